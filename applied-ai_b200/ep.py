"""Expert-parallel MoE layer: experts sharded across ranks, tokens data-parallel.

Rank r of P owns experts [r*E/P, (r+1)*E/P) and T/P tokens.  One exchange each way:

    route by global expert  ->  counts all-to-all  ->  payload all-to-all (rows sorted by
    destination rank, then expert)  ->  re-sort arrivals by local expert  ->  grouped GEMM
    (gate+up, SwiGLU)  ->  grouped GEMM (down, stored back in arrival order)  ->  return
    all-to-all  ->  weighted top-k combine on the home rank

The reference has no distributed code at all (`fused_moe` assumes every expert is local,
kernels/triton/inference/col_major_moe_gemm/v0_moe_fused.py:249); this layer extends the
same computation to the expert-parallel configuration of the benchmark.  The collectives
are torch.distributed all_to_all_single (NCCL over NVLink on GPUs); received rows land
in local memory before any kernel touches them.

Every routed row is computed by the same kernel with the same reduction order whatever P
is, and the combine sums in fixed top-k order on the home rank, so outputs do not depend
on the number of ranks.

The compute steps come from an `ops` object.  The default, `CudaOps`, calls
libb200moe.so; there is no CPU implementation in this package (the CPU tests of the
exchange logic inject their own checker ops).
"""
import torch
import torch.distributed as dist


class CudaOps:
    """The layer's compute steps on the GPU.  mode: "bf16" or "fp8_blockwise"."""

    def __init__(self, w1, w2, mode="bf16", cta_group=0, fuse_requant=True):
        """fuse_requant (fp8_blockwise, default): the gate+up GEMM's epilogue quantises the fp32 SwiGLU
        values 1x128 itself (same formula and bytes as float8_groupwise_quantize on those values);
        False rounds them to bf16 first and runs the separate quantiser pass."""
        from . import groupgemm, moe, quant
        self._gg, self._moe, self._quant = groupgemm, moe, quant
        self.mode = mode
        self.cta_group = cta_group
        self.fuse_requant = bool(fuse_requant)
        if mode == "bf16":
            self.w1, self.w2 = w1.contiguous(), w2.contiguous()
        elif mode == "fp8_blockwise":
            self.w1, self.w1_scale = self._quantize_weight(w1)
            self.w2, self.w2_scale = self._quantize_weight(w2)
        else:
            raise ValueError("mode must be 'bf16' or 'fp8_blockwise'")

    @classmethod
    def from_quantized(cls, w1q, w1_scale, w2q, w2_scale, cta_group=0, fuse_requant=True):
        """fp8_blockwise ops from weights that are already e4m3 with 128x128 block scales
        (w [E, N, K] float8_e4m3fn, scales [E, ceil(N/128), K/128] fp32), e.g. loaded from a
        checkpoint or quantised expert by expert to bound the set-up memory."""
        if w1q.dtype != torch.float8_e4m3fn or w2q.dtype != torch.float8_e4m3fn:
            raise ValueError("from_quantized takes float8_e4m3fn weights")
        self = cls.__new__(cls)
        from . import groupgemm, moe, quant
        self._gg, self._moe, self._quant = groupgemm, moe, quant
        self.mode, self.cta_group, self.fuse_requant = "fp8_blockwise", cta_group, bool(fuse_requant)
        self.w1, self.w1_scale = w1q.contiguous(), w1_scale.contiguous()
        self.w2, self.w2_scale = w2q.contiguous(), w2_scale.contiguous()
        return self

    def _quantize_weight(self, w):
        if w.dtype == torch.float8_e4m3fn:
            raise ValueError("pass unquantised weights; block scales are computed here")
        q = torch.empty(w.shape, dtype=torch.float8_e4m3fn, device=w.device)
        s = torch.empty(w.shape[0], (w.shape[1] + 127) // 128, w.shape[2] // 128, dtype=torch.float32,
                        device=w.device)
        for e in range(w.shape[0]):  # one expert at a time bounds the fp32 temporaries
            q[e], s[e] = self._quant.quantize_fp8_block(w[e])
        return q, s

    def route(self, ids, num_experts):
        return self._moe.route(ids, num_experts, check=False)

    def gather(self, src, idx, div=1):
        return self._moe.gather_rows(src, idx, div=div)

    def dispatch_payloads(self, hidden):
        """What travels per token: the bf16 row, or its e4m3 bytes plus the 1x128 scales."""
        if self.mode == "bf16":
            return [hidden]
        q, s = self._quant.float8_groupwise_quantize(hidden)
        return [q.view(torch.uint8), s]

    def expert_ffn(self, rows, m_sizes, out_row_map=None, experts=None, peer=None):
        """rows: payload tensors sorted by local expert -> [R, H] bf16.  With out_row_map the
        down GEMM stores sorted row r at row out_row_map[r] (leaving expert order in the
        same pass).  experts=(lo, hi) restricts the call to that range of local experts.
        peer=(tags, bases, n_peers, rows_per_buffer): the down GEMM stores every row into the
        buffer of the rank named by its tag (nothing is returned)."""
        gg = self._gg
        lo, hi = experts if experts is not None else (0, self.w1.shape[0])
        if peer is not None:
            tags, bases, n_peers, y_rows = peer
            if self.mode == "bf16":
                h = gg.grouped_gemm(rows[0], self.w1, m_sizes, epilogue="swiglu", check=False,
                                    cta_group=self.cta_group)
                return gg.grouped_gemm_ex(gg.KIND_BF16, h, self.w2, m_sizes, cta_group=self.cta_group,
                                          out_row_tags=tags, peer_bases=bases, n_peers=n_peers, out_rows=y_rows)
            xq, xs = rows[0].view(torch.float8_e4m3fn), rows[1]
            hq, hs = self._gate_up_fp8(xq, xs, self.w1, self.w1_scale, m_sizes)
            return gg.grouped_gemm_ex(gg.KIND_FP8_BLOCKWISE, hq, self.w2, m_sizes, x_scale=hs, w_scale=self.w2_scale,
                                      cta_group=self.cta_group, out_row_tags=tags, peer_bases=bases,
                                      n_peers=n_peers, out_rows=y_rows)
        if self.mode == "bf16":
            h = gg.grouped_gemm(rows[0], self.w1[lo:hi], m_sizes, epilogue="swiglu", check=False,
                                cta_group=self.cta_group)
            return gg.grouped_gemm(h, self.w2[lo:hi], m_sizes, check=False, cta_group=self.cta_group,
                                   out_row_map=out_row_map)
        xq, xs = rows[0].view(torch.float8_e4m3fn), rows[1]
        hq, hs = self._gate_up_fp8(xq, xs, self.w1[lo:hi], self.w1_scale[lo:hi], m_sizes)
        return gg.grouped_gemm_fp8_blockwise(hq, self.w2[lo:hi], m_sizes, hs, self.w2_scale[lo:hi], check=False,
                                             cta_group=self.cta_group, out_row_map=out_row_map)

    def _gate_up_fp8(self, xq, xs, w1, w1_scale, m_sizes):
        """gate+up GEMM with SwiGLU -> (e4m3 rows, 1x128 scales) for the down GEMM."""
        gg = self._gg
        if self.fuse_requant:
            return gg.grouped_gemm_ex(gg.KIND_FP8_BLOCKWISE, xq, w1, m_sizes, x_scale=xs, w_scale=w1_scale,
                                      epilogue="swiglu_fp8", cta_group=self.cta_group)
        h = gg.grouped_gemm_fp8_blockwise(xq, w1, m_sizes, xs, w1_scale, epilogue="swiglu", check=False,
                                          cta_group=self.cta_group)
        return self._quant.float8_groupwise_quantize(h)

    def combine(self, y, inv_perm, topk_weights, num_tokens, top_k):
        return self._moe.combine_topk(y, inv_perm, topk_weights, num_tokens, top_k)

    def payload_row_bytes(self, hidden_size):
        """Bytes per token of each payload part, matching dispatch_payloads."""
        if self.mode == "bf16":
            return [2 * hidden_size]
        return [hidden_size, 4 * (hidden_size // 128)]


class PeerBuffers:
    """This rank's receive side of the peer-memory exchange — payload rows (capacity_rows per
    part), their (rank, row) tags and the buffer the experts' results come home to — in ONE
    allocation that every other rank of the group maps with CUDA IPC (opened with its own
    device current, checked with a copy-engine round trip before any kernel uses it).
    Built once; every rank must build it at the same time."""

    def __init__(self, group, device, capacity_rows, part_row_bytes, home_rows, hidden_size):
        import ctypes

        from . import _lib
        self.P = dist.get_world_size(group)
        self.me = dist.get_rank(group)
        self.cap, self.home_rows, self.H = int(capacity_rows), int(home_rows), int(hidden_size)
        self.part_row_bytes = list(part_row_bytes)
        # ... + the flag words of the stream barrier (2 slots x P ranks), last so the other offsets keep their order
        sizes = [self.cap * b for b in part_row_bytes] + [self.cap * 8, self.home_rows * self.H * 2, 2 * self.P * 4]
        self.offsets, total = [], 0
        for sz in sizes:
            self.offsets.append(total)
            total += (sz + 255) // 256 * 256
        self.arena = torch.zeros(max(total, 1 << 21), dtype=torch.uint8, device=device)
        a = self.arena
        self.parts = [a[o:o + sz] for o, sz in zip(self.offsets[:-3], sizes[:-3])]
        self.tags = a[self.offsets[-3]:self.offsets[-3] + sizes[-3]].view(torch.int64)
        self.y_home = a[self.offsets[-2]:self.offsets[-2] + sizes[-2]].view(torch.bfloat16).view(self.home_rows, self.H)
        self.epoch = 0   # stream-barrier epoch: the same on every rank because every rank makes the same calls
        # export: (handle of the allocation the arena lives in, byte offset of the arena inside it)
        lib = _lib.load()
        hbuf = ctypes.create_string_buffer(64)
        off = ctypes.c_uint64(0)
        with torch.cuda.device(device):
            _lib.check(lib.b200moe_ipc_export(a.data_ptr(), hbuf, ctypes.byref(off)), "ipc_export")
        handle, off_in_block = hbuf.raw, int(off.value)
        gathered = [None] * self.P
        dist.all_gather_object(gathered, (handle, off_in_block), group=group)
        self._opened = []
        scratch = torch.zeros(8, dtype=torch.uint8, device=device)
        bases = []
        with torch.cuda.device(device):
            for r in range(self.P):
                if r == self.me:
                    bases.append(a.data_ptr())
                    continue
                h, off = gathered[r]
                base = ctypes.c_void_p()
                _lib.check(lib.b200moe_ipc_open(h, ctypes.byref(base)), "ipc_open")
                self._opened.append(base.value)
                torch.cuda.synchronize()
                # every rank probes its own word of the peer's arena, so concurrent probes cannot collide
                _lib.check(lib.b200moe_peer_probe(base.value + off + 8 * self.me, scratch.data_ptr()), "peer_probe")
                bases.append(base.value + off)
        # device tables of base addresses, one per buffer kind, indexed by rank
        self.tables = [torch.tensor([bases[r] + o for r in range(self.P)], dtype=torch.int64, device=device)
                       for o in self.offsets]
        self.sync = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def barrier(self, slot, status_word, stream, limit_ns=2_000_000_000):
        """Orders this rank's stream after every rank's kernels enqueued so far (flag words in the peers'
        arenas, no collective, no host synchronisation).  Called in the same order on every rank."""
        from . import _lib
        if slot == 0:
            self.epoch += 1
        _lib.check(_lib.load().b200moe_ep_barrier(self.tables[-1].data_ptr(), self.P, self.me, slot, self.epoch,
                                                  limit_ns, status_word.data_ptr(), stream), "ep_barrier")

    def close(self):
        from . import _lib
        lib = _lib.load()
        for base in self._opened:
            lib.b200moe_ipc_close(base)
        self._opened = []


def expert_ids_from_counts(recv_counts, total):
    """Local expert id of every received row.  recv_counts [P, E_local]: rows arrive
    grouped by source rank and, inside one source, by expert."""
    P, e_local = recv_counts.shape
    ids = torch.arange(e_local, device=recv_counts.device, dtype=torch.int32).repeat(P)
    return torch.repeat_interleave(ids, recv_counts.reshape(-1).to(torch.int64), output_size=total)


class ExpertParallelMoE:
    """One MoE FFN layer under expert parallelism.

    ops          compute steps holding this rank's expert weights (CudaOps)
    num_experts  global expert count E (divisible by the group size)
    group        torch.distributed process group (None: default group, or no exchange at
                 all when torch.distributed is not initialised — the single-GPU case)
    waves        the local experts are cut into this many consecutive chunks; each chunk has
                 its own dispatch and return all-to-all, issued asynchronously, so the
                 exchange of one chunk runs under the GEMMs of its neighbours.  Must divide
                 E / P (it is lowered to the nearest divisor otherwise).
    """

    def __init__(self, ops, num_experts, group=None, waves=1, exchange="nccl", max_tokens=None, top_k=None,
                 hidden_size=None, capacity_factor=1.5, barrier="flags"):
        """exchange="nccl": all_to_all_single collectives (rows land in local buffers first).
        exchange="peer": rows are written straight into the owner's memory by the sender's push
        kernel and come home through the down GEMM's store (ordinary stores or non-multicast
        shared->global bulk copies over NVLink into CUDA IPC mappings; peer memory is never read); needs max_tokens (per rank), top_k and hidden_size up front because the
        shared buffers are built once, and a receive capacity of capacity_factor times the
        rows a rank sends.  No host synchronisation happens in that mode, so a routing skew that
        overflows a rank's receive buffer cannot raise inside forward(): the surplus rows are
        dropped (they contribute zero to their tokens), status 24 is recorded on the device, and
        raise_on_status() reports it."""
        self.ops = ops
        self.group = group
        self.E = int(num_experts)
        self.P = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        if self.E % self.P:
            raise ValueError(f"{self.E} experts cannot be split evenly over {self.P} ranks")
        self.e_local = self.E // self.P
        waves = max(1, min(int(waves), self.e_local))
        while self.e_local % waves:
            waves -= 1
        self.W = waves
        self.e_wave = self.e_local // self.W
        self.last_plan = None
        self._remap = None
        self.exchange = exchange
        if barrier not in ("flags", "nccl"):
            raise ValueError("barrier must be 'flags' or 'nccl'")
        self.barrier = barrier   # exchange="peer": how the ranks' streams meet ("nccl": one-element all-reduces)
        self.peer = None
        self.profile = False     # when True, forward() records CUDA-event timings of its phases
        self.timings = []        # [(phase, milliseconds)] of the last profiled forward
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange must be 'nccl' or 'peer'")
        if exchange == "peer" and self.P > 1:
            if not (max_tokens and top_k and hidden_size):
                raise ValueError("exchange='peer' needs max_tokens, top_k and hidden_size")
            dev = torch.device("cuda", torch.cuda.current_device())
            home_rows = int(max_tokens) * int(top_k)
            cap = int(home_rows * float(capacity_factor) + 127) // 128 * 128
            self.peer = PeerBuffers(group, dev, cap, ops.payload_row_bytes(int(hidden_size)), home_rows,
                                    int(hidden_size))

    def _forward_peer(self, hidden, topk_weights, topk_ids):
        """Dispatch by remote stores, return inside the down GEMM; two stream barriers (flag words in
        the peers' arenas, or one-element all-reduces with barrier="nccl") order "rows have landed"
        and "results are home" on every rank."""
        import ctypes

        from . import _lib
        from . import groupgemm as gg
        ops, P, pb = self.ops, self.P, self.peer
        T, H = hidden.shape
        k = topk_ids.shape[1]
        R = T * k
        if R > pb.home_rows or H != pb.H:
            raise RuntimeError("more routed rows or another hidden size than the peer buffers were built for")
        dev = hidden.device
        lib = _lib.load()
        stream = torch.cuda.current_stream().cuda_stream
        word = gg._status_word(dev)
        marks = []

        def mark(name):
            if self.profile:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        m_glob, offsets, perm, inv_perm = ops.route(topk_ids, self.E)
        counts = torch.empty((P, self.E), dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(counts, m_glob, group=self.group)
        dst_base = torch.empty(self.E, dtype=torch.int32, device=dev)
        m_loc = torch.empty(self.e_local, dtype=torch.int32, device=dev)
        _lib.check(lib.b200moe_ep_plan(counts.data_ptr(), P, self.E, pb.me, pb.cap, dst_base.data_ptr(),
                                       m_loc.data_ptr(), word.data_ptr(), stream), "ep_plan")
        mark("route+plan")
        parts = ops.dispatch_payloads(hidden)
        mark("quantise tokens")
        p1 = parts[1] if len(parts) > 1 else None
        rc = lib.b200moe_ep_push(parts[0].data_ptr(), pb.part_row_bytes[0], 0 if p1 is None else p1.data_ptr(),
                                 pb.part_row_bytes[1] if p1 is not None else 0, perm.data_ptr(), k,
                                 offsets.data_ptr(), dst_base.data_ptr(), R, self.E, P, pb.me, pb.cap, T,
                                 pb.tables[0].data_ptr(), pb.tables[1].data_ptr() if p1 is not None else 0,
                                 pb.tables[len(parts)].data_ptr(), pb.y_home.data_ptr(), 2 * H, stream)
        _lib.check(rc, "ep_push")
        mark("push")
        self._stream_barrier(0, word, stream)                # every rank's rows have landed everywhere
        mark("barrier 1")
        rows = []
        for buf, nbytes, part in zip(pb.parts, pb.part_row_bytes, parts):
            rows.append(buf.view(part.dtype).view(pb.cap, nbytes // part.element_size()))
        ops.expert_ffn(rows, m_loc, peer=(pb.tags, pb.tables[len(parts) + 1], P, pb.home_rows))
        mark("experts (down GEMM stores home)")
        self._stream_barrier(1, word, stream)                # every result row is home
        mark("barrier 2")
        out = ops.combine(pb.y_home[:R], inv_perm, topk_weights, T, k)
        mark("combine")
        if self.profile:
            torch.cuda.synchronize()
            self.timings = [(marks[i][0], marks[i - 1][1].elapsed_time(marks[i][1])) for i in range(1, len(marks))]
        return out

    def _stream_barrier(self, slot, word, stream):
        if self.barrier == "flags":
            self.peer.barrier(slot, word, stream)
        else:
            dist.all_reduce(self.peer.sync, group=self.group)

    def raise_on_status(self):
        """Deferred check of everything this layer has enqueued on the current device so far.  The
        layer itself never synchronises with the host; call this wherever a synchronisation is
        acceptable (after a step, every N steps, before results are trusted).  Raises
        B200MoeError when a rank's receive buffer overflowed (status 24: rows past the capacity
        were dropped, their experts' contributions are missing from the outputs of that step — build the layer with a larger
        capacity_factor, or use exchange="nccl", which sizes its buffers per step) or when a
        device-side wait ran out; ValueError for invalid expert ids."""
        from . import groupgemm as gg
        gg.pending_status()

    def _key_table(self, device):
        """Sort key of every global expert: (wave, destination rank, expert inside the wave), so
        that the rows of one wave are contiguous and, inside it, grouped by destination."""
        if self._remap is None or self._remap.device != device:
            e = torch.arange(self.E, device=device)
            dest, el = e // self.e_local, e % self.e_local
            wave, ew = el // self.e_wave, el % self.e_wave
            self._remap = (wave * (self.P * self.e_wave) + dest * self.e_wave + ew).to(torch.int32)
        return self._remap

    def _a2a(self, out, inp, out_splits, in_splits):
        return dist.all_to_all_single(out, inp, output_split_sizes=out_splits, input_split_sizes=in_splits,
                                      group=self.group, async_op=True)

    def forward(self, hidden, topk_weights, topk_ids):
        """hidden [T_local, H]; topk_ids [T_local, k] GLOBAL expert ids; returns [T_local, H] bf16."""
        ops, P, W, ew = self.ops, self.P, self.W, self.e_wave
        T, H = hidden.shape
        k = topk_ids.shape[1]
        dev = hidden.device

        if P == 1:
            # every expert is local: the routed order already is the expert order
            m_glob, _, perm, inv_perm = ops.route(topk_ids, self.E)
            rows = [ops.gather(pay, perm, div=k) for pay in ops.dispatch_payloads(hidden)]
            y_home = ops.expert_ffn(rows, m_glob)
            self.last_plan = {"send_splits": [int(topk_ids.numel())], "recv_splits": [int(topk_ids.numel())]}
            return ops.combine(y_home, inv_perm, topk_weights, T, k)

        if self.peer is not None:
            return self._forward_peer(hidden, topk_weights, topk_ids)

        # 1. sort this rank's routed rows by (wave, destination rank, expert)
        keys = self._key_table(dev)[topk_ids.reshape(-1).long()]
        m_key, _, perm, inv_perm = ops.route(keys, W * P * ew)
        send_counts = m_key.reshape(W, P, ew).permute(1, 0, 2).contiguous().to(torch.int64)   # [dest, wave, expert]

        # 2. counts exchange, then ONE host read of all split sizes
        recv_counts = torch.empty_like(send_counts)                                            # [src, wave, expert]
        self._a2a(recv_counts, send_counts, None, None).wait()
        sizes = torch.stack([send_counts.sum(2), recv_counts.sum(2)]).cpu()                    # [2, P, W]
        send_pw, recv_pw = sizes[0], sizes[1]
        n_send = int(send_pw.sum())
        send_off = [0]
        for w in range(W):
            send_off.append(send_off[-1] + int(send_pw[:, w].sum()))
        self.last_plan = {"send_splits": send_pw.sum(1).tolist(), "recv_splits": recv_pw.sum(1).tolist(),
                          "waves": W}

        # 3. dispatch: every wave's payload all-to-all is issued now, in wave order
        send_bufs = [ops.gather(pay, perm, div=k) for pay in ops.dispatch_payloads(hidden)]
        pending = []
        for w in range(W):
            in_splits, out_splits = send_pw[:, w].tolist(), recv_pw[:, w].tolist()
            n_recv = sum(out_splits)
            bufs, works = [], []
            for sb in send_bufs:
                rb = torch.empty((n_recv, sb.shape[1]), dtype=sb.dtype, device=dev)
                works.append(self._a2a(rb, sb[send_off[w]:send_off[w + 1]], out_splits, in_splits))
                bufs.append(rb)
            pending.append((bufs, works, n_recv, in_splits, out_splits))

        # 4. per wave: wait for its rows, sort arrivals by expert, run the experts, send results home
        y_home = None
        returns = []
        for w, (bufs, works, n_recv, in_splits, out_splits) in enumerate(pending):
            for wk in works:
                wk.wait()
            # arrivals are ordered (source rank, expert); the GEMM wants (expert, source rank)
            ids_recv = expert_ids_from_counts(recv_counts[:, w, :], n_recv)
            m_loc, _, perm2, _ = ops.route(ids_recv, ew)
            rows = [ops.gather(r, perm2) for r in bufs]
            # the down GEMM stores each row straight back at its arrival position
            y_arrival = ops.expert_ffn(rows, m_loc, out_row_map=perm2, experts=(w * ew, (w + 1) * ew))
            if y_home is None:
                y_home = torch.empty((n_send, H), dtype=y_arrival.dtype, device=dev)
            returns.append((self._a2a(y_home[send_off[w]:send_off[w + 1]], y_arrival, in_splits, out_splits),
                            y_arrival))

        # 5. weighted sum over the top-k on the home rank
        for wk, _ in returns:
            wk.wait()
        return ops.combine(y_home, inv_perm, topk_weights, T, k)

    __call__ = forward
