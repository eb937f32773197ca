"""Benchmark of the MoE grouped-GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c5|c3]

Default workload ("c2"): bf16 grouped GEMM at the DeepSeek-V3 routed-expert gate+up
shape — G=8 experts, K=7168, N=4096, 16384 rows, group sizes multiples of 128, seeded
synthetic data.  One step = one grouped GEMM over the whole batch.  Metric: TFLOPS
(2*M*N*K / time).  With N > 1 GPUs every rank holds its own 8 experts and 16384 rows
(expert-sharded, no exchange in this path) and the value is the sum over ranks.

Prints ONE JSON line (rank 0).  `--impl reference` times the reference's own ground
truth for this path — the torch per-expert matmul loop on the host CPU cores — on a
bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (G, M, N, K)
    "c2": (8, 16384, 4096, 7168),
    "c5": (128, 8192, 1408, 2048),
    "c2_fp8_rowwise": (8, 16384, 4096, 7168),
    "c2_fp8_blockwise": (8, 16384, 4096, 7168),
    # one rank's share of the DeepSeek-V3 layer at 8-way expert parallelism: 32 experts, 32768 routed rows
    "c4_gate_up": (32, 32768, 4096, 7168),
    "c4_down": (32, 32768, 7168, 2048),
    "c2_backward": (8, 16384, 4096, 7168),  # grad_x and grad_w of the C2 forward
}
WORKLOAD_KIND = {"c2": "bf16", "c5": "bf16", "c2_fp8_rowwise": "fp8_rowwise", "c2_fp8_blockwise": "fp8_blockwise",
                 "c4_gate_up": "fp8_blockwise", "c4_down": "fp8_blockwise", "c2_backward": "bf16_backward"}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        d = json.load(open(path))
        return {"bf16_tflops": float(d["bf16_tflops"]), "bf16_tflops_sustained": float(d["bf16_tflops_sustained"]),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    except Exception:
        return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.thread = [], None, None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [r for r in self.rows if t0 - 0.05 <= r[0] <= t1 + 0.05] or self.rows
        for _, line in rows:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        med = sm[len(sm) // 2] if sm else None
        return {"sm_mhz": med, "sm_max_mhz": smax, "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def cpu_loop_tflops(G, N, K, rows_per_group, repeats, seed=1001):
    """The reference's per-expert loop (dev/triton_groupGEMM/testing/base_testing.py:125-131)
    in fp32 on the host cores, over `rows_per_group` rows of each group."""
    from oracle import grouped as O
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(seed)
    M = G * rows_per_group
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(G, N, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    m_sizes = torch.full((G,), rows_per_group, dtype=torch.int32)
    xf, wf = x.float(), w.float()
    O.grouped_gemm_ref(xf[: G * 8], wf, torch.full((G,), 8, dtype=torch.int32))  # touch pages, spin up threads
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        O.grouped_gemm_ref(xf, wf, m_sizes)
        times.append(time.perf_counter() - t0)
    times.sort()
    t = times[len(times) // 2]
    return 2.0 * M * N * K / t / 1e12, t, M


def run_reference_layer(args):
    """The reference's `torch_moe` procedure (kernels/triton/inference/col_major_moe_gemm/
    test_moe_gemm.py:16-30) in fp32 on the host cores, on a token sample of the layer."""
    from oracle import grouped as O
    T, H, I, E, k, mode = LAYERS[args.workload]
    torch.set_num_threads(os.cpu_count() or 1)
    ns, es = 64, min(E, 8)
    g = torch.Generator().manual_seed(9)
    a = torch.randn(ns, H, generator=g)
    w1 = torch.randn(es, 2 * I, H, generator=g) * H ** -0.5
    w2 = torch.randn(es, H, I, generator=g) * I ** -0.5
    tw, ids = torch.topk(torch.softmax(torch.randn(ns, es, generator=g), -1), min(k, es))
    for _ in range(max(1, min(args.warmup, 2))):
        O.torch_moe_ref(a, w1, w2, tw, ids)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.torch_moe_ref(a, w1, w2, tw, ids)
    dt = (time.perf_counter() - t0) / args.steps
    v = ns / dt
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: MoE FFN layer T={T} H={H} I={I} E={E} top-{k}", "sampled_tokens": ns},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "reference",
                         "sample": f"{ns} tokens over {es} experts top-{min(k, es)}, full H and I, fp32"},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    if args.workload in LAYERS:
        return run_reference_layer(args)
    G, M, N, K = WORKLOADS[args.workload]
    rows = 256 if M // G >= 256 else max(8, M // G)
    G = min(G, 8)
    torch.set_num_threads(os.cpu_count() or 1)
    from oracle import grouped as O
    g = torch.Generator().manual_seed(1001)
    Ms = G * rows
    x = torch.randn(Ms, K, generator=g).to(torch.bfloat16).float()
    w = (torch.randn(G, N, K, generator=g) * K ** -0.5).to(torch.bfloat16).float()
    m_sizes = torch.full((G,), rows, dtype=torch.int32)
    for _ in range(max(1, min(args.warmup, 3))):
        O.grouped_gemm_ref(x, w, m_sizes)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.grouped_gemm_ref(x, w, m_sizes)
    dt = (time.perf_counter() - t0) / args.steps
    tflops = 2.0 * Ms * N * K / dt / 1e12
    sample = f"{rows} rows of each of the {G} groups ({Ms} of {M} rows), full N and K, fp32 torch.matmul loop"
    line = {
        "impl": "reference", "metric": "grouped_gemm_tflops", "value": tflops, "unit": "TFLOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: grouped GEMM G={G} K={K} N={N} M={M}", "sampled_rows": Ms},
        "cpu_baseline": {"value": tflops, "unit": "TFLOPS", "cores": torch.get_num_threads(), "kind": "reference",
                         "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def fp8_peak_tflops():
    """Dense FP8 tensor peak of this GPU, measured here the way the bf16 peaks were
    (library GEMM 8192^3, best of 10): torch._scaled_mm, e4m3 x e4m3 -> bf16."""
    n = 8192
    a = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn).t()
    one = torch.ones((), device="cuda")
    best = None
    for i in range(13):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        e1.record()
        torch.cuda.synchronize()
        if i >= 3:
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
    return 2.0 * n ** 3 / (best * 1e-3) / 1e12


PROFILED_TRAFFIC_BYTES = {
    "c2": 1.160e9,                # profiles/gg_kernel_bf16_c2_deepseek_gate_up.md
    "c5": 750.5e6,                # profiles/gg_kernel_bf16_c5_skewed_routing.md
    "c2_fp8_rowwise": 471.0e6,    # profiles/gg_kernel_fp8_rowwise_c2_shape.md
    "c2_fp8_blockwise": 477.1e6,  # profiles/gg_fp8_block_kernel_c2_shape.md
}


def vendor_grouped_mm(wl, y_ours, iters=10):
    """The bf16 grouped GEMM of the installed torch (`torch._grouped_mm`, a library kernel) on the same
    resident inputs, as a second baseline next to the CPU loop.  Returns a dict for the JSON line; never
    raises.  The FP8 counterpart (`torch._scaled_grouped_mm`) is not called: in this torch build its kernel
    is compiled for another architecture and aborts on the device, which costs the process its context."""
    try:
        m_sizes = wl["m_sizes"]
        offs = torch.cumsum(m_sizes, 0).to(torch.int32)
        if wl["kind"] == "bf16":
            x, w = wl["x"], wl["w"]
            name = "torch._grouped_mm"
            fn = lambda: torch._grouped_mm(x, w.transpose(-2, -1), offs=offs)
        else:
            return None
        out = fn()
        torch.cuda.synchronize()
        rows = wl["rows"]
        diff = float((out[:rows].float() - y_ours[:rows].float()).abs().max() / y_ours[:rows].float().abs().max())
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        return {"kind": name, "value": wl["flops"] / (ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": ms,
                "max_rel_diff_vs_this_engine": diff, "note": "library kernel of the installed torch, same resident inputs"}
    except Exception as exc:  # missing op, unsupported shape or dtype on this build
        return {"kind": "torch grouped mm", "unavailable": f"{type(exc).__name__}: {str(exc)[:160]}"}


def make_workload(name, rank, dev, cta_group):
    """Builds device-resident inputs and the step function of one workload."""
    import applied_ai_b200 as B
    from applied_ai_b200 import configs
    G, M, N, K = WORKLOADS[name]
    kind = WORKLOAD_KIND[name]
    wl = {"G": G, "M": M, "N": N, "K": K, "kind": kind, "epilogue": "none"}
    if name == "c5":
        x, w, m_sizes = configs.c5_skew(seed=1004 + 17 * rank, device=dev)
        wl["m_desc"] = "m_sizes multinomial Zipf(1.2), 8 empty groups"
    else:
        x, w, m_sizes = configs.c2_deepseek_gate_up(seed=1001 + 17 * rank, M=M, K=K, N=N, G=G, device=dev)
        wl["m_desc"] = "m_sizes multinomial x128"
    wl["m_sizes"] = m_sizes
    wl["rows"] = int(m_sizes.sum())
    n_out = N
    if kind == "bf16":
        wl.update(x=x, w=w, act=[x], elem=2)
        wl["step"] = lambda a=x: B.grouped_gemm(a, w, m_sizes, cta_group=cta_group)
        wl["step_with"] = lambda act, ms: B.grouped_gemm(act[0], w, ms, cta_group=cta_group)
        wl["ref_rows"] = lambda rows, e: x[rows].cpu().float() @ w[e].cpu().float().T
        wl["tol"] = 1e-2
    elif kind == "bf16_backward":
        from applied_ai_b200.tgroup_gemm_backwards import grouped_gemm_backward
        gd = torch.Generator(device=dev).manual_seed(4242 + rank)
        dy = torch.randn(M, N, generator=gd, device=dev).to(torch.bfloat16)
        wl.update(x=x, w=w, act=[dy], elem=2)
        wl["step"] = lambda a=dy: grouped_gemm_backward(a, x, w, m_sizes, cta_group=cta_group, check=False)[0]
        wl["step_with"] = lambda act, ms: grouped_gemm_backward(act[0], x, w, ms, cta_group=cta_group, check=False)[0]
        wl["ref_rows"] = lambda rows, e: dy[rows].cpu().float() @ w[e].cpu().float()
        wl["tol"] = 1e-2
    elif kind == "fp8_rowwise":
        xq, xs = B.quantize_fp8_row(x)
        wq, ws = B.quantize_fp8_row(w.reshape(G * N, K))
        del x, w
        wl.update(act=[xq, xs], elem=1)
        wl["step"] = lambda a=xq, s=xs: B.grouped_gemm_fp8_rowwise(a, wq, m_sizes, s, ws, cta_group=cta_group)
        wl["step_with"] = lambda act, ms: B.grouped_gemm_fp8_rowwise(act[0], wq, ms, act[1], ws, cta_group=cta_group)
        wl["ref_rows"] = lambda rows, e: (xq[rows].cpu().float() @ wq[e * N:(e + 1) * N].cpu().float().T
                                          * xs[rows].cpu()[:, None] * ws[e * N:(e + 1) * N].cpu()[None, :])
        wl["tol"] = 2e-2
    else:  # fp8_blockwise
        xq, xs = B.float8_groupwise_quantize(x)
        wq = torch.empty(G, N, K, dtype=torch.float8_e4m3fn, device=dev)
        ws = torch.empty(G, (N + 127) // 128, K // 128, dtype=torch.float32, device=dev)
        for e in range(G):
            wq[e], ws[e] = B.quantize_fp8_block(w[e])
        del x, w
        epi = "swiglu" if name == "c4_gate_up" else "none"
        wl["epilogue"] = epi
        n_out = N // 2 if epi == "swiglu" else N
        wl.update(act=[xq, xs], elem=1)
        wl["step"] = lambda a=xq, s=xs: B.grouped_gemm_fp8_blockwise(a, wq, m_sizes, s, ws, epilogue=epi,
                                                                     cta_group=cta_group)
        wl["step_with"] = lambda act, ms: B.grouped_gemm_fp8_blockwise(act[0], wq, ms, act[1], ws, epilogue=epi,
                                                                       cta_group=cta_group)

        def ref_rows(rows, e):
            xd = xq[rows].cpu().float() * xs[rows].cpu().repeat_interleave(128, dim=1)
            wd = wq[e].cpu().float() * ws[e].cpu().repeat_interleave(128, dim=0)[:N].repeat_interleave(128, dim=1)
            r = xd @ wd.T
            if epi == "swiglu":
                r = torch.nn.functional.silu(r[:, :N // 2]) * r[:, N // 2:]
            return r
        wl["ref_rows"] = ref_rows
        wl["tol"] = 2e-2
    wl["n_out"] = K if kind == "bf16_backward" else n_out
    wl["flops"] = (4.0 if kind == "bf16_backward" else 2.0) * wl["rows"] * N * K
    nonempty = int((m_sizes > 0).sum())
    act_bytes = sum(t.numel() * t.element_size() for t in wl["act"])
    wl["act_bytes"] = act_bytes
    wl["alg_bytes"] = act_bytes + nonempty * N * K * wl["elem"] + wl["rows"] * n_out * 2
    return wl


def run_ours(args):
    import applied_ai_b200 as B
    from applied_ai_b200 import _lib

    rank, world, local = dist_env()
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_DEBUG", "WARN")  # keep NCCL's version banner off stdout
        dist.init_process_group("nccl", device_id=dev)
    _lib.load(build_if_missing=False)
    B.set_default_check(False)

    wl = make_workload(args.workload, rank, dev, args.cta_group)
    G, M, N, K = wl["G"], wl["M"], wl["N"], wl["K"]
    m_sizes, step, flops = wl["m_sizes"], wl["step"], wl["flops"]

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    y = step()
    torch.cuda.synchronize()
    status = int(B.groupgemm._status_word(dev).item())
    assert status == 0, f"device status {status}"

    # correctness guard on the timed configuration: a sample of rows against the host loop
    if rank == 0:
        from oracle import grouped as O
        gsel = torch.Generator().manual_seed(7)
        start, worst = 0, 0.0
        ms = m_sizes.cpu()
        for e in range(G):
            mg = int(ms[e])
            if mg and e % max(1, G // 8) == 0:
                pick = (start + torch.randint(0, mg, (2,), generator=gsel)).to(dev)
                worst = max(worst, O.rel_err(y[pick].cpu().float(), wl["ref_rows"](pick, e)))
            start += mg
        assert worst <= wl["tol"], f"bench output fails parity: {worst}"

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid))
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    launches0 = _lib.launch_count()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    launches = _lib.launch_count() - launches0   # kernels of this library enqueued inside the timed region
    barrier()
    t_wall1 = time.time()
    ms_total = ev0.elapsed_time(ev1)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None

    vendor = vendor_grouped_mm(wl, y) if (rank == 0 and world == 1) else None

    # end to end: pinned host activations (and their scales) -> device, the public API call, result -> host,
    # every step.  Copies and compute of consecutive steps overlap the way a caller streaming batches
    # would run them: an upload stream, the compute stream and a download stream over two sets of buffers.
    act_host = [t.cpu().pin_memory() for t in wl["act"]]
    m_host = m_sizes.cpu().pin_memory()
    nbuf = 2
    act_dev = [[torch.empty_like(t) for t in wl["act"]] for _ in range(nbuf)]
    m_dev = [torch.empty_like(m_sizes) for _ in range(nbuf)]
    y_host = [torch.empty((M, wl["n_out"]), dtype=torch.bfloat16).pin_memory() for _ in range(nbuf)]
    s_up, s_cmp, s_down = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_up = [torch.cuda.Event() for _ in range(nbuf)]
    ev_cmp = [torch.cuda.Event() for _ in range(nbuf)]
    ev_down = [torch.cuda.Event() for _ in range(nbuf)]
    outs = [None] * nbuf

    def e2e_run(n):
        for i in range(n):
            b = i % nbuf
            with torch.cuda.stream(s_up):
                s_up.wait_event(ev_cmp[b])          # the GEMM that read this input buffer two steps ago
                for d, h in zip(act_dev[b], act_host):
                    d.copy_(h, non_blocking=True)
                m_dev[b].copy_(m_host, non_blocking=True)
                ev_up[b].record(s_up)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_up[b])
                s_cmp.wait_event(ev_down[b])        # the download that read this output slot two steps ago
                outs[b] = wl["step_with"](act_dev[b], m_dev[b])
                ev_cmp[b].record(s_cmp)
            with torch.cuda.stream(s_down):
                s_down.wait_event(ev_cmp[b])
                y_host[b].copy_(outs[b], non_blocking=True)
                ev_down[b].record(s_down)

    e2e_steps = max(4, min(args.steps, 20))
    e2e_run(2)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(s_up)
    e2e_run(e2e_steps)
    s_down.wait_stream(s_cmp)
    s_down.wait_stream(s_up)
    e1.record(s_down)
    barrier()
    ms_e2e = e0.elapsed_time(e1) / e2e_steps

    t = torch.tensor([ms_total, ms_e2e, flops], dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        ms_total, ms_e2e, flops_all = float(tmax[0]), float(tmax[1]), float(tsum[2])
    else:
        flops_all = flops
    ms_step = ms_total / args.steps

    if rank == 0:
        peaks = load_peaks()
        tflops = flops_all / (ms_step * 1e-3) / 1e12
        per_gpu = flops / (ms_step * 1e-3) / 1e12
        if args.workload == "c5":
            gbs = wl["alg_bytes"] / (ms_step * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"], "traffic": args.traffic, "peak_source": peaks["source"]}
        elif wl["kind"] in ("bf16", "bf16_backward"):
            roof = {"bound": "tensor", "achieved": per_gpu, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": per_gpu / peaks["bf16_tflops"], "traffic": args.traffic,
                    "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
                    "frac_of_sustained": per_gpu / peaks["bf16_tflops_sustained"]}
        else:
            fp8_peak = fp8_peak_tflops()
            roof = {"bound": "tensor", "achieved": per_gpu, "peak": fp8_peak, "unit": "TFLOP/s",
                    "frac": per_gpu / fp8_peak, "traffic": args.traffic,
                    "peak_source": "measured in this run (torch._scaled_mm e4m3 8192^3, best of 10)"}
        cpu_rows = 1024 if M // G >= 1024 else max(8, M // G)
        cpu_tf, cpu_t, cpu_M = cpu_loop_tflops(min(G, 8), N, K, cpu_rows, repeats=3)
        dtype = {"bf16": "bf16", "bf16_backward": "bf16", "fp8_rowwise": "fp8_e4m3", "fp8_blockwise": "fp8_e4m3"}[wl["kind"]]
        line = {
            "metric": "grouped_gemm_tflops", "value": tflops, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": f"{args.workload}: grouped GEMM {wl['kind']} G={G} K={K} N={N} M={M} per GPU, "
                                   f"{wl['m_desc']}, epilogue {wl['epilogue']}",
                       "cta_group": args.cta_group or "auto",
                       "l2": f"operands {wl['alg_bytes'] >> 20} MiB per step > 126 MiB L2",
                       "sharding": "experts across ranks, no exchange" if world > 1 else "single GPU"},
            "roofline": roof,
            "cpu_baseline": {"value": cpu_tf, "unit": "TFLOPS", "cores": torch.get_num_threads(), "kind": "reference",
                             "sample": f"{cpu_rows} rows of each of {min(G, 8)} groups ({cpu_M} rows), fp32 torch "
                                       f"per-expert loop, median of 3, {cpu_t:.2f} s each"},
            "e2e": {"value": flops_all / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOPS",
                    "h2d_bytes_per_step": wl["act_bytes"] + G * 4, "d2h_bytes_per_step": M * wl["n_out"] * 2,
                    "ms_per_step": ms_e2e,
                    "note": "every step: activations (+scales) and m_sizes from pinned host memory, result to pinned host "
                            "memory; weights resident; uploads, compute and downloads of consecutive steps overlap "
                            "(3 streams, 2 buffer sets)"},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if vendor is not None:
            line["vendor_baseline"] = vendor
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


LAYERS = {
    # name: (T tokens global, H, I, E, k, mode)
    "c3": (4096, 4096, 14336, 8, 2, "bf16"),            # Mixtral-8x7B FFN layer shapes, 1 GPU
    "c4": (32768, 7168, 2048, 256, 8, "fp8_blockwise"),  # DeepSeek-V3 routed-expert layer shapes, expert parallel
    # what ONE rank computes in c4 at 8-way expert parallelism (32 experts, 32768 routed rows), without the exchange
    "c4_rank8": (4096, 7168, 2048, 32, 8, "fp8_blockwise"),
}


def run_layer(args):
    """MoE layer throughput in tokens/s: route -> (dispatch all-to-all) -> gate+up GEMM with
    SwiGLU -> down GEMM -> (return all-to-all) -> weighted top-k combine.  The token count is
    fixed (strong scaling): each of N ranks holds T/N tokens and E/N experts."""
    import applied_ai_b200 as B
    from applied_ai_b200 import _lib
    from applied_ai_b200.ep import CudaOps, ExpertParallelMoE

    rank, world, local = dist_env()
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_DEBUG", "WARN")  # keep NCCL's version banner off stdout
        dist.init_process_group("nccl", device_id=dev)
    _lib.load(build_if_missing=False)
    B.set_default_check(False)
    T, H, I, E, k, mode = LAYERS[args.workload]
    if args.workload in ("c3", "c4_rank8") and world > 1:
        raise SystemExit(f"{args.workload} is a single-GPU workload")
    t_loc, e_loc = T // world, E // world

    # routing from one global seeded draw (identical on every rank), tokens and weights per owner
    g = torch.Generator().manual_seed(1002 if args.workload == "c3" else 1003)
    score = torch.softmax(torch.randn(T, E, generator=g), dim=-1)
    topk_w, topk_ids = torch.topk(score, k)
    sl = slice(rank * t_loc, (rank + 1) * t_loc)
    topk_w, topk_ids = topk_w[sl].to(dev), topk_ids[sl].to(torch.int32).to(dev)
    gd = torch.Generator(device=dev).manual_seed(5000 + rank)
    hidden = torch.randn(t_loc, H, generator=gd, device=dev).to(torch.bfloat16)
    w1 = torch.empty(e_loc, 2 * I, H, dtype=torch.bfloat16, device=dev)
    w2 = torch.empty(e_loc, H, I, dtype=torch.bfloat16, device=dev)
    for e in range(e_loc):
        w1[e] = (torch.randn(2 * I, H, generator=gd, device=dev) * H ** -0.5).to(torch.bfloat16)
        w2[e] = (torch.randn(H, I, generator=gd, device=dev) * I ** -0.5).to(torch.bfloat16)
    ops = CudaOps(w1, w2, mode=mode, cta_group=args.cta_group, fuse_requant=args.fuse_requant)
    if mode != "bf16":
        del w1, w2
    layer = ExpertParallelMoE(ops, E, waves=args.waves, exchange=args.exchange, max_tokens=t_loc, top_k=k,
                              hidden_size=H, capacity_factor=1.25)

    def step(h=hidden):
        return layer(h, topk_w, topk_ids)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    out = step()
    torch.cuda.synchronize()
    status = int(B.groupgemm._status_word(dev).item())
    assert status == 0, f"device status {status}"
    assert bool(torch.isfinite(out.float()).all())
    phase_ms = None
    if layer.peer is not None:
        step()
        layer.profile = True
        step()
        layer.profile = False
        phase_ms = {name: round(ms, 3) for name, ms in layer.timings}

    if world == 1 and rank == 0:
        # parity guard: a few tokens through the host restatement of the same layer
        from oracle import grouped as O
        pick = torch.tensor([0, t_loc // 2, t_loc - 1])
        hp = hidden[pick.to(dev)].cpu()
        ids_p, w_p = topk_ids[pick.to(dev)].cpu(), topk_w[pick.to(dev)].cpu()
        ref = torch.zeros(len(pick), H)
        for i in range(len(pick)):
            for j in range(k):
                e = int(ids_p[i, j])
                if mode == "bf16":
                    hcur = O.silu_and_mul_ref(hp[i:i + 1].float() @ ops.w1[e].cpu().float().T)
                    hcur = hcur.to(torch.bfloat16).float()
                    ye = hcur @ ops.w2[e].cpu().float().T
                else:
                    xq, xs = O.quant_1x128_ref(hp[i:i + 1])
                    one = torch.tensor([1], dtype=torch.int32)
                    h1 = O.silu_and_mul_ref(O.grouped_gemm_fp8_blockwise_ref(
                        xq, ops.w1[e].cpu()[None], one, xs, ops.w1_scale[e].cpu()[None]))
                    hq, hs = O.quant_1x128_ref(h1 if ops.fuse_requant else h1.to(torch.bfloat16))
                    ye = O.grouped_gemm_fp8_blockwise_ref(hq, ops.w2[e].cpu()[None], one, hs,
                                                          ops.w2_scale[e].cpu()[None])
                ref[i] += float(w_p[i, j]) * ye.to(torch.bfloat16).float()[0]
        err = O.rel_err(out[pick.to(dev)].cpu().float(), ref)
        assert err <= (1e-2 if mode == "bf16" else 2e-2), f"bench output fails parity: {err}"

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid))
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    launches0 = _lib.launch_count()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    launches = _lib.launch_count() - launches0   # this rank's kernels of this library inside the timed region
    barrier()
    t_wall1 = time.time()
    ms_total = ev0.elapsed_time(ev1)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None

    # end to end: this rank's tokens from pinned host memory, the layer, its output back to the host
    h_host = hidden.cpu().pin_memory()
    h_dev = torch.empty_like(hidden)
    o_host = torch.empty((t_loc, H), dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        h_dev.copy_(h_host, non_blocking=True)
        o_host.copy_(step(h_dev), non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1) / e2e_steps

    t = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step, ms_e2e = float(t[0]) / args.steps, float(t[1])

    if rank == 0:
        peaks = load_peaks()
        flops = 2.0 * T * k * (2 * I * H + H * I)            # all ranks
        per_gpu = flops / world / (ms_step * 1e-3) / 1e12
        if mode == "bf16":
            peak, src = peaks["bf16_tflops"], peaks["source"] + " (burst cuBLAS bf16)"
        else:
            peak, src = fp8_peak_tflops(), "measured in this run (torch._scaled_mm e4m3 8192^3, best of 10)"
        # CPU baseline: the reference's torch_moe procedure (test_moe_gemm.py:16-30) on a token sample
        from oracle import grouped as O
        torch.set_num_threads(os.cpu_count() or 1)
        ns, es = 64, min(E, 8)
        gs = torch.Generator().manual_seed(9)
        a = torch.randn(ns, H, generator=gs)
        cw1 = torch.randn(es, 2 * I, H, generator=gs) * H ** -0.5
        cw2 = torch.randn(es, H, I, generator=gs) * I ** -0.5
        cs = torch.softmax(torch.randn(ns, es, generator=gs), -1)
        ctw, cids = torch.topk(cs, min(k, es))
        O.torch_moe_ref(a[:8], cw1, cw2, ctw[:8], cids[:8])
        t0 = time.perf_counter()
        O.torch_moe_ref(a, cw1, cw2, ctw, cids)
        cpu_s = time.perf_counter() - t0
        line = {
            "metric": "moe_layer_tokens_per_s", "value": T / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if mode == "bf16" else "fp8_e4m3",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: MoE FFN layer T={T} H={H} I={I} E={E} top-{k} {mode}, "
                                   f"{t_loc} tokens and {e_loc} experts per GPU",
                       "l2": "weights per GPU exceed the 126 MiB L2",
                       "intermediate": ("bf16" if mode == "bf16" else
                                        "e4m3 + 1x128 scales written by the gate+up GEMM's epilogue" if ops.fuse_requant
                                        else "bf16, then the separate 1x128 quantiser"),
                       "exchange": ("none (1 GPU)" if world == 1 else
                                    f"NCCL all_to_all_single (counts, payload, return), {layer.W} waves"
                                    if args.exchange == "nccl" else
                                    "peer memory: push kernel + down-GEMM stores over NVLink, 2 one-element all-reduces")},
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s",
                         "frac": per_gpu / peak, "traffic": args.traffic, "peak_source": src,
                         "note": "whole layer (route, gather, 2 GEMMs, quantise, combine, exchange) against the GEMM peak"},
            "cpu_baseline": {"value": ns / cpu_s, "unit": "tokens/s", "cores": torch.get_num_threads(),
                             "kind": "reference",
                             "sample": f"torch_moe procedure, {ns} tokens over {es} experts top-{min(k, es)}, fp32, {cpu_s:.2f} s"},
            "e2e": {"value": T / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": t_loc * H * 2,
                    "d2h_bytes_per_step": t_loc * H * 2, "ms_per_step": ms_e2e,
                    "note": "per-rank token shard from pinned host memory, output back to host; weights resident"},
            "gpu_launches": launches,
            "phase_ms_rank0": phase_ms,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def run_dense(args):
    """Dense fp16 GEMM D = A @ B^T (fp32 out) at one expert's worth of the C2 shape: this
    package's single-group mode next to the reference's own Blackwell kernel
    (launch_sm100_gemm_f16_tma, built by oracle/build_ref.py into oracle/_ref/)."""
    import ctypes
    from applied_ai_b200 import _lib, sm100_gemm as S
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    _lib.load(build_if_missing=False)
    dev = torch.device("cuda", 0)
    M, N, K = 16384, 4096, 7168
    g = torch.Generator(device=dev).manual_seed(77)
    A = torch.randn(M, K, generator=g, device=dev).to(torch.float16)
    Bm = (torch.randn(N, K, generator=g, device=dev) * K ** -0.5).to(torch.float16)
    C = torch.zeros(M, N, dtype=torch.float32, device=dev)
    flops = 2.0 * M * N * K

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps

    D = S.sm100_gemm_f16(A, Bm, C)
    from oracle import grouped as O
    pick = torch.tensor([0, M // 3, M - 1], device=dev)
    err = O.rel_err(D[pick].cpu(), A[pick].cpu().float() @ Bm.cpu().float().T)
    assert err <= 1e-3, err
    ms_ours = timed(lambda: S.sm100_gemm_f16(A, Bm, C))
    ref_info = {"unavailable": "oracle/_ref/libsm100_gemm_ref.so not built"}
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libsm100_gemm_ref.so")
    if os.path.exists(ref_path):
        ref = ctypes.CDLL(ref_path)
        fn = ref.launch_sm100_gemm_f16_tma
        fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 3 + [ctypes.c_float] * 2 + [ctypes.c_void_p]
        fn.restype = ctypes.c_int
        D2 = torch.empty_like(C)
        rc = fn(A.data_ptr(), Bm.data_ptr(), C.data_ptr(), D2.data_ptr(), M, N, K, 1.0, 0.0, None)
        torch.cuda.synchronize()
        if rc == 0:
            ms_ref = timed(lambda: fn(A.data_ptr(), Bm.data_ptr(), C.data_ptr(), D2.data_ptr(), M, N, K, 1.0, 0.0, None))
            ref_info = {"ms_per_step": ms_ref, "tflops": flops / (ms_ref * 1e-3) / 1e12,
                        "max_rel_diff_vs_ours": O.rel_err(D2[pick].cpu(), D[pick].cpu()),
                        "what": "kernels/blackwell/cute_gemm_02_tma/sm100_gemm.cu built unmodified"}
        else:
            ref_info = {"unavailable": f"reference launcher returned {rc}"}
    peaks = load_peaks()
    tf = flops / (ms_ours * 1e-3) / 1e12
    line = {"metric": "dense_gemm_tflops", "value": tf, "unit": "TFLOPS", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_ours, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"dense: D = A @ B^T, fp16 in, fp32 out, M={M} N={N} K={K}",
                       "l2": "operands 561 MiB > 126 MiB L2"},
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": tf / peaks["bf16_tflops"], "traffic": args.traffic,
                         "peak_source": peaks["source"] + " (burst cuBLAS bf16)"},
            "reference_kernel": ref_info, "gpu_launches": args.steps}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + sorted(LAYERS) + ["dense"])
    ap.add_argument("--cta-group", type=int, default=0, dest="cta_group")
    ap.add_argument("--waves", type=int, default=2,
                    help="expert-parallel layers: chunks of local experts whose exchange overlaps compute")
    ap.add_argument("--exchange", default="peer", choices=["nccl", "peer"],
                    help="expert-parallel layers: NCCL all-to-all, or remote stores into peer memory")
    ap.add_argument("--fuse-requant", action=argparse.BooleanOptionalAction, default=True, dest="fuse_requant",
                    help="FP8 layers: quantise the SwiGLU output inside the gate+up GEMM (default; "
                         "--no-fuse-requant runs the separate quantiser on a bf16 intermediate)")
    ap.add_argument("--traffic", type=float, default=None,
                    help="DRAM bytes per launch from an ncu capture, echoed into the roofline object")
    args = ap.parse_args()
    if args.traffic is None and args.cta_group == 0:
        # dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel, one launch, from the ncu
        # captures summarised under profiles/ (same workload and tiling); not measured in this run
        args.traffic = PROFILED_TRAFFIC_BYTES.get(args.workload)
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "dense":
        run_dense(args)
    elif args.workload in LAYERS:
        run_layer(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
