"""Expert-parallel exchange logic on CPU: world_size-2 (and 4) gloo ranks, with the layer's
compute steps supplied by the CPU oracle.  Checks that sharding experts over ranks gives
every rank exactly the rows the unsharded layer computes for its tokens, for bf16-style
payloads and for two-part (quantised bytes + scales) payloads."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from applied_ai_b200.ep import ExpertParallelMoE, expert_ids_from_counts
from oracle import grouped as O


class CpuRefOps:
    """Checker implementation of the layer's compute steps (fp32, oracle functions)."""

    def __init__(self, w1, w2, two_part=False):
        self.w1, self.w2, self.two_part = w1.float(), w2.float(), two_part

    def route(self, ids, num_experts):
        return O.route_ref(ids, num_experts)

    def gather(self, src, idx, div=1):
        return src[(idx.long() // div)]

    def dispatch_payloads(self, hidden):
        if not self.two_part:
            return [hidden]
        q, s = O.quant_1x128_ref(hidden)
        return [q.view(torch.uint8), s]

    def expert_ffn(self, rows, m_sizes, out_row_map=None, experts=None):
        lo, hi = experts if experts is not None else (0, self.w1.shape[0])
        x = rows[0]
        if self.two_part:
            x = rows[0].view(torch.float8_e4m3fn).float() * rows[1].repeat_interleave(128, dim=1)
        h = O.silu_and_mul_ref(O.grouped_gemm_ref(x, self.w1[lo:hi], m_sizes))
        y = O.grouped_gemm_ref(h, self.w2[lo:hi], m_sizes)
        if out_row_map is None:
            return y
        out = torch.empty_like(y)
        out[out_row_map.long()] = y
        return out

    def combine(self, y, inv_perm, topk_weights, num_tokens, top_k):
        return (y[inv_perm.long()].view(num_tokens, top_k, -1) * topk_weights.float().view(num_tokens, top_k, 1)).sum(1)


def make_problem(T, H, I, E, k, seed):
    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(T, H, generator=g)
    w1 = torch.randn(E, 2 * I, H, generator=g) * H ** -0.5
    w2 = torch.randn(E, H, I, generator=g) * I ** -0.5
    score = torch.softmax(torch.randn(T, E, generator=g), -1)
    # skew the routing so some experts (and one whole rank's worth at P=4) get few or no rows
    score[:, : E // 4] *= 0.05
    tw, ids = torch.topk(score, k)
    return hidden, w1, w2, tw, ids.to(torch.int32)


def _worker(rank, world, port, two_part, waves, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T, H, I, E, k = 64, 128, 128, 8, 2
        hidden, w1, w2, tw, ids = make_problem(T, H, I, E, k, seed=11)
        t_loc, e_loc = T // world, E // world
        sl = slice(rank * t_loc, (rank + 1) * t_loc)
        ops = CpuRefOps(w1[rank * e_loc:(rank + 1) * e_loc], w2[rank * e_loc:(rank + 1) * e_loc], two_part)
        layer = ExpertParallelMoE(ops, E, waves=waves)
        out = layer(hidden[sl], tw[sl], ids[sl])
        hid_ref = hidden
        if two_part:
            q, s = O.quant_1x128_ref(hidden)
            hid_ref = q.float() * s.repeat_interleave(128, dim=1)
        ref = O.torch_moe_ref(hid_ref, w1, w2, tw, ids)[sl]
        results[rank] = (float((out - ref).abs().max()), float(ref.abs().max()), layer.last_plan)
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


@pytest.mark.parametrize("world,two_part,waves", [(2, False, 1), (2, True, 2), (4, False, 2), (2, False, 4)])
def test_expert_parallel_matches_unsharded_layer(world, two_part, waves):
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), two_part, waves, results), nprocs=world, join=True)
    assert len(results) == world
    sent = 0
    for r in range(world):
        err, scale, plan = results[r]
        assert err <= 1e-4 * scale, (r, err, scale)
        assert len(plan["send_splits"]) == world and len(plan["recv_splits"]) == world
        sent += sum(plan["send_splits"])
    assert sent == 64 * 2  # every routed row travelled exactly once
    # what rank a sends to rank b is what b receives from a
    for a in range(world):
        for b in range(world):
            assert results[a][2]["send_splits"][b] == results[b][2]["recv_splits"][a]


def test_single_process_layer_needs_no_process_group():
    hidden, w1, w2, tw, ids = make_problem(32, 128, 128, 4, 2, seed=3)
    layer = ExpertParallelMoE(CpuRefOps(w1, w2), 4)
    assert layer.P == 1
    out = layer(hidden, tw, ids)
    ref = O.torch_moe_ref(hidden, w1, w2, tw, ids)
    assert float((out - ref).abs().max()) <= 1e-4 * float(ref.abs().max())


def test_expert_ids_from_counts():
    counts = torch.tensor([[2, 0, 1], [0, 3, 1]])
    assert expert_ids_from_counts(counts, 7).tolist() == [0, 0, 2, 1, 1, 1, 2]
