"""Expert-parallel layer on GPUs: the single-rank layer against the oracle and against
fused_moe, and (as far as GPUs are visible) 2, 4 and 8 NCCL ranks against one."""
import os
import socket

import pytest
import torch

import applied_ai_b200 as B
from applied_ai_b200 import _lib
from applied_ai_b200.ep import CudaOps, ExpertParallelMoE
from oracle import grouped as O
from tests.helpers import BF16_REL_TOL, FP8_REL_TOL

pytestmark = pytest.mark.gpu


def problem(T, H, I, E, k, seed):
    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * H ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * I ** -0.5).to(torch.bfloat16)
    tw, ids = torch.topk(torch.softmax(torch.randn(T, E, generator=g), -1), k)
    return hidden, w1, w2, tw, ids.to(torch.int32)


def test_single_rank_bf16_equals_fused_moe():
    hidden, w1, w2, tw, ids = problem(300, 256, 384, 8, 2, 1)
    d = "cuda"
    layer = ExpertParallelMoE(CudaOps(w1.to(d), w2.to(d), "bf16"), 8)
    out = layer(hidden.to(d), tw.to(d), ids.to(d))
    assert torch.equal(out, B.fused_moe(hidden.to(d), w1.to(d), w2.to(d), tw.to(d), ids.to(d)))
    assert O.rel_err(out.cpu().float(), O.torch_moe_ref(hidden, w1, w2, tw, ids)) <= BF16_REL_TOL


def fp8_layer_reference(hidden, ops, tw, ids):
    """The layer on the same quantised operands: 1x128-quantised tokens, block-quantised
    weights, intermediate quantised 1x128 again (from fp32) before the down GEMM."""
    E = ops.w1.shape[0]
    xq, xs = O.quant_1x128_ref(hidden)
    T, k = ids.shape
    out = torch.zeros(T, ops.w2.shape[1])
    w1, s1, w2, s2 = ops.w1.cpu(), ops.w1_scale.cpu(), ops.w2.cpu(), ops.w2_scale.cpu()
    for e in range(E):
        for j in range(k):
            rows = torch.nonzero(ids[:, j] == e).reshape(-1)
            if rows.numel() == 0:
                continue
            m = torch.tensor([rows.numel()], dtype=torch.int32)
            h = O.silu_and_mul_ref(O.grouped_gemm_fp8_blockwise_ref(xq[rows], w1[e][None], m, xs[rows], s1[e][None]))
            hq, hs = O.quant_1x128_ref(h.to(torch.bfloat16) if not ops.fuse_requant else h)
            y = O.grouped_gemm_fp8_blockwise_ref(hq, w2[e][None], m, hs, s2[e][None]).to(torch.bfloat16).float()
            out[rows] += tw[rows, j:j + 1].float() * y
    return out


@pytest.mark.parametrize("fuse", [False, True])
def test_single_rank_fp8_blockwise_layer(fuse):
    hidden, w1, w2, tw, ids = problem(200, 256, 256, 4, 2, 2)
    d = "cuda"
    ops = CudaOps(w1.to(d), w2.to(d), "fp8_blockwise", fuse_requant=fuse)
    out = ExpertParallelMoE(ops, 4)(hidden.to(d), tw.to(d), ids.to(d))
    ref = fp8_layer_reference(hidden, ops, tw, ids)
    assert O.rel_err(out.cpu().float(), ref) <= FP8_REL_TOL


def _worker(rank, world, port, mode, waves, ret, exchange="nccl", skew=False):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    d = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=d)
    try:
        T, H, I, E, k = PROBLEM
        hidden, w1, w2, tw, ids = problem(T, H, I, E, k, 3)
        tl, el = T // world, E // world
        sl = slice(rank * tl, (rank + 1) * tl)
        ops = CudaOps(w1[rank * el:(rank + 1) * el].to(d), w2[rank * el:(rank + 1) * el].to(d), mode, cta_group=2)
        layer = ExpertParallelMoE(ops, E, waves=waves, exchange=exchange, max_tokens=tl, top_k=k, hidden_size=H)
        out = layer(hidden[sl].to(d), tw[sl].to(d), ids[sl].to(d))
        if exchange == "peer":   # the shared buffers are reused from call to call
            if skew:
                # every token of every rank to the experts of rank 0: it would receive `world` times
                # the rows it sends, more than its buffer holds.  Nothing faults: surplus rows are
                # dropped, the status word says so, and the next ordinary call is unaffected.
                ids_skew = (ids[sl] % el).to(d)
                bad = layer(hidden[sl].to(d), tw[sl].to(d), ids_skew)
                assert bool(torch.isfinite(bad.float()).all())
                raised = False
                try:
                    layer.raise_on_status()
                except _lib.B200MoeError as exc:
                    raised = "receive buffer" in str(exc)
                ret[f"raised{rank}"] = raised
                layer.raise_on_status()          # the word was cleared by the first read
            out2 = layer(hidden[sl].to(d), tw[sl].to(d), ids[sl].to(d))
            assert torch.equal(out, out2)
            layer.raise_on_status()
        torch.cuda.synchronize()
        ret[rank] = out.cpu()
    finally:
        dist.destroy_process_group()


PROBLEM = (512, 256, 256, 8, 2)   # T, H, I, E, top-k
WORLDS = [2, 4, 8]


def _run_ranks(world, mode, waves, exchange, skew=False):
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, mode, waves, ret, exchange, skew), nprocs=world, join=True)
    return ret


def _one_rank(mode):
    T, H, I, E, k = PROBLEM
    hidden, w1, w2, tw, ids = problem(T, H, I, E, k, 3)
    d = "cuda"
    return ExpertParallelMoE(CudaOps(w1.to(d), w2.to(d), mode, cta_group=2), E)(hidden.to(d), tw.to(d), ids.to(d)).cpu()


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("mode,waves", [("bf16", 1), ("fp8_blockwise", 2), ("bf16", 4)])
def test_ranks_equal_one_rank_bit_for_bit(world, mode, waves):
    """NCCL all-to-all exchange: 2, 4 and 8 ranks give the bits of the single-rank layer."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ret = _run_ranks(world, mode, waves, "nccl")
    assert torch.equal(_one_rank(mode), torch.cat([ret[r] for r in range(world)]))


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("mode", ["bf16", "fp8_blockwise"])
def test_peer_memory_exchange_equals_one_rank_bit_for_bit(world, mode):
    """Dispatch by remote stores and return inside the down GEMM's store, against the single-rank layer."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ret = _run_ranks(world, mode, 1, "peer")
    assert torch.equal(_one_rank(mode), torch.cat([ret[r] for r in range(world)]))


@pytest.mark.parametrize("world", [2, 4])
def test_peer_exchange_capacity_overflow_is_reported_not_silent(world):
    """Routing skew beyond the receive capacity: rows are dropped without any out-of-bounds access, the
    deferred check raises on every rank, and the layer keeps working afterwards."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ret = _run_ranks(world, "bf16", 1, "peer", skew=True)
    assert all(ret[f"raised{r}"] for r in range(world))
    assert torch.equal(_one_rank("bf16"), torch.cat([ret[r] for r in range(world)]))


def test_ep_plan_reports_overflow_and_clamps_the_owner_sizes():
    """b200moe_ep_plan through the C ABI on one GPU: counts that exceed the capacity of rank 0."""
    lib = _lib.load()
    P, E, cap = 2, 4, 100
    counts = torch.tensor([[60, 30, 5, 5], [40, 20, 5, 5]], dtype=torch.int32, device="cuda")   # rank 0 would get 150
    for me, want_m in ((0, [100, 0]), (1, [10, 10])):
        dst = torch.full((E,), -1, dtype=torch.int32, device="cuda")
        m_loc = torch.full((E // P,), -1, dtype=torch.int32, device="cuda")
        word = torch.zeros(1, dtype=torch.int32, device="cuda")
        rc = lib.b200moe_ep_plan(counts.data_ptr(), P, E, me, cap, dst.data_ptr(), m_loc.data_ptr(), word.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert int(word.item()) == 24
        assert m_loc.tolist() == want_m
        # first row of my rows per global expert: rows of lower ranks come first inside an expert
        assert dst.tolist() == ([0, 100, 0, 10] if me == 0 else [60, 130, 5, 15])
