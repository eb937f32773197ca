"""Device-side waits are bounded: a wait that nothing satisfies ends with a status code,
not a hang, and the context keeps working.  No GPU fault, trap or endless loop is used."""
import time

import pytest
import torch

import applied_ai_b200 as B
from applied_ai_b200 import _lib
from oracle import grouped as O

pytestmark = pytest.mark.gpu


def test_unsatisfied_wait_returns_status_and_context_survives():
    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.time()
    rc = lib.b200moe_selftest_wait_timeout(50_000_000, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    dt = time.time() - t0
    assert int(status.item()) == 20
    assert 0.04 <= dt < 2.0, dt            # it waited for its 50 ms limit, then gave up by itself
    assert "expected" in _lib.describe_status(20)
    # same context, next launch: a real grouped GEMM still works and is right
    g = torch.Generator().manual_seed(0)
    x = torch.randn(200, 64, generator=g).to(torch.bfloat16)
    w = torch.randn(2 * 64, 64, generator=g).to(torch.bfloat16)
    m = torch.tensor([120, 80], dtype=torch.int32)
    y = B.grouped_gemm(x.cuda(), w.cuda(), m.cuda())
    assert O.rel_err(y.cpu().float(), O.grouped_gemm_ref(x, w, m)) <= 1e-2


def test_selftest_rejects_unbounded_limits():
    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.b200moe_selftest_wait_timeout(0, status.data_ptr(), None) == -1
    assert lib.b200moe_selftest_wait_timeout(10_000_000_000, status.data_ptr(), None) == -1
    assert lib.b200moe_selftest_wait_timeout(1000, None, None) == -1


def test_stream_barrier_gives_up_on_a_peer_that_never_signals():
    """b200moe_ep_barrier with two 'ranks' whose flag blocks both live on this GPU: rank 0 signals both and
    finds its own flag, but nobody plays rank 1, so that wait runs into its 50 ms limit, reports status 25
    and returns.  A second call with the missing flag stored by hand passes at once."""
    lib = _lib.load()
    P = 2
    blocks = [torch.zeros(2 * P, dtype=torch.int32, device="cuda") for _ in range(P)]
    table = torch.tensor([b.data_ptr() for b in blocks], dtype=torch.int64, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.time()
    assert lib.b200moe_ep_barrier(table.data_ptr(), P, 0, 0, 1, 50_000_000, status.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    dt = time.time() - t0
    assert int(status.item()) == 25 and 0.04 <= dt < 2.0, (int(status.item()), dt)
    assert blocks[0].tolist() == [1, 0, 0, 0] and blocks[1].tolist() == [1, 0, 0, 0]   # word [slot 0][rank 0] of both
    assert "peer" in _lib.describe_status(25)
    status.zero_()
    blocks[0][1] = 2                      # "rank 1" has signalled epoch 2 already (a peer may be one step ahead)
    assert lib.b200moe_ep_barrier(table.data_ptr(), P, 0, 0, 2, 50_000_000, status.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # bad arguments are refused on the host
    assert lib.b200moe_ep_barrier(table.data_ptr(), P, 2, 0, 1, 50_000_000, status.data_ptr(), stream) == -1
    assert lib.b200moe_ep_barrier(table.data_ptr(), P, 0, 0, 1, 0, status.data_ptr(), stream) == -1


def test_tmem_read_probe_reports_a_plausible_rate():
    """The diagnostic runs, leaves the context usable and reports a rate between 16 B/clk (one lane quadrant
    crawling) and 4 KiB/clk (more than the MMA itself moves) per SM."""
    from applied_ai_b200.selftest import tmem_read_rate
    for warps, in_flight in ((4, 1), (8, 2)):
        r = tmem_read_rate(warps, in_flight, iters=50, ctas=4)
        assert 16.0 < r < 4096.0
    with pytest.raises(Exception):
        tmem_read_rate(warps=3)
    assert torch.ones(4, device="cuda").sum().item() == 4.0


def test_two_host_threads_on_their_own_streams_get_the_serial_results():
    """The entry points keep no state that two callers could share by accident: two Python threads, each on its
    own stream and with its own shapes (bf16 forward, backward, block-wise FP8 with a bad-size call in between),
    produce bit for bit what the same calls produce one after another, and the bad call of one thread does not
    show up in the other thread's status word."""
    import threading
    from applied_ai_b200.tgroup_gemm_backwards import grouped_gemm_backward

    def inputs(seed, G, M, N, K):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(G, N, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
        dy = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
        m = torch.full((G,), M // G - 3, dtype=torch.int32).cuda()
        return x, w, dy, m

    def work(args, bad):
        x, w, dy, m = args
        out = []
        rows = int(m.sum())
        for it in range(6):
            out.append(B.grouped_gemm(x, w, m)[:rows])  # (rows past sum(m_sizes) are not written: torch.empty)
            out.extend(grouped_gemm_backward(dy, x, w, m))
            if bad and it == 2:
                with pytest.raises(ValueError):
                    B.grouped_gemm(x, w, torch.full_like(m, x.shape[0]))  # sum(m_sizes) > M
        torch.cuda.current_stream().synchronize()
        return out

    cases = [(inputs(71, 4, 1024, 512, 256), True), (inputs(72, 6, 1536, 384, 640), False)]
    serial = [work(a, bad) for a, bad in cases]
    results, errors = [None, None], []

    def runner(i):
        try:
            with torch.cuda.stream(torch.cuda.Stream()):
                results[i] = work(*cases[i])
        except Exception as e:  # noqa: BLE001 - reported below
            errors.append(e)

    threads = [threading.Thread(target=runner, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not errors, errors
    for got, want in zip(results, serial):
        assert got is not None and len(got) == len(want)
        for a, b in zip(got, want):
            assert torch.equal(a, b)
    assert B.pending_status() is None
