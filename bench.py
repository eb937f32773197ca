"""Benchmark of the MoE grouped-GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default run (workload "c2"): the headline metric is the bf16 grouped GEMM at the DeepSeek-V3
routed-expert gate+up shape — G=8 experts, K=7168, N=4096, 16384 rows, group sizes multiples of
128, seeded synthetic data.  One step = one grouped GEMM over the whole batch.  Metric: TFLOPS
(2*M*N*K / time).  With N > 1 GPUs every rank holds its own 8 experts and 16384 rows (replicas:
this GEMM has no exchange step) and the value is the sum over ranks.

The same JSON line carries, measured in the same run:
  "sustained"  the same GEMM back to back for at least two seconds (the rate under the power cap),
  "also"       the other single-GPU workloads (FP8 row-wise / block-wise, the DeepSeek-V3 per-rank
               GEMM shapes, the skewed-routing case, the Mixtral layer, the backward), N = 1 only,
  "ep_layer"   the expert-parallel DeepSeek-V3 MoE layer (FP8 block-wise, 32768 tokens top-8 over 256
               experts) on the N GPUs of this run: experts and tokens sharded over the ranks, dispatch
               and return through peer memory and, separately, through NCCL all-to-all, each with a
               per-rank parity check against the CPU restatement of the layer.

Prints ONE JSON line (rank 0).  `--impl reference` times the reference's own ground truth for this
path — the torch per-expert matmul loop on the host CPU cores — on a bounded sample of the workload.
"""
import argparse
import datetime
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
LAYERS = {
    # name: (T tokens global, H, I, E, k, mode)
    "c3": (4096, 4096, 14336, 8, 2, "bf16"),            # Mixtral-8x7B FFN layer shapes, 1 GPU
    "c4": (32768, 7168, 2048, 256, 8, "fp8_blockwise"),  # DeepSeek-V3 routed-expert layer shapes, expert parallel
    # what ONE rank computes in c4 at 8-way expert parallelism (32 experts, 32768 routed rows), without the exchange
    "c4_rank8": (4096, 7168, 2048, 32, 8, "fp8_blockwise"),
}
ALSO_DEFAULT = ["c2_fp8_blockwise", "c2_fp8_rowwise", "c4_gate_up", "c4_down", "c5", "c3", "c4_rank8", "c2_backward"]
# rows of each group in the CPU sample that both the in-line cpu_baseline and `--impl reference` time
CPU_SAMPLE_ROWS_PER_GROUP = 256


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        d = json.load(open(path))
        return {"bf16_tflops": float(d["bf16_tflops"]), "bf16_tflops_sustained": float(d["bf16_tflops_sustained"]),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    except Exception:
        return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock, power and throttle reasons with nvidia-smi from start() to stop(); window(t0, t1)
    summarises the samples taken between two wall-clock times."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_id):
        self.rows, self.proc, self.thread = [], None, None
        self.gpu_id = gpu_id

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_id), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()

    def window(self, t0, t1, slack=0.03):
        sm, power, smax, reasons = [], [], None, set()
        for t, line in list(self.rows):
            if not (t0 - slack <= t <= t1 + slack):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(self.NAMES, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power) if power else None}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def numa_cpus_of_gpu(dev):
    """CPUs of the NUMA node the GPU's PCIe slot hangs off that this process may run on, or None."""
    try:
        p = torch.cuda.get_device_properties(dev)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read())
        if node < 0:
            return None, None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        return (cpus or None), node
    except Exception:
        return None, None


class numa_local:
    """While active, the calling thread runs on the GPU's NUMA node, so that host buffers allocated and
    first touched inside land in that node's memory."""

    def __init__(self, dev):
        self.cpus, self.node = numa_cpus_of_gpu(dev)
        self.saved = None

    def __enter__(self):
        if self.cpus:
            try:
                self.saved = os.sched_getaffinity(0)
                os.sched_setaffinity(0, self.cpus)
            except OSError:
                self.saved = None
        return self

    def __exit__(self, *exc):
        if self.saved is not None:
            os.sched_setaffinity(0, self.saved)


def pinned_copy(t):
    h = torch.empty(t.shape, dtype=t.dtype).pin_memory()
    h.copy_(t)
    return h


# ------------------------------------------------------------------ CPU baseline (the port of the reference loop)

def cpu_sample(G, N, K):
    """Inputs of the CPU sample: CPU_SAMPLE_ROWS_PER_GROUP rows of each of (at most 8) groups, full N and K."""
    G = min(G, 8)
    rows = CPU_SAMPLE_ROWS_PER_GROUP
    g = torch.Generator().manual_seed(1001)
    x = torch.randn(G * rows, K, generator=g).to(torch.bfloat16).float()
    w = (torch.randn(G, N, K, generator=g) * K ** -0.5).to(torch.bfloat16).float()
    return x, w, torch.full((G,), rows, dtype=torch.int32), G, rows


def cpu_loop_tflops(G, N, K, seconds=10.0, max_repeats=200):
    """The reference's per-expert loop (dev/triton_groupGEMM/testing/base_testing.py:125-131) in fp32 on the
    host cores over the CPU sample; repeated for about `seconds`, median step time."""
    from oracle import grouped as O
    torch.set_num_threads(os.cpu_count() or 1)
    x, w, m_sizes, Gs, rows = cpu_sample(G, N, K)
    O.grouped_gemm_ref(x, w, m_sizes)  # touch pages, spin up threads
    times, t_start = [], time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_start < seconds and len(times) < max_repeats):
        t0 = time.perf_counter()
        O.grouped_gemm_ref(x, w, m_sizes)
        times.append(time.perf_counter() - t0)
    times.sort()
    t = times[len(times) // 2]
    sample = (f"{rows} rows of each of {Gs} groups ({Gs * rows} rows), full N and K, fp32 torch per-expert loop, "
              f"median of {len(times)} runs, {t:.3f} s each")
    return 2.0 * Gs * rows * N * K / t / 1e12, sample


def cpu_layer_tokens_per_s(H, I, E, k, repeats=1):
    """The reference's `torch_moe` procedure (kernels/triton/inference/col_major_moe_gemm/test_moe_gemm.py:16-30)
    in fp32 on the host cores, on a 64-token sample over at most 8 experts."""
    from oracle import grouped as O
    torch.set_num_threads(os.cpu_count() or 1)
    ns, es = 64, min(E, 8)
    g = torch.Generator().manual_seed(9)
    a = torch.randn(ns, H, generator=g)
    w1 = torch.randn(es, 2 * I, H, generator=g) * H ** -0.5
    w2 = torch.randn(es, H, I, generator=g) * I ** -0.5
    tw, ids = torch.topk(torch.softmax(torch.randn(ns, es, generator=g), -1), min(k, es))
    O.torch_moe_ref(a[:8], w1, w2, tw[:8], ids[:8])
    t0 = time.perf_counter()
    for _ in range(repeats):
        O.torch_moe_ref(a, w1, w2, tw, ids)
    dt = (time.perf_counter() - t0) / repeats
    return ns / dt, dt, f"torch_moe procedure, {ns} tokens over {es} experts top-{min(k, es)}, full H and I, fp32, {dt:.2f} s"


def run_reference(args):
    """`--impl reference`: the CPU port of the reference's ground-truth loop, all host threads, rank 0 only."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from oracle import grouped as O
    if args.workload in LAYERS:
        T, H, I, E, k, mode = LAYERS[args.workload]
        v, dt, sample = cpu_layer_tokens_per_s(H, I, E, k, repeats=max(1, args.steps))
        metric, unit, cfg = "moe_layer_tokens_per_s", "tokens/s", f"{args.workload}: MoE FFN layer T={T} H={H} I={I} E={E} top-{k}"
        scaling = "strong"
    else:
        G, M, N, K = WORKLOADS[args.workload]
        torch.set_num_threads(os.cpu_count() or 1)
        x, w, m_sizes, Gs, rows = cpu_sample(G, N, K)
        for _ in range(max(1, min(args.warmup, 3))):
            O.grouped_gemm_ref(x, w, m_sizes)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            O.grouped_gemm_ref(x, w, m_sizes)
        dt = (time.perf_counter() - t0) / args.steps
        v = 2.0 * Gs * rows * N * K / dt / 1e12
        sample = f"{rows} rows of each of {Gs} groups ({Gs * rows} of {M} rows), full N and K, fp32 torch.matmul loop"
        metric, unit, cfg, scaling = "grouped_gemm_tflops", "TFLOPS", f"{args.workload}: grouped GEMM G={G} K={K} N={N} M={M}", "weak"
    line = {
        "impl": "reference", "metric": metric, "value": v, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg, "sample": sample},
        "cpu_baseline": {"value": v, "unit": unit, "cores": torch.get_num_threads(), "kind": "port", "sample": sample,
                         "note": "CPU port of the reference's ground-truth loop (its Triton kernels cannot run here)"},
        "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU helpers

_fp8_peak = None


def fp8_peak_tflops():
    """Dense FP8 tensor peak of this GPU, measured here the way the bf16 peaks were
    (library GEMM 8192^3, best of 10): torch._scaled_mm, e4m3 x e4m3 -> bf16.  Measured once per run."""
    global _fp8_peak
    if _fp8_peak is not None:
        return _fp8_peak
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
    _fp8_peak = 2.0 * n ** 3 / (best * 1e-3) / 1e12
    return _fp8_peak


FP8_PEAK_SOURCE = "measured in this run (torch._scaled_mm e4m3 8192^3, best of 10)"

# dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel, one launch, from earlier ncu captures of
# the same workload and tiling (not measured in this run; the line says so in roofline.traffic_source)
PROFILED_TRAFFIC_BYTES = {
    "c2": 1.160e9,
    "c5": 750.5e6,
    "c2_fp8_rowwise": 471.0e6,
    "c2_fp8_blockwise": 477.1e6,
}


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def reduce_max(values, dev, world):
    t = torch.tensor(values, dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


def reduce_sum(values, dev, world):
    t = torch.tensor(values, dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return [float(v) for v in t]


def time_steps(step, steps, warmup, world):
    """W untimed steps, then exactly `steps` steps between two events on the launching stream, a barrier and a
    device synchronisation on both sides.  Returns (ms total on this rank, kernels enqueued, wall t0, wall t1)."""
    from applied_ai_b200 import _lib
    for _ in range(max(warmup, 3)):
        step()
    barrier(world)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    n0 = _lib.launch_count()
    ev0.record()
    for _ in range(steps):
        step()
    ev1.record()
    launches = _lib.launch_count() - n0
    barrier(world)
    return ev0.elapsed_time(ev1), launches, t0, time.time()


def vendor_grouped_mm(wl, y_ours, iters=10):
    """The bf16 grouped GEMM of the installed torch (`torch._grouped_mm`, a library kernel) on the same
    resident inputs, as a second baseline next to the CPU loop.  Returns a dict for the JSON line; never
    raises.  The FP8 counterpart (`torch._scaled_grouped_mm`) is not called: in this torch build its kernel
    is compiled for another architecture and aborts on the device, which costs the process its context."""
    try:
        if wl["kind"] != "bf16":
            return None
        m_sizes = wl["m_sizes"]
        offs = torch.cumsum(m_sizes, 0).to(torch.int32)
        x, w = wl["x"], wl["w"]
        fn = lambda: torch._grouped_mm(x, w.transpose(-2, -1), offs=offs)
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
        return {"kind": "torch._grouped_mm", "value": wl["flops"] / (ms * 1e-3) / 1e12, "unit": "TFLOPS",
                "ms_per_step": ms, "max_rel_diff_vs_this_engine": diff,
                "note": "library kernel of the installed torch, same resident inputs"}
    except Exception as exc:  # missing op, unsupported shape or dtype on this build
        return {"kind": "torch grouped mm", "unavailable": f"{type(exc).__name__}: {str(exc)[:160]}"}


def make_workload(name, rank, dev, cta_group):
    """Builds device-resident inputs and the step function of one grouped-GEMM workload."""
    import applied_ai_b200 as B
    from applied_ai_b200 import configs
    G, M, N, K = WORKLOADS[name]
    kind = WORKLOAD_KIND[name]
    wl = {"name": name, "G": G, "M": M, "N": N, "K": K, "kind": kind, "epilogue": "none"}
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
    wl["dtype"] = {"bf16": "bf16", "bf16_backward": "bf16", "fp8_rowwise": "fp8_e4m3", "fp8_blockwise": "fp8_e4m3"}[kind]
    return wl


def parity_of_workload(wl, y, dev):
    """A sample of output rows against the host loop (two rows of up to eight groups)."""
    from oracle import grouped as O
    gsel = torch.Generator().manual_seed(7)
    start, worst, checked = 0, 0.0, 0
    ms = wl["m_sizes"].cpu()
    G = wl["G"]
    for e in range(G):
        mg = int(ms[e])
        if mg and e % max(1, G // 8) == 0:
            pick = (start + torch.randint(0, mg, (2,), generator=gsel)).to(dev)
            worst = max(worst, O.rel_err(y[pick].cpu().float(), wl["ref_rows"](pick, e)))
            checked += 2
        start += mg
    return {"max_rel_err": worst, "tol": wl["tol"], "rows_checked": checked}


def roofline_of_workload(wl, ms_step, peaks, traffic):
    per_gpu = wl["flops"] / (ms_step * 1e-3) / 1e12
    src = "ncu capture of an earlier build, same workload and tiling; not measured in this run" if traffic else None
    if wl["name"] == "c5":
        gbs = wl["alg_bytes"] / (ms_step * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": gbs / peaks["hbm_gbs"], "traffic": traffic, "traffic_source": src,
                "peak_source": peaks["source"] + " (copy bandwidth)", "algorithmic_bytes": wl["alg_bytes"]}
    if wl["kind"] in ("bf16", "bf16_backward"):
        return {"bound": "tensor", "achieved": per_gpu, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": per_gpu / peaks["bf16_tflops"], "traffic": traffic, "traffic_source": src,
                "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
                "frac_of_sustained": per_gpu / peaks["bf16_tflops_sustained"]}
    peak = fp8_peak_tflops()
    return {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu / peak,
            "traffic": traffic, "traffic_source": src, "peak_source": FP8_PEAK_SOURCE}


def also_gemm(name, dev, cta_group, steps, peaks):
    """One of the other single-GPU grouped-GEMM workloads: parity sample, then `steps` timed steps."""
    import applied_ai_b200 as B
    wl = make_workload(name, 0, dev, cta_group)
    y = wl["step"]()
    torch.cuda.synchronize()
    B.pending_status()
    par = parity_of_workload(wl, y, dev)
    del y
    ms_total, launches, _, _ = time_steps(wl["step"], steps, 3, 1)
    B.pending_status()
    ms = ms_total / steps
    res = {"value": wl["flops"] / (ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": ms, "steps": steps,
           "dtype": wl["dtype"],
           "workload": f"{wl['kind']} G={wl['G']} K={wl['K']} N={wl['N']} M={wl['M']}, {wl['m_desc']}, epilogue {wl['epilogue']}",
           "roofline": roofline_of_workload(wl, ms, peaks, PROFILED_TRAFFIC_BYTES.get(name) if cta_group == 0 else None),
           "parity": par, "gpu_launches": launches}
    assert par["max_rel_err"] <= par["tol"], f"{name} fails parity: {par}"
    return res


# ------------------------------------------------------------------ MoE layers

def expert_weights(e, H, I, dev):
    """bf16 weights of GLOBAL expert e, from a generator seeded by e alone: any rank can rebuild any expert."""
    g = torch.Generator(device=dev).manual_seed(7000 + e)
    w1 = (torch.randn(2 * I, H, generator=g, device=dev) * H ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(H, I, generator=g, device=dev) * I ** -0.5).to(torch.bfloat16)
    return w1, w2


def build_layer_ops(name, rank, world, dev, cta_group, fuse_requant):
    """This rank's expert weights (experts [rank*E/world, (rank+1)*E/world)) as the layer's compute object."""
    import applied_ai_b200 as B
    from applied_ai_b200.ep import CudaOps
    T, H, I, E, k, mode = LAYERS[name]
    e_loc = E // world
    if mode == "bf16":
        w1 = torch.empty(e_loc, 2 * I, H, dtype=torch.bfloat16, device=dev)
        w2 = torch.empty(e_loc, H, I, dtype=torch.bfloat16, device=dev)
        for i in range(e_loc):
            w1[i], w2[i] = expert_weights(rank * e_loc + i, H, I, dev)
        return CudaOps(w1, w2, mode="bf16", cta_group=cta_group)
    w1q = torch.empty(e_loc, 2 * I, H, dtype=torch.float8_e4m3fn, device=dev)
    w2q = torch.empty(e_loc, H, I, dtype=torch.float8_e4m3fn, device=dev)
    s1 = torch.empty(e_loc, 2 * I // 128, H // 128, dtype=torch.float32, device=dev)
    s2 = torch.empty(e_loc, H // 128, I // 128, dtype=torch.float32, device=dev)
    for i in range(e_loc):  # expert by expert: the bf16 originals never exist all at once
        a, b = expert_weights(rank * e_loc + i, H, I, dev)
        w1q[i], s1[i] = B.quantize_fp8_block(a)
        w2q[i], s2[i] = B.quantize_fp8_block(b)
    return CudaOps.from_quantized(w1q, s1, w2q, s2, cta_group=cta_group, fuse_requant=fuse_requant)


def layer_inputs(name, rank, world, dev):
    """Routing from one global seeded draw (identical on every rank); this rank's slice of tokens."""
    T, H, I, E, k, mode = LAYERS[name]
    t_loc = T // world
    g = torch.Generator().manual_seed(1002 if name == "c3" else 1003)
    score = torch.softmax(torch.randn(T, E, generator=g), dim=-1)
    topk_w, topk_ids = torch.topk(score, k)
    sl = slice(rank * t_loc, (rank + 1) * t_loc)
    gd = torch.Generator(device=dev).manual_seed(5000 + rank)
    hidden = torch.randn(t_loc, H, generator=gd, device=dev).to(torch.bfloat16)
    return hidden, topk_w[sl].to(dev), topk_ids[sl].to(torch.int32).to(dev)


def layer_parity(name, ops, out, hidden, topk_w, topk_ids, rank, world, dev, n_tokens=2):
    """`n_tokens` of THIS rank's tokens through the CPU restatement of the layer on the same quantised
    operands.  The experts a token visits may live on other ranks: their weights are rebuilt here from the
    per-expert seed and quantised by the same code."""
    import applied_ai_b200 as B
    from oracle import grouped as O
    T, H, I, E, k, mode = LAYERS[name]
    t_loc = hidden.shape[0]
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // max(1, world)))
    pick = torch.linspace(0, t_loc - 1, n_tokens).long()
    hp = hidden[pick.to(dev)].cpu()
    ids_p, w_p = topk_ids[pick.to(dev)].cpu(), topk_w[pick.to(dev)].cpu()
    ref = torch.zeros(len(pick), H)
    one = torch.tensor([1], dtype=torch.int32)
    cache = {}
    for i in range(len(pick)):
        for j in range(k):
            e = int(ids_p[i, j])
            if e not in cache:
                a, b = expert_weights(e, H, I, dev)
                if mode == "bf16":
                    cache[e] = (a.cpu().float(), b.cpu().float())
                else:
                    (aq, as_), (bq, bs) = B.quantize_fp8_block(a), B.quantize_fp8_block(b)
                    cache[e] = (aq.cpu(), as_.cpu(), bq.cpu(), bs.cpu())
                del a, b
            if mode == "bf16":
                w1f, w2f = cache[e]
                hcur = O.silu_and_mul_ref(hp[i:i + 1].float() @ w1f.T).to(torch.bfloat16).float()
                ye = hcur @ w2f.T
            else:
                aq, as_, bq, bs = cache[e]
                xq, xs = O.quant_1x128_ref(hp[i:i + 1])
                h1 = O.silu_and_mul_ref(O.grouped_gemm_fp8_blockwise_ref(xq, aq[None], one, xs, as_[None]))
                hq, hs = O.quant_1x128_ref(h1 if ops.fuse_requant else h1.to(torch.bfloat16))
                ye = O.grouped_gemm_fp8_blockwise_ref(hq, bq[None], one, hs, bs[None])
            ref[i] += float(w_p[i, j]) * ye.to(torch.bfloat16).float()[0]
    err = O.rel_err(out[pick.to(dev)].cpu().float(), ref)
    return err, len(pick)


def measure_layer(name, exchange, ops, rank, world, dev, args, steps, parity_tokens=2):
    """Times one MoE layer configuration on the ranks of this run.  Returns (dict for the JSON line, output of
    one step).  Every rank checks some of its own tokens against the CPU restatement before the timed steps,
    and the status words are read again after them."""
    import applied_ai_b200 as B
    from applied_ai_b200.ep import ExpertParallelMoE
    T, H, I, E, k, mode = LAYERS[name]
    t_loc, e_loc = T // world, E // world
    hidden, topk_w, topk_ids = layer_inputs(name, rank, world, dev)
    layer = ExpertParallelMoE(ops, E, waves=args.waves, exchange=exchange, max_tokens=t_loc, top_k=k,
                              hidden_size=H, capacity_factor=1.25)

    def step(h=hidden):
        return layer(h, topk_w, topk_ids)

    out = step()
    torch.cuda.synchronize()
    layer.raise_on_status()
    err, n_checked = layer_parity(name, ops, out, hidden, topk_w, topk_ids, rank, world, dev, parity_tokens)
    tol = 1e-2 if mode == "bf16" else 2e-2
    finite = float(bool(torch.isfinite(out.float()).all()))
    err_all = reduce_max([err, 1.0 - finite], dev, world)
    phase_ms = None
    if layer.peer is not None:
        step()
        layer.profile = True
        step()
        layer.profile = False
        phase_ms = {pname: round(ms, 3) for pname, ms in layer.timings}

    ms_total, launches, _, _ = time_steps(step, steps, args.warmup, world)
    status_ok = 1.0
    try:
        layer.raise_on_status()
    except Exception:
        status_ok = 0.0

    # end to end: this rank's tokens from pinned host memory, the layer, its output back to the host
    with numa_local(dev):
        h_host = pinned_copy(hidden.cpu())
        o_host = torch.empty((t_loc, H), dtype=torch.bfloat16).pin_memory()
        o_host.zero_()
    h_dev = torch.empty_like(hidden)

    def e2e_step():
        h_dev.copy_(h_host, non_blocking=True)
        o_host.copy_(step(h_dev), non_blocking=True)

    e2e_steps = max(3, min(steps, 10))
    for _ in range(2):
        e2e_step()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier(world)
    ms_step, ms_e2e, bad_status = reduce_max([ms_total / steps, e0.elapsed_time(e1) / e2e_steps, 1.0 - status_ok], dev, world)

    flops = 2.0 * T * k * (2 * I * H + H * I)            # all ranks
    per_gpu = flops / world / (ms_step * 1e-3) / 1e12
    peaks = load_peaks()
    if mode == "bf16":
        peak, src = peaks["bf16_tflops"], peaks["source"] + " (burst cuBLAS bf16)"
    else:
        peak, src = fp8_peak_tflops(), FP8_PEAK_SOURCE
    res = {
        "workload": f"{name}: MoE FFN layer T={T} H={H} I={I} E={E} top-{k} {mode}, {t_loc} tokens and {e_loc} experts per GPU",
        "exchange": ("none (every expert is local)" if world == 1 else
                     f"NCCL all_to_all_single (counts, payload, return), {layer.W} waves, one host read of the split sizes"
                     if exchange == "nccl" else
                     "peer memory: push kernel + down-GEMM epilogue stores over NVLink, no host synchronisation"),
        "intermediate": ("bf16" if mode == "bf16" else
                         "e4m3 + 1x128 scales written by the gate+up GEMM's epilogue" if ops.fuse_requant
                         else "bf16, then the separate 1x128 quantiser"),
        "metric": "moe_layer_tokens_per_s", "value": T / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "scaling": "strong", "ms_per_step": ms_step, "steps": steps,
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu / peak,
                     "peak_source": src,
                     "note": "whole layer (route, gather/dispatch, 2 GEMMs, quantise, return, combine) against the GEMM peak"},
        "phase_ms_rank0": phase_ms,
        "e2e": {"value": T / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": t_loc * H * 2, "d2h_bytes_per_step": t_loc * H * 2,
                "note": "per-rank token shard from pinned host memory, output back to pinned host memory; weights resident"},
        "parity": {"max_rel_err": err_all[0], "tol": tol, "rows_checked": n_checked * world,
                   "what": "tokens of every rank against the CPU restatement of the layer on the same quantised operands",
                   "all_finite": err_all[1] == 0.0},
        "status_word": "0 on every rank after the timed steps" if bad_status == 0.0 else "SET on some rank",
        "gpu_launches_rank0": launches,
    }
    if layer.peer is not None:
        layer.peer.close()
    assert err_all[0] <= tol and err_all[1] == 0.0, f"{name} ({exchange}) fails parity: {res['parity']}"
    assert bad_status == 0.0, f"{name} ({exchange}): a device status word was set during the timed steps"
    return res, out


def ep_layer_section(rank, world, dev, args):
    """The expert-parallel DeepSeek-V3 layer on the GPUs of this run, both exchanges."""
    ops = build_layer_ops("c4", rank, world, dev, args.cta_group, args.fuse_requant)
    steps = args.steps
    if world == 1:
        res, _ = measure_layer("c4", "nccl", ops, rank, world, dev, args, steps)
        return res
    res, out_peer = measure_layer("c4", "peer", ops, rank, world, dev, args, steps)
    nccl, out_nccl = measure_layer("c4", "nccl", ops, rank, world, dev, args, steps)
    same = float(torch.equal(out_peer, out_nccl))
    same = -reduce_max([-same], dev, world)[0]
    res["parity"]["peer_equals_nccl_bit_for_bit"] = bool(same == 1.0)
    for key in ("workload", "intermediate", "metric", "unit", "n_gpus", "scaling"):
        nccl.pop(key, None)
    res["nccl"] = nccl
    return res


def run_layer(args):
    """`--workload c3|c4|c4_rank8`: the MoE layer as the run's headline (tokens/s)."""
    from applied_ai_b200 import _lib
    import applied_ai_b200 as B
    rank, world, local = dist_env()
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_DEBUG", "WARN")  # keep NCCL's version banner off stdout
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=240))
    _lib.load(build_if_missing=False)
    B.set_default_check(False)
    name = args.workload
    if name in ("c3", "c4_rank8") and world > 1:
        raise SystemExit(f"{name} is a single-GPU workload")
    T, H, I, E, k, mode = LAYERS[name]
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid))
    if rank == 0:
        sampler.start()
    ops = build_layer_ops(name, rank, world, dev, args.cta_group, args.fuse_requant)
    t0 = time.time()
    res, _ = measure_layer(name, args.exchange, ops, rank, world, dev, args, args.steps)
    t1 = time.time()
    if rank == 0:
        sampler.stop()
        v, dt, sample = cpu_layer_tokens_per_s(H, I, E, k)
        line = {
            "metric": "moe_layer_tokens_per_s", "value": res["value"], "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": res["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16" if mode == "bf16" else "fp8_e4m3", "data": "synthetic",
            "config": {"workload": res["workload"], "l2": "weights per GPU exceed the 126 MiB L2",
                       "intermediate": res["intermediate"], "exchange": res["exchange"]},
            "roofline": dict(res["roofline"], traffic=args.traffic),
            "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample} if world == 1 else None,
            "e2e": res["e2e"], "gpu_launches": res["gpu_launches_rank0"], "phase_ms_rank0": res["phase_ms_rank0"],
            "parity": res["parity"], "status_word": res["status_word"],
            "clocks": sampler.window(t0, t1),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def also_layer(name, dev, args, steps):
    ops = build_layer_ops(name, 0, 1, dev, args.cta_group, args.fuse_requant)
    res, _ = measure_layer(name, "nccl", ops, 0, 1, dev, args, steps)
    for key in ("metric", "n_gpus", "scaling", "exchange"):
        res.pop(key, None)
    return res


# ------------------------------------------------------------------ the default run

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
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=240))
    _lib.load(build_if_missing=False)
    B.set_default_check(False)
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid))
    if rank == 0:
        sampler.start()   # early: nvidia-smi needs a moment before its first sample

    wl = make_workload(args.workload, rank, dev, args.cta_group)
    G, M, N, K = wl["G"], wl["M"], wl["N"], wl["K"]
    m_sizes, step, flops = wl["m_sizes"], wl["step"], wl["flops"]

    y = step()
    torch.cuda.synchronize()
    B.pending_status()
    # correctness guard on the timed configuration: a sample of rows of every rank against the host loop
    par = parity_of_workload(wl, y, dev)
    par["max_rel_err"] = reduce_max([par["max_rel_err"]], dev, world)[0]
    par["rows_checked"] *= world
    assert par["max_rel_err"] <= wl["tol"], f"bench output fails parity: {par}"

    ms_total, launches, t_wall0, t_wall1 = time_steps(step, args.steps, args.warmup, world)
    B.pending_status()
    clocks = sampler.window(t_wall0, t_wall1) if rank == 0 else None

    # the same step back to back for at least two seconds: the rate under the board's power limit
    sustained = None
    if args.sustained:
        n_sus = max(args.steps, int(2200.0 / max(ms_total / args.steps, 1e-3)) + 1)
        barrier(world)
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ts0 = time.time()
        s0.record()
        for _ in range(n_sus):
            step()
        s1.record()
        barrier(world)
        ts1 = time.time()
        ms_sus = reduce_max([s0.elapsed_time(s1)], dev, world)[0]
        sustained = (n_sus, ms_sus, ts0, ts1)

    vendor = vendor_grouped_mm(wl, y) if (rank == 0 and world == 1) else None
    del y

    # end to end: pinned host activations (and their scales) -> device, the public API call, result -> host,
    # every step.  Copies and compute of consecutive steps overlap the way a caller streaming batches
    # would run them: an upload stream, the compute stream and a download stream over two sets of buffers.
    # The pinned buffers are allocated and first touched on the GPU's NUMA node.
    nbuf = 2
    with numa_local(dev) as numa:
        act_host = [pinned_copy(t.cpu()) for t in wl["act"]]
        m_host = pinned_copy(m_sizes.cpu())
        y_host = [torch.empty((M, wl["n_out"]), dtype=torch.bfloat16).pin_memory() for _ in range(nbuf)]
        for t in y_host:
            t.zero_()
    act_dev = [[torch.empty_like(t) for t in wl["act"]] for _ in range(nbuf)]
    m_dev = [torch.empty_like(m_sizes) for _ in range(nbuf)]
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
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(s_up)
    e2e_run(e2e_steps)
    s_down.wait_stream(s_cmp)
    s_down.wait_stream(s_up)
    e1.record(s_down)
    barrier(world)
    B.pending_status()
    ms_e2e_rank = e0.elapsed_time(e1) / e2e_steps
    del act_dev, outs, y_host, act_host

    ms_total, ms_e2e = reduce_max([ms_total, ms_e2e_rank], dev, world)
    flops_all = reduce_sum([flops], dev, world)[0]
    ms_step = ms_total / args.steps
    h2d, d2h = wl["act_bytes"] + G * 4, M * wl["n_out"] * 2

    peaks = load_peaks()
    line = None
    if rank == 0:
        tflops = flops_all / (ms_step * 1e-3) / 1e12
        traffic = args.traffic
        if traffic is None and args.cta_group == 0:
            traffic = PROFILED_TRAFFIC_BYTES.get(args.workload)
        line = {
            "metric": "grouped_gemm_tflops", "value": tflops, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
            "config": {"workload": f"{args.workload}: grouped GEMM {wl['kind']} G={G} K={K} N={N} M={M} per GPU, "
                                   f"{wl['m_desc']}, epilogue {wl['epilogue']}",
                       "cta_group": args.cta_group or "auto",
                       "l2": f"operands {wl['alg_bytes'] >> 20} MiB per step > 126 MiB L2",
                       "sharding": "replicas only: every rank runs its own 8 experts and 16384 rows, no exchange "
                                   "(the expert-parallel exchange is measured in ep_layer)" if world > 1 else "single GPU"},
            "roofline": roofline_of_workload(wl, ms_step, peaks, traffic),
            "parity": par,
            "e2e": {"value": flops_all / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOPS", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e,
                    "h2d_gbs_rank0": h2d / (ms_e2e_rank * 1e-3) / 1e9, "d2h_gbs_rank0": d2h / (ms_e2e_rank * 1e-3) / 1e9,
                    "pinned_buffers_numa_node": numa.node if numa.cpus else None,
                    "note": "every step: activations (+scales) and m_sizes from pinned host memory, result to pinned host "
                            "memory; weights resident; uploads, compute and downloads of consecutive steps overlap "
                            "(3 streams, 2 buffer sets); PCIe-bound, and with N ranks the copies of all ranks share "
                            "the host's memory and root complexes"},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if sustained is not None:
            n_sus, ms_sus, ts0, ts1 = sustained
            v = flops_all / (ms_sus / n_sus * 1e-3) / 1e12
            per_gpu = v / world
            line["sustained"] = {"steps": n_sus, "seconds": ms_sus * 1e-3, "ms_per_step": ms_sus / n_sus, "value": v,
                                 "unit": "TFLOPS",
                                 "frac_of_sustained_peak": per_gpu / peaks["bf16_tflops_sustained"]
                                 if wl["kind"].startswith("bf16") else None,
                                 "frac_of_burst_peak": per_gpu / peaks["bf16_tflops"]
                                 if wl["kind"].startswith("bf16") else None,
                                 "clocks": sampler.window(ts0, ts1)}
        if vendor is not None:
            line["vendor_baseline"] = vendor
    del wl, step
    torch.cuda.empty_cache()

    if args.also and world == 1 and rank == 0:
        also = {}
        for name in args.also_list:
            try:
                if name in LAYERS:
                    also[name] = also_layer(name, dev, args, max(5, min(args.steps, 10)))
                else:
                    also[name] = also_gemm(name, dev, args.cta_group, max(5, min(args.steps, 10)), peaks)
            except AssertionError as exc:   # a parity failure must be visible in the line, not hide the rest of it
                also[name] = {"failed": str(exc)[:300]}
            torch.cuda.empty_cache()
        line["also"] = also

    if args.ep_layer:
        t0 = time.time()
        try:
            ep = ep_layer_section(rank, world, dev, args)
        except AssertionError as exc:
            ep = {"failed": str(exc)[:300]}
        if rank == 0:
            ep["clocks"] = sampler.window(t0, time.time())
            line["ep_layer"] = ep
        torch.cuda.empty_cache()

    if rank == 0:
        sampler.stop()
        if world == 1:
            cpu_tf, sample = cpu_loop_tflops(G, N, K, seconds=args.cpu_seconds)
            line["cpu_baseline"] = {"value": cpu_tf, "unit": "TFLOPS", "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": sample,
                                    "note": "CPU port of the reference's ground-truth loop (its Triton kernels cannot run here)"}
        else:
            line["cpu_baseline"] = None   # timed at N = 1 only
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
                    help="expert-parallel layers, NCCL exchange: chunks of local experts with their own all-to-all")
    ap.add_argument("--exchange", default="peer", choices=["nccl", "peer"],
                    help="--workload c4: NCCL all-to-all, or remote stores into peer memory")
    ap.add_argument("--fuse-requant", action=argparse.BooleanOptionalAction, default=True, dest="fuse_requant",
                    help="FP8 layers: quantise the SwiGLU output inside the gate+up GEMM (default; "
                         "--no-fuse-requant runs the separate quantiser on a bf16 intermediate)")
    ap.add_argument("--traffic", type=float, default=None,
                    help="DRAM bytes per launch from an ncu capture, echoed into the roofline object")
    ap.add_argument("--sustained", action=argparse.BooleanOptionalAction, default=None,
                    help="also run the step back to back for two seconds (default: on for the default workload)")
    ap.add_argument("--also", action=argparse.BooleanOptionalAction, default=None,
                    help="N = 1: also measure the other single-GPU workloads (default: on for the default workload)")
    ap.add_argument("--also-list", default=",".join(ALSO_DEFAULT), dest="also_list")
    ap.add_argument("--ep-layer", action=argparse.BooleanOptionalAction, default=None, dest="ep_layer",
                    help="also measure the expert-parallel DeepSeek-V3 layer on the GPUs of this run "
                         "(default: on for the default workload)")
    ap.add_argument("--cpu-seconds", type=float, default=10.0, dest="cpu_seconds",
                    help="N = 1: how long the CPU baseline repeats its sample")
    args = ap.parse_args()
    default_run = args.workload == "c2" and args.cta_group == 0
    for flag in ("sustained", "also", "ep_layer"):
        if getattr(args, flag) is None:
            setattr(args, flag, default_run)
    args.also_list = [n for n in args.also_list.split(",") if n]
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
