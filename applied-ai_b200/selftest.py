"""Diagnostics of the library that have no counterpart in the reference.

`tmem_read_rate()` times raw `tcgen05.ld` traffic (b200moe_selftest_tmem_read): the bytes per SM clock at which
an accumulator can be brought out of tensor memory, which bounds every epilogue and, in the block-wise FP8
kernel, the promotion that follows each 128-deep K block.

    python -c "import applied_ai_b200.selftest as s; s.main()"
"""
import torch

from . import _lib

ACC_BYTES = 128 * 256 * 4  # one CTA's 128-lane x 256-column fp32 accumulator


def tmem_read_rate(warps=8, in_flight=2, iters=200, ctas=1, device=None):
    """Bytes per SM clock (slowest CTA) at which `ctas` CTAs drain an accumulator with 32x32b.x32 loads."""
    if not torch.cuda.is_available():
        raise RuntimeError("tmem_read_rate needs a CUDA device (there is no CPU path)")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    lib = _lib.load()
    cycles = torch.zeros(ctas, dtype=torch.int64, device=device)
    with torch.cuda.device(device):
        for _ in range(2):  # the first launch pays for loading the kernel
            rc = lib.b200moe_selftest_tmem_read(warps, in_flight, iters, ctas, cycles.data_ptr(),
                                                torch.cuda.current_stream().cuda_stream)
            _lib.check(rc, "selftest_tmem_read")
        torch.cuda.synchronize(device)
    worst = int(cycles.max().item())
    if worst <= 0:
        raise RuntimeError("the probe kernel did not run (wrong architecture?)")
    return ACC_BYTES * iters / worst


def main():
    for ctas in (1, 148):
        for warps in (4, 8):
            for in_flight in (1, 2, 4):
                r = tmem_read_rate(warps, in_flight, 200, ctas)
                print(f"ctas={ctas:3d} warps={warps} loads_in_flight={in_flight}: {r:7.1f} B/clk/SM, "
                      f"{ACC_BYTES / r:7.1f} clk per 128x256 fp32 accumulator")


if __name__ == "__main__":
    main()
