// Two diagnostics.
// (1) A wait that nothing will ever satisfy, to show what every wait in the GEMM kernels does
// when its limit runs out: it stops polling, leaves a code in the status word and the
// kernel returns normally, so the context stays usable.  No fault, trap or endless loop
// is involved.
// (2) The raw read rate of tensor memory (tcgen05.ld), further down.
#include <cuda_runtime.h>
#include <stdint.h>

#include "b200moe_internal.h"
#include "ptx.cuh"

namespace b200moe {

__global__ void selftest_wait_kernel(uint64_t limit_ns, int32_t* status) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&bar, 1);  // one arrival expected; none will come
        mbar_init_fence();
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) ok = mbar_wait(&bar, 0, &abort_flag, limit_ns);
    __syncthreads();
    // the other threads see the shared flag, exactly as the roles of a GEMM CTA do
    if (threadIdx.x == 32 && abort_flag && status != nullptr) atomicCAS(status, 0, kStatusSelfTestTimeout);
    (void)ok;
}

int selftest_wait_launch(uint64_t limit_ns, int32_t* status, cudaStream_t stream) {
    if (status == nullptr || limit_ns == 0 || limit_ns > 2000000000ull) return kErrBadArgument;
    selftest_wait_kernel<<<1, 64, 0, stream>>>(limit_ns, status);
    note_launch();
    return static_cast<int>(cudaGetLastError());
}

// Raw rate of tcgen05.ld out of tensor memory, the quantity that bounds an epilogue (or the per-K-block
// promotion of the block-wise FP8 kernel) that has to bring a whole 128 x 256 fp32 accumulator into registers:
// `warps` (4 or 8) warps of one CTA read one accumulator's worth (128 lanes x 256 columns, 128 KiB) `iters`
// times with 32x32b.x32 loads, IN_FLIGHT loads issued before each wait, and cycles_out[cta] receives the
// clock64() ticks warp 0 saw around its loop.  Nothing is computed, nothing waits on anything else.
template <int IN_FLIGHT>
__global__ void __launch_bounds__(256, 1) tmem_read_probe_kernel(int iters, long long* cycles_out, uint32_t* sink) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL)
    __shared__ uint32_t tmem_base_s;
    const int warp = threadIdx.x >> 5;
    const int warps = blockDim.x >> 5;
    if (warp == 0) {
        tmem_alloc<1>(&tmem_base_s, 256);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    // 8 warps: warps 0-3 take columns 0-127, warps 4-7 columns 128-255; 4 warps: all 256 columns each
    const int col0 = warps == 8 ? (warp >> 2) * 128 : 0;
    const int loads = (warps == 8 ? 128 : 256) / 32;  // x32 loads per pass of this warp
    const uint32_t t0 = tmem_base_s + lane_base + static_cast<uint32_t>(col0);
    uint32_t acc = 0;
    uint32_t v[IN_FLIGHT][32];
    __syncthreads();
    const long long c0 = clock64();
    for (int it = 0; it < iters; ++it) {
        for (int l = 0; l < loads; l += IN_FLIGHT) {
#pragma unroll
            for (int j = 0; j < IN_FLIGHT; ++j) tmem_ld_32x32(t0 + static_cast<uint32_t>((l + j) * 32), v[j]);
#pragma unroll
            for (int j = 0; j < IN_FLIGHT; ++j) tmem_ld_wait(v[j]);
#pragma unroll
            for (int j = 0; j < IN_FLIGHT; ++j) acc ^= v[j][0] ^ v[j][31];
        }
    }
    const long long c1 = clock64();
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) cycles_out[blockIdx.x] = c1 - c0;
    if (acc == 0x9e3779b9u && sink != nullptr) sink[0] = acc;  // keeps the loads alive
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc<1>(tmem_base_s, 256);
    }
#endif
}

int selftest_tmem_read_launch(int warps, int in_flight, int iters, int ctas, long long* cycles_out,
                              cudaStream_t stream) {
    if ((warps != 4 && warps != 8) || (in_flight != 1 && in_flight != 2 && in_flight != 4) || iters <= 0 ||
        iters > 100000 || ctas <= 0 || ctas > 1024 || cycles_out == nullptr)
        return kErrBadArgument;
    const dim3 grid(static_cast<unsigned>(ctas)), block(static_cast<unsigned>(warps * 32));
    if (in_flight == 1) tmem_read_probe_kernel<1><<<grid, block, 0, stream>>>(iters, cycles_out, nullptr);
    if (in_flight == 2) tmem_read_probe_kernel<2><<<grid, block, 0, stream>>>(iters, cycles_out, nullptr);
    if (in_flight == 4) tmem_read_probe_kernel<4><<<grid, block, 0, stream>>>(iters, cycles_out, nullptr);
    note_launch();
    return static_cast<int>(cudaGetLastError());
}

}  // namespace b200moe
