// A wait that nothing will ever satisfy, to show what every wait in the GEMM kernels does
// when its limit runs out: it stops polling, leaves a code in the status word and the
// kernel returns normally, so the context stays usable.  No fault, trap or endless loop
// is involved.
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

}  // namespace b200moe
