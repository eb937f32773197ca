// Expert-parallel dispatch over peer memory: the sender writes every routed row straight
// into the destination rank's receive buffer, at its final expert-sorted position, with
// plain 16-byte stores over NVLink.  No staging buffer, no all-to-all, no re-sort on the
// receiver.  (The way back is the grouped GEMM's epilogue storing through (rank, row)
// tags.)  The reference has no distributed code; this implements the dispatch/combine
// exchange that the expert-parallel benchmark configuration asks for.
//
// Every rank knows the full count matrix C[src][global expert] (one small all-gather), so
// it can compute where its rows land on every destination without asking anyone:
//   row(dest d, local expert e, i-th row of mine)
//       = sum_{e' < e} total[d][e']  +  sum_{s < me} C[s][d*El + e]  +  i
// which is the stable (expert, source rank, source order) ordering.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "b200moe_internal.h"
#include "moe_kernels.h"

namespace b200moe {

// One block.  counts: [P][E] int32, source-major.  Outputs: dst_base[E] (first row, on the
// owning rank, of my rows for each global expert) and m_loc[El] (rows per local expert
// that this rank receives in total).
__global__ void __launch_bounds__(256)
ep_plan_kernel(const int32_t* __restrict__ counts, int P, int E, int e_local, int me, int cap,
               int32_t* __restrict__ dst_base, int32_t* __restrict__ m_loc, int32_t* status) {
    extern __shared__ int32_t sm[];
    int32_t* tot = sm;         // [E] rows of every rank for the expert
    int32_t* before = sm + E;  // [E] rows of ranks below me for the expert
    for (int ge = threadIdx.x; ge < E; ge += blockDim.x) {
        int t = 0, b = 0;
        for (int s = 0; s < P; ++s) {
            const int c = counts[static_cast<size_t>(s) * E + ge];
            t += c;
            if (s < me) b += c;
        }
        tot[ge] = t;
        before[ge] = b;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < P; d += blockDim.x) {
        int running = 0;
        for (int e = 0; e < e_local; ++e) {
            const int ge = d * e_local + e;
            dst_base[ge] = running + before[ge];
            // the owner computes the rows that fit: positions are in expert order, so what is
            // dropped is a suffix and the group sizes stay consistent with the rows that arrive
            if (d == me) m_loc[e] = max(0, min(tot[ge], cap - running));
            running += tot[ge];
        }
        // a destination that would overflow its buffer: rows past `cap` are dropped by the
        // push kernel (their results count as zero), and everybody learns about it here
        if (running > cap && status != nullptr) atomicCAS(status, 0, kStatusCapacity);
    }
}

// One warp per routed row (sorted position p).  parts: up to two byte arrays per token
// (e.g. e4m3 row and its fp32 scales); tags: (my rank << 32 | p) so the owner of the
// expert can send the result back to row p of my buffer.
__global__ void __launch_bounds__(256)
ep_push_kernel(const uint8_t* __restrict__ part0, long long bytes0, const uint8_t* __restrict__ part1,
               long long bytes1, const int32_t* __restrict__ perm, int k, const int32_t* __restrict__ offsets,
               const int32_t* __restrict__ dst_base, int R, int E, int e_local, int me, int cap, int tokens,
               uint8_t* const* __restrict__ peer0, uint8_t* const* __restrict__ peer1,
               long long* const* __restrict__ peer_tag, uint8_t* __restrict__ home, long long home_row_bytes) {
    const int lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    // Every rank starts its walk over the (destination-sorted) rows at a different place, so
    // that at any moment the ranks write to different destinations instead of all to the same.
    const int rot = static_cast<int>(static_cast<long long>(me) * R / (E / e_local));
    for (int p0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p0 < R; p0 += warps_total) {
        const int p = p0 + rot < R ? p0 + rot : p0 + rot - R;
        int lo = 0, hi = E - 1;  // global expert of sorted position p: last ge with offsets[ge] <= p
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (__ldg(offsets + mid) <= p) lo = mid; else hi = mid - 1;
        }
        const int ge = lo;
        const int d = ge / e_local;
        const int row = __ldg(dst_base + ge) + (p - __ldg(offsets + ge));
        const int flat = __ldg(perm + p);
        const int tok = flat / k;
        if (row < 0 || row >= cap || flat < 0 || tok >= tokens) {
            // a row its owner has no room for is never computed: its result row, which the combine
            // reads from this rank's home buffer, is zeroed here instead of keeping an older step's values
            if (home != nullptr) {
                uint4* z = reinterpret_cast<uint4*>(home + static_cast<size_t>(p) * home_row_bytes);
                for (int v = lane; v < static_cast<int>(home_row_bytes >> 4); v += 32) z[v] = make_uint4(0u, 0u, 0u, 0u);
            }
            continue;
        }
        {
            const uint4* src = reinterpret_cast<const uint4*>(part0 + static_cast<size_t>(tok) * bytes0);
            uint4* dst = reinterpret_cast<uint4*>(peer0[d] + static_cast<size_t>(row) * bytes0);
            const int n = static_cast<int>(bytes0 >> 4);
            int v = lane;
            for (; v + 96 < n; v += 128) {
                const uint4 r0 = __ldg(src + v), r1 = __ldg(src + v + 32), r2 = __ldg(src + v + 64),
                            r3 = __ldg(src + v + 96);
                dst[v] = r0;
                dst[v + 32] = r1;
                dst[v + 64] = r2;
                dst[v + 96] = r3;
            }
            for (; v < n; v += 32) dst[v] = __ldg(src + v);
        }
        if (part1 != nullptr) {
            if ((bytes1 & 15) == 0) {
                const uint4* src = reinterpret_cast<const uint4*>(part1 + static_cast<size_t>(tok) * bytes1);
                uint4* dst = reinterpret_cast<uint4*>(peer1[d] + static_cast<size_t>(row) * bytes1);
                const int n = static_cast<int>(bytes1 >> 4);
                for (int v = lane; v < n; v += 32) dst[v] = __ldg(src + v);
            } else {  // short rows (a few scales): 4 bytes at a time
                const uint32_t* src = reinterpret_cast<const uint32_t*>(part1 + static_cast<size_t>(tok) * bytes1);
                uint32_t* dst = reinterpret_cast<uint32_t*>(peer1[d] + static_cast<size_t>(row) * bytes1);
                const int n = static_cast<int>(bytes1 >> 2);
                for (int v = lane; v < n; v += 32) dst[v] = __ldg(src + v);
            }
        }
        if (lane == 0) peer_tag[d][row] = (static_cast<long long>(me) << 32) | static_cast<long long>(p);
    }
    __threadfence_system();  // rows are on their way to other GPUs: order them before the kernel ends
}

// Barrier between the ranks' streams without a collective: thread p tells rank p "my kernels up to
// here are done" by storing `epoch` into word [slot][me] of rank p's flag block, then waits until
// rank p has stored the same epoch (or a later one) into this rank's block.  One block of P threads.
// Everything this rank enqueued before is complete when this kernel starts (stream order), the
// release store orders it before the flag for the peer, and the acquire load orders the peer's data
// before whatever this stream runs next.  The wait is bounded: after limit_ns the thread records
// kStatusPeerTimeout and returns, nothing is left spinning.
__global__ void __launch_bounds__(64)
ep_barrier_kernel(int32_t* const* __restrict__ flag_blocks, int P, int me, int slot, int32_t epoch,
                  unsigned long long limit_ns, int32_t* status) {
    const int p = threadIdx.x;
    if (p >= P) return;
    __threadfence_system();
    int32_t* theirs = flag_blocks[p] + slot * P + me;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
    const int32_t* mine = flag_blocks[me] + slot * P + p;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (unsigned spins = 0;; ++spins) {
        int32_t seen;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if (seen - epoch >= 0) break;  // epochs only grow; the difference also survives a wrap
        if ((spins & 0x3f) == 0x3f) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (now - t0 > limit_ns) {
                if (status != nullptr) atomicCAS(status, 0, kStatusPeerTimeout);
                break;
            }
        }
    }
}

int ep_barrier_launch(int32_t* const* flag_blocks, int P, int me, int slot, int epoch, unsigned long long limit_ns,
                      int32_t* status, cudaStream_t stream) {
    if (flag_blocks == nullptr || P <= 0 || P > 64 || me < 0 || me >= P || slot < 0 || slot > 1 || limit_ns == 0 ||
        limit_ns > 10ull * 1000 * 1000 * 1000)
        return kErrBadArgument;
    ep_barrier_kernel<<<1, 64, 0, stream>>>(flag_blocks, P, me, slot, epoch, limit_ns, status);
    note_launch();
    return static_cast<int>(cudaGetLastError());
}

int ep_plan_launch(const int32_t* counts, int P, int E, int me, int cap, int32_t* dst_base, int32_t* m_loc,
                   int32_t* status, cudaStream_t stream) {
    if (counts == nullptr || dst_base == nullptr || m_loc == nullptr || P <= 0 || E <= 0 || E % P != 0 || me < 0 ||
        me >= P || cap <= 0 || E > 4096)
        return kErrBadArgument;
    ep_plan_kernel<<<1, 256, sizeof(int32_t) * 2 * E, stream>>>(counts, P, E, E / P, me, cap, dst_base, m_loc, status);
    note_launch();
    return static_cast<int>(cudaGetLastError());
}

int ep_push_launch(const void* part0, long long bytes0, const void* part1, long long bytes1, const int32_t* perm,
                   int k, const int32_t* offsets, const int32_t* dst_base, int R, int E, int P, int me, int cap,
                   int tokens, void* const* peer0, void* const* peer1, long long* const* peer_tag, void* home,
                   long long home_row_bytes, cudaStream_t stream) {
    if (part0 == nullptr || perm == nullptr || offsets == nullptr || dst_base == nullptr || peer0 == nullptr ||
        peer_tag == nullptr || k <= 0 || R < 0 || E <= 0 || P <= 0 || E % P != 0 || bytes0 <= 0 || (bytes0 & 15) ||
        (part1 != nullptr && (peer1 == nullptr || bytes1 <= 0 || (bytes1 & 3))))
        return kErrBadArgument;
    if ((reinterpret_cast<uintptr_t>(part0) & 15u) || (reinterpret_cast<uintptr_t>(part1) & 15u)) return kErrAlignment;
    if (home != nullptr && (home_row_bytes <= 0 || (home_row_bytes & 15) || (reinterpret_cast<uintptr_t>(home) & 15u)))
        return kErrAlignment;
    // rows of part 1 start at multiples of bytes1 inside 256-byte aligned buffers: 4-byte aligned at least
    if (R == 0) return 0;
    int blocks = (R + 7) / 8;
    if (blocks > 148 * 8) blocks = 148 * 8;
    ep_push_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(part0), bytes0,
                                               static_cast<const uint8_t*>(part1), bytes1, perm, k, offsets, dst_base,
                                               R, E, E / P, me, cap, tokens,
                                               reinterpret_cast<uint8_t* const*>(peer0),
                                               reinterpret_cast<uint8_t* const*>(peer1), peer_tag,
                                               static_cast<uint8_t*>(home), home_row_bytes);
    note_launch();
    return static_cast<int>(cudaGetLastError());
}

int enable_peer_access(int peer_device) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (peer_device == dev) return 0;
    int can = 0;
    e = cudaDeviceCanAccessPeer(&can, dev, peer_device);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (!can) return kErrWrongDevice;
    e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();  // clear the sticky-less error state
        return 0;
    }
    return static_cast<int>(e);
}

// Maps another process's allocation (exported with cudaIpcGetMemHandle) into this process
// with THIS rank's device current, so the mapping is made for access from this device and
// peer access is switched on as part of the call.
int ipc_open(const void* handle_bytes, void** base) {
    if (handle_bytes == nullptr || base == nullptr) return kErrBadArgument;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle_bytes, sizeof(h));
    return static_cast<int>(cudaIpcOpenMemHandle(base, h, cudaIpcMemLazyEnablePeerAccess));
}

// Export side: the handle of the cudaMalloc allocation that contains dev_ptr, and the byte
// offset of dev_ptr inside that allocation (the importer gets the allocation's base back).
int ipc_export(const void* dev_ptr, void* handle_out64, unsigned long long* offset_out) {
    if (dev_ptr == nullptr || handle_out64 == nullptr || offset_out == nullptr) return kErrBadArgument;
    using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || sym == nullptr)
        return kErrNoDriverEntry;
    CUdeviceptr base = 0;
    size_t size = 0;
    if (reinterpret_cast<RangeFn>(sym)(&base, &size, reinterpret_cast<CUdeviceptr>(dev_ptr)) != CUDA_SUCCESS)
        return kErrBadArgument;
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
    if (e != cudaSuccess) return static_cast<int>(e);
    memcpy(handle_out64, &h, sizeof(h));
    *offset_out = static_cast<unsigned long long>(reinterpret_cast<CUdeviceptr>(dev_ptr) - base);
    return 0;
}

int ipc_close(void* base) { return static_cast<int>(cudaIpcCloseMemHandle(base)); }

// Set-up time check of a mapping without any kernel touching it: copy a word into the
// peer buffer and back with the copy engine and compare.  A broken mapping shows up as an
// error code here instead of a fault in a kernel later.
int peer_probe(void* peer_ptr, void* local_scratch8) {
    if (peer_ptr == nullptr || local_scratch8 == nullptr) return kErrBadArgument;
    const unsigned int pattern = 0x5EEDB200u;
    unsigned int back = 0, saved = 0;
    cudaError_t e = cudaMemcpy(&saved, peer_ptr, 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaMemcpy(local_scratch8, &pattern, 4, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaMemcpy(peer_ptr, local_scratch8, 4, cudaMemcpyDeviceToDevice);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaMemcpy(static_cast<char*>(local_scratch8) + 4, peer_ptr, 4, cudaMemcpyDeviceToDevice);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaMemcpy(&back, static_cast<char*>(local_scratch8) + 4, 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaMemcpy(peer_ptr, &saved, 4, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return static_cast<int>(e);
    return back == pattern ? 0 : kErrWrongDevice;
}

}  // namespace b200moe
