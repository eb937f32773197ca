// The memory-bound steps that surround the expert GEMMs in an MoE layer: routing
// (stable counting sort of the flattened top-k expert ids), row gather, SwiGLU,
// weighted top-k combine and 1x128 e4m3 quantisation.  In the reference these are
// vLLM ops and ATen calls around the Triton GEMM
// (kernels/triton/inference/col_major_moe_gemm/v0_moe_fused.py:138-180, :276-296) and a
// Triton quantiser (kernels/triton/inference/fp8/float8_groupwise_quant.py:20-50).
// All are HBM-bound: 16-byte vector accesses, one pass over the data, no atomics whose
// order could change a result.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <mutex>

#include "b200moe_internal.h"
#include "moe_kernels.h"

namespace b200moe {

// ------------------------------------------------------------------ routing
//
// Input: ids[R] (R = tokens * top_k, flattened row-major, so flat index i = t*k + j).
// Output: m_sizes[E] (rows per expert), offsets[E+1] (exclusive prefix), perm[R]
// (sorted position -> flat index) and inv_perm[R] (flat index -> sorted position).
// The order is the stable sort by expert id: inside one expert, ascending flat index.
//
// Three launches over C chunks of the id list (one warp per chunk):
//   count   : counts[c][e] = number of ids equal to e in chunk c
//   scan    : per expert, exclusive prefix over chunks (in place) and the total
//   scatter : position = offsets[e] + counts[c][e] + rank inside the chunk
// `counts` is the scratch memory (C*E int32).  Ids outside [0, E) are dropped
// (inv_perm = -1) and reported through the status word.

constexpr int kRouteWarps = 4;

__global__ void __launch_bounds__(kRouteWarps * 32)
route_count_kernel(const int32_t* __restrict__ ids, int R, int E, int chunk_len, int num_chunks,
                   int32_t* __restrict__ counts, int32_t* status) {
    extern __shared__ int32_t hist_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunk = blockIdx.x * kRouteWarps + warp;
    if (chunk >= num_chunks) return;
    int32_t* hist = hist_all + warp * E;
    for (int e = lane; e < E; e += 32) hist[e] = 0;
    __syncwarp();
    const int begin = chunk * chunk_len;
    const int end = min(R, begin + chunk_len);
    for (int i0 = begin; i0 < end; i0 += 32) {
        const int i = i0 + lane;
        int e = i < end ? ids[i] : -1;
        if (i < end && (e < 0 || e >= E)) {
            if (status) atomicCAS(status, 0, kStatusBadGroupSizes);
            e = -1;
        }
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && (peers & ((1u << lane) - 1u)) == 0) hist[e] += __popc(peers);
        __syncwarp();
    }
    for (int e = lane; e < E; e += 32) counts[static_cast<size_t>(chunk) * E + e] = hist[e];
}

// One warp per expert: exclusive scan of counts[:, e] over the chunks, 32 at a time.
__global__ void __launch_bounds__(256)
route_scan_kernel(int32_t* __restrict__ counts, int E, int num_chunks, int32_t* __restrict__ m_sizes) {
    const int lane = threadIdx.x & 31;
    const int e = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (e >= E) return;
    int carry = 0;
    for (int c0 = 0; c0 < num_chunks; c0 += 32) {
        const int c = c0 + lane;
        const int v = c < num_chunks ? counts[static_cast<size_t>(c) * E + e] : 0;
        int s = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, s, d);
            if (lane >= d) s += o;
        }
        if (c < num_chunks) counts[static_cast<size_t>(c) * E + e] = carry + s - v;
        carry += __shfl_sync(0xffffffffu, s, 31);
    }
    if (lane == 0) m_sizes[e] = carry;
}

__global__ void __launch_bounds__(kRouteWarps * 32)
route_scatter_kernel(const int32_t* __restrict__ ids, int R, int E, int chunk_len, int num_chunks,
                     const int32_t* __restrict__ counts, const int32_t* __restrict__ m_sizes,
                     int32_t* __restrict__ offsets, int32_t* __restrict__ perm, int32_t* __restrict__ inv_perm) {
    extern __shared__ int32_t sm[];
    int32_t* off = sm;                 // [E] exclusive prefix of m_sizes
    int32_t* cursors = sm + E;         // [kRouteWarps][E]
    __shared__ int32_t warp_tot[kRouteWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Exclusive prefix of m_sizes over experts, computed by the whole block in slabs
    // of blockDim.x experts (E is at most a few thousand).
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += blockDim.x) {
        const int e = e0 + threadIdx.x;
        const int v = e < E ? m_sizes[e] : 0;
        int s = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, s, d);
            if (lane >= d) s += o;
        }
        if (lane == 31) warp_tot[warp] = s;
        __syncthreads();
        int before = 0, slab = 0;
        for (int w = 0; w < kRouteWarps; ++w) {
            if (w < warp) before += warp_tot[w];
            slab += warp_tot[w];
        }
        if (e < E) off[e] = carry + before + s - v;
        carry += slab;
        __syncthreads();
    }
    if (blockIdx.x == 0) {
        for (int e = threadIdx.x; e < E; e += blockDim.x) offsets[e] = off[e];
        if (threadIdx.x == 0) offsets[E] = carry;
    }

    const int chunk = blockIdx.x * kRouteWarps + warp;
    if (chunk >= num_chunks) return;
    int32_t* cur = cursors + warp * E;
    for (int e = lane; e < E; e += 32) cur[e] = off[e] + counts[static_cast<size_t>(chunk) * E + e];
    __syncwarp();
    const int begin = chunk * chunk_len;
    const int end = min(R, begin + chunk_len);
    for (int i0 = begin; i0 < end; i0 += 32) {
        const int i = i0 + lane;
        int e = i < end ? ids[i] : -1;
        if (e < 0 || e >= E) e = -1;
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const unsigned lower = peers & ((1u << lane) - 1u);
        int pos = -1;
        if (e >= 0) pos = cur[e] + __popc(lower);
        __syncwarp();
        if (e >= 0 && lower == 0) cur[e] += __popc(peers);
        __syncwarp();
        if (i < end) {
            inv_perm[i] = pos;
            if (pos >= 0) perm[pos] = i;
        }
    }
}

int route_plan(int R, int E, int* chunk_len, int* num_chunks) {
    if (R < 0 || E <= 0 || E > kRouteMaxExperts) return kErrBadArgument;
    int len = 256;
    const int need = (R + kRouteMaxChunks - 1) / kRouteMaxChunks;
    if (need > len) len = ((need + 31) / 32) * 32;
    *chunk_len = len;
    *num_chunks = R == 0 ? 0 : (R + len - 1) / len;
    return 0;
}

int route_launch(const int32_t* ids, int R, int E, int32_t* m_sizes, int32_t* offsets, int32_t* perm,
                 int32_t* inv_perm, int32_t* counts, int32_t* status, cudaStream_t stream) {
    int chunk_len = 0, num_chunks = 0;
    if (int e = route_plan(R, E, &chunk_len, &num_chunks)) return e;
    if (R == 0) {
        cudaError_t e1 = cudaMemsetAsync(m_sizes, 0, sizeof(int32_t) * E, stream);
        if (e1 != cudaSuccess) return static_cast<int>(e1);
        e1 = cudaMemsetAsync(offsets, 0, sizeof(int32_t) * (E + 1), stream);
        return static_cast<int>(e1);
    }
    const int blocks = (num_chunks + kRouteWarps - 1) / kRouteWarps;
    route_count_kernel<<<blocks, kRouteWarps * 32, sizeof(int32_t) * kRouteWarps * E, stream>>>(
        ids, R, E, chunk_len, num_chunks, counts, status);
    note_launch();
    route_scan_kernel<<<(E + 7) / 8, 256, 0, stream>>>(counts, E, num_chunks, m_sizes);
    note_launch();
    route_scatter_kernel<<<blocks, kRouteWarps * 32, sizeof(int32_t) * (kRouteWarps + 1) * E, stream>>>(
        ids, R, E, chunk_len, num_chunks, counts, m_sizes, offsets, perm, inv_perm);
    note_launch();
    return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ padded layout (vLLM format)
// From the routing result, the three arrays moe_align_block_size returns
// (kernels/triton/inference/col_major_moe_gemm/v0_moe_fused.py:138-180): every expert's rows
// padded to a multiple of block_size with the pad id `numel`, one expert id per block, and
// the padded total.  sorted_ids must arrive pre-filled with the pad id.
__global__ void __launch_bounds__(256)
align_blocks_kernel(const int32_t* __restrict__ m_sizes, const int32_t* __restrict__ offsets,
                    const int32_t* __restrict__ perm, int R, int E, int block_size,
                    int32_t* __restrict__ sorted_ids, int32_t* __restrict__ expert_ids,
                    int32_t* __restrict__ num_tokens_post_pad) {
    extern __shared__ int32_t padded_off[];  // [E + 1] exclusive prefix of the padded sizes
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < E; ++e) {
            padded_off[e] = acc;
            acc += (m_sizes[e] + block_size - 1) / block_size * block_size;
        }
        padded_off[E] = acc;
        if (blockIdx.x == 0) num_tokens_post_pad[0] = acc;
    }
    __syncthreads();
    const int stride = gridDim.x * blockDim.x;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;
    // one expert id per block of the padded layout
    const int nblocks = padded_off[E] / block_size;
    for (int b = tid; b < nblocks; b += stride) {
        const int pos = b * block_size;
        int lo = 0, hi = E - 1;  // last e with padded_off[e] <= pos and a non-empty padded range
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (padded_off[mid] <= pos) lo = mid; else hi = mid - 1;
        }
        expert_ids[b] = lo;
    }
    // routed rows to their padded positions
    for (int p = tid; p < R; p += stride) {
        int lo = 0, hi = E - 1;  // expert of sorted position p: last e with offsets[e] <= p
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (offsets[mid] <= p) lo = mid; else hi = mid - 1;
        }
        sorted_ids[padded_off[lo] + (p - offsets[lo])] = perm[p];
    }
}

__global__ void fill_i32_kernel(int32_t* dst, long long n, int32_t value) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        dst[i] = value;
}

int align_blocks_launch(const int32_t* ids, int R, int E, int block_size, int32_t* sorted_ids, int32_t* expert_ids,
                        int32_t* num_tokens_post_pad, int32_t* scratch, int32_t* status, cudaStream_t stream) {
    if (block_size <= 0) return kErrBadArgument;
    int chunk_len = 0, num_chunks = 0;
    if (int e = route_plan(R, E, &chunk_len, &num_chunks)) return e;
    // scratch: m_sizes[E] | offsets[E+1] | perm[R] | inv_perm[R] | counts[num_chunks*E]
    int32_t* m_sizes = scratch;
    int32_t* offsets = m_sizes + E;
    int32_t* perm = offsets + E + 1;
    int32_t* inv_perm = perm + R;
    int32_t* counts = inv_perm + R;
    if (int e = route_launch(ids, R, E, m_sizes, offsets, perm, inv_perm, counts, status, stream)) return e;
    const long long n_sorted = static_cast<long long>(R) + static_cast<long long>(E) * (block_size - 1);
    fill_i32_kernel<<<static_cast<int>(std::min<long long>((n_sorted + 255) / 256, 1184)), 256, 0, stream>>>(
        sorted_ids, n_sorted, R);
    note_launch();
    const int blocks = std::max(1, std::min((R + 255) / 256, 592));
    align_blocks_kernel<<<blocks, 256, sizeof(int32_t) * (E + 1), stream>>>(m_sizes, offsets, perm, R, E, block_size,
                                                                             sorted_ids, expert_ids,
                                                                             num_tokens_post_pad);
    note_launch();
    return static_cast<int>(cudaGetLastError());
}

long long align_blocks_scratch_ints(int R, int E) {
    int chunk_len = 0, num_chunks = 0;
    if (route_plan(R, E, &chunk_len, &num_chunks)) return -1;
    return static_cast<long long>(E) + (E + 1) + 2ll * R + static_cast<long long>(std::max(num_chunks, 1)) * E;
}

// ------------------------------------------------------------------ routing, scratch held by the library
//
// Same three launches as route_launch, with the chunk counts kept in an array that is
// part of the library image instead of a buffer from the caller.  Each GPU that loads
// the library carries the array (1 MiB) until the process exits.
constexpr int kRouteStaticInts = 1024 * 256;
constexpr int kRouteStaticMaxDevices = 64;
static __device__ __align__(256) int32_t g_route_static_counts[kRouteStaticInts];

int route_static_capacity_ints() { return kRouteStaticInts; }

int route_static_launch(const int32_t* ids, int R, int E, int32_t* m_sizes, int32_t* offsets, int32_t* perm,
                        int32_t* inv_perm, int32_t* status, cudaStream_t stream) {
    int chunk_len = 0, num_chunks = 0;
    if (int e = route_plan(R, E, &chunk_len, &num_chunks)) return e;
    if (static_cast<long long>(num_chunks) * E > kRouteStaticInts) return kErrTooLarge;
    int dev = 0;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    if (dev < 0 || dev >= kRouteStaticMaxDevices) return kErrBadArgument;
    // In host code the array's name is only a handle for the runtime; the address the
    // kernels need is a per-device value that has to be asked for, once, while that
    // device is current.
    static std::mutex mu;
    static int32_t* dev_ptr[kRouteStaticMaxDevices] = {};
    int32_t* counts = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev_ptr[dev] == nullptr) {
            void* p = nullptr;
            ce = cudaGetSymbolAddress(&p, g_route_static_counts);
            if (ce != cudaSuccess) return static_cast<int>(ce);
            dev_ptr[dev] = static_cast<int32_t*>(p);
        }
        counts = dev_ptr[dev];
    }
    // Every counts[c][e] with c < num_chunks is overwritten by the count kernel before it
    // is read, so what an earlier call left in the array does not matter.
    return route_launch(ids, R, E, m_sizes, offsets, perm, inv_perm, counts, status, stream);
}

// ------------------------------------------------------------------ gather
// dst[p, :] = src[idx[p] / div, :]   (row_bytes bytes per row), one warp per row.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint8_t* __restrict__ src, const int32_t* __restrict__ idx, int div, uint8_t* __restrict__ dst,
                   int rows, long long row_bytes, int src_rows, int vec_ok) {
    const int lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    for (int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < rows; p += warps_total) {
        const int i = idx[p];
        const int s = i / div;
        if (i < 0 || s >= src_rows) continue;  // never read outside src
        const uint8_t* a = src + static_cast<size_t>(s) * row_bytes;
        uint8_t* b = dst + static_cast<size_t>(p) * row_bytes;
        if (vec_ok) {
            const uint4* a4 = reinterpret_cast<const uint4*>(a);
            uint4* b4 = reinterpret_cast<uint4*>(b);
            const int n = static_cast<int>(row_bytes >> 4);
            int v = lane;
            for (; v + 96 < n; v += 128) {
                const uint4 r0 = __ldg(a4 + v), r1 = __ldg(a4 + v + 32), r2 = __ldg(a4 + v + 64),
                            r3 = __ldg(a4 + v + 96);
                b4[v] = r0;
                b4[v + 32] = r1;
                b4[v + 64] = r2;
                b4[v + 96] = r3;
            }
            for (; v < n; v += 32) b4[v] = __ldg(a4 + v);
        } else {
            for (long long v = lane; v < row_bytes; v += 32) b[v] = a[v];
        }
    }
}

int gather_rows_launch(const void* src, const int32_t* idx, int div, void* dst, int rows, long long row_bytes,
                       int src_rows, cudaStream_t stream) {
    if (rows < 0 || row_bytes <= 0 || div <= 0 || src_rows < 0) return kErrBadArgument;
    if (rows == 0) return 0;
    const int vec_ok = (row_bytes % 16 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) &&
                       ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
    int blocks = (rows + 7) / 8;
    if (blocks > 148 * 8) blocks = 148 * 8;
    gather_rows_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(src), idx, div,
                                                   static_cast<uint8_t*>(dst), rows, row_bytes, src_rows, vec_ok);
    note_launch();
    return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ SwiGLU
// out[r, j] = silu(in[r, j]) * in[r, d + j], bf16 in / bf16 out, fp32 math.
__global__ void __launch_bounds__(256)
swiglu_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, long long rows, int d) {
    const int vec_per_row = d >> 3;
    const long long total = rows * vec_per_row;
    for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < total;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = v / vec_per_row;
        const int c = static_cast<int>(v - r * vec_per_row) << 3;
        const uint4 g4 = *reinterpret_cast<const uint4*>(in + r * 2 * d + c);
        const uint4 u4 = *reinterpret_cast<const uint4*>(in + r * 2 * d + d + c);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
        uint4 o4;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 g = __bfloat1622float2(g2[q]);
            const float2 u = __bfloat1622float2(u2[q]);
            o2[q] = __floats2bfloat162_rn(g.x / (1.0f + __expf(-g.x)) * u.x, g.y / (1.0f + __expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + r * d + c) = o4;
    }
}

int swiglu_launch(const void* in, void* out, long long rows, int d, cudaStream_t stream) {
    if (rows < 0 || d <= 0 || (d % 8) != 0) return kErrBadArgument;
    if ((reinterpret_cast<uintptr_t>(in) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) return kErrAlignment;
    if (rows == 0) return 0;
    const long long total = rows * (d >> 3);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    swiglu_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(in),
                                                                static_cast<__nv_bfloat16*>(out), rows, d);
    note_launch();
    return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ combine
// out[t, :] = sum_{j<k} weight[t, j] * y[inv_perm[t*k + j], :], fp32 accumulation in
// ascending j, one rounding to bf16.  One thread owns 8 consecutive columns.
__global__ void __launch_bounds__(256)
combine_topk_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ inv_perm,
                    const float* __restrict__ weight, __nv_bfloat16* __restrict__ out, int T, int k, int H,
                    int y_rows) {
    const int vec_per_row = H >> 3;
    const long long total = static_cast<long long>(T) * vec_per_row;
    for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < total;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int t = static_cast<int>(v / vec_per_row);
        const int c = static_cast<int>(v - static_cast<long long>(t) * vec_per_row) << 3;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        // four rows at a time: their loads are all in flight before the first FMA (sum order stays j = 0, 1, ...)
        for (int j0 = 0; j0 < k; j0 += 4) {
            int pj[4];
            float wj[4];
            uint4 rj[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u;
                pj[u] = j < k ? __ldg(inv_perm + static_cast<size_t>(t) * k + j) : -1;
                wj[u] = (j < k && weight) ? __ldg(weight + static_cast<size_t>(t) * k + j) : 1.0f;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const bool live = pj[u] >= 0 && pj[u] < y_rows;
                rj[u] = live ? *reinterpret_cast<const uint4*>(y + static_cast<size_t>(pj[u]) * H + c)
                             : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (pj[u] < 0 || pj[u] >= y_rows) continue;
                const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rj[u]);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = __bfloat1622float2(r2[q]);
                    acc[2 * q] = fmaf(wj[u], f.x, acc[2 * q]);
                    acc[2 * q + 1] = fmaf(wj[u], f.y, acc[2 * q + 1]);
                }
            }
        }
        uint4 o4;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int q = 0; q < 4; ++q) o2[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
        *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + c) = o4;
    }
}

int combine_topk_launch(const void* y, const int32_t* inv_perm, const float* weight, void* out, int T, int k, int H,
                        int y_rows, cudaStream_t stream) {
    if (T < 0 || k <= 0 || H <= 0 || (H % 8) != 0 || y_rows < 0) return kErrBadArgument;
    if ((reinterpret_cast<uintptr_t>(y) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) return kErrAlignment;
    if (T == 0) return 0;
    const long long total = static_cast<long long>(T) * (H >> 3);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    combine_topk_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(y), inv_perm, weight, static_cast<__nv_bfloat16*>(out), T, k, H, y_rows);
    note_launch();
    return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ 1x128 quantiser
// For every run of 128 consecutive elements: scale = max(amax, 1e-12) / 448,
// q = clamp(x / scale, +-448) rounded to e4m3 (nearest even).  Sixteen lanes per run,
// 8 elements (one 16-byte load for bf16) per lane, so a warp covers two runs at a time.
// IEEE division, so results match the same formula evaluated in fp32 on the host bit for
// bit.
template <typename In>
__global__ void __launch_bounds__(256)
quant_1x128_kernel(const In* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scales, long long groups) {
    const int lane = threadIdx.x & 31;
    const int sub = lane & 15;  // position inside the run
    const long long halves_total = static_cast<long long>(gridDim.x) * (blockDim.x >> 4);
    for (long long grp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 4;
         grp < ((groups + 1) & ~1ll); grp += halves_total) {
        const bool live = grp < groups;  // odd tail: the idle half-warp still joins the shuffles
        float f[8];
        if (live) {
            const In* src = x + grp * 128 + sub * 8;
            if constexpr (sizeof(In) == 2) {
                const uint4 raw = *reinterpret_cast<const uint4*>(src);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 a = __bfloat1622float2(h[j]);
                    f[2 * j] = a.x;
                    f[2 * j + 1] = a.y;
                }
            } else {
                const float4 r0 = *reinterpret_cast<const float4*>(src);
                const float4 r1 = *reinterpret_cast<const float4*>(src + 4);
                f[0] = r0.x; f[1] = r0.y; f[2] = r0.z; f[3] = r0.w;
                f[4] = r1.x; f[5] = r1.y; f[6] = r1.z; f[7] = r1.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = 0.0f;
        }
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
#pragma unroll
        for (int d = 8; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
        const float scale = __fdiv_rn(fmaxf(amax, 1e-12f), 448.0f);
        uint32_t packed[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float v = __fdiv_rn(f[j], scale);
            v = fminf(fmaxf(v, -448.0f), 448.0f);
            const __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
            packed[j >> 2] |= static_cast<uint32_t>(b) << (8 * (j & 3));
        }
        if (live) {
            *reinterpret_cast<uint2*>(q + grp * 128 + sub * 8) = make_uint2(packed[0], packed[1]);
            if (sub == 0) scales[grp] = scale;
        }
    }
}

int quant_1x128_launch(const void* x, int x_is_fp32, void* q, float* scales, long long rows, int K,
                       cudaStream_t stream) {
    if (rows < 0 || K <= 0 || (K % 128) != 0) return kErrBadArgument;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(q) & 7u)) return kErrAlignment;
    const long long groups = rows * (K / 128);
    if (groups == 0) return 0;
    long long blocks = (groups + 15) / 16;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (x_is_fp32) {
        quant_1x128_kernel<float><<<static_cast<int>(blocks), 256, 0, stream>>>(
            static_cast<const float*>(x), static_cast<uint8_t*>(q), scales, groups);
        note_launch();
    } else {
        quant_1x128_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scales, groups);
        note_launch();
    }
    return static_cast<int>(cudaGetLastError());
}

}  // namespace b200moe
