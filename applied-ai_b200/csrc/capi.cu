// extern "C" entry points of libb200moe.so; declarations and contracts are in
// include/b200moe.h.  Each one validates its arguments on the host, enqueues kernels
// on the caller's stream and returns a code; none allocates, synchronises or throws.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200moe.h"
#include "b200moe_internal.h"
#include "moe_kernels.h"

using namespace b200moe;

static_assert(B200MOE_EBADARG == kErrBadArgument && B200MOE_EALIGN == kErrAlignment &&
                  B200MOE_ETOOMANYGROUPS == kErrTooManyGroups && B200MOE_ENODRIVER == kErrNoDriverEntry &&
                  B200MOE_ETENSORMAP == kErrTensorMap && B200MOE_EWRONGDEVICE == kErrWrongDevice &&
                  B200MOE_ETOOLARGE == kErrTooLarge,
              "public and internal error codes must agree");
static_assert(B200MOE_SBADSIZES == kStatusBadGroupSizes && B200MOE_STIMEOUT_FIRST == kStatusTimeoutProducer &&
                  B200MOE_STIMEOUT_LAST == kStatusTimeoutEpilogue && B200MOE_SSELFTEST == kStatusSelfTestTimeout && B200MOE_SCAPACITY == kStatusCapacity && B200MOE_SPEERTIMEOUT == kStatusPeerTimeout && B200MOE_SWRONGARCH == kStatusWrongArch,
              "public and internal status codes must agree");

#include <atomic>
namespace b200moe {
static std::atomic<long long> g_launches{0};
void note_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launches_so_far() { return g_launches.load(std::memory_order_relaxed); }
}  // namespace b200moe

extern "C" {

int b200moe_version(void) { return 1; }
long long b200moe_kernel_launches(void) { return launches_so_far(); }

#ifndef B200MOE_BUILD_ID
#define B200MOE_BUILD_ID 0
#endif
int b200moe_build_id(void) { return B200MOE_BUILD_ID; }

int b200moe_grouped_gemm_bf16(const void* x, const void* w, const int32_t* m_sizes, void* y, int M, int N, int K,
                              int G, int64_t ldy, int64_t y_col_group_stride, int epilogue, int cta_group,
                              const int32_t* y_row_map, int y_rows, int32_t* status, b200moe_stream_t stream) {
    GGLaunch a{};
    a.x = x;
    a.w = w;
    a.m_sizes = m_sizes;
    a.y = y;
    a.status = status;
    a.row_map = y_row_map;
    a.y_rows = y_rows;
    a.ldy = ldy;
    a.y_col_group_stride = y_col_group_stride;
    a.M = M;
    a.N = N;
    a.K = K;
    a.G = G;
    a.elem_bytes = 2;
    a.scale_mode = 0;
    a.epilogue = epilogue;
    a.cta_group = cta_group;
    a.stream = static_cast<cudaStream_t>(stream);
    if (ldy <= 0 || y_col_group_stride < 0 || (y_row_map != nullptr && y_rows <= 0)) return kErrBadArgument;
    return grouped_gemm_launch(a);
}

int b200moe_grouped_gemm_fp8_rowwise(const void* xq, const void* wq, const float* x_scale, const float* w_scale,
                                     const int32_t* m_sizes, void* y, int M, int N, int K, int G, int64_t ldy,
                                     int64_t y_col_group_stride, int cta_group, const int32_t* y_row_map,
                                     int y_rows, int32_t* status, b200moe_stream_t stream) {
    GGLaunch a{};
    a.x = xq;
    a.w = wq;
    a.m_sizes = m_sizes;
    a.y = y;
    a.x_scale = x_scale;
    a.w_scale = w_scale;
    a.status = status;
    a.row_map = y_row_map;
    a.y_rows = y_rows;
    a.ldy = ldy;
    a.y_col_group_stride = y_col_group_stride;
    a.M = M;
    a.N = N;
    a.K = K;
    a.G = G;
    a.elem_bytes = 1;
    a.scale_mode = 1;
    a.epilogue = 0;
    a.cta_group = cta_group;
    a.stream = static_cast<cudaStream_t>(stream);
    if (ldy <= 0 || y_col_group_stride < 0 || (y_row_map != nullptr && y_rows <= 0)) return kErrBadArgument;
    return grouped_gemm_launch(a);
}

int b200moe_grouped_gemm_fp8_blockwise(const void* xq, const void* wq, const float* x_scale, const float* w_scale,
                                       const int32_t* m_sizes, void* y, int M, int N, int K, int G, int64_t ldy,
                                       int64_t y_col_group_stride, int epilogue, int cta_group,
                                       const int32_t* y_row_map, int y_rows, int32_t* status,
                                       b200moe_stream_t stream) {
    GGLaunch a{};
    a.x = xq;
    a.w = wq;
    a.m_sizes = m_sizes;
    a.y = y;
    a.x_scale = x_scale;
    a.w_scale = w_scale;
    a.status = status;
    a.row_map = y_row_map;
    a.y_rows = y_rows;
    a.ldy = ldy;
    a.y_col_group_stride = y_col_group_stride;
    a.M = M;
    a.N = N;
    a.K = K;
    a.G = G;
    a.elem_bytes = 1;
    a.scale_mode = 2;
    a.epilogue = epilogue;
    a.cta_group = cta_group;
    a.stream = static_cast<cudaStream_t>(stream);
    if (ldy <= 0 || y_col_group_stride < 0 || (y_row_map != nullptr && y_rows <= 0)) return kErrBadArgument;
    return grouped_gemm_fp8_block_launch(a);
}

int b200moe_grouped_gemm_ex(const b200moe_gemm_desc* d, b200moe_stream_t stream) {
    if (d == nullptr) return kErrBadArgument;
    GGLaunch a{};
    a.x = d->x;
    a.w = d->w;
    a.m_sizes = d->m_sizes;
    a.y = d->y;
    a.x_scale = d->x_scale;
    a.w_scale = d->w_scale;
    a.status = d->status;
    a.row_map = d->y_row_map;
    a.row_tags = reinterpret_cast<const long long*>(d->y_row_tags);
    a.peer_y = d->y_peer_bases;
    a.n_peers = d->n_peers;
    a.y_rows = d->y_rows;
    a.ldy = d->ldy;
    a.y_col_group_stride = d->y_col_group_stride;
    a.M = d->M;
    a.N = d->N;
    a.K = d->K;
    a.G = d->G;
    a.epilogue = d->epilogue;
    a.cta_group = d->cta_group;
    a.stream = static_cast<cudaStream_t>(stream);
    if (d->ldy <= 0 || d->y_col_group_stride < 0 || d->m_sizes == nullptr) return kErrBadArgument;
    if ((d->y_row_map != nullptr || d->y_row_tags != nullptr) && d->y_rows <= 0) return kErrBadArgument;
    if (d->epilogue != B200MOE_EPI_NONE && d->epilogue != B200MOE_EPI_SWIGLU &&
        !(d->epilogue == B200MOE_EPI_SWIGLU_FP8 && d->kind == B200MOE_KIND_FP8_BLOCKWISE))
        return kErrBadArgument;
    a.y_scale_out = d->y_scale_out;
    a.y_f32_out = d->y_fp32_out;
    switch (d->kind) {
        case B200MOE_KIND_BF16:
            a.elem_bytes = 2;
            a.scale_mode = 0;
            return grouped_gemm_launch(a);
        case B200MOE_KIND_FP8_ROWWISE:
            a.elem_bytes = 1;
            a.scale_mode = 1;
            return grouped_gemm_launch(a);
        case B200MOE_KIND_FP8_BLOCKWISE:
            a.elem_bytes = 1;
            a.scale_mode = 2;
            return grouped_gemm_fp8_block_launch(a);
        default:
            return kErrBadArgument;
    }
}

int b200moe_ep_plan(const int32_t* counts, int P, int E, int my_rank, int capacity_rows, int32_t* dst_base,
                    int32_t* m_local, int32_t* status, b200moe_stream_t stream) {
    return ep_plan_launch(counts, P, E, my_rank, capacity_rows, dst_base, m_local, status,
                          static_cast<cudaStream_t>(stream));
}

int b200moe_ep_push(const void* part0, int64_t row_bytes0, const void* part1, int64_t row_bytes1,
                    const int32_t* perm, int top_k, const int32_t* offsets, const int32_t* dst_base, int R, int E,
                    int P, int my_rank, int capacity_rows, int tokens, void* const* peer_part0,
                    void* const* peer_part1, int64_t* const* peer_tags, void* home_rows, int64_t home_row_bytes,
                    b200moe_stream_t stream) {
    return ep_push_launch(part0, row_bytes0, part1, row_bytes1, perm, top_k, offsets, dst_base, R, E, P, my_rank,
                          capacity_rows, tokens, peer_part0, peer_part1,
                          reinterpret_cast<long long* const*>(peer_tags), home_rows, home_row_bytes,
                          static_cast<cudaStream_t>(stream));
}

int b200moe_ep_barrier(int32_t* const* flag_blocks, int P, int my_rank, int slot, int epoch, uint64_t limit_ns,
                       int32_t* status, b200moe_stream_t stream) {
    return ep_barrier_launch(flag_blocks, P, my_rank, slot, epoch, limit_ns, status, static_cast<cudaStream_t>(stream));
}

int b200moe_enable_peer_access(int peer_device) { return enable_peer_access(peer_device); }
int b200moe_ipc_open(const void* handle64, void** base) { return ipc_open(handle64, base); }
int b200moe_ipc_export(const void* dev_ptr, void* handle_out64, uint64_t* offset_out) {
    unsigned long long off = 0;
    const int rc = ipc_export(dev_ptr, handle_out64, &off);
    if (rc == 0) *offset_out = off;
    return rc;
}
int b200moe_ipc_close(void* base) { return ipc_close(base); }
int b200moe_peer_probe(void* peer_ptr, void* local_scratch8) { return peer_probe(peer_ptr, local_scratch8); }

int b200moe_sm100_gemm_f16(const void* A, const void* B, const void* C, void* D, int M, int N, int K, float alpha,
                           float beta, b200moe_stream_t stream) {
    GGLaunch a{};
    a.x = A;
    a.w = B;
    a.m_sizes = nullptr;  // one group: every row
    a.y = D;
    a.c_in = static_cast<const float*>(C);
    a.alpha = alpha;
    a.beta = beta;
    a.is_f16 = 1;
    a.ldy = N;
    a.y_col_group_stride = 0;
    a.M = M;
    a.N = N;
    a.K = K;
    a.G = 1;
    a.elem_bytes = 2;
    a.scale_mode = 0;
    a.epilogue = 2;
    a.cta_group = 0;
    a.stream = static_cast<cudaStream_t>(stream);
    return grouped_gemm_launch(a);
}

int b200moe_backward_workspace_bytes(int M, int N, int K, int G, size_t* bytes) {
    if (bytes == nullptr || M < 0 || N <= 0 || K <= 0 || G <= 0) return kErrBadArgument;
    *bytes = dw_workspace_bytes(N, K, G) + 256;
    return 0;
}

int b200moe_grouped_gemm_backward(const void* grad_y, const void* x, const void* w, const int32_t* m_sizes,
                                  void* grad_x, void* grad_w, int M, int N, int K, int G, int64_t grad_y_ld,
                                  int64_t grad_y_col_group_stride, void* workspace, size_t workspace_bytes,
                                  int cta_group, int32_t* status, b200moe_stream_t stream) {
    size_t need = 0;
    if (int e = b200moe_backward_workspace_bytes(M, N, K, G, &need)) return e;
    if (grad_y == nullptr || x == nullptr || w == nullptr || m_sizes == nullptr || grad_x == nullptr ||
        grad_w == nullptr || workspace == nullptr || grad_y_ld < N || grad_y_col_group_stride < 0)
        return kErrBadArgument;
    // every operand is read in place by TMA: 16-byte row pitches
    if (N % 8 != 0 || K % 8 != 0 || grad_y_ld % 8 != 0 || grad_y_col_group_stride % 8 != 0) return kErrAlignment;
    if (workspace_bytes < need) return kErrTooLarge;
    if (M == 0) return 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The two gradients are independent of each other, so the grad_w kernel is launched to start on the SMs the
    // grad_x kernel gives back while its last round of tiles drains (overlap_role); the small packing kernel that
    // grad_w needs runs first so that nothing stands between the two.
    const uintptr_t tail_ws = (reinterpret_cast<uintptr_t>(workspace) + 255) & ~static_cast<uintptr_t>(255);
    if (int e = dw_tail_pack_launch(grad_y, grad_y_ld, grad_y_col_group_stride, x, m_sizes, M, N, K, G,
                                    reinterpret_cast<void*>(tail_ws), s))
        return e;
    // grad_x[rows of g] = grad_y[rows of g, block g] @ w[g]: the forward kernel with w[g] [N, K] read as an
    // MN-major operand (the contraction walks its rows)
    GGLaunch a{};
    a.x = grad_y;
    a.w = w;
    a.w_mn_major = 1;
    a.overlap_role = 1;
    a.m_sizes = m_sizes;
    a.y = grad_x;
    a.status = status;
    a.ldy = K;
    a.x_ld = grad_y_ld;
    a.x_col_group_stride = grad_y_col_group_stride;
    a.M = M;
    a.N = K;   // output columns
    a.K = N;   // contraction length
    a.G = G;
    a.elem_bytes = 2;
    a.cta_group = cta_group;
    a.stream = s;
    if (int e = grouped_gemm_launch(a)) return e;
    // grad_w[g] = grad_y[rows of g, block g]^T @ x[rows of g]
    return grouped_gemm_dw_launch(grad_y, grad_y_ld, grad_y_col_group_stride, x, m_sizes, grad_w, M, N, K, G,
                                  reinterpret_cast<const void*>(tail_ws), cta_group, /*overlapped=*/true, status, s);
}

int b200moe_selftest_wait_timeout(uint64_t limit_ns, int32_t* status, b200moe_stream_t stream) {
    return selftest_wait_launch(limit_ns, status, static_cast<cudaStream_t>(stream));
}

int b200moe_selftest_tmem_read(int warps, int in_flight, int iters, int ctas, long long* cycles,
                               b200moe_stream_t stream) {
    return selftest_tmem_read_launch(warps, in_flight, iters, ctas, cycles, static_cast<cudaStream_t>(stream));
}

int b200moe_route_workspace_bytes(int R, int E, size_t* bytes) {
    if (bytes == nullptr) return kErrBadArgument;
    int chunk_len = 0, num_chunks = 0;
    if (int e = route_plan(R, E, &chunk_len, &num_chunks)) return e;
    *bytes = sizeof(int32_t) * static_cast<size_t>(num_chunks > 0 ? num_chunks : 1) * static_cast<size_t>(E);
    return 0;
}

int b200moe_route(const int32_t* ids, int R, int E, int32_t* m_sizes, int32_t* offsets, int32_t* perm,
                  int32_t* inv_perm, void* workspace, size_t workspace_bytes, int32_t* status,
                  b200moe_stream_t stream) {
    size_t need = 0;
    if (int e = b200moe_route_workspace_bytes(R, E, &need)) return e;
    if (m_sizes == nullptr || offsets == nullptr) return kErrBadArgument;
    if (R > 0 && (ids == nullptr || perm == nullptr || inv_perm == nullptr || workspace == nullptr))
        return kErrBadArgument;
    if (R > 0 && workspace_bytes < need) return kErrTooLarge;
    return route_launch(ids, R, E, m_sizes, offsets, perm, inv_perm, static_cast<int32_t*>(workspace), status,
                        static_cast<cudaStream_t>(stream));
}

int b200moe_route_noalloc(const int32_t* ids, int R, int E, int32_t* m_sizes, int32_t* offsets, int32_t* perm,
                          int32_t* inv_perm, int32_t* status, b200moe_stream_t stream) {
    if (m_sizes == nullptr || offsets == nullptr) return kErrBadArgument;
    if (R > 0 && (ids == nullptr || perm == nullptr || inv_perm == nullptr)) return kErrBadArgument;
    return route_static_launch(ids, R, E, m_sizes, offsets, perm, inv_perm, status,
                               static_cast<cudaStream_t>(stream));
}

int b200moe_moe_align_workspace_bytes(int R, int E, size_t* bytes) {
    if (bytes == nullptr) return kErrBadArgument;
    const long long n = align_blocks_scratch_ints(R, E);
    if (n < 0) return kErrBadArgument;
    *bytes = sizeof(int32_t) * static_cast<size_t>(n);
    return 0;
}

int b200moe_moe_align_block_size(const int32_t* ids, int R, int E, int block_size, int32_t* sorted_ids,
                                 int32_t* expert_ids, int32_t* num_tokens_post_pad, void* workspace,
                                 size_t workspace_bytes, int32_t* status, b200moe_stream_t stream) {
    size_t need = 0;
    if (int e = b200moe_moe_align_workspace_bytes(R, E, &need)) return e;
    if (sorted_ids == nullptr || expert_ids == nullptr || num_tokens_post_pad == nullptr || workspace == nullptr ||
        (R > 0 && ids == nullptr))
        return kErrBadArgument;
    if (workspace_bytes < need) return kErrTooLarge;
    return align_blocks_launch(ids, R, E, block_size, sorted_ids, expert_ids, num_tokens_post_pad,
                               static_cast<int32_t*>(workspace), status, static_cast<cudaStream_t>(stream));
}

int b200moe_gather_rows(const void* src, const int32_t* idx, int div, void* dst, int rows, int64_t row_bytes,
                        int src_rows, b200moe_stream_t stream) {
    if (rows > 0 && (src == nullptr || idx == nullptr || dst == nullptr)) return kErrBadArgument;
    return gather_rows_launch(src, idx, div, dst, rows, row_bytes, src_rows, static_cast<cudaStream_t>(stream));
}

int b200moe_swiglu(const void* in, void* out, int64_t rows, int d, b200moe_stream_t stream) {
    if (rows > 0 && (in == nullptr || out == nullptr)) return kErrBadArgument;
    return swiglu_launch(in, out, rows, d, static_cast<cudaStream_t>(stream));
}

int b200moe_combine_topk(const void* y, const int32_t* inv_perm, const float* weight, void* out, int T, int k,
                         int H, int y_rows, b200moe_stream_t stream) {
    if (T > 0 && (y == nullptr || inv_perm == nullptr || out == nullptr)) return kErrBadArgument;
    return combine_topk_launch(y, inv_perm, weight, out, T, k, H, y_rows, static_cast<cudaStream_t>(stream));
}

int b200moe_quant_1x128(const void* x, int x_is_fp32, void* q, float* scales, int64_t rows, int K,
                        b200moe_stream_t stream) {
    if (rows > 0 && (x == nullptr || q == nullptr || scales == nullptr)) return kErrBadArgument;
    return quant_1x128_launch(x, x_is_fp32, q, scales, rows, K, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
