// Types shared by the translation units of libb200moe.so (not part of the public ABI).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200moe {

// Values a kernel may leave in the caller's status word (0 = nothing to report).
enum : int32_t {
    kStatusBadGroupSizes = 1,     // a negative group size, or the sizes add up to more rows than x has
    kStatusTimeoutProducer = 16,  // TMA producer gave up waiting for a free stage
    kStatusTimeoutMmaFull = 17,   // MMA issuer gave up waiting for a filled stage
    kStatusTimeoutMmaAcc = 18,    // MMA issuer gave up waiting for a drained accumulator
    kStatusTimeoutEpilogue = 19,  // epilogue gave up waiting for a finished accumulator
    kStatusSelfTestTimeout = 20,  // the self-test's deliberately unsatisfied wait ran out (expected)
    kStatusCapacity = 24,         // expert-parallel dispatch: a rank would receive more rows than its buffer holds
    kStatusPeerTimeout = 25,      // expert-parallel barrier: a peer's flag did not arrive within the limit
    kStatusWrongArch = 32,        // kernel image was not built for sm_100a
};

// Negative return codes of the C entry points (positive values are cudaError_t).
enum : int {
    kErrBadArgument = -1,
    kErrAlignment = -2,
    kErrTooManyGroups = -3,
    kErrNoDriverEntry = -4,
    kErrTensorMap = -5,
    kErrWrongDevice = -6,
    kErrTooLarge = -7,
};

struct GGParams {
    const int32_t* m_sizes;
    void* y;
    const float* x_scale;
    const float* w_scale;
    int32_t* status;
    const int32_t* row_map;        // optional: row r of the result is stored at row row_map[r] of y
    const long long* row_tags;     // optional: row r goes to peer_y[tag >> 32] at row (tag & 0xffffffff)
    void* const* peer_y;           //   bases of y on every rank (device array, n_peers entries)
    int n_peers;
    float* y_scale_out;            // EPI 3: fp32 scales of the e4m3 output, [M, n_out/128]
    float* y_f32_out;              // EPI 3, optional: the fp32 values that were quantised, [M, n_out]
    const float* c_in;             // fp32 epilogue: the C operand of alpha*acc + beta*C (same layout as y)
    float alpha, beta;
    uint32_t idesc;                // tcgen05 instruction descriptor (operand formats, tile shape)
    uint32_t idesc_half;           // same with N = 128, for the split tiles of the last round
    int y_rows;                    // rows of y (bounds for row_map)
    long long ldy;                 // elements between consecutive rows of y
    long long y_col_group_stride;  // first column of group g's block is g * this (0: all groups share columns)
    int M, N, K, G;
    long long x_col_group_stride;  // group g's K range in x starts at column g * this (0: shared columns)
    int n_out;    // output columns per group (N, or N/2 with SwiGLU)
    int n_tiles;  // column tiles per group
    int tile_mode;  // which row blocks this launch covers (kTilesAll / kTilesMain / kTilesTails)
    int overlap_role;  // 0 none; 1: a second launch of the same GEMM follows and may start on the SMs this one gives
                       // back (launch_dependents at start); 2: that second launch (griddep_wait before it exits, so
                       // that it never completes before the first one)
};

struct GGLaunch {
    const void* x;
    const void* w;
    const int32_t* m_sizes;
    void* y;
    const float* x_scale;
    const float* w_scale;
    int32_t* status;
    const int32_t* row_map;
    const long long* row_tags;
    void* const* peer_y;
    int n_peers;
    float* y_scale_out;
    float* y_f32_out;
    const float* c_in;
    float alpha, beta;
    int is_f16;      // 2-byte operands are IEEE half instead of bf16
    int w_mn_major;  // w is [G, K, N] (N contiguous) instead of [G, N, K]; 16-bit operands, plain epilogue only
    int overlap_role;  // GGParams::overlap_role for a caller that pairs this launch with an independent one
    int y_rows;
    long long ldy;
    long long y_col_group_stride;
    long long x_ld;                // elements per row of x when it is wider than K (0: K)
    long long x_col_group_stride;  // see GGParams
    int M, N, K, G;
    int elem_bytes;  // 2 bf16/f16, 1 e4m3
    int scale_mode;  // 0 none, 1 row-wise
    int epilogue;    // 0 plain, 1 SwiGLU, 2 fp32 out = alpha*acc + beta*C, 3 SwiGLU -> e4m3 + 1x128 scales
    int cta_group;   // 0 auto, 1 or 2
    cudaStream_t stream;
};

// Kernels this library has enqueued in this process (every launch site calls note_launch right after its launch).
void note_launch(int n = 1);
long long launches_so_far();

int grouped_gemm_launch(const GGLaunch& a);
// Weight gradient (grouped_gemm_dw.cu): dY [M, dy_ld] and x [M, K] are read in place; tail_ws holds the
// zero-padded copies of the groups' partial last 64-row blocks (dw_workspace_bytes).
size_t dw_workspace_bytes(int N, int K, int G);
// Step 1 (tail_pack_kernel) fills tail_ws; step 2 is the GEMM.  overlapped: the kernel launched just before in
// the stream is independent of this one and has executed launch_dependents, so this one may start on the SMs
// that one gives back (it then waits for that kernel before it exits).
int dw_tail_pack_launch(const void* dy, long long dy_ld, long long dy_col_group_stride, const void* x,
                        const int32_t* m_sizes, int M, int N, int K, int G, void* tail_ws, cudaStream_t stream);
int grouped_gemm_dw_launch(const void* dy, long long dy_ld, long long dy_col_group_stride, const void* x,
                           const int32_t* m_sizes, void* dw, int M, int N, int K, int G, const void* tail_ws,
                           int cta_group, bool overlapped, int32_t* status, cudaStream_t stream);
int selftest_wait_launch(uint64_t limit_ns, int32_t* status, cudaStream_t stream);
int selftest_tmem_read_launch(int warps, int in_flight, int iters, int ctas, long long* cycles_out,
                              cudaStream_t stream);
// FP8 with 1x128 activation scales [M, K/128] and 128x128 weight scales [G, ceil(N/128), K/128].
int grouped_gemm_fp8_block_launch(const GGLaunch& a);

}  // namespace b200moe
