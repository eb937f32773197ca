/* libb200moe.so — C ABI of the B200 (sm_100a) MoE grouped-GEMM engine.
 *
 * Every entry point takes raw DEVICE pointers, plain integers and a CUDA stream
 * (a cudaStream_t passed as void*; NULL = the default stream), enqueues its work on
 * that stream and returns without synchronising.  Nothing here allocates device
 * memory.  The device that owns the pointers must be current on the calling thread.
 *
 * Return value: 0 = enqueued; > 0 = a cudaError_t from the runtime; < 0 = one of
 * the B200MOE_E* codes below.  Entry points never throw and never abort.
 *
 * `status` (optional, may be NULL) points to one zero-initialised int32 in device
 * memory.  A kernel that meets bad data or gives up a bounded wait writes a non-zero
 * B200MOE_S* code there (first writer wins) and does no further work; the caller reads
 * it after synchronising.  The word is never reset by the library.
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* b200moe_stream_t;

/* negative return codes */
#define B200MOE_EBADARG (-1)       /* null pointer, non-positive size, unknown mode */
#define B200MOE_EALIGN (-2)        /* pointer not 16-byte aligned, or K * element size not a multiple of 16 */
#define B200MOE_ETOOMANYGROUPS (-3) /* G > 1024 */
#define B200MOE_ENODRIVER (-4)     /* cuTensorMapEncodeTiled could not be resolved */
#define B200MOE_ETENSORMAP (-5)    /* the driver rejected a tensor map */
#define B200MOE_EWRONGDEVICE (-6)  /* current device is not compute capability 10.x */
#define B200MOE_ETOOLARGE (-7)     /* workspace too small / size beyond a stated maximum */

/* device status word */
#define B200MOE_SBADSIZES 1        /* negative m_sizes entry, sum(m_sizes) > M, or an expert id outside [0, E) */
#define B200MOE_STIMEOUT_FIRST 16  /* 16..19: a bounded wait inside the GEMM kernel ran out */
#define B200MOE_STIMEOUT_LAST 19
#define B200MOE_SSELFTEST 20       /* b200moe_selftest_wait_timeout: the unsatisfied wait ran out, as it should */
#define B200MOE_SCAPACITY 24       /* expert-parallel dispatch: a receive buffer is too small for the routed rows */
#define B200MOE_SPEERTIMEOUT 25    /* expert-parallel barrier: a peer rank's flag did not arrive within the limit */
#define B200MOE_SWRONGARCH 32

/* flags of the grouped GEMM entry points */
#define B200MOE_EPI_NONE 0
#define B200MOE_EPI_SWIGLU 1  /* w[g] = [gate rows 0..N/2) ; up rows N/2..N); y gets N/2 columns: silu(gate)*up */
#define B200MOE_EPI_SWIGLU_FP8 3 /* block-wise FP8 kind via b200moe_grouped_gemm_ex only: silu(gate)*up quantised in the
                                   epilogue to e4m3 [M, N/2] (y, row pitch ldy BYTES) + fp32 scales [M, N/256] (y_scale_out) */
#define B200MOE_CTA_AUTO 0    /* 1 = one CTA per 128x256 tile, 2 = a CTA pair per 256x256 tile */

int b200moe_version(void);
/* Id of the source files this binary was compiled from (0 when the build did not set one).
 * The Python loader compares it with the sources on disk and refuses a library that does
 * not match them.  No counterpart in the reference (its kernels are compiled on first use). */
int b200moe_build_id(void);
/* How many kernels this library has enqueued in this process so far (all devices, all streams).
 * For callers that report their launch counts; a grouped GEMM may be one or two kernels.
 * No counterpart in the reference. */
long long b200moe_kernel_launches(void);

/* y[rows of group g, g*y_col_group_stride + (0..N)] = x[rows of group g, :] @ w[g]^T
 * x [M,K] bf16 row-major, w [G,N,K] bf16 row-major, m_sizes [G] int32 (device; zeros
 * allowed; sum <= M, trailing rows of y are then left untouched), y bf16 with `ldy`
 * elements between rows.  fp32 accumulation, one rounding to bf16.
 * y_col_group_stride = 0, ldy = N gives the [M,N] layout of
 *   grouped_gemm(x, w, m_sizes)            dev/triton_groupGEMM/groupgemm.py:518 (-> :407);
 * y_col_group_stride = N, ldy = N*G gives the [M, N*G] block layout of
 *   grouped_gemm_forward(x, w, m_sizes)    kernels/MoE/group_GEMM/triton/tgroup_gemm_forward.py:626 (-> :485).
 * With B200MOE_EPI_SWIGLU the activation of v0_moe_fused.py:284 (silu_and_mul) is
 * applied to the accumulators and y has N/2 columns per group.
 * y_row_map (device, may be NULL): when given, row r of the result is stored at row
 * y_row_map[r] of y (y has y_rows rows; entries outside [0, y_rows) are skipped).  This
 * is the scatter the reference's GEMM does through sorted_token_ids
 * (v0_moe_fused.py:132-135), used here to leave expert-sorted order in the same pass.
 * The FP8 entry points take the same two arguments. */
int b200moe_grouped_gemm_bf16(const void* x, const void* w, const int32_t* m_sizes, void* y, int M, int N, int K,
                              int G, int64_t ldy, int64_t y_col_group_stride, int epilogue, int cta_group,
                              const int32_t* y_row_map, int y_rows, int32_t* status, b200moe_stream_t stream);

/* Row-wise scaled FP8: y = (xq @ wq[g]^T) * x_scale[row] * w_scale[g*N + col].
 * xq [M,K], wq [G,N,K] float8_e4m3fn; x_scale [M] fp32; w_scale [G*N] fp32; y bf16.
 * Replaces grouped_gemm_fp8_rowwise(x, w, m_sizes, x_scale, w_scale)
 *   dev/triton_groupGEMM/groupgemm.py:524, kernels/MoE/group_GEMM/triton/tgroup_gemm_forward.py:632. */
int b200moe_grouped_gemm_fp8_rowwise(const void* xq, const void* wq, const float* x_scale, const float* w_scale,
                                     const int32_t* m_sizes, void* y, int M, int N, int K, int G, int64_t ldy,
                                     int64_t y_col_group_stride, int cta_group, const int32_t* y_row_map,
                                     int y_rows, int32_t* status, b200moe_stream_t stream);

/* Block-wise scaled FP8 (1x128 activation scales, 128x128 weight scales):
 *   y[m,n] = sum_kb (xq[m, kb*128:(kb+1)*128] . wq[g][n, same]) * x_scale[m, kb] * w_scale[g][n/128][kb]
 * xq [M,K], wq [G,N,K] float8_e4m3fn; x_scale [M, K/128] fp32; w_scale [G, ceil(N/128), K/128]
 * fp32; y bf16; K a multiple of 128.  epilogue = B200MOE_EPI_SWIGLU (N a multiple of 256)
 * writes silu(gate)*up with N/2 columns.  Not present in the reference (its block-wise
 * kernels are the absent FBGEMM ones named at kernels/needs_perf_help/fp8_gemm_bench.py:16-21);
 * the activation-scale convention is float8_groupwise_quant.py:36-46. */
int b200moe_grouped_gemm_fp8_blockwise(const void* xq, const void* wq, const float* x_scale, const float* w_scale,
                                       const int32_t* m_sizes, void* y, int M, int N, int K, int G, int64_t ldy,
                                       int64_t y_col_group_stride, int epilogue, int cta_group,
                                       const int32_t* y_row_map, int y_rows, int32_t* status,
                                       b200moe_stream_t stream);

/* One grouped GEMM described by a struct: everything the three entry points above can do,
 * plus a second way to place result rows — y_row_tags[r] = (rank << 32) | row sends result
 * row r to row `row` of y_peer_bases[rank] (bf16, pitch ldy, y_rows rows each), which may
 * be another GPU's memory mapped into this process: the return leg of the expert-parallel
 * exchange happens inside the GEMM's store over NVLink: ordinary st.global from the bf16
 * kernel, shared->global bulk copies (cp.async.bulk, never multicast) from the block-wise FP8
 * kernel.  Peer memory is only ever a store destination: no load of any kind reads it.  No counterpart
 * in the reference (it has no distributed code). */
#define B200MOE_KIND_BF16 0
#define B200MOE_KIND_FP8_ROWWISE 1
#define B200MOE_KIND_FP8_BLOCKWISE 2
typedef struct b200moe_gemm_desc {
    const void* x;            /* [M, K] */
    const void* w;            /* [G, N, K] */
    const int32_t* m_sizes;   /* [G] device */
    void* y;                  /* bf16 output (may be NULL when y_row_tags is set) */
    const float* x_scale;     /* FP8 kinds */
    const float* w_scale;
    int M, N, K, G;
    int64_t ldy, y_col_group_stride;
    int kind;                 /* B200MOE_KIND_* */
    int epilogue;             /* B200MOE_EPI_* */
    int cta_group;
    int y_rows;               /* rows of the destination buffer(s) when a map or tags are given */
    const int32_t* y_row_map; /* optional */
    const int64_t* y_row_tags;/* optional, excludes y_row_map */
    void* const* y_peer_bases;/* device array of n_peers base pointers */
    int n_peers;
    int32_t* status;
    float* y_scale_out;       /* B200MOE_EPI_SWIGLU_FP8: scales of the quantised output */
    float* y_fp32_out;        /* B200MOE_EPI_SWIGLU_FP8, optional (NULL: off): the fp32 silu(gate)*up values
                                 [M, N/2] that were quantised, 16-byte aligned; for checking the quantiser */
} b200moe_gemm_desc;
int b200moe_grouped_gemm_ex(const b200moe_gemm_desc* desc, b200moe_stream_t stream);

/* Expert-parallel dispatch over peer memory (no counterpart in the reference).
 * b200moe_ep_plan: from counts[P][E] (rows every rank routes to every global expert, after
 * an all-gather) compute, for rank my_rank, dst_base[E] = first row in the owner's receive
 * buffer for my rows of each expert, and m_local[E/P] = rows this rank receives per local
 * expert.  Order on the owner: expert, then source rank, then source order.  Sets status
 * B200MOE_SCAPACITY if some rank would receive more than capacity_rows rows.
 * b200moe_ep_push: for every routed row p (sorted by global expert: perm, offsets from
 * b200moe_route) copy its token's bytes (part0, row size a multiple of 16, and optionally
 * part1, row size a multiple of 4) into the owner's buffers peer_part0[d] / peer_part1[d] at row dst_base[e] + i and
 * write peer_tags[d][row] = (my_rank << 32) | p.  Rows past capacity_rows are dropped: the owner's
 * m_local counts only the rows that fit (a prefix in expert order), the sender zeroes the dropped
 * row's result in its own home buffer (home_rows: [R] rows of home_row_bytes bytes, a multiple of
 * 16; may be NULL), so the layer's output then lacks those experts' contributions, and
 * B200MOE_SCAPACITY in the status word says so.
 * The peer_* arrays are DEVICE arrays of P pointers into buffers of capacity_rows rows on
 * each rank, mapped into this process (CUDA IPC); call b200moe_enable_peer_access for each
 * peer device once.  The caller orders "all pushes done" before the GEMMs with a
 * collective on the stream. */
int b200moe_ep_plan(const int32_t* counts, int P, int E, int my_rank, int capacity_rows, int32_t* dst_base,
                    int32_t* m_local, int32_t* status, b200moe_stream_t stream);
int b200moe_ep_push(const void* part0, int64_t row_bytes0, const void* part1, int64_t row_bytes1,
                    const int32_t* perm, int top_k, const int32_t* offsets, const int32_t* dst_base, int R, int E,
                    int P, int my_rank, int capacity_rows, int tokens, void* const* peer_part0,
                    void* const* peer_part1, int64_t* const* peer_tags, void* home_rows, int64_t home_row_bytes,
                    b200moe_stream_t stream);
/* Barrier between the P ranks' streams through flag words in peer-mapped memory, in place of a
 * collective (a one-element all-reduce costs tens of microseconds, this a few).  flag_blocks is a DEVICE
 * array of P pointers, entry r = rank r's flag block of 2*P int32 (zero before first use, mapped into
 * this process like the other exchange buffers).  Thread p stores `epoch` into word [slot][my_rank] of rank
 * p's block, then waits until rank p has stored an epoch >= `epoch` into word [slot][p] of this rank's
 * block.  The caller passes the same, growing epoch on every rank (1, 2, 3, ... per call and slot; two
 * slots so that the two barriers of a step do not share words).  What this rank enqueued before the call
 * is complete before its flags are stored; what it enqueues after starts after every peer's flag has
 * been seen.  The wait gives up after limit_ns (1 .. 1e10): status gets B200MOE_SPEERTIMEOUT and the
 * kernel returns.  No counterpart in the reference, which has no multi-GPU code. */
int b200moe_ep_barrier(int32_t* const* flag_blocks, int P, int my_rank, int slot, int epoch, uint64_t limit_ns,
                       int32_t* status, b200moe_stream_t stream);
int b200moe_enable_peer_access(int peer_device);
/* b200moe_ipc_export: the 64-byte IPC handle of the cudaMalloc allocation containing dev_ptr
 * and dev_ptr's byte offset in it.  b200moe_ipc_open: map such an allocation into this
 * process; call with this rank's device current.  b200moe_peer_probe copies one word into
 * the mapped buffer and back with the copy engine (synchronous, set-up time only) and
 * returns 0 when the mapping works; local_scratch8 is 8 bytes of this rank's device memory. */
int b200moe_ipc_export(const void* dev_ptr, void* handle_out64, uint64_t* offset_out);
int b200moe_ipc_open(const void* handle64, void** base);
int b200moe_ipc_close(void* base);
int b200moe_peer_probe(void* peer_ptr, void* local_scratch8);

/* Dense D = alpha * A @ B^T + beta * C with the grouped kernel's G = 1 mode.
 * A [M,K], B [N,K] IEEE half (float16), C and D [M,N] float32, row-major; C may be NULL
 * when beta == 0.  Same arguments as
 *   launch_sm100_gemm_f16_tma(void* A, void* B, void* C, void* D, int M, int N, int K,
 *                             float alpha, float beta, cudaStream_t)
 * kernels/blackwell/cute_gemm_02_tma/sm100_gemm.h:33-36, without its alignment rules
 * (M % 128, N % 256, K % 64): any M, N and K % 8 == 0 work, and the stream argument is honoured. */
int b200moe_sm100_gemm_f16(const void* A, const void* B, const void* C, void* D, int M, int N, int K, float alpha,
                           float beta, b200moe_stream_t stream);

/* Backward of the grouped GEMM:
 *   grad_x[rows of g] = grad_y[rows of g, block g] @ w[g]            [M, K] bf16
 *   grad_w[g]         = grad_y[rows of g, block g]^T @ x[rows of g]  [G, N, K] bf16 (zeros for empty groups)
 * grad_y is [M, N*G] (block layout: grad_y_ld = N*G, grad_y_col_group_stride = N) or [M, N]
 * (grad_y_ld = N, stride 0), bf16.  Rows of grad_x past sum(m_sizes) are not written.
 * Replaces grouped_gemm_backward(grad_output, x, w, m_sizes)
 *   kernels/MoE/group_GEMM/triton/tgroup_gemm_backwards.py:382 (per-group definition:
 *   testing/pytorch_reference_backwards.py:165-197).  grad_y, x and w are read where they lie (N, K,
 * grad_y_ld and grad_y_col_group_stride must be multiples of 8, else B200MOE_EALIGN); `workspace`
 * (b200moe_backward_workspace_bytes: 128 * G * (N + K) bytes and some slack) holds the zero-padded copies of
 * the groups' last partial 64-row blocks that grad_w contracts over. */
int b200moe_backward_workspace_bytes(int M, int N, int K, int G, size_t* bytes);
int b200moe_grouped_gemm_backward(const void* grad_y, const void* x, const void* w, const int32_t* m_sizes,
                                  void* grad_x, void* grad_w, int M, int N, int K, int G, int64_t grad_y_ld,
                                  int64_t grad_y_col_group_stride, void* workspace, size_t workspace_bytes,
                                  int cta_group, int32_t* status, b200moe_stream_t stream);

/* Failure-path self-test: launches one small kernel whose only wait can never be
 * satisfied and whose limit is limit_ns (1 .. 2e9).  After the limit the kernel stops
 * polling, writes B200MOE_SSELFTEST to *status and returns; nothing faults and the
 * context stays usable.  Every wait inside the GEMM kernels ends the same way (codes
 * 16..19, limit 0.4 s).  No counterpart in the reference, which has no bounded waits. */
int b200moe_selftest_wait_timeout(uint64_t limit_ns, int32_t* status, b200moe_stream_t stream);

/* Diagnostic without a counterpart in the reference: the raw rate of tcgen05.ld.  `ctas` CTAs of `warps` (4 or
 * 8) warps each read one 128-lane x 256-column fp32 accumulator (128 KiB of tensor memory) `iters` times with
 * 32x32b.x32 loads, `in_flight` (1, 2 or 4) loads issued before each wait; cycles[cta] (device memory, `ctas`
 * entries) receives the SM clock ticks of the loop.  128 KiB * iters / cycles is the bytes per clock an
 * epilogue, or the per-K-block promotion of the block-wise FP8 kernel, can at best drain. */
int b200moe_selftest_tmem_read(int warps, int in_flight, int iters, int ctas, long long* cycles,
                               b200moe_stream_t stream);

/* Routing: stable counting sort of ids[R] (R = tokens*top_k, flat index t*top_k + j)
 * by expert.  m_sizes[E], offsets[E+1], perm[R] (sorted position -> flat index),
 * inv_perm[R] (flat index -> sorted position, -1 for an id outside [0,E)).
 * Takes the place of vLLM's moe_align_block_size as called at
 * kernels/triton/inference/col_major_moe_gemm/v0_moe_fused.py:138-180, without the
 * padding (the GEMM handles ragged groups).  E <= 2048.  `workspace` is scratch of at
 * least b200moe_route_workspace_bytes(R, E) bytes. */
int b200moe_route_workspace_bytes(int R, int E, size_t* bytes);
int b200moe_route(const int32_t* ids, int R, int E, int32_t* m_sizes, int32_t* offsets, int32_t* perm,
                  int32_t* inv_perm, void* workspace, size_t workspace_bytes, int32_t* status,
                  b200moe_stream_t stream);

/* b200moe_route for callers that have no device buffer to lend and no way to get one.
 * (No counterpart in the reference: it exists for hosts such as an inference server
 * that has handed every free byte of HBM to its own cache pool, or a plugin that runs
 * under an allocator it does not own.  There cudaMalloc can fail outright, and even
 * when it succeeds it stalls the whole device.)  Same inputs, outputs and ordering
 * as b200moe_route; the chunk counts live in a 1 MiB array that is part of the library
 * image, so every GPU that loads the library holds that 1 MiB until the process exits.
 * Limit: chunks * E <= 262144, where chunks = ceil(R / max(256, 32*ceil(R/32768)));
 * in practice any R with E <= 256, or E <= 2048 with R <= 32768.  Beyond that the call
 * returns B200MOE_ETOOLARGE and enqueues nothing.  It never calls cudaMalloc, cudaFree
 * or any allocating library routine.
 * The first call on each device looks up the array's device address (the device must
 * be current); make that first call before starting any stream capture.  All calls on a
 * device share the one array: two calls whose kernels can overlap on the GPU (different
 * streams, no ordering between them) race on it.  Nothing in it has to start at zero:
 * each call overwrites every entry it later reads. */
int b200moe_route_noalloc(const int32_t* ids, int R, int E, int32_t* m_sizes, int32_t* offsets, int32_t* perm,
                          int32_t* inv_perm, int32_t* status, b200moe_stream_t stream);

/* The padded layout of moe_align_block_size(topk_ids, block_size, num_experts)
 * (kernels/triton/inference/col_major_moe_gemm/v0_moe_fused.py:138-180), for code written
 * against that format: sorted_ids[R + E*(block_size-1)] = routed rows grouped by expert,
 * each expert padded to a multiple of block_size with the pad id R; expert_ids[>= R/block_size + E]
 * = expert of every block (entries past the used blocks are not written); num_tokens_post_pad[1]. */
int b200moe_moe_align_workspace_bytes(int R, int E, size_t* bytes);
int b200moe_moe_align_block_size(const int32_t* ids, int R, int E, int block_size, int32_t* sorted_ids,
                                 int32_t* expert_ids, int32_t* num_tokens_post_pad, void* workspace,
                                 size_t workspace_bytes, int32_t* status, b200moe_stream_t stream);

/* dst[p, :] = src[idx[p] / div, :] for p < rows; row_bytes bytes per row.  The
 * indexed load the reference's GEMM does per tile (v0_moe_fused.py:95, offs_token //
 * top_k), as one pass.  Entries with idx < 0 or a source row >= src_rows are skipped. */
int b200moe_gather_rows(const void* src, const int32_t* idx, int div, void* dst, int rows, int64_t row_bytes,
                        int src_rows, b200moe_stream_t stream);

/* out[r, 0..d) = silu(in[r, 0..d)) * in[r, d..2d), bf16 (ops.silu_and_mul, v0_moe_fused.py:284). */
int b200moe_swiglu(const void* in, void* out, int64_t rows, int d, b200moe_stream_t stream);

/* out[t, :] = sum_j weight[t,j] * y[inv_perm[t*k+j], :]  (bf16 in/out, fp32 sum in
 * ascending j; weight may be NULL = 1).  The routed-weight multiply and torch.sum of
 * v0_moe_fused.py:122-126, :291-296. */
int b200moe_combine_topk(const void* y, const int32_t* inv_perm, const float* weight, void* out, int T, int k,
                         int H, int y_rows, b200moe_stream_t stream);

/* 1x128 e4m3 quantiser: scale = max(amax,1e-12)/448, q = clamp(x/scale, +-448).
 * x [rows,K] bf16 (x_is_fp32 = 0) or fp32 (1); q [rows,K] e4m3; scales [rows,K/128].
 * float8_groupwise_quantize, kernels/triton/inference/fp8/float8_groupwise_quant.py:53. */
int b200moe_quant_1x128(const void* x, int x_is_fp32, void* q, float* scales, int64_t rows, int K,
                        b200moe_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
