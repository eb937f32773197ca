// Weight gradient of the grouped GEMM:  dW[g] = dY[rows of g]^T @ X[rows of g]   ([N, K] per group),
// the second half of grouped_gemm_backward (kernels/MoE/group_GEMM/triton/tgroup_gemm_backwards.py:382;
// per-group definition in testing/pytorch_reference_backwards.py:165-197).
//
// The contraction runs over the ragged row dimension m_g.  dY and X are read where they lie, as MN-major
// operands (make_sw128_mnmajor_desc: the operand's own dimension, n or k, is the contiguous one, the
// contraction index m walks the rows), 64 rows of the group per stage, so nothing is transposed.  A group's
// last block may be partial; its rows would run into the next group, so tail_pack_kernel first copies every
// group's partial last block (fewer than 64 rows) into a zero-padded 64-row block of a small side buffer
// ([G*64, N] and [G*64, K]; an empty group gets an all-zero block, which makes its dW zero), and the producer
// fetches that one block from the side buffer.  Nothing else is copied.
//
// The kernel uses the forward kernel's TMA ring, tcgen05 pipeline and CTA-pair tiles; only the tile walk
// differs: every group owns the same number of (n, k) tiles and the K loop length is the group's row count / 64,
// rounded up (1 for an empty group).
#include "gg_common.cuh"

namespace b200moe {

constexpr int kDwThreads = 192;
constexpr int kDwEpiWarps = 4;

struct DWParams {
    const int32_t* m_sizes;
    void* dw;           // [G, N, K] bf16
    int32_t* status;
    int M, N, K, G;     // M = rows of x / dY; N, K = weight dims
    int tiles_n, tiles_k;
    uint32_t idesc;
    int overlapped;                 // launched beside the independent kernel in front of it: wait for that one before exiting
    long long dy_col_group_stride;  // first column of group g's block of dY = g * this
};

// Run by one warp: row_off[g] = first row of group g (row_off[G] = rows in all groups), kcnt[g] = 64-row
// blocks to contract (1 for an empty group: the all-zero block of the side buffer); *bad_out is set when a
// size is negative or the sizes add up to more than M.
__device__ __forceinline__ void build_row_layout(const int32_t* m_sizes, int G, int M, int lane, int* row_off,
                                                 int* kcnt, int* bad_out) {
    int rows = 0, bad = 0;
    for (int base = 0; base < G; base += 32) {
        const int g = base + lane;
        int m = g < G ? m_sizes[g] : 0;
        if (m < 0) {
            bad = 1;
            m = 0;
        }
        int rs = m;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int r2 = __shfl_up_sync(0xffffffffu, rs, d);
            if (lane >= d) rs += r2;
        }
        if (g < G) {
            row_off[g] = rows + rs - m;
            kcnt[g] = m == 0 ? 1 : (m + 63) >> 6;
        }
        rows += __shfl_sync(0xffffffffu, rs, 31);
        if (rows > M) bad = 1;
    }
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) {
        row_off[G] = rows;
        *bad_out = bad;
    }
    __syncwarp();
}

struct DwSmemTail {
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    int invalid;
    int kcnt[kMaxGroups + 1];     // 64-row blocks the group contracts
    int row_off[kMaxGroups + 1];  // first row of the group in dY / X
};

template <int CTAS>
constexpr size_t dw_smem_bytes() {
    return 1024 + StageCfg<CTAS, 0>::kRingBytes + sizeof(DwSmemTail);
}

// Rows of group g's last block that are real: 0 = the block is whole (no side-buffer copy), 1..63 = that many
// rows and zeros after them, 64 = empty group (the side buffer holds 64 zero rows to contract).
__device__ __forceinline__ int tail_rows_of(int m) { return m <= 0 ? 64 : (m & 63); }

// Side buffer: block g of dy_tail [G*64, N] and x_tail [G*64, K] is the zero-padded copy of
// the group's partial last block.  grid = (G, ceil((N + K) / 8 / 256) rounded into y), 256 threads; every thread
// moves 16 bytes (8 bf16) of one column chunk for all 64 rows.
__global__ void __launch_bounds__(256)
tail_pack_kernel(const __nv_bfloat16* __restrict__ dy, long long dy_ld, long long dy_col_group_stride,
                 const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ m_sizes, int G, int M, int N, int K,
                 __nv_bfloat16* __restrict__ dy_tail, __nv_bfloat16* __restrict__ x_tail) {
    const int g = blockIdx.x;
    __shared__ int s_row_end;
    if (threadIdx.x < 32) {  // rows up to and including group g
        int sum = 0;
        for (int i = threadIdx.x; i <= g; i += 32) sum += max(m_sizes[i], 0);
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
        if (threadIdx.x == 0) s_row_end = sum;
    }
    __syncthreads();
    const int row_end = s_row_end, m = max(m_sizes[g], 0);
    if (row_end > M) return;  // invalid sizes: the GEMM kernel reports them and writes nothing
    const int valid = tail_rows_of(m);
    if (valid == 0) return;  // whole last block: read in place
    const int real = valid == 64 ? 0 : valid;
    const long long first = static_cast<long long>(row_end) - real;  // first row of the partial block
    const int chunk = blockIdx.y * 256 + threadIdx.x;                // 8-element column chunk over [dY | X]
    const int n_chunks = N / 8, k_chunks = K / 8;
    if (chunk >= n_chunks + k_chunks) return;
    const bool is_dy = chunk < n_chunks;
    const int c = (is_dy ? chunk : chunk - n_chunks) * 8;
    const __nv_bfloat16* src = is_dy ? dy + first * dy_ld + g * dy_col_group_stride + c : x + first * K + c;
    const long long src_ld = is_dy ? dy_ld : K;
    __nv_bfloat16* dst = is_dy ? dy_tail + static_cast<long long>(g) * 64 * N + c
                               : x_tail + static_cast<long long>(g) * 64 * K + c;
    const int dst_ld = is_dy ? N : K;
    for (int r = 0; r < 64; ++r) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < real) v = *reinterpret_cast<const uint4*>(src + r * src_ld);
        *reinterpret_cast<uint4*>(dst + static_cast<long long>(r) * dst_ld) = v;
    }
}

// tm_a = dY [M rows, ld cols], tm_b = X [M rows, K cols], tm_a_tail = dy_tail [G*64, N], tm_b_tail = x_tail
// [G*64, K], all 2-D maps with boxes of 64 rows x 64 columns.
template <int CTAS>
__global__ void __launch_bounds__(kDwThreads, 1)
gg_dw_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
             const __grid_constant__ CUtensorMap tm_a_tail, const __grid_constant__ CUtensorMap tm_b_tail,
             const DWParams p) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL)
    using Cfg = StageCfg<CTAS, 0>;
    constexpr int kTileRows = kRowsPerCta * CTAS;
    constexpr uint32_t kTxBytes = static_cast<uint32_t>(Cfg::kStageBytes) * CTAS;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t ring_addr = (raw_addr + 1023u) & ~1023u;
    DwSmemTail* st = reinterpret_cast<DwSmemTail*>(smem_raw + (ring_addr - raw_addr) + Cfg::kRingBytes);
    volatile int* abort_flag = &st->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = CTAS == 1 ? 0u : cluster_ctarank();
    const int cluster_id = blockIdx.x / CTAS;
    const int num_clusters = gridDim.x / CTAS;

    if (threadIdx.x == 0) {
        st->abort_flag = 0;
        st->invalid = 0;
    }
    __syncthreads();
    if (warp == 0) {
        build_row_layout(p.m_sizes, p.G, p.M, lane, st->row_off, st->kcnt, &st->invalid);
        if (lane == 0) {
            if (st->invalid) report(p.status, kStatusBadGroupSizes);
            for (int s = 0; s < Cfg::kStages; ++s) {
                mbar_init(&st->full[s], 1);
                mbar_init(&st->empty[s], 1);
            }
            for (int b = 0; b < 2; ++b) {
                mbar_init(&st->acc_full[b], 1);
                mbar_init(&st->acc_empty[b], kDwEpiWarps * CTAS);
            }
            mbar_init_fence();
            prefetch_tensormap(&tm_a);
            prefetch_tensormap(&tm_b);
        }
    } else if (warp == 1) {
        tmem_alloc<CTAS>(&st->tmem_base, kTmemCols);
        tmem_relinquish<CTAS>();
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (CTAS == 2) cluster_sync_all();
    tc_fence_after();

    const uint32_t tmem_base = st->tmem_base;
    const int tiles_per_group = p.tiles_n * p.tiles_k;
    const int total_tiles = st->invalid ? 0 : p.G * tiles_per_group;

    if (warp == 0) {
        // TMA producer: the warp walks the loop, one elected lane issues the copies
        {
            const bool leader = elect_one();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = cluster_id; ok && t < total_tiles; t += num_clusters) {
                const int g = t / tiles_per_group, local = t - g * tiles_per_group;
                const int n_idx = local % p.tiles_n, k_idx = local / p.tiles_n;
                const int row0 = n_idx * kTileRows + static_cast<int>(cta_rank) * kRowsPerCta;
                const int kcol0 = k_idx * kTileN;
                const int nkb = st->kcnt[g];
                // the group's rows, and whether its last block comes from the side buffer
                const int grow0 = st->row_off[g];
                const bool has_tail = tail_rows_of(st->row_off[g + 1] - grow0) != 0;
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!__all_sync(0xffffffffu, mbar_wait(&st->empty[stage], phase ^ 1u, abort_flag))) {
                        report(p.status, kStatusTimeoutProducer);
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = ring_addr + stage * Cfg::kStageBytes;
                    const uint32_t b_dst = a_dst + kABytes;
                    // boxes of 64 rows x 64 columns, 8192 bytes each: this CTA's 128 columns of dY (its rows
                    // of dW) and its share of the tile's 256 columns of X
                    const bool tail = has_tail && kb == nkb - 1;
                    const CUtensorMap* ma = tail ? &tm_a_tail : &tm_a;
                    const CUtensorMap* mb = tail ? &tm_b_tail : &tm_b;
                    const int r = tail ? g * 64 : grow0 + kb * 64;
                    const int ac = row0 + (tail ? 0 : static_cast<int>(g * p.dy_col_group_stride));
                    const int bc = kcol0 + (CTAS == 2 ? static_cast<int>(cta_rank) * 128 : 0);
                    const uint32_t bar =
                        CTAS == 1 ? smem_u32(&st->full[stage]) : mapa_shared(smem_u32(&st->full[stage]), 0);
                    if (leader) {
                        if (cta_rank == 0) mbar_arrive_expect_tx(&st->full[stage], kTxBytes);
                        if constexpr (CTAS == 1) {
                            tma_load_2d(ma, bar, a_dst, ac, r);
                            tma_load_2d(ma, bar, a_dst + 8192, ac + 64, r);
#pragma unroll
                            for (int j = 0; j < 4; ++j) tma_load_2d(mb, bar, b_dst + j * 8192, bc + j * 64, r);
                        } else {
                            tma_load_2d_pair(ma, bar, a_dst, ac, r);
                            tma_load_2d_pair(ma, bar, a_dst + 8192, ac + 64, r);
                            tma_load_2d_pair(mb, bar, b_dst, bc, r);
                            tma_load_2d_pair(mb, bar, b_dst + 8192, bc + 64, r);
                        }
                    }
                    __syncwarp();
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // the whole warp walks the loop (warp-uniform descriptors), one elected lane issues
        if (cta_rank == 0) {
            const bool leader = elect_one();
            int stage = 0, buf = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int t = cluster_id; ok && t < total_tiles; t += num_clusters) {
                const int nkb = st->kcnt[t / tiles_per_group];
                if (!__all_sync(0xffffffffu, mbar_wait(&st->acc_empty[buf], acc_phase ^ 1u, abort_flag))) {
                    report(p.status, kStatusTimeoutMmaAcc);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * kTileN);
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!__all_sync(0xffffffffu, mbar_wait(&st->full[stage], phase, abort_flag))) {
                        report(p.status, kStatusTimeoutMmaFull);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = ring_addr + stage * Cfg::kStageBytes;
                    const uint64_t a_desc = make_sw128_mnmajor_desc(a_addr);
                    const uint64_t b_desc = make_sw128_mnmajor_desc(a_addr + kABytes);
                    // per MMA: 16 rows of 128 bytes of each tile, +128 in the descriptor's 16-byte units
                    constexpr uint32_t kStep = 128u;
                    if (leader) {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma<CTAS, false>(d_tmem, a_desc + kStep * k, b_desc + kStep * k, p.idesc,
                                              (kb > 0 || k > 0) ? 1u : 0u);
                        umma_commit<CTAS>(&st->empty[stage]);
                    }
                    __syncwarp();
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                if (leader) umma_commit<CTAS>(&st->acc_full[buf]);
                __syncwarp();
                buf ^= 1;
                if (buf == 0) acc_phase ^= 1u;
            }
        }
    } else {
        const int quarter = warp & 3;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t acc_empty_leader =
            CTAS == 1 ? smem_u32(&st->acc_empty[0]) : mapa_shared(smem_u32(&st->acc_empty[0]), 0);
        __nv_bfloat16* const dw = static_cast<__nv_bfloat16*>(p.dw);
        int buf = 0;
        uint32_t acc_phase = 0;
        for (int t = cluster_id; t < total_tiles; t += num_clusters) {
            const int g = t / tiles_per_group, local = t - g * tiles_per_group;
            const int n_idx = local % p.tiles_n, k_idx = local / p.tiles_n;
            int ok = 1;
            if (lane == 0) ok = mbar_wait(&st->acc_full[buf], acc_phase, abort_flag) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (lane == 0) report(p.status, kStatusTimeoutEpilogue);
                break;
            }
            tc_fence_after();
            const int row = n_idx * kTileRows + static_cast<int>(cta_rank) * kRowsPerCta + quarter * 32 + lane;
            const bool row_ok = row < p.N;
            const uint32_t t_acc = tmem_base + lane_base + static_cast<uint32_t>(buf * kTileN);
            __nv_bfloat16* const out_row = dw + (static_cast<size_t>(g) * p.N + (row_ok ? row : 0)) * p.K;
            const int col0 = k_idx * kTileN;
#pragma unroll 1
            for (int c = 0; c < kTileN / 32; ++c) {
                const int col = col0 + c * 32;
                if (col >= p.K) break;
                uint32_t v[32];
                float f[32];
                tmem_ld_32x32(t_acc + static_cast<uint32_t>(c * 32), v);
                tmem_ld_wait(v);
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
                if (row_ok) store_row_chunk(out_row, col, p.K, f);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_leader + static_cast<uint32_t>(buf) * 8u);
            buf ^= 1;
            if (buf == 0) acc_phase ^= 1u;
        }
    }

    __syncwarp();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (CTAS == 2) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<CTAS>(tmem_base, kTmemCols);
    }
    if (p.overlapped && threadIdx.x == 0) griddep_wait();
#else
    if (threadIdx.x == 0 && blockIdx.x == 0) report(p.status, kStatusWrongArch);
#endif
}

template <int CTAS>
static int launch_dw(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_a_tail,
                     const CUtensorMap& tm_b_tail, const DWParams& p, int sms, cudaStream_t stream) {
    auto kernel = gg_dw_kernel<CTAS>;
    constexpr size_t smem = dw_smem_bytes<CTAS>();
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured_dev = dev;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>((sms / CTAS) * CTAS), 1, 1);
    cfg.blockDim = dim3(kDwThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.overlapped ? 2 : 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b, tm_a_tail, tm_b_tail, p);
    if (e == cudaSuccess) note_launch();
    return static_cast<int>(e);
}

// A [rows, ld] bf16 matrix read as an MN-major operand: boxes of 64 rows x 64 columns, 128-byte swizzle.
static int encode_mn_map_2d(CUtensorMap* m, const void* base, long long rows, long long ld) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return kErrNoDriverEntry;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(ld), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    cuuint32_t box[2] = {64, 64};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : kErrTensorMap;
}

size_t dw_workspace_bytes(int N, int K, int G) {
    return 2ull * 64ull * static_cast<size_t>(G) * (static_cast<size_t>(N) + K) + 256;
}

// dy [M, dy_ld] (group g's block starts at column g * dy_col_group_stride), x [M, K], dw [G, N, K], all bf16 and
// read / written in place; tail_ws: dw_workspace_bytes(N, K, G) bytes, 16-byte aligned, filled by
// dw_tail_pack_launch with the same arguments.
static int check_dw_args(const void* dy, long long dy_ld, long long dy_col_group_stride, const void* x,
                         const int32_t* m_sizes, int M, int N, int K, int G, const void* tail_ws) {
    if (dy == nullptr || x == nullptr || m_sizes == nullptr || tail_ws == nullptr || M <= 0 || N <= 0 || K <= 0 ||
        G <= 0 || dy_ld < N || dy_col_group_stride < 0)
        return kErrBadArgument;
    if (G > kMaxGroups) return kErrTooManyGroups;
    if (N % 8 != 0 || K % 8 != 0 || dy_ld % 8 != 0 || dy_col_group_stride % 8 != 0 ||
        (reinterpret_cast<uintptr_t>(dy) & 15u) || (reinterpret_cast<uintptr_t>(x) & 15u) ||
        (reinterpret_cast<uintptr_t>(tail_ws) & 15u))
        return kErrAlignment;
    return 0;
}

int dw_tail_pack_launch(const void* dy, long long dy_ld, long long dy_col_group_stride, const void* x,
                        const int32_t* m_sizes, int M, int N, int K, int G, void* tail_ws, cudaStream_t stream) {
    if (int e = check_dw_args(dy, dy_ld, dy_col_group_stride, x, m_sizes, M, N, K, G, tail_ws)) return e;
    __nv_bfloat16* dy_tail = static_cast<__nv_bfloat16*>(tail_ws);
    __nv_bfloat16* x_tail = dy_tail + 64ull * G * N;  // 128 * G * N bytes in: still 16-byte aligned
    const dim3 grid(static_cast<unsigned>(G), static_cast<unsigned>(((N + K) / 8 + 255) / 256), 1);
    tail_pack_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(dy), dy_ld, dy_col_group_stride,
                                               static_cast<const __nv_bfloat16*>(x), m_sizes, G, M, N, K, dy_tail,
                                               x_tail);
    if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return static_cast<int>(e);
    note_launch();
    return 0;
}

int grouped_gemm_dw_launch(const void* dy, long long dy_ld, long long dy_col_group_stride, const void* x,
                           const int32_t* m_sizes, void* dw, int M, int N, int K, int G, const void* tail_ws,
                           int cta_group, bool overlapped, int32_t* status, cudaStream_t stream) {
    if (dw == nullptr) return kErrBadArgument;
    if (int e = check_dw_args(dy, dy_ld, dy_col_group_stride, x, m_sizes, M, N, K, G, tail_ws)) return e;
    DeviceInfo di;
    if (int e = get_device_info(&di)) return e;
    if (di.cc_major != 10) return kErrWrongDevice;
    const __nv_bfloat16* dy_tail = static_cast<const __nv_bfloat16*>(tail_ws);
    const __nv_bfloat16* x_tail = dy_tail + 64ull * G * N;
    CUtensorMap tm_a, tm_b, tm_a_tail, tm_b_tail;
    if (int e = encode_mn_map_2d(&tm_a, dy, M, dy_ld)) return e;
    if (int e = encode_mn_map_2d(&tm_b, x, M, K)) return e;
    if (int e = encode_mn_map_2d(&tm_a_tail, dy_tail, 64ll * G, N)) return e;
    if (int e = encode_mn_map_2d(&tm_b_tail, x_tail, 64ll * G, K)) return e;
    const int ctas = cta_group == 1 ? 1 : cta_group == 2 ? 2 : (N >= 256 ? 2 : 1);
    DWParams p;
    p.m_sizes = m_sizes;
    p.dw = dw;
    p.status = status;
    p.M = M;
    p.N = N;
    p.K = K;
    p.G = G;
    p.tiles_n = (N + 128 * ctas - 1) / (128 * ctas);
    p.tiles_k = (K + kTileN - 1) / kTileN;
    p.idesc = make_idesc(false, 128 * ctas, kTileN, false, true, true);
    p.overlapped = overlapped ? 1 : 0;
    p.dy_col_group_stride = dy_col_group_stride;
    return ctas == 1 ? launch_dw<1>(tm_a, tm_b, tm_a_tail, tm_b_tail, p, di.sms, stream)
                     : launch_dw<2>(tm_a, tm_b, tm_a_tail, tm_b_tail, p, di.sms, stream);
}

}  // namespace b200moe
