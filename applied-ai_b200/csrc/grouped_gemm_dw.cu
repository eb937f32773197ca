// Weight gradient of the grouped GEMM:  dW[g] = dY[rows of g]^T @ X[rows of g]   ([N, K] per group),
// the second half of grouped_gemm_backward (kernels/MoE/group_GEMM/triton/tgroup_gemm_backwards.py:382;
// per-group definition in testing/pytorch_reference_backwards.py:165-197).
//
// The contraction runs over the ragged row dimension m_g, so both operands are first brought
// into "rows contiguous" form by transpose_pad_kernel (below): dYT [N, Mpad] and XT [K, Mpad],
// where every group's columns start at a multiple of 64 and are zero-padded to a multiple of
// 64, and one extra block of 64 zero columns stands in for empty groups.  After that the
// problem has the forward kernel's shape — D[n, k] += A[n, m] * B[k, m]^T with both operands
// K-major — and uses the same TMA ring, tcgen05 pipeline and CTA-pair tiles; only the tile
// walk differs: every group owns the same number of (n, k) tiles and the K loop length is the
// group's padded row count / 64.
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
};

// Padded column layout shared by the transpose kernel and the dW kernel.
// koff[g] = first padded column of group g, kcnt[g] = 64-column blocks to contract
// (empty groups contract the one all-zero block that follows the last group).
// Optional outputs: pstart[g] = padded start of every group in order (empty groups have
// pstart[g] == pstart[g+1]; pstart[G] = total), row_off[g] = first real row of the group.
__device__ __forceinline__ void build_padded_layout(const int32_t* m_sizes, int G, int M, int lane, int* koff,
                                                    int* kcnt, int* total_blocks, int* bad_out,
                                                    int* pstart = nullptr, int* row_off = nullptr) {
    int carry = 0, rows = 0, bad = 0;
    for (int base = 0; base < G; base += 32) {
        const int g = base + lane;
        int m = g < G ? m_sizes[g] : 0;
        if (m < 0) {
            bad = 1;
            m = 0;
        }
        const int blocks = (m + 63) >> 6;
        int bs = blocks, rs = m;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int b2 = __shfl_up_sync(0xffffffffu, bs, d);
            const int r2 = __shfl_up_sync(0xffffffffu, rs, d);
            if (lane >= d) {
                bs += b2;
                rs += r2;
            }
        }
        if (g < G) {
            koff[g] = (carry + bs - blocks) << 6;
            kcnt[g] = blocks;
            if (pstart != nullptr) pstart[g] = (carry + bs - blocks) << 6;
            if (row_off != nullptr) row_off[g] = rows + rs - m;
        }
        carry += __shfl_sync(0xffffffffu, bs, 31);
        rows += __shfl_sync(0xffffffffu, rs, 31);
        if (rows > M) bad = 1;
    }
    bad = __any_sync(0xffffffffu, bad);
    __syncwarp();
    for (int g = lane; g < G; g += 32)
        if (kcnt[g] == 0) {  // empty group: contract the zero block
            koff[g] = carry << 6;
            kcnt[g] = 1;
        }
    if (lane == 0) {
        *total_blocks = carry;
        *bad_out = bad;
        if (pstart != nullptr) pstart[G] = carry << 6;
        if (row_off != nullptr) row_off[G] = rows;
    }
}

// One 64x64 bf16 tile through shared memory, run by 256 threads.
// Reads src[r][c] for r < rows_in, c < cols_in (zeros elsewhere) with 16-byte loads when the
// tile is whole and aligned, writes dst[c][r] for c < rows_out, r < cols_out the same way.
__device__ __forceinline__ void transpose_tile_64(const __nv_bfloat16* src, long long src_ld, int rows_in, int cols_in,
                                                  __nv_bfloat16* dst, long long dst_ld, int rows_out, int cols_out,
                                                  __nv_bfloat16 (*tile)[66]) {
    const bool vec_in = rows_in > 0 && cols_in == 64 && (src_ld % 8) == 0 &&
                        (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
    if (vec_in) {
        for (int idx = threadIdx.x; idx < 64 * 8; idx += blockDim.x) {
            const int r = idx >> 3, v = idx & 7;
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            if (r < rows_in) raw = __ldg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * src_ld) + v);
            const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
            uint32_t* t = reinterpret_cast<uint32_t*>(&tile[r][v * 8]);  // rows are 132 bytes apart: 4-byte aligned
            t[0] = w[0]; t[1] = w[1]; t[2] = w[2]; t[3] = w[3];
        }
    } else {
        for (int idx = threadIdx.x; idx < 64 * 64; idx += blockDim.x) {
            const int r = idx >> 6, c = idx & 63;
            tile[r][c] = (r < rows_in && c < cols_in) ? src[static_cast<size_t>(r) * src_ld + c] : __float2bfloat16(0.0f);
        }
    }
    __syncthreads();
    const bool vec_out = cols_out == 64 && (dst_ld % 8) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
    if (vec_out) {
        for (int idx = threadIdx.x; idx < 64 * 8; idx += blockDim.x) {
            const int c = idx >> 3, v = idx & 7;  // output row c, 8 consecutive output columns r = 8v..8v+7
            if (c >= rows_out) continue;
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const unsigned short lo = *reinterpret_cast<const unsigned short*>(&tile[v * 8 + 2 * j][c]);
                const unsigned short hi = *reinterpret_cast<const unsigned short*>(&tile[v * 8 + 2 * j + 1][c]);
                w[j] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
            }
            reinterpret_cast<uint4*>(dst + static_cast<size_t>(c) * dst_ld)[v] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
        for (int idx = threadIdx.x; idx < 64 * 64; idx += blockDim.x) {
            const int c = idx >> 6, r = idx & 63;
            if (c < rows_out && r < cols_out) dst[static_cast<size_t>(c) * dst_ld + r] = tile[r][c];
        }
    }
}

// out[c, koff_g + i] = src[off_g + i, col0_g + c]  (i < m_g), zeros in the padding and in the
// extra zero block.  src has `ld` elements per row; col0_g = g * col_group_stride.
// grid: x = padded 64-column blocks (upper bound M/64 + G + 1), y = C / 64 (rounded up).
__global__ void __launch_bounds__(256)
transpose_pad_kernel(const __nv_bfloat16* __restrict__ src, long long ld, long long col_group_stride, int C,
                     const int32_t* __restrict__ m_sizes, int G, int M, __nv_bfloat16* __restrict__ out,
                     long long mpad) {
    __shared__ int koff[kMaxGroups + 1], kcnt[kMaxGroups + 1], pstart[kMaxGroups + 1], row_off[kMaxGroups + 1];
    __shared__ int total_blocks, bad;
    __shared__ __nv_bfloat16 tile[64][66];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) build_padded_layout(m_sizes, G, M, lane, koff, kcnt, &total_blocks, &bad, pstart, row_off);
    __syncthreads();
    if (bad) return;
    const int blk = blockIdx.x;
    if (blk > total_blocks) return;  // blk == total_blocks is the all-zero block
    const int c0 = blockIdx.y * 64;
    int g = 0, i0 = 0, valid = 0;
    if (blk < total_blocks) {
        const int col = blk << 6;
        int lo = 0, hi = G - 1;  // last g with pstart[g] <= col: the group that owns the block
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (pstart[mid] <= col) lo = mid; else hi = mid - 1;
        }
        g = lo;
        i0 = col - pstart[g];
        valid = min(64, (row_off[g + 1] - row_off[g]) - i0);
    }
    // load 64 rows x 64 columns (zeros outside), transposed through shared memory
    const __nv_bfloat16* src_tile =
        src + static_cast<size_t>(row_off[g] + i0) * ld + static_cast<size_t>(g) * col_group_stride + c0;
    __nv_bfloat16* dst_tile = out + static_cast<size_t>(c0) * mpad + (static_cast<size_t>(blk) << 6);
    transpose_tile_64(src_tile, ld, valid, min(64, C - c0), dst_tile, mpad, min(64, C - c0), 64, tile);
}

// Batched plain transpose: dst[b, c, r] = src[b, r, c]  (src [B, R, C], dst [B, C, R]).
__global__ void __launch_bounds__(256)
transpose_batched_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, int R, int C) {
    __shared__ __nv_bfloat16 tile[64][66];
    const size_t base = static_cast<size_t>(blockIdx.z) * R * C;
    const int r0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
    transpose_tile_64(src + base + static_cast<size_t>(r0) * C + c0, C, min(64, R - r0), min(64, C - c0),
                      dst + base + static_cast<size_t>(c0) * R + r0, R, min(64, C - c0), min(64, R - r0), tile);
}

struct DwSmemTail {
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    int invalid;
    int total_blocks;
    int koff[kMaxGroups + 1];
    int kcnt[kMaxGroups + 1];
};

template <int CTAS>
constexpr size_t dw_smem_bytes() {
    return 1024 + StageCfg<CTAS, 0>::kRingBytes + sizeof(DwSmemTail);
}

// tm_a: dYT [N rows, Mpad cols] (2-D map, box 128 x 64); tm_b: XT viewed as [1, K rows, Mpad cols].
template <int CTAS>
__global__ void __launch_bounds__(kDwThreads, 1)
gg_dw_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const DWParams p) {
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
        build_padded_layout(p.m_sizes, p.G, p.M, lane, st->koff, st->kcnt, &st->total_blocks, &st->invalid);
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
                const int koff = st->koff[g], nkb = st->kcnt[g];
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!__all_sync(0xffffffffu, mbar_wait(&st->empty[stage], phase ^ 1u, abort_flag))) {
                        report(p.status, kStatusTimeoutProducer);
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = ring_addr + stage * Cfg::kStageBytes;
                    const uint32_t b_dst = a_dst + kABytes;
                    const int c0 = koff + kb * 64;
                    if constexpr (CTAS == 1) {
                        const uint32_t bar = smem_u32(&st->full[stage]);
                        if (leader) {
                            mbar_arrive_expect_tx(&st->full[stage], kTxBytes);
                            tma_load_2d(&tm_a, bar, a_dst, c0, row0);
                            tma_load_3d(&tm_b, bar, b_dst, c0, kcol0, 0);
                            tma_load_3d(&tm_b, bar, b_dst + kSubBoxBytes, c0, kcol0 + 128, 0);
                        }
                    } else {
                        const uint32_t bar = mapa_shared(smem_u32(&st->full[stage]), 0);
                        if (leader) {
                            if (cta_rank == 0) mbar_arrive_expect_tx(&st->full[stage], kTxBytes);
                            tma_load_2d_pair(&tm_a, bar, a_dst, c0, row0);
                            tma_load_3d_pair(&tm_b, bar, b_dst, c0, kcol0 + static_cast<int>(cta_rank) * 128, 0);
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
                    const uint64_t a_desc = make_sw128_kmajor_desc(a_addr);
                    const uint64_t b_desc = make_sw128_kmajor_desc(a_addr + kABytes);
                    if (leader) {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma<CTAS, false>(d_tmem, a_desc + 2u * k, b_desc + 2u * k, p.idesc,
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
#else
    if (threadIdx.x == 0 && blockIdx.x == 0) report(p.status, kStatusWrongArch);
#endif
}

template <int CTAS>
static int launch_dw(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const DWParams& p, int sms, cudaStream_t stream) {
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
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b, p);
    if (e == cudaSuccess) note_launch();
    return static_cast<int>(e);
}

long long dw_padded_cols(int M, int G) { return ((static_cast<long long>(M) + 63) / 64 + G + 1) * 64; }

int transpose_pad_launch(const void* src, long long ld, long long col_group_stride, int C, const int32_t* m_sizes,
                         int G, int M, void* out, long long mpad, cudaStream_t stream) {
    if (src == nullptr || out == nullptr || m_sizes == nullptr || C <= 0 || G <= 0 || G > kMaxGroups || M < 0 ||
        mpad < dw_padded_cols(M, G))
        return kErrBadArgument;
    const dim3 grid(static_cast<unsigned>(mpad / 64), static_cast<unsigned>((C + 63) / 64), 1);
    transpose_pad_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), ld, col_group_stride, C,
                                                   m_sizes, G, M, static_cast<__nv_bfloat16*>(out), mpad);
    note_launch();
    return static_cast<int>(cudaGetLastError());
}

int transpose_batched_launch(const void* src, void* dst, int B, int R, int C, cudaStream_t stream) {
    if (src == nullptr || dst == nullptr || B <= 0 || R <= 0 || C <= 0 || B > 65535) return kErrBadArgument;
    const dim3 grid(static_cast<unsigned>((R + 63) / 64), static_cast<unsigned>((C + 63) / 64),
                    static_cast<unsigned>(B));
    transpose_batched_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src),
                                                       static_cast<__nv_bfloat16*>(dst), R, C);
    note_launch();
    return static_cast<int>(cudaGetLastError());
}

// dyt [N, mpad], xt [K, mpad] (outputs of transpose_pad_launch with the same m_sizes), dw [G, N, K].
int grouped_gemm_dw_launch(const void* dyt, const void* xt, const int32_t* m_sizes, void* dw, int M, int N, int K,
                           int G, long long mpad, int cta_group, int32_t* status, cudaStream_t stream) {
    if (dyt == nullptr || xt == nullptr || m_sizes == nullptr || dw == nullptr || M < 0 || N <= 0 || K <= 0 ||
        G <= 0 || mpad < dw_padded_cols(M, G) || (mpad % 8) != 0)
        return kErrBadArgument;
    if (G > kMaxGroups) return kErrTooManyGroups;
    if ((reinterpret_cast<uintptr_t>(dyt) & 15u) || (reinterpret_cast<uintptr_t>(xt) & 15u)) return kErrAlignment;
    DeviceInfo di;
    if (int e = get_device_info(&di)) return e;
    if (di.cc_major != 10) return kErrWrongDevice;
    CUtensorMap tm_a, tm_b;
    if (int e = encode_x_map(&tm_a, dyt, N, static_cast<int>(mpad), 2)) return e;
    if (int e = encode_w_map(&tm_b, xt, 1, K, static_cast<int>(mpad), 2)) return e;
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
    p.idesc = make_idesc(false, 128 * ctas, kTileN);
    return ctas == 1 ? launch_dw<1>(tm_a, tm_b, p, di.sms, stream) : launch_dw<2>(tm_a, tm_b, p, di.sms, stream);
}

}  // namespace b200moe
