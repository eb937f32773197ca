// Ragged ("grouped") GEMM for MoE experts on sm_100a:
//     y[rows of group g, :] = x[rows of group g, :] @ w[g]^T
// x is [M, K] row-major, w is [G, N, K] row-major (K-major operands for both), the
// rows of x are partitioned into G consecutive groups by m_sizes[G] (device memory,
// zeros allowed).  This replaces the persistent Triton kernels of the reference
// (dev/triton_groupGEMM/groupgemm.py:131-254 bf16, :270-404 fp8 row-wise;
// kernels/MoE/group_GEMM/triton/tgroup_gemm_forward.py:136-293, :311-482).
//
// Structure of one CTA (192 threads), persistent over output tiles:
//   warp 0      TMA producer: fills a ring of shared-memory stages with a
//               128-row box of x and this CTA's share of a 256-row box of w[g].
//   warp 1      MMA issuer: one thread issues tcgen05.mma (4 per stage) into one of
//               two TMEM accumulators (256 fp32 columns each); tcgen05.commit
//               releases stages and publishes finished accumulators.
//   warps 2..5  epilogue: tcgen05.ld the accumulator, apply scales / SwiGLU,
//               convert to bf16, store the valid rows and columns.
// With CTAS == 2 two CTAs of a cluster form one 256x256 tile: each loads its own 128
// rows of x and its own 128 rows of w[g], the leader issues cta_group::2 MMAs, and
// both epilogues drain their own 128 accumulator rows.  No load is multicast.
//
// Tile order: groups in the order given; inside a group, row blocks vary fastest
// within one 256-column panel of w[g], so tiles that run together share the panel.
// Tile t of the global list belongs to cluster (t mod #clusters): static, no atomics,
// so results are bit-identical from run to run.
#include "gg_common.cuh"

namespace b200moe {

constexpr int kThreads = 192;
constexpr int kEpiWarps = 4;

// ELEM_BYTES: 2 = bf16 operands, 1 = e4m3 operands.
// SCALE: 0 none, 1 row-wise (x_scale[M], w_scale[G*N]).
// EPI: 0 plain, 1 SwiGLU (w[g] = [gate rows 0..I) ; up rows I..2I), output has I columns),
//      2 fp32 output alpha*acc + beta*C (the dense D = alpha*A*B^T + beta*C of
//        kernels/blackwell/cute_gemm_02_tma/sm100_gemm.cu:157-173).
// B_MN: w is [G, K, N] with N contiguous instead of [G, N, K] (y = x @ w[g] without a transpose: the input
//      gradient of the layer reads the forward weights as they lie).  16-bit operands only.
template <int ELEM_BYTES, int CTAS, int SCALE, int EPI, bool B_MN = false>
__global__ void __launch_bounds__(kThreads, 1)
gg_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const GGParams p) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL)
    using Cfg = StageCfg<CTAS, 0>;
    constexpr bool kFp8 = ELEM_BYTES == 1;
    constexpr int kElemsPerStage = kRowBytes / ELEM_BYTES;  // K elements per stage
    constexpr int kTileRows = kRowsPerCta * CTAS;

    extern __shared__ uint8_t smem_raw[];
    const SmemView sv = carve_smem<CTAS, 0>(smem_raw);
    const uint32_t ring_addr = sv.ring_addr;
    SmemTail* st = sv.tail;
    volatile int* abort_flag = &st->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = CTAS == 1 ? 0u : cluster_ctarank();
    const int cluster_id = blockIdx.x / CTAS;
    const int num_clusters = gridDim.x / CTAS;

    // ---- prologue: group tables, barriers, TMEM
    if (threadIdx.x == 0) {
        st->abort_flag = 0;
        st->invalid = 0;
    }
    __syncthreads();
    if (warp == 0) {
        build_tables_and_barriers<CTAS, 0>(st, p, lane, kTileRows, kEpiWarps * CTAS);
        if (lane == 0) {
            prefetch_tensormap(&tm_x);
            prefetch_tensormap(&tm_w);
        }
    } else if (warp == 1) {
        tmem_alloc<CTAS>(&st->tmem_base, kTmemCols);
        tmem_relinquish<CTAS>();
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (CTAS == 2) cluster_sync_all();  // peer barriers exist before anything signals them
    tc_fence_after();

    const uint32_t tmem_base = st->tmem_base;
    const int total_tiles = st->total_tiles;
    const int num_kb = (p.K + kElemsPerStage - 1) / kElemsPerStage;
    // an independent kernel follows in the stream: its CTAs may take each SM as soon as this kernel's CTA there is done
    if (p.overlap_role == 1 && threadIdx.x == 0) griddep_launch_dependents();
    const WorkSplit ws = make_work_split(total_tiles, num_clusters, CTAS == 2);

    if (warp == 0) {
        // ================= TMA producer (the warp walks the loop, one elected lane issues)
        producer_loop<CTAS, 0, EPI == 1, true, B_MN>(&tm_x, &tm_w, st, ring_addr, p, cta_rank, cluster_id,
                                                     num_clusters, kElemsPerStage, num_kb);
    } else if (warp == 1) {
        // ================= MMA issuer (leader CTA; the warp walks the loop, one elected lane issues)
        if (cta_rank == 0) {
            const bool leader = elect_one();
            int stage = 0, buf = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int wk = cluster_id; ok && wk < ws.total_work; wk += num_clusters) {
                const uint32_t idesc = wk < ws.split_from ? p.idesc : p.idesc_half;
                // waits are warp-collective so that every lane takes the same way out
                if (!__all_sync(0xffffffffu, mbar_wait(&st->acc_empty[buf], acc_phase ^ 1u, abort_flag))) {
                    report(p.status, kStatusTimeoutMmaAcc);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * kTileN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!__all_sync(0xffffffffu, mbar_wait(&st->full[stage], phase, abort_flag))) {
                        report(p.status, kStatusTimeoutMmaFull);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = ring_addr + stage * Cfg::kStageBytes;
                    const uint64_t a_desc = make_sw128_kmajor_desc(a_addr);
                    const uint64_t b_desc =
                        B_MN ? make_sw128_mnmajor_desc(a_addr + kABytes) : make_sw128_kmajor_desc(a_addr + kABytes);
                    // per MMA: 32 bytes along K of a K-major tile (+2 in the descriptor's 16-byte units),
                    // 16 rows of 128 bytes of an MN-major one (+128)
                    constexpr uint32_t kBStep = B_MN ? 128u : 2u;
                    if (leader) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            umma<CTAS, kFp8>(d_tmem, a_desc + 2u * k, b_desc + kBStep * k, idesc,
                                             (kb > 0 || k > 0) ? 1u : 0u);
                        }
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
        // ================= epilogue (4 warps; warp w owns TMEM lanes 32*(w%4)..+31)
        const int quarter = warp & 3;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t acc_empty_leader =
            CTAS == 1 ? smem_u32(&st->acc_empty[0]) : mapa_shared(smem_u32(&st->acc_empty[0]), 0);
        int g = 0, buf = 0;
        uint32_t acc_phase = 0;
        for (int wk = cluster_id; wk < ws.total_work; wk += num_clusters) {
            int t, half;
            decode_work(wk, ws, &t, &half);
            const TileCoord tc = locate_tile(t, g, st->tile_off, st->row_off, kTileRows, p.tile_mode);
            int ok = 1;
            if (lane == 0) ok = mbar_wait(&st->acc_full[buf], acc_phase, abort_flag) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (lane == 0) report(p.status, kStatusTimeoutEpilogue);
                break;
            }
            tc_fence_after();
            const int row = tc.row0 + static_cast<int>(cta_rank) * kRowsPerCta + quarter * 32 + lane;
            const bool row_ok = row < tc.row_end;
            const uint32_t t_acc = tmem_base + lane_base + static_cast<uint32_t>(buf * kTileN);
            float x_scale = 1.0f;
            if constexpr (SCALE == 1) x_scale = row_ok ? p.x_scale[row] : 0.0f;

            constexpr int kOutCols = EPI == 1 ? 128 : kTileN;  // output columns per tile
            constexpr int kOutElem = EPI == 2 ? 4 : 2;         // bytes per output element
            constexpr int kSlabCols = 128 / kOutElem;          // columns in one 128-byte staged run
            // a half tile covers half of the tile's output columns; with SwiGLU its up columns
            // sit 64 (not 128) accumulator columns after the gate columns
            const int tile_cols = half >= 0 ? kOutCols / 2 : kOutCols;
            const int up_off = half >= 0 ? 64 : 128;
            const int col0 = tc.n_idx * kOutCols + (half > 0 ? kOutCols / 2 : 0);  // first output column (within group)
            // Destination row: the row itself, where the caller's row map sends it, or a row of
            // another rank's buffer.
            RowDest rd;
            const bool store_ok = resolve_row_dest(p, row, row_ok, &rd);
            char* const my_row = store_ok ? reinterpret_cast<char*>(rd.base) +
                                                (static_cast<size_t>(rd.drow) * p.ldy +
                                                 static_cast<size_t>(tc.g) * p.y_col_group_stride) * kOutElem
                                          : nullptr;
            const char* const my_c =
                (EPI == 2 && store_ok && p.beta != 0.0f)
                    ? reinterpret_cast<const char*>(p.c_in) + static_cast<size_t>(rd.drow) * p.ldy * sizeof(float)
                    : nullptr;
            const float* const w_scale_g = SCALE == 1 ? p.w_scale + static_cast<size_t>(tc.g) * p.N : nullptr;
            uint4* const stage = sv.warp_stage + (warp - 2) * (kWarpStageBytes / 16);
            const bool to_peers = p.row_tags != nullptr;  // kernel-uniform

#pragma unroll 1
            for (int slab = 0; slab < tile_cols / kSlabCols; ++slab) {
                const int scol = col0 + slab * kSlabCols;
                if (scol >= p.n_out) break;  // warp-uniform: nothing left to store in this tile
#pragma unroll
                for (int part = 0; part < kSlabCols / 32; ++part) {
                    const int c = slab * (kSlabCols / 32) + part;  // 32-column chunk inside the tile
                    const int col = col0 + c * 32;
                    uint32_t v[32];
                    float f[32];
                    tmem_ld_32x32(t_acc + static_cast<uint32_t>(c * 32), v);
                    if constexpr (EPI == 1) {
                        uint32_t u[32];
                        tmem_ld_32x32(t_acc + static_cast<uint32_t>(up_off + c * 32), u);
                        tmem_ld_wait(v);
                        tmem_ld_wait(u);
#pragma unroll
                        for (int j = 0; j < 32; ++j) f[j] = silu_mul(__uint_as_float(v[j]), __uint_as_float(u[j]));
                    } else {
                        tmem_ld_wait(v);
#pragma unroll
                        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
                    }
                    if constexpr (SCALE == 1) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int cj = col + j;
                            const float ws = cj < p.n_out ? __ldg(w_scale_g + cj) : 0.0f;
                            f[j] = f[j] * x_scale * ws;
                        }
                    }
                    if constexpr (EPI == 2) {
                        if (store_ok)
                            store_row_chunk_axpby(reinterpret_cast<float*>(my_row),
                                                  reinterpret_cast<const float*>(my_c), col, p.n_out, f, p.alpha,
                                                  p.beta);
                    } else if (!to_peers) {
                        if (store_ok) store_row_chunk(reinterpret_cast<__nv_bfloat16*>(my_row), col, p.n_out, f);
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            stage_put<128>(stage, lane, part * 4 + q,
                                      make_uint4(pack_bf16x2(f[q * 8 + 0], f[q * 8 + 1]),
                                                 pack_bf16x2(f[q * 8 + 2], f[q * 8 + 3]),
                                                 pack_bf16x2(f[q * 8 + 4], f[q * 8 + 5]),
                                                 pack_bf16x2(f[q * 8 + 6], f[q * 8 + 7])));
                    }
                }
                if constexpr (EPI != 2) {
                    if (to_peers) {
                        __syncwarp();
                        stage_flush<2, 128>(stage, lane,
                                       my_row != nullptr ? my_row + static_cast<size_t>(scol) * kOutElem : nullptr,
                                       min(128, (p.n_out - scol) * kOutElem));
                        __syncwarp();
                    }
                }
            }
            // Accumulator drained: hand it back to the MMA issuer.
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_leader + static_cast<uint32_t>(buf) * 8u);
            buf ^= 1;
            if (buf == 0) acc_phase ^= 1u;
        }
    }

    // ---- teardown: everyone meets, then the allocating warp frees TMEM
    __syncwarp();
    if (*abort_flag) {
        // A wait gave up.  Give copies already issued time to land before the CTA exits.
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (CTAS == 2) cluster_sync_all();  // the peer may still read this CTA's shared memory until here
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<CTAS>(tmem_base, kTmemCols);
    }
    // started early, beside an independent kernel: do not end before that one (what follows waits for this one only)
    if (p.overlap_role == 2 && threadIdx.x == 0) griddep_wait();
#else
    if (threadIdx.x == 0 && blockIdx.x == 0) report(p.status, kStatusWrongArch);
#endif
}

// ------------------------------------------------------------------ host side

template <int ELEM_BYTES, int CTAS, int SCALE, int EPI, bool B_MN = false>
static int launch_variant(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const GGParams& p, int sms,
                          cudaStream_t stream) {
    static_assert(!B_MN || ELEM_BYTES == 2, "MN-major operands exist for 16-bit types only");
    auto kernel = gg_kernel<ELEM_BYTES, CTAS, SCALE, EPI, B_MN>;
    constexpr size_t smem = gg_smem_bytes<CTAS, 0, kEpiWarps * kWarpStageBytes>();
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
    cfg.blockDim = dim3(kThreads, 1, 1);
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
    cfg.numAttrs = p.overlap_role == 2 ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tm_x, tm_w, p);
    if (e == cudaSuccess) note_launch();
    return static_cast<int>(e);
}

int grouped_gemm_launch(const GGLaunch& a) {
    // y may be null when every row leaves through (rank, row) tags: the peer table names the buffers
    if (a.M < 0 || a.N <= 0 || a.K <= 0 || a.G <= 0 || a.x == nullptr || a.w == nullptr ||
        (a.y == nullptr && a.row_tags == nullptr) || (a.m_sizes == nullptr && a.G != 1))
        return kErrBadArgument;
    if (a.G > kMaxGroups) return kErrTooManyGroups;
    if (a.elem_bytes != 1 && a.elem_bytes != 2) return kErrBadArgument;
    if ((static_cast<long long>(a.K) * a.elem_bytes) % 16 != 0) return kErrAlignment;  // TMA row pitch
    if (a.x_col_group_stride != 0 && (a.x_col_group_stride * a.elem_bytes) % 16 != 0) return kErrAlignment;
    if ((reinterpret_cast<uintptr_t>(a.x) & 15u) || (reinterpret_cast<uintptr_t>(a.w) & 15u)) return kErrAlignment;
    if (a.scale_mode == 1 && (a.x_scale == nullptr || a.w_scale == nullptr)) return kErrBadArgument;
    if (a.epilogue == 2 && (a.elem_bytes != 2 || a.scale_mode != 0 || a.y_col_group_stride != 0 ||
                            (a.beta != 0.0f && a.c_in == nullptr) || a.row_map != nullptr || a.row_tags != nullptr))
        return kErrBadArgument;
    if (a.scale_mode != 0 && a.scale_mode != 1) return kErrBadArgument;
    if (a.epilogue == 1 && (a.N % 2 != 0)) return kErrBadArgument;
    if (a.epilogue < 0 || a.epilogue > 2) return kErrBadArgument;
    if (a.row_tags != nullptr && (a.peer_y == nullptr || a.n_peers <= 0 || a.y_rows <= 0)) return kErrBadArgument;
    if (a.epilogue == 1 && a.scale_mode != 0) return kErrBadArgument;
    if (a.w_mn_major && (a.elem_bytes != 2 || a.epilogue != 0 || a.scale_mode != 0)) return kErrBadArgument;
    if (a.w_mn_major && (static_cast<long long>(a.N) * 2) % 16 != 0) return kErrAlignment;  // TMA row pitch of w
    if (a.M == 0) return 0;

    DeviceInfo di;
    if (int e = get_device_info(&di)) return e;
    if (di.cc_major != 10) return kErrWrongDevice;

    CUtensorMap tm_x, tm_w;
    // x may be wider than K (a group's K range is then a column block of it)
    const long long x_ld = a.x_ld > 0 ? a.x_ld : a.K;
    if ((x_ld * a.elem_bytes) % 16 != 0 || x_ld > 0x7fffffffll) return kErrAlignment;
    if (int e = encode_x_map(&tm_x, a.x, a.M, static_cast<int>(x_ld), a.elem_bytes, a.is_f16 != 0)) return e;
    if (a.w_mn_major) {
        if (int e = encode_w_mn_map(&tm_w, a.w, a.G, a.K, a.N, a.is_f16 != 0)) return e;
    } else if (int e = encode_w_map(&tm_w, a.w, a.G, a.N, a.K, a.elem_bytes, a.is_f16 != 0)) {
        return e;
    }

    GGParams p;
    p.m_sizes = a.m_sizes;
    p.y = a.y;
    p.x_scale = a.x_scale;
    p.w_scale = a.w_scale;
    p.status = a.status;
    p.row_map = a.row_map;
    p.row_tags = a.row_tags;
    p.peer_y = a.peer_y;
    p.n_peers = a.n_peers;
    p.y_rows = (a.row_map || a.row_tags) ? a.y_rows : a.M;
    p.M = a.M;
    p.N = a.N;
    p.K = a.K;
    p.G = a.G;
    p.ldy = a.ldy;
    p.x_col_group_stride = a.x_col_group_stride;
    p.y_col_group_stride = a.y_col_group_stride;
    p.n_out = a.epilogue == 1 ? a.N / 2 : a.N;
    p.n_tiles = a.epilogue == 1 ? (p.n_out + 127) / 128 : (p.n_out + kTileN - 1) / kTileN;

    // A CTA pair computes 256 rows at a time; with few rows per group most of that tile
    // would be padding, so small groups use the single-CTA 128-row tile.
    // Auto tiling: CTA pairs from 192 rows per group on average (measured with 32 ragged groups, N=4096,
    // K=7168: 910 vs 794 TFLOP/s at 192 rows per group, 1242 vs 1107 at 1024); below that the 128-row
    // tiles of the single-CTA kernel waste less (skewed 64-row average: 0.142 vs 0.174 ms).
    const int ctas = a.cta_group == 1 ? 1 : a.cta_group == 2 ? 2 : (a.M / a.G >= 192 ? 2 : 1);
    const bool fp8 = a.elem_bytes == 1;
    p.y_scale_out = nullptr;
    p.y_f32_out = nullptr;
    p.c_in = a.c_in;
    p.alpha = a.alpha;
    p.beta = a.beta;
    // The main/tails split of group_row_tiles() (a group's last row block of at most 128 rows in a second,
    // single-CTA launch) is NOT used here: this kernel is bound by the MMAs, a 128x256 single-CTA tile keeps
    // one SM busy about as long as the half-empty pair tile keeps two, and the second launch adds its own
    // partial wave.  Mixtral-shaped layer (8 groups of ~1024 rows, half of them with such a block):
    // gate+up 1.458 ms split vs 1.430 ms pairs only, down 0.744 vs 0.720.  With the second launch started on the
    // SMs the first gives back (overlap_role, as the block-wise kernel does) it still loses: DeepSeek gate+up shape
    // 0.686 vs 0.668 ms, the Mixtral layer 2.29-2.30 vs 2.25-2.27 ms.  (The block-wise FP8 kernel, which is bound
    // by latency instead, gains 5-10 % from the split.)
    const bool split_tails = false;
    auto launch = [&](int nctas, int mode) -> int {
        p.tile_mode = mode;
        p.overlap_role = a.overlap_role;
        p.idesc = make_idesc(fp8, 128 * nctas, kTileN, a.is_f16 != 0, a.w_mn_major != 0);
        p.idesc_half = make_idesc(fp8, 128 * nctas, kTileN / 2, a.is_f16 != 0, a.w_mn_major != 0);
        if (a.w_mn_major)
            return nctas == 1 ? launch_variant<2, 1, 0, 0, true>(tm_x, tm_w, p, di.sms, a.stream)
                              : launch_variant<2, 2, 0, 0, true>(tm_x, tm_w, p, di.sms, a.stream);
#define B200MOE_LAUNCH(EB, SC, EP)                                                          \
    (nctas == 1 ? launch_variant<EB, 1, SC, EP>(tm_x, tm_w, p, di.sms, a.stream)             \
                : launch_variant<EB, 2, SC, EP>(tm_x, tm_w, p, di.sms, a.stream))
        if (!fp8 && a.epilogue == 0) return B200MOE_LAUNCH(2, 0, 0);
        if (!fp8 && a.epilogue == 1) return B200MOE_LAUNCH(2, 0, 1);
        if (!fp8 && a.epilogue == 2) return B200MOE_LAUNCH(2, 0, 2);
        if (fp8 && a.scale_mode == 1) return B200MOE_LAUNCH(1, 1, 0);
        if (fp8 && a.scale_mode == 0 && a.epilogue == 0) return B200MOE_LAUNCH(1, 0, 0);
#undef B200MOE_LAUNCH
        return kErrBadArgument;
    };
    if (!split_tails) return launch(ctas, kTilesAll);
    if (int e = launch(2, kTilesMain)) return e;
    return launch(1, kTilesTails);
}

}  // namespace b200moe
