// FP8 grouped GEMM with block-wise scales (the DeepSeek-V3 recipe):
//     y[m, n] = sum over K blocks kb of
//               (xq[m, kb] . wq[g][n, kb]) * x_scale[m, kb] * w_scale[g][n / 128][kb]
// xq [M, K] e4m3 with one fp32 scale per row and 128 columns (1x128), wq [G, N, K] e4m3
// with one fp32 scale per 128x128 block, y bf16.  The reference has no such kernel (its
// block-wise path lives in FBGEMM, kernels/needs_perf_help/fp8_gemm_bench.py:16-21); the
// 1x128 scale convention is that of kernels/triton/inference/fp8/float8_groupwise_quant.py.
//
// The scales change along K, so they cannot wait for the end of the tile.  One
// shared-memory stage holds exactly one 128-deep K block.  The MMA issuer accumulates
// each block on its own (4 MMAs, the first one overwriting) into one of two 256-column
// TMEM buffers and publishes it; the epilogue warps pull it out with tcgen05.ld and fold
// it into fp32 REGISTER accumulators with the block's combined scale while the tensor
// core already works on the next block in the other buffer.
//
// 384 threads in three warpgroups: warp 0 TMA producer, warp 1 MMA issuer, warps 2 and 3 send
// finished rows to global memory (bulk-copy epilogue; otherwise they only help set up), warps
// 4..11 promote.  Promotion warp w owns TMEM lanes 32*(w%4).. (a hardware rule) and half of the
// tile's columns, i.e. 128 accumulators per thread; setmaxnreg moves registers from the first
// warpgroup to the two promotion warpgroups so those accumulators stay in registers.  Tile
// shapes, scheduler and the CTA-pair mode are those of the bf16 kernel (grouped_gemm.cu).
//
// What bounds it: only two K blocks fit in TMEM, so the tensor pipe (512 cycles per block) waits
// for the round trip MMA done -> promotion warps see the commit (~130-400 cycles later) -> TMEM
// loads and the first half of the FMAs (~330) -> "drained" arrivals reach the issuer (~260) ->
// next MMAs issued (~170): ~950 cycles per block in cycle stamps.  Everything the promotion
// warps do besides that sits on this path, so the first scales of a tile are fetched one tile
// ahead and finished rows are handed to other warps instead of being stored by them.
//
// In auto mode on ragged groups the launcher runs two kernels: CTA pairs on 256-row tiles, then single CTAs on
// the groups' last blocks of at most 128 rows (group_row_tiles).  The second is a programmatic dependent of the
// first (overlap_role): its CTAs start on each SM as the first kernel's CTA there exits.
#include <cuda_fp8.h>

#include "gg_common.cuh"

namespace b200moe {

constexpr int kBlkThreads = 384;
constexpr int kBlkEpiWarps = 8;
// Register split after start-up (setmaxnreg): the control warpgroup keeps 24 registers per thread, the two
// promotion warpgroups take 240.  The registers moved come out of what the CTA got at launch
// (168 per thread for 384 threads), never out of the rest of the SM: a split that adds up to more than
// that leaves the raising warps waiting forever.
#define B200MOE_BLK_CTL_REGS 24
#define B200MOE_BLK_EPI_REGS 240
#define B200MOE_STR2(x) #x
#define B200MOE_STR(x) B200MOE_STR2(x)
static_assert(128 * B200MOE_BLK_CTL_REGS + 256 * B200MOE_BLK_EPI_REGS <= kBlkThreads * 168,
              "setmaxnreg split exceeds the registers the CTA is launched with");
constexpr int kBlkStageBytes = 32 * 64;  // peer-store staging per warp: 32 rows x 64 bytes
// Bulk-copy epilogue: one staging slot per promotion thread for the bf16 results of its row (128 of them =
// 256 bytes for the plain epilogue, 64 = 128 bytes after SwiGLU, 64 e4m3 bytes when they are quantised) +
// 16 bytes that keep the slots of neighbouring lanes off the same banks, and one destination pointer per
// slot.  The promotion warps only park their rows there; the two control warps that have no other job send
// every slot with one asynchronous bulk copy while the promotion warps are already at the next tile.
// (Issued by the promotion warps themselves the copies cost ~2300 cycles per warp and tile — the instruction
// is carried out lane by lane — on the one set of warps the tensor pipe waits for; sending them a few lanes
// per K block, or writing the rows out with ordinary coalesced stores, at once or one store per K block,
// slowed every K block down instead.)
template <int EPI, int CTAS>
struct BulkCfg {
    static constexpr int kRowBytes = EPI == 0 ? 256 : (EPI == 1 ? 128 : 64);
    static constexpr int kSlotBytes = kRowBytes + 16;
    static constexpr int kSlots = kBlkEpiWarps * 32;
    static constexpr int kStagingBytes = kSlots * kSlotBytes + kSlots * 8;   // slots, then the pointer table
    static constexpr int kLess = (CTAS == 2 && EPI == 0) ? 2 : 1;             // ring stages given up for them
};

// Developer aid: with -DB200MOE_TRACE the first two CTAs record clock64() stamps of their roles per K block
// (read back with b200moe_debug_read_trace); without it the macro vanishes.
#ifdef B200MOE_TRACE
__device__ unsigned long long g_trace[2][10][160][4];
#define B200MOE_TR(role, k, slot)                                                       \
    do {                                                                                \
        if (blockIdx.x < 2 && (k) < 160 && (threadIdx.x & 31) == 0)                     \
            g_trace[blockIdx.x][role][k][slot] = static_cast<unsigned long long>(clock64()); \
    } while (0)
#else
#define B200MOE_TR(role, k, slot) do { } while (0)
#endif

// EPI: 0 plain, 1 SwiGLU -> bf16, 3 SwiGLU -> e4m3 with one fp32 scale per row and 128 columns
//      (the 1x128 quantiser of float8_groupwise_quant.py:36-46 applied to the fp32 values in
//      registers, so the intermediate never exists in bf16).
// BULK (EPI 0 and 1 with outputs made of whole 16-byte aligned runs; EPI 3 always): the bulk-copy epilogue
//      described at BulkCfg.  Without it: direct 16-byte stores (local output) or 64-byte runs through a small
//      staging buffer (rows that go to other GPUs); both also handle ragged N.
template <int CTAS, int EPI, bool BULK = false>
__global__ void __launch_bounds__(kBlkThreads, 1)
gg_fp8_block_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                    const GGParams p) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL)
    constexpr int kLess = BULK ? BulkCfg<EPI, CTAS>::kLess : 0;  // ring stages the bulk slots cost
    constexpr int kBulkSlotBytes = BulkCfg<EPI, CTAS>::kSlotBytes;
    constexpr int kBulkStagingBytes = BulkCfg<EPI, CTAS>::kStagingBytes;
    constexpr int kRun = 64;                 // bytes per staged row of the ordinary-store path
    using Cfg = StageCfg<CTAS, kLess>;
    constexpr int kTileRows = kRowsPerCta * CTAS;
    constexpr bool kSwiglu = EPI == 1 || EPI == 3;

    extern __shared__ uint8_t smem_raw[];
    const SmemView sv = carve_smem<CTAS, kLess>(smem_raw);
    const uint32_t ring_addr = sv.ring_addr;
    SmemTail* st = sv.tail;
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
    // Mailbox through which the two warps that share 32 rows exchange their half-row maxima
    // (EPI 3): amax[slot][half][row] and a sequence word per (slot, half, lane quarter).
    float* const mail_amax =
        reinterpret_cast<float*>(sv.warp_stage) + (BULK ? kBulkStagingBytes / 4 : 0);  // after the bulk slots
    volatile int* const mail_seq = reinterpret_cast<volatile int*>(mail_amax + 2 * 2 * 128);
    if constexpr (EPI == 3) {
        if (threadIdx.x < 16) mail_seq[threadIdx.x] = 0;
    }
    __syncthreads();
    if (warp == 0) {
        build_tables_and_barriers<CTAS, kLess>(st, p, lane, kTileRows, kBlkEpiWarps * CTAS);
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
    if constexpr (CTAS == 2) cluster_sync_all();
    tc_fence_after();

    const uint32_t tmem_base = st->tmem_base;
    const int total_tiles = st->total_tiles;
    const int num_kb = p.K / 128;  // the launcher guarantees K % 128 == 0
    // main launch of a main + tails pair: the tails kernel writes other rows and needs nothing from this one, so
    // its CTAs may take each SM as soon as this kernel's CTA there is done
    if (p.overlap_role == 1 && threadIdx.x == 0) griddep_launch_dependents();

    // Register budget: one light warpgroup + two promotion warpgroups (see B200MOE_BLK_*_REGS).
    if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 " B200MOE_STR(B200MOE_BLK_CTL_REGS) ";");
      if (warp == 0) {
        producer_loop<CTAS, kLess, kSwiglu>(&tm_x, &tm_w, st, ring_addr, p, cta_rank, cluster_id, num_clusters, 128,
                                          num_kb);
      } else if (warp == 1) {
        // ================= MMA issuer: one K block per stage, one TMEM buffer per K block
        // (the whole warp walks the loop so that descriptors are warp-uniform; one elected lane issues)
        if (cta_rank == 0) {
            const bool leader = elect_one();
            int stage = 0, buf = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            [[maybe_unused]] int kc = 0;
            for (int t = cluster_id; ok && t < total_tiles; t += num_clusters) {
                for (int kb = 0; kb < num_kb; ++kb, ++kc) {
                    // operands first: they are almost always there long before the accumulator is free, and
                    // the accumulator's release is what the whole pipeline waits for
                    if (!__all_sync(0xffffffffu, mbar_wait(&st->full[stage], phase, abort_flag))) {
                        report(p.status, kStatusTimeoutMmaFull);
                        ok = false;
                        break;
                    }
                    B200MOE_TR(8, kc, 1);
                    if (!__all_sync(0xffffffffu, mbar_wait(&st->acc_empty[buf], acc_phase ^ 1u, abort_flag))) {
                        report(p.status, kStatusTimeoutMmaAcc);
                        ok = false;
                        break;
                    }
                    B200MOE_TR(8, kc, 0);
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * kTileN);
                    const uint32_t a_addr = ring_addr + stage * Cfg::kStageBytes;
                    const uint64_t a_desc = make_sw128_kmajor_desc(a_addr);
                    const uint64_t b_desc = make_sw128_kmajor_desc(a_addr + kABytes);
                    if (leader) {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma<CTAS, true>(d_tmem, a_desc + 2u * k, b_desc + 2u * k, p.idesc, k > 0 ? 1u : 0u);
                        // One commit serves two waiters: the producer (stage free) and the promotion
                        // warps (this K block's product is in TMEM) both watch empty[stage].
                        umma_commit<CTAS>(&st->empty[stage]);
                    }
                    __syncwarp();
                    B200MOE_TR(8, kc, 2);
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                    buf ^= 1;
                    if (buf == 0) acc_phase ^= 1u;
                }
            }
        }
      } else if constexpr (BULK) {
        // ================= sending warps (2 and 3): per tile, one bulk copy per parked slot, 128 slots each
        const int sw = warp - 2;
        char* const* const slot_ptrs = reinterpret_cast<char* const*>(
            reinterpret_cast<const char*>(sv.warp_stage) + BulkCfg<EPI, CTAS>::kSlots * kBulkSlotBytes);
        const uint32_t slots_addr = smem_u32(sv.warp_stage);
        uint32_t out_phase = 0;
        for (int t = cluster_id; t < total_tiles; t += num_clusters) {
            if (!__all_sync(0xffffffffu, mbar_wait(&st->out_full, out_phase, abort_flag))) {
                report(p.status, kStatusTimeoutEpilogue);
                break;
            }
#pragma unroll 1
            for (int round = 0; round < 4; ++round) {
                const int slot = sw * 128 + round * 32 + lane;
                char* const dst = slot_ptrs[slot];
                if (dst != nullptr)
                    bulk_store(dst, slots_addr + static_cast<uint32_t>(slot * kBulkSlotBytes),
                               BulkCfg<EPI, CTAS>::kRowBytes);
            }
            bulk_commit();
            bulk_wait_read();  // every copy of this thread has read its slot
            __syncwarp();
            if (lane == 0) mbar_arrive(&st->out_empty);
            out_phase ^= 1u;
        }
        bulk_wait_all();
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 " B200MOE_STR(B200MOE_BLK_EPI_REGS) ";");
        // ================= epilogue / promotion (8 warps)
        const int ew = warp - 4;          // 0..7
        const int quarter = warp & 3;     // TMEM lane quarter this warp may read
        const int half = ew >> 2;         // which half of the tile's columns
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t acc_empty_leader =
            CTAS == 1 ? smem_u32(&st->acc_empty[0]) : mapa_shared(smem_u32(&st->acc_empty[0]), 0);
        const int kblocks = num_kb;                    // scales per row of x
        const int nblocks = (p.N + 127) / 128;         // scale blocks per expert along N
        int g = 0, buf = 0, tiles_done = 0, stage = 0;
        uint32_t stage_phase = 0;
        bool ok = true;
        [[maybe_unused]] int kc = 0;
        // The thread's 128 columns are four runs of 32: two scale blocks at most.
        //   plain : columns half*128 + [0,128)            -> scale block 2*n_idx + half
        //   SwiGLU: gate columns half*64 + [0,64) (block n_idx) and the matching up
        //           columns 128 + half*64 + [0,64) (block I/128 + n_idx)
        const int col_a = kSwiglu ? half * 64 : half * 128;
        const int col_b = kSwiglu ? 128 + half * 64 : half * 128 + 64;
        // Bulk-copy epilogue, promotion side: park the row in this thread's slot, leave its destination in the
        // pointer table, and tell the sending warps; before the next tile's rows are parked, wait until the
        // copies of this one have read the slots (normally long past).
        uint4* const my_slot = sv.warp_stage + (ew * 32 + lane) * (kBulkSlotBytes / 16);
        char** const my_slot_ptr = reinterpret_cast<char**>(reinterpret_cast<char*>(sv.warp_stage) +
                                                            BulkCfg<EPI, CTAS>::kSlots * kBulkSlotBytes) + ew * 32 + lane;
        uint32_t tiles_parked = 0;
        auto slots_free = [&]() -> bool {   // all lanes
            if (tiles_parked == 0) return true;
            return __all_sync(0xffffffffu, mbar_wait(&st->out_empty, (tiles_parked - 1) & 1u, abort_flag));
        };
        auto hand_over = [&](char* dst) {   // all lanes, after the slot has been written
            *my_slot_ptr = dst;
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&st->out_full);
            ++tiles_parked;
        };
        // Per-tile state kept small (registers are what this kernel runs out of): the thread's row (-1:
        // past the group's end), group, column tile and the element offset of its (first) row of w
        // scales.  With SwiGLU the up columns' scale row lies a fixed distance after the gate columns'
        // (N is a multiple of 256 there, so no block index needs clamping).  The first block's scales
        // of a tile are fetched one tile ahead (before the previous tile's stores), so no tile
        // begins by waiting for global memory.
        struct TileState {
            int row, g, n_idx, wa_off;
        };
        const int wb_delta = kSwiglu ? (p.n_out / 128) * kblocks : 0;
        auto enter_tile = [&](int t) {
            const TileCoord c = locate_tile(t, g, st->tile_off, st->row_off, kTileRows, p.tile_mode);
            const int r = c.row0 + static_cast<int>(cta_rank) * kRowsPerCta + quarter * 32 + lane;
            const int blk_a = kSwiglu ? c.n_idx : 2 * c.n_idx + half;
            TileState s;
            s.row = r < c.row_end ? r : -1;
            s.g = c.g;
            s.n_idx = c.n_idx;
            s.wa_off = (c.g * nblocks + min(blk_a, nblocks - 1)) * kblocks;  // (the launcher bounds these below 2^31)
            return s;
        };
        float xs_next = 0.0f, wa_next = 0.0f, wb_next = 0.0f;
        TileState nxt{};
        auto fetch_scales = [&](const TileState& s, int kb) {
            xs_next = s.row >= 0 ? __ldg(p.x_scale + s.row * kblocks + kb) : 0.0f;
            wa_next = __ldg(p.w_scale + s.wa_off + kb);
            wb_next = kSwiglu ? __ldg(p.w_scale + s.wa_off + wb_delta + kb) : wa_next;
        };
        if (cluster_id < total_tiles) {
            nxt = enter_tile(cluster_id);
            fetch_scales(nxt, 0);
        }
        for (int t = cluster_id; ok && t < total_tiles; t += num_clusters) {
            const TileState cur = nxt;   // set one iteration ago
            const int cur_row = cur.row >= 0 ? cur.row : 0;
            const bool cur_row_ok = cur.row >= 0;

            float acc[128];
#pragma unroll
            for (int j = 0; j < 128; ++j) acc[j] = 0.0f;

            for (int kb = 0; kb < num_kb; ++kb, ++kc) {
                const float sa = xs_next * wa_next;
                const float sb = xs_next * wb_next;
                if (kb + 1 < num_kb) {  // fetch the next block's scales while waiting
                    fetch_scales(cur, kb + 1);
                } else if (t + num_clusters < total_tiles) {  // ... or the first block's scales of the next tile
                    nxt = enter_tile(t + num_clusters);
                    fetch_scales(nxt, 0);
                }
                // every lane polls: the flip is seen without a shuffle hop
                const int got = __all_sync(0xffffffffu, mbar_wait(&st->empty[stage], stage_phase, abort_flag) ? 1 : 0);
                if (!got) {
                    if (lane == 0) report(p.status, kStatusTimeoutEpilogue);
                    ok = false;
                    break;
                }
                B200MOE_TR(ew, kc, 0);
                tc_fence_after();
                const uint32_t t_acc = tmem_base + lane_base + static_cast<uint32_t>(buf * kTileN);
                // Four runs of 32 columns through two staging buffers; the TMEM buffer goes back
                // to the MMA issuer as soon as the last load has landed, before the last FMAs.
                uint32_t v0[32], v1[32];
                tmem_ld_32x32(t_acc + static_cast<uint32_t>(col_a), v0);
                tmem_ld_32x32(t_acc + static_cast<uint32_t>(col_a + 32), v1);
                tmem_ld_wait(v0);
                tmem_ld_wait(v1);
                B200MOE_TR(ew, kc, 1);
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[j] = fmaf(__uint_as_float(v0[j]), sa, acc[j]);
                tmem_ld_32x32(t_acc + static_cast<uint32_t>(col_b), v0);
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[32 + j] = fmaf(__uint_as_float(v1[j]), sa, acc[32 + j]);
                tmem_ld_32x32(t_acc + static_cast<uint32_t>(col_b + 32), v1);
                tmem_ld_wait(v0);
                tmem_ld_wait(v1);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(acc_empty_leader + static_cast<uint32_t>(buf) * 8u);
                B200MOE_TR(ew, kc, 2);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    acc[64 + j] = fmaf(__uint_as_float(v0[j]), sb, acc[64 + j]);
                    acc[96 + j] = fmaf(__uint_as_float(v1[j]), sb, acc[96 + j]);
                }
                B200MOE_TR(ew, kc, 3);
                buf ^= 1;
                if (++stage == Cfg::kStages) {
                    stage = 0;
                    stage_phase ^= 1u;
                }
            }
            if (!ok) break;

            if constexpr (EPI == 3) {
                // ---- SwiGLU, then 1x128 quantisation of the 128 output columns this tile owns for
                // the row; this thread holds 64 of them, the warp with the other half holds the rest.
                ++tiles_done;
                float f[64];
                float amax = 0.0f;
#pragma unroll
                for (int j = 0; j < 64; ++j) {
                    f[j] = silu_mul(acc[j], acc[64 + j]);
                    amax = fmaxf(amax, fabsf(f[j]));
                }
                const int slot = tiles_done & 1;
                const int rix = quarter * 32 + lane;
                mail_amax[(slot * 2 + half) * 128 + rix] = amax;
                __threadfence_block();
                __syncwarp();
                if (lane == 0) mail_seq[(slot * 2 + half) * 4 + quarter] = tiles_done;
                // bounded wait for the partner warp's half
                int seen = 0;
                if (lane == 0) {
                    const uint64_t t0 = globaltimer_ns();
                    uint32_t spins = 0;
                    seen = 1;
                    while (mail_seq[(slot * 2 + (half ^ 1)) * 4 + quarter] != tiles_done) {
                        if (((++spins) & 0x3F) == 0 && (*abort_flag || globaltimer_ns() - t0 > kWaitLimitNs)) {
                            *abort_flag = 1;
                            seen = 0;
                            break;
                        }
                    }
                }
                seen = __shfl_sync(0xffffffffu, seen, 0);
                if (!seen) {
                    if (lane == 0) report(p.status, kStatusTimeoutEpilogue);
                    ok = false;
                    break;
                }
                __threadfence_block();
                amax = fmaxf(amax, mail_amax[(slot * 2 + (half ^ 1)) * 128 + rix]);
                // the quantiser's own formula (float8_groupwise_quant.py:39-46), IEEE division included, so
                // that the bytes equal those of quant_1x128_kernel run on these fp32 values
                const float scale = __fdiv_rn(fmaxf(amax, 1e-12f), 448.0f);
                const int col = cur.n_idx * 128 + half * 64;
                if (p.y_f32_out != nullptr && cur_row_ok && col < p.n_out) {  // optional copy of the values quantised
                    float4* f_row = reinterpret_cast<float4*>(p.y_f32_out + static_cast<size_t>(cur_row) * p.n_out + col);
#pragma unroll
                    for (int j = 0; j < 16; ++j) f_row[j] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
                }
                const bool q_ok = cur_row_ok && col < p.n_out;
                if constexpr (BULK) {
                    if (!slots_free()) {
                        if (lane == 0) report(p.status, kStatusTimeoutEpilogue);
                        ok = false;
                        break;
                    }
                }
                uint8_t* const q_row = static_cast<uint8_t*>(p.y) + static_cast<size_t>(cur_row) * p.ldy + col;
                // f / scale for 64 values that share the divisor: with y = RN(1 / scale), q0 = RN(f * y),
                // r = f - q0 * scale (exact in an FMA) and q1 = RN(q0 + r * y), q1 is the correctly rounded
                // quotient (Markstein's correction step) — three instructions per value instead of a full
                // division.  A divisor whose significand is all ones, where the reciprocal step is not
                // covered, takes the ordinary division.
                const float inv_scale = __frcp_rn(scale);
                if ((__float_as_uint(scale) & 0x007fffffu) != 0x007fffffu) {
#pragma unroll
                    for (int j = 0; j < 64; ++j) {
                        const float q0 = f[j] * inv_scale;
                        f[j] = fmaf(fmaf(-q0, scale, f[j]), inv_scale, q0);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 64; ++j) f[j] = __fdiv_rn(f[j], scale);
                }
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float v[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) v[j] = fminf(fmaxf(f[c4 * 16 + i * 4 + j], -448.0f), 448.0f);
                        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0], v[1]), __NV_SATFINITE, __NV_E4M3);
                        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2], v[3]), __NV_SATFINITE, __NV_E4M3);
                        w[i] = lo | (hi << 16);
                    }
                    if constexpr (BULK)
                        my_slot[c4] = make_uint4(w[0], w[1], w[2], w[3]);
                    else if (q_ok)
                        *reinterpret_cast<uint4*>(q_row + c4 * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                // (the launcher checked that rows of y start 16-byte aligned and hold whole 128-column runs)
                if constexpr (BULK) hand_over(q_ok ? reinterpret_cast<char*>(q_row) : nullptr);
                if (q_ok && half == 0)
                    p.y_scale_out[static_cast<size_t>(cur_row) * (p.n_out / 128) + cur.n_idx] = scale;
                continue;
            }
            // ---- store: the thread's row, its (up to) 128 output columns, 64 at a time through
            // the warp's staging buffer so that whole 128-byte runs of a row go out together
            RowDest rd;
            const bool store_ok = resolve_row_dest(p, cur_row, cur_row_ok, &rd);
            char* const my_row = store_ok ? reinterpret_cast<char*>(rd.base) +
                                                (static_cast<size_t>(rd.drow) * p.ldy +
                                                 static_cast<size_t>(cur.g) * p.y_col_group_stride) * 2
                                          : nullptr;
            uint4* const stage = sv.warp_stage + ew * (32 * kRun / 16);  // (the ordinary-store path's buffer)
            if constexpr (BULK) {
                // (built for whole runs only: n_out % 128 == 0, aligned pitch; the launcher sees to it)
                constexpr int kMine = EPI == 1 ? 64 : 128;  // results this thread holds for its row
                const int col0 = EPI == 1 ? cur.n_idx * 128 + half * 64 : cur.n_idx * kTileN + half * 128;
                if (!slots_free()) {
                    if (lane == 0) report(p.status, kStatusTimeoutEpilogue);
                    ok = false;
                    break;
                }
#pragma unroll
                for (int q = 0; q < kMine / 8; ++q) {
                    float f[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if constexpr (EPI == 1)
                            f[j] = silu_mul(acc[q * 8 + j], acc[64 + q * 8 + j]);
                        else
                            f[j] = acc[q * 8 + j];
                    }
                    my_slot[q] = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                            pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
                }
                char* dst = (store_ok && col0 < p.n_out) ? my_row + static_cast<size_t>(col0) * 2 : nullptr;
                if (dst != nullptr && (reinterpret_cast<uintptr_t>(dst) & 15u) != 0) {
                    // a destination buffer that is not 16-byte aligned cannot take a bulk copy: element stores, now
                    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(my_slot);
                    for (int j = 0; j < kMine; ++j) reinterpret_cast<__nv_bfloat16*>(dst)[j] = src[j];
                    dst = nullptr;
                }
                hand_over(dst);
                continue;
            }
            constexpr int kSlabs = EPI == 1 ? 1 : 2;
            const int col_first = EPI == 1 ? cur.n_idx * 128 + half * 64 : cur.n_idx * kTileN + half * 128;
            const bool to_peers = p.row_tags != nullptr;  // kernel-uniform
#pragma unroll
            for (int sl = 0; sl < kSlabs; ++sl) {
                const int scol = col_first + sl * 64;
                if (scol >= p.n_out) continue;  // warp-uniform
                if (!to_peers) {
                    if (store_ok) {
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            float f[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if constexpr (EPI == 1)
                                    f[j] = silu_mul(acc[c * 32 + j], acc[64 + c * 32 + j]);
                                else
                                    f[j] = acc[sl * 64 + c * 32 + j];
                            }
                            store_row_chunk(reinterpret_cast<__nv_bfloat16*>(my_row), scol + c * 32, p.n_out, f);
                        }
                    }
                } else {
#pragma unroll
                    for (int hrun = 0; hrun < 2; ++hrun) {  // two 64-byte runs (32 columns each)
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            float f[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const int jj = hrun * 32 + q * 8 + j;
                                if constexpr (EPI == 1)
                                    f[j] = silu_mul(acc[jj], acc[64 + jj]);
                                else
                                    f[j] = acc[sl * 64 + jj];
                            }
                            stage_put<64>(stage, lane, q,
                                          make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                                     pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7])));
                        }
                        __syncwarp();
                        const int rcol = scol + hrun * 32;
                        if (rcol < p.n_out)
                            stage_flush<2, 64>(stage, lane,
                                               my_row != nullptr ? my_row + static_cast<size_t>(rcol) * 2 : nullptr,
                                               min(64, (p.n_out - rcol) * 2));
                        __syncwarp();
                    }
                }
            }
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
    // tails launch: what follows in the stream waits for this kernel only, so it must not end before the main one
    if (p.overlap_role == 2 && threadIdx.x == 0) griddep_wait();
#else
    if (threadIdx.x == 0 && blockIdx.x == 0) report(p.status, kStatusWrongArch);
#endif
}

template <int CTAS, int EPI, bool BULK = false>
static int launch_block_variant(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const GGParams& p, int sms,
                                cudaStream_t stream) {
    const bool overlapped = p.overlap_role == 2;  // may start before the kernel in front of it has finished
    auto kernel = gg_fp8_block_kernel<CTAS, EPI, BULK>;
    constexpr size_t smem = gg_smem_bytes<CTAS, BULK ? BulkCfg<EPI, CTAS>::kLess : 0,
                                           BULK ? BulkCfg<EPI, CTAS>::kStagingBytes + (EPI == 3 ? 2304 : 0)
                                                : kBlkEpiWarps * kBlkStageBytes>();
    static_assert(smem <= 232448, "shared memory per CTA");
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
    cfg.blockDim = dim3(kBlkThreads, 1, 1);
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
    cfg.numAttrs = overlapped ? 2 : 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tm_x, tm_w, p);
    if (e == cudaSuccess) note_launch();
    return static_cast<int>(e);
}

#ifdef B200MOE_TRACE
extern "C" int b200moe_debug_read_trace(void* dst, unsigned long long bytes) {
    return static_cast<int>(cudaMemcpyFromSymbol(dst, g_trace, bytes < sizeof(g_trace) ? bytes : sizeof(g_trace)));
}
#endif

int grouped_gemm_fp8_block_launch(const GGLaunch& a) {
    // y may be null when every row leaves through (rank, row) tags: the peer table names the buffers
    if (a.M < 0 || a.N <= 0 || a.K <= 0 || a.G <= 0 || a.x == nullptr || a.w == nullptr ||
        (a.y == nullptr && a.row_tags == nullptr) || a.m_sizes == nullptr || a.x_scale == nullptr ||
        a.w_scale == nullptr)
        return kErrBadArgument;
    if (a.G > kMaxGroups) return kErrTooManyGroups;
    if (a.K % 128 != 0) return kErrAlignment;  // whole scale blocks along K
    // scale offsets are 32-bit in the kernel
    if (static_cast<long long>(a.M) * (a.K / 128) > 0x7fffffffll ||
        static_cast<long long>(a.G) * ((a.N + 127) / 128) * (a.K / 128) > 0x7fffffffll)
        return kErrTooLarge;
    if ((reinterpret_cast<uintptr_t>(a.x) & 15u) || (reinterpret_cast<uintptr_t>(a.w) & 15u)) return kErrAlignment;
    if (a.epilogue != 0 && a.epilogue != 1 && a.epilogue != 3) return kErrBadArgument;
    if (a.epilogue == 3 && a.y_f32_out != nullptr && (reinterpret_cast<uintptr_t>(a.y_f32_out) & 15u) != 0)
        return kErrAlignment;
    if (a.epilogue == 3 && (a.y_scale_out == nullptr || a.row_map != nullptr || a.row_tags != nullptr ||
                            a.y_col_group_stride != 0 || (a.ldy & 15) != 0 ||
                            (reinterpret_cast<uintptr_t>(a.y) & 15u) != 0))
        return kErrBadArgument;
    if (a.row_tags != nullptr && (a.peer_y == nullptr || a.n_peers <= 0 || a.y_rows <= 0)) return kErrBadArgument;
    if (a.epilogue != 0 && (a.N % 256 != 0)) return kErrBadArgument;  // gate and up halves in whole scale blocks
    if (a.M == 0) return 0;

    DeviceInfo di;
    if (int e = get_device_info(&di)) return e;
    if (di.cc_major != 10) return kErrWrongDevice;
    CUtensorMap tm_x, tm_w;
    if (int e = encode_x_map(&tm_x, a.x, a.M, a.K, 1)) return e;
    if (int e = encode_w_map(&tm_w, a.w, a.G, a.N, a.K, 1)) return e;

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
    p.n_out = a.epilogue != 0 ? a.N / 2 : a.N;
    p.n_tiles = a.epilogue != 0 ? (p.n_out + 127) / 128 : (p.n_out + kTileN - 1) / kTileN;
    p.y_scale_out = a.y_scale_out;
    p.y_f32_out = a.epilogue == 3 ? a.y_f32_out : nullptr;

    // Auto tiling: this kernel is bound by the promotion round trip, not by the MMA, so CTA pairs buy nothing
    // until the padding of 128-row tiles stops mattering.  32 ragged groups, N=4096, K=7168, single vs pair:
    // 96 rows per group 1003 vs 723 TFLOP/s, 256: 1383 vs 1317, 512: 1688 vs 1571, 768: 1851 vs 1840,
    // 1024: 1932 vs 1935, 2048: 1855 vs 1890.
    const int ctas = a.cta_group == 1 ? 1 : a.cta_group == 2 ? 2 : (a.M / a.G >= 640 ? 2 : 1);
    p.c_in = nullptr;
    p.alpha = 1.0f;
    p.beta = 0.0f;
    // outputs made of whole, 16-byte aligned runs leave through bulk copies
    const bool bulk = p.n_out % 128 == 0 && a.ldy % 8 == 0 && a.y_col_group_stride % 8 == 0 &&
                      (a.row_tags != nullptr || (reinterpret_cast<uintptr_t>(a.y) & 15u) == 0);
    // CTA pairs on ragged groups in auto mode: two launches, see group_row_tiles() (a group's last row block
    // of at most 128 rows goes to a single-CTA launch instead of filling half of a pair tile)
    const bool split_tails = a.cta_group == 0 && ctas == 2;
    auto launch = [&](int nctas, int mode) -> int {
        p.tile_mode = mode;
        p.overlap_role = mode == kTilesMain ? 1 : (mode == kTilesTails ? 2 : 0);
        p.idesc = make_idesc(true, 128 * nctas, kTileN);
        p.idesc_half = p.idesc;
        if (a.epilogue == 3)  // (its argument checks above already demand aligned, whole 128-column runs)
            return nctas == 1 ? launch_block_variant<1, 3, true>(tm_x, tm_w, p, di.sms, a.stream)
                              : launch_block_variant<2, 3, true>(tm_x, tm_w, p, di.sms, a.stream);
        if (a.epilogue == 0) {
            if (bulk)
                return nctas == 1 ? launch_block_variant<1, 0, true>(tm_x, tm_w, p, di.sms, a.stream)
                                  : launch_block_variant<2, 0, true>(tm_x, tm_w, p, di.sms, a.stream);
            return nctas == 1 ? launch_block_variant<1, 0>(tm_x, tm_w, p, di.sms, a.stream)
                              : launch_block_variant<2, 0>(tm_x, tm_w, p, di.sms, a.stream);
        }
        if (bulk)
            return nctas == 1 ? launch_block_variant<1, 1, true>(tm_x, tm_w, p, di.sms, a.stream)
                              : launch_block_variant<2, 1, true>(tm_x, tm_w, p, di.sms, a.stream);
        return nctas == 1 ? launch_block_variant<1, 1>(tm_x, tm_w, p, di.sms, a.stream)
                          : launch_block_variant<2, 1>(tm_x, tm_w, p, di.sms, a.stream);
    };
    if (!split_tails) return launch(ctas, kTilesAll);
    if (int e = launch(2, kTilesMain)) return e;
    return launch(1, kTilesTails);
}

}  // namespace b200moe
