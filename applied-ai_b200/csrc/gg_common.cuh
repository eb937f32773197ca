// Pieces shared by the grouped-GEMM kernels: tile geometry, the shared-memory tail
// (barriers + group tables), the ragged tile walk, the TMA producer loop and the
// host-side tensor-map encoders.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "b200moe_internal.h"
#include "ptx.cuh"

namespace b200moe {

constexpr int kMaxGroups = 1024;
constexpr int kRowsPerCta = 128;                    // accumulator rows (TMEM lanes) per CTA
constexpr int kTileN = 256;                         // accumulator columns per tile
constexpr int kRowBytes = 128;                      // one swizzle row: 64 bf16 or 128 e4m3 along K
constexpr int kABytes = kRowsPerCta * kRowBytes;    // 16 KiB
constexpr int kSubBoxBytes = 128 * kRowBytes;       // a 128-row box of w: 16 KiB
constexpr int kTmemCols = 2 * kTileN;               // two accumulators

// LESS = stages given up (each kernel trades ring depth against epilogue staging space).
template <int CTAS, int LESS = 0>
struct StageCfg {
    static constexpr int kBBytes = (2 / CTAS) * kSubBoxBytes;  // this CTA's share of the w box
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = (CTAS == 1 ? 4 : 6) - LESS;
    static constexpr int kRingBytes = kStages * kStageBytes;   // 192 KiB at full depth
};

constexpr int kWarpStageBytes = 32 * 128;  // epilogue staging per warp: 32 rows x 128 bytes

struct SmemTail {
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t out_full;   // block-wise FP8 kernel: the promotion warps have parked a tile's rows for the sending warps
    uint64_t out_empty;  //   ... the sending warps' copies have read them
    uint32_t tmem_base;
    int abort_flag;
    int invalid;
    int total_tiles;
    int row_off[kMaxGroups + 1];
    int tile_off[kMaxGroups + 1];
};

template <int CTAS, int LESS, int STAGING_BYTES>
constexpr size_t gg_smem_bytes() {
    return 1024 + StageCfg<CTAS, LESS>::kRingBytes + sizeof(SmemTail) + 16 + STAGING_BYTES;
}

// Carves the dynamic shared memory: a 1024-byte aligned stage ring followed by the tail.
struct SmemView {
    uint32_t ring_addr;
    SmemTail* tail;
    uint4* warp_stage;  // EPI_WARPS x kWarpStageBytes, 16-byte aligned
};
template <int CTAS, int LESS>
__device__ __forceinline__ SmemView carve_smem(uint8_t* smem_raw) {
    const uint32_t raw_addr = smem_u32(smem_raw);
    SmemView v;
    v.ring_addr = (raw_addr + 1023u) & ~1023u;
    uint8_t* tail = smem_raw + (v.ring_addr - raw_addr) + StageCfg<CTAS, LESS>::kRingBytes;
    v.tail = reinterpret_cast<SmemTail*>(tail);
    v.warp_stage = reinterpret_cast<uint4*>(tail + ((sizeof(SmemTail) + 15) & ~size_t(15)));
    return v;
}

// ---- epilogue staging, used when rows go to ANOTHER GPU: a warp parks 32 rows x 128 bytes
// (lane = row) in shared memory and writes them out again row by row, so that one store
// instruction covers whole 128-byte runs of 4 rows instead of 16 bytes of 32 different rows
// (NVLink carries 16-byte writes poorly).  For local memory the direct stores below are
// faster: the extra shared-memory traffic competes with the MMA's operand reads.  16-byte chunks are XOR-swizzled by
// row so neither direction has bank conflicts.
// RUN = bytes per staged row (128 or 64); a warp's buffer is 32 * RUN bytes.
template <int RUN = 128>
__device__ __forceinline__ void stage_put(uint4* stage, int lane, int chunk, uint4 v) {
    constexpr int kChunks = RUN / 16;
    stage[lane * kChunks + (chunk ^ (lane & (kChunks - 1)))] = v;
}
__device__ __forceinline__ char* shfl_ptr(char* p, int src_lane) {
    const unsigned long long v = reinterpret_cast<unsigned long long>(p);
    const unsigned lo = __shfl_sync(0xffffffffu, static_cast<unsigned>(v), src_lane);
    const unsigned hi = __shfl_sync(0xffffffffu, static_cast<unsigned>(v >> 32), src_lane);
    return reinterpret_cast<char*>((static_cast<unsigned long long>(hi) << 32) | lo);
}
// my_dst: where this lane's row (row = lane) starts its 128-byte run, or nullptr to skip the
// row.  valid_bytes (warp-uniform): how much of the run lies inside the output's columns.
// ELEM: bytes per element, for the ragged last chunk and for unaligned destinations.
template <int ELEM, int RUN = 128>
__device__ __forceinline__ void stage_flush(const uint4* stage, int lane, char* my_dst, int valid_bytes) {
    constexpr int kChunks = RUN / 16;            // 16-byte chunks per row
    constexpr int kRowsPerStep = 32 / kChunks;   // rows covered by one store instruction
#pragma unroll
    for (int i = 0; i < 32 / kRowsPerStep; ++i) {
        const int r = i * kRowsPerStep + lane / kChunks;
        const int c = lane % kChunks;
        char* dst = shfl_ptr(my_dst, r);
        if (dst == nullptr || c * 16 >= valid_bytes) continue;
        const uint4 v = stage[r * kChunks + (c ^ (r & (kChunks - 1)))];
        dst += c * 16;
        if (c * 16 + 16 <= valid_bytes && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
            *reinterpret_cast<uint4*>(dst) = v;
        } else {
            const int n = min(16, valid_bytes - c * 16) / ELEM;
            if constexpr (ELEM == 2) {
                const unsigned short* e = reinterpret_cast<const unsigned short*>(&v);
                for (int j = 0; j < n; ++j) reinterpret_cast<unsigned short*>(dst)[j] = e[j];
            } else {
                const unsigned* e = reinterpret_cast<const unsigned*>(&v);
                for (int j = 0; j < n; ++j) reinterpret_cast<unsigned*>(dst)[j] = e[j];
            }
        }
    }
}

__device__ __forceinline__ void report(int32_t* status, int code) {
    if (status != nullptr) atomicCAS(status, 0, code);
}

struct TileCoord {
    int g, row0, row_end, n_idx;
};

// Which row blocks of a group one launch covers.  A ragged group whose last 256-row pair tile would hold
// at most 128 rows wastes half of that tile's MMAs, so the launcher may run two kernels: the "main" one
// (CTA pairs, 256-row tiles) leaves such a last block out, and the "tails" one (single CTAs, 128-row tiles)
// computes just those blocks.  Rows are padded to 128 that way instead of 256.
constexpr int kTilesAll = 0;    // every row block of the group, ceil(m / tile_rows) tiles
constexpr int kTilesMain = 1;   // tile_rows = 256: a last block of 1..128 rows is left to the tails kernel
constexpr int kTilesTails = 2;  // tile_rows = 128: only that left-out block (one tile, or none)
__host__ __device__ __forceinline__ int group_row_tiles(int m, int tile_rows, int mode) {
    if (mode == kTilesMain) return (m + 127) / 256;
    if (mode == kTilesTails) return ((m & 255) >= 1 && (m & 255) <= 128) ? 1 : 0;
    return (m + tile_rows - 1) / tile_rows;
}
__host__ __device__ __forceinline__ int group_first_row(int m, int mode) { return mode == kTilesTails ? (m & ~255) : 0; }

// Maps a global tile number to its group and position.  `g` only moves forward.
__device__ __forceinline__ TileCoord locate_tile(int t, int& g, const int* tile_off, const int* row_off,
                                                 int tile_rows, int mode = kTilesAll) {
    while (tile_off[g + 1] <= t) ++g;
    const int local = t - tile_off[g];
    const int m_g = row_off[g + 1] - row_off[g];
    const int tiles_m = group_row_tiles(m_g, tile_rows, mode);
    TileCoord c;
    c.g = g;
    c.row0 = row_off[g] + group_first_row(m_g, mode) + (local % tiles_m) * tile_rows;
    c.row_end = row_off[g + 1];
    c.n_idx = local / tiles_m;
    return c;
}

// The last, partial round of tiles.  With C clusters and T tiles, r = T mod C tiles remain
// after the full rounds; when they would occupy at most half of the clusters, each is cut
// into two 128-column halves so the round takes half as long.  Work item w < split_from is
// tile w; the items after that are (tile, half) pairs.
struct WorkSplit {
    int split_from, total_work;
};
__device__ __forceinline__ WorkSplit make_work_split(int total_tiles, int num_clusters, bool allow) {
    const int r = total_tiles % num_clusters;
    WorkSplit ws;
    if (allow && r > 0 && 2 * r <= num_clusters) {
        ws.split_from = total_tiles - r;
        ws.total_work = total_tiles + r;
    } else {
        ws.split_from = total_tiles;
        ws.total_work = total_tiles;
    }
    return ws;
}
__device__ __forceinline__ void decode_work(int w, const WorkSplit& ws, int* tile, int* half) {
    if (w < ws.split_from) {
        *tile = w;
        *half = -1;
    } else {
        const int h = w - ws.split_from;
        *tile = ws.split_from + (h >> 1);
        *half = h & 1;
    }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float silu_mul(float gate, float up) { return gate / (1.0f + __expf(-gate)) * up; }

// Where result row `row` is stored: y itself, y through the caller's row map, or another
// rank's y through a (rank, row) tag.  Returns false when the row must not be stored.
struct RowDest {
    __nv_bfloat16* base;  // start of the destination row's buffer (before the column offset)
    long long drow;
};
__device__ __forceinline__ bool resolve_row_dest(const GGParams& p, int row, bool row_ok, RowDest* out) {
    out->base = static_cast<__nv_bfloat16*>(p.y);
    out->drow = row;
    if (!row_ok) return false;
    if (p.row_tags != nullptr) {
        const long long tag = p.row_tags[row];
        const int rank = static_cast<int>(tag >> 32);
        const long long pos = tag & 0xffffffffll;
        if (rank < 0 || rank >= p.n_peers || pos >= p.y_rows) return false;
        out->base = static_cast<__nv_bfloat16*>(p.peer_y[rank]);
        out->drow = pos;
        return true;
    }
    if (p.row_map != nullptr) {
        const int d = __ldg(p.row_map + row);
        if (d < 0 || d >= p.y_rows) return false;
        out->drow = d;
    }
    return true;
}

// Direct store of 32 consecutive fp32 values of one output row as bf16 at columns
// [col, col+32), clipped to n_out columns; 16-byte stores when the run is whole and aligned.
// Used for local memory, where L2 merges the partial lines of neighbouring rows.
__device__ __forceinline__ void store_row_chunk(__nv_bfloat16* y_row, int col, int n_out, const float* f) {
    if (col >= n_out) return;
    __nv_bfloat16* dst = y_row + col;
    if ((col + 32 <= n_out) && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
        uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16x2(f[q * 8 + 0], f[q * 8 + 1]);
            o.y = pack_bf16x2(f[q * 8 + 2], f[q * 8 + 3]);
            o.z = pack_bf16x2(f[q * 8 + 4], f[q * 8 + 5]);
            o.w = pack_bf16x2(f[q * 8 + 6], f[q * 8 + 7]);
            d4[q] = o;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col + j < n_out) dst[j] = __float2bfloat16_rn(f[j]);
    }
}
// Same for the fp32 output alpha * acc + beta * C (c_row may be nullptr when beta == 0).
__device__ __forceinline__ void store_row_chunk_axpby(float* d_row, const float* c_row, int col, int n_out,
                                                      const float* f, float alpha, float beta) {
    if (col >= n_out) return;
    float* dst = d_row + col;
    const float* c = c_row != nullptr ? c_row + col : nullptr;
    if ((col + 32 <= n_out) && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) &&
        ((reinterpret_cast<uintptr_t>(c) & 15u) == 0)) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            float4 cv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c != nullptr) cv = __ldg(reinterpret_cast<const float4*>(c) + q);
            reinterpret_cast<float4*>(dst)[q] =
                make_float4(alpha * f[q * 4 + 0] + beta * cv.x, alpha * f[q * 4 + 1] + beta * cv.y,
                            alpha * f[q * 4 + 2] + beta * cv.z, alpha * f[q * 4 + 3] + beta * cv.w);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col + j < n_out) dst[j] = alpha * f[j] + (c != nullptr ? beta * c[j] : 0.0f);
    }
}

// Run by ONE warp: exclusive prefix sums of rows and tiles over the groups (32 groups per
// step), validation of m_sizes, and initialisation of the barriers.  `acc_empty_count` is
// the number of arrivals that hand an accumulator back to the MMA issuer.
template <int CTAS, int LESS>
__device__ __forceinline__ void build_tables_and_barriers(SmemTail* st, const GGParams& p, int lane, int tile_rows,
                                                          int acc_empty_count) {
    int row_carry = 0, tile_carry = 0, bad = 0;
    for (int base = 0; base < p.G; base += 32) {
        const int g = base + lane;
        // no size array = one group holding every row (the dense case)
        int m = g < p.G ? (p.m_sizes != nullptr ? p.m_sizes[g] : p.M) : 0;
        if (m < 0) {
            bad = 1;
            m = 0;
        }
        int tiles = group_row_tiles(m, tile_rows, p.tile_mode) * p.n_tiles;
        int rs = m, ts = tiles;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int r2 = __shfl_up_sync(0xffffffffu, rs, d);
            const int t2 = __shfl_up_sync(0xffffffffu, ts, d);
            if (lane >= d) {
                rs += r2;
                ts += t2;
            }
        }
        if (g < p.G) {
            st->row_off[g] = row_carry + rs - m;
            st->tile_off[g] = tile_carry + ts - tiles;
        }
        row_carry += __shfl_sync(0xffffffffu, rs, 31);
        tile_carry += __shfl_sync(0xffffffffu, ts, 31);
        if (row_carry > p.M) bad = 1;  // also stops int overflow of the running sum
    }
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) {
        st->row_off[p.G] = row_carry;
        st->tile_off[p.G] = tile_carry;
        st->total_tiles = bad ? 0 : tile_carry;
        st->invalid = bad;
        if (bad) report(p.status, kStatusBadGroupSizes);
        for (int s = 0; s < StageCfg<CTAS, LESS>::kStages; ++s) {
            mbar_init(&st->full[s], 1);
            mbar_init(&st->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&st->acc_full[b], 1);
            mbar_init(&st->acc_empty[b], acc_empty_count);
        }
        mbar_init(&st->out_full, 8);   // one arrival per promotion warp
        mbar_init(&st->out_empty, 2);  // one per sending warp
        mbar_init_fence();
    }
}

// TMA producer, run by ONE thread per CTA: for every tile of this cluster and every
// 128-byte slice of K, wait for a free stage and fetch this CTA's 128 rows of x and its
// share of the tile's two 128-row boxes of w[g] (rows nb0.. and nb1..).
//
// B_MN (16-bit operands only): w is [G, K, N] with N contiguous (an MN-major B operand, see
// make_sw128_mnmajor_desc).  The CTA's share of the tile's columns then arrives as boxes of 64 contraction
// rows x 64 columns, 8192 bytes each, one after another: columns c0.., c0+64.. (and two more when one CTA
// holds all 256 columns).  A half tile uses the first box of each CTA only; the second is fetched all the
// same so that every stage carries the same byte count.
template <int CTAS, int LESS, bool SWIGLU, bool HALF = false, bool B_MN = false>
__device__ __forceinline__ void producer_loop(const CUtensorMap* tm_x, const CUtensorMap* tm_w, SmemTail* st,
                                              uint32_t ring_addr, const GGParams& p, uint32_t cta_rank,
                                              int cluster_id, int num_clusters, int elems_per_stage, int num_kb) {
    using Cfg = StageCfg<CTAS, LESS>;
    constexpr int kTileRows = kRowsPerCta * CTAS;
    constexpr uint32_t kTxBytes = static_cast<uint32_t>(Cfg::kStageBytes) * CTAS;
    volatile int* abort_flag = &st->abort_flag;
    const int total_tiles = st->total_tiles;
    int g = 0, stage = 0;
    uint32_t phase = 0;
    const WorkSplit ws = make_work_split(total_tiles, num_clusters, HALF && CTAS == 2);
    // Called by the whole producer warp: coordinates and addresses are computed in warp-uniform
    // code, one elected lane issues the copies.
    const bool leader = elect_one();
    for (int wk = cluster_id; wk < ws.total_work; wk += num_clusters) {
        int t, half;
        decode_work(wk, ws, &t, &half);
        const TileCoord tc = locate_tile(t, g, st->tile_off, st->row_off, kTileRows, p.tile_mode);
        const int row0 = tc.row0 + static_cast<int>(cta_rank) * kRowsPerCta;
        int nb0 = SWIGLU ? tc.n_idx * 128 : tc.n_idx * kTileN;
        int nb1 = SWIGLU ? p.n_out + tc.n_idx * 128 : tc.n_idx * kTileN + 128;
        if (HALF && half >= 0) {
            // half tile (CTA pair only): each CTA still fetches a 128-row box of w, of which the
            // N = 128 MMA uses the first 64 rows
            nb0 = SWIGLU ? tc.n_idx * 128 + half * 64 : tc.n_idx * kTileN + half * 128;
            nb1 = SWIGLU ? p.n_out + tc.n_idx * 128 + half * 64 : tc.n_idx * kTileN + half * 128 + 64;
        }
        // B_MN: first column of this CTA's share (nb0 / nb1 above are exactly that for both tile kinds)
        const int mn_c0 = (CTAS == 1 || cta_rank == 0) ? nb0 : nb1;
        for (int kb = 0; kb < num_kb; ++kb) {
            if (!__all_sync(0xffffffffu, mbar_wait(&st->empty[stage], phase ^ 1u, abort_flag))) {
                report(p.status, kStatusTimeoutProducer);
                return;
            }
            const uint32_t a_dst = ring_addr + stage * Cfg::kStageBytes;
            const uint32_t b_dst = a_dst + kABytes;
            const int k0 = kb * elems_per_stage;                                     // position along K
            const int kx = k0 + static_cast<int>(tc.g * p.x_col_group_stride);      // column of x it sits at
            if constexpr (CTAS == 1) {
                const uint32_t bar = smem_u32(&st->full[stage]);
                if (leader) {
                    mbar_arrive_expect_tx(&st->full[stage], kTxBytes);
                    tma_load_2d(tm_x, bar, a_dst, kx, row0);
                    if constexpr (B_MN) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) tma_load_3d(tm_w, bar, b_dst + j * 8192, mn_c0 + j * 64, k0, tc.g);
                    } else {
                        tma_load_3d(tm_w, bar, b_dst, k0, nb0, tc.g);
                        tma_load_3d(tm_w, bar, b_dst + kSubBoxBytes, k0, nb1, tc.g);
                    }
                }
            } else {
                // Bytes of both CTAs are counted on the leader's barrier.
                const uint32_t bar = mapa_shared(smem_u32(&st->full[stage]), 0);
                if (leader) {
                    if (cta_rank == 0) mbar_arrive_expect_tx(&st->full[stage], kTxBytes);
                    tma_load_2d_pair(tm_x, bar, a_dst, kx, row0);
                    if constexpr (B_MN) {
                        tma_load_3d_pair(tm_w, bar, b_dst, mn_c0, k0, tc.g);
                        tma_load_3d_pair(tm_w, bar, b_dst + 8192, mn_c0 + 64, k0, tc.g);
                    } else {
                        tma_load_3d_pair(tm_w, bar, b_dst, k0, cta_rank == 0 ? nb0 : nb1, tc.g);
                    }
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

// ------------------------------------------------------------------ host side

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so the library links against the
// CUDA runtime only.
inline EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// x viewed as [rows, K]; box = 128 rows x 128 bytes, 128-byte swizzle.
inline int encode_x_map(CUtensorMap* m, const void* x, int rows, int K, int elem_bytes, bool is_f16 = false) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return kErrNoDriverEntry;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * elem_bytes};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(kRowBytes / elem_bytes), 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, elem_bytes == 2 ? (is_f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16)
                                     : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                     const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : kErrTensorMap;
}

// w viewed as [G, rows_per_group, K]; box = 1 group x 128 rows x 128 bytes.  The group
// is its own dimension so a box that runs past a group's last row is zero-filled
// instead of reading the next expert's weights.
inline int encode_w_map(CUtensorMap* m, const void* w, int G, int rows_per_group, int K, int elem_bytes,
                        bool is_f16 = false) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return kErrNoDriverEntry;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows_per_group),
                          static_cast<cuuint64_t>(G)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(K) * elem_bytes,
                             static_cast<cuuint64_t>(K) * elem_bytes * rows_per_group};
    cuuint32_t box[3] = {static_cast<cuuint32_t>(kRowBytes / elem_bytes), 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(m, elem_bytes == 2 ? (is_f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16)
                                     : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                     const_cast<void*>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : kErrTensorMap;
}

// w viewed as [G, K rows, N] with N contiguous (16-bit elements); box = 64 rows x 64 columns (128 bytes),
// 128-byte swizzle: the MN-major B operand of producer_loop<..., B_MN = true>.
inline int encode_w_mn_map(CUtensorMap* m, const void* w, int G, int K, int N, bool is_f16 = false) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return kErrNoDriverEntry;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(G)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(N) * 2, static_cast<cuuint64_t>(N) * 2 * K};
    cuuint32_t box[3] = {64, 64, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(m, is_f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                     const_cast<void*>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : kErrTensorMap;
}

struct DeviceInfo {
    int sms = 0;
    int cc_major = 0, cc_minor = 0;
};
inline int get_device_info(DeviceInfo* out) {
    static thread_local int cached_dev = -1;
    static thread_local DeviceInfo cached;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev != cached_dev) {
        cudaDeviceProp prop;
        e = cudaGetDeviceProperties(&prop, dev);
        if (e != cudaSuccess) return static_cast<int>(e);
        cached.sms = prop.multiProcessorCount;
        cached.cc_major = prop.major;
        cached.cc_minor = prop.minor;
        cached_dev = dev;
    }
    *out = cached;
    return 0;
}

}  // namespace b200moe
