// Launchers of the memory-bound MoE helper kernels (internal to libb200moe.so).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200moe {

// Per-warp histograms of E counters must fit the default 48 KiB of dynamic shared memory.
constexpr int kRouteMaxExperts = 2048;
constexpr int kRouteMaxChunks = 1024;

// Splits R ids into chunks for the routing kernels; scratch needed = num_chunks * E int32.
int route_plan(int R, int E, int* chunk_len, int* num_chunks);
int route_launch(const int32_t* ids, int R, int E, int32_t* m_sizes, int32_t* offsets, int32_t* perm,
                 int32_t* inv_perm, int32_t* counts, int32_t* status, cudaStream_t stream);
// Routing with the scratch in a fixed array inside the library (num_chunks * E <= capacity).
int route_static_capacity_ints();
int route_static_launch(const int32_t* ids, int R, int E, int32_t* m_sizes, int32_t* offsets, int32_t* perm,
                        int32_t* inv_perm, int32_t* status, cudaStream_t stream);
// vLLM-format padded layout built on the routing kernels; scratch = align_blocks_scratch_ints() int32.
long long align_blocks_scratch_ints(int R, int E);
int align_blocks_launch(const int32_t* ids, int R, int E, int block_size, int32_t* sorted_ids, int32_t* expert_ids,
                        int32_t* num_tokens_post_pad, int32_t* scratch, int32_t* status, cudaStream_t stream);
int gather_rows_launch(const void* src, const int32_t* idx, int div, void* dst, int rows, long long row_bytes,
                       int src_rows, cudaStream_t stream);
int swiglu_launch(const void* in, void* out, long long rows, int d, cudaStream_t stream);
int combine_topk_launch(const void* y, const int32_t* inv_perm, const float* weight, void* out, int T, int k, int H,
                        int y_rows, cudaStream_t stream);
int quant_1x128_launch(const void* x, int x_is_fp32, void* q, float* scales, long long rows, int K,
                       cudaStream_t stream);

// Expert-parallel dispatch over peer memory (ep_kernels.cu).
int ep_plan_launch(const int32_t* counts, int P, int E, int me, int cap, int32_t* dst_base, int32_t* m_loc,
                   int32_t* status, cudaStream_t stream);
int ep_barrier_launch(int32_t* const* flag_blocks, int P, int me, int slot, int epoch, unsigned long long limit_ns,
                      int32_t* status, cudaStream_t stream);
int ep_push_launch(const void* part0, long long bytes0, const void* part1, long long bytes1, const int32_t* perm,
                   int k, const int32_t* offsets, const int32_t* dst_base, int R, int E, int P, int me, int cap,
                   int tokens, void* const* peer0, void* const* peer1, long long* const* peer_tag, void* home,
                   long long home_row_bytes, cudaStream_t stream);
int enable_peer_access(int peer_device);
int ipc_open(const void* handle_bytes, void** base);
int ipc_export(const void* dev_ptr, void* handle_out64, unsigned long long* offset_out);
int ipc_close(void* base);
int peer_probe(void* peer_ptr, void* local_scratch8);

}  // namespace b200moe
