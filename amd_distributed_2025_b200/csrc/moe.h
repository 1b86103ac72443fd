// Host-callable launchers of the MoE expert-parallel kernels (no torch types here).
//
// Capability: dispatch -> expert op -> combine of the reference task
// (all2all/reference.py:68-234; device kernels all2all/hipv8.py:60-226).  The reference
// moves rows through packed staging buffers and four library all-to-alls; here the
// dispatch kernel stores every row straight into the owning rank's expert buffer over
// NVLink and the combine kernel pulls expert outputs from peer memory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "status.h"

namespace b200 {

struct MoeLayout {
  // Byte offsets inside every rank's symmetric heap (identical on all ranks).
  uint64_t off_counts;       // int32 [world][num_experts]; row s is written by rank s
  uint64_t off_expert_x;     // in_dtype [E_local][max_recv][hidden]
  uint64_t off_expert_meta;  // int32 [E_local][max_recv][5]
  uint64_t off_expert_y;     // out_dtype [E_local][max_recv][hidden]
};

struct MoeDispatchParams {
  const void* x;             // [T, hidden] rows of row_bytes each
  const int32_t* indices;    // [T, k]
  int32_t num_tokens, k, num_experts, num_local_experts, world_size, rank, max_recv;
  uint32_t row_bytes;        // hidden * sizeof(in_dtype)
  uint64_t epoch;
  uint64_t timeout_ns;
  uint64_t peer_base[kMaxWorldSize];  // this process's mapping of every rank's heap
  MoeLayout layout;
  // Local scratch (never touched by peers).
  int32_t* blk_hist;         // [count_blocks][num_experts]
  int32_t* local_rank;       // [T*k] position of an entry among equal experts inside its chunk
  int2* route;               // [T*k] (owner rank, row index e_local*max_recv+slot); row -1 = dropped
  int32_t* expert_num_tokens;  // [E_local] output
  uint32_t* sync_counters;   // [2]: grid barrier, finished CTAs; zero between launches
  StatusBlock* status;
  int32_t count_blocks;      // CTAs that take part in counting (<= grid)
  int32_t chunk;             // entries per counting CTA
};

struct MoeCombineParams {
  void* out;                 // [T, hidden] out_dtype
  const float* weights;      // [T, k]
  const int2* route;         // [T*k] from dispatch
  int32_t num_tokens, k, hidden, world_size, rank, max_recv;
  int32_t dtype;             // 0 = fp16, 1 = bf16, 2 = fp32
  uint64_t epoch;
  uint64_t timeout_ns;
  uint64_t peer_base[kMaxWorldSize];
  uint64_t off_expert_y;
  StatusBlock* status;
};

// Number of CTAs the dispatch kernel may use on the current device (co-resident).
int moe_dispatch_max_blocks(int device);

cudaError_t launch_moe_dispatch(const MoeDispatchParams& p, int grid, cudaStream_t stream);

// Variant for small problems (a few thousand (token, k) entries): same protocol and layouts,
// but every CTA derives the slots from the full index list, so there is no in-GPU barrier.
// blk_hist, local_rank, count_blocks and chunk of the parameters are not used.
bool moe_dispatch_small_applies(int num_entries, int num_experts);
cudaError_t launch_moe_dispatch_small(const MoeDispatchParams& p, int grid, cudaStream_t stream);

// expert_y[e, j, :] = cast(expert_x[e, j, :]) * scale for j < expert_num_tokens[e];
// padding rows are not touched (all2all/reference.py:262 scales the padded buffer too,
// but only valid rows are ever read back).
cudaError_t launch_moe_expert_scale(const void* expert_x, void* expert_y, const int32_t* expert_num_tokens,
                                    int num_local_experts, int max_recv, int hidden, int in_dtype,
                                    int out_dtype, float scale, cudaStream_t stream);

cudaError_t launch_moe_combine(const MoeCombineParams& p, cudaStream_t stream);

}  // namespace b200
