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

// ---------------------------------------------------------------------------------------
// De-duplicating protocol ("dedup" mode, the default)
// ---------------------------------------------------------------------------------------
// The reference sends one row per (token, k) entry in both directions
// (all2all/reference.py:79-86,107-112; all2all/hipv8.py:80-97,144-161).  Here a token's
// row crosses NVLink once per DESTINATION RANK: the sender stores it into a landing
// buffer on the owner, indexed by (source rank, token), together with the final row
// index of each of the token's entries on that owner.  The owner then replicates the
// landed row into expert_x[e_local, slot] with local copies, so the dispatch layouts
// stay those of the reference.  On the way back the owner forms, per (source, token),
// the weighted sum over its local experts in fp32 and pushes that ONE row into the
// source's return buffer; the source adds the rows of the owners it used.
struct MoeDedupLayout {
  uint64_t off_counts;       // int32 [world][num_experts]; row s is written by rank s
  uint64_t off_expert_x;     // dtype [E_local][max_recv][hidden]
  uint64_t off_expert_meta;  // int32 [E_local][max_recv][5]
  uint64_t off_expert_y;     // dtype [E_local][max_recv][hidden]
  uint64_t off_land;         // dtype [world][max_tokens][hidden]: row (s, t) = token t of rank s
  uint64_t off_tok_rec;      // int32 [world][max_tokens][rec_ints]: one record per (source s, token t), written by
                             // the sender with ONE coalesced store: [0] low word of the dispatch epoch that landed
                             // it, [1, 1+k) final row of entry k on this rank or -1, [1+k, 1+2k) its routing weight
  uint64_t off_ret;          // dtype or float [world][max_tokens][hidden]: row (d, t) = owner d's partial of my token t
};

struct MoeDedupDispatchParams {
  const void* x;             // [T, hidden]
  const int32_t* indices;    // [T, k]
  const float* weights;      // [T, k] or nullptr (then combine sends them)
  int32_t num_tokens, k, num_experts, num_local_experts, world_size, rank, max_recv, max_tokens;
  int32_t rec_ints;          // int32 words per (source, token) record: 1 + 2k rounded up to a multiple of 4
  int32_t dtype;             // 0 = fp16, 1 = bf16, 2 = fp32
  uint32_t row_bytes;
  int32_t pieces;            // a row is landed by this many warps (small problems)
  int32_t rep_pieces;        // a landed row is replicated by this many warps (evens out the warps' shares)
  int32_t chunks;            // the large kernel lands its tokens in this many chunks, each with its own
                             // "delivered" flag, so that the owners replicate chunk c while c + 1 is in flight
  int32_t bulk_landing;      // 1: rows cross to the owners as bulk copies through shared memory (cp.async.bulk),
                             // 0: as 16-byte stores from registers
  int32_t fuse_scale;        // 1: the replication pass also writes expert_y = expert_x * scale
  float scale;
  uint64_t epoch, timeout_ns;
  uint64_t peer_base[kMaxWorldSize];
  MoeDedupLayout layout;
  void* expert_y;            // where the fused expert op writes (this rank's buffer)
  int32_t* blk_hist;         // [grid][num_experts] (large kernel only)
  int2* route;               // [T*k] (owner rank, row) or (-1, -1)
  int32_t* expert_num_tokens;
  uint32_t* sync_counters;   // [0] grid barrier, [1] finished CTAs, [4] CTAs that have published their count rows
  StatusBlock* status;
  uint64_t* trace;           // optional [8] globaltimer stamps of CTA 0: start, counted, rows issued,
                             // counts arrived, metadata stored, all sources delivered, replicated, (max) exit
};

struct MoeDedupCombineParams {
  void* out;                 // [T, hidden]
  const float* weights;      // [T, k]
  const int2* route;         // from dispatch
  const void* expert_y;      // this rank's expert outputs, dispatch layout (any local tensor)
  int32_t num_tokens, k, hidden, num_local_experts, world_size, rank, max_recv, max_tokens;
  int32_t rec_ints;
  int32_t dtype;
  int32_t partial_fp32;      // return rows travel as fp32 instead of dtype
  int32_t weights_sent;      // dispatch already delivered the weights
  int32_t pieces;
  uint64_t epoch, dispatch_epoch, timeout_ns;
  uint64_t peer_base[kMaxWorldSize];
  MoeDedupLayout layout;
  uint32_t* sync_counters;   // [2] weights pushed, [3] partial rows pushed
  StatusBlock* status;
  uint64_t* trace;           // optional [8]: start, weights exchanged, partials pushed, all partials arrived, (max) exit
};

// True when a problem of this size takes the barrier-free small dispatch kernel.
bool moe_dedup_is_small(int num_entries, int num_experts);
// Co-resident grid sizes (cooperative launches) for the current device.
int moe_dedup_dispatch_max_blocks(int device, int num_experts, int num_entries, int bulk_landing);
int moe_dedup_combine_max_blocks(int device);
cudaError_t launch_moe_dedup_dispatch(const MoeDedupDispatchParams& p, int grid, cudaStream_t stream);
cudaError_t launch_moe_dedup_combine(const MoeDedupCombineParams& p, int grid, cudaStream_t stream);

}  // namespace b200
