// The two operators on CPU ranks of one node, over the shared-memory heap (host_shm_heap.h).
//
// These are the device kernels' protocols restated for ordinary processes: the same flag
// rows and epochs, the same buffer layouts, the same one-sided data movement (a sender
// writes rows straight into the owner's expert buffer, or once per destination rank into
// its landing buffer with a record of the final rows; combine pulls rows out of the
// owners' output buffers, or the owners push one pre-reduced row per token back; a rank
// stores its partial row blocks into the owners' staging slots), the same bounded waits
// and status records.  They give the framework a CPU
// backend that needs no collective library, and they let the multi-rank protocol -- slot
// arithmetic, who signals whom, why no barrier is needed between calls -- run under real
// concurrency on any number of ranks without a GPU.  Only protocol and data movement live
// here; the arithmetic (expert scale, weighted sum, sum of partials) is done with the tensor
// library's vectorised CPU kernels by the callers in bindings.cpp.
//
// The reference's CPU path is its oracle: Python loops around gloo collectives
// (all2all/reference.py:63-234, gemm-rs/reference.py:52-59).
#pragma once
#include <stdint.h>

#include "host_shm_heap.h"
#include "status.h"

namespace b200 {

enum HostDtype : int { HOST_F16 = 0, HOST_BF16 = 1, HOST_F32 = 2 };

inline int host_dtype_bytes(int dt) { return dt == HOST_F32 ? 4 : 2; }

// Slab regions (byte offsets from the slab base, identical on every rank).
struct HostMoeLayout {
  uint64_t counts;       // int32 [world][num_experts]; row s written by rank s
  uint64_t expert_x;     // in_dtype [local_experts][max_recv][hidden]
  uint64_t expert_meta;  // int32 [local_experts][max_recv][5]
  uint64_t expert_y;     // out_dtype [local_experts][max_recv][hidden]
};

struct HostMoeShape {
  int num_experts, topk, hidden, max_recv;
  int in_dtype, out_dtype;  // HostDtype
};

// Dispatch.  x [num_tokens][hidden] in_dtype, indices [num_tokens][topk] int32.
// route [num_tokens * topk][3] int32 receives (owner rank, local expert, slot) per entry;
// expert_num_tokens [local_experts] int32 receives the rows every local expert holds.
// Rows of one expert are ordered by source rank, then by (token, k).
StatusWord host_moe_dispatch(HostShmHeap& heap, const HostMoeLayout& lay, const HostMoeShape& s, const void* x,
                             const int32_t* indices, int num_tokens, int32_t* route, int32_t* expert_num_tokens,
                             uint64_t epoch, uint64_t timeout_ns);

// First half of combine: announces this rank's expert_y, waits for everybody's, then copies the
// rows named by `route` out of their owners' expert_y into rows [num_tokens * topk][hidden]
// (out_dtype; zeros for entries that dispatch skipped).  The weighted sum is the caller's.
StatusWord host_moe_pull(HostShmHeap& heap, const HostMoeLayout& lay, const HostMoeShape& s, const int32_t* route,
                         int num_tokens, void* rows, uint64_t epoch, uint64_t timeout_ns);

// ---- the "dedup" protocol of the device kernels (moe_dedup.cu), between CPU ranks -----------
// A token's row crosses to every destination RANK once (into that rank's landing buffer), with
// one record per (source, token) naming the final rows of its entries there; the owner copies
// the landed row into those rows of expert_x itself and writes expert_meta.  Combine sends one
// pre-reduced row per (token, owner rank) back.  Same regions and record format as the device
// layout (moe.h, MoeDedupLayout).
struct HostMoeDedupLayout {
  uint64_t counts;       // int32 [world][num_experts]
  uint64_t expert_x;     // in_dtype [local_experts][max_recv][hidden]
  uint64_t expert_meta;  // int32 [local_experts][max_recv][5]
  uint64_t expert_y;     // out_dtype [local_experts][max_recv][hidden]
  uint64_t land;         // in_dtype [world][max_tokens][hidden]: row (s, t) = token t of rank s
  uint64_t tok_rec;      // int32 [world][max_tokens][rec_ints]: [0] low word of the dispatch call number,
                         // [1, 1+k) final row of entry k on this rank or -1, [1+k, 1+2k) its routing weight
  uint64_t ret;          // [world][max_tokens][hidden] of ret_elem_bytes: row (d, t) = owner d's partial of my token t
};

struct HostMoeDedupShape {
  int num_experts, topk, hidden, max_recv, max_tokens, rec_ints;
  int in_dtype, out_dtype;  // HostDtype
  int chunks;               // this rank lands its tokens in so many chunks, each announced by its own flag value
};

// Dispatch.  route [num_tokens * topk][2] int32 receives (owner rank, row on the owner =
// local expert * max_recv + slot, or -1 for an entry that was dropped); expert_num_tokens as above.
// Returns when the rows of every source have been copied into this rank's expert_x.
StatusWord host_moe_dedup_dispatch(HostShmHeap& heap, const HostMoeDedupLayout& lay, const HostMoeDedupShape& s,
                                   const void* x, const int32_t* indices, int num_tokens, int32_t* route,
                                   int32_t* expert_num_tokens, uint64_t epoch, uint64_t timeout_ns);

// Combine, step 1: the routing weights of this rank's tokens go into the records on the owners;
// returns when every source's weights are here.  (The owner's weighted sums are the caller's.)
StatusWord host_moe_dedup_send_weights(HostShmHeap& heap, const HostMoeDedupLayout& lay, const HostMoeDedupShape& s,
                                       const int32_t* route, const float* weights, int num_tokens, uint64_t epoch,
                                       uint64_t timeout_ns);

// Combine, step 2, after the caller has stored its partial rows into the sources' return buffers:
// "my partials are in place" to everyone; returns when every owner's partials are here.
StatusWord host_moe_dedup_return(HostShmHeap& heap, uint64_t epoch, uint64_t timeout_ns);

// Data movement of the reduce-scatter.  partial [M][N] is this rank's GEMM output; row block r
// goes to slot [src = this rank] of rank r's staging area stage[world][M / world][N] (the own
// block is not copied).  Returns once every peer's block for this rank has arrived; the sum
// is the caller's.
StatusWord host_rs_exchange(HostShmHeap& heap, uint64_t stage_offset, const void* partial, int m, int n,
                            int elem_bytes, uint64_t epoch, uint64_t timeout_ns);

}  // namespace b200
