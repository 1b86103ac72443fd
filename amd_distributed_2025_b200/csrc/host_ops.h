// The two operators on CPU ranks of one node, over the shared-memory heap (host_shm_heap.h).
//
// These are the device kernels' protocols restated for ordinary processes: the same flag
// rows and epochs, the same buffer layouts, the same one-sided data movement (a sender
// writes rows straight into the owner's expert buffer; combine pulls rows out of the
// owners' output buffers; a rank stores its partial row blocks into the owners' staging
// slots), the same bounded waits and status records.  They give the framework a CPU
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

// Data movement of the reduce-scatter.  partial [M][N] is this rank's GEMM output; row block r
// goes to slot [src = this rank] of rank r's staging area stage[world][M / world][N] (the own
// block is not copied).  Returns once every peer's block for this rank has arrived; the sum
// is the caller's.
StatusWord host_rs_exchange(HostShmHeap& heap, uint64_t stage_offset, const void* partial, int m, int n,
                            int elem_bytes, uint64_t epoch, uint64_t timeout_ns);

}  // namespace b200
