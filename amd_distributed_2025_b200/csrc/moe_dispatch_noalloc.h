// Single-GPU MoE dispatch for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference.
//
// Who needs it: code that runs where cudaMalloc is off limits -- inside a latency-critical
// serving loop whose memory was carved up front, under a host framework that owns the
// whole device heap and forbids foreign allocations, or in a plug-in loaded by a process
// that has already handed every free byte to its own pool, so that a late cudaMalloc
// would fail or stall the device.  The regular path (MoEAllToAll.dispatch) creates a
// symmetric workspace with cudaMalloc and lets torch allocate its scratch tensors; this
// variant takes the caller's input and output buffers and keeps every intermediate
// (count matrix, per-chunk histograms, per-entry ranks, flags, barrier counters, status)
// in one file-scope __device__ array inside this library.
//
// Limits (checked; a call beyond them returns an error and launches nothing):
//   world size 1 only (all experts are local), num_experts <= 1024,
//   num_tokens * experts_per_token <= 65536, at most 160 SMs.
// The scratch array is B200_NOALLOC_SCRATCH_BYTES (1 MiB) and is resident on every GPU
// that loads this library until the process exits.
//
// Behaviour to know about:
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress) and caches it; make that first call outside any stream
//     capture.  Later calls do no set-up.
//   * All calls on a device share the one array.  Two calls whose kernels can overlap on
//     the GPU (different streams, no dependency) race on it; serialise them.
//   * The array keeps what the previous call left.  Each call clears, on the given
//     stream, the words that must start at zero (barrier counters, status); flags are
//     compared against a call number that only grows, so old values are harmless.
//   * An entry whose expert id is outside [0, num_experts), or whose slot would not fit
//     max_recv, is dropped: its route is (-1, -1), the other entries are served and
//     b200_moe_dispatch_noalloc_status() reports 2.
//   * Call numbers are handed out under a lock in the order the host threads get there; two
//     host threads that call concurrently may launch in the opposite order, which the flag
//     comparison tolerates only if their kernels do not overlap -- one more reason to
//     serialise callers.  Kernel waits are bounded at 2 seconds.
//   * Nothing here calls cudaMalloc, cudaFree, cudaHostAlloc or any torch allocator.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define B200_NOALLOC_SCRATCH_BYTES (1u << 20)
#define B200_NOALLOC_MAX_EXPERTS 1024
#define B200_NOALLOC_MAX_ENTRIES 65536
#define B200_NOALLOC_MAX_SMS 160

#ifdef __cplusplus
extern "C" {
#endif

// Dispatch the rows of x[num_tokens, row_bytes] to their experts on this GPU.
//   indices          [num_tokens, experts_per_token] int32 expert ids
//   expert_x         out: [num_experts, max_recv, row_bytes] bytes
//   expert_meta      out: [num_experts, max_recv, 5] int32 (expert, 0, token, k, 0)
//   expert_num_tokens out: [num_experts] int32
//   route            out: [num_tokens * experts_per_token, 2] int32 (0, expert * max_recv + slot)
// All pointers are device pointers owned by the caller; row_bytes is hidden * element size.
// Returns 0 on success, a negative value on a rejected argument (see
// b200_moe_dispatch_noalloc_error) or a positive cudaError_t from the runtime.
int b200_moe_dispatch_noalloc(const void* x, const int32_t* indices, int num_tokens, int experts_per_token,
                              int row_bytes, int num_experts, int max_recv, void* expert_x, int32_t* expert_meta,
                              int32_t* expert_num_tokens, int32_t* route, cudaStream_t stream);

// Text for the last non-zero return value of the calling thread.
const char* b200_moe_dispatch_noalloc_error(void);

// Synchronises the device and reports what the last kernel recorded: 0 = clean,
// 1 = a bounded wait expired, 2 = an out-of-range expert id or slot was skipped.
int b200_moe_dispatch_noalloc_status(void);

#ifdef __cplusplus
}
#endif
