// Allocation-free single-GPU MoE dispatch (see moe_dispatch_noalloc.h).
#include "moe_dispatch_noalloc.h"

#include <algorithm>
#include <cstdio>
#include <mutex>

#include "moe.h"
#include "status.h"

namespace {

// Every intermediate of the dispatch kernel lives here.  In host code `g_scratch` is only
// a handle for the runtime, never an address a kernel may use: the device address comes
// from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_scratch[B200_NOALLOC_SCRATCH_BYTES];

// Carving of the array (byte offsets).  The first block mirrors a symmetric-heap header so
// the unchanged kernel finds its flags at "heap base + row * 16 + slot".
constexpr uint64_t kOffFlags = 0;
constexpr uint64_t kOffCounts = b200::kHeapHeaderBytes;                                    // int32 [1][1024]
constexpr uint64_t kOffSync = kOffCounts + B200_NOALLOC_MAX_EXPERTS * 4;                   // uint32 [64]
constexpr uint64_t kOffStatus = kOffSync + 256;                                           // StatusBlock
constexpr uint64_t kOffLocalRank = kOffStatus + 256;                                      // int32 [65536]
constexpr uint64_t kOffBlkHist = kOffLocalRank + (uint64_t)B200_NOALLOC_MAX_ENTRIES * 4;  // int32 [blocks][experts]
constexpr uint64_t kBlkHistBytes = B200_NOALLOC_SCRATCH_BYTES - kOffBlkHist;
static_assert(kOffBlkHist < B200_NOALLOC_SCRATCH_BYTES, "scratch array too small");
static_assert(sizeof(b200::StatusBlock) <= 256, "status block does not fit its slot");

constexpr int kMaxDevices = 64;
struct DeviceState {
  unsigned char* base = nullptr;  // device address of g_scratch on this device
  uint64_t epoch = 0;             // call number; flags are compared against it
  int sms = 0;
};
DeviceState g_state[kMaxDevices];
std::mutex g_mutex;

thread_local char g_error[256] = "";

int fail(int code, const char* msg) {
  std::snprintf(g_error, sizeof(g_error), "%s", msg);
  return code;
}

}  // namespace

extern "C" int b200_moe_dispatch_noalloc(const void* x, const int32_t* indices, int num_tokens, int experts_per_token,
                                         int row_bytes, int num_experts, int max_recv, void* expert_x,
                                         int32_t* expert_meta, int32_t* expert_num_tokens, int32_t* route,
                                         cudaStream_t stream) {
  if (num_tokens < 0 || experts_per_token <= 0 || row_bytes <= 0 || (row_bytes & 1) || max_recv <= 0)
    return fail(-1, "b200_moe_dispatch_noalloc: num_tokens, experts_per_token, row_bytes (even) and max_recv must be positive");
  if (num_experts <= 0 || num_experts > B200_NOALLOC_MAX_EXPERTS)
    return fail(-2, "b200_moe_dispatch_noalloc: num_experts exceeds the built-in maximum of 1024");
  const long long n = (long long)num_tokens * experts_per_token;
  if (n > B200_NOALLOC_MAX_ENTRIES)
    return fail(-3, "b200_moe_dispatch_noalloc: num_tokens * experts_per_token exceeds the built-in maximum of 65536");
  if ((long long)num_experts * max_recv >= (1ll << 31))
    return fail(-4, "b200_moe_dispatch_noalloc: num_experts * max_recv does not fit 32-bit row ids");
  if ((n > 0 && (x == nullptr || indices == nullptr || route == nullptr)) || expert_x == nullptr ||
      expert_meta == nullptr || expert_num_tokens == nullptr)
    return fail(-5, "b200_moe_dispatch_noalloc: null buffer");

  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  if (dev < 0 || dev >= kMaxDevices) return fail(-6, "b200_moe_dispatch_noalloc: device ordinal out of range");

  DeviceState* st;
  uint64_t epoch;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    st = &g_state[dev];
    if (st->base == nullptr) {
      // One-time set-up for this device (it is the current device): resolve the device
      // address of the scratch array.  Not an allocation; do it outside stream capture.
      void* ptr = nullptr;
      err = cudaGetSymbolAddress(&ptr, g_scratch);
      if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
      err = cudaDeviceGetAttribute(&st->sms, cudaDevAttrMultiProcessorCount, dev);
      if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
      st->base = static_cast<unsigned char*>(ptr);
    }
  }
  if (st->sms > B200_NOALLOC_MAX_SMS)
    return fail(-7, "b200_moe_dispatch_noalloc: device has more SMs than the scratch array was sized for");

  // Same work split as the regular path: contiguous chunks of (token, k) entries per CTA.
  const int max_blocks = st->sms;
  long long chunk = (n + max_blocks - 1) / max_blocks;
  if (chunk < 32) chunk = 32;
  const long long count_blocks = (n + chunk - 1) / chunk;
  if ((uint64_t)std::max<long long>(count_blocks, 1) * num_experts * 4 > kBlkHistBytes)
    return fail(-8, "b200_moe_dispatch_noalloc: histogram does not fit the scratch array");
  int grid = max_blocks;
  const long long want = std::max<long long>(std::max<long long>(count_blocks, (n + 7) / 8), 1);
  if (want < grid) grid = (int)want;
  {
    // every argument check has passed: only now does the call take a call number
    std::lock_guard<std::mutex> lock(g_mutex);
    epoch = ++st->epoch;
  }

  unsigned char* base = st->base;
  // Words that must start at zero: barrier counters and the status block.  Flags and the
  // count row are overwritten or compared against `epoch`, the rest is written before use.
  err = cudaMemsetAsync(base + kOffSync, 0, 512, stream);
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));

  b200::MoeDispatchParams p;
  p.x = x;
  p.indices = indices;
  p.num_tokens = num_tokens;
  p.k = experts_per_token;
  p.num_experts = num_experts;
  p.num_local_experts = num_experts;
  p.world_size = 1;
  p.rank = 0;
  p.max_recv = max_recv;
  p.row_bytes = (uint32_t)row_bytes;
  p.epoch = epoch;
  p.timeout_ns = 2000000000ull;
  for (int r = 0; r < b200::kMaxWorldSize; ++r) p.peer_base[r] = 0;
  const uint64_t heap = reinterpret_cast<uint64_t>(base);
  p.peer_base[0] = heap;
  // The kernel addresses outputs as "heap base + offset"; the caller's buffers are
  // expressed as (unsigned, wrapping) offsets from the scratch base.
  p.layout.off_counts = kOffCounts;
  p.layout.off_expert_x = reinterpret_cast<uint64_t>(expert_x) - heap;
  p.layout.off_expert_meta = reinterpret_cast<uint64_t>(expert_meta) - heap;
  p.layout.off_expert_y = 0;
  p.blk_hist = reinterpret_cast<int32_t*>(base + kOffBlkHist);
  p.local_rank = reinterpret_cast<int32_t*>(base + kOffLocalRank);
  p.route = reinterpret_cast<int2*>(route);
  p.expert_num_tokens = expert_num_tokens;
  p.sync_counters = reinterpret_cast<uint32_t*>(base + kOffSync);
  p.status = reinterpret_cast<b200::StatusBlock*>(base + kOffStatus);  // host_mirror stays null
  p.count_blocks = (int32_t)count_blocks;
  p.chunk = (int32_t)chunk;
  err = b200::launch_moe_dispatch(p, grid, stream);
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  g_error[0] = '\0';
  return 0;
}

extern "C" const char* b200_moe_dispatch_noalloc_error(void) { return g_error; }

extern "C" int b200_moe_dispatch_noalloc_status(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  unsigned char* base;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    base = g_state[dev].base;
  }
  if (base == nullptr) return 0;
  b200::StatusBlock blk;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpy(&blk, base + kOffStatus, sizeof(blk), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return (int)blk.word.code;
}
