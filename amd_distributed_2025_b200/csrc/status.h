// Status words shared by device kernels and the host runtime.
//
// Every device-side wait in this library is bounded.  When a wait gives up, the kernel
// records *where* in a StatusWord that lives in mapped pinned host memory, stops
// waiting and returns normally, so the CUDA context stays usable and the host can turn
// the record into an exception.  The reference has no counterpart: a lost rank hangs
// its collective forever (all2all/hipv8.py:281,305).
#pragma once
#include <stdint.h>

namespace b200 {

enum StatusCode : uint32_t {
  STATUS_OK = 0,
  STATUS_TIMEOUT = 1,       // a bounded wait expired (phase/peer say which)
  STATUS_BAD_INDEX = 2,     // an expert id, slot or offset was out of range and was skipped
  STATUS_BAD_ARGUMENT = 3,  // host-side validation failed
};

enum Phase : uint32_t {
  PHASE_NONE = 0,
  PHASE_GRID_BARRIER = 1,
  PHASE_MOE_COUNTS = 2,      // waiting for the peers' per-expert count rows
  PHASE_MOE_DATA = 3,        // waiting for the peers' "rows delivered" flag
  PHASE_MOE_Y_READY = 4,     // waiting for the peers' "expert output ready" flag
  PHASE_RS_PARTIALS = 5,     // waiting for partial tiles of a reduce-scatter block
  PHASE_GEMM_PIPELINE = 6,   // an mbarrier of the GEMM pipeline
  PHASE_BARRIER = 7,         // stand-alone cross-GPU barrier
  PHASE_TEST = 8,            // wait used by the timeout self-test
  PHASE_MOE_WEIGHTS = 9,     // waiting for the sources' routing weights (combine without a fused dispatch)
  PHASE_MOE_RETURN = 10,     // waiting for the owners' pre-reduced return rows
};

struct StatusWord {
  uint32_t code;    // StatusCode; first error wins
  uint32_t phase;   // Phase
  int32_t peer;     // peer rank the wait was on, or -1
  int32_t detail;   // kernel specific (block id, expert id, ...)
  uint64_t epoch;   // call number of the failing wait
  uint64_t seen;    // last value read from the flag
};

// Device-resident status record.  `word` is updated with device atomics; when a failure
// is recorded its fields are also copied, with plain stores, to `host_mirror` (mapped
// pinned host memory) so the host can poll it without synchronising the stream.
struct StatusBlock {
  StatusWord word;
  StatusWord* host_mirror;
};

constexpr int kMaxWorldSize = 16;

// Flag rows inside the symmetric heap header; each row has kMaxWorldSize 64-bit slots,
// slot s of a row on rank d is written only by rank s.
enum FlagRow : int {
  FLAG_BARRIER = 0,
  FLAG_MOE_COUNTS = 1,
  FLAG_MOE_DATA = 2,
  FLAG_MOE_Y_READY = 3,
  FLAG_RS_DONE = 4,
  FLAG_TEST = 5,
  FLAG_MOE_RET = 6,
  FLAG_MOE_INFO = 7,   // per source: how it cut its tokens into chunks (not a flag anybody waits on)
  FLAG_ROWS = 8,
};

constexpr uint64_t kFlagBytes = uint64_t(FLAG_ROWS) * kMaxWorldSize * sizeof(uint64_t);
// Header of every symmetric heap: flags, then padding up to 4 KiB.
constexpr uint64_t kHeapHeaderBytes = 4096;

}  // namespace b200
