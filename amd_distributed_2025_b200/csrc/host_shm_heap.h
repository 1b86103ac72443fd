// Host-memory stand-in for the symmetric heap: one POSIX shared-memory slab per rank, mapped
// by every rank of a node, with the same header of epoch flags and the same bounded-wait /
// status semantics as the device runtime (symm_heap.h, signal.cuh).
//
// It exists so that the signalling protocol -- who writes which flag slot, epochs instead of
// resets, a wait that gives up and reports where -- can be exercised by ordinary CPU
// processes: with a peer that signals late, never signals, or exits.  The reference has no
// counterpart (its ranks meet only inside library collectives, all2all/hipv8.py:281).
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "status.h"

namespace b200 {

class HostShmHeap {
 public:
  // Creates this rank's slab "/<prefix>_<rank>" of `bytes` (>= header); a fresh segment is all zero.
  HostShmHeap(const std::string& prefix, int rank, int world_size, uint64_t bytes);
  ~HostShmHeap();
  HostShmHeap(const HostShmHeap&) = delete;
  HostShmHeap& operator=(const HostShmHeap&) = delete;

  // Maps the peers' slabs, waiting up to timeout_ns for them to appear.  Returns false on timeout.
  bool open_peers(uint64_t timeout_ns);
  void close();
  // Removes the slab's name; mappings stay valid.  Once every rank has mapped every slab (a
  // barrier after open_peers) the names are no longer needed, and a rank that is killed
  // later leaves nothing behind in /dev/shm.
  void unlink();

  int rank() const { return rank_; }
  int world_size() const { return world_; }
  uint64_t bytes() const { return bytes_; }
  uint8_t* base(int r) const { return base_[r]; }

  // rank -> dst: "my value for `row` is now `epoch`" (release store into slot [row][rank] on dst).
  void signal(int row, int dst, uint64_t epoch);
  // Wait until slot [row][src] of the own slab reaches `epoch`; STATUS_TIMEOUT (with phase, peer,
  // epoch, last value seen) after timeout_ns.  The first failure is also kept in last_status().
  StatusWord wait(int row, int src, uint64_t epoch, uint64_t timeout_ns, uint32_t phase);
  // Current value of slot [row][src] of the own slab (acquire load); for words that carry data
  // rather than a call number, read after the flag that was raised behind them.
  uint64_t peek(int row, int src) const;
  // The device barrier's protocol on FLAG_BARRIER: signal everyone, then wait for everyone.
  StatusWord barrier(uint64_t epoch, uint64_t timeout_ns);

  StatusWord last_status() const { return status_; }
  void reset_status();

 private:
  std::string prefix_;
  int rank_, world_;
  uint64_t bytes_;
  uint8_t* base_[kMaxWorldSize];
  StatusWord status_;
};

}  // namespace b200
