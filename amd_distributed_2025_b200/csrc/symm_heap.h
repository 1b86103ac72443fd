// Symmetric heap: one device allocation per rank, mapped into every peer process.
//
// The reference exchanges data only through library collectives on ordinary tensors
// (all2all/hipv8.py:281,305,332,359; gemm-rs/reference.py:59).  Here every rank owns a
// slab of device memory whose layout is identical on all ranks; peers map it through
// CUDA IPC handles exchanged once over the host process group, and kernels then
// address "offset X on rank r" as peer_base[r] + X with plain loads and stores that
// travel over NVLink.  The first kHeapHeaderBytes hold the signalling flags.
//
// Host-only: no torch types.  The Python side (parallel/symm_mem.py) drives the
// collective parts (handle exchange) and sub-allocates the slab.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "status.h"

namespace b200 {

class SymmHeap {
 public:
  // Allocates and zeroes `bytes` (rounded up to 2 MiB) on `device`.
  SymmHeap(int rank, int world_size, uint64_t bytes, int device);
  ~SymmHeap();
  SymmHeap(const SymmHeap&) = delete;
  SymmHeap& operator=(const SymmHeap&) = delete;

  // 64-byte CUDA IPC handle of the local slab.
  std::string ipc_handle() const;
  // Maps the peers' slabs.  handles[r] is rank r's ipc_handle(); the own entry is ignored.
  void open_peers(const std::vector<std::string>& handles);
  // Unmaps peers and frees the slab.  All ranks must have stopped using it.  Ranks that
  // tear down together should call close_peers() first, meet on the host, then close():
  // a slab must not be freed while a peer still maps it.
  void close();
  void close_peers();

  int rank() const { return rank_; }
  int world_size() const { return world_; }
  int device() const { return device_; }
  uint64_t bytes() const { return bytes_; }
  void* local_base() const { return base_[rank_]; }
  uint64_t peer_base(int r) const { return reinterpret_cast<uint64_t>(base_[r]); }
  const void* const* bases() const { return base_; }
  bool peers_open() const { return peers_open_; }

  StatusBlock* status_device() const { return status_dev_; }
  // Snapshot of the host mirror (no stream synchronisation).
  StatusWord status_host() const;
  // Reads the device copy (synchronises the device).
  StatusWord status_sync() const;
  // Clears both copies and the kernels' grid-sync counters; call only when idle.
  void reset_status();

  // Local scratch words used by kernels' intra-GPU barriers; zero between launches.
  uint32_t* sync_counters() const { return sync_counters_; }

 private:
  int rank_, world_, device_;
  uint64_t bytes_;
  void* base_[kMaxWorldSize];
  bool peers_open_;
  StatusBlock* status_dev_;
  StatusWord* status_host_;  // mapped pinned
  uint32_t* sync_counters_;
};

// A cross-GPU barrier on FLAG_BARRIER: every rank stores `epoch` into its slot on every
// peer and waits until all slots of its own row reach `epoch`.
cudaError_t launch_symm_barrier(const SymmHeap& heap, uint64_t epoch, uint64_t timeout_ns, cudaStream_t stream);

// Self-test of the bounded wait: waits on FLAG_TEST slot `slot` of the local heap for a
// value that nothing writes; must come back with STATUS_TIMEOUT after ~timeout_ns.
cudaError_t launch_wait_selftest(const SymmHeap& heap, int slot, uint64_t want, uint64_t timeout_ns,
                                 cudaStream_t stream);

// Peer-store bandwidth probe (link_probe.cu): copies `bytes` from this rank's slab at
// src_offset into rank `peer`'s slab at dst_offset with 16-byte stores (mode 0) or bulk
// copies of `chunk` bytes through shared memory (mode 1), and ends with a system-scope fence.
cudaError_t launch_link_probe(const SymmHeap& heap, int peer, uint64_t src_offset, uint64_t dst_offset, uint64_t bytes,
                              int mode, int chunk, int grid, uint64_t timeout_ns, cudaStream_t stream);

}  // namespace b200
