// NVLink multicast (NVLS) region: one physical allocation per rank, bound into ONE multicast
// object that NVSwitch resolves to all of them.
//
// A load with `multimem.ld_reduce` from the multicast address returns the SUM of the values
// that the ranks hold at that offset, added inside the switch: the owner of an output row
// receives one reduced stream instead of world_size partial rows.  The reference reaches its
// peers only through library collectives (gemm-rs/reference.py:59); this is the in-switch
// counterpart of that reduce-scatter, used by the fused GEMM when B200_RS_MODE=nvls.
//
// Set-up is collective and driven from Python (parallel/symm_mem.py: McastWorkspace):
//   rank 0   create_and_export()            -> file descriptor of the multicast object
//   others   import_from(pid of rank 0, fd) (the descriptor is duplicated with pidfd_getfd)
//   all      add_device(); <host barrier>; bind_and_map(); <host barrier>
// and tear-down likewise: <all idle, host barrier>; close().  A rank must never exit while
// its memory is still bound and peers may still read through the multicast address.
//
// Host-only header: no torch types.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace b200 {

class McastRegion {
 public:
  // Whether the device and driver expose multicast objects at all (no allocation is made).
  static bool supported(int device, std::string* why);

  McastRegion(int rank, int world_size, uint64_t bytes, int device);
  ~McastRegion();
  McastRegion(const McastRegion&) = delete;
  McastRegion& operator=(const McastRegion&) = delete;

  int create_and_export();                 // rank 0 only
  void import_from(int64_t pid, int fd);   // every other rank
  void add_device();
  void bind_and_map();
  void close();

  int rank() const { return rank_; }
  int world_size() const { return world_; }
  int device() const { return device_; }
  uint64_t bytes() const { return bytes_; }
  void* local_ptr() const { return local_va_; }   // this rank's own memory (ordinary loads and stores)
  void* mc_ptr() const { return mc_va_; }         // the multicast address (multimem.* instructions only)
  bool mapped() const { return mc_va_ != nullptr; }

 private:
  int rank_, world_, device_;
  uint64_t bytes_;
  unsigned long long mc_handle_, mem_handle_;  // CUmemGenericAllocationHandle
  bool have_mc_, have_mem_, bound_, device_added_;
  void* local_va_;
  void* mc_va_;
  int export_fd_;
};

// Self-test: out[i] = sum over ranks of the bf16 pairs at element pair i of the region, formed by
// multimem.ld_reduce (fp32 accumulation), for `n_vec` 16-byte vectors starting at byte `offset`.
cudaError_t launch_mcast_selftest(const McastRegion& region, uint64_t offset, void* out, uint64_t n_vec,
                                  cudaStream_t stream);

}  // namespace b200
