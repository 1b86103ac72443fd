// Symmetric heap implementation and the two small kernels that exercise the flags.
#include "symm_heap.h"

#include <cstring>
#include <stdexcept>

#include "signal.cuh"

namespace b200 {

namespace {

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
  }
}

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    else prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

constexpr uint64_t kSlabAlign = 2ull << 20;

}  // namespace

SymmHeap::SymmHeap(int rank, int world_size, uint64_t bytes, int device)
    : rank_(rank), world_(world_size), device_(device), bytes_(0), peers_open_(false), status_dev_(nullptr),
      status_host_(nullptr), sync_counters_(nullptr) {
  if (world_size < 1 || world_size > kMaxWorldSize) throw std::runtime_error("world_size out of range");
  if (rank < 0 || rank >= world_size) throw std::runtime_error("rank out of range");
  if (bytes < kHeapHeaderBytes) bytes = kHeapHeaderBytes;
  bytes_ = (bytes + kSlabAlign - 1) / kSlabAlign * kSlabAlign;
  for (int r = 0; r < kMaxWorldSize; ++r) base_[r] = nullptr;
  DeviceGuard guard(device_);
  check(cudaMalloc(&base_[rank_], bytes_), "cudaMalloc(symmetric slab)");
  check(cudaMemset(base_[rank_], 0, bytes_), "cudaMemset(symmetric slab)");
  check(cudaMalloc(reinterpret_cast<void**>(&status_dev_), sizeof(StatusBlock)), "cudaMalloc(status)");
  check(cudaHostAlloc(reinterpret_cast<void**>(&status_host_), sizeof(StatusWord), cudaHostAllocMapped),
        "cudaHostAlloc(status mirror)");
  std::memset(status_host_, 0, sizeof(StatusWord));
  StatusBlock blk;
  std::memset(&blk, 0, sizeof(blk));
  StatusWord* mirror_dev = nullptr;
  check(cudaHostGetDevicePointer(reinterpret_cast<void**>(&mirror_dev), status_host_, 0), "cudaHostGetDevicePointer");
  blk.host_mirror = mirror_dev;
  check(cudaMemcpy(status_dev_, &blk, sizeof(blk), cudaMemcpyHostToDevice), "cudaMemcpy(status)");
  check(cudaMalloc(reinterpret_cast<void**>(&sync_counters_), 64 * sizeof(uint32_t)), "cudaMalloc(sync counters)");
  check(cudaMemset(sync_counters_, 0, 64 * sizeof(uint32_t)), "cudaMemset(sync counters)");
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  if (world_ == 1) peers_open_ = true;
}

SymmHeap::~SymmHeap() {
  try {
    close();
  } catch (...) {
  }
}

std::string SymmHeap::ipc_handle() const {
  DeviceGuard guard(device_);
  cudaIpcMemHandle_t h;
  check(cudaIpcGetMemHandle(&h, base_[rank_]), "cudaIpcGetMemHandle");
  return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void SymmHeap::open_peers(const std::vector<std::string>& handles) {
  if ((int)handles.size() != world_) throw std::runtime_error("open_peers: need one handle per rank");
  if (peers_open_ && world_ > 1) throw std::runtime_error("open_peers: peers already mapped");
  DeviceGuard guard(device_);
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    if (handles[r].size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("open_peers: bad handle size");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handles[r].data(), sizeof(h));
    check(cudaIpcOpenMemHandle(&base_[r], h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  }
  peers_open_ = true;
}

void SymmHeap::close_peers() {
  if (base_[rank_] == nullptr) return;
  DeviceGuard guard(device_);
  cudaDeviceSynchronize();
  for (int r = 0; r < world_; ++r) {
    if (r == rank_ || base_[r] == nullptr) continue;
    cudaIpcCloseMemHandle(base_[r]);
    base_[r] = nullptr;
  }
  if (world_ > 1) peers_open_ = false;
}

void SymmHeap::close() {
  if (base_[rank_] == nullptr) return;
  close_peers();
  DeviceGuard guard(device_);
  cudaFree(base_[rank_]);
  base_[rank_] = nullptr;
  if (status_dev_) cudaFree(status_dev_);
  if (status_host_) cudaFreeHost(status_host_);
  if (sync_counters_) cudaFree(sync_counters_);
  status_dev_ = nullptr;
  status_host_ = nullptr;
  sync_counters_ = nullptr;
  peers_open_ = false;
}

StatusWord SymmHeap::status_host() const {
  StatusWord w;
  std::memset(&w, 0, sizeof(w));
  if (status_host_ == nullptr) return w;
  const volatile StatusWord* v = status_host_;
  w.code = v->code;
  w.phase = v->phase;
  w.peer = v->peer;
  w.detail = v->detail;
  w.epoch = v->epoch;
  w.seen = v->seen;
  return w;
}

StatusWord SymmHeap::status_sync() const {
  DeviceGuard guard(device_);
  StatusBlock blk;
  check(cudaMemcpy(&blk, status_dev_, sizeof(blk), cudaMemcpyDeviceToHost), "cudaMemcpy(status)");
  return blk.word;
}

void SymmHeap::reset_status() {
  DeviceGuard guard(device_);
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  check(cudaMemset(&status_dev_->word, 0, sizeof(StatusWord)), "cudaMemset(status)");
  std::memset(status_host_, 0, sizeof(StatusWord));
  check(cudaMemset(sync_counters_, 0, 64 * sizeof(uint32_t)), "cudaMemset(sync counters)");
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
}

// ---------------------------------------------------------------------------------------

struct BarrierParams {
  uint64_t peer_base[kMaxWorldSize];
  int rank, world_size;
  uint64_t epoch, timeout_ns;
  StatusBlock* status;
};

__global__ void symm_barrier_kernel(const BarrierParams p) {
  const int tid = threadIdx.x;
  if (tid < p.world_size) {
    __threadfence_system();
    st_release_sys(flag_ptr(p.peer_base[tid], FLAG_BARRIER, p.rank), p.epoch);
    wait_flag_ge(flag_ptr(p.peer_base[p.rank], FLAG_BARRIER, tid), p.epoch, p.timeout_ns, p.status, PHASE_BARRIER,
                 tid, 0);
  }
}

cudaError_t launch_symm_barrier(const SymmHeap& heap, uint64_t epoch, uint64_t timeout_ns, cudaStream_t stream) {
  BarrierParams p;
  for (int r = 0; r < kMaxWorldSize; ++r) p.peer_base[r] = r < heap.world_size() ? heap.peer_base(r) : 0;
  p.rank = heap.rank();
  p.world_size = heap.world_size();
  p.epoch = epoch;
  p.timeout_ns = timeout_ns;
  p.status = heap.status_device();
  symm_barrier_kernel<<<1, 32, 0, stream>>>(p);
  return cudaGetLastError();
}

__global__ void wait_selftest_kernel(const uint64_t* flag, uint64_t want, uint64_t timeout_ns, StatusBlock* status,
                                     int slot) {
  if (threadIdx.x == 0) wait_flag_ge(flag, want, timeout_ns, status, PHASE_TEST, slot, 0);
}

cudaError_t launch_wait_selftest(const SymmHeap& heap, int slot, uint64_t want, uint64_t timeout_ns,
                                 cudaStream_t stream) {
  if (slot < 0 || slot >= kMaxWorldSize) return cudaErrorInvalidValue;
  wait_selftest_kernel<<<1, 32, 0, stream>>>(flag_ptr(heap.peer_base(heap.rank()), FLAG_TEST, slot), want,
                                             timeout_ns, heap.status_device(), slot);
  return cudaGetLastError();
}

}  // namespace b200
