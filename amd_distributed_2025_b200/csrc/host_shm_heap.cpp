#include "host_shm_heap.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <stdexcept>
#include <thread>

namespace b200 {

namespace {

uint64_t now_ns() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
             std::chrono::steady_clock::now().time_since_epoch())
      .count();
}

std::string seg_name(const std::string& prefix, int rank) { return "/" + prefix + "_" + std::to_string(rank); }

std::atomic<uint64_t>* flag_slot(uint8_t* base, int row, int src) {
  static_assert(sizeof(std::atomic<uint64_t>) == sizeof(uint64_t), "flag slots are plain 64-bit words");
  return reinterpret_cast<std::atomic<uint64_t>*>(base) + (row * kMaxWorldSize + src);
}

}  // namespace

HostShmHeap::HostShmHeap(const std::string& prefix, int rank, int world_size, uint64_t bytes)
    : prefix_(prefix), rank_(rank), world_(world_size), bytes_(bytes < kHeapHeaderBytes ? kHeapHeaderBytes : bytes) {
  if (world_size < 1 || world_size > kMaxWorldSize || rank < 0 || rank >= world_size)
    throw std::runtime_error("HostShmHeap: rank / world_size out of range");
  for (int r = 0; r < kMaxWorldSize; ++r) base_[r] = nullptr;
  std::memset(&status_, 0, sizeof(status_));
  const std::string name = seg_name(prefix_, rank_);
  shm_unlink(name.c_str());
  int fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0) throw std::runtime_error("HostShmHeap: shm_open(create) failed for " + name);
  if (ftruncate(fd, (off_t)bytes_) != 0) {
    ::close(fd);
    throw std::runtime_error("HostShmHeap: ftruncate failed");
  }
  void* p = mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  ::close(fd);
  if (p == MAP_FAILED) throw std::runtime_error("HostShmHeap: mmap failed");
  base_[rank_] = static_cast<uint8_t*>(p);
  // The segment was created exclusively just above, so every page is zero-filled by the kernel.
  // It is NOT cleared here: a peer may map it as soon as it has its full size and could already
  // have stored a flag that a late memset would wipe out.
}

HostShmHeap::~HostShmHeap() { close(); }

bool HostShmHeap::open_peers(uint64_t timeout_ns) {
  const uint64_t t0 = now_ns();
  for (int r = 0; r < world_; ++r) {
    if (r == rank_ || base_[r] != nullptr) continue;
    const std::string name = seg_name(prefix_, r);
    while (true) {
      int fd = shm_open(name.c_str(), O_RDWR, 0600);
      if (fd >= 0) {
        struct stat st;
        if (fstat(fd, &st) == 0 && (uint64_t)st.st_size >= bytes_) {
          void* p = mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
          ::close(fd);
          if (p == MAP_FAILED) return false;
          base_[r] = static_cast<uint8_t*>(p);
          break;
        }
        ::close(fd);  // created but not sized yet
      }
      if (now_ns() - t0 > timeout_ns) return false;
      std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
  }
  return true;
}

void HostShmHeap::close() {
  for (int r = 0; r < world_; ++r) {
    if (base_[r] != nullptr) {
      munmap(base_[r], bytes_);
      base_[r] = nullptr;
    }
  }
  if (!prefix_.empty()) shm_unlink(seg_name(prefix_, rank_).c_str());
  prefix_.clear();
}

void HostShmHeap::unlink() {
  if (!prefix_.empty()) shm_unlink(seg_name(prefix_, rank_).c_str());
}

void HostShmHeap::signal(int row, int dst, uint64_t epoch) {
  if (row < 0 || row >= FLAG_ROWS || dst < 0 || dst >= world_ || base_[dst] == nullptr)
    throw std::runtime_error("HostShmHeap::signal: bad row / destination");
  flag_slot(base_[dst], row, rank_)->store(epoch, std::memory_order_release);
}

StatusWord HostShmHeap::wait(int row, int src, uint64_t epoch, uint64_t timeout_ns, uint32_t phase) {
  StatusWord w;
  std::memset(&w, 0, sizeof(w));
  if (row < 0 || row >= FLAG_ROWS || src < 0 || src >= world_) {
    w.code = STATUS_BAD_ARGUMENT;
    return w;
  }
  std::atomic<uint64_t>* slot = flag_slot(base_[rank_], row, src);
  const uint64_t t0 = now_ns();
  uint64_t seen = slot->load(std::memory_order_acquire);
  uint32_t spins = 0;
  while (seen < epoch) {
    if ((++spins & 63u) == 0) {
      if (now_ns() - t0 > timeout_ns) {
        w.code = STATUS_TIMEOUT;
        w.phase = phase;
        w.peer = src;
        w.detail = row;
        w.epoch = epoch;
        w.seen = seen;
        if (status_.code == STATUS_OK) status_ = w;  // first error wins
        return w;
      }
      std::this_thread::yield();
    }
    seen = slot->load(std::memory_order_acquire);
  }
  return w;
}

uint64_t HostShmHeap::peek(int row, int src) const {
  if (row < 0 || row >= FLAG_ROWS || src < 0 || src >= world_) throw std::runtime_error("HostShmHeap::peek: bad row / source");
  return flag_slot(base_[rank_], row, src)->load(std::memory_order_acquire);
}

StatusWord HostShmHeap::barrier(uint64_t epoch, uint64_t timeout_ns) {
  for (int r = 0; r < world_; ++r) signal(FLAG_BARRIER, r, epoch);
  StatusWord ok;
  std::memset(&ok, 0, sizeof(ok));
  for (int r = 0; r < world_; ++r) {
    StatusWord w = wait(FLAG_BARRIER, r, epoch, timeout_ns, PHASE_BARRIER);
    if (w.code != STATUS_OK) return w;
  }
  return ok;
}

void HostShmHeap::reset_status() { std::memset(&status_, 0, sizeof(status_)); }

}  // namespace b200
