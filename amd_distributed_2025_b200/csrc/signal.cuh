// Device-side signalling over NVLink peer memory: release/acquire flag accesses at
// system scope, bounded waits, and an in-GPU grid barrier.
//
// Protocol rules used by every kernel in this library:
//  * payload stores (plain st.global to a peer mapping) are followed by
//    __threadfence_system() and then a st.release.sys / red.release.sys of the flag;
//  * the consumer polls the flag with ld.acquire.sys and only then touches the payload,
//    with L1-bypassing loads (ld.global.cg) when the payload is in peer memory;
//  * flags carry the call number (epoch), which only grows, so nothing is ever reset;
//  * a wait that exceeds its time limit records a StatusWord and returns false.
//
// The reference synchronises only through host-blocking library collectives
// (all2all/hipv8.py:278-305); it has no device-side signalling.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "status.h"

namespace b200 {

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Relaxed forms: ordering comes from an explicit fence issued once before a batch of them
// (every .release form pays for its own fence).
__device__ __forceinline__ void red_relaxed_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_relaxed_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t ld_relaxed_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// First error wins; later errors are dropped so the original cause survives.
__device__ __forceinline__ void record_status(StatusBlock* st, uint32_t code, uint32_t phase, int peer,
                                              int detail, uint64_t epoch, uint64_t seen) {
  if (st == nullptr) return;
  if (atomicCAS(&st->word.code, (uint32_t)STATUS_OK, code) == STATUS_OK) {
    st->word.phase = phase;
    st->word.peer = peer;
    st->word.detail = detail;
    st->word.epoch = epoch;
    st->word.seen = seen;
    StatusWord* h = st->host_mirror;
    if (h != nullptr) {
      volatile StatusWord* hv = h;
      hv->phase = phase;
      hv->peer = peer;
      hv->detail = detail;
      hv->epoch = epoch;
      hv->seen = seen;
      __threadfence_system();
      hv->code = code;
    }
    __threadfence_system();
  }
}

__device__ __forceinline__ bool status_failed(const StatusBlock* st) {
  return st != nullptr && *reinterpret_cast<const volatile uint32_t*>(&st->word.code) != STATUS_OK;
}

__device__ __forceinline__ bool status_timed_out(const StatusBlock* st) {
  return st != nullptr && *reinterpret_cast<const volatile uint32_t*>(&st->word.code) == STATUS_TIMEOUT;
}

// Spin until *flag >= want.  Gives up after limit_ns (or as soon as another thread has
// recorded a failure), records STATUS_TIMEOUT and returns false.
__device__ __forceinline__ bool wait_flag_ge(const uint64_t* flag, uint64_t want, uint64_t limit_ns,
                                             StatusBlock* st, uint32_t phase, int peer, int detail) {
  uint64_t seen = ld_acquire_sys(flag);
  if (seen >= want) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    seen = ld_acquire_sys(flag);
    if (seen >= want) return true;
    if ((++spins & 63u) == 0) {
      if (global_timer_ns() - t0 > limit_ns || status_timed_out(st)) break;
    }
    __nanosleep(20);
  }
  record_status(st, STATUS_TIMEOUT, phase, peer, detail, want, seen);
  return false;
}

__device__ __forceinline__ bool wait_u32_ge(const uint32_t* ctr, uint32_t want, uint64_t limit_ns,
                                            StatusBlock* st, uint32_t phase, int peer, int detail,
                                            bool sys_scope) {
  uint32_t seen = sys_scope ? ld_acquire_sys_u32(ctr) : ld_acquire_gpu_u32(ctr);
  if (seen >= want) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    seen = sys_scope ? ld_acquire_sys_u32(ctr) : ld_acquire_gpu_u32(ctr);
    if (seen >= want) return true;
    if ((++spins & 63u) == 0) {
      if (global_timer_ns() - t0 > limit_ns || status_timed_out(st)) break;
    }
    __nanosleep(20);
  }
  record_status(st, STATUS_TIMEOUT, phase, peer, detail, want, seen);
  return false;
}

// Barrier over all CTAs of a co-resident (cooperatively launched) grid.  `counter` only
// grows during a launch; `target` is the caller's running expectation and is advanced
// by gridDim.x per barrier.  The last CTA of the kernel zeroes the counter again.
__device__ __forceinline__ bool grid_barrier(uint32_t* counter, uint32_t& target, uint64_t limit_ns,
                                             StatusBlock* st) {
  __shared__ int ok_shared;
  __syncthreads();
  target += gridDim.x;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
    ok_shared = wait_u32_ge(counter, target, limit_ns, st, PHASE_GRID_BARRIER, -1, (int)blockIdx.x, false);
    __threadfence();
  }
  __syncthreads();
  return ok_shared != 0;
}

template <typename T>
__device__ __forceinline__ T* peer_ptr(uint64_t base, uint64_t byte_offset) {
  return reinterpret_cast<T*>(base + byte_offset);
}

__host__ __device__ __forceinline__ uint64_t* flag_ptr(uint64_t heap_base, int row, int src) {
  return reinterpret_cast<uint64_t*>(heap_base) + (row * kMaxWorldSize + src);
}

}  // namespace b200
