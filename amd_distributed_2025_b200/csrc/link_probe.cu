// Peer-store bandwidth probe: how fast can THIS GPU push bytes into a peer's slab, and with
// which mechanism?  It supplies the link denominator of the roofline of the fused kernels.
// The reference has nothing like it: its traffic goes through library collectives
// (all2all/hipv8.py:281-359, gemm-rs/reference.py:59).
//
//   mode 0  16-byte stores from registers (eight loads in flight per lane, then eight stores)
//   mode 1  bulk copies through shared memory: cp.async.bulk global -> shared, then
//           cp.async.bulk shared -> peer global, two stages per warp, `chunk` bytes per copy
//
// The kernel ends with a system-scope fence per CTA, so its duration (CUDA events on the
// sender) includes the time until the peer has acknowledged every byte.
#include <cuda_runtime.h>
#include <stdint.h>

#include "signal.cuh"
#include "sm100_ptx.cuh"
#include "symm_heap.h"

namespace b200 {

namespace {

constexpr int kProbeThreads = 256;
constexpr int kProbeWarps = kProbeThreads / 32;
constexpr int kProbeMaxChunk = 8192;

__global__ void __launch_bounds__(kProbeThreads) link_probe_kernel(const uint8_t* __restrict__ src, uint8_t* dst,
                                                                   uint64_t bytes, int mode, int chunk,
                                                                   uint64_t timeout_ns, StatusBlock* status) {
  extern __shared__ __align__(128) uint8_t probe_smem[];
  __shared__ uint64_t bars[kProbeWarps];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const uint64_t gw = (uint64_t)blockIdx.x * kProbeWarps + warp;
  const uint64_t W = (uint64_t)gridDim.x * kProbeWarps;
  if (mode == 1) {
    if (threadIdx.x == 0) {
      for (int w = 0; w < kProbeWarps; ++w) ptx::mbar_init(ptx::smem_u32(&bars[w]), 1);
      ptx::fence_mbar_init();
      ptx::fence_proxy_async_smem();
    }
    __syncthreads();
    if (lane == 0) {
      const uint32_t stage = ptx::smem_u32(probe_smem + (size_t)warp * 2 * kProbeMaxChunk);
      const uint32_t bar = ptx::smem_u32(&bars[warp]);
      uint32_t parity = 0, n = 0;
      const uint64_t chunks = bytes / (uint64_t)chunk;
      for (uint64_t c = gw; c < chunks; c += W, ++n) {
        const uint32_t st = stage + (n & 1u) * kProbeMaxChunk;
        ptx::bulk_wait_group_read<1>();
        ptx::mbar_arrive_expect_tx(bar, (uint32_t)chunk);
        ptx::bulk_load(st, src + c * chunk, (uint32_t)chunk, bar);
        const uint64_t t0 = global_timer_ns();
        bool ok = true;
        while (!ptx::mbar_try_wait(bar, parity)) {
          if (global_timer_ns() - t0 > timeout_ns) {
            record_status(status, STATUS_TIMEOUT, PHASE_TEST, -1, (int)blockIdx.x, 0, parity);
            ok = false;
            break;
          }
        }
        if (!ok) break;
        parity ^= 1u;
        ptx::fence_proxy_async_smem();
        ptx::bulk_store(dst + c * chunk, st, (uint32_t)chunk);
        ptx::bulk_commit_group();
      }
      ptx::bulk_wait_group<0>();
      asm volatile("fence.proxy.async.global;" ::: "memory");
    }
  } else {
    const int4* s4 = reinterpret_cast<const int4*>(src);
    int4* d4 = reinterpret_cast<int4*>(dst);
    const uint64_t nv = bytes >> 4;
    // a warp moves runs of 8 x 512 bytes
    for (uint64_t base = gw * 256; base < nv; base += W * 256) {
      int4 r[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint64_t idx = base + lane + 32 * u;
        if (idx < nv) r[u] = __ldcg(s4 + idx);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint64_t idx = base + lane + 32 * u;
        if (idx < nv) d4[idx] = r[u];
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) __threadfence_system();
}

}  // namespace

cudaError_t launch_link_probe(const SymmHeap& heap, int peer, uint64_t src_offset, uint64_t dst_offset, uint64_t bytes,
                              int mode, int chunk, int grid, uint64_t timeout_ns, cudaStream_t stream) {
  if (peer < 0 || peer >= heap.world_size() || (mode != 0 && mode != 1)) return cudaErrorInvalidValue;
  if (chunk < 16 || chunk > kProbeMaxChunk || (chunk & 15) || (bytes & 15) || (src_offset & 15) || (dst_offset & 15))
    return cudaErrorInvalidValue;
  if (src_offset + bytes > heap.bytes() || dst_offset + bytes > heap.bytes() || src_offset < kHeapHeaderBytes ||
      dst_offset < kHeapHeaderBytes)
    return cudaErrorInvalidValue;
  const size_t smem = mode == 1 ? (size_t)kProbeWarps * 2 * kProbeMaxChunk : 0;
  static bool opted_in = false;
  if (mode == 1 && !opted_in) {
    cudaError_t e = cudaFuncSetAttribute(link_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    opted_in = true;
  }
  const uint8_t* src = static_cast<const uint8_t*>(heap.local_base()) + src_offset;
  uint8_t* dst = reinterpret_cast<uint8_t*>(heap.peer_base(peer)) + dst_offset;
  link_probe_kernel<<<grid, kProbeThreads, smem, stream>>>(src, dst, bytes, mode, chunk, timeout_ns, heap.status_device());
  return cudaGetLastError();
}

}  // namespace b200
