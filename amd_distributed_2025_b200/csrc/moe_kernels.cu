// MoE expert-parallel dispatch / expert scale / combine kernels for sm_100a.
//
// What the reference does with six kernels, two packed staging buffers and four library
// all-to-alls per call (all2all/hipv8.py:60-226, 266-372) is done here by two kernels
// that talk to the peers' memory directly:
//
//   moe_dispatch_kernel  counts entries per expert, publishes the count row to every
//                        peer, derives each entry's final slot in the owner's
//                        expert buffer (reference order: source rank, then (t, k)),
//                        and stores the row + its 5-int metadata straight into the
//                        owner's memory over NVLink.  No pack buffer, no unpack pass.
//   moe_combine_kernel   for every output element pulls the k expert rows from the
//                        owners' memory and forms the weighted sum in fp32 registers in
//                        fixed k order, one rounding.  No atomics, no fp32 scratch.
//
// All cross-GPU waits are bounded (signal.cuh).
#include <cuda_runtime.h>
#include <stdint.h>

#include "moe.h"
#include "moe_common.cuh"
#include "signal.cuh"

namespace b200 {

namespace {

using namespace moe;

constexpr int kDispatchThreads = 256;
constexpr int kMetaDim = 5;

// One warp copies `bytes` from src to dst (dst may be peer memory).
__device__ __forceinline__ void warp_copy_row(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                              uint32_t bytes, int lane) {
  const bool vec16 = ((bytes & 15u) == 0) && ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) &&
                     ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
  if (vec16) {
    const int4* s = reinterpret_cast<const int4*>(src);
    int4* d = reinterpret_cast<int4*>(dst);
    const int nv = bytes >> 4;
    for (int v = lane; v < nv; v += 32 * 8) {
      int4 r[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = v + u * 32;
        if (idx < nv) r[u] = __ldg(s + idx);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = v + u * 32;
        if (idx < nv) d[idx] = r[u];
      }
    }
  } else if ((bytes & 3u) == 0 && ((reinterpret_cast<uintptr_t>(src) & 3u) == 0) &&
             ((reinterpret_cast<uintptr_t>(dst) & 3u) == 0)) {
    const uint32_t* s = reinterpret_cast<const uint32_t*>(src);
    uint32_t* d = reinterpret_cast<uint32_t*>(dst);
    const int nv = bytes >> 2;
    for (int v = lane; v < nv; v += 32) d[v] = __ldg(s + v);
  } else {
    const uint16_t* s = reinterpret_cast<const uint16_t*>(src);
    uint16_t* d = reinterpret_cast<uint16_t*>(dst);
    const int nv = bytes >> 1;
    for (int v = lane; v < nv; v += 32) d[v] = __ldg(s + v);
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------
// dispatch
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kDispatchThreads, 1) moe_dispatch_kernel(const MoeDispatchParams p) {
  extern __shared__ int32_t smem_run[];  // [num_experts] running per-expert count of this chunk
  __shared__ int is_last_shared;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int n = p.num_tokens * p.k;
  const int E = p.num_experts;
  const int G = gridDim.x;
  const uint64_t my_base = p.peer_base[p.rank];
  uint32_t bar_target = 0;

  // ---- phase A: per-chunk ordered ranks and histogram --------------------------------
  if ((int)blockIdx.x < p.count_blocks) {
    for (int e = tid; e < E; e += blockDim.x) smem_run[e] = 0;
    __syncthreads();
    if (warp == 0) {
      const int lo = blockIdx.x * p.chunk;
      const int hi = min(n, lo + p.chunk);
      for (int base = lo; base < hi; base += 32) {
        const int i = base + lane;
        int e = -1;
        if (i < hi) {
          e = p.indices[i];
          if (e < 0 || e >= E) {
            record_status(p.status, STATUS_BAD_INDEX, PHASE_NONE, -1, i, p.epoch, (uint64_t)(int64_t)e);
            p.local_rank[i] = -1;
            e = -1;
          }
        }
        const unsigned active = __ballot_sync(0xffffffffu, e >= 0);
        if (e >= 0) {
          const unsigned same = __match_any_sync(active, e);
          const int before = __popc(same & ((1u << lane) - 1u));
          const int cur = smem_run[e];
          __syncwarp(active);
          p.local_rank[i] = cur + before;
          if (before == 0) smem_run[e] = cur + __popc(same);
        }
        __syncwarp();
      }
    }
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) p.blk_hist[(size_t)blockIdx.x * E + e] = smem_run[e];
  }
  grid_barrier(&p.sync_counters[0], bar_target, p.timeout_ns, p.status);

  // ---- phase B: publish my per-expert totals to every rank, then collect theirs ------
  for (int dst = blockIdx.x; dst < p.world_size; dst += G) {
    int32_t* remote = peer_ptr<int32_t>(p.peer_base[dst], p.layout.off_counts) + (size_t)p.rank * E;
    for (int e = tid; e < E; e += blockDim.x) {
      int total = 0;
      for (int g = 0; g < p.count_blocks; ++g) total += p.blk_hist[(size_t)g * E + e];
      remote[e] = total;
    }
    __syncthreads();
    if (tid == 0) {
      __threadfence_system();
      st_release_sys(flag_ptr(p.peer_base[dst], FLAG_MOE_COUNTS, p.rank), p.epoch);
    }
  }
  if (tid < p.world_size) {
    wait_flag_ge(flag_ptr(my_base, FLAG_MOE_COUNTS, tid), p.epoch, p.timeout_ns, p.status, PHASE_MOE_COUNTS,
                 tid, (int)blockIdx.x);
  }
  __syncthreads();
  const int32_t* counts = peer_ptr<const int32_t>(my_base, p.layout.off_counts);  // [world][E]

  if (blockIdx.x == 0) {
    for (int el = tid; el < p.num_local_experts; el += blockDim.x) {
      int total = 0;
      for (int s = 0; s < p.world_size; ++s)
        total += __ldcg(counts + (size_t)s * E + p.rank * p.num_local_experts + el);
      p.expert_num_tokens[el] = min(total, p.max_recv);
    }
  }

  // ---- phase C: one warp per (token, k) entry: slot, row copy, metadata, route --------
  if (!status_timed_out(p.status)) {
    const int warps_total = G * (kDispatchThreads / 32);
    const uint8_t* xbytes = reinterpret_cast<const uint8_t*>(p.x);
    for (int i = blockIdx.x * (kDispatchThreads / 32) + warp; i < n; i += warps_total) {
      const int e = p.indices[i];
      if (e < 0 || e >= E) {
        if (lane == 0) p.route[i] = make_int2(-1, -1);
        continue;
      }
      const int chunk_id = i / p.chunk;
      int part = 0;
      for (int g = lane; g < chunk_id; g += 32) part += p.blk_hist[(size_t)g * E + e];
      if (lane < p.rank) part += __ldcg(counts + (size_t)lane * E + e);
      part = warp_sum(part);
      const int slot = part + p.local_rank[i];
      const int dst = e / p.num_local_experts;
      const int el = e - dst * p.num_local_experts;
      if (slot < 0 || slot >= p.max_recv) {
        if (lane == 0) {
          record_status(p.status, STATUS_BAD_INDEX, PHASE_NONE, dst, i, p.epoch, (uint64_t)(int64_t)slot);
          p.route[i] = make_int2(-1, -1);
        }
        continue;
      }
      const int64_t row = (int64_t)el * p.max_recv + slot;
      const int t = i / p.k;
      const int kk = i - t * p.k;
      const uint64_t dst_base = p.peer_base[dst];
      warp_copy_row(xbytes + (size_t)t * p.row_bytes,
                    peer_ptr<uint8_t>(dst_base, p.layout.off_expert_x) + (size_t)row * p.row_bytes, p.row_bytes,
                    lane);
      if (lane < kMetaDim) {
        int32_t mv = 0;
        if (lane == 0) mv = e;
        else if (lane == 1) mv = p.rank;
        else if (lane == 2) mv = t;
        else if (lane == 3) mv = kk;
        peer_ptr<int32_t>(dst_base, p.layout.off_expert_meta)[(size_t)row * kMetaDim + lane] = mv;
      }
      if (lane == 0) p.route[i] = make_int2(dst, (int)row);
    }
  }

  // ---- phase D: when every CTA has delivered, tell the owners; wait for theirs -------
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    const uint32_t done = atomicAdd(&p.sync_counters[1], 1u);
    is_last_shared = (done == (uint32_t)G - 1u);
  }
  __syncthreads();
  if (is_last_shared) {
    if (tid == 0) {
      __threadfence_system();  // one fence orders every CTA's row stores (observed through the counter) ...
      for (int dst = 0; dst < p.world_size; ++dst)  // ... before these relaxed flag stores
        st_relaxed_sys(flag_ptr(p.peer_base[dst], FLAG_MOE_DATA, p.rank), p.epoch);
      p.sync_counters[0] = 0;
      p.sync_counters[1] = 0;
    }
    if (tid < p.world_size) {
      wait_flag_ge(flag_ptr(my_base, FLAG_MOE_DATA, tid), p.epoch, p.timeout_ns, p.status, PHASE_MOE_DATA, tid,
                   (int)blockIdx.x);
    }
  }
}

// ---------------------------------------------------------------------------------------
// dispatch, small problems (decode): no in-GPU barrier
// ---------------------------------------------------------------------------------------
// With a few thousand (token, k) entries every CTA can afford to read ALL of them: it builds
// the full per-expert histogram in shared memory itself and finds an entry's position among
// equal experts by scanning the entries before it.  That removes the per-chunk counting
// pass, the grid-wide barrier and the histogram round trip through global memory from the
// latency chain; the cross-GPU protocol (count rows, flags, row stores, done flags) is the
// same as in moe_dispatch_kernel, and so are the resulting layouts.
__global__ void __launch_bounds__(kDispatchThreads) moe_dispatch_small_kernel(const MoeDispatchParams p) {
  extern __shared__ int32_t smem_small[];  // [n] expert ids (or -1), then [num_experts] histogram
  __shared__ int is_last_shared;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int n = p.num_tokens * p.k;
  const int E = p.num_experts;
  const int G = gridDim.x;
  const uint64_t my_base = p.peer_base[p.rank];
  int32_t* s_idx = smem_small;
  int32_t* s_hist = smem_small + ((n + 31) & ~31);

  for (int e = tid; e < E; e += blockDim.x) s_hist[e] = 0;
  for (int i = tid; i < n; i += blockDim.x) {
    int e = p.indices[i];
    if (e < 0 || e >= E) {
      if (blockIdx.x == 0) record_status(p.status, STATUS_BAD_INDEX, PHASE_NONE, -1, i, p.epoch, (uint64_t)(int64_t)e);
      e = -1;
    }
    s_idx[i] = e;
  }
  __syncthreads();
  for (int i = tid; i < n; i += blockDim.x) {
    const int e = s_idx[i];
    if (e >= 0) atomicAdd(&s_hist[e], 1);
  }
  __syncthreads();

  // publish this rank's per-expert totals to every rank, then collect theirs
  for (int dst = blockIdx.x; dst < p.world_size; dst += G) {
    int32_t* remote = peer_ptr<int32_t>(p.peer_base[dst], p.layout.off_counts) + (size_t)p.rank * E;
    for (int e = tid; e < E; e += blockDim.x) remote[e] = s_hist[e];
    __syncthreads();
    if (tid == 0) {
      __threadfence_system();
      st_release_sys(flag_ptr(p.peer_base[dst], FLAG_MOE_COUNTS, p.rank), p.epoch);
    }
  }
  if (tid < p.world_size) {
    wait_flag_ge(flag_ptr(my_base, FLAG_MOE_COUNTS, tid), p.epoch, p.timeout_ns, p.status, PHASE_MOE_COUNTS,
                 tid, (int)blockIdx.x);
  }
  __syncthreads();
  const int32_t* counts = peer_ptr<const int32_t>(my_base, p.layout.off_counts);  // [world][E]

  if (blockIdx.x == 0) {
    for (int el = tid; el < p.num_local_experts; el += blockDim.x) {
      int total = 0;
      for (int s = 0; s < p.world_size; ++s)
        total += __ldcg(counts + (size_t)s * E + p.rank * p.num_local_experts + el);
      p.expert_num_tokens[el] = min(total, p.max_recv);
    }
  }

  if (!status_timed_out(p.status)) {
    const int warps_total = G * (kDispatchThreads / 32);
    const uint8_t* xbytes = reinterpret_cast<const uint8_t*>(p.x);
    for (int i = blockIdx.x * (kDispatchThreads / 32) + warp; i < n; i += warps_total) {
      const int e = s_idx[i];
      if (e < 0) {
        if (lane == 0) p.route[i] = make_int2(-1, -1);
        continue;
      }
      // entries of this rank with the same expert that come before entry i, plus the rows
      // that lower ranks send to that expert: the slot in the reference's order
      int part = 0;
      for (int j = lane; j < i; j += 32) part += (s_idx[j] == e) ? 1 : 0;
      if (lane < p.rank) part += __ldcg(counts + (size_t)lane * E + e);
      const int slot = warp_sum(part);
      const int dst = e / p.num_local_experts;
      const int el = e - dst * p.num_local_experts;
      if (slot >= p.max_recv) {
        if (lane == 0) {
          record_status(p.status, STATUS_BAD_INDEX, PHASE_NONE, dst, i, p.epoch, (uint64_t)(int64_t)slot);
          p.route[i] = make_int2(-1, -1);
        }
        continue;
      }
      const int64_t row = (int64_t)el * p.max_recv + slot;
      const int t = i / p.k;
      const int kk = i - t * p.k;
      const uint64_t dst_base = p.peer_base[dst];
      warp_copy_row(xbytes + (size_t)t * p.row_bytes,
                    peer_ptr<uint8_t>(dst_base, p.layout.off_expert_x) + (size_t)row * p.row_bytes, p.row_bytes,
                    lane);
      if (lane < kMetaDim) {
        int32_t mv = 0;
        if (lane == 0) mv = e;
        else if (lane == 1) mv = p.rank;
        else if (lane == 2) mv = t;
        else if (lane == 3) mv = kk;
        peer_ptr<int32_t>(dst_base, p.layout.off_expert_meta)[(size_t)row * kMetaDim + lane] = mv;
      }
      if (lane == 0) p.route[i] = make_int2(dst, (int)row);
    }
  }

  // when every CTA has delivered, tell the owners; wait for theirs
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    const uint32_t done = atomicAdd(&p.sync_counters[1], 1u);
    is_last_shared = (done == (uint32_t)G - 1u);
  }
  __syncthreads();
  if (is_last_shared) {
    if (tid == 0) {
      __threadfence_system();
      for (int dst = 0; dst < p.world_size; ++dst)
        st_relaxed_sys(flag_ptr(p.peer_base[dst], FLAG_MOE_DATA, p.rank), p.epoch);
      p.sync_counters[1] = 0;
    }
    if (tid < p.world_size) {
      wait_flag_ge(flag_ptr(my_base, FLAG_MOE_DATA, tid), p.epoch, p.timeout_ns, p.status, PHASE_MOE_DATA, tid,
                   (int)blockIdx.x);
    }
  }
}

bool moe_dispatch_small_applies(int num_entries, int num_experts) {
  return num_entries <= 4096 && num_experts <= 4096;
}

cudaError_t launch_moe_dispatch_small(const MoeDispatchParams& p, int grid, cudaStream_t stream) {
  const int n = p.num_tokens * p.k;
  const size_t smem = ((size_t)((n + 31) & ~31) + (size_t)p.num_experts) * sizeof(int32_t);
  if (smem > 48 * 1024) return cudaErrorInvalidValue;
  moe_dispatch_small_kernel<<<grid, kDispatchThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

int moe_dispatch_max_blocks(int device) {
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  return sms > 0 ? sms : 1;
}

cudaError_t launch_moe_dispatch(const MoeDispatchParams& p, int grid, cudaStream_t stream) {
  const size_t smem = (size_t)p.num_experts * sizeof(int32_t);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(moe_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  MoeDispatchParams params = p;
  void* args[] = {&params};
  // Cooperative launch: the kernel's CTAs wait on one another, so they must be co-resident.
  return cudaLaunchCooperativeKernel((const void*)moe_dispatch_kernel, dim3(grid), dim3(kDispatchThreads), args,
                                     smem, stream);
}

// ---------------------------------------------------------------------------------------
// expert op of the task: a scale over the valid rows
// ---------------------------------------------------------------------------------------
template <typename TIn, typename TOut>
__global__ void moe_expert_scale_kernel(const TIn* __restrict__ x, TOut* __restrict__ y,
                                        const int32_t* __restrict__ num_tokens, int num_local_experts,
                                        int max_recv, int hidden, float scale) {
  extern __shared__ int32_t prefix[];  // [E_local + 1] exclusive prefix of the valid row counts
  // Block-wide exclusive scan, 32 experts per step of warp 0.
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int carry = 0;
    for (int base = 0; base < num_local_experts; base += 32) {
      const int e = base + lane;
      const int v = e < num_local_experts ? min(max(num_tokens[e], 0), max_recv) : 0;
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      if (e < num_local_experts) prefix[e] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) prefix[num_local_experts] = carry;
  }
  __syncthreads();
  const int total_rows = prefix[num_local_experts];
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < total_rows; r += gridDim.x * warps_per_block) {
    int lo = 0, hi = num_local_experts;  // largest e with prefix[e] <= r
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (prefix[mid] <= r) lo = mid; else hi = mid;
    }
    const size_t row = (size_t)lo * max_recv + (r - prefix[lo]);
    const TIn* src = x + row * hidden;
    TOut* dst = y + row * hidden;
    // The reference rounds the scale to out_dtype before multiplying in out_dtype
    // (tensor * python int); (1 + rank) is exactly representable, so one rounding of
    // the fp32 product gives the same value.
    constexpr int kVec = 16 / sizeof(TIn);
    if (sizeof(TIn) == sizeof(TOut) && hidden % kVec == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0 &&
        (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      const int nv = hidden / kVec;
      const int4* s4 = reinterpret_cast<const int4*>(src);
      int4* d4 = reinterpret_cast<int4*>(dst);
      for (int v = lane; v < nv; v += 32 * 4) {
        int4 r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v + u * 32 < nv) r[u] = __ldcg(s4 + v + u * 32);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (v + u * 32 < nv) {
            TIn* e = reinterpret_cast<TIn*>(&r[u]);
            int4 o;
            TOut* eo = reinterpret_cast<TOut*>(&o);
#pragma unroll
            for (int j = 0; j < kVec; ++j) eo[j] = from_f32<TOut>(to_f32(e[j]) * scale);
            d4[v + u * 32] = o;
          }
        }
      }
    } else {
      for (int h = lane; h < hidden; h += 32) dst[h] = from_f32<TOut>(to_f32(src[h]) * scale);
    }
  }
}

template <typename TIn, typename TOut>
static cudaError_t launch_scale_typed(const void* x, void* y, const int32_t* cnt, int el, int max_recv, int hidden,
                                      float scale, cudaStream_t stream) {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = sms * 4;
  moe_expert_scale_kernel<TIn, TOut><<<grid, 256, (el + 1) * sizeof(int32_t), stream>>>(
      reinterpret_cast<const TIn*>(x), reinterpret_cast<TOut*>(y), cnt, el, max_recv, hidden, scale);
  return cudaGetLastError();
}

cudaError_t launch_moe_expert_scale(const void* expert_x, void* expert_y, const int32_t* expert_num_tokens,
                                    int num_local_experts, int max_recv, int hidden, int in_dtype, int out_dtype,
                                    float scale, cudaStream_t stream) {
  if (in_dtype != out_dtype) return cudaErrorInvalidValue;
  switch (in_dtype) {
    case 0: return launch_scale_typed<__half, __half>(expert_x, expert_y, expert_num_tokens, num_local_experts, max_recv, hidden, scale, stream);
    case 1: return launch_scale_typed<__nv_bfloat16, __nv_bfloat16>(expert_x, expert_y, expert_num_tokens, num_local_experts, max_recv, hidden, scale, stream);
    case 2: return launch_scale_typed<float, float>(expert_x, expert_y, expert_num_tokens, num_local_experts, max_recv, hidden, scale, stream);
    default: return cudaErrorInvalidValue;
  }
}

// ---------------------------------------------------------------------------------------
// combine
// ---------------------------------------------------------------------------------------
namespace {

constexpr int kCombineThreads = 256;
constexpr int kCombineBatch = 8;  // peer loads kept in flight per thread

}  // namespace

template <typename T, bool VEC>
__global__ void __launch_bounds__(kCombineThreads) moe_combine_kernel(const MoeCombineParams p) {
  const int tid = threadIdx.x;
  const uint64_t my_base = p.peer_base[p.rank];

  // My expert outputs were produced by earlier kernels of this stream; tell every rank.
  if (blockIdx.x == 0 && tid < p.world_size) {
    __threadfence_system();
    st_release_sys(flag_ptr(p.peer_base[tid], FLAG_MOE_Y_READY, p.rank), p.epoch);
  }
  if (tid < p.world_size) {
    wait_flag_ge(flag_ptr(my_base, FLAG_MOE_Y_READY, tid), p.epoch, p.timeout_ns, p.status, PHASE_MOE_Y_READY,
                 tid, (int)blockIdx.x);
  }
  __syncthreads();
  if (status_timed_out(p.status)) return;

  const size_t row_bytes = (size_t)p.hidden * sizeof(T);
  if (VEC) {
    constexpr int N = Vec16<T>::N;
    const int nv = p.hidden / N;
    const long long total = (long long)p.num_tokens * nv;
    for (long long idx = (long long)blockIdx.x * blockDim.x + tid; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
      const int t = (int)(idx / nv);
      const int v = (int)(idx - (long long)t * nv);
      float acc[N];
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] = 0.f;
      for (int k0 = 0; k0 < p.k; k0 += kCombineBatch) {
        int4 vals[kCombineBatch];
        float w[kCombineBatch];
#pragma unroll
        for (int u = 0; u < kCombineBatch; ++u) {
          const int kk = k0 + u;
          w[u] = 0.f;
          vals[u] = make_int4(0, 0, 0, 0);
          if (kk < p.k) {
            const int2 r = __ldg(p.route + (size_t)t * p.k + kk);
            if (r.y >= 0) {
              const int4* src =
                  reinterpret_cast<const int4*>(p.peer_base[r.x] + p.off_expert_y + (uint64_t)r.y * row_bytes) + v;
              vals[u] = __ldcg(src);
              w[u] = __ldg(p.weights + (size_t)t * p.k + kk);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kCombineBatch; ++u) fma_vec<T>(acc, vals[u], w[u]);
      }
      reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(p.out) + (size_t)t * row_bytes)[v] = pack_vec<T>(acc);
    }
  } else {
    const long long total = (long long)p.num_tokens * p.hidden;
    for (long long idx = (long long)blockIdx.x * blockDim.x + tid; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
      const int t = (int)(idx / p.hidden);
      const int h = (int)(idx - (long long)t * p.hidden);
      float acc = 0.f;
      for (int kk = 0; kk < p.k; ++kk) {
        const int2 r = __ldg(p.route + (size_t)t * p.k + kk);
        if (r.y < 0) continue;
        const T* src = reinterpret_cast<const T*>(p.peer_base[r.x] + p.off_expert_y + (uint64_t)r.y * row_bytes) + h;
        acc = fmaf(to_f32(__ldcg(src)), __ldg(p.weights + (size_t)t * p.k + kk), acc);
      }
      reinterpret_cast<T*>(p.out)[(size_t)t * p.hidden + h] = from_f32<T>(acc);
    }
  }
}

template <typename T>
static cudaError_t launch_combine_typed(const MoeCombineParams& p, cudaStream_t stream) {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const bool vec = ((size_t)p.hidden * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(p.out) % 16 == 0) &&
                   (p.off_expert_y % 16 == 0);
  const long long items = vec ? (long long)p.num_tokens * (p.hidden / Vec16<T>::N) : (long long)p.num_tokens * p.hidden;
  long long want = (items + kCombineThreads - 1) / kCombineThreads;
  // CTA 0 raises this rank's flag while every CTA polls the peers' flags: keep the whole
  // grid resident so CTA 0 can never be queued behind spinning CTAs.
  int per_sm = 1;
  if (vec) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_combine_kernel<T, true>, kCombineThreads, 0);
  else cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_combine_kernel<T, false>, kCombineThreads, 0);
  if (per_sm < 1) per_sm = 1;
  const long long cap = (long long)sms * per_sm;
  int grid = (int)(want < 1 ? 1 : (want > cap ? cap : want));
  if (vec) moe_combine_kernel<T, true><<<grid, kCombineThreads, 0, stream>>>(p);
  else moe_combine_kernel<T, false><<<grid, kCombineThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_moe_combine(const MoeCombineParams& p, cudaStream_t stream) {
  switch (p.dtype) {
    case 0: return launch_combine_typed<__half>(p, stream);
    case 1: return launch_combine_typed<__nv_bfloat16>(p, stream);
    case 2: return launch_combine_typed<float>(p, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace b200
