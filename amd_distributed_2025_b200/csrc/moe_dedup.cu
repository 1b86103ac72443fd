// MoE expert-parallel dispatch and combine with one row per (token, destination rank).
//
// The reference (all2all/reference.py:79-86,107-112,226-232; all2all/hipv8.py:80-97,144-226)
// moves one row per (token, k) entry in both directions.  With top-8 routing over 8 ranks a
// token reaches about 5 distinct ranks, and with skewed routing the hot rank receives the same
// token through several of its experts, so most of those bytes are duplicates.  Here:
//
//   dispatch  (one cooperative launch per rank)
//     A  count entries per expert (all warps; the order inside a rank is (token, k))
//     B  store the per-expert totals into every rank's count matrix, raise COUNTS
//     C  land rows: token t goes ONCE to every rank that owns one of its experts, into
//        that rank's landing buffer at (source rank, t) -- needs no slot, so it starts
//        before the counts of the other ranks have arrived
//     D  when the counts are in: final slot of every entry in the reference's order
//        (source rank, token, k); store its 5-int metadata at the final place, and per
//        (token, destination) the row indices + routing weights + an epoch mark
//     E  last CTA raises DATA on every rank
//     F  owner side: as each source's DATA arrives, copy its landed rows into
//        expert_x[e_local, slot] (local traffic only), optionally applying the task's
//        elementwise expert op into expert_y on the way
//   combine   (one cooperative launch per rank)
//     0  (only when dispatch did not carry the weights) push weights, raise/await WEIGHTS
//     1  owner side: per landed (source, token) the fp32 sum over its local entries of
//        w * expert_y[row], pushed as ONE row into the source's return buffer
//     2  last CTA raises RET; source side: out[t] = sum over the owners it used
//
// Calls must alternate dispatch, combine: a rank enters call n+1 only after every owner's
// RET flag of call n, i.e. after every rank finished reading what call n+1 overwrites.
// All cross-GPU waits are bounded (signal.cuh); row indices read from memory that peers
// write are range-checked before use (STATUS_BAD_INDEX, access skipped).
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <cstdlib>

#include "moe.h"
#include "moe_common.cuh"
#include "signal.cuh"
#include "sm100_ptx.cuh"

namespace b200 {

namespace {

using namespace moe;

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMetaDim = 5;
constexpr int kU = 8;  // 16-byte vectors per lane held in registers per chunk (4 KiB per warp)
constexpr int kMaxChunks = 8;
constexpr int kLandStage = 4096;  // bytes per landing stage; two stages per warp
constexpr int kLandBytes = kWarps * 2 * kLandStage;  // dynamic shared memory of the landing stages per CTA

struct Dst2 {
  int4* x;
  int4* y;
};

// One warp copies vectors [v_lo, v_hi) of a row to up to `n_dst` destinations: the chunk is
// loaded once into registers and stored to every destination.  dst_of(j) is evaluated by
// the whole warp (it may shuffle) and returns {nullptr, nullptr} to skip.  With SCALE the
// second pointer receives the row multiplied by `scale`.
template <typename T, bool SCALE, typename F>
__device__ __forceinline__ void warp_fanout(const int4* __restrict__ src, int v_lo, int v_hi, int lane, int n_dst,
                                            float scale, F&& dst_of) {
  for (int v0 = v_lo; v0 < v_hi; v0 += 32 * kU) {
    int4 r[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int idx = v0 + lane + 32 * u;
      if (idx < v_hi) r[u] = __ldcg(src + idx);
    }
    for (int j = 0; j < n_dst; ++j) {
      const Dst2 d = dst_of(j);
      if (d.x == nullptr) continue;
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int idx = v0 + lane + 32 * u;
        if (idx < v_hi) {
          d.x[idx] = r[u];
          if (SCALE) d.y[idx] = scale_vec<T>(r[u], scale);
        }
      }
    }
  }
}

// Same for rows that are not a whole number of aligned 16-byte vectors: element loop.
template <typename T, bool SCALE, typename F>
__device__ __forceinline__ void warp_fanout_scalar(const T* __restrict__ src, int hidden, int lane, int n_dst, float scale,
                                                   F&& dst_of) {
  for (int j = 0; j < n_dst; ++j) {
    const Dst2 d = dst_of(j);
    if (d.x == nullptr) continue;
    T* dx = reinterpret_cast<T*>(d.x);
    T* dy = reinterpret_cast<T*>(d.y);
    for (int h = lane; h < hidden; h += 32) {
      const T v = src[h];
      dx[h] = v;
      if (SCALE) dy[h] = from_f32<T>(to_f32(v) * scale);
    }
  }
}

__device__ __forceinline__ void stamp(uint64_t* trace, int slot) {
  if (trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) trace[slot] = global_timer_ns();
}

// Threads 0..world-1 wait for the `row` flags of all sources; returns false on expiry.
__device__ __forceinline__ bool cta_wait_all(uint64_t my_base, int row, uint64_t epoch, int world, uint64_t limit,
                                             StatusBlock* st, uint32_t phase) {
  if ((int)threadIdx.x < world) {
    wait_flag_ge(flag_ptr(my_base, row, threadIdx.x), epoch, limit, st, phase, threadIdx.x, (int)blockIdx.x);
  }
  __syncthreads();
  return !status_timed_out(st);
}

// After every CTA of the grid has passed here, exactly one of them (the last) gets true.
// Every CTA's earlier stores are ordered before anything the last CTA does afterwards.
__device__ __forceinline__ bool last_cta_arrives(uint32_t* counter) {
  __shared__ int is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t done = atomicAdd(counter, 1u);
    is_last = (done == gridDim.x - 1u);
    if (is_last) __threadfence_system();
  }
  __syncthreads();
  return is_last != 0;
}

// ---- weighted sum of rows through shared memory ------------------------------------------------
// Register loads keep at most a few KiB per warp in flight, which leaves a reduction over
// scattered 8-16 KiB rows latency-bound at under half of the memory bandwidth.  Here every row's
// run of bytes is fetched by ONE bulk copy (cp.async.bulk, completion counted on the warp's
// mbarrier), so a warp has its whole stage in flight and sixteen warps keep ~190 KiB per SM
// moving; the sum is then formed from shared memory.
constexpr int kStageBytes = 12288;  // per warp

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint64_t limit_ns, StatusBlock* st,
                                                  uint32_t phase) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!ptx::mbar_try_wait(bar, parity)) {
    if ((++spins & 255u) == 0 && global_timer_ns() - t0 > limit_ns) {
      record_status(st, STATUS_TIMEOUT, phase, -1, (int)blockIdx.x, 0, parity);
      return false;
    }
  }
  return true;
}

// One warp: dst[v] = sum over c < cnt (ascending) of w_c * row_c[v] for the 16-byte vectors
// v in [v_lo, v_hi) of rows of T.  Lane c holds row_c (a local pointer, 16-byte aligned) and w_c.
// `stage` / `stage_u32` is this warp's shared-memory stage, `bar` its mbarrier (count 1), `parity`
// the phase to wait for next.  With OUT_FP32 the sums are stored un-rounded (4 bytes per element).
// Returns false if a copy did not complete within the limit (recorded).
template <typename T, bool OUT_FP32>
__device__ __forceinline__ bool warp_weighted_sum_bulk(const uint8_t* row, float w, int cnt, int v_lo, int v_hi,
                                                       uint8_t* dst_row, const uint8_t* stage, uint32_t stage_u32,
                                                       uint32_t bar, uint32_t& parity, int lane, uint64_t limit_ns,
                                                       StatusBlock* st) {
  constexpr int N = Vec16<T>::N;
  constexpr int CU = 4;
  int cv = kStageBytes / 16 / cnt;  // vectors per row that fit the stage together with the other rows
  cv = cv >= 32 ? (cv & ~31) : cv;
  for (int vc = v_lo; vc < v_hi; vc += cv) {
    const int nvc = min(cv, v_hi - vc);
    const uint32_t cb = (uint32_t)nvc * 16u;
    if (lane == 0) ptx::mbar_arrive_expect_tx(bar, cb * (uint32_t)cnt);
    __syncwarp();
    if (lane < cnt) ptx::bulk_load(stage_u32 + (uint32_t)lane * cb, row + (size_t)vc * 16, cb, bar);
    if (!mbar_wait_bounded(bar, parity, limit_ns, st, PHASE_MOE_RETURN)) return false;
    parity ^= 1u;
    for (int v0 = 0; v0 < nvc; v0 += 32 * CU) {
      float acc[CU][N];
#pragma unroll
      for (int u = 0; u < CU; ++u)
#pragma unroll
        for (int e = 0; e < N; ++e) acc[u][e] = 0.f;
      for (int c = 0; c < cnt; ++c) {
        const float wc = __shfl_sync(0xffffffffu, w, c);
        const int4* srow = reinterpret_cast<const int4*>(stage + (size_t)c * cb);
#pragma unroll
        for (int u = 0; u < CU; ++u) {
          const int idx = v0 + lane + 32 * u;
          if (idx < nvc) fma_vec<T>(acc[u], srow[idx], wc);
        }
      }
#pragma unroll
      for (int u = 0; u < CU; ++u) {
        const int idx = v0 + lane + 32 * u;
        if (idx >= nvc) continue;
        const size_t gv = (size_t)vc + idx;
        if (OUT_FP32) {
          float4* d4 = reinterpret_cast<float4*>(dst_row) + gv * (N / 4);
#pragma unroll
          for (int q = 0; q < N / 4; ++q)
            d4[q] = make_float4(acc[u][4 * q], acc[u][4 * q + 1], acc[u][4 * q + 2], acc[u][4 * q + 3]);
        } else {
          reinterpret_cast<int4*>(dst_row)[gv] = pack_vec<T>(acc[u]);
        }
      }
    }
    // every lane is done reading the stage before the next copies may overwrite it
    ptx::fence_proxy_async_smem();
    __syncwarp();
  }
  return true;
}

}  // namespace

// ---------------------------------------------------------------------------------------
// dispatch
// ---------------------------------------------------------------------------------------
// SMALL: a few thousand entries.  Every CTA reads all expert ids and builds the whole
// histogram itself, and an entry's position among equal experts is found by scanning the
// entries before it: no in-GPU barrier on the latency chain, and a row can be split over
// several warps.  Otherwise CTAs own contiguous token ranges, count them with all warps
// and meet once on a grid barrier.
template <typename T, bool SMALL>
__global__ void __launch_bounds__(kThreads) moe_dedup_dispatch_kernel(const MoeDedupDispatchParams p) {
  // dynamic shared memory: [landing stages: kLandBytes, only with bulk landing] [int32 work arrays]
  extern __shared__ __align__(128) uint8_t smem_dispatch[];
  int32_t* smem_i32 = reinterpret_cast<int32_t*>(smem_dispatch + (p.bulk_landing ? kLandBytes : 0));
  __shared__ uint64_t land_bars[kWarps];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  if (p.bulk_landing) {
    if (tid == 0) {
      for (int wi = 0; wi < kWarps; ++wi) ptx::mbar_init(ptx::smem_u32(&land_bars[wi]), 1);
      ptx::fence_mbar_init();
      ptx::fence_proxy_async_smem();
    }
    __syncthreads();
  }
  const int E = p.num_experts;
  const int El = p.num_local_experts;
  const int k = p.k;
  const int T_tok = p.num_tokens;
  const int n = T_tok * k;
  const int G = gridDim.x;
  const int W = G * kWarps;
  const int gw = blockIdx.x * kWarps + warp;
  const int P = SMALL ? p.pieces : 1;   // pieces of a row in the landing pass
  const int PR = p.rep_pieces;           // ... and in the replication pass
  const uint64_t my_base = p.peer_base[p.rank];
  const uint32_t epoch32 = (uint32_t)p.epoch;
  const bool vec16 = (p.row_bytes & 15u) == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15u) == 0;
  const int nv = (int)(p.row_bytes >> 4);
  const int pv = (nv + P - 1) / P;  // vectors per piece
  const int pvr = (nv + PR - 1) / PR;
  const int hidden = (int)(p.row_bytes / sizeof(T));
  const uint8_t* xbytes = reinterpret_cast<const uint8_t*>(p.x);
  uint32_t bar_target = 0;
  stamp(p.trace, 0);

  // shared memory: SMALL: ids[n padded to 32] | hist[E] | base[E];  else: whist[8][E] | base[E] | tot[E]
  int32_t* s_idx = smem_i32;
  int32_t* s_hist = SMALL ? smem_i32 + ((n + 31) & ~31) : smem_i32;
  int32_t* s_base = SMALL ? s_hist + E : smem_i32 + kWarps * E;
  int32_t* s_tot = s_base + E;  // !SMALL only
  int32_t* whist = smem_i32 + warp * E;  // !SMALL: this warp's row

  // token range of this CTA / warp (!SMALL)
  const int tpc = (T_tok + G - 1) / G;
  const int tpw = (tpc + kWarps - 1) / kWarps;
  const int cta_t0 = min(T_tok, (int)blockIdx.x * tpc);
  const int cta_t1 = min(T_tok, cta_t0 + tpc);
  const int w_t0 = min(cta_t1, cta_t0 + warp * tpw);
  const int w_t1 = min(cta_t1, w_t0 + tpw);

  // ---- phase A: count --------------------------------------------------------------------
  if (SMALL) {
    for (int e = tid; e < 2 * E; e += kThreads) s_hist[e] = 0;
    for (int i = tid; i < n; i += kThreads) {
      int e = p.indices[i];
      if (e < 0 || e >= E) {
        if (blockIdx.x == 0) record_status(p.status, STATUS_BAD_INDEX, PHASE_NONE, -1, i, p.epoch, (uint64_t)(int64_t)e);
        e = -1;
      }
      s_idx[i] = e;
    }
    __syncthreads();
    for (int i = tid; i < n; i += kThreads) {
      const int e = s_idx[i];
      if (e >= 0) atomicAdd(&s_hist[e], 1);
    }
    __syncthreads();
  } else {
    for (int e = tid; e < (kWarps + 2) * E; e += kThreads) smem_i32[e] = 0;
    __syncthreads();
    for (int t = w_t0; t < w_t1; ++t) {
      int e = -1;
      if (lane < k) {
        e = p.indices[(size_t)t * k + lane];
        if (e < 0 || e >= E) {
          record_status(p.status, STATUS_BAD_INDEX, PHASE_NONE, -1, t * k + lane, p.epoch, (uint64_t)(int64_t)e);
          e = -1;
        }
      }
      const unsigned active = __ballot_sync(0xffffffffu, e >= 0);
      if (e >= 0) {
        const unsigned same = __match_any_sync(active, e);
        if ((same & ((1u << lane) - 1u)) == 0) whist[e] += __popc(same);
      }
      __syncwarp();
    }
    __syncthreads();
    // per expert: exclusive prefix over the warps of this CTA (in place), CTA total to global
    for (int e = tid; e < E; e += kThreads) {
      int run = 0;
      for (int w = 0; w < kWarps; ++w) {
        const int c = smem_i32[w * E + e];
        smem_i32[w * E + e] = run;
        run += c;
      }
      p.blk_hist[(size_t)blockIdx.x * E + e] = run;
    }
    grid_barrier(&p.sync_counters[0], bar_target, p.timeout_ns, p.status);
  }
  stamp(p.trace, 1);

  // ---- phase B: publish this rank's per-expert totals to every rank -----------------------
  if (SMALL) {
    for (int dst = blockIdx.x; dst < p.world_size; dst += G) {
      int32_t* remote = peer_ptr<int32_t>(p.peer_base[dst], p.layout.off_counts) + (size_t)p.rank * E;
      for (int e = tid; e < E; e += kThreads) remote[e] = s_hist[e];
    }
  } else {
    // base[e] = entries of this rank in lower CTAs; tot[e] = all of them (publishing CTAs only).
    // One coalesced pass over the histogram rows with shared-memory adds keeps every thread busy.
    const int rows = ((int)blockIdx.x < p.world_size) ? G : (int)blockIdx.x;
    const int lim = rows * E;
    for (int base = tid; base < lim; base += kThreads * 8) {
      int c[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {  // eight loads in flight per thread
        const int idx = base + u * kThreads;
        c[u] = idx < lim ? __ldcg(p.blk_hist + idx) : 0;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (c[u] == 0) continue;
        const int idx = base + u * kThreads;
        const int g = idx / E;
        const int e = idx - g * E;
        if (g < (int)blockIdx.x) atomicAdd(&s_base[e], c[u]);
        atomicAdd(&s_tot[e], c[u]);
      }
    }
    __syncthreads();
    for (int dst = blockIdx.x; dst < p.world_size; dst += G) {
      int32_t* remote = peer_ptr<int32_t>(p.peer_base[dst], p.layout.off_counts) + (size_t)p.rank * E;
      for (int e = tid; e < E; e += kThreads) remote[e] = s_tot[e];
    }
  }
  __syncthreads();
  const int C = SMALL ? 1 : max(1, min(p.chunks, kMaxChunks));  // chunks of this rank's tokens, each with its own DATA flag
  if (tid == 0 && (int)blockIdx.x < p.world_size) {
    // how this rank cuts its tokens into chunks travels with the counts: epoch | chunks | grid | tokens
    const uint64_t info = ((p.epoch & 0xffffffull) << 40) | ((uint64_t)C << 36) | ((uint64_t)(SMALL ? 0 : G) << 24) |
                          (uint64_t)T_tok;
    for (int dst = blockIdx.x; dst < p.world_size; dst += G)
      st_relaxed_sys(flag_ptr(p.peer_base[dst], FLAG_MOE_INFO, p.rank), info);
    __threadfence_system();
    for (int dst = blockIdx.x; dst < p.world_size; dst += G)
      st_release_sys(flag_ptr(p.peer_base[dst], FLAG_MOE_COUNTS, p.rank), p.epoch);
    if (!SMALL) atomicAdd(&p.sync_counters[4], 1u);
  }
  if (!SMALL && p.world_size > 1) {
    // The count rows must leave before the first row does: a GPU's stores to all its peers share
    // one way out, and a few hundred bytes queued behind megabytes bound for a busy peer arrive
    // when those have drained -- far too late for the peers that wait for them.
    if (tid == 0)
      wait_u32_ge(&p.sync_counters[4], (uint32_t)min(p.world_size, G), p.timeout_ns, p.status, PHASE_GRID_BARRIER, -1,
                  (int)blockIdx.x, false);
    __syncthreads();
  }

  // Counts of all ranks -> where this rank's rows start in every expert buffer.  The small kernel
  // does this after its rows have left (their flight hides the count exchange); the large one
  // before its first chunk, because every chunk needs final slots for its records.
  bool alive = true;
  const int32_t* counts = peer_ptr<const int32_t>(my_base, p.layout.off_counts);  // [world][E]
  auto await_counts = [&]() {
    alive = cta_wait_all(my_base, FLAG_MOE_COUNTS, p.epoch, p.world_size, p.timeout_ns, p.status, PHASE_MOE_COUNTS);
    stamp(p.trace, 3);
    if (!alive) return;
    for (int e = tid; e < E; e += kThreads) {
      int lower = 0;
      for (int s = 0; s < p.rank; ++s) lower += __ldcg(counts + (size_t)s * E + e);
      s_base[e] += lower;
    }
    if (blockIdx.x == 0) {
      for (int el = tid; el < El; el += kThreads) {
        int total = 0;
        for (int s = 0; s < p.world_size; ++s) total += __ldcg(counts + (size_t)s * E + p.rank * El + el);
        p.expert_num_tokens[el] = min(total, p.max_recv);
      }
    }
    __syncthreads();
  };
  if (!SMALL) await_counts();

  // ---- phase C: land every token once per destination rank --------------------------------
  // (token, piece) items: this warp's own tokens, or strided over all warps when SMALL
  const uint32_t land_stage_u32 = ptx::smem_u32(smem_dispatch + (size_t)warp * 2 * kLandStage);
  const uint32_t land_bar = ptx::smem_u32(&land_bars[warp]);
  uint32_t land_parity = 0, land_chunks = 0;
  bool land_ok = true;
  const int w_len = w_t1 - w_t0;
  for (int c = 0; c < C; ++c) {
  // chunk c of this warp's tokens: those with (i * C) / w_len == c, i counted from w_t0
  const int c_t0 = w_t0 + (c * w_len + C - 1) / C;
  const int c_t1 = w_t0 + ((c + 1) * w_len + C - 1) / C;
  {
    const int item0 = SMALL ? gw : c_t0;
    const int item1 = SMALL ? T_tok * P : c_t1;
    const int step = SMALL ? W : 1;
    for (int item = item0; item < item1; item += step) {
      const int t = SMALL ? item / P : item;
      const int piece = SMALL ? item - t * P : 0;
      int e = -1;
      if (lane < k) {
        e = SMALL ? s_idx[t * k + lane] : p.indices[(size_t)t * k + lane];
        if (e < 0 || e >= E) e = -1;
      }
      const unsigned mask = __reduce_or_sync(0xffffffffu, e >= 0 ? (1u << (e / El)) : 0u) & ~(1u << p.rank);
      if (mask == 0) continue;
      const uint64_t land_off = p.layout.off_land + ((uint64_t)p.rank * p.max_tokens + t) * p.row_bytes;
      auto dst_of = [&](int j) {
        int d = p.rank + 1 + j;
        if (d >= p.world_size) d -= p.world_size;
        Dst2 r{nullptr, nullptr};
        if ((mask >> d) & 1u) r.x = peer_ptr<int4>(p.peer_base[d], land_off);
        return r;
      };
      if (vec16 && p.bulk_landing) {
        // One lane drives the copies: a run of the row comes into a stage with one bulk load and
        // leaves with one bulk store per destination; the second stage is loaded while the stores
        // of the first drain, and no register or issue slot is tied up by NVLink back-pressure.
        if (lane == 0 && land_ok) {
          const uint8_t* src = xbytes + (size_t)t * p.row_bytes;
          const int v_lo = piece * pv, v_hi = min(nv, (piece + 1) * pv);
          for (int vc = v_lo; vc < v_hi; vc += kLandStage / 16) {
            const uint32_t bytes = (uint32_t)min(kLandStage / 16, v_hi - vc) * 16u;
            const uint32_t st = land_stage_u32 + (land_chunks & 1u) * kLandStage;
            ptx::bulk_wait_group_read<1>();  // the stores that used this stage two runs ago have read it
            ptx::mbar_arrive_expect_tx(land_bar, bytes);
            ptx::bulk_load(st, src + (size_t)vc * 16, bytes, land_bar);
            if (!mbar_wait_bounded(land_bar, land_parity, p.timeout_ns, p.status, PHASE_MOE_DATA)) {
              land_ok = false;
              break;
            }
            land_parity ^= 1u;
            ptx::fence_proxy_async_smem();
            for (int j = 0; j < p.world_size - 1; ++j) {
              const Dst2 d = dst_of(j);
              if (d.x != nullptr) ptx::bulk_store(reinterpret_cast<uint8_t*>(d.x) + (size_t)vc * 16, st, bytes);
            }
            ptx::bulk_commit_group();
            ++land_chunks;
          }
        }
        __syncwarp();
      } else if (vec16) {
        warp_fanout<T, false>(reinterpret_cast<const int4*>(xbytes + (size_t)t * p.row_bytes), piece * pv,
                              min(nv, (piece + 1) * pv), lane, p.world_size - 1, 0.f, dst_of);
      } else if (piece == 0) {
        warp_fanout_scalar<T, false>(reinterpret_cast<const T*>(xbytes + (size_t)t * p.row_bytes), hidden, lane,
                                     p.world_size - 1, 0.f, dst_of);
      }
    }
  }
  if (p.bulk_landing && lane == 0) {
    ptx::bulk_wait_group<0>();  // this warp's bulk stores have been performed ...
    asm volatile("fence.proxy.async.global;" ::: "memory");  // ... and are ordered before the flag stores below
  }
  __syncwarp();
  stamp(p.trace, 2);

  // ---- phase D: final slots of the chunk's entries; one record per (token, destination) ------
  if (SMALL) await_counts();
  if (alive) {
    const int item0 = SMALL ? gw : c_t0;
    const int item1 = SMALL ? T_tok : c_t1;
    const int step = SMALL ? W : 1;
    for (int t = item0; t < item1; t += step) {
      int e = -1;
      if (lane < k) {
        e = SMALL ? s_idx[t * k + lane] : p.indices[(size_t)t * k + lane];
        if (e < 0 || e >= E) e = -1;
      }
      int slot = -1;
      if (SMALL) {
        // entries of this rank with the same expert before entry (t, kk): scan by the warp
        for (int kk = 0; kk < k; ++kk) {
          const int ek = __shfl_sync(0xffffffffu, e, kk);
          if (ek < 0) continue;
          const int upto = t * k + kk;
          int part = 0;
          for (int j = lane; j < upto; j += 32) part += (s_idx[j] == ek) ? 1 : 0;
          part = warp_sum(part);
          if (lane == kk) slot = s_base[ek] + part;
        }
      } else {
        const unsigned active = __ballot_sync(0xffffffffu, e >= 0);
        if (e >= 0) {
          const unsigned same = __match_any_sync(active, e);
          const int before = __popc(same & ((1u << lane) - 1u));
          const int cur = whist[e];
          __syncwarp(active);
          slot = s_base[e] + cur + before;
          if (before == 0) whist[e] = cur + __popc(same);
        }
        __syncwarp();
      }
      int dst = -1, row = -1;
      if (e >= 0) {
        dst = e / El;
        if (slot >= 0 && slot < p.max_recv) {
          row = (e - dst * El) * p.max_recv + slot;
        } else {
          record_status(p.status, STATUS_BAD_INDEX, PHASE_NONE, dst, t * k + lane, p.epoch, (uint64_t)(int64_t)slot);
        }
      }
      if (lane < k) p.route[(size_t)t * k + lane] = make_int2(row >= 0 ? dst : -1, row);
      const float w = (p.weights != nullptr && lane < k) ? p.weights[(size_t)t * k + lane] : 0.f;
      unsigned mask = __reduce_or_sync(0xffffffffu, e >= 0 ? (1u << dst) : 0u);
      // The record of (this rank, t) on every destination: lane 0 carries the mark, lanes 1..k the
      // final rows, lanes k+1..2k the weights -- one coalesced store per destination.  (The 5-int
      // metadata rows of the reference layout are written by the owner when it replicates.)
      const int from = lane == 0 ? 0 : (lane <= k ? lane - 1 : lane - 1 - k);
      const int row_f = __shfl_sync(0xffffffffu, row, from);
      const int dst_f = __shfl_sync(0xffffffffu, dst, from);
      const float w_f = __shfl_sync(0xffffffffu, w, from);
      const int words = p.weights != nullptr ? 1 + 2 * k : 1 + k;
      const uint64_t rec = ((uint64_t)p.rank * p.max_tokens + t) * p.rec_ints;
      while (mask) {
        const int d = __ffs(mask) - 1;
        mask &= mask - 1;
        if (lane < words) {
          int32_t v;
          if (lane == 0) v = (int32_t)epoch32;
          else if (lane <= k) v = (dst_f == d) ? row_f : -1;
          else v = __float_as_int((dst_f == d) ? w_f : 0.f);
          peer_ptr<int32_t>(p.peer_base[d], p.layout.off_tok_rec)[rec + lane] = v;
        }
      }
    }
  }
  stamp(p.trace, 4);

  // ---- phase E: every CTA has delivered its part of the chunk -> tell the owners -------------
  if (last_cta_arrives(&p.sync_counters[16 + c])) {
    if (tid == 0) {
      if (!status_timed_out(p.status)) {  // no CTA of this rank gave up: everything was stored
        const uint64_t done = (p.epoch << 8) | (uint64_t)(c + 1);
        for (int d = 0; d < p.world_size; ++d) st_relaxed_sys(flag_ptr(p.peer_base[d], FLAG_MOE_DATA, p.rank), done);
      }
      p.sync_counters[16 + c] = 0;
      if (c == C - 1) {
        p.sync_counters[0] = 0;
        p.sync_counters[4] = 0;
      }
    }
  }
  }  // chunks

  // ---- phase F: replicate landed rows into the expert buffers, chunk by chunk, source by source
  // A source's chunk c is complete when its DATA flag reaches (epoch << 8) | (c + 1); the chunks of
  // the sources are replicated while their later chunks are still crossing the links.
  const uint8_t* land = peer_ptr<const uint8_t>(my_base, p.layout.off_land);
  uint8_t* ex = peer_ptr<uint8_t>(my_base, p.layout.off_expert_x);
  uint8_t* ey = reinterpret_cast<uint8_t*>(p.expert_y);
  const int32_t* tok_rec = peer_ptr<const int32_t>(my_base, p.layout.off_tok_rec);
  int32_t* meta = peer_ptr<int32_t>(my_base, p.layout.off_expert_meta);
  const int total_rows = El * p.max_recv;
  // how every source cut its tokens (its info word is in place once its counts flag is)
  __shared__ int src_T[kMaxWorldSize], src_G[kMaxWorldSize], src_C[kMaxWorldSize];
  if (tid < p.world_size) {
    const uint64_t info = ld_acquire_sys(flag_ptr(my_base, FLAG_MOE_INFO, tid));
    const bool fresh = ((info >> 40) & 0xffffffull) == (p.epoch & 0xffffffull);
    src_T[tid] = fresh ? min((int)(info & 0xffffffull), p.max_tokens) : 0;
    src_G[tid] = fresh ? (int)((info >> 24) & 0xfffull) : 0;
    src_C[tid] = fresh ? max(1, (int)((info >> 36) & 0xfull)) : 1;
  }
  __syncthreads();
  int c_max = 1;
  for (int s = 0; s < p.world_size; ++s) c_max = max(c_max, src_C[s]);
  // Chunk by chunk, and inside a chunk source by source as the flags come in (this rank's own rows
  // first): the replication of one source's chunk overlaps the arrival of the next one's.
  for (int c = 0; c < c_max && alive; ++c) {
  for (int j = 0; j < p.world_size && alive; ++j) {
    int s = p.rank + j;
    if (s >= p.world_size) s -= p.world_size;
    const int Cs = src_C[s];
    if (c >= Cs) continue;
    if (tid == 0)
      wait_flag_ge(flag_ptr(my_base, FLAG_MOE_DATA, s), (p.epoch << 8) | (uint64_t)(c + 1), p.timeout_ns, p.status,
                   PHASE_MOE_DATA, s, (int)blockIdx.x);
    __syncthreads();
    alive = !status_timed_out(p.status);
    if (!alive) break;
    if (c == c_max - 1 && j == p.world_size - 1) stamp(p.trace, 5);
    // the source's partition of its tokens: CTA g owns tpc tokens, its warp w tpw of those
    const int Ts = src_T[s];
    const int Gs = max(src_G[s], 1);
    const int s_tpc = (Ts + Gs - 1) / Gs;
    const int s_tpw = (s_tpc + kWarps - 1) / kWarps;
    // Dense numbering of the chunk's tokens: (source warp, position inside its share of the chunk,
    // piece) -- so that consecutive items are live and every warp here gets its share of them.
    const int max_sub = (s_tpw + Cs - 1) / Cs;
    const int n_items = Gs * kWarps * max_sub * PR;
    for (int item = gw; item < n_items; item += W) {
      const int piece = item % PR;
      const int q = item / PR;
      const int sub = q % max_sub;
      const int pair = q / max_sub;
      const int g = pair / kWarps;
      const int w = pair - g * kWarps;
      const int len = min(s_tpw, min(s_tpc, Ts - g * s_tpc) - w * s_tpw);  // tokens of that source warp
      if (len <= 0) continue;
      const int i = (c * len + Cs - 1) / Cs + sub;
      if (i >= ((c + 1) * len + Cs - 1) / Cs) continue;
      const int t = g * s_tpc + w * s_tpw + i;
      const uint64_t rec = (uint64_t)s * p.max_tokens + t;
      // lane 0 reads the mark, lanes 1..k the rows of the record: one load for the warp
      int word = 0;
      if (lane <= k) word = __ldcg(tok_rec + rec * p.rec_ints + lane);
      if ((uint32_t)__shfl_sync(0xffffffffu, word, 0) != epoch32) continue;
      int row = __shfl_down_sync(0xffffffffu, word, 1);  // lane kk < k: row of entry kk
      if (lane >= k) row = -1;
      if (row >= total_rows) {
        record_status(p.status, STATUS_BAD_INDEX, PHASE_MOE_DATA, s, t, p.epoch, (uint64_t)(int64_t)row);
        row = -1;
      }
      if (__ballot_sync(0xffffffffu, row >= 0) == 0) continue;
      if (piece == 0 && row >= 0) {
        // metadata row of the reference layout: (global expert, source rank, token, k, 0)
        int32_t* m = meta + (size_t)row * kMetaDim;
        m[0] = p.rank * El + row / p.max_recv;
        m[1] = s;
        m[2] = t;
        m[3] = lane;
        m[4] = 0;
      }
      const uint8_t* src = (s == p.rank) ? xbytes + (size_t)t * p.row_bytes : land + rec * p.row_bytes;
      auto dst_of = [&](int kk) {
        const int r = __shfl_sync(0xffffffffu, row, kk);
        Dst2 d{nullptr, nullptr};
        if (r >= 0) {
          d.x = reinterpret_cast<int4*>(ex + (size_t)r * p.row_bytes);
          d.y = reinterpret_cast<int4*>(ey + (size_t)r * p.row_bytes);
        }
        return d;
      };
      if (vec16) {
        const int v_lo = piece * pvr, v_hi = min(nv, (piece + 1) * pvr);
        if (p.fuse_scale) warp_fanout<T, true>(reinterpret_cast<const int4*>(src), v_lo, v_hi, lane, k, p.scale, dst_of);
        else warp_fanout<T, false>(reinterpret_cast<const int4*>(src), v_lo, v_hi, lane, k, 0.f, dst_of);
      } else if (piece == 0) {
        if (p.fuse_scale) warp_fanout_scalar<T, true>(reinterpret_cast<const T*>(src), hidden, lane, k, p.scale, dst_of);
        else warp_fanout_scalar<T, false>(reinterpret_cast<const T*>(src), hidden, lane, k, 0.f, dst_of);
      }
    }
  }
  }  // chunks
  stamp(p.trace, 6);
  if (p.trace != nullptr && tid == 0) atomicMax(reinterpret_cast<unsigned long long*>(p.trace + 7), global_timer_ns());
}

// ---------------------------------------------------------------------------------------
// combine
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads) moe_dedup_combine_kernel(const MoeDedupCombineParams p) {
  constexpr int N = Vec16<T>::N;
  constexpr int CU = 4;  // vectors per lane per chunk
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int k = p.k;
  const int G = gridDim.x;
  const int W = G * kWarps;
  const int gw = blockIdx.x * kWarps + warp;
  const int P = p.pieces;
  const uint64_t my_base = p.peer_base[p.rank];
  const uint32_t mark32 = (uint32_t)p.dispatch_epoch;
  const size_t row_bytes = (size_t)p.hidden * sizeof(T);
  const bool vec16 = (row_bytes & 15u) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15u) == 0 &&
                     (reinterpret_cast<uintptr_t>(p.expert_y) & 15u) == 0;
  const int nv = (int)(row_bytes >> 4);
  const int pv = (nv + P - 1) / P;
  const size_t ret_row_bytes = p.partial_fp32 ? (size_t)p.hidden * 4 : row_bytes;
  stamp(p.trace, 0);
  bool alive = true;

  // this warp's stage and mbarrier for the bulk-copy reductions
  extern __shared__ __align__(128) uint8_t smem_stage[];
  __shared__ uint64_t stage_bars[kWarps];
  const uint8_t* stage = smem_stage + (size_t)warp * kStageBytes;
  const uint32_t stage_u32 = ptx::smem_u32(stage);
  const uint32_t bar = ptx::smem_u32(&stage_bars[warp]);
  uint32_t parity = 0;
  if (tid == 0) {
    for (int wi = 0; wi < kWarps; ++wi) ptx::mbar_init(ptx::smem_u32(&stage_bars[wi]), 1);
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  __syncthreads();

  // ---- phase 0: deliver the routing weights to the owners (when dispatch did not) ----------
  if (!p.weights_sent) {
    for (int t = gw; t < p.num_tokens; t += W) {
      int dst = -1;
      float w = 0.f;
      if (lane < k) {
        const int2 rt = __ldg(p.route + (size_t)t * k + lane);
        if (rt.y >= 0 && rt.x >= 0 && rt.x < p.world_size) dst = rt.x;
        w = __ldg(p.weights + (size_t)t * k + lane);
      }
      unsigned mask = __reduce_or_sync(0xffffffffu, dst >= 0 ? (1u << dst) : 0u);
      const uint64_t rec = ((uint64_t)p.rank * p.max_tokens + t) * p.rec_ints + 1 + k;
      while (mask) {
        const int d = __ffs(mask) - 1;
        mask &= mask - 1;
        if (lane < k) peer_ptr<float>(p.peer_base[d], p.layout.off_tok_rec)[rec + lane] = (dst == d) ? w : 0.f;
      }
    }
    if (last_cta_arrives(&p.sync_counters[2])) {
      if (tid == 0) {
        for (int d = 0; d < p.world_size; ++d)
          st_relaxed_sys(flag_ptr(p.peer_base[d], FLAG_MOE_Y_READY, p.rank), p.epoch);
        p.sync_counters[2] = 0;
      }
    }
    alive = cta_wait_all(my_base, FLAG_MOE_Y_READY, p.epoch, p.world_size, p.timeout_ns, p.status, PHASE_MOE_WEIGHTS);
  }
  stamp(p.trace, 1);

  // ---- phase 1: per landed (source, token): fp32 sum over the local entries, one row back ----
  const int32_t* tok_rec = peer_ptr<const int32_t>(my_base, p.layout.off_tok_rec);
  const uint8_t* ey = reinterpret_cast<const uint8_t*>(p.expert_y);
  const int total_rows = p.num_local_experts * p.max_recv;
  const bool direct_out = p.world_size == 1;  // the only owner is the source: write the result itself
  bool warp_ok = true;
  for (int j = 0; j < p.world_size && alive && warp_ok; ++j) {
    int s = p.rank + 1 + j;  // remote sources first, rotated so that the ranks do not all push to the same one
    if (s >= p.world_size) s -= p.world_size;
    for (int item = gw; item < p.max_tokens * P; item += W) {
      const int t = item / P;
      const int piece = item - t * P;
      const uint64_t rec = (uint64_t)s * p.max_tokens + t;
      // one load for the warp: lane 0 the mark, lanes 1..k the rows, lanes k+1..2k the weights
      int word = 0;
      if (lane <= 2 * k) word = __ldcg(tok_rec + rec * p.rec_ints + lane);
      if ((uint32_t)__shfl_sync(0xffffffffu, word, 0) != mark32) continue;
      int row = __shfl_sync(0xffffffffu, word, (lane + 1) & 31);
      float w = __int_as_float(__shfl_sync(0xffffffffu, word, (lane + 1 + k) & 31));
      if (lane >= k) {
        row = -1;
        w = 0.f;
      }
      if (row >= total_rows) {
        record_status(p.status, STATUS_BAD_INDEX, PHASE_MOE_RETURN, s, t, p.epoch, (uint64_t)(int64_t)row);
        row = -1;
      }
      // compact the valid entries to lanes 0..cnt-1, keeping ascending k
      const unsigned valid = __ballot_sync(0xffffffffu, row >= 0);
      const int cnt = __popc(valid);
      if (cnt == 0) continue;
      const int from = __fns(valid, 0, lane + 1);  // lane of the (lane+1)-th valid entry, or -1
      const int crow = __shfl_sync(0xffffffffu, row, from < 0 ? 0 : from);
      const float cw = __shfl_sync(0xffffffffu, w, from < 0 ? 0 : from);
      uint8_t* dst_row = direct_out
                             ? reinterpret_cast<uint8_t*>(p.out) + (size_t)t * row_bytes
                             : peer_ptr<uint8_t>(p.peer_base[s], p.layout.off_ret) +
                                   ((uint64_t)p.rank * p.max_tokens + t) * ret_row_bytes;
      if (vec16) {
        const int v_lo = piece * pv, v_hi = min(nv, (piece + 1) * pv);
        const uint8_t* my_row = ey + (size_t)(lane < cnt ? crow : 0) * row_bytes;
        bool ok;
        if (p.partial_fp32 && !direct_out) {
          ok = warp_weighted_sum_bulk<T, true>(my_row, cw, cnt, v_lo, v_hi, dst_row, stage, stage_u32, bar, parity, lane,
                                               p.timeout_ns, p.status);
        } else {
          ok = warp_weighted_sum_bulk<T, false>(my_row, cw, cnt, v_lo, v_hi, dst_row, stage, stage_u32, bar, parity, lane,
                                                p.timeout_ns, p.status);
        }
        if (!ok) {  // recorded as a timeout: the CTA-wide waits below will see it and give up together
          warp_ok = false;
          break;
        }
      } else if (piece == 0) {
        // the trip count is the same for every lane: the shuffles below need the whole warp
        for (int h0 = 0; h0 < p.hidden; h0 += 32) {
          const int h = h0 + lane;
          float acc = 0.f;
          for (int c = 0; c < cnt; ++c) {
            const int r = __shfl_sync(0xffffffffu, crow, c);
            const float wc = __shfl_sync(0xffffffffu, cw, c);
            if (h < p.hidden) acc = fmaf(to_f32(__ldcg(reinterpret_cast<const T*>(ey + (size_t)r * row_bytes) + h)), wc, acc);
          }
          if (h < p.hidden) {
            if (p.partial_fp32 && !direct_out) reinterpret_cast<float*>(dst_row)[h] = acc;
            else reinterpret_cast<T*>(dst_row)[h] = from_f32<T>(acc);
          }
        }
      }
    }
  }
  stamp(p.trace, 2);

  if (direct_out) {
    // tokens none of whose entries was delivered still get a defined (zero) row
    for (int t = gw; t < p.num_tokens; t += W) {
      bool any = false;
      if (lane < k) any = __ldg(p.route + (size_t)t * k + lane).y >= 0;
      if (__ballot_sync(0xffffffffu, any) != 0) continue;
      T* o = reinterpret_cast<T*>(p.out) + (size_t)t * p.hidden;
      for (int h = lane; h < p.hidden; h += 32) o[h] = from_f32<T>(0.f);
    }
    if (p.trace != nullptr && tid == 0) atomicMax(reinterpret_cast<unsigned long long*>(p.trace + 7), global_timer_ns());
    return;
  }

  // ---- phase 2: all partial rows pushed -> tell the sources; add up what came back ----------
  if (last_cta_arrives(&p.sync_counters[3])) {
    if (tid == 0) {
      if (!status_timed_out(p.status)) {
        for (int d = 0; d < p.world_size; ++d) st_relaxed_sys(flag_ptr(p.peer_base[d], FLAG_MOE_RET, p.rank), p.epoch);
      }
      p.sync_counters[3] = 0;
    }
  }
  if (alive) alive = cta_wait_all(my_base, FLAG_MOE_RET, p.epoch, p.world_size, p.timeout_ns, p.status, PHASE_MOE_RETURN);
  stamp(p.trace, 3);
  if (alive) {
    const uint8_t* ret = peer_ptr<const uint8_t>(my_base, p.layout.off_ret);
    for (int item = gw; item < p.num_tokens * P; item += W) {
      const int t = item / P;
      const int piece = item - t * P;
      int dst = -1;
      if (lane < k) {
        const int2 rt = __ldg(p.route + (size_t)t * k + lane);
        if (rt.y >= 0 && rt.x >= 0 && rt.x < p.world_size) dst = rt.x;
      }
      const unsigned mask = __reduce_or_sync(0xffffffffu, dst >= 0 ? (1u << dst) : 0u);
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) + (size_t)t * row_bytes;
      if (vec16 && !p.partial_fp32) {
        const int v_lo = piece * pv, v_hi = min(nv, (piece + 1) * pv);
        const int cnt = __popc(mask);
        if (cnt == 0) {  // nothing was delivered for this token: a defined (zero) row
          for (int idx = v_lo + lane; idx < v_hi; idx += 32) reinterpret_cast<int4*>(orow)[idx] = make_int4(0, 0, 0, 0);
          continue;
        }
        const int d = (int)__fns(mask, 0, lane + 1);  // lane c: the c-th owner in ascending rank order
        const uint8_t* my_row = ret + ((uint64_t)(lane < cnt ? d : 0) * p.max_tokens + t) * ret_row_bytes;
        if (!warp_weighted_sum_bulk<T, false>(my_row, 1.f, cnt, v_lo, v_hi, orow, stage, stage_u32, bar, parity, lane,
                                              p.timeout_ns, p.status))
          break;
      } else if (vec16) {
        const int v_lo = piece * pv, v_hi = min(nv, (piece + 1) * pv);
        for (int v0 = v_lo; v0 < v_hi; v0 += 32 * CU) {
          float acc[CU][N];
#pragma unroll
          for (int u = 0; u < CU; ++u)
#pragma unroll
            for (int e = 0; e < N; ++e) acc[u][e] = 0.f;
          unsigned m = mask;
          while (m) {  // ascending owner rank
            const int d = __ffs(m) - 1;
            m &= m - 1;
            const uint8_t* rrow = ret + ((uint64_t)d * p.max_tokens + t) * ret_row_bytes;
            if (p.partial_fp32) {
              float4 f[CU][N / 4];
#pragma unroll
              for (int u = 0; u < CU; ++u) {
                const int idx = v0 + lane + 32 * u;
#pragma unroll
                for (int q = 0; q < N / 4; ++q)
                  f[u][q] = idx < v_hi ? __ldcg(reinterpret_cast<const float4*>(rrow) + (size_t)idx * (N / 4) + q)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
              }
#pragma unroll
              for (int u = 0; u < CU; ++u)
#pragma unroll
                for (int q = 0; q < N / 4; ++q) {
                  acc[u][4 * q] += f[u][q].x;
                  acc[u][4 * q + 1] += f[u][q].y;
                  acc[u][4 * q + 2] += f[u][q].z;
                  acc[u][4 * q + 3] += f[u][q].w;
                }
            } else {
              int4 a[CU];
#pragma unroll
              for (int u = 0; u < CU; ++u) {
                const int idx = v0 + lane + 32 * u;
                a[u] = idx < v_hi ? __ldcg(reinterpret_cast<const int4*>(rrow) + idx) : make_int4(0, 0, 0, 0);
              }
#pragma unroll
              for (int u = 0; u < CU; ++u) fma_vec<T>(acc[u], a[u], 1.f);
            }
          }
#pragma unroll
          for (int u = 0; u < CU; ++u) {
            const int idx = v0 + lane + 32 * u;
            if (idx < v_hi) reinterpret_cast<int4*>(orow)[idx] = pack_vec<T>(acc[u]);
          }
        }
      } else if (piece == 0) {
        for (int h = lane; h < p.hidden; h += 32) {
          float acc = 0.f;
          unsigned m = mask;
          while (m) {
            const int d = __ffs(m) - 1;
            m &= m - 1;
            const uint8_t* rrow = ret + ((uint64_t)d * p.max_tokens + t) * ret_row_bytes;
            acc += p.partial_fp32 ? __ldcg(reinterpret_cast<const float*>(rrow) + h)
                                  : to_f32(__ldcg(reinterpret_cast<const T*>(rrow) + h));
          }
          reinterpret_cast<T*>(orow)[h] = from_f32<T>(acc);
        }
      }
    }
  }
  if (p.trace != nullptr && tid == 0) atomicMax(reinterpret_cast<unsigned long long*>(p.trace + 7), global_timer_ns());
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
namespace {

bool dedup_small(int num_entries, int num_experts) { return num_entries <= 4096 && num_experts <= 2048; }

// Kernels without a grid barrier wait only on flags that the LAST CTA of a grid raises, so all
// they need is that every CTA gets an SM eventually: the grid is sized to fit the device at
// once (occupancy x SMs) and launched the ordinary way, which costs several microseconds less
// per launch than a cooperative launch.  B200_COOP_LAUNCH=1 makes the runtime enforce the
// co-residency (e.g. when other work shares the device).  Waits are bounded either way.
bool force_cooperative() {
  static const bool on = [] {
    const char* v = std::getenv("B200_COOP_LAUNCH");
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  return on;
}

size_t dispatch_smem(bool small, int num_entries, int num_experts, bool bulk_landing) {
  const size_t stages = bulk_landing ? (size_t)kLandBytes : 0;
  if (small) return stages + ((size_t)((num_entries + 31) & ~31) + 2 * (size_t)num_experts) * sizeof(int32_t);
  return stages + (size_t)(kWarps + 2) * num_experts * sizeof(int32_t);
}

template <typename T, bool SMALL>
cudaError_t launch_dispatch_typed(const MoeDedupDispatchParams& p, int grid, size_t smem, cudaStream_t stream) {
  auto kernel = moe_dedup_dispatch_kernel<T, SMALL>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  if (SMALL && !force_cooperative()) {
    kernel<<<grid, kThreads, smem, stream>>>(p);
    return cudaGetLastError();
  }
  MoeDedupDispatchParams params = p;
  void* args[] = {&params};
  // Cooperative launch: CTAs meet on a grid barrier, so they must be co-resident.
  return cudaLaunchCooperativeKernel((const void*)kernel, dim3(grid), dim3(kThreads), args, smem, stream);
}

template <typename T>
int dispatch_occupancy(bool small, size_t smem) {
  int per_sm = 0;
  if (small) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_dedup_dispatch_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_dedup_dispatch_kernel<T, true>, kThreads, smem);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_dedup_dispatch_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_dedup_dispatch_kernel<T, false>, kThreads, smem);
  }
  return per_sm;
}

}  // namespace

bool moe_dedup_is_small(int num_entries, int num_experts) { return dedup_small(num_entries, num_experts); }

int moe_dedup_dispatch_max_blocks(int device, int num_experts, int num_entries, int bulk_landing) {
  // Occupancy of the bf16 instantiation stands for all three (same code up to conversions).
  struct Key { int device, experts, small_entries, bulk; int blocks; };
  static thread_local Key cache[8];
  static thread_local int used = 0;
  const bool small = dedup_small(num_entries, num_experts);
  const int small_entries = small ? ((num_entries + 31) & ~31) : -1;
  for (int i = 0; i < used; ++i)
    if (cache[i].device == device && cache[i].experts == num_experts && cache[i].small_entries == small_entries &&
        cache[i].bulk == bulk_landing)
      return cache[i].blocks;
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (sms <= 0) sms = 1;
  const size_t smem = dispatch_smem(small, num_entries, num_experts, bulk_landing != 0);
  int per_sm = dispatch_occupancy<__nv_bfloat16>(small, smem);
  if (per_sm < 1) per_sm = 1;
  // the large kernel sums one histogram row per CTA: more than one CTA per SM does not pay there
  const int blocks = sms * (small ? std::min(per_sm, 2) : 1);
  Key& slot = cache[used < 8 ? used++ : 7];
  slot = {device, num_experts, small_entries, bulk_landing, blocks};
  return blocks;
}

int moe_dedup_combine_max_blocks(int device) {
  static thread_local int cached_device = -1, cached = 0;
  if (cached_device == device) return cached;
  int sms = 0, per_sm = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int smem = kWarps * kStageBytes;
  cudaFuncSetAttribute(moe_dedup_combine_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaFuncSetAttribute(moe_dedup_combine_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaFuncSetAttribute(moe_dedup_combine_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_dedup_combine_kernel<__nv_bfloat16>, kThreads, smem);
  int other = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&other, moe_dedup_combine_kernel<float>, kThreads, smem);
  per_sm = std::max(1, std::min(std::min(per_sm, other), 3));
  cached_device = device;
  cached = std::max(sms, 1) * per_sm;
  return cached;
}

cudaError_t launch_moe_dedup_dispatch(const MoeDedupDispatchParams& p, int grid, cudaStream_t stream) {
  const int n = p.num_tokens * p.k;
  if (p.k < 1 || p.k > 32 || p.world_size > kMaxWorldSize || p.num_tokens > p.max_tokens) return cudaErrorInvalidValue;
  const bool small = dedup_small(n, p.num_experts);
  const size_t smem = dispatch_smem(small, n, p.num_experts, p.bulk_landing != 0);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  if (small) {
    switch (p.dtype) {
      case 0: return launch_dispatch_typed<__half, true>(p, grid, smem, stream);
      case 1: return launch_dispatch_typed<__nv_bfloat16, true>(p, grid, smem, stream);
      case 2: return launch_dispatch_typed<float, true>(p, grid, smem, stream);
      default: return cudaErrorInvalidValue;
    }
  }
  switch (p.dtype) {
    case 0: return launch_dispatch_typed<__half, false>(p, grid, smem, stream);
    case 1: return launch_dispatch_typed<__nv_bfloat16, false>(p, grid, smem, stream);
    case 2: return launch_dispatch_typed<float, false>(p, grid, smem, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_moe_dedup_combine(const MoeDedupCombineParams& p, int grid, cudaStream_t stream) {
  if (p.k < 1 || p.k > 32 || p.world_size > kMaxWorldSize) return cudaErrorInvalidValue;
  // the opt-in to this much dynamic shared memory was made by moe_dedup_combine_max_blocks(), which
  // every caller needs first to size the grid
  const size_t smem = (size_t)kWarps * kStageBytes;
  if (!force_cooperative()) {
    switch (p.dtype) {
      case 0: moe_dedup_combine_kernel<__half><<<grid, kThreads, smem, stream>>>(p); break;
      case 1: moe_dedup_combine_kernel<__nv_bfloat16><<<grid, kThreads, smem, stream>>>(p); break;
      case 2: moe_dedup_combine_kernel<float><<<grid, kThreads, smem, stream>>>(p); break;
      default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
  }
  MoeDedupCombineParams params = p;
  void* args[] = {&params};
  const void* kernel = nullptr;
  switch (p.dtype) {
    case 0: kernel = (const void*)moe_dedup_combine_kernel<__half>; break;
    case 1: kernel = (const void*)moe_dedup_combine_kernel<__nv_bfloat16>; break;
    case 2: kernel = (const void*)moe_dedup_combine_kernel<float>; break;
    default: return cudaErrorInvalidValue;
  }
  return cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(kThreads), args, smem, stream);
}

}  // namespace b200
