// Fused GEMM + reduce-scatter kernel for sm_100a (see gemm_rs.h for the capability).
//
// Two schedules share the code: one CTA per 128 x BN tile, or a CTA pair (cluster of two,
// tcgen05 cta_group::2) per 256 x BN tile, where each CTA loads half of the W tile and the
// leader's single MMA instruction feeds both tensor-memory halves.  No load is multicast.
//
// Warp roles inside one persistent CTA (224 threads, one CTA per SM):
//   warp 0        TMA producer: fills a ring of shared-memory stages with A and W tiles
//   warp 1        MMA issuer: one lane issues tcgen05.mma, accumulating in tensor memory;
//                 also owns the tensor-memory allocation
//   warps 2..5    epilogue: tcgen05.ld the accumulator, round to bf16, transpose through a
//                 double-buffered, 128-byte-swizzled shared-memory slab, then either TMA-store
//                 the rows into the owner's staging block (peer memory; asynchronous, so NVLink
//                 back-pressure never stalls the warp) or store them per lane as whole
//                 256-byte row segments (direct output, mixed-ownership tiles, fp32 slices)
//   warp 6        signaller: after a tile's rows are stored, fences once and bumps the
//                 owners' arrival counters, keeping that latency off the epilogue warps
//   warps 7..10   reducers: from the start of the kernel they take this rank's staged output
//                 units (a 32-row quarter of a tile, or a whole tile) in the order in which
//                 they complete, wait (bounded) until all partials of a unit have arrived, add
//                 them in rank order in fp32 and write the result -- while the other warps,
//                 and the other SMs, still multiply.  When a CTA's GEMM tiles are done its
//                 seven other warps join them.
// A rank's own rows are finished either in the epilogue of its own tiles (peers' staged rows
// added there; default up to 4 ranks) or by the reducers; tiles that straddle an ownership
// boundary and K-sliced problems always go to the reducers.
//
// Staging buffers and counters exist in two parities that calls alternate between.  A rank
// reaches call n+2 only after it received every peer's partials of call n+1, so every peer
// has started call n+1 and hence finished reading parity n%2: no barrier between calls.
//
// Every wait (mbarrier or peer counter) is bounded; on expiry the kernel records a status,
// lets copies in flight land, frees tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <cstring>

#include "gemm_rs.h"
#include "signal.cuh"
#include "sm100_ptx.cuh"

namespace b200 {

namespace {

constexpr int BM = kGemmRsBlockM;  // 128: one TMEM lane per output row
constexpr int BK = kGemmRsBlockK;  // 64 bf16 = one 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int kMainThreads = 224;  // producer, MMA issuer, 4 epilogue warps, signaller
constexpr int kReducerWarps = 4;
constexpr int kThreads = kMainThreads + 32 * kReducerWarps;
constexpr int kEpilogueWarps = 4;
constexpr int kSmemLimit = 232448;  // 227 KiB opt-in maximum per CTA

// BN: tile width.  CTAS: 1 = one CTA per 128 x BN tile; 2 = a CTA pair (cluster of two) owns a
// 256 x BN tile: each CTA loads its own 128 rows of A and HALF of the W tile, the leader
// issues one M=256 MMA for both, and each CTA's tensor memory receives its 128 rows.
template <int BN, int CTAS>
struct Cfg {
  static constexpr int kABytes = BM * BK * 2;           // 16 KiB
  static constexpr int kBRows = BN / CTAS;              // W rows this CTA loads per stage
  static constexpr int kBBytes = kBRows * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTxBytes = CTAS * kStageBytes;   // bytes counted on the (leader's) full barrier
  static constexpr int kEpiCols = (BN % 128 == 0) ? 128 : 64;  // columns transposed at a time
  static constexpr int kSlabBytes = 32 * kEpiCols * 2;  // one transpose buffer of an epilogue warp:
                                                        // kEpiCols / 64 sub-slabs of 32 rows x 128 bytes
  static constexpr int kSlabBuffers = 2;                // filled alternately; TMA drains one while the other fills
  static constexpr int kEpiBytes = kEpilogueWarps * kSlabBuffers * kSlabBytes;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kStagesRaw = (kSmemLimit - 1024 - kEpiBytes - kBarrierBytes) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kEpiBytes + kBarrierBytes;
  static constexpr int kAccStride = BN <= 64 ? 64 : (BN <= 128 ? 128 : 256);  // TMEM columns per accumulator
  static constexpr int kTmemCols = 2 * kAccStride;                             // two accumulators; power of two
  static_assert(CTAS == 1 || CTAS == 2, "one CTA or a CTA pair");
  static_assert(kStages >= 3, "pipeline too shallow");
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "TMEM columns must be a power of two <= 512");
  static_assert(kBRows % 8 == 0 && kBRows <= 256, "W box rows");
  static_assert(BN % kEpiCols == 0 && BN % 16 == 0 && BN <= 256, "tile width");
};

struct KernelParams {
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;
  int M, N, K, world_size, rank;
  int rows_per_rank;
  int m_tiles, n_tiles, num_kb;  // m_tiles counts 128-row blocks
  int m_groups;  // row groups of 128 * CTAS rows: the scheduling unit along M
  int m_start;   // first row group of the rotated order (the one after this rank's rows)
  int band;      // row groups visited together, column tile by column tile, so that concurrently
                 // running tiles share A and W tiles in L2
  int splits;    // K is cut into this many slices per tile; each slice is one work item whose
                 // bf16 partial is staged like a rank's partial ("virtual ranks")
  int kb_per_split;
  float bias_scale;
  int bias_at_source;  // 1: every rank adds the bias to its rounded partial (the reference's order of operations)
  uint64_t peer_base[kMaxWorldSize];
  uint64_t off_stage, off_counters;
  uint64_t epoch, timeout_ns;
  StatusBlock* status;
  uint64_t* trace;  // optional [gridDim.x][8] globaltimer stamps: 0 start, 1 pipeline ready, 2 GEMM tiles done,
                    // 3 exit; with own tiles finished in the epilogue: 4 first own tile reached, 5 its peers'
                    // rows arrived, 6 last own tile stored; else, for the first epilogue warp once it has
                    // joined the reducers: 5 its first unit complete, 6 its last unit reduced
  int debug;        // measurement aids (results are wrong when set): 1 = stage into this GPU's own memory
                    // instead of the owner's, 2 = skip the staging stores
  int fuse_own;     // 1: a rank finishes its own tiles in their epilogue (adds the peers' rows there);
                    // 0: it stages them like everybody else and all CTAs reduce after the GEMM tiles
  int direct;       // 1: one rank, K not sliced: tiles are written straight to `out`, nothing is staged
  int tma_store;    // 1: whole 32-row groups go to one owner and there are tensor maps for every owner:
                    // staged tiles leave through TMA stores instead of per-lane stores
  int nvls;         // 1: every rank stages ALL its partial tiles in its own multicast-bound memory (layout
                    // [M][N]); owners pull the sum through NVSwitch with multimem.ld_reduce
  uint64_t nvls_local, nvls_mc;  // this parity's staging: own memory, and the multicast address
  int checked;      // 1: every staging store first proves that its owner and byte range lie inside the
                    // staging region of one parity; a violation is recorded (STATUS_BAD_INDEX) and skipped
  uint64_t stage_capacity;  // bytes of one parity's staging region
};

constexpr int kMaxStageMaps = 8;
struct StageMaps {
  CUtensorMap m[kMaxStageMaps];  // m[o]: rank o's staging block for partials coming from this rank, bf16 [R, N]
};

__device__ __forceinline__ void trace_stamp(const KernelParams& p, int slot) {
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[(size_t)blockIdx.x * 8 + slot] = global_timer_ns();
}
__device__ __forceinline__ void trace_stamp_any(const KernelParams& p, int slot, bool first_only) {
  if (p.trace == nullptr) return;
  uint64_t* w = p.trace + (size_t)blockIdx.x * 8 + slot;
  if (first_only && *w != 0) return;
  *w = global_timer_ns();
}

struct PipeState {
  uint32_t stage = 0, phase = 0;
  __device__ __forceinline__ void advance(uint32_t n) {
    if (++stage == n) {
      stage = 0;
      phase ^= 1;
    }
  }
};

// Bounded mbarrier wait.  Returns false (and raises *abort) when the limit expires or
// another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort, uint64_t limit_ns,
                                          StatusBlock* st, int detail) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((++spins & 255u) == 0) {
      if (*abort) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        record_status(st, STATUS_TIMEOUT, PHASE_GEMM_PIPELINE, -1, detail, 0, parity);
        *abort = 1;
        return false;
      }
    }
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Work item t of this CTA (pair): K slice, row group (rotated so the rank's own rows come
// last, visited in bands) and column tile; `mb` is the 128-row block this CTA computes.
template <int CTAS>
__device__ __forceinline__ void tile_coords(const KernelParams& p, int t, uint32_t cta_rank, int& mb, int& nb,
                                            int& split) {
  const int tile = t / p.splits;
  split = t - tile * p.splits;
  const int per_band = p.band * p.n_tiles;
  const int b = tile / per_band;
  const int start = b * p.band;
  const int size = min(p.band, p.m_groups - start);
  const int within = tile - start * p.n_tiles;
  nb = within / size;
  int mg = p.m_start + start + (within - nb * size);
  if (mg >= p.m_groups) mg -= p.m_groups;
  mb = mg * CTAS + (int)cta_rank;
}

// True when every row of m-tile `mb` belongs to this rank (and lies inside M) and K is not
// sliced: such a tile is finished in the epilogue of the rank itself.
__device__ __forceinline__ bool tile_owned(const KernelParams& p, int mb) {
  const int lo = mb * BM;
  const int row_lo = p.rank * p.rows_per_rank;
  return p.fuse_own && p.splits == 1 && lo >= row_lo && lo + BM <= row_lo + p.rows_per_rank && lo + BM <= p.M;
}

// For two output vectors out[rl[u], nn[u]..+8): sum of the world_size bf16 partial vectors in
// rank order, in fp32, plus the bias, rounded once.  This rank's own partials come from
// registers (`own`), the peers' from the staging buffer; all 2 x (world - 1) loads are
// issued before the first use.
__device__ __forceinline__ void reduce_partials2(const KernelParams& p, const __nv_bfloat16* stage, const int (&rl)[2],
                                                 const int (&nn)[2], const bool (&live)[2], const uint4 (&own)[2],
                                                 uint4 (&res)[2]) {
  const size_t R = (size_t)p.rows_per_rank;
  float acc[2][8];
#pragma unroll
  for (int u = 0; u < 2; ++u)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
  for (int s0 = 0; s0 < p.world_size; s0 += 8) {
    uint4 vals[2][8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int s = s0 + k;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (s < p.world_size && s != p.rank && live[u]) {
          vals[u][k] = __ldcg(reinterpret_cast<const uint4*>(stage + ((size_t)s * R + rl[u]) * p.N + nn[u]));
        } else {
          vals[u][k] = (s == p.rank) ? own[u] : make_uint4(0, 0, 0, 0);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&vals[u][k]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          acc[u][2 * e] += f.x;
          acc[u][2 * e + 1] += f.y;
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    if (p.bias != nullptr && !p.bias_at_source && live[u]) {
      const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + nn[u]);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[u][2 * e] = fmaf(f.x, p.bias_scale, acc[u][2 * e]);
        acc[u][2 * e + 1] = fmaf(f.y, p.bias_scale, acc[u][2 * e + 1]);
      }
    }
    res[u].x = pack_bf16x2(acc[u][0], acc[u][1]);
    res[u].y = pack_bf16x2(acc[u][2], acc[u][3]);
    res[u].z = pack_bf16x2(acc[u][4], acc[u][5]);
    res[u].w = pack_bf16x2(acc[u][6], acc[u][7]);
  }
}

// One warp reduces the 16-byte output vectors [item_lo, items) of the block rows [r0, ...) x
// columns [c0, c0 + 8 * vec_per_row) (vectors numbered row by row).  Every lane keeps 4 vectors of 4 sources in flight (the
// reduction is latency-bound otherwise), adds sources in (virtual) rank order in fp32 and
// rounds once.
__device__ __forceinline__ void reduce_block(const KernelParams& p, const __nv_bfloat16* stage, int r0, int row_lo,
                                             int c0, int vec_per_row, int item_lo, int items, int lane) {
  constexpr int U = 4;
  constexpr int S = 4;
  const size_t R = (size_t)p.rows_per_rank;
  const size_t src_stride = R * p.N;
  const int sources = p.world_size * p.splits;
  for (int base = item_lo + lane; base < items; base += 32 * U) {
    float acc[U][8];
    size_t off[U];  // element offset of the vector inside one source's [R, N] block; ~0 = past the end
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + u * 32;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
      if (i < items) {
        const int rl = r0 + i / vec_per_row - row_lo;
        const int n = c0 + ((i % vec_per_row) << 3);
        off[u] = (size_t)rl * p.N + n;
      } else {
        off[u] = ~(size_t)0;
      }
    }
    for (int s = 0; s < sources; s += S) {
      uint4 v[S][U];
#pragma unroll
      for (int q = 0; q < S; ++q) {
        const bool have = s + q < sources;
        const __nv_bfloat16* src = stage + (size_t)(s + q) * src_stride;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          v[q][u] = (have && off[u] != ~(size_t)0) ? __ldcg(reinterpret_cast<const uint4*>(src + off[u]))
                                                   : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int q = 0; q < S; ++q) {  // ascending (virtual) rank
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[q][u]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            acc[u][2 * e] += f.x;
            acc[u][2 * e + 1] += f.y;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (off[u] == ~(size_t)0) continue;
      if (p.bias != nullptr && !p.bias_at_source) {
        const int n = (int)(off[u] % (size_t)p.N);
        const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + n);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          acc[u][2 * e] = fmaf(f.x, p.bias_scale, acc[u][2 * e]);
          acc[u][2 * e + 1] = fmaf(f.y, p.bias_scale, acc[u][2 * e + 1]);
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[u][0], acc[u][1]);
      o.y = pack_bf16x2(acc[u][2], acc[u][3]);
      o.z = pack_bf16x2(acc[u][4], acc[u][5]);
      o.w = pack_bf16x2(acc[u][6], acc[u][7]);
      *reinterpret_cast<uint4*>(p.out + off[u]) = o;
    }
  }
}

// NVLS form: the partials of all ranks sit at the same offset of their own multicast-bound
// staging ([M][N] bf16); one multimem.ld_reduce per 16 bytes returns their sum, formed in fp32
// inside the switch and rounded once.  A bias that is added once goes on top (second rounding).
__device__ __forceinline__ void reduce_block_nvls(const KernelParams& p, int r0, int row_lo, int c0, int vec_per_row,
                                                  int item_lo, int items, int lane) {
  constexpr int U = 4;
  const __nv_bfloat16* mc = reinterpret_cast<const __nv_bfloat16*>(p.nvls_mc);
  for (int base = item_lo + lane; base < items; base += 32 * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + u * 32;
      if (i < items) {
        const size_t off = (size_t)(r0 + i / vec_per_row) * p.N + c0 + ((i % vec_per_row) << 3);
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                     : "l"(mc + off)
                     : "memory");
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + u * 32;
      if (i >= items) continue;
      const int m = r0 + i / vec_per_row;
      const int n = c0 + ((i % vec_per_row) << 3);
      uint4 o = v[u];
      if (p.bias != nullptr && !p.bias_at_source) {
        const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + n);
        const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&bv);
        const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
        uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 fb = __bfloat1622float2(hb[e]);
          const float2 fv = __bfloat1622float2(hv[e]);
          po[e] = pack_bf16x2(fmaf(fb.x, p.bias_scale, fv.x), fmaf(fb.y, p.bias_scale, fv.y));
        }
      }
      *reinterpret_cast<uint4*>(p.out + (size_t)(m - row_lo) * p.N + n) = o;
    }
  }
}

// Same for a K-sliced problem, whose staging holds fp32 slices [world * splits][R][N].  The
// slices of one rank are summed in fp32 and rounded to bf16 -- that is the rank's matmul
// output in the reference -- the bias is added per rank in bf16 if the reference order was
// asked for, and the ranks are then summed in fp32 and rounded once.
__device__ __forceinline__ void reduce_block_sliced(const KernelParams& p, const float* stage, int r0, int row_lo,
                                                    int c0, int vec_per_row, int item_lo, int items, int lane) {
  constexpr int U = 2;
  const size_t R = (size_t)p.rows_per_rank;
  for (int base = item_lo + lane; base < items; base += 32 * U) {
    float acc[U][8];
    size_t off[U];
    float bias_f[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + u * 32;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        acc[u][e] = 0.f;
        bias_f[u][e] = 0.f;
      }
      off[u] = ~(size_t)0;
      if (i < items) {
        const int rl = r0 + i / vec_per_row - row_lo;
        const int n = c0 + ((i % vec_per_row) << 3);
        off[u] = (size_t)rl * p.N + n;
        if (p.bias != nullptr) {
          const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + n);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            bias_f[u][2 * e] = f.x;
            bias_f[u][2 * e + 1] = f.y;
          }
        }
      }
    }
    for (int r = 0; r < p.world_size; ++r) {
      float part[U][8];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int e = 0; e < 8; ++e) part[u][e] = 0.f;
      for (int sl = 0; sl < p.splits; sl += 2) {
        const float* src0 = stage + (size_t)(r * p.splits + sl) * R * p.N;
        const float* src1 = src0 + R * p.N;
        const bool two = sl + 1 < p.splits;
        uint4 lo0[U], hi0[U], lo1[U], hi1[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const bool live = off[u] != ~(size_t)0;
          lo0[u] = live ? __ldcg(reinterpret_cast<const uint4*>(src0 + off[u])) : make_uint4(0, 0, 0, 0);
          hi0[u] = live ? __ldcg(reinterpret_cast<const uint4*>(src0 + off[u] + 4)) : make_uint4(0, 0, 0, 0);
          lo1[u] = (live && two) ? __ldcg(reinterpret_cast<const uint4*>(src1 + off[u])) : make_uint4(0, 0, 0, 0);
          hi1[u] = (live && two) ? __ldcg(reinterpret_cast<const uint4*>(src1 + off[u] + 4)) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          part[u][0] = (part[u][0] + __uint_as_float(lo0[u].x)) + __uint_as_float(lo1[u].x);
          part[u][1] = (part[u][1] + __uint_as_float(lo0[u].y)) + __uint_as_float(lo1[u].y);
          part[u][2] = (part[u][2] + __uint_as_float(lo0[u].z)) + __uint_as_float(lo1[u].z);
          part[u][3] = (part[u][3] + __uint_as_float(lo0[u].w)) + __uint_as_float(lo1[u].w);
          part[u][4] = (part[u][4] + __uint_as_float(hi0[u].x)) + __uint_as_float(hi1[u].x);
          part[u][5] = (part[u][5] + __uint_as_float(hi0[u].y)) + __uint_as_float(hi1[u].y);
          part[u][6] = (part[u][6] + __uint_as_float(hi0[u].z)) + __uint_as_float(hi1[u].z);
          part[u][7] = (part[u][7] + __uint_as_float(hi0[u].w)) + __uint_as_float(hi1[u].w);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float v = __bfloat162float(__float2bfloat16_rn(part[u][e]));
          if (p.bias_at_source) v = __bfloat162float(__float2bfloat16_rn(v + bias_f[u][e]));
          acc[u][e] += v;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (off[u] == ~(size_t)0) continue;
      if (!p.bias_at_source) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[u][e] = fmaf(bias_f[u][e], p.bias_scale, acc[u][e]);
      }
      uint4 o;
      o.x = pack_bf16x2(acc[u][0], acc[u][1]);
      o.y = pack_bf16x2(acc[u][2], acc[u][3]);
      o.z = pack_bf16x2(acc[u][4], acc[u][5]);
      o.w = pack_bf16x2(acc[u][6], acc[u][7]);
      *reinterpret_cast<uint4*>(p.out + off[u]) = o;
    }
  }
}

// The reduction of this rank's staged output, shared by the reducer warps (from the start of
// the kernel) and by the other warps (once their GEMM tiles are done).  Units are numbered in
// the order in which they complete -- column tile by column tile over the rank's row blocks,
// as the tile schedule visits them -- and dealt to the CTAs round robin; inside a CTA a
// shared counter hands the next unit to whichever warp asks, and that warp waits (bounded)
// for the unit's arrival counters before it reduces.  Tiles that straddle an ownership
// boundary (always the case when a rank owns fewer than 128 rows) and all tiles of a K-sliced
// problem were staged by every (virtual) rank, this one included.
template <int BN>
__device__ __forceinline__ void reduce_staged_units(const KernelParams& p, int* next_unit, volatile int* abort, int lane,
                                                    bool stamps) {
  const int G = gridDim.x;
  const int R = p.rows_per_rank;
  const int row_lo = p.rank * R;
  const int mb_lo = row_lo / BM;
  const int mb_hi = (row_lo + R - 1) / BM;
  // staged row blocks: all of [mb_lo, mb_hi], or only its (at most two) partly owned ends
  const bool lo_staged = !tile_owned(p, mb_lo);
  const bool hi_staged = mb_hi != mb_lo && !tile_owned(p, mb_hi);
  const bool all_staged = !(p.fuse_own && p.splits == 1);
  const int n_mb = all_staged ? (mb_hi - mb_lo + 1) : ((lo_staged ? 1 : 0) + (hi_staged ? 1 : 0));
  if (n_mb == 0) return;
  // Unit of work: a whole 128 x BN tile (four counters) when there are plenty of tiles, else one
  // 32-row quarter of a tile (one counter) so that a small problem still occupies every CTA.
  const int parts = (n_mb * p.n_tiles >= 2 * G) ? 1 : kEpilogueWarps;
  const int rows_per_part = BM / parts;
  const int ctrs_per_part = kEpilogueWarps / parts;
  const int total_units = p.n_tiles * n_mb * parts;
  // A unit is cut further into `cuts` runs of its output vectors when there are fewer units than
  // warps: one warp on a whole unit is a long chain of dependent loads, and the last units to
  // complete decide when the kernel ends.
  const int unit_items = rows_per_part * (BN / 8);
  int cuts = (2 * G * (kThreads / 32) + total_units - 1) / total_units;
  cuts = max(1, min(min(cuts, unit_items / 128), 16));
  const int cut_items = (unit_items + cuts - 1) / cuts;
  const long long total_work = (long long)total_units * cuts;
  const uint32_t want = (uint32_t)(p.world_size * p.splits);
  uint32_t* counters = peer_ptr<uint32_t>(p.peer_base[p.rank], p.off_counters);
  const __nv_bfloat16* stage = peer_ptr<const __nv_bfloat16>(p.peer_base[p.rank], p.off_stage);
  const int first = G - 1 - (int)blockIdx.x;  // CTAs with fewer GEMM tiles get the earlier units
  while (!*abort) {
    int li = 0;
    if (lane == 0) li = atomicAdd(next_unit, 1);
    li = __shfl_sync(0xffffffffu, li, 0);
    const long long j = (long long)first + (long long)li * G;
    if (j >= total_work) break;
    const int cut = (int)(j % cuts);
    const int unit = (int)(j / cuts);
    const int part = unit % parts;
    const int rest = unit / parts;
    const int mi = rest % n_mb;
    const int nb = rest / n_mb;
    const int mb = all_staged ? mb_lo + mi : ((mi == 0 && lo_staged) ? mb_lo : mb_hi);
    uint32_t* ctr = counters + ((size_t)mb * p.n_tiles + nb) * kEpilogueWarps + part * ctrs_per_part;
    int ok = 1;
    if (lane < ctrs_per_part) {
      // long sleeps: this wait can last for most of the kernel and must not steal issue slots
      // from the warps that feed the tensor cores
      const uint32_t* c = ctr + lane;
      const bool sys = p.world_size > 1;
      uint32_t seen = sys ? ld_acquire_sys_u32(c) : ld_acquire_gpu_u32(c);
      if (seen < want) {
        const uint64_t t0 = global_timer_ns();
        while (true) {
          __nanosleep(400);
          seen = sys ? ld_acquire_sys_u32(c) : ld_acquire_gpu_u32(c);
          if (seen >= want) break;
          if (*abort || global_timer_ns() - t0 > p.timeout_ns) {
            if (!*abort) record_status(p.status, STATUS_TIMEOUT, PHASE_RS_PARTIALS, -1, mb * p.n_tiles + nb, want, seen);
            *abort = 1;
            ok = 0;
            break;
          }
        }
      }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    if (stamps && lane == 0) trace_stamp_any(p, 5, true);  // first unit of this warp is complete
    const int r0 = max(mb * BM + part * rows_per_part, row_lo);
    const int r1 = min(min(mb * BM + (part + 1) * rows_per_part, row_lo + R), p.M);
    if (r1 > r0) {
      const int c0 = nb * BN;
      const int c1 = min(c0 + BN, p.N);
      const int vec_per_row = (c1 - c0) >> 3;
      const int items = (r1 - r0) * vec_per_row;
      const int lo = cut * cut_items;
      const int hi = min(items, lo + cut_items);
      if (lo < hi) {
        if (p.nvls) reduce_block_nvls(p, r0, row_lo, c0, vec_per_row, lo, hi, lane);
        else if (p.splits > 1) reduce_block_sliced(p, reinterpret_cast<const float*>(stage), r0, row_lo, c0, vec_per_row, lo, hi, lane);
        else reduce_block(p, stage, r0, row_lo, c0, vec_per_row, lo, hi, lane);
      }
    }
    __syncwarp();
    if (lane < ctrs_per_part) {
      // Every cut of the unit adds one to its counters when it is done; the one that sees all the
      // others' marks zeroes them (this parity's counters are next used two calls from now).
      const uint32_t old = atomicAdd(ctr + lane, 1u);
      if (old == want + (uint32_t)cuts - 1u) ctr[lane] = 0;
    }
    if (stamps && lane == 0) trace_stamp_any(p, 6, false);  // latest unit this warp has finished
  }
}

}  // namespace

template <int BN, int CTAS>
__global__ void __launch_bounds__(kThreads, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const __grid_constant__ StageMaps stage_maps, const KernelParams p) {
  using C = Cfg<BN, CTAS>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int abort_flag;
  __shared__ uint32_t tmem_base_shared;
  __shared__ int next_unit_shared;  // next reduction unit of this CTA to hand out

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  trace_stamp(p, 0);
  const uint32_t cta_rank = CTAS == 2 ? ptx::cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;

  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_a0 = smem_base;                              // stage s: + s * kStageBytes
  const uint32_t smem_epi = smem_base + C::kStages * C::kStageBytes;
  const uint32_t bar_base = smem_epi + C::kEpiBytes;
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (C::kStages + s); };
  auto tfull_bar = [&](uint32_t s) { return bar_base + 8u * (2 * C::kStages + s); };
  auto tempty_bar = [&](uint32_t s) { return bar_base + 8u * (2 * C::kStages + 2 + s); };
  auto sfull_bar = [&](uint32_t s) { return bar_base + 8u * (2 * C::kStages + 4 + s); };   // tile stored by all 4 warps
  auto sempty_bar = [&](uint32_t s) { return bar_base + 8u * (2 * C::kStages + 6 + s); };  // signaller took it

  if (tid == 0) {
    abort_flag = 0;
    next_unit_shared = 0;
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);   // one arrive (with the byte count) per phase, by the leader's producer
      ptx::mbar_init(empty_bar(s), 1);  // one commit per phase, by the MMA issuer (to both CTAs of a pair)
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(tfull_bar(s), 1);
      ptx::mbar_init(tempty_bar(s), kEpilogueWarps * CTAS);  // every epilogue warp of the pair
      ptx::mbar_init(sfull_bar(s), kEpilogueWarps);
      ptx::mbar_init(sempty_bar(s), 1);
    }
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&tma_a);
    ptx::prefetch_tensormap(&tma_b);
  }
  if (warp == 1) {
    if (CTAS == 2) {
      ptx::tmem_alloc_pair(ptx::smem_u32(&tmem_base_shared), C::kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(&tmem_base_shared), C::kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  if (CTAS == 2) ptx::cluster_sync_all();  // the peer's barriers exist before anything signals them
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_shared;
  trace_stamp(p, 1);

  const int total_tiles = p.m_groups * p.n_tiles * p.splits;
  const int G = gridDim.x;              // CTAs
  const int GG = G / CTAS;              // CTAs or CTA pairs: the schedulers
  const int gidx = (int)blockIdx.x / CTAS;
  const uint64_t limit = p.timeout_ns;

  if (warp == 0) {
    // ================================ TMA producer =====================================
    // Runs in every CTA: its own 128 rows of A and its share of the W tile.
    if (lane == 0) {
      PipeState ps;
      for (int t = gidx; t < total_tiles && !abort_flag; t += GG) {
        int mb, nb, split;
        tile_coords<CTAS>(p, t, cta_rank, mb, nb, split);
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(ps.stage), ps.phase ^ 1u, &abort_flag, limit, p.status, 100 + (int)ps.stage)) break;
          const uint32_t sa = smem_a0 + ps.stage * C::kStageBytes;
          const uint32_t sb = sa + C::kABytes;
          if (CTAS == 2) {
            if (leader) ptx::mbar_arrive_expect_tx(full_bar(ps.stage), C::kTxBytes);
            ptx::tma_load_2d_pair(sa, &tma_a, full_bar(ps.stage), kb * BK, mb * BM);
            ptx::tma_load_2d_pair(sb, &tma_b, full_bar(ps.stage), kb * BK, nb * BN + (int)cta_rank * C::kBRows);
          } else {
            ptx::mbar_arrive_expect_tx(full_bar(ps.stage), C::kTxBytes);
            ptx::tma_load_2d(sa, &tma_a, full_bar(ps.stage), kb * BK, mb * BM);
            ptx::tma_load_2d(sb, &tma_b, full_bar(ps.stage), kb * BK, nb * BN);
          }
          ps.advance(C::kStages);
        }
      }
    }
  } else if (warp == 1) {
    // ================================ MMA issuer =======================================
    // One lane of the (leader) CTA; in a pair the same instruction drives both CTAs.
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = ptx::make_idesc_bf16_f32(BM * CTAS, BN);
      PipeState ps;
      uint32_t it = 0;
      for (int t = gidx; t < total_tiles && !abort_flag; t += GG, ++it) {
        const uint32_t acc = it & 1u;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, &abort_flag, limit, p.status, 200 + (int)acc)) break;
        ptx::tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * C::kAccStride;
        const int split = t % p.splits;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(ps.stage), ps.phase, &abort_flag, limit, p.status, 300 + (int)ps.stage)) {
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after();
          const uint32_t sa = smem_a0 + ps.stage * C::kStageBytes;
          const uint32_t sb = sa + C::kABytes;
          const uint64_t da = ptx::make_smem_desc_k_sw128(sa);
          const uint64_t db = ptx::make_smem_desc_k_sw128(sb);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j) {
            // advancing K by 16 bf16 = 32 bytes = 2 descriptor address units
            if (CTAS == 2) ptx::umma_bf16_pair(tmem_d, da + 2u * j, db + 2u * j, idesc, (kb > kb0 || j > 0) ? 1u : 0u);
            else ptx::umma_bf16(tmem_d, da + 2u * j, db + 2u * j, idesc, (kb > kb0 || j > 0) ? 1u : 0u);
          }
          // stage reusable (in both CTAs of a pair) once these MMAs have read it
          if (CTAS == 2) ptx::umma_commit_pair(empty_bar(ps.stage), 3);
          else ptx::umma_commit(empty_bar(ps.stage));
          ps.advance(C::kStages);
        }
        if (!ok) break;
        // accumulator complete: wake the epilogue warps (of both CTAs)
        if (CTAS == 2) ptx::umma_commit_pair(tfull_bar(acc), 3);
        else ptx::umma_commit(tfull_bar(acc));
      }
    }
  } else if (warp < 6) {
    // ================================ epilogue =========================================
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const uint32_t slab0 = smem_epi + (uint32_t)(warp - 2) * (C::kSlabBuffers * C::kSlabBytes);
    constexpr int kChunksPerRow = C::kEpiCols / 8;       // 16-byte chunks per tile row held in a buffer
    constexpr int kRowsPerStore = 32 / kChunksPerRow;    // rows covered by one warp store
    constexpr int kSubBytes = 32 * 128;                  // one sub-slab: 32 rows x 128 bytes, 128B-swizzled
    // 16-byte chunk `chunk` of row `row`: sub-slab chunk / 8, position (chunk % 8) ^ (row % 8).
    // This is the layout a 128-byte-swizzled TMA box {64 bf16, 32 rows} expects.
    auto slab_addr = [&](uint32_t buf, int row, int chunk) {
      return buf + (uint32_t)(chunk >> 3) * kSubBytes + (uint32_t)row * 128u + (uint32_t)(((chunk & 7) ^ (row & 7)) << 4);
    };
    uint32_t pass_count = 0;
    const bool direct = p.direct != 0;
    const bool sliced = p.splits > 1;
    const int R = p.rows_per_rank;
    const int row_lo = p.rank * R;
    uint32_t* my_counters = peer_ptr<uint32_t>(p.peer_base[p.rank], p.off_counters);
    const __nv_bfloat16* my_stage = peer_ptr<const __nv_bfloat16>(p.peer_base[p.rank], p.off_stage);
    uint32_t it = 0;
    for (int t = gidx; t < total_tiles && !abort_flag; t += GG, ++it) {
      int mb, nb, split;
      tile_coords<CTAS>(p, t, cta_rank, mb, nb, split);
      const uint32_t acc = it & 1u;
      const uint32_t acc_phase = (it >> 1) & 1u;
      if (!mbar_wait(tfull_bar(acc), acc_phase, &abort_flag, limit, p.status, 400 + (int)acc)) break;
      ptx::tcgen05_fence_after();
      const int m0 = mb * BM + q * 32;
      const int n0 = nb * BN;
      // A tile whose rows all belong to this rank is finished here: the peers' partial rows
      // are added in the store loop and the result goes straight to `out`.
      const bool owned = !direct && tile_owned(p, mb);
      const size_t ctr_index = ((size_t)mb * p.n_tiles + nb) * kEpilogueWarps + q;
      bool peers_ok = true;
      // One pass fills the warp's slab (32 rows x kEpiCols * 2 bytes): kEpiCols bf16 columns,
      // or half as many fp32 columns for a K-sliced problem (staged un-rounded).
      const int cols_per_pass = sliced ? C::kEpiCols / 2 : C::kEpiCols;
      const int passes = BN / cols_per_pass;
      // Whole 32-row groups of a staged tile leave through TMA stores (asynchronous, so NVLink
      // back-pressure never blocks this warp); everything else takes the per-lane store loop.
      const bool tma_tile = p.tma_store && !direct && !owned && !sliced && m0 < p.M;
      const int owner0 = tma_tile ? m0 / R : 0;
#pragma unroll 1
      for (int half = 0; half < passes; ++half, ++pass_count) {
        const uint32_t slab = slab0 + (pass_count & 1u) * C::kSlabBytes;
        // the TMA store that last read this buffer (two passes ago) must be done with it
        if (lane == 0) ptx::bulk_wait_group_read<1>();
        __syncwarp();
        // ---- TMEM -> registers -> (bf16) -> swizzled slab (row = lane) ------------------
#pragma unroll 1
        for (int c = 0; c < cols_per_pass / 32; ++c) {
          uint32_t v[32];
          const uint32_t taddr =
              tmem_base + ((uint32_t)(q * 32) << 16) + acc * C::kAccStride + half * cols_per_pass + c * 32;
          ptx::tmem_ld_32x32b_x32(taddr, v);
          ptx::tmem_ld_wait();
          if (sliced) {
#pragma unroll
            for (int j8 = 0; j8 < 8; ++j8) {
              const int chunk = c * 8 + j8;  // 16-byte chunk = 4 fp32 columns
              const uint32_t addr = slab_addr(slab, lane, chunk);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v[4 * j8]), "r"(v[4 * j8 + 1]),
                           "r"(v[4 * j8 + 2]), "r"(v[4 * j8 + 3])
                           : "memory");
            }
            continue;
          }
          if (p.bias != nullptr && (direct || p.bias_at_source)) {
            const int nbase = n0 + half * cols_per_pass + c * 32;
            if (p.bias_at_source) {
              // reference order: round the product to bf16, add the bf16 bias, round again
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int n = nbase + j;
                const float b = (n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
                v[j] = __float_as_uint(__bfloat162float(__float2bfloat16_rn(__uint_as_float(v[j]))) + b);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int n = nbase + j;
                const float b = (n < p.N) ? __bfloat162float(p.bias[n]) * p.bias_scale : 0.f;
                v[j] = __float_as_uint(__uint_as_float(v[j]) + b);
              }
            }
          }
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
            uint4 pk;
            pk.x = pack_bf16x2(__uint_as_float(v[8 * j4 + 0]), __uint_as_float(v[8 * j4 + 1]));
            pk.y = pack_bf16x2(__uint_as_float(v[8 * j4 + 2]), __uint_as_float(v[8 * j4 + 3]));
            pk.z = pack_bf16x2(__uint_as_float(v[8 * j4 + 4]), __uint_as_float(v[8 * j4 + 5]));
            pk.w = pack_bf16x2(__uint_as_float(v[8 * j4 + 6]), __uint_as_float(v[8 * j4 + 7]));
            const int chunk = c * 4 + j4;
            const uint32_t addr = slab_addr(slab, lane, chunk);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk.x), "r"(pk.y), "r"(pk.z),
                         "r"(pk.w)
                         : "memory");
          }
        }
        if (half == passes - 1) {
          // all TMEM reads of this accumulator are done: hand it back to the MMA warp
          ptx::tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (CTAS == 2) ptx::mbar_arrive_cluster(tempty_bar(acc), 0);  // the leader's barrier
            else ptx::mbar_arrive(tempty_bar(acc));
          }
        }
        __syncwarp();
        if (owned && half == 0) {
          // Rows q*32..q*32+31 of this tile were stored by warp q of every peer; wait for
          // their world_size - 1 arrivals on this warp's counter.
          int ok = 1;
          if (warp == 2 && lane == 0) trace_stamp_any(p, 4, true);
          if (lane == 0) {
            ok = wait_u32_ge(my_counters + ctr_index, (uint32_t)(p.world_size - 1), limit, p.status, PHASE_RS_PARTIALS,
                             -1, (int)(mb * p.n_tiles + nb), true)
                     ? 1
                     : 0;
          }
          if (warp == 2 && lane == 0) trace_stamp_any(p, 5, true);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          peers_ok = ok != 0;
          if (!peers_ok) abort_flag = 1;
        }
        if (tma_tile) {
          // ---- slab -> owner's staging block, one TMA box per 64 columns -------------------
          ptx::fence_proxy_async_smem();  // this lane's slab writes, for the async proxy
          __syncwarp();
          bool in_range = true;
          if (p.checked && !p.nvls) {
            const long long rl0 = (long long)m0 - (long long)owner0 * R;
            in_range = owner0 >= 0 && owner0 < p.world_size && rl0 >= 0 && rl0 + 32 <= R &&
                       ((uint64_t)(p.rank + 1) * R * p.N * 2ull) <= p.stage_capacity;
            if (!in_range && lane == 0)
              record_status(p.status, STATUS_BAD_INDEX, PHASE_RS_PARTIALS, owner0, (int)(mb * p.n_tiles + nb), p.epoch, (uint64_t)m0);
          }
          if (lane == 0 && p.debug != 2 && in_range) {
            // nvls: one map over this rank's own [M, N] staging; else the owner's block for this rank
            const void* map = &stage_maps.m[p.nvls ? 0 : (p.debug == 1 ? p.rank : owner0)];
            const int y = p.nvls ? m0 : m0 - owner0 * R;
#pragma unroll
            for (int sub = 0; sub < C::kEpiCols / 64; ++sub) {
              const int x = n0 + half * cols_per_pass + sub * 64;
              if (x < p.N) ptx::tma_store_2d(map, slab + sub * kSubBytes, x, y);
            }
            ptx::bulk_commit_group();
          }
          __syncwarp();
          continue;
        }
        if (owned) {
          // ---- own tile: add the peers' staged rows to this rank's partial, two row segments
          // per step so that 2 x (world - 1) loads are in flight per lane ----------------------
          if (peers_ok) {
#pragma unroll 1
            for (int s = 0; s < kChunksPerRow; s += 2) {
              uint4 own[2];
              int rl[2], nn[2];
              bool live[2];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int rr = (s + u) * kRowsPerStore + lane / kChunksPerRow;
                const int cc = lane % kChunksPerRow;
                const uint32_t addr = slab_addr(slab, rr, cc);
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(own[u].x), "=r"(own[u].y), "=r"(own[u].z), "=r"(own[u].w)
                             : "r"(addr));
                rl[u] = m0 + rr - row_lo;
                nn[u] = n0 + half * cols_per_pass + cc * 8;
                live[u] = (m0 + rr < p.M) && (nn[u] < p.N);
              }
              uint4 res[2];
              reduce_partials2(p, my_stage, rl, nn, live, own, res);
#pragma unroll
              for (int u = 0; u < 2; ++u)
                if (live[u]) *reinterpret_cast<uint4*>(p.out + (size_t)rl[u] * p.N + nn[u]) = res[u];
            }
          }
          __syncwarp();
          continue;
        }
        // ---- slab -> global, whole row segments per store ------------------------------
#pragma unroll 2
        for (int s = 0; s < kChunksPerRow; ++s) {
          const int rr = s * kRowsPerStore + lane / kChunksPerRow;
          const int cc = lane % kChunksPerRow;
          const uint32_t addr = slab_addr(slab, rr, cc);
          uint4 val;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                       : "r"(addr)
                       : "memory");
          const int m = m0 + rr;
          const int n = n0 + half * cols_per_pass + cc * (sliced ? 4 : 8);
          if (m < p.M && n < p.N) {
            if (p.nvls && !direct) {
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.nvls_local) + (size_t)m * p.N + n) = val;
              continue;
            }
            if (p.checked && !direct) {
              const int owner = m / R;
              const uint64_t elem = ((uint64_t)(p.rank * p.splits + split) * R + (uint64_t)(m - owner * R)) * p.N + n;
              const uint64_t end = sliced ? (elem + 4) * 4ull : (elem + 8) * 2ull;
              if (owner >= p.world_size || end > p.stage_capacity) {
                record_status(p.status, STATUS_BAD_INDEX, PHASE_RS_PARTIALS, owner, (int)(mb * p.n_tiles + nb), p.epoch, end);
                continue;
              }
            }
            if (sliced) {
              const int owner = m / R;
              const int rl = m - owner * R;
              float* dst = peer_ptr<float>(p.peer_base[owner], p.off_stage) +
                           ((size_t)(p.rank * p.splits + split) * R + rl) * p.N + n;
              *reinterpret_cast<uint4*>(dst) = val;
            } else if (direct) {
              *reinterpret_cast<uint4*>(p.out + (size_t)m * p.N + n) = val;
            } else if (p.debug != 2) {
              const int owner = m / R;
              const int rl = m - owner * R;
              __nv_bfloat16* dst = peer_ptr<__nv_bfloat16>(p.peer_base[p.debug == 1 ? p.rank : owner], p.off_stage) +
                                   ((size_t)(p.rank * p.splits + split) * R + rl) * p.N + n;
              *reinterpret_cast<uint4*>(dst) = val;
            }
          }
        }
        __syncwarp();
      }
      if (owned) {
        if (lane == 0) my_counters[ctr_index] = 0;  // next used by the call after next
        if (warp == 2 && lane == 0) trace_stamp_any(p, 6, false);
      }
      // Hand the stored tile to the signaller warp: it pays for the fence that must precede
      // the arrival counters, so this warp can start on the next accumulator right away.
      if (tma_tile && lane == 0) {
        ptx::bulk_wait_group<0>();  // the tile's TMA stores have been performed
        asm volatile("fence.proxy.async.global;" ::: "memory");  // order them before the generic-proxy signal
      }
      __syncwarp();
      if (!direct && lane == 0) {
        if (mbar_wait(sempty_bar(acc), acc_phase ^ 1u, &abort_flag, limit, p.status, 500 + (int)acc))
          ptx::mbar_arrive(sfull_bar(acc));
      }
      // reconverge: the next tile starts with warp-wide (.sync.aligned) tensor-memory loads
      __syncwarp();
    }
  } else if (warp == 6) {
    // ================================ signaller ========================================
    // For every staged tile: once all four epilogue warps have stored their rows, make the
    // stores visible (one fence for the whole CTA's tile) and bump the owners' counters.
    if (lane == 0 && !p.direct) {
      const int R = p.rows_per_rank;
      uint32_t it = 0;
      for (int t = gidx; t < total_tiles && !abort_flag; t += GG, ++it) {
        int mb, nb, split;
        tile_coords<CTAS>(p, t, cta_rank, mb, nb, split);
        const uint32_t acc = it & 1u;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(sfull_bar(acc), acc_phase, &abort_flag, limit, p.status, 600 + (int)acc)) break;
        if (!tile_owned(p, mb)) {
          const int m_lo = mb * BM;
          const int m_hi = min(p.M, m_lo + BM) - 1;
          const int o_lo = m_lo / R;
          const int o_hi = m_hi / R;
          if (o_lo <= o_hi) {
            // device scope is enough (and much cheaper) when the only owner is this GPU
            if (o_lo == p.rank && o_hi == p.rank && !p.nvls) __threadfence();
            else __threadfence_system();
            const size_t base_index = ((size_t)mb * p.n_tiles + nb) * kEpilogueWarps;
            for (int o = o_lo; o <= o_hi; ++o) {
              uint32_t* ctr = peer_ptr<uint32_t>(p.peer_base[o], p.off_counters) + base_index;
#pragma unroll
              for (int w = 0; w < kEpilogueWarps; ++w) {
                // relaxed: the fence above already orders the tile's stores before these
                if (o == p.rank) red_relaxed_gpu_add(ctr + w, 1u);
                else red_relaxed_sys_add(ctr + w, 1u);
              }
            }
          }
        }
        ptx::mbar_arrive(sempty_bar(acc));
      }
    }
  } else {
    // ================================ reducers ==========================================
    if (!p.direct) reduce_staged_units<BN>(p, &next_unit_shared, &abort_flag, lane, false);
  }

  // ================================ end of the GEMM phase ================================
  if (warp < kMainThreads / 32) {
    if (abort_flag) {
      // give copies still in flight time to land before shared memory is released
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 200000) __nanosleep(1000);
    }
    // the seven GEMM warps meet among themselves (the reducers are still at work) ...
    __syncwarp();
    asm volatile("bar.sync 1, %0;" ::"n"(kMainThreads) : "memory");
    trace_stamp(p, 2);
    // ... and help with what is left of the reduction
    if (!p.direct && !abort_flag) reduce_staged_units<BN>(p, &next_unit_shared, &abort_flag, lane, warp == 2 && !p.fuse_own);
  }

  // ================================ teardown =============================================
  ptx::tcgen05_fence_before();
  __syncthreads();
  // A CTA of a pair must not retire while its partner may still signal its barriers or
  // read its shared memory through the shared MMA.
  if (CTAS == 2) ptx::cluster_sync_all();
  ptx::tcgen05_fence_after();
  if (warp == 1) {
    __syncwarp();
    if (CTAS == 2) ptx::tmem_dealloc_pair(tmem_base, C::kTmemCols);
    else ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
  trace_stamp(p, 3);
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// Row-major bf16 [rows, cols] tensor, box = [box_rows, 64 columns], 128-byte swizzle,
// out-of-range elements read as zero.  Encoded maps are kept in a small per-thread cache:
// a serving loop calls with the same weight (and often the same activation buffer) again
// and again, and the driver call is a visible part of a short launch.
bool make_tensor_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  struct Entry {
    const void* base;
    uint64_t rows, cols;
    uint32_t box_rows;
    CUtensorMap map;
  };
  constexpr int kEntries = 64;
  thread_local Entry cache[kEntries];
  thread_local int used = 0, next = 0;
  for (int i = 0; i < used; ++i) {
    const Entry& e = cache[i];
    if (e.base == base && e.rows == rows && e.cols == cols && e.box_rows == box_rows) {
      *map = e.map;
      return true;
    }
  }
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  Entry& slot = cache[next];
  slot.base = base;
  slot.rows = rows;
  slot.cols = cols;
  slot.box_rows = box_rows;
  slot.map = *map;
  next = (next + 1) % kEntries;
  if (used < kEntries) ++used;
  return true;
}

// Tile shape and K slicing from the problem size.  Cost model: waves of work items times
// the time of one item (proportional to its k-blocks and its width, with a penalty for
// narrow tiles, which use the tensor pipe less well).
GemmRsPlan make_plan(int M, int N, int K, int world_size, int sms, int force_bn, int force_pair, int force_splits) {
  const int m_tiles = (M + BM - 1) / BM;
  const int num_kb = (K + BK - 1) / BK;
  GemmRsPlan best = {};
  double best_cost = 1e300;
  struct Cand { int bn, ctas; double penalty; };
  const Cand cands[] = {{256, 2, 1.0}, {192, 2, 1.06}, {128, 2, 1.5}, {256, 1, 1.18}, {128, 1, 1.55}, {64, 1, 2.9}};
  for (const Cand& c : cands) {
    if (force_bn > 0 && c.bn != force_bn) continue;
    if (force_pair >= 0 && (c.ctas == 2) != (force_pair != 0)) continue;
    const int schedulers = std::max(sms / c.ctas, 1);
    const int tiles = ((m_tiles + c.ctas - 1) / c.ctas) * ((N + c.bn - 1) / c.bn);
    int max_splits = 1;
    // Slices travel as fp32 and cost a fence and a counter per tile and owner: across GPUs they
    // only pay when the problem leaves most of the machine idle.
    const int idle_factor = world_size > 1 ? 4 : 2;
    if (force_splits > 0) max_splits = force_splits;
    else if (tiles * idle_factor <= schedulers) max_splits = std::min(std::min(schedulers / tiles, num_kb / 4), 8);
    for (int sp = (force_splits > 0 ? force_splits : 1); sp <= std::max(max_splits, 1); ++sp) {
      int per = (num_kb + sp - 1) / sp;
      if ((sp - 1) * per >= num_kb) continue;  // an empty slice
      const double waves = std::ceil((double)tiles * sp / schedulers);
      // Item time in units of (k-blocks x columns); 1536 stands for the fixed ramp-up and
      // epilogue of an item, 400 per slice for staging and re-reading the partial tile.
      const double cost = waves * (per * c.bn * c.penalty + 1536.0) + (sp > 1 ? 400.0 * sp : 0.0);
      if (cost < best_cost) {
        best_cost = cost;
        best.block_n = c.bn;
        best.cta_pair = c.ctas == 2 ? 1 : 0;
        best.splits = sp;
      }
    }
  }
  if (best.block_n == 0) {
    best.block_n = force_bn > 0 ? force_bn : 128;
    best.cta_pair = 0;
    best.splits = 1;
  }
  // bf16 partials per rank, or fp32 slices when K is cut
  best.stage_bytes = best.splits > 1 ? (uint64_t)best.splits * (uint64_t)M * (uint64_t)N * 4ull
                                     : (uint64_t)M * (uint64_t)N * 2ull;
  const uint64_t n_tiles = (N + 63) / 64;
  best.counter_bytes = ((uint64_t)m_tiles * n_tiles * kEpilogueWarps * 4 + 255) / 256 * 256;
  (void)world_size;
  return best;
}

template <int BN, int CTAS>
cudaError_t launch_typed(const GemmRsArgs& a, int sms, int splits, cudaStream_t stream) {
  using C = Cfg<BN, CTAS>;
  CUtensorMap map_a, map_b;
  if (!make_tensor_map(&map_a, a.a, (uint64_t)a.M, (uint64_t)a.K, BM)) return cudaErrorInvalidValue;
  if (!make_tensor_map(&map_b, a.w, (uint64_t)a.N, (uint64_t)a.K, C::kBRows)) return cudaErrorInvalidValue;

  KernelParams p;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(a.bias);
  p.out = reinterpret_cast<__nv_bfloat16*>(a.out);
  p.M = a.M;
  p.N = a.N;
  p.K = a.K;
  p.world_size = a.world_size;
  p.rank = a.rank;
  p.rows_per_rank = a.M / a.world_size;
  p.m_tiles = (a.M + BM - 1) / BM;
  p.n_tiles = (a.N + BN - 1) / BN;
  p.num_kb = (a.K + BK - 1) / BK;
  p.m_groups = (p.m_tiles + CTAS - 1) / CTAS;
  // rotated order: start with the first row group wholly after this rank's rows
  const int64_t group_rows = (int64_t)BM * CTAS;
  p.m_start = (int)((((int64_t)(a.rank + 1) * p.rows_per_rank + group_rows - 1) / group_rows) % p.m_groups);
  p.splits = splits;
  p.kb_per_split = (p.num_kb + splits - 1) / splits;
  // bands of up to 8 row groups, never mixing a rank's own rows into a band that starts elsewhere
  const int groups_per_rank = std::max((int)(p.rows_per_rank / group_rows), 1);
  p.band = std::max(1, std::min(std::min(8, groups_per_rank), p.m_groups));
  p.bias_scale = a.bias_scale;
  p.bias_at_source = a.bias_at_source;
  for (int r = 0; r < kMaxWorldSize; ++r) p.peer_base[r] = a.peer_base[r];
  p.off_stage = a.off_stage;
  p.off_counters = a.off_counters;
  p.epoch = a.epoch;
  p.timeout_ns = a.timeout_ns;
  p.status = a.status;
  p.trace = a.trace;
  p.debug = a.debug;
  p.fuse_own = a.fuse_own;
  p.checked = a.checked;
  p.stage_capacity = a.stage_capacity;
  // NVLS: bf16 partials only (K slices travel as fp32 and keep the peer-to-peer path), at least two ranks
  p.nvls = (a.nvls_mc != 0 && a.nvls_local != 0 && a.world_size > 1 && splits == 1) ? 1 : 0;
  p.nvls_local = a.nvls_local;
  p.nvls_mc = a.nvls_mc;
  if (p.nvls) {
    // Everybody visits the tiles in the SAME order (no rotation), so that a tile is complete on all
    // ranks at about the same time and its owner can pull it at once: the transfers spread over the
    // whole run instead of piling up at its end.
    p.m_start = 0;
    p.fuse_own = 0;
  }
  p.direct = (a.world_size == 1 && splits == 1 && !a.force_staged) ? 1 : 0;
  StageMaps maps;
  std::memset(&maps, 0, sizeof(maps));
  p.tma_store = 0;
  if (p.nvls && a.tma_store != 0) {
    p.tma_store = 1;
    if (!make_tensor_map(&maps.m[0], reinterpret_cast<const void*>(a.nvls_local), (uint64_t)a.M, (uint64_t)a.N, 32))
      return cudaErrorInvalidValue;
  } else if (a.world_size <= kMaxStageMaps && splits == 1 && !p.direct && p.rows_per_rank % 32 == 0 && a.tma_store != 0) {
    p.tma_store = 1;
    for (int o = 0; o < a.world_size; ++o) {
      const uint8_t* base = reinterpret_cast<const uint8_t*>(a.peer_base[o]) + a.off_stage +
                            (uint64_t)a.rank * p.rows_per_rank * a.N * 2ull;
      if (!make_tensor_map(&maps.m[o], base, (uint64_t)p.rows_per_rank, (uint64_t)a.N, 32)) return cudaErrorInvalidValue;
    }
  }

  auto kernel = gemm_rs_kernel<BN, CTAS>;
  // Per kernel variant and device, once: opt in to the large dynamic shared memory and ask
  // how many CTA pairs can be resident (both calls are slow enough to matter per launch).
  struct VariantInfo {
    bool ready = false;
    int max_clusters = 0;
  };
  static VariantInfo info[64];
  int dev = 0;
  cudaGetDevice(&dev);
  VariantInfo& vi = info[dev & 63];

  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (!vi.ready) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    vi.max_clusters = sms / CTAS;
    if (CTAS == 2) {
      cfg.gridDim = dim3((unsigned)(sms / CTAS * CTAS));
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess && n > 0) vi.max_clusters = std::min(n, sms / CTAS);
    }
    vi.ready = true;
  }

  const int total = p.m_groups * p.n_tiles * splits;
  int schedulers = std::min(total, vi.max_clusters);  // never more CTAs (pairs) than can be resident at once
  if (a.max_ctas > 0) schedulers = std::min(schedulers, std::max(a.max_ctas / CTAS, 1));
  if (schedulers < 1) schedulers = 1;
  cfg.gridDim = dim3((unsigned)(schedulers * CTAS));
  return cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, maps, p);
}

}  // namespace

GemmRsPlan gemm_rs_plan(int M, int N, int K, int world_size, int block_n, int cta_pair, int splits) {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  return make_plan(M, N, K, world_size, sms, block_n, cta_pair, splits);
}

cudaError_t launch_gemm_rs(const GemmRsArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.world_size < 1 || a.M % a.world_size != 0) return cudaErrorInvalidValue;
  if (a.K % 8 != 0 || a.N % 8 != 0) return cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const GemmRsPlan plan = make_plan(a.M, a.N, a.K, a.world_size, sms, a.block_n, a.cta_pair, a.splits);
  const int sp = plan.splits;
  if (plan.cta_pair) {
    switch (plan.block_n) {
      case 256: return launch_typed<256, 2>(a, sms, sp, stream);
      case 192: return launch_typed<192, 2>(a, sms, sp, stream);
      case 128: return launch_typed<128, 2>(a, sms, sp, stream);
      default: return cudaErrorInvalidValue;
    }
  }
  switch (plan.block_n) {
    case 256: return launch_typed<256, 1>(a, sms, sp, stream);
    case 128: return launch_typed<128, 1>(a, sms, sp, stream);
    case 64: return launch_typed<64, 1>(a, sms, sp, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace b200
