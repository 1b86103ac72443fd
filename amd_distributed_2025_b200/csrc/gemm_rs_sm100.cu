// Fused GEMM + reduce-scatter kernel for sm_100a (see gemm_rs.h for the capability).
//
// Warp roles inside one persistent CTA (192 threads, one CTA per SM):
//   warp 0        TMA producer: fills a ring of shared-memory stages with A and W tiles
//   warp 1        MMA issuer: one lane issues tcgen05.mma, accumulating in tensor memory;
//                 also owns the tensor-memory allocation
//   warps 2..5    epilogue: tcgen05.ld the accumulator, round to bf16, transpose through
//                 shared memory so that every warp store covers whole 256-byte row
//                 segments, store to the owner's staging buffer (peer memory), signal
// After its share of GEMM tiles every CTA joins the reduction of this rank's own rows.
//
// Every wait (mbarrier or peer counter) is bounded; on expiry the kernel records a status,
// lets copies in flight land, frees tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "gemm_rs.h"
#include "signal.cuh"
#include "sm100_ptx.cuh"

namespace b200 {

namespace {

constexpr int BM = kGemmRsBlockM;  // 128: one TMEM lane per output row
constexpr int BK = kGemmRsBlockK;  // 64 bf16 = one 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kEpilogueWarps = 4;
constexpr int kSmemLimit = 232448;  // 227 KiB opt-in maximum per CTA

template <int BN>
struct Cfg {
  static constexpr int kABytes = BM * BK * 2;           // 16 KiB
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiCols = BN < 128 ? BN : 128;  // columns transposed at a time
  static constexpr int kSlabBytes = 32 * kEpiCols * 2;  // per epilogue warp
  static constexpr int kEpiBytes = kEpilogueWarps * kSlabBytes;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kStagesRaw = (kSmemLimit - 1024 - kEpiBytes - kBarrierBytes) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kEpiBytes + kBarrierBytes;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;  // two accumulators; power of two >= 32
  static_assert(kStages >= 3, "pipeline too shallow");
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "TMEM columns must be a power of two <= 512");
};

struct KernelParams {
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;
  int M, N, K, world_size, rank;
  int rows_per_rank;
  int m_tiles, n_tiles, num_kb;
  int m_start;  // first m-tile of the rotated order (the one after this rank's rows)
  float bias_scale;
  uint64_t peer_base[kMaxWorldSize];
  uint64_t off_stage, off_counters;
  uint64_t epoch, timeout_ns;
  StatusBlock* status;
};

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

__device__ __forceinline__ void tile_coords(const KernelParams& p, int t, int& mb, int& nb) {
  const int j = t / p.n_tiles;
  nb = t - j * p.n_tiles;
  mb = p.m_start + j;
  if (mb >= p.m_tiles) mb -= p.m_tiles;
}

}  // namespace

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const KernelParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int abort_flag;
  __shared__ uint32_t tmem_base_shared;
  __shared__ int wait_ok_shared;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t smem_a0 = smem_base;                              // stage s: + s * kStageBytes
  const uint32_t smem_epi = smem_base + C::kStages * C::kStageBytes;
  const uint32_t bar_base = smem_epi + C::kEpiBytes;
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (C::kStages + s); };
  auto tfull_bar = [&](uint32_t s) { return bar_base + 8u * (2 * C::kStages + s); };
  auto tempty_bar = [&](uint32_t s) { return bar_base + 8u * (2 * C::kStages + 2 + s); };

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(tfull_bar(s), 1);
      ptx::mbar_init(tempty_bar(s), kEpilogueWarps);
    }
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&tma_a);
    ptx::prefetch_tensormap(&tma_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tmem_base_shared), C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_shared;

  const int total_tiles = p.m_tiles * p.n_tiles;
  const int G = gridDim.x;
  const uint64_t limit = p.timeout_ns;

  if (warp == 0) {
    // ================================ TMA producer =====================================
    if (lane == 0) {
      PipeState ps;
      for (int t = blockIdx.x; t < total_tiles && !abort_flag; t += G) {
        int mb, nb;
        tile_coords(p, t, mb, nb);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(empty_bar(ps.stage), ps.phase ^ 1u, &abort_flag, limit, p.status, 100 + (int)ps.stage)) break;
          const uint32_t sa = smem_a0 + ps.stage * C::kStageBytes;
          const uint32_t sb = sa + C::kABytes;
          ptx::mbar_arrive_expect_tx(full_bar(ps.stage), C::kStageBytes);
          ptx::tma_load_2d(sa, &tma_a, full_bar(ps.stage), kb * BK, mb * BM);
          ptx::tma_load_2d(sb, &tma_b, full_bar(ps.stage), kb * BK, nb * BN);
          ps.advance(C::kStages);
        }
      }
    }
  } else if (warp == 1) {
    // ================================ MMA issuer =======================================
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc_bf16_f32(BM, BN);
      PipeState ps;
      uint32_t it = 0;
      for (int t = blockIdx.x; t < total_tiles && !abort_flag; t += G, ++it) {
        const uint32_t acc = it & 1u;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, &abort_flag, limit, p.status, 200 + (int)acc)) break;
        ptx::tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < p.num_kb; ++kb) {
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
            ptx::umma_bf16(tmem_d, da + 2u * j, db + 2u * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
          }
          ptx::umma_commit(empty_bar(ps.stage));  // stage reusable once these MMAs have read it
          ps.advance(C::kStages);
        }
        if (!ok) break;
        ptx::umma_commit(tfull_bar(acc));  // accumulator complete
      }
    }
  } else {
    // ================================ epilogue =========================================
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const uint32_t slab = smem_epi + (uint32_t)(warp - 2) * C::kSlabBytes;
    constexpr int kChunksPerRow = C::kEpiCols / 8;       // 16-byte chunks per slab row
    constexpr int kRowsPerStore = 32 / kChunksPerRow;    // slab rows covered by one warp store
    constexpr int kRowPitch = C::kEpiCols * 2;
    const bool direct = (p.world_size == 1);
    const uint64_t my_counter_off = p.off_counters;
    uint32_t it = 0;
    for (int t = blockIdx.x; t < total_tiles && !abort_flag; t += G, ++it) {
      int mb, nb;
      tile_coords(p, t, mb, nb);
      const uint32_t acc = it & 1u;
      const uint32_t acc_phase = (it >> 1) & 1u;
      if (!mbar_wait(tfull_bar(acc), acc_phase, &abort_flag, limit, p.status, 400 + (int)acc)) break;
      ptx::tcgen05_fence_after();
      const int m0 = mb * BM + q * 32;
      const int n0 = nb * BN;
#pragma unroll 1
      for (int half = 0; half < BN / C::kEpiCols; ++half) {
        // ---- TMEM -> registers -> bf16 -> swizzled slab (row = lane) --------------------
#pragma unroll 1
        for (int c = 0; c < C::kEpiCols / 32; ++c) {
          uint32_t v[32];
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + half * C::kEpiCols + c * 32;
          ptx::tmem_ld_32x32b_x32(taddr, v);
          ptx::tmem_ld_wait();
          if (direct && p.bias != nullptr) {
            const int nbase = n0 + half * C::kEpiCols + c * 32;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int n = nbase + j;
              const float b = (n < p.N) ? __bfloat162float(p.bias[n]) * p.bias_scale : 0.f;
              v[j] = __float_as_uint(__uint_as_float(v[j]) + b);
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
            const uint32_t addr = slab + lane * kRowPitch + (uint32_t)((chunk ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk.x), "r"(pk.y), "r"(pk.z),
                         "r"(pk.w)
                         : "memory");
          }
        }
        if (half == BN / C::kEpiCols - 1) {
          // all TMEM reads of this accumulator are done: hand it back to the MMA warp
          ptx::tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
        }
        __syncwarp();
        // ---- slab -> global, whole row segments per store ------------------------------
#pragma unroll
        for (int s = 0; s < kChunksPerRow; ++s) {
          const int rr = s * kRowsPerStore + lane / kChunksPerRow;
          const int cc = lane % kChunksPerRow;
          const uint32_t addr = slab + rr * kRowPitch + (uint32_t)((cc ^ (rr & 7)) << 4);
          uint4 val;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                       : "r"(addr)
                       : "memory");
          const int m = m0 + rr;
          const int n = n0 + half * C::kEpiCols + cc * 8;
          if (m < p.M && n < p.N) {
            if (direct) {
              *reinterpret_cast<uint4*>(p.out + (size_t)m * p.N + n) = val;
            } else {
              const int owner = m / p.rows_per_rank;
              const int rl = m - owner * p.rows_per_rank;
              __nv_bfloat16* dst = peer_ptr<__nv_bfloat16>(p.peer_base[owner], p.off_stage) +
                                   ((size_t)p.rank * p.rows_per_rank + rl) * p.N + n;
              *reinterpret_cast<uint4*>(dst) = val;
            }
          }
        }
        __syncwarp();
      }
      if (!direct) {
        // Tell every owner with rows in this tile that this warp's part has been stored.
        __syncwarp();
        if (lane == 0) {
          __threadfence_system();
          const int m_lo = mb * BM;
          const int m_hi = min(p.M, m_lo + BM) - 1;
          const int o_lo = m_lo / p.rows_per_rank;
          const int o_hi = m_hi / p.rows_per_rank;
          for (int o = o_lo; o <= o_hi; ++o) {
            uint32_t* ctr = peer_ptr<uint32_t>(p.peer_base[o], my_counter_off) + ((size_t)mb * p.n_tiles + nb);
            red_release_sys_add(ctr, 1u);
          }
        }
      }
    }
  }

  // ================================ teardown of the GEMM phase ===========================
  if (abort_flag) {
    // give copies still in flight time to land before shared memory is released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000) __nanosleep(1000);
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if (p.world_size == 1 || abort_flag) return;

  // ================================ reduction of this rank's rows ========================
  // Blocks of the global tiling that contain rows owned by this rank; block j is reduced
  // by CTA (G-1 - j % G) so that CTAs with fewer GEMM tiles start first.
  const int R = p.rows_per_rank;
  const int row_lo = p.rank * R;
  const int mb_lo = row_lo / BM;
  const int mb_hi = (row_lo + R - 1) / BM;
  const int blocks = (mb_hi - mb_lo + 1) * p.n_tiles;
  const uint32_t want = (uint32_t)(p.world_size * kEpilogueWarps);
  uint32_t* counters = peer_ptr<uint32_t>(p.peer_base[p.rank], p.off_counters);
  const __nv_bfloat16* stage = peer_ptr<const __nv_bfloat16>(p.peer_base[p.rank], p.off_stage);
  (void)smem_gen;
  for (int j = (G - 1 - (int)blockIdx.x); j < blocks; j += G) {
    const int mb = mb_lo + j / p.n_tiles;
    const int nb = j % p.n_tiles;
    uint32_t* ctr = counters + ((size_t)mb * p.n_tiles + nb);
    if (tid == 0) {
      wait_ok_shared = wait_u32_ge(ctr, want, limit, p.status, PHASE_RS_PARTIALS, -1, mb * p.n_tiles + nb, true);
    }
    __syncthreads();
    const bool ok = wait_ok_shared != 0;
    if (ok) {
      const int r0 = max(mb * BM, row_lo);
      const int r1 = min(min((mb + 1) * BM, row_lo + R), p.M);
      const int c0 = nb * BN;
      const int c1 = min(c0 + BN, p.N);
      const int vec_per_row = (c1 - c0) >> 3;
      const int items = (r1 - r0) * vec_per_row;
      for (int i = tid; i < items; i += kThreads) {
        const int r = r0 + i / vec_per_row;
        const int n = c0 + ((i % vec_per_row) << 3);
        const int rl = r - row_lo;
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        for (int s0 = 0; s0 < p.world_size; s0 += 8) {
          uint4 vals[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int s = s0 + u;
            if (s < p.world_size) {
              vals[u] = __ldcg(reinterpret_cast<const uint4*>(stage + ((size_t)s * R + rl) * p.N + n));
            } else {
              vals[u] = make_uint4(0, 0, 0, 0);
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&vals[u]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(h[e]);
              acc[2 * e] += f.x;
              acc[2 * e + 1] += f.y;
            }
          }
        }
        if (p.bias != nullptr) {
          const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + n);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            acc[2 * e] = fmaf(f.x, p.bias_scale, acc[2 * e]);
            acc[2 * e + 1] = fmaf(f.y, p.bias_scale, acc[2 * e + 1]);
          }
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(p.out + (size_t)rl * p.N + n) = o;
      }
    }
    __syncthreads();
    if (tid == 0) *ctr = 0;  // this parity's counter is next used two calls from now
    if (!ok) break;
  }
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
// out-of-range elements read as zero.
bool make_tensor_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int pick_block_n(int M, int N, int sms) {
  const int m_tiles = (M + BM - 1) / BM;
  // widest tile that still gives every SM a tile; narrow tiles only for small problems
  for (int bn : {256, 128}) {
    const int tiles = m_tiles * ((N + bn - 1) / bn);
    if (tiles >= sms) return bn;
  }
  return 64;
}

template <int BN>
cudaError_t launch_typed(const GemmRsArgs& a, int sms, cudaStream_t stream) {
  using C = Cfg<BN>;
  CUtensorMap map_a, map_b;
  if (!make_tensor_map(&map_a, a.a, (uint64_t)a.M, (uint64_t)a.K, BM)) return cudaErrorInvalidValue;
  if (!make_tensor_map(&map_b, a.w, (uint64_t)a.N, (uint64_t)a.K, BN)) return cudaErrorInvalidValue;

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
  // rotated order: start with the first tile wholly after this rank's rows
  p.m_start = (int)((((int64_t)(a.rank + 1) * p.rows_per_rank + BM - 1) / BM) % p.m_tiles);
  p.bias_scale = a.bias_scale;
  for (int r = 0; r < kMaxWorldSize; ++r) p.peer_base[r] = a.peer_base[r];
  p.off_stage = a.off_stage;
  p.off_counters = a.off_counters;
  p.epoch = a.epoch;
  p.timeout_ns = a.timeout_ns;
  p.status = a.status;

  {
    cudaError_t e = cudaFuncSetAttribute(gemm_rs_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
  }
  const int total = p.m_tiles * p.n_tiles;
  int grid = std::min(total, sms);
  if (a.max_ctas > 0) grid = std::min(grid, a.max_ctas);
  if (grid < 1) grid = 1;
  gemm_rs_kernel<BN><<<grid, kThreads, C::kSmemBytes, stream>>>(map_a, map_b, p);
  return cudaGetLastError();
}

}  // namespace

uint64_t gemm_rs_stage_bytes(int M, int N, int world_size) {
  (void)world_size;
  return (uint64_t)M * (uint64_t)N * 2ull;  // world * (M / world) * N bf16
}

uint64_t gemm_rs_counter_bytes(int M, int N, int world_size) {
  (void)world_size;
  const uint64_t m_tiles = (M + BM - 1) / BM;
  const uint64_t n_tiles = (N + 63) / 64;
  return (m_tiles * n_tiles * 4 + 255) / 256 * 256;
}

cudaError_t launch_gemm_rs(const GemmRsArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.world_size < 1 || a.M % a.world_size != 0) return cudaErrorInvalidValue;
  if (a.K % 8 != 0 || a.N % 8 != 0) return cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int bn = a.block_n > 0 ? a.block_n : pick_block_n(a.M, a.N, sms);
  switch (bn) {
    case 256: return launch_typed<256>(a, sms, stream);
    case 128: return launch_typed<128>(a, sms, stream);
    case 64: return launch_typed<64>(a, sms, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace b200
