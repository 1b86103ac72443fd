// Block-scaled fp8 (e4m3) GEMM for sm_100a:  C[m, n] = sum_kb (A_kb[m, :] . B_kb[n, :]) * as[m, kb] * bs[n / 128, kb]
//
// The reference tree carries a template for this operation that belongs to neither of
// its two tasks (all2all/hip.py:17-59, identical copy in gemm-rs/hip.py): one thread per
// output element, K walked in blocks of 128, the block's partial product multiplied by a
// per-row scale of A and a per-128x128-block scale of B, bf16 result.  Here the block
// products run on the tensor cores: per 128-wide K block four tcgen05.mma.kind::f8f6f4
// instructions (K = 32 each) write a fresh 128 x 128 fp32 partial into one of two
// tensor-memory buffers, and the four epilogue warps pull it out, multiply by the
// block's scales and accumulate in registers while the next block is being multiplied.
// Operands are K-major (row-major [m, k] and [n, k]); TMA stages them with the 128-byte
// swizzle exactly as in the bf16 GEMM (a 128-byte row now holds 128 fp8 values).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "fp8_gemm.h"
#include "signal.cuh"
#include "sm100_ptx.cuh"

namespace b200 {

namespace {

constexpr int FBM = 128, FBN = 128, FBK = 128;  // FBK = the scale block of the operation
constexpr int kFp8Threads = 192;                // producer, MMA issuer, 4 epilogue warps
constexpr int kFp8Stages = 6;
constexpr int kFp8ABytes = FBM * FBK;           // 16 KiB
constexpr int kFp8BBytes = FBN * FBK;
constexpr int kFp8StageBytes = kFp8ABytes + kFp8BBytes;
constexpr int kFp8SmemBytes = 1024 + kFp8Stages * kFp8StageBytes + 1024;

struct Fp8Params {
  const float* a_scale;  // [m, k_blocks], element (m, kb) at m * as_stride_m + kb * as_stride_k
  const float* b_scale;  // [n_blocks, k_blocks], element (nb, kb) at nb * bs_stride_n + kb * bs_stride_k
  __nv_bfloat16* c;      // [m, n] row-major
  int M, N, K, k_blocks;
  long long as_stride_m, as_stride_k, bs_stride_n, bs_stride_k;
  uint64_t timeout_ns;
  int* error_flag;  // set to 1 if a pipeline wait expired
};

// Instruction descriptor of tcgen05.mma.kind::f8f6f4 with e4m3 A and B (both K-major) and fp32
// accumulation: bits [4,6) D format (1 = f32), [7,10) A format (0 = e4m3), [10,13) B format,
// [17,23) N >> 3, [24,29) M >> 4.
constexpr uint32_t make_idesc_e4m3_f32(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void umma_fp8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ bool fp8_wait(uint32_t bar, uint32_t parity, volatile int* abort, uint64_t limit_ns,
                                         int* error_flag) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((++spins & 255u) == 0) {
      if (*abort) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *abort = 1;
        if (error_flag != nullptr) *error_flag = 1;
        return false;
      }
    }
  }
}

}  // namespace

__global__ void __launch_bounds__(kFp8Threads, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                const Fp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int abort_flag;
  __shared__ uint32_t tmem_base_shared;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + kFp8Stages * kFp8StageBytes;
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (kFp8Stages + s); };
  auto tfull_bar = [&](uint32_t s) { return bar_base + 8u * (2 * kFp8Stages + s); };
  auto tempty_bar = [&](uint32_t s) { return bar_base + 8u * (2 * kFp8Stages + 2 + s); };

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < kFp8Stages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(tfull_bar(s), 1);
      ptx::mbar_init(tempty_bar(s), 4);
    }
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tmem_base_shared), 2 * FBN);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_shared;

  const int m_tiles = (p.M + FBM - 1) / FBM;
  const int n_tiles = (p.N + FBN - 1) / FBN;
  const int total = m_tiles * n_tiles;
  const int G = gridDim.x;
  const uint64_t limit = p.timeout_ns;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int t = blockIdx.x; t < total && !abort_flag; t += G) {
        const int mb = t / n_tiles, nb = t % n_tiles;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!fp8_wait(empty_bar(stage), phase ^ 1u, &abort_flag, limit, p.error_flag)) break;
          const uint32_t sa = smem_base + stage * kFp8StageBytes;
          ptx::mbar_arrive_expect_tx(full_bar(stage), kFp8StageBytes);
          ptx::tma_load_2d(sa, &tma_a, full_bar(stage), kb * FBK, mb * FBM);
          ptx::tma_load_2d(sa + kFp8ABytes, &tma_b, full_bar(stage), kb * FBK, nb * FBN);
          if (++stage == kFp8Stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_e4m3_f32(FBM, FBN);
      uint32_t stage = 0, phase = 0, it = 0;  // `it` counts K blocks over all tiles: one TMEM buffer each
      for (int t = blockIdx.x; t < total && !abort_flag; t += G) {
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t acc = it & 1u;
          if (!fp8_wait(tempty_bar(acc), ((it >> 1) & 1u) ^ 1u, &abort_flag, limit, p.error_flag)) break;
          if (!fp8_wait(full_bar(stage), phase, &abort_flag, limit, p.error_flag)) break;
          ptx::tcgen05_fence_after();
          const uint32_t sa = smem_base + stage * kFp8StageBytes;
          const uint64_t da = ptx::make_smem_desc_k_sw128(sa);
          const uint64_t db = ptx::make_smem_desc_k_sw128(sa + kFp8ABytes);
#pragma unroll
          for (int j = 0; j < FBK / 32; ++j) {
            // 32 fp8 = 32 bytes of K per instruction = 2 descriptor address units
            umma_fp8(tmem_base + acc * FBN, da + 2u * j, db + 2u * j, idesc, j > 0 ? 1u : 0u);
          }
          ptx::umma_commit(empty_bar(stage));
          ptx::umma_commit(tfull_bar(acc));
          if (++stage == kFp8Stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t it = 0;
    for (int t = blockIdx.x; t < total && !abort_flag; t += G) {
      const int mb = t / n_tiles, nb = t % n_tiles;
      const int m = mb * FBM + q * 32 + lane;
      float accum[FBN];
#pragma unroll
      for (int j = 0; j < FBN; ++j) accum[j] = 0.f;
      bool ok = true;
      for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
        const uint32_t acc = it & 1u;
        if (!fp8_wait(tfull_bar(acc), (it >> 1) & 1u, &abort_flag, limit, p.error_flag)) {
          ok = false;
          break;
        }
        ptx::tcgen05_fence_after();
        float scale = 0.f;
        if (m < p.M) {
          scale = p.a_scale[(long long)m * p.as_stride_m + (long long)kb * p.as_stride_k] *
                  p.b_scale[(long long)nb * p.bs_stride_n + (long long)kb * p.bs_stride_k];
        }
#pragma unroll
        for (int c = 0; c < FBN / 32; ++c) {
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * FBN + c * 32, v);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) accum[c * 32 + j] = fmaf(__uint_as_float(v[j]), scale, accum[c * 32 + j]);
        }
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
        __syncwarp();
      }
      if (ok && m < p.M) {
        __nv_bfloat16* row = p.c + (size_t)m * p.N + (size_t)nb * FBN;
        const int ncols = min(FBN, p.N - nb * FBN);
        if ((p.N & 7) == 0) {
#pragma unroll
          for (int j = 0; j < FBN; j += 8) {
            if (j < ncols) {
              uint4 o;
              __nv_bfloat162 h;
              h = __floats2bfloat162_rn(accum[j], accum[j + 1]);
              o.x = *reinterpret_cast<uint32_t*>(&h);
              h = __floats2bfloat162_rn(accum[j + 2], accum[j + 3]);
              o.y = *reinterpret_cast<uint32_t*>(&h);
              h = __floats2bfloat162_rn(accum[j + 4], accum[j + 5]);
              o.z = *reinterpret_cast<uint32_t*>(&h);
              h = __floats2bfloat162_rn(accum[j + 6], accum[j + 7]);
              o.w = *reinterpret_cast<uint32_t*>(&h);
              *reinterpret_cast<uint4*>(row + j) = o;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < FBN; ++j)
            if (j < ncols) row[j] = __float2bfloat16_rn(accum[j]);
        }
      }
    }
  }

  if (abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000) __nanosleep(1000);
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, 2 * FBN);
  }
}

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool make_fp8_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return false;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols};
  cuuint32_t box[2] = {(cuuint32_t)FBK, box_rows};
  cuuint32_t elem_strides[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

cudaError_t launch_fp8_gemm(const Fp8GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.K % 16 != 0) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  if (!make_fp8_map(&map_a, a.a, (uint64_t)a.M, (uint64_t)a.K, FBM)) return cudaErrorInvalidValue;
  if (!make_fp8_map(&map_b, a.b, (uint64_t)a.N, (uint64_t)a.K, FBN)) return cudaErrorInvalidValue;
  Fp8Params p;
  p.a_scale = a.a_scale;
  p.b_scale = a.b_scale;
  p.c = reinterpret_cast<__nv_bfloat16*>(a.c);
  p.M = a.M;
  p.N = a.N;
  p.K = a.K;
  p.k_blocks = (a.K + FBK - 1) / FBK;
  p.as_stride_m = a.as_stride_m;
  p.as_stride_k = a.as_stride_k;
  p.bs_stride_n = a.bs_stride_n;
  p.bs_stride_k = a.bs_stride_k;
  p.timeout_ns = a.timeout_ns;
  p.error_flag = a.error_flag;
  cudaError_t e = cudaFuncSetAttribute(fp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFp8SmemBytes);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int total = ((a.M + FBM - 1) / FBM) * ((a.N + FBN - 1) / FBN);
  const int grid = std::max(1, std::min(total, sms));
  fp8_gemm_kernel<<<grid, kFp8Threads, kFp8SmemBytes, stream>>>(map_a, map_b, p);
  return cudaGetLastError();
}

}  // namespace b200
