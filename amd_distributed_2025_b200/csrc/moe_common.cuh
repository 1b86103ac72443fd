// Element conversions and 16-byte vector helpers shared by the MoE kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {
namespace moe {

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T> struct Vec16;  // 16-byte vector of T
template <> struct Vec16<__half> { static constexpr int N = 8; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };
template <> struct Vec16<float> { static constexpr int N = 4; };

// acc[0..N) += w * raw[0..N)
template <typename T>
__device__ __forceinline__ void fma_vec(float* acc, const int4& raw, float w);

template <>
__device__ __forceinline__ void fma_vec<__half>(float* acc, const int4& raw, float w) {
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(h[j]);
    acc[2 * j] = fmaf(f.x, w, acc[2 * j]);
    acc[2 * j + 1] = fmaf(f.y, w, acc[2 * j + 1]);
  }
}
template <>
__device__ __forceinline__ void fma_vec<__nv_bfloat16>(float* acc, const int4& raw, float w) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(h[j]);
    acc[2 * j] = fmaf(f.x, w, acc[2 * j]);
    acc[2 * j + 1] = fmaf(f.y, w, acc[2 * j + 1]);
  }
}
template <>
__device__ __forceinline__ void fma_vec<float>(float* acc, const int4& raw, float w) {
  const float* f = reinterpret_cast<const float*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) acc[j] = fmaf(f[j], w, acc[j]);
}

template <typename T>
__device__ __forceinline__ int4 pack_vec(const float* acc);
template <>
__device__ __forceinline__ int4 pack_vec<__half>(const float* acc) {
  int4 out;
  __half2* h = reinterpret_cast<__half2*>(&out);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
  return out;
}
template <>
__device__ __forceinline__ int4 pack_vec<__nv_bfloat16>(const float* acc) {
  int4 out;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
  return out;
}
template <>
__device__ __forceinline__ int4 pack_vec<float>(const float* acc) {
  int4 out;
  float* f = reinterpret_cast<float*>(&out);
#pragma unroll
  for (int j = 0; j < 4; ++j) f[j] = acc[j];
  return out;
}

// 16 bytes of T, every element multiplied by `s` (fp32 product, one rounding).
template <typename T>
__device__ __forceinline__ int4 scale_vec(const int4& raw, float s) {
  float acc[Vec16<T>::N];
#pragma unroll
  for (int j = 0; j < Vec16<T>::N; ++j) acc[j] = 0.f;
  fma_vec<T>(acc, raw, s);
  return pack_vec<T>(acc);
}

}  // namespace moe
}  // namespace b200
