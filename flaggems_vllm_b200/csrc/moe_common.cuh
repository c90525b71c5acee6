// Shared helpers for the sm_100a MoE kernels: error reporting for the C ABI,
// dtype tags, small device utilities.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/moe_sm100.h"

namespace moe {

// Records a host-side failure text for moe_last_error(); returns `code`.
int fail(int code, const char* fmt, ...);
// Checks the launch error of the kernel just enqueued; returns 0 or the cudaError_t.
int check_launch(const char* what);
// Limit, in nanoseconds, of every bounded barrier wait of the kernels launched from now on
// (moe_set_wait_limit_ns; 2 s unless changed).
unsigned long long wait_limit_ns();

template <typename T> struct ToF32;
template <> struct ToF32<float> {
  static __device__ __forceinline__ float get(float v) { return v; }
};
template <> struct ToF32<__half> {
  static __device__ __forceinline__ float get(__half v) { return __half2float(v); }
};
template <> struct ToF32<__nv_bfloat16> {
  static __device__ __forceinline__ float get(__nv_bfloat16 v) { return __bfloat162float(v); }
};

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float fp8e4m3_to_f32(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ uint8_t f32_to_fp8e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// SiLU(g) * u with the sigmoid written as the reference kernel does,
// g / (1 + exp(-g)) in fp32 (src/flaggems_vllm/ops/fused_moe.py:1795).
__device__ __forceinline__ float silu_mul(float g, float u) {
  return (g / (1.0f + expf(-g))) * u;
}

__device__ __forceinline__ void set_status(int32_t* status, int bit) {
  if (status != nullptr) atomicOr(status, bit);
}

// Eight consecutive elements as fp32 (one or two 16-byte loads).
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}

constexpr float kFp8Max = 448.0f;
constexpr float kQuantEps = 1e-10f;

}  // namespace moe
