// Shared device helpers for the PoPE kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pope_b200.h"

namespace pope {

// ---- element access in fp32 regardless of storage type ------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// ---- the PoPE magnitude and its derivative -------------------------------------------------
// softplus with the cut-over at 20 used by torch.nn.functional.softplus and by the reference
// kernels (PoPE_pytorch/triton_pope.py:18-24).
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// softplus(x) = max(x,0) + log1p(exp(-|x|)); beyond x = 20 the second term is below 2.1e-9,
// i.e. the reference's cut-over to the identity is reproduced to fp32 rounding.
__device__ __forceinline__ float softplus_fast(float x) {
  const float t = ex2_approx(-fabsf(x) * 1.4426950408889634f);
  return fmaxf(x, 0.f) + lg2_approx(1.f + t) * 0.6931471805599453f;
}

// sin / cos for phases up to ~1e5 rad at ~1e-6 absolute error: two-constant Cody-Waite reduction to [-pi, pi]
// (k * 6.28125 is exact for |k| < 2^15), then the special-function unit.  The accurate sincosf costs five times the
// instructions; this form is for results that are rounded or tolerance-checked at 1e-5 or coarser.
__device__ __forceinline__ void sincos_reduced(float x, float* s, float* c) {
  const float k = rintf(x * 0.15915494309189535f);
  float r = fmaf(-k, 6.28125f, x);
  r = fmaf(-k, 1.9353071795864769e-3f, r);
  *s = __sinf(r), *c = __cosf(r);
}

// Addressing of one (batch, head) unit of a strided tensor.
struct Strides {
  int64_t b, h, n;
  __host__ __device__ Strides() : b(0), h(0), n(0) {}
  __host__ __device__ Strides(const PopeStride3& s) : b(s.b), h(s.h), n(s.n) {}
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace pope
