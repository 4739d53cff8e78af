// Helpers shared by the tensor-core (tcgen05) attention kernels: operand formats, packing,
// fast device math and the per-position (cos, sin) phase table.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "common.cuh"
#include "tc05.cuh"

namespace pope {

using namespace tc;

// device address of the sticky status word (bit 0 = a bounded wait gave up) on the current device
unsigned int* tc_status_ptr();

constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

template <typename T> struct TcFmt;
template <> struct TcFmt<__nv_bfloat16> { static constexpr uint32_t fmt = FMT_BF16; };
template <> struct TcFmt<__half> { static constexpr uint32_t fmt = FMT_F16; };

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t u);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) {
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}

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

// table[pos][c] = (cos, sin) of freqs[pos][c] as half2, built once per call in the workspace
cudaError_t launch_trig_table(const float* freqs, int64_t sfn, int n, int r, __half2* table, cudaStream_t st);

// Expand ROWS rows (row0 .. row0+ROWS) of a (rows, D) operand into the K-major operand layout
// (chunk-major storage: chunk*ROWS*16 + row*16 bytes): chunks [0, D/8) hold a*cos for rotated
// features and the raw feature otherwise, chunks [D/8, D/8 + r/8) hold a*sin.  Phases come from
// the table row (pos0 + row); rows at or beyond `nrows` are zero-filled.  256 threads.
template <int D, int ROWS, typename T>
__device__ __forceinline__ void stage_xform_table(const T* base, int64_t sn, int row0, int nrows, const __half2* table,
                                                  int pos0, int r, uint8_t* buf, int tid) {
  constexpr int DC = D / 8;
  const int RC = r >> 3;
#pragma unroll
  for (int it = 0; it < (ROWS * DC) / 256; ++it) {
    const int task = tid + it * 256;
    const int row = task % ROWS, c = task / ROWS;
    const int j = row0 + row;
    const bool ok = j < nrows;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (ok) raw = *reinterpret_cast<const uint4*>(base + (int64_t)j * sn + c * 8);
    if (c < RC) {
      uint4 t0 = make_uint4(0, 0, 0, 0), t1 = t0;
      if (ok) {
        const uint4* tp = reinterpret_cast<const uint4*>(table + (int64_t)(pos0 + j) * r + c * 8);
        t0 = tp[0], t1 = tp[1];
      }
      const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
      const uint32_t tw[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
      uint32_t oc[4], os[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x = unpack2<T>(rw[e]);
        const float a0 = softplus_fast(x.x), a1 = softplus_fast(x.y);
        const float2 cs0 = __half22float2(*reinterpret_cast<const __half2*>(&tw[2 * e]));
        const float2 cs1 = __half22float2(*reinterpret_cast<const __half2*>(&tw[2 * e + 1]));
        oc[e] = ok ? pack2<T>(a0 * cs0.x, a1 * cs1.x) : 0u;
        os[e] = ok ? pack2<T>(a0 * cs0.y, a1 * cs1.y) : 0u;
      }
      *reinterpret_cast<uint4*>(buf + c * (ROWS * 16) + row * 16) = make_uint4(oc[0], oc[1], oc[2], oc[3]);
      *reinterpret_cast<uint4*>(buf + (DC + c) * (ROWS * 16) + row * 16) = make_uint4(os[0], os[1], os[2], os[3]);
    } else {
      *reinterpret_cast<uint4*>(buf + c * (ROWS * 16) + row * 16) = raw;
    }
  }
}

// Copy ROWS rows of a (rows, D) operand unchanged into the same chunk-major layout.  256 threads.
template <int D, int ROWS, typename T>
__device__ __forceinline__ void stage_plain(const T* base, int64_t sn, int row0, int nrows, uint8_t* buf, int tid) {
  constexpr int DC = D / 8;
#pragma unroll
  for (int it = 0; it < (ROWS * DC) / 256; ++it) {
    const int task = tid + it * 256;
    const int row = task % ROWS, c = task / ROWS;
    const int j = row0 + row;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (j < nrows) raw = *reinterpret_cast<const uint4*>(base + (int64_t)j * sn + c * 8);
    *reinterpret_cast<uint4*>(buf + c * (ROWS * 16) + row * 16) = raw;
  }
}

// Exact (sincosf, log1pf) transform of 128 resident rows, phase = freqs[pos0 + row] + sign*bias.
// Same layout as above with ROWS = 128.  256 threads: thread handles row tid%128, chunks tid/128 + 2k.
template <int D, typename T>
__device__ __forceinline__ void stage_xform_exact128(const T* base, int64_t sn, int row0, int nrows, const float* freqs,
                                                     int64_t sfn, int pos0, const float* bias, float sign, int r,
                                                     uint8_t* buf, int tid) {
  constexpr int DC = D / 8;
  const int RC = r >> 3;
  const int row = tid & 127, j = row0 + row;
  const bool ok = j < nrows;
  const T* src = base + (int64_t)j * sn;
  const float* frow = r > 0 ? freqs + (int64_t)(pos0 + j) * sfn : nullptr;
  for (int c = tid >> 7; c < DC; c += 2) {
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (ok) raw = *reinterpret_cast<const uint4*>(src + c * 8);
    if (c < RC) {
      const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
      uint32_t oc[4] = {0, 0, 0, 0}, os[4] = {0, 0, 0, 0};
      if (ok) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = unpack2<T>(rw[e]);
          float s0, c0, s1, c1;
          sincosf(frow[c * 8 + 2 * e] + sign * bias[c * 8 + 2 * e], &s0, &c0);
          sincosf(frow[c * 8 + 2 * e + 1] + sign * bias[c * 8 + 2 * e + 1], &s1, &c1);
          const float a0 = softplus_f(x.x), a1 = softplus_f(x.y);
          oc[e] = pack2<T>(a0 * c0, a1 * c1);
          os[e] = pack2<T>(a0 * s0, a1 * s1);
        }
      }
      *reinterpret_cast<uint4*>(buf + c * (128 * 16) + row * 16) = make_uint4(oc[0], oc[1], oc[2], oc[3]);
      *reinterpret_cast<uint4*>(buf + (DC + c) * (128 * 16) + row * 16) = make_uint4(os[0], os[1], os[2], os[3]);
    } else {
      *reinterpret_cast<uint4*>(buf + c * (128 * 16) + row * 16) = raw;
    }
  }
}

}  // namespace pope
