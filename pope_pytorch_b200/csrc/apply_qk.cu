// Stand-alone PoPE transform (sm_100a): q, k -> q', k' of width 2r + (d - r) in the reference's interleaved layout
// [a0 cos, a0 sin, a1 cos, a1 sin, ..., pass-through features], fp32, for callers that feed their own attention.
// Replaces the chain of elementwise PyTorch kernels of PoPE_pytorch/pope.py:37-86 (softplus, add, cos, sin, two
// products, stack, reshape, cat: about ten passes over the data) by ONE pass: bytes = inputs + outputs, HBM-bound.
// Phases as the reference computes them: query row i uses freqs[Nk - Nq + i] (:64), key row j uses fl(freqs[j] + bias[h])
// (:56); accurate sincosf and log1pf / expf, since the result IS the user-visible value here (no 16-bit rounding
// follows).  The backward is the chain rule of the same map:
//   dx = (g_c cos + g_s sin) sigmoid(x),  dphase = a (g_s cos - g_c sin)  -> dfreqs (query and key rows), dbias (key rows).
#include "kernels.h"
#include "common.cuh"

namespace pope {

struct ApplySide {
  const void* x;      // (units, rows, d) input
  Strides sx;
  float* y;           // (units, rows, d + r) output / its gradient
  Strides sy;
  void* dx;           // backward only
  Strides sdx;
  int heads, rows, pos0;
  const float* bias;  // key side: per-head phase; query side: null
  int64_t bias_sh;
  float* dbias;       // backward, key side only (may be null)
  int64_t dbias_sh;
};

struct ApplyP {
  ApplySide side[2];  // 0 = queries, 1 = keys
  int B, d, r;
  const float* freqs;
  Strides sf;
  float* dfreqs;      // backward (may be null)
  Strides sdf;
};

constexpr int AP_THREADS = 256;
constexpr int AP_ROWS = 16;   // rows per block: the bias gradient of a block is reduced before it touches global memory

// grid (row blocks, units, 2 sides); thread = (row within the block, feature): DP = features rounded up to a power of two
template <typename T, bool BACKWARD>
__global__ void __launch_bounds__(AP_THREADS) apply_qk_kernel(ApplyP p, int DP) {
  const ApplySide& s = p.side[blockIdx.z];
  const int u = blockIdx.y, b = u / s.heads, h = u % s.heads;
  if (b >= p.B) return;
  const int c = threadIdx.x % DP, lane_row = threadIdx.x / DP, rows_per_pass = AP_THREADS / DP;
  const int row_begin = blockIdx.x * AP_ROWS;
  if (row_begin >= s.rows) return;
  const bool live = c < p.d;
  const bool rot = c < p.r;
  const float hb = (rot && s.bias) ? s.bias[h * s.bias_sh + c] : 0.f;
  float dbias_acc = 0.f;
  for (int rr = lane_row; rr < AP_ROWS; rr += rows_per_pass) {
    const int i = row_begin + rr;
    if (i >= s.rows || !live) continue;
    const T* xr = static_cast<const T*>(s.x) + b * s.sx.b + h * s.sx.h + (int64_t)i * s.sx.n;
    float* yr = s.y + b * s.sy.b + h * s.sy.h + (int64_t)i * s.sy.n;
    const float x = to_f32<T>(xr[c]);
    if (rot) {
      const int pos = s.pos0 + i;
      const float f = p.freqs[b * p.sf.b + h * p.sf.h + (int64_t)pos * p.sf.n + c];
      float sn, cs;
      sincosf(s.bias ? f + hb : f, &sn, &cs);
      const float a = softplus_f(x);
      if (!BACKWARD) {
        *reinterpret_cast<float2*>(yr + 2 * c) = make_float2(a * cs, a * sn);
      } else {
        const float2 g = *reinterpret_cast<const float2*>(yr + 2 * c);
        T* dxr = static_cast<T*>(s.dx) + b * s.sdx.b + h * s.sdx.h + (int64_t)i * s.sdx.n;
        dxr[c] = from_f32<T>((g.x * cs + g.y * sn) * sigmoid_f(x));
        const float dphase = a * (g.y * cs - g.x * sn);
        if (p.dfreqs) atomicAdd(p.dfreqs + b * p.sdf.b + h * p.sdf.h + (int64_t)pos * p.sdf.n + c, dphase);
        dbias_acc += dphase;
      }
    } else {
      if (!BACKWARD) {
        yr[p.r + c] = x;
      } else {
        T* dxr = static_cast<T*>(s.dx) + b * s.sdx.b + h * s.sdx.h + (int64_t)i * s.sdx.n;
        dxr[c] = from_f32<T>(yr[p.r + c]);
      }
    }
  }
  if (BACKWARD && s.dbias) {
    // one atomic per (block, feature): the row lanes of a feature are summed through shared memory first
    __shared__ float red[AP_THREADS];
    red[threadIdx.x] = dbias_acc;
    __syncthreads();
    if (lane_row == 0 && rot) {
      float sum = 0.f;
      for (int l = 0; l < rows_per_pass; ++l) sum += red[l * DP + c];
      atomicAdd(s.dbias + h * s.dbias_sh + c, sum);
    }
  }
}

static int pow2_at_least(int x) {
  int p = 1;
  while (p < x) p <<= 1;
  return p;
}

template <typename T, bool BACKWARD>
static cudaError_t launch_apply(const ApplyP& p, int units_max, int rows_max, cudaStream_t st) {
  const int DP = pow2_at_least(p.d);
  if (DP > AP_THREADS) return cudaErrorInvalidValue;
  const dim3 grid((unsigned)((rows_max + AP_ROWS - 1) / AP_ROWS), (unsigned)units_max, 2);
  apply_qk_kernel<T, BACKWARD><<<grid, AP_THREADS, 0, st>>>(p, DP);
  return cudaGetLastError();
}

static ApplyP apply_params(const PopeShape& s, const PopeEmbed& e) {
  ApplyP p = {};
  p.B = s.B, p.d = s.d, p.r = s.r;
  p.freqs = e.freqs, p.sf = Strides(e.sf);
  p.side[0].heads = s.H, p.side[0].rows = s.Nq, p.side[0].pos0 = s.Nk - s.Nq;
  p.side[1].heads = s.Hk, p.side[1].rows = s.Nk, p.side[1].pos0 = 0;
  p.side[1].bias = s.r > 0 ? e.bias : nullptr, p.side[1].bias_sh = e.bias_stride_h;
  return p;
}

cudaError_t apply_qk_fwd(const PopeApplyArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  ApplyP p = apply_params(s, a.embed);
  p.side[0].x = a.q, p.side[0].sx = Strides(a.sq), p.side[0].y = a.q_out, p.side[0].sy = Strides(a.sqo);
  p.side[1].x = a.k, p.side[1].sx = Strides(a.sk), p.side[1].y = a.k_out, p.side[1].sy = Strides(a.sko);
  const int units = s.B * (s.H > s.Hk ? s.H : s.Hk);
  switch (s.dtype) {
    case POPE_F32: return launch_apply<float, false>(p, units, s.Nk, st);
    case POPE_BF16: return launch_apply<__nv_bfloat16, false>(p, units, s.Nk, st);
    default: return launch_apply<__half, false>(p, units, s.Nk, st);
  }
}

cudaError_t apply_qk_bwd(const PopeApplyBwdArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  ApplyP p = apply_params(s, a.embed);
  p.side[0].x = a.q, p.side[0].sx = Strides(a.sq), p.side[0].y = const_cast<float*>(a.dq_out), p.side[0].sy = Strides(a.sdqo);
  p.side[0].dx = a.dq, p.side[0].sdx = Strides(a.sdq);
  p.side[1].x = a.k, p.side[1].sx = Strides(a.sk), p.side[1].y = const_cast<float*>(a.dk_out), p.side[1].sy = Strides(a.sdko);
  p.side[1].dx = a.dk, p.side[1].sdx = Strides(a.sdk);
  p.side[1].dbias = s.r > 0 ? a.dbias : nullptr, p.side[1].dbias_sh = a.dbias_stride_h;
  p.dfreqs = s.r > 0 ? a.dfreqs : nullptr, p.sdf = Strides(a.sdf);
  const int units = s.B * (s.H > s.Hk ? s.H : s.Hk);
  switch (s.dtype) {
    case POPE_F32: return launch_apply<float, true>(p, units, s.Nk, st);
    case POPE_BF16: return launch_apply<__nv_bfloat16, true>(p, units, s.Nk, st);
    default: return launch_apply<__half, true>(p, units, s.Nk, st);
  }
}

}  // namespace pope
