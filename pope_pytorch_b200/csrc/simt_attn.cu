// Full-precision (fp32 FMA) PoPE attention: forward (with a split over the keys for short
// query ranges), and backward.  Any shape / stride / dtype the C ABI accepts runs here; the
// tensor-core family takes over the shapes it implements.
//
// Reference semantics: PoPE_pytorch/triton_pope_flash_attn.py:23-218.
//
// Expanded operand layout used inside these kernels (never leaves shared memory):
//   columns [0, HDP)        : a*cos(phase) for c < r, the raw feature for r <= c < d, zero padding
//   columns [HDP, HDP + RP) : a*sin(phase) for c < r, zero padding
// with HDP = d rounded up to 32 and RP = r rounded up to 32.
#include <math_constants.h>

#include "common.cuh"
#include "kernels.h"

namespace pope {

constexpr int AM = 32;  // rows owned by a CTA (8 warps x 4 rows)
constexpr int AN = 32;  // rows of the opposite operand per step (one per lane)

struct AttnP {
  int B, H, Hk, Nq, Nk, d, r;
  int causal, nsplit, split_len;
  float scale;
  const void *q, *k, *v, *out, *dout;
  Strides sq, sk, sv, so, sdo, sf, sdq, sdk, sdv, sdf;
  const float *freqs, *bias, *lse_in, *delta;
  int64_t bias_sh, dbias_sh;
  const uint8_t* mask;
  int64_t msb, msn;
  void *o, *dq, *dk, *dv;
  float *lse, *dfreqs, *dbias;
  float *part_o, *part_ml;  // split-KV partials
};

// Transform one feature of one row into its (cos-part, sin-part) pair.
template <typename T>
__device__ __forceinline__ void xform(const T* row, const float* frow, const float* bias, int c, int d, int r,
                                      float& vc, float& vs) {
  vc = 0.f, vs = 0.f;
  if (c < d) {
    const float x = to_f32(row[c]);
    if (c < r) {
      float th = frow[c];
      if (bias) th += bias[c];
      float sn, cs;
      sincosf(th, &sn, &cs);
      const float a = softplus_f(x);
      vc = a * cs, vs = a * sn;
    } else {
      vc = x;
    }
  }
}

// Stage 32 rows feature-major: XT[c][row] (row stride 32 floats), cos block then sin block.
template <typename T>
__device__ __forceinline__ void stage_feature_major(float* XT, const T* base, int64_t sn, const float* f, int64_t fsn,
                                                    const float* bias, int row0, int nrows, int pos0, int d, int r,
                                                    int HDP, int RP, int tid) {
  const int row = tid & 31, grow = row0 + row;
  for (int c = tid >> 5; c < HDP; c += 8) {
    float vc = 0.f, vs = 0.f;
    if (grow < nrows) xform<T>(base + (int64_t)grow * sn, f ? f + (int64_t)(pos0 + grow) * fsn : nullptr, bias, c, d, r, vc, vs);
    XT[c * 32 + row] = vc;
    if (c < RP) XT[(HDP + c) * 32 + row] = vs;
  }
}

// Stage 32 rows row-major with odd stride ld: X[row][c].
template <typename T>
__device__ __forceinline__ void stage_row_major(float* X, int ld, const T* base, int64_t sn, const float* f, int64_t fsn,
                                                const float* bias, int row0, int nrows, int pos0, int d, int r,
                                                int HDP, int RP, int tid) {
  const int row = tid >> 3, grow = row0 + row;
  for (int c = tid & 7; c < HDP; c += 8) {
    float vc = 0.f, vs = 0.f;
    if (grow < nrows) xform<T>(base + (int64_t)grow * sn, f ? f + (int64_t)(pos0 + grow) * fsn : nullptr, bias, c, d, r, vc, vs);
    X[row * ld + c] = vc;
    if (c < RP) X[row * ld + HDP + c] = vs;
  }
}

// Plain (untransformed) staging, row-major / feature-major.
template <typename T>
__device__ __forceinline__ void stage_plain_row_major(float* X, int ld, const T* base, int64_t sn, int row0, int nrows,
                                                      int d, int HDP, int tid) {
  const int row = tid >> 3, grow = row0 + row;
  for (int c = tid & 7; c < HDP; c += 8) X[row * ld + c] = (grow < nrows && c < d) ? to_f32(base[(int64_t)grow * sn + c]) : 0.f;
}
template <typename T>
__device__ __forceinline__ void stage_plain_feature_major(float* XT, const T* base, int64_t sn, int row0, int nrows,
                                                          int d, int HDP, int tid) {
  const int row = tid & 31, grow = row0 + row;
  for (int c = tid >> 5; c < HDP; c += 8) XT[c * 32 + row] = (grow < nrows && c < d) ? to_f32(base[(int64_t)grow * sn + c]) : 0.f;
}

// dot of this warp's 4 owned rows (feature-major tile AT, float4 per feature) with the lane's row of X
__device__ __forceinline__ void dot4(const float* AT, int w, const float* xrow, int n, float (&s)[4]) {
  s[0] = s[1] = s[2] = s[3] = 0.f;
#pragma unroll 8
  for (int c = 0; c < n; ++c) {
    const float4 a = *reinterpret_cast<const float4*>(AT + c * 32 + w * 4);
    const float x = xrow[c];
    s[0] = fmaf(a.x, x, s[0]), s[1] = fmaf(a.y, x, s[1]), s[2] = fmaf(a.z, x, s[2]), s[3] = fmaf(a.w, x, s[3]);
  }
}

// ---- forward -------------------------------------------------------------------------------
template <typename T, int DCH>
__global__ void __launch_bounds__(256) attn_fwd_simt_kernel(AttnP p) {
  extern __shared__ __align__(16) float smem[];
  const int HDP = DCH * 32, RP = (p.r + 31) / 32 * 32, KD = HDP + RP;
  float* QT = smem;                    // [KD][32]
  float* Ks = QT + KD * 32;            // [32][KD+1]
  float* Vs = Ks + 32 * (KD + 1);      // [32][HDP+1]
  float* Ps = Vs + 32 * (HDP + 1);     // [8][32][4]
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int u = blockIdx.y, b = u / p.H, h = u % p.H, hk = h % p.Hk;
  const int i0 = blockIdx.x * AM;
  const int qoff = p.Nk - p.Nq;
  const T* q = (const T*)p.q + b * p.sq.b + h * p.sq.h;
  const T* k = (const T*)p.k + b * p.sk.b + hk * p.sk.h;
  const T* v = (const T*)p.v + b * p.sv.b + hk * p.sv.h;
  const float* fq = p.r > 0 ? p.freqs + b * p.sf.b + h * p.sf.h : nullptr;
  const float* fk = p.r > 0 ? p.freqs + b * p.sf.b + hk * p.sf.h : nullptr;
  const float* bias = p.r > 0 ? p.bias + hk * p.bias_sh : nullptr;
  const uint8_t* mask = p.mask ? p.mask + b * p.msb : nullptr;

  stage_feature_major<T>(QT, q, p.sq.n, fq, p.sf.n, nullptr, i0, p.Nq, qoff, p.d, p.r, HDP, RP, tid);

  int kb = blockIdx.z * p.split_len, ke = min(p.Nk, kb + p.split_len);
  if (p.causal) ke = min(ke, min(i0 + AM, p.Nq));  // key j is visible to row i iff j <= i
  float m[4], l[4], o[4][DCH];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -CUDART_INF_F, l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < DCH; ++c) o[i][c] = 0.f;
  }

  for (int n0 = kb; n0 < ke; n0 += AN) {
    __syncthreads();  // previous tile fully consumed (also orders the Q staging on the first pass)
    stage_row_major<T>(Ks, KD + 1, k, p.sk.n, fk, p.sf.n, bias, n0, ke, 0, p.d, p.r, HDP, RP, tid);
    stage_plain_row_major<T>(Vs, HDP + 1, v, p.sv.n, n0, ke, p.d, HDP, tid);
    __syncthreads();
    float s[4];
    dot4(QT, w, Ks + lane * (KD + 1), KD, s);
    const int j = n0 + lane;
    const bool key_ok = j < ke && (!mask || mask[(int64_t)j * p.msn]);
    float pr[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int gi = i0 + w * 4 + i;
      const bool ok = key_ok && (!p.causal || j <= gi);
      const float sv = ok ? s[i] * p.scale : -CUDART_INF_F;
      const float mnew = fmaxf(m[i], warp_max(sv));
      float alpha = 1.f, pv = 0.f;
      if (mnew != -CUDART_INF_F) {
        alpha = __expf(m[i] - mnew);  // m = -inf gives 0
        pv = ok ? expf(sv - mnew) : 0.f;
      }
      l[i] = l[i] * alpha + warp_sum(pv);
      m[i] = mnew;
      pr[i] = pv;
#pragma unroll
      for (int c = 0; c < DCH; ++c) o[i][c] *= alpha;
    }
    *reinterpret_cast<float4*>(Ps + (w * 32 + lane) * 4) = make_float4(pr[0], pr[1], pr[2], pr[3]);
    __syncwarp();
#pragma unroll 4
    for (int jj = 0; jj < AN; ++jj) {
      const float4 pp = *reinterpret_cast<const float4*>(Ps + (w * 32 + jj) * 4);
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        const float vv = Vs[jj * (HDP + 1) + lane + 32 * c];
        o[0][c] = fmaf(pp.x, vv, o[0][c]), o[1][c] = fmaf(pp.y, vv, o[1][c]);
        o[2][c] = fmaf(pp.z, vv, o[2][c]), o[3][c] = fmaf(pp.w, vv, o[3][c]);
      }
    }
    __syncwarp();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gi = i0 + w * 4 + i;
    if (gi >= p.Nq) continue;
    if (p.nsplit == 1) {
      const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
      T* orow = (T*)p.o + b * p.so.b + h * p.so.h + (int64_t)gi * p.so.n;
#pragma unroll
      for (int c = 0; c < DCH; ++c)
        if (lane + 32 * c < p.d) orow[lane + 32 * c] = from_f32<T>(o[i][c] * inv);
      if (lane == 0) p.lse[((int64_t)u * p.Nq) + gi] = l[i] > 0.f ? m[i] + logf(l[i]) : -CUDART_INF_F;
    } else {
      const int64_t slot = ((int64_t)u * p.nsplit + blockIdx.z) * p.Nq + gi;
#pragma unroll
      for (int c = 0; c < DCH; ++c) p.part_o[slot * HDP + lane + 32 * c] = o[i][c];
      if (lane == 0) p.part_ml[slot * 2] = m[i], p.part_ml[slot * 2 + 1] = l[i];
    }
  }
}

// Merge the per-split partial results: one warp per (unit, row).
template <typename T>
__global__ void attn_fwd_combine_kernel(AttnP p, int HDP) {
  // (behind the streaming decode kernel this one is launched as its programmatic dependent: wait for that grid before the
  // partials are read; after an ordinary launch the wait returns at once)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int64_t rowid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (rowid >= (int64_t)p.B * p.H * p.Nq) return;
  const int u = rowid / p.Nq, gi = rowid % p.Nq, b = u / p.H, h = u % p.H;
  float M = -CUDART_INF_F;
  for (int s = 0; s < p.nsplit; ++s) M = fmaxf(M, p.part_ml[(((int64_t)u * p.nsplit + s) * p.Nq + gi) * 2]);
  float L = 0.f;
  T* orow = (T*)p.o + b * p.so.b + h * p.so.h + (int64_t)gi * p.so.n;
  for (int c = lane; c < p.d; c += 32) {
    float acc = 0.f;
    L = 0.f;
    for (int s = 0; s < p.nsplit; ++s) {
      const int64_t slot = ((int64_t)u * p.nsplit + s) * p.Nq + gi;
      const float ms = p.part_ml[slot * 2], ls = p.part_ml[slot * 2 + 1];
      const float wgt = (ms == -CUDART_INF_F) ? 0.f : expf(ms - M);
      L += ls * wgt;
      acc += p.part_o[slot * HDP + c] * wgt;
    }
    orow[c] = from_f32<T>(L > 0.f ? acc / L : 0.f);
  }
  if (lane == 0) {
    L = 0.f;
    for (int s = 0; s < p.nsplit; ++s) {
      const int64_t slot = ((int64_t)u * p.nsplit + s) * p.Nq + gi;
      const float ms = p.part_ml[slot * 2];
      L += (ms == -CUDART_INF_F) ? 0.f : p.part_ml[slot * 2 + 1] * expf(ms - M);
    }
    p.lse[(int64_t)u * p.Nq + gi] = L > 0.f ? M + logf(L) : -CUDART_INF_F;
  }
}

// delta[u, i] = <out_i, dout_i>: one warp per row (PoPE_pytorch/triton_pope_flash_attn.py:119-130).
template <typename T>
__global__ void attn_bwd_delta_kernel(const T* out, Strides so, const T* dout, Strides sdo, float* delta, int B, int H,
                                      int Nq, int d) {
  const int lane = threadIdx.x & 31;
  const int64_t rowid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (rowid >= (int64_t)B * H * Nq) return;
  const int u = rowid / Nq, gi = rowid % Nq, b = u / H, h = u % H;
  const T* o = out + b * so.b + h * so.h + (int64_t)gi * so.n;
  const T* g = dout + b * sdo.b + h * sdo.h + (int64_t)gi * sdo.n;
  float acc = 0.f;
  for (int c = lane; c < d; c += 32) acc = fmaf(to_f32(o[c]), to_f32(g[c]), acc);
  acc = warp_sum(acc);
  if (lane == 0) delta[rowid] = acc;
}

template <typename T>
static cudaError_t delta_t(const PopeAttnBwdArgs& a, float* delta, cudaStream_t st) {
  const PopeShape& s = a.shape;
  const int64_t rows = (int64_t)s.B * s.H * s.Nq;
  attn_bwd_delta_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const T*)a.out, Strides(a.so), (const T*)a.dout,
                                                                      Strides(a.sdo), delta, s.B, s.H, s.Nq, s.d);
  return cudaGetLastError();
}
cudaError_t attn_bwd_delta(const PopeAttnBwdArgs& a, float* delta, cudaStream_t st) {
  switch (a.shape.dtype) {
    case POPE_F32: return delta_t<float>(a, delta, st);
    case POPE_BF16: return delta_t<__nv_bfloat16>(a, delta, st);
    default: return delta_t<__half>(a, delta, st);
  }
}

// ---- decode: one query row against a long key range ------------------------------------------------
// Memory-bound (every K and V row is read once per unit), so the work is laid out for coalescing: a warp
// takes one key at a time, lane l holds features 4l .. 4l+3 (and 128 + 4l .. for d > 128) of the key, of V and
// of the accumulator; the score is a warp reduction.  Key phases come from fp32 (cos f, sin f) tables built
// once per call and shared by all units, rotated by the head's bias held in registers.  Each (unit, key
// range) CTA writes a partial (o, m, l) that attn_fwd_combine_kernel merges.
constexpr int DEC_WARPS = 8;
constexpr int DEC_KU = 4;   // keys per warp and loop iteration

struct DecodeP {
  int H, Hk, Nk, d, r, nsplit, split_len;
  float scale;
  const void *q, *k, *v;
  Strides sq, sk, sv;
  const float *freqs, *bias, *ctab, *stab;   // freqs: query row only; tables: keys
  int64_t sfn, bias_sh;
  const uint8_t* mask;
  int64_t msb, msn;
  float *part_o, *part_ml;
  int HDP;
};

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&x)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&x)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  x[0] = a.x, x[1] = a.y, x[2] = a.z, x[3] = a.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[4]) {
  const uint2 a = *reinterpret_cast<const uint2*>(p);
  x[0] = __uint_as_float(a.x << 16), x[1] = __uint_as_float(a.x & 0xffff0000u);
  x[2] = __uint_as_float(a.y << 16), x[3] = __uint_as_float(a.y & 0xffff0000u);
}
template <> __device__ __forceinline__ void load4<__half>(const __half* p, float (&x)[4]) {
  const uint2 a = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&a.x)), hi = __half22float2(*reinterpret_cast<const __half2*>(&a.y));
  x[0] = lo.x, x[1] = lo.y, x[2] = hi.x, x[3] = hi.y;
}

template <typename T, int DM>   // DM = feature groups of 128 (1: d <= 128, 2: d <= 256)
__global__ void __launch_bounds__(DEC_WARPS * 32) attn_decode_kernel(DecodeP p) {
  __shared__ float red_o[DEC_WARPS][DM * 128];
  __shared__ float red_ml[DEC_WARPS][2];
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int u = blockIdx.y, b = u / p.H, h = u % p.H, hk = h % p.Hk;
  const T* qrow = (const T*)p.q + b * p.sq.b + h * p.sq.h;            // the single query row
  const T* kbase = (const T*)p.k + b * p.sk.b + hk * p.sk.h;
  const T* vbase = (const T*)p.v + b * p.sv.b + hk * p.sv.h;
  const uint8_t* mask = p.mask ? p.mask + b * p.msb : nullptr;
  const int kb = blockIdx.x * p.split_len, ke = min(p.Nk, kb + p.split_len);

  // this lane's slice of q' (exact transform, phase of the last position) and of the bias rotation
  float qc[DM][4], qs[DM][4], cb[DM][4], sb[DM][4];
  bool live[DM], rot[DM];
#pragma unroll
  for (int m = 0; m < DM; ++m) {
    const int c0 = m * 128 + lane * 4;
    live[m] = c0 < p.d, rot[m] = c0 < p.r;     // d and r are multiples of 4: a lane's 4 features share their fate
#pragma unroll
    for (int e = 0; e < 4; ++e) qc[m][e] = qs[m][e] = cb[m][e] = sb[m][e] = 0.f;
    if (live[m]) {
      float x[4];
      load4<T>(qrow + c0, x);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (rot[m]) {
          float sn, cs;
          sincosf(p.freqs[(int64_t)(p.Nk - 1) * p.sfn + c0 + e], &sn, &cs);
          const float a = softplus_f(x[e]);
          qc[m][e] = a * cs, qs[m][e] = a * sn;
          sincosf(p.bias[hk * p.bias_sh + c0 + e], &sb[m][e], &cb[m][e]);
        } else {
          qc[m][e] = x[e];
        }
      }
    }
  }

  float mrun = -CUDART_INF_F, lrun = 0.f, o[DM][4];
#pragma unroll
  for (int m = 0; m < DM; ++m)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[m][e] = 0.f;

  // DEC_KU keys per warp and iteration: their loads are issued together, their warp reductions interleave, and
  // the running maximum / rescale of the accumulator is paid once per group instead of once per key.
  for (int j0 = kb + w; j0 < ke; j0 += DEC_WARPS * DEC_KU) {
    float part[DEC_KU], vv[DEC_KU][DM][4];
    bool ok[DEC_KU];
#pragma unroll
    for (int u = 0; u < DEC_KU; ++u) {
      const int j = j0 + u * DEC_WARPS;
      const bool in = j < ke;
      ok[u] = in && (!mask || mask[(int64_t)j * p.msn] != 0);   // warp-uniform
      part[u] = 0.f;
#pragma unroll
      for (int m = 0; m < DM; ++m) {
        const int c0 = m * 128 + lane * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) vv[u][m][e] = 0.f;
        if (!live[m] || !in) continue;
        float x[4];
        load4<T>(kbase + (int64_t)j * p.sk.n + c0, x);
        load4<T>(vbase + (int64_t)j * p.sv.n + c0, vv[u][m]);
        if (rot[m]) {
          float ct[4], stt[4];
          load4<float>(p.ctab + (int64_t)j * p.r + c0, ct);
          load4<float>(p.stab + (int64_t)j * p.r + c0, stt);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float a = softplus_fast(x[e]);   // ex2.approx / lg2.approx: 2^-22, a sixth of the instructions
            const float kc = a * (ct[e] * cb[m][e] - stt[e] * sb[m][e]);
            const float ks = a * (stt[e] * cb[m][e] + ct[e] * sb[m][e]);
            part[u] = fmaf(qc[m][e], kc, fmaf(qs[m][e], ks, part[u]));
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) part[u] = fmaf(qc[m][e], x[e], part[u]);
        }
      }
    }
    float sc[DEC_KU], mnew = mrun;
#pragma unroll
    for (int u = 0; u < DEC_KU; ++u) {
      sc[u] = ok[u] ? warp_sum(part[u]) * p.scale : -CUDART_INF_F;
      mnew = fmaxf(mnew, sc[u]);
    }
    if (mnew == -CUDART_INF_F) continue;   // nothing visible so far (warp-uniform)
    const float alpha = expf(mrun - mnew);   // exp(-inf) = 0 on the first visible group
    float pj[DEC_KU], psum = 0.f;
#pragma unroll
    for (int u = 0; u < DEC_KU; ++u) pj[u] = expf(sc[u] - mnew), psum += pj[u];
    lrun = lrun * alpha + psum;
    mrun = mnew;
#pragma unroll
    for (int m = 0; m < DM; ++m)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float acc = o[m][e] * alpha;
#pragma unroll
        for (int u = 0; u < DEC_KU; ++u) acc = fmaf(pj[u], vv[u][m][e], acc);
        o[m][e] = acc;
      }
  }

  // merge the 8 warps of the CTA, then hand the partial to the cross-split combine
#pragma unroll
  for (int m = 0; m < DM; ++m)
#pragma unroll
    for (int e = 0; e < 4; ++e) red_o[w][m * 128 + lane * 4 + e] = o[m][e];
  if (lane == 0) red_ml[w][0] = mrun, red_ml[w][1] = lrun;
  __syncthreads();
  float M = -CUDART_INF_F;
#pragma unroll
  for (int ww = 0; ww < DEC_WARPS; ++ww) M = fmaxf(M, red_ml[ww][0]);
  const int64_t slot = (int64_t)u * p.nsplit + blockIdx.x;     // Nq = 1
  for (int c = tid; c < p.HDP; c += DEC_WARPS * 32) {
    float acc = 0.f;
    if (c < DM * 128)
#pragma unroll
      for (int ww = 0; ww < DEC_WARPS; ++ww)
        acc += red_ml[ww][0] == -CUDART_INF_F ? 0.f : red_o[ww][c] * expf(red_ml[ww][0] - M);
    p.part_o[slot * p.HDP + c] = acc;
  }
  if (tid == 0) {
    float L = 0.f;
#pragma unroll
    for (int ww = 0; ww < DEC_WARPS; ++ww) L += red_ml[ww][0] == -CUDART_INF_F ? 0.f : red_ml[ww][1] * expf(red_ml[ww][0] - M);
    p.part_ml[slot * 2] = M, p.part_ml[slot * 2 + 1] = L;
  }
}

static bool decode_applies(const PopeAttnArgs& a) {
  const PopeShape& s = a.shape;
  if (s.Nq != 1 || a.causal || s.Nk < 1024 || s.d > 256 || s.d % 4 != 0 || s.r % 4 != 0) return false;
  if (s.r > 0 && (a.embed.sf.b != 0 || a.embed.sf.h != 0)) return false;
  const int esz = s.dtype == POPE_F32 ? 4 : 2;
  auto ok = [&](const void* ptr, const PopeStride3& st) {
    const int al = 4 * esz;   // 4 features per lane
    return reinterpret_cast<uintptr_t>(ptr) % al == 0 && (st.b * esz) % al == 0 && (st.h * esz) % al == 0 && (st.n * esz) % al == 0;
  };
  return ok(a.q, a.sq) && ok(a.k, a.sk) && ok(a.v, a.sv);
}

static void decode_plan(const PopeShape& s, int& nsplit, int& split_len) {
  const int64_t units = (int64_t)s.B * s.H;
  int want = (int)((8 * 148 + units - 1) / units);      // about eight CTAs per SM in flight
  const int maxs = s.Nk / 256;
  nsplit = want < maxs ? want : maxs;
  if (nsplit < 1) nsplit = 1;
  split_len = (s.Nk + nsplit - 1) / nsplit;
  nsplit = (s.Nk + split_len - 1) / split_len;
}

cudaError_t launch_trig_table_f32(const PopeEmbed& e, int n, int r, float* ctab, float* stab, cudaStream_t st);

// ---- forward launch --------------------------------------------------------------------------
static void plan_split(const PopeShape& s, int causal, int& nsplit, int& split_len) {
  // Few query tiles against a long key range: split the keys so every SM has work.
  const int64_t ctas = (int64_t)((s.Nq + AM - 1) / AM) * s.B * s.H;
  nsplit = 1, split_len = s.Nk;
  if (!causal && ctas < 2 * 148 && s.Nk >= 2048) {
    int want = (int)((4 * 148 + ctas - 1) / ctas);
    int maxs = s.Nk / 512;
    nsplit = want < maxs ? want : maxs;
    if (nsplit < 1) nsplit = 1;
    split_len = round_up((s.Nk + nsplit - 1) / nsplit, AN);
    nsplit = (s.Nk + split_len - 1) / split_len;
  }
}

size_t attn_fwd_simt_workspace(const PopeAttnArgs& a) {
  if (decode_applies(a)) {
    int dns, dsl;
    decode_plan(a.shape, dns, dsl);
    const int HDP = simt_dch(a.shape.d) * 32;
    const size_t slots = (size_t)a.shape.B * a.shape.H * dns;
    return slots * (HDP + 2) * sizeof(float) + 256 + (size_t)a.shape.Nk * a.shape.r * 2 * sizeof(float);
  }
  int ns, sl;
  plan_split(a.shape, a.causal, ns, sl);
  if (ns == 1) return 0;
  const int HDP = simt_dch(a.shape.d) * 32;
  const size_t slots = (size_t)a.shape.B * a.shape.H * ns * a.shape.Nq;
  return slots * (HDP + 2) * sizeof(float);
}

template <typename T, int DCH>
static cudaError_t launch_attn_fwd(const PopeAttnArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  AttnP p = {};
  p.B = s.B, p.H = s.H, p.Hk = s.Hk, p.Nq = s.Nq, p.Nk = s.Nk, p.d = s.d, p.r = s.r;
  p.causal = a.causal, p.scale = a.softmax_scale;
  plan_split(s, a.causal, p.nsplit, p.split_len);
  p.q = a.q, p.k = a.k, p.v = a.v, p.sq = a.sq, p.sk = a.sk, p.sv = a.sv, p.so = a.so, p.sf = a.embed.sf;
  p.freqs = a.embed.freqs, p.bias = a.embed.bias, p.bias_sh = a.embed.bias_stride_h;
  p.mask = a.mask, p.msb = a.mask_stride_b, p.msn = a.mask_stride_n;
  p.o = a.out, p.lse = a.lse;
  const int HDP = DCH * 32, RP = round_up(s.r, 32), KD = HDP + RP;
  if (p.nsplit > 1) {
    const size_t slots = (size_t)s.B * s.H * p.nsplit * s.Nq;
    p.part_o = (float*)a.workspace;
    p.part_ml = p.part_o + slots * HDP;
  }
  const size_t smem = sizeof(float) * ((size_t)KD * 32 + 32 * (KD + 1) + 32 * (HDP + 1) + 8 * 32 * 4);
  cudaError_t e = cudaFuncSetAttribute(attn_fwd_simt_kernel<T, DCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid((s.Nq + AM - 1) / AM, s.B * s.H, p.nsplit);
  attn_fwd_simt_kernel<T, DCH><<<grid, 256, smem, st>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess || p.nsplit == 1) return e;
  const int64_t rows = (int64_t)s.B * s.H * s.Nq;
  attn_fwd_combine_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(p, HDP);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_decode(const PopeAttnArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  DecodeP p = {};
  p.H = s.H, p.Hk = s.Hk, p.Nk = s.Nk, p.d = s.d, p.r = s.r, p.scale = a.softmax_scale;
  decode_plan(s, p.nsplit, p.split_len);
  p.q = a.q, p.k = a.k, p.v = a.v, p.sq = a.sq, p.sk = a.sk, p.sv = a.sv;
  p.freqs = a.embed.freqs, p.bias = a.embed.bias, p.sfn = a.embed.sf.n, p.bias_sh = a.embed.bias_stride_h;
  p.mask = a.mask, p.msb = a.mask_stride_b, p.msn = a.mask_stride_n;
  p.HDP = simt_dch(s.d) * 32;
  const size_t slots = (size_t)s.B * s.H * p.nsplit;
  p.part_o = (float*)a.workspace;
  p.part_ml = p.part_o + slots * p.HDP;
  float* ctab = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(a.workspace) + (slots * (p.HDP + 2) * sizeof(float) + 255) / 256 * 256);
  float* stab = ctab + (size_t)s.Nk * s.r;
  p.ctab = ctab, p.stab = stab;
  cudaError_t e = cudaSuccess;
  if (s.r > 0 && (e = launch_trig_table_f32(a.embed, s.Nk, s.r, ctab, stab, st)) != cudaSuccess) return e;
  dim3 grid(p.nsplit, s.B * s.H);
  if (s.d <= 128) attn_decode_kernel<T, 1><<<grid, DEC_WARPS * 32, 0, st>>>(p);
  else attn_decode_kernel<T, 2><<<grid, DEC_WARPS * 32, 0, st>>>(p);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  AttnP c = {};
  c.B = s.B, c.H = s.H, c.Nq = 1, c.d = s.d, c.nsplit = p.nsplit, c.so = a.so, c.o = a.out, c.lse = a.lse;
  c.part_o = p.part_o, c.part_ml = p.part_ml;
  const int64_t rows = (int64_t)s.B * s.H;
  attn_fwd_combine_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(c, p.HDP);
  return cudaGetLastError();
}

// Merge of per-split partials (one query row per unit) for the streaming decode kernel.
cudaError_t launch_split_combine(const PopeAttnArgs& a, int nsplit, float* part_o, float* part_ml, cudaStream_t st) {
  const PopeShape& s = a.shape;
  AttnP c = {};
  c.B = s.B, c.H = s.H, c.Nq = s.Nq, c.d = s.d, c.nsplit = nsplit, c.so = a.so, c.o = a.out, c.lse = a.lse;
  c.part_o = part_o, c.part_ml = part_ml;
  const int HDP = simt_dch(s.d) * 32;
  const int64_t rows = (int64_t)s.B * s.H * s.Nq;
  const unsigned blocks = (unsigned)((rows + 7) / 8);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks), cfg.blockDim = dim3(256), cfg.dynamicSmemBytes = 0, cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  switch (s.dtype) {
    case POPE_F32: return cudaLaunchKernelEx(&cfg, attn_fwd_combine_kernel<float>, c, HDP);
    case POPE_BF16: return cudaLaunchKernelEx(&cfg, attn_fwd_combine_kernel<__nv_bfloat16>, c, HDP);
    default: return cudaLaunchKernelEx(&cfg, attn_fwd_combine_kernel<__half>, c, HDP);
  }
}

template <typename T>
static cudaError_t attn_fwd_dch(const PopeAttnArgs& a, cudaStream_t st) {
  if (a.shape.d > 256) return cudaErrorInvalidValue;
  if (decode_applies(a)) return launch_decode<T>(a, st);
  switch (simt_dch(a.shape.d)) {
    case 1: return launch_attn_fwd<T, 1>(a, st);
    case 2: return launch_attn_fwd<T, 2>(a, st);
    case 3: return launch_attn_fwd<T, 3>(a, st);
    case 4: return launch_attn_fwd<T, 4>(a, st);
    default: return launch_attn_fwd<T, 8>(a, st);
  }
}

cudaError_t attn_fwd_simt(const PopeAttnArgs& a, cudaStream_t st) {
  switch (a.shape.dtype) {
    case POPE_F32: return attn_fwd_dch<float>(a, st);
    case POPE_BF16: return attn_fwd_dch<__nv_bfloat16>(a, st);
    default: return attn_fwd_dch<__half>(a, st);
  }
}

}  // namespace pope

#include "simt_attn_bwd.inl"
