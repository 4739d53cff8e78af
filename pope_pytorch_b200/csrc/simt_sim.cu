// Full-precision (fp32 FMA) similarity kernels: sim = q' k'^T and its backward.
// These are the exact-arithmetic family: every shape, stride and dtype the C ABI accepts runs
// here; the tensor-core family takes over the shapes it implements.
//
// Reference semantics: PoPE_pytorch/triton_pope.py:28-83 (forward), :85-256 (backward).
#include "common.cuh"
#include "kernels.h"

namespace pope {

struct SimP {
  int B, H, Hk, Nq, Nk, d, r;
  const void *q, *k;
  Strides sq, sk, sf, ss;
  const float *freqs, *bias;
  int64_t bias_sh;
  void* sim;
};

constexpr int ST = 64;   // output tile edge
constexpr int SFC = 16;  // features per staging step
constexpr int SLD = ST + 4;

// Stage SFC features of 64 rows into feature-major shared tiles, applying the PoPE transform:
// c < r: (a cos, a sin); r <= c < d: (x, 0); else zeros.
template <typename T>
__device__ __forceinline__ void stage_rows(float (*C)[SLD], float (*S)[SLD], const T* base, int64_t srow,
                                           const float* fbase, int64_t frow, const float* bias, int row0,
                                           int nrows, int pos0, int c0, int d, int r, int tid) {
  const int row = tid & 63, cg = tid >> 6;
  const int grow = row0 + row;
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    const int c = c0 + cg * 4 + kk;
    float vc = 0.f, vs = 0.f;
    if (grow < nrows && c < d) {
      float x = to_f32(base[(int64_t)grow * srow + c]);
      if (c < r) {
        float th = fbase[(int64_t)(pos0 + grow) * frow + c];
        if (bias) th += bias[c];
        float sn, cs;
        sincosf(th, &sn, &cs);
        float a = softplus_f(x);
        vc = a * cs;
        vs = a * sn;
      } else {
        vc = x;
      }
    }
    C[cg * 4 + kk][row] = vc;
    S[cg * 4 + kk][row] = vs;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) sim_fwd_simt_kernel(SimP p) {
  __shared__ __align__(16) float Qc[SFC][SLD], Qs[SFC][SLD], Kc[SFC][SLD], Ks[SFC][SLD];
  const int tid = threadIdx.x;
  const int u = blockIdx.z, b = u / p.H, h = u % p.H, hk = h % p.Hk;
  const int i0 = blockIdx.y * ST, j0 = blockIdx.x * ST;
  const T* q = (const T*)p.q + b * p.sq.b + h * p.sq.h;
  const T* k = (const T*)p.k + b * p.sk.b + hk * p.sk.h;
  const float* fq = p.freqs ? p.freqs + b * p.sf.b + h * p.sf.h : nullptr;
  const float* fk = p.freqs ? p.freqs + b * p.sf.b + hk * p.sf.h : nullptr;
  const float* bias = p.r > 0 ? p.bias + hk * p.bias_sh : nullptr;
  const int qoff = p.Nk - p.Nq;

  float acc[4][4] = {};
  const int ty = tid >> 4, tx = tid & 15;
  for (int c0 = 0; c0 < p.d; c0 += SFC) {
    stage_rows<T>(Qc, Qs, q, p.sq.n, fq, p.sf.n, nullptr, i0, p.Nq, qoff, c0, p.d, p.r, tid);
    stage_rows<T>(Kc, Ks, k, p.sk.n, fk, p.sf.n, bias, j0, p.Nk, 0, c0, p.d, p.r, tid);
    __syncthreads();
    const bool has_sin = c0 < p.r;
#pragma unroll
    for (int c = 0; c < SFC; ++c) {
      float4 a = *reinterpret_cast<const float4*>(&Qc[c][ty * 4]);
      float4 bb = *reinterpret_cast<const float4*>(&Kc[c][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      if (has_sin) {
        float4 a2 = *reinterpret_cast<const float4*>(&Qs[c][ty * 4]);
        float4 b2 = *reinterpret_cast<const float4*>(&Ks[c][tx * 4]);
        const float av2[4] = {a2.x, a2.y, a2.z, a2.w}, bv2[4] = {b2.x, b2.y, b2.z, b2.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av2[i], bv2[j], acc[i][j]);
      }
    }
    __syncthreads();
  }
  T* out = (T*)p.sim + b * p.ss.b + h * p.ss.h;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gi = i0 + ty * 4 + i;
    if (gi >= p.Nq) continue;
    T* row = out + (int64_t)gi * p.ss.n;
    const int gj = j0 + tx * 4;
    if (sizeof(T) == 4 && gj + 3 < p.Nk && ((reinterpret_cast<uintptr_t>(row + gj) & 15) == 0)) {
      *reinterpret_cast<float4*>(row + gj) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (gj + j < p.Nk) row[gj + j] = from_f32<T>(acc[i][j]);
    }
  }
}

// ---- backward ------------------------------------------------------------------------------
struct SimBwdP {
  int B, H, Hk, Nq, Nk, d, r;
  const void *q, *k, *ds;
  Strides sq, sk, sf, sds, sdq, sdk, sdf;
  const float *freqs, *bias;
  int64_t bias_sh, dbias_sh;
  void *dq, *dk;
  float *dfreqs, *dbias;
};

constexpr int BR = 64;  // output rows per CTA
constexpr int BF = 16;  // output features per CTA
constexpr int BI = 32;  // inner (contracted) rows per step

// One CTA produces 64 rows x 16 features of dq (KEY_SIDE = false) or dk (KEY_SIDE = true):
//   dXc = G Yc, dXs = G Ys with G = dS (or dS^T) and Y the transformed opposite operand, then
//   dx = (dXc cos + dXs sin) sigmoid(x), dphase = a (dXs cos - dXc sin)   for c < r
//   dx = dXc                                                                 otherwise
// (PoPE_pytorch/triton_pope.py:129-151, 174-194, 246-256).
template <typename T, bool KEY_SIDE>
__global__ void __launch_bounds__(256) sim_bwd_simt_kernel(SimBwdP p) {
  __shared__ float G[BR][BI + 1];
  __shared__ float Yc[BI][BF], Ys[BI][BF];
  __shared__ float red[16][BF];
  const int tid = threadIdx.x;
  const int u = blockIdx.z;
  const int R = KEY_SIDE ? p.Nk : p.Nq;          // rows of the output
  const int NI = KEY_SIDE ? p.Nq : p.Nk;         // inner length per head
  const int heads_out = KEY_SIDE ? p.Hk : p.H;
  const int b = u / heads_out, ho = u % heads_out;
  const int hk = KEY_SIDE ? ho : ho % p.Hk;
  const int groups = KEY_SIDE ? p.H / p.Hk : 1;
  const int row0 = blockIdx.x * BR, c0 = blockIdx.y * BF;
  const int qoff = p.Nk - p.Nq;
  const float* bias = p.r > 0 ? p.bias + hk * p.bias_sh : nullptr;
  // phases of the row operand (head ho) and, per group, of the contracted operand
  const float* f_row = p.r > 0 ? p.freqs + b * p.sf.b + ho * p.sf.h : nullptr;

  const int rg = tid >> 4, fx = tid & 15;  // 4 rows x 1 feature per thread
  float ac[4] = {}, as[4] = {};
  const bool has_sin = c0 < p.r;

  for (int g = 0; g < groups; ++g) {
    const int hq = KEY_SIDE ? g * p.Hk + hk : ho;
    const T* ds = (const T*)p.ds + b * p.sds.b + hq * p.sds.h;
    // the operand being contracted: keys for dq, queries for dk
    const T* y = KEY_SIDE ? (const T*)p.q + b * p.sq.b + hq * p.sq.h : (const T*)p.k + b * p.sk.b + hk * p.sk.h;
    const int64_t ysn = KEY_SIDE ? p.sq.n : p.sk.n;
    const int ypos0 = KEY_SIDE ? qoff : 0;
    const float* f = p.r > 0 ? p.freqs + b * p.sf.b + (KEY_SIDE ? hq : hk) * p.sf.h : nullptr;
    for (int n0 = 0; n0 < NI; n0 += BI) {
      // G tile
      if (KEY_SIDE) {  // G[row j][inner i] = dS[i][j]; j contiguous in memory
        const int row = tid & 63;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const int in = (tid >> 6) + kk * 4;
          const int gi = n0 + in, gj = row0 + row;
          G[row][in] = (gi < NI && gj < R) ? to_f32(ds[(int64_t)gi * p.sds.n + gj]) : 0.f;
        }
      } else {  // G[row i][inner j] = dS[i][j]
        const int in = tid & 31;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const int row = (tid >> 5) + kk * 8;
          const int gi = row0 + row, gj = n0 + in;
          G[row][in] = (gi < R && gj < NI) ? to_f32(ds[(int64_t)gi * p.sds.n + gj]) : 0.f;
        }
      }
      // transformed Y tile: 32 inner rows x 16 features
      {
        const int in = tid >> 3;
        const int gn = n0 + in;
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const int fl = (tid & 7) * 2 + kk, c = c0 + fl;
          float vc = 0.f, vs = 0.f;
          if (gn < NI && c < p.d) {
            float x = to_f32(y[(int64_t)gn * ysn + c]);
            if (c < p.r) {
              float th = f[(int64_t)(ypos0 + gn) * p.sf.n + c];
              if (!KEY_SIDE) th += bias[c];
              float sn, cs;
              sincosf(th, &sn, &cs);
              float a = softplus_f(x);
              vc = a * cs, vs = a * sn;
            } else {
              vc = x;
            }
          }
          Yc[in][fl] = vc, Ys[in][fl] = vs;
        }
      }
      __syncthreads();
#pragma unroll 8
      for (int in = 0; in < BI; ++in) {
        const float yc = Yc[in][fx], ys = Ys[in][fx];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float gv = G[rg * 4 + i][in];
          ac[i] = fmaf(gv, yc, ac[i]);
          if (has_sin) as[i] = fmaf(gv, ys, as[i]);
        }
      }
      __syncthreads();
    }
  }

  // epilogue: chain rule through the transform of the row operand
  const int c = c0 + fx;
  const T* x = KEY_SIDE ? (const T*)p.k + b * p.sk.b + ho * p.sk.h : (const T*)p.q + b * p.sq.b + ho * p.sq.h;
  const int64_t xsn = KEY_SIDE ? p.sk.n : p.sq.n;
  T* dx = KEY_SIDE ? (T*)p.dk + b * p.sdk.b + ho * p.sdk.h : (T*)p.dq + b * p.sdq.b + ho * p.sdq.h;
  const int64_t dxsn = KEY_SIDE ? p.sdk.n : p.sdq.n;
  const int pos0 = KEY_SIDE ? 0 : qoff;
  float dphase_sum = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gr = row0 + rg * 4 + i;
    if (gr >= R || c >= p.d) continue;
    float g = ac[i];
    if (c < p.r) {
      const float xv = to_f32(x[(int64_t)gr * xsn + c]);
      float th = f_row[(int64_t)(pos0 + gr) * p.sf.n + c];
      if (KEY_SIDE) th += bias[c];
      float sn, cs;
      sincosf(th, &sn, &cs);
      const float a = softplus_f(xv);
      g = (ac[i] * cs + as[i] * sn) * sigmoid_f(xv);
      const float dph = a * (as[i] * cs - ac[i] * sn);
      dphase_sum += dph;
      if (p.dfreqs) atomicAdd(p.dfreqs + b * p.sdf.b + ho * p.sdf.h + (int64_t)(pos0 + gr) * p.sdf.n + c, dph);
    }
    dx[(int64_t)gr * dxsn + c] = from_f32<T>(g);
  }
  if (KEY_SIDE && p.dbias && has_sin) {  // block-uniform condition
    red[rg][fx] = dphase_sum;
    __syncthreads();
    if (tid < BF) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) s += red[i][tid];
      if (c0 + tid < p.r) atomicAdd(p.dbias + hk * p.dbias_sh + c0 + tid, s);
    }
  }
}

template <typename T>
static cudaError_t launch_sim_fwd(const PopeSimArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  SimP p;
  p.B = s.B, p.H = s.H, p.Hk = s.Hk, p.Nq = s.Nq, p.Nk = s.Nk, p.d = s.d, p.r = s.r;
  p.q = a.q, p.k = a.k, p.sq = a.sq, p.sk = a.sk, p.sf = a.embed.sf, p.ss = a.ss;
  p.freqs = s.r > 0 ? a.embed.freqs : nullptr, p.bias = a.embed.bias, p.bias_sh = a.embed.bias_stride_h;
  p.sim = a.sim;
  dim3 grid((s.Nk + ST - 1) / ST, (s.Nq + ST - 1) / ST, s.B * s.H);
  sim_fwd_simt_kernel<T><<<grid, 256, 0, st>>>(p);
  return cudaGetLastError();
}

cudaError_t sim_fwd_simt(const PopeSimArgs& a, cudaStream_t st) {
  switch (a.shape.dtype) {
    case POPE_F32: return launch_sim_fwd<float>(a, st);
    case POPE_BF16: return launch_sim_fwd<__nv_bfloat16>(a, st);
    default: return launch_sim_fwd<__half>(a, st);
  }
}

template <typename T>
static cudaError_t launch_sim_bwd(const PopeSimBwdArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  SimBwdP p;
  p.B = s.B, p.H = s.H, p.Hk = s.Hk, p.Nq = s.Nq, p.Nk = s.Nk, p.d = s.d, p.r = s.r;
  p.q = a.q, p.k = a.k, p.ds = a.dsim;
  p.sq = a.sq, p.sk = a.sk, p.sf = a.embed.sf, p.sds = a.sds, p.sdq = a.sdq, p.sdk = a.sdk, p.sdf = a.sdf;
  p.freqs = a.embed.freqs, p.bias = a.embed.bias, p.bias_sh = a.embed.bias_stride_h, p.dbias_sh = a.dbias_stride_h;
  p.dq = a.dq, p.dk = a.dk, p.dfreqs = s.r > 0 ? a.dfreqs : nullptr, p.dbias = s.r > 0 ? a.dbias : nullptr;
  const int fchunks = (s.d + BF - 1) / BF;
  dim3 gq((s.Nq + BR - 1) / BR, fchunks, s.B * s.H);
  sim_bwd_simt_kernel<T, false><<<gq, 256, 0, st>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  dim3 gk((s.Nk + BR - 1) / BR, fchunks, s.B * s.Hk);
  sim_bwd_simt_kernel<T, true><<<gk, 256, 0, st>>>(p);
  return cudaGetLastError();
}

cudaError_t sim_bwd_simt(const PopeSimBwdArgs& a, cudaStream_t st) {
  switch (a.shape.dtype) {
    case POPE_F32: return launch_sim_bwd<float>(a, st);
    case POPE_BF16: return launch_sim_bwd<__nv_bfloat16>(a, st);
    default: return launch_sim_bwd<__half>(a, st);
  }
}

}  // namespace pope
