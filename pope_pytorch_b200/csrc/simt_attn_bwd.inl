// Backward of the fp32 PoPE attention family (included by simt_attn.cu).
//
// Two kernels, no atomics on dq/dk/dv, deterministic:
//   dq   : each CTA owns 32 query rows and sweeps the key tiles
//   dkdv : each CTA owns 32 key rows and sweeps the query tiles (all query heads of its group)
// Both recompute P = exp(S*scale - lse) and dS = P (dP - delta) scale
// (PoPE_pytorch/triton_pope_flash_attn.py:190-199) and finish with the chain rule through the
// transform (:202-210).  dfreqs / dbias are accumulated with fp32 atomics when requested.
namespace pope {

template <typename T, int DCH>
__global__ void __launch_bounds__(256) attn_bwd_dq_simt_kernel(AttnP p) {
  extern __shared__ __align__(16) float smem[];
  const int HDP = DCH * 32, RP = (p.r + 31) / 32 * 32, KD = HDP + RP, RCH = RP / 32;
  float* QT = smem;                     // [KD][32]   transformed queries, feature-major
  float* GT = QT + KD * 32;             // [HDP][32]  dout, feature-major
  float* Ks = GT + HDP * 32;            // [32][KD+1]
  float* Vs = Ks + 32 * (KD + 1);       // [32][HDP+1]
  float* Ds = Vs + 32 * (HDP + 1);      // [8][32][4]
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int u = blockIdx.y, b = u / p.H, h = u % p.H, hk = h % p.Hk;
  const int i0 = blockIdx.x * AM;
  const int qoff = p.Nk - p.Nq;
  const T* q = (const T*)p.q + b * p.sq.b + h * p.sq.h;
  const T* k = (const T*)p.k + b * p.sk.b + hk * p.sk.h;
  const T* v = (const T*)p.v + b * p.sv.b + hk * p.sv.h;
  const T* g = (const T*)p.dout + b * p.sdo.b + h * p.sdo.h;
  const float* fq = p.r > 0 ? p.freqs + b * p.sf.b + h * p.sf.h : nullptr;
  const float* fk = p.r > 0 ? p.freqs + b * p.sf.b + hk * p.sf.h : nullptr;
  const float* bias = p.r > 0 ? p.bias + hk * p.bias_sh : nullptr;
  const uint8_t* mask = p.mask ? p.mask + b * p.msb : nullptr;

  stage_feature_major<T>(QT, q, p.sq.n, fq, p.sf.n, nullptr, i0, p.Nq, qoff, p.d, p.r, HDP, RP, tid);
  stage_plain_feature_major<T>(GT, g, p.sdo.n, i0, p.Nq, p.d, HDP, tid);

  float lse[4], dl[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gi = i0 + w * 4 + i;
    lse[i] = gi < p.Nq ? p.lse_in[(int64_t)u * p.Nq + gi] : -CUDART_INF_F;
    dl[i] = gi < p.Nq ? p.delta[(int64_t)u * p.Nq + gi] : 0.f;
  }
  float dqc[4][DCH], dqs[4][DCH];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < DCH; ++c) dqc[i][c] = 0.f, dqs[i][c] = 0.f;

  int ke = p.Nk;
  if (p.causal) ke = min(ke, min(i0 + AM, p.Nq));
  for (int n0 = 0; n0 < ke; n0 += AN) {
    __syncthreads();
    stage_row_major<T>(Ks, KD + 1, k, p.sk.n, fk, p.sf.n, bias, n0, ke, 0, p.d, p.r, HDP, RP, tid);
    stage_plain_row_major<T>(Vs, HDP + 1, v, p.sv.n, n0, ke, p.d, HDP, tid);
    __syncthreads();
    float s[4], dp[4];
    dot4(QT, w, Ks + lane * (KD + 1), KD, s);
    dot4(GT, w, Vs + lane * (HDP + 1), HDP, dp);
    const int j = n0 + lane;
    const bool key_ok = j < ke && (!mask || mask[(int64_t)j * p.msn]);
    float ds[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int gi = i0 + w * 4 + i;
      const bool ok = key_ok && (!p.causal || j <= gi) && lse[i] != -CUDART_INF_F;
      const float pv = ok ? expf(s[i] * p.scale - lse[i]) : 0.f;
      ds[i] = pv * (dp[i] - dl[i]) * p.scale;
    }
    *reinterpret_cast<float4*>(Ds + (w * 32 + lane) * 4) = make_float4(ds[0], ds[1], ds[2], ds[3]);
    __syncwarp();
#pragma unroll 2
    for (int jj = 0; jj < AN; ++jj) {
      const float4 dd = *reinterpret_cast<const float4*>(Ds + (w * 32 + jj) * 4);
      const float* krow = Ks + jj * (KD + 1) + lane;
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        const float kc = krow[32 * c];
        dqc[0][c] = fmaf(dd.x, kc, dqc[0][c]), dqc[1][c] = fmaf(dd.y, kc, dqc[1][c]);
        dqc[2][c] = fmaf(dd.z, kc, dqc[2][c]), dqc[3][c] = fmaf(dd.w, kc, dqc[3][c]);
        if (c < RCH) {
          const float ks = krow[HDP + 32 * c];
          dqs[0][c] = fmaf(dd.x, ks, dqs[0][c]), dqs[1][c] = fmaf(dd.y, ks, dqs[1][c]);
          dqs[2][c] = fmaf(dd.z, ks, dqs[2][c]), dqs[3][c] = fmaf(dd.w, ks, dqs[3][c]);
        }
      }
    }
    __syncwarp();
  }

  T* dq = (T*)p.dq + b * p.sdq.b + h * p.sdq.h;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gi = i0 + w * 4 + i;
    if (gi >= p.Nq) continue;
#pragma unroll
    for (int cc = 0; cc < DCH; ++cc) {
      const int c = lane + 32 * cc;
      if (c >= p.d) continue;
      float gq = dqc[i][cc];
      if (c < p.r) {
        const float x = to_f32(q[(int64_t)gi * p.sq.n + c]);
        const float th = fq[(int64_t)(qoff + gi) * p.sf.n + c];
        float sn, cs;
        sincosf(th, &sn, &cs);
        gq = (dqc[i][cc] * cs + dqs[i][cc] * sn) * sigmoid_f(x);
        if (p.dfreqs) {
          const float dph = softplus_f(x) * (dqs[i][cc] * cs - dqc[i][cc] * sn);
          atomicAdd(p.dfreqs + b * p.sdf.b + h * p.sdf.h + (int64_t)(qoff + gi) * p.sdf.n + c, dph);
        }
      }
      dq[(int64_t)gi * p.sdq.n + c] = from_f32<T>(gq);
    }
  }
}

template <typename T, int DCH>
__global__ void __launch_bounds__(256) attn_bwd_dkdv_simt_kernel(AttnP p) {
  extern __shared__ __align__(16) float smem[];
  const int HDP = DCH * 32, RP = (p.r + 31) / 32 * 32, KD = HDP + RP, RCH = RP / 32;
  float* KT = smem;                     // [KD][32]   transformed keys, feature-major
  float* VT = KT + KD * 32;             // [HDP][32]
  float* Qs = VT + HDP * 32;            // [32][KD+1] transformed queries of the current tile
  float* Gs = Qs + 32 * (KD + 1);       // [32][HDP+1] dout of the current tile
  float* Ps = Gs + 32 * (HDP + 1);      // [8][32][4]
  float* Ds = Ps + 8 * 32 * 4;          // [8][32][4]
  float* Ls = Ds + 8 * 32 * 4;          // [32] lse, [32] delta
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int u = blockIdx.y, b = u / p.Hk, hk = u % p.Hk;
  const int j0 = blockIdx.x * AM;
  const int qoff = p.Nk - p.Nq;
  const int groups = p.H / p.Hk;
  const T* k = (const T*)p.k + b * p.sk.b + hk * p.sk.h;
  const T* v = (const T*)p.v + b * p.sv.b + hk * p.sv.h;
  const float* fk = p.r > 0 ? p.freqs + b * p.sf.b + hk * p.sf.h : nullptr;
  const float* bias = p.r > 0 ? p.bias + hk * p.bias_sh : nullptr;
  const uint8_t* mask = p.mask ? p.mask + b * p.msb : nullptr;

  stage_feature_major<T>(KT, k, p.sk.n, fk, p.sf.n, bias, j0, p.Nk, 0, p.d, p.r, HDP, RP, tid);
  stage_plain_feature_major<T>(VT, v, p.sv.n, j0, p.Nk, p.d, HDP, tid);

  bool key_ok[4];
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    const int j = j0 + w * 4 + kk;
    key_ok[kk] = j < p.Nk && (!mask || mask[(int64_t)j * p.msn]);
  }
  float dv[4][DCH], dkc[4][DCH], dks[4][DCH];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < DCH; ++c) dv[i][c] = 0.f, dkc[i][c] = 0.f, dks[i][c] = 0.f;

  const int m_begin = p.causal ? (j0 / AN) * AN : 0;  // rows i < j see nothing of this key tile
  for (int gidx = 0; gidx < groups; ++gidx) {
    const int h = gidx * p.Hk + hk, uq = b * p.H + h;
    const T* q = (const T*)p.q + b * p.sq.b + h * p.sq.h;
    const T* g = (const T*)p.dout + b * p.sdo.b + h * p.sdo.h;
    const float* fq = p.r > 0 ? p.freqs + b * p.sf.b + h * p.sf.h : nullptr;
    for (int m0 = m_begin; m0 < p.Nq; m0 += AN) {
      __syncthreads();
      stage_row_major<T>(Qs, KD + 1, q, p.sq.n, fq, p.sf.n, nullptr, m0, p.Nq, qoff, p.d, p.r, HDP, RP, tid);
      stage_plain_row_major<T>(Gs, HDP + 1, g, p.sdo.n, m0, p.Nq, p.d, HDP, tid);
      if (tid < 32) {
        const int gi = m0 + tid;
        Ls[tid] = gi < p.Nq ? p.lse_in[(int64_t)uq * p.Nq + gi] : -CUDART_INF_F;
        Ls[32 + tid] = gi < p.Nq ? p.delta[(int64_t)uq * p.Nq + gi] : 0.f;
      }
      __syncthreads();
      float s[4], dp[4];
      dot4(KT, w, Qs + lane * (KD + 1), KD, s);
      dot4(VT, w, Gs + lane * (HDP + 1), HDP, dp);
      const int gi = m0 + lane;
      const float lse = Ls[lane], dl = Ls[32 + lane];
      float pt[4], dst[4];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int j = j0 + w * 4 + kk;
        const bool ok = key_ok[kk] && gi < p.Nq && (!p.causal || j <= gi) && lse != -CUDART_INF_F;
        pt[kk] = ok ? expf(s[kk] * p.scale - lse) : 0.f;
        dst[kk] = pt[kk] * (dp[kk] - dl) * p.scale;
      }
      *reinterpret_cast<float4*>(Ps + (w * 32 + lane) * 4) = make_float4(pt[0], pt[1], pt[2], pt[3]);
      *reinterpret_cast<float4*>(Ds + (w * 32 + lane) * 4) = make_float4(dst[0], dst[1], dst[2], dst[3]);
      __syncwarp();
#pragma unroll 2
      for (int ii = 0; ii < AN; ++ii) {
        const float4 pp = *reinterpret_cast<const float4*>(Ps + (w * 32 + ii) * 4);
        const float4 dd = *reinterpret_cast<const float4*>(Ds + (w * 32 + ii) * 4);
        const float* grow = Gs + ii * (HDP + 1) + lane;
        const float* qrow = Qs + ii * (KD + 1) + lane;
#pragma unroll
        for (int c = 0; c < DCH; ++c) {
          const float gv = grow[32 * c], qc = qrow[32 * c];
          dv[0][c] = fmaf(pp.x, gv, dv[0][c]), dv[1][c] = fmaf(pp.y, gv, dv[1][c]);
          dv[2][c] = fmaf(pp.z, gv, dv[2][c]), dv[3][c] = fmaf(pp.w, gv, dv[3][c]);
          dkc[0][c] = fmaf(dd.x, qc, dkc[0][c]), dkc[1][c] = fmaf(dd.y, qc, dkc[1][c]);
          dkc[2][c] = fmaf(dd.z, qc, dkc[2][c]), dkc[3][c] = fmaf(dd.w, qc, dkc[3][c]);
          if (c < RCH) {
            const float qs = qrow[HDP + 32 * c];
            dks[0][c] = fmaf(dd.x, qs, dks[0][c]), dks[1][c] = fmaf(dd.y, qs, dks[1][c]);
            dks[2][c] = fmaf(dd.z, qs, dks[2][c]), dks[3][c] = fmaf(dd.w, qs, dks[3][c]);
          }
        }
      }
      __syncwarp();
    }
  }

  // epilogue: dv, dk through the transform, phase gradients
  T* dkp = (T*)p.dk + b * p.sdk.b + hk * p.sdk.h;
  T* dvp = (T*)p.dv + b * p.sdv.b + hk * p.sdv.h;
  __syncthreads();
  float* red = Qs;  // [8][RP] per-warp partial sums of the phase gradient
#pragma unroll
  for (int cc = 0; cc < DCH; ++cc) {
    const int c = lane + 32 * cc;
    float dph_sum = 0.f;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const int j = j0 + w * 4 + kk;
      if (j >= p.Nk || c >= p.d) continue;
      dvp[(int64_t)j * p.sdv.n + c] = from_f32<T>(dv[kk][cc]);
      float gk = dkc[kk][cc];
      if (c < p.r) {
        const float x = to_f32(k[(int64_t)j * p.sk.n + c]);
        const float th = fk[(int64_t)j * p.sf.n + c] + bias[c];
        float sn, cs;
        sincosf(th, &sn, &cs);
        gk = (dkc[kk][cc] * cs + dks[kk][cc] * sn) * sigmoid_f(x);
        const float dph = softplus_f(x) * (dks[kk][cc] * cs - dkc[kk][cc] * sn);
        dph_sum += dph;
        if (p.dfreqs) atomicAdd(p.dfreqs + b * p.sdf.b + hk * p.sdf.h + (int64_t)j * p.sdf.n + c, dph);
      }
      dkp[(int64_t)j * p.sdk.n + c] = from_f32<T>(gk);
    }
    if (cc < RCH) red[w * RP + c] = dph_sum;
  }
  if (p.dbias && p.r > 0) {
    __syncthreads();
    for (int c = tid; c < p.r; c += 256) {
      float sacc = 0.f;
#pragma unroll
      for (int ww = 0; ww < 8; ++ww) sacc += red[ww * RP + c];
      atomicAdd(p.dbias + hk * p.dbias_sh + c, sacc);
    }
  }
}

size_t attn_bwd_simt_workspace(const PopeAttnBwdArgs& a) {
  return (size_t)a.shape.B * a.shape.H * a.shape.Nq * sizeof(float);  // delta
}

template <typename T, int DCH>
static cudaError_t launch_attn_bwd(const PopeAttnBwdArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  float* delta = (float*)a.workspace;
  cudaError_t e = attn_bwd_delta(a, delta, st);
  if (e != cudaSuccess) return e;
  AttnP p = {};
  p.B = s.B, p.H = s.H, p.Hk = s.Hk, p.Nq = s.Nq, p.Nk = s.Nk, p.d = s.d, p.r = s.r;
  p.causal = a.causal, p.scale = a.softmax_scale, p.nsplit = 1, p.split_len = s.Nk;
  p.q = a.q, p.k = a.k, p.v = a.v, p.out = a.out, p.dout = a.dout;
  p.sq = a.sq, p.sk = a.sk, p.sv = a.sv, p.so = a.so, p.sdo = a.sdo, p.sf = a.embed.sf;
  p.sdq = a.sdq, p.sdk = a.sdk, p.sdv = a.sdv, p.sdf = a.sdf;
  p.freqs = a.embed.freqs, p.bias = a.embed.bias, p.bias_sh = a.embed.bias_stride_h, p.dbias_sh = a.dbias_stride_h;
  p.lse_in = a.lse, p.delta = delta;
  p.mask = a.mask, p.msb = a.mask_stride_b, p.msn = a.mask_stride_n;
  p.dq = a.dq, p.dk = a.dk, p.dv = a.dv;
  p.dfreqs = s.r > 0 ? a.dfreqs : nullptr, p.dbias = s.r > 0 ? a.dbias : nullptr;
  const int HDP = DCH * 32, RP = round_up(s.r, 32), KD = HDP + RP;
  const size_t smem_q = sizeof(float) * ((size_t)KD * 32 + HDP * 32 + 32 * (KD + 1) + 32 * (HDP + 1) + 8 * 32 * 4);
  const size_t smem_k = smem_q + sizeof(float) * (8 * 32 * 4 + 64);
  e = cudaFuncSetAttribute(attn_bwd_dq_simt_kernel<T, DCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(attn_bwd_dkdv_simt_kernel<T, DCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_k);
  if (e != cudaSuccess) return e;
  attn_bwd_dq_simt_kernel<T, DCH><<<dim3((s.Nq + AM - 1) / AM, s.B * s.H), 256, smem_q, st>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  attn_bwd_dkdv_simt_kernel<T, DCH><<<dim3((s.Nk + AM - 1) / AM, s.B * s.Hk), 256, smem_k, st>>>(p);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t attn_bwd_dch(const PopeAttnBwdArgs& a, cudaStream_t st) {
  if (a.shape.d > 256) return cudaErrorInvalidValue;
  switch (simt_dch(a.shape.d)) {
    case 1: return launch_attn_bwd<T, 1>(a, st);
    case 2: return launch_attn_bwd<T, 2>(a, st);
    case 3: return launch_attn_bwd<T, 3>(a, st);
    case 4: return launch_attn_bwd<T, 4>(a, st);
    default: return launch_attn_bwd<T, 8>(a, st);
  }
}

cudaError_t attn_bwd_simt(const PopeAttnBwdArgs& a, cudaStream_t st) {
  switch (a.shape.dtype) {
    case POPE_F32: return attn_bwd_dch<float>(a, st);
    case POPE_BF16: return attn_bwd_dch<__nv_bfloat16>(a, st);
    default: return attn_bwd_dch<__half>(a, st);
  }
}

}  // namespace pope
