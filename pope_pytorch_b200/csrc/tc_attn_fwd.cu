// PoPE flash-attention forward on the Blackwell tensor cores (tcgen05 + TMEM), sm_100a only.
//
// One CTA owns 256 query rows (two 128-row MMA tiles) of one (batch, head) unit and sweeps
// the keys 64 at a time.  Per key tile:
//   1. all 256 threads turn the raw K rows into the expanded operand K' = [a cos | pass | a sin]
//      in registers and write it to shared memory in the tensor core's K-major layout
//      (double buffered); V is staged MN-major; nothing expanded ever goes to global memory
//   2. one thread issues tcgen05.mma  S_t = Q'_t K'^T  into TMEM (t = 0,1)
//   3. every thread owns one query row: it pulls its 64 scores out of TMEM, applies the
//      causal / key-padding masks, keeps the running max and sum, and writes P (bf16) back
//      into TMEM over the scores
//   4. one thread issues  O_t += P_t V  with P read straight from TMEM
// The MMAs of step 2 run while the threads do step 3 of the previous tile, those of step 4
// while they do step 1 of the next.
//
// The per-head phase bias is folded into the QUERY phase (cos(fq - fk - b) is symmetric in
// where b is applied), so the key-side transform needs only a per-position table of
// (cos f, sin f) that a small pre-pass builds once per call in the caller's workspace.
//
// Semantics follow PoPE_pytorch/triton_pope_flash_attn.py:23-117 (top-left causal mask,
// bottom-right positions, mask True = keep, zero output and -inf LSE for empty rows).
#include <mutex>

#include "kernels.h"
#include "tc_common.cuh"

namespace pope {

__device__ unsigned int g_tc_status = 0;  // sticky: bit 0 = a bounded wait gave up

unsigned int* tc_status_ptr() {
  void* p = nullptr;
  return cudaGetSymbolAddress(&p, g_tc_status) == cudaSuccess ? static_cast<unsigned int*>(p) : nullptr;
}

unsigned int tc_read_status() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v));
  return v;
}

// ---- pre-pass: table[pos][c] = (cos, sin) of freqs[pos][c] as half2 ---------------------------
__global__ void pope_trig_table_kernel(const float* freqs, int64_t sfn, int n, int r, __half2* table) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)n * r) return;
  const int pos = idx / r, c = idx % r;
  float sn, cs;
  sincosf(freqs[pos * sfn + c], &sn, &cs);
  table[idx] = __floats2half2_rn(cs, sn);
}

cudaError_t launch_trig_table(const float* freqs, int64_t sfn, int n, int r, __half2* table, cudaStream_t st) {
  const int64_t total = (int64_t)n * r;
  pope_trig_table_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(freqs, sfn, n, r, table);
  return cudaGetLastError();
}

struct TcFwdP {
  int H, Hk, Nq, Nk, r, causal;
  float scale_log2;  // softmax_scale * log2(e)
  const void *q, *k, *v;
  void* o;
  float* lse;
  Strides sq, sk, sv, so;
  const float* freqs;
  int64_t sfn;
  const float* bias;
  int64_t bias_sh;
  const __half2* table;
  const uint8_t* mask;
  int64_t msb, msn;
};

constexpr int TQ = 128;   // rows per MMA tile
constexpr int TK = 64;    // keys per step

// Expand 64 key rows starting at n0 into Kbuf (K-major, chunk-major storage: chunk*1024 + row*16),
// stage the matching V rows MN-major (chunk*1024 + key*16) and publish the key-validity bits.
template <int D, typename T>
__device__ __forceinline__ void stage_keys(const TcFwdP& p, const T* kbase, const T* vbase, const uint8_t* maskb, int n0,
                                           uint8_t* Kbuf, uint8_t* Vbuf, uint32_t* kbits, int tid) {
  constexpr int DC = D / 8;
  const int RC = p.r >> 3;
#pragma unroll
  for (int it = 0; it < (TK * DC) / 256; ++it) {
    const int task = tid + it * 256;
    const int row = task & (TK - 1), c = task >> 6;
    const int j = n0 + row;
    const bool ok = j < p.Nk;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (ok) raw = *reinterpret_cast<const uint4*>(kbase + (int64_t)j * p.sk.n + c * 8);
    if (c < RC) {
      uint4 t0 = make_uint4(0, 0, 0, 0), t1 = t0;
      if (ok) {
        const uint4* tp = reinterpret_cast<const uint4*>(p.table + (int64_t)j * p.r + c * 8);
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
      *reinterpret_cast<uint4*>(Kbuf + c * (TK * 16) + row * 16) = make_uint4(oc[0], oc[1], oc[2], oc[3]);
      *reinterpret_cast<uint4*>(Kbuf + (DC + c) * (TK * 16) + row * 16) = make_uint4(os[0], os[1], os[2], os[3]);
    } else {
      *reinterpret_cast<uint4*>(Kbuf + c * (TK * 16) + row * 16) = raw;
    }
  }
  // the sin block of K' only spans chunks [DC, DC + RC); nothing to clear beyond it
#pragma unroll
  for (int it = 0; it < (TK * DC) / 256; ++it) {
    const int task = tid + it * 256;
    const int row = task & (TK - 1), c = task >> 6;
    const int j = n0 + row;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (j < p.Nk) raw = *reinterpret_cast<const uint4*>(vbase + (int64_t)j * p.sv.n + c * 8);
    *reinterpret_cast<uint4*>(Vbuf + c * (TK * 16) + row * 16) = raw;
  }
  if (tid < TK) {
    const int j = n0 + tid;
    const bool ok = j < p.Nk && (!maskb || maskb[(int64_t)j * p.msn] != 0);
    const uint32_t bits = __ballot_sync(0xffffffffu, ok);
    if ((tid & 31) == 0) kbits[tid >> 5] = bits;
  }
}

template <int D, typename T>
__global__ void __launch_bounds__(256, 1) attn_fwd_tc_kernel(TcFwdP p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int DC = D / 8;
  const int RC = p.r >> 3, KD = D + p.r, KSTEPS = KD >> 4;
  uint8_t* Qs = smem;                              // 2 tiles x [KD/8 chunks][128 rows][16 B]
  uint8_t* Ks = Qs + 2 * TQ * KD * 2;              // 2 bufs  x [KD/8 chunks][64 rows][16 B]
  uint8_t* Vs = Ks + 2 * TK * KD * 2;              // 2 bufs  x [D/8 chunks][64 keys][16 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(Vs + 2 * TK * D * 2);  // s[0], s[1], pv[0], pv[1]
  uint32_t* kbits = reinterpret_cast<uint32_t*>(bars + 4);           // [2 bufs][2 words]
  uint32_t* tmem_slot = kbits + 4;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int u = blockIdx.y, b = u / p.H, h = u % p.H, hk = h % p.Hk;
  const int i0 = (gridDim.x - 1 - blockIdx.x) * (2 * TQ);  // heavy (late) row blocks first
  const int qoff = p.Nk - p.Nq;
  const T* qbase = (const T*)p.q + b * p.sq.b + h * p.sq.h;
  const T* kbase = (const T*)p.k + b * p.sk.b + hk * p.sk.h;
  const T* vbase = (const T*)p.v + b * p.sv.b + hk * p.sv.h;
  const uint8_t* maskb = p.mask ? p.mask + b * p.msb : nullptr;
  const float* biasr = p.r > 0 ? p.bias + hk * p.bias_sh : nullptr;

  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    for (int i = 0; i < 4; ++i) mbar_init(&bars[i], 1);
    mbar_init_fence();
  }

  // ---- Q' for both tiles: thread = row -------------------------------------------------------
  {
    const int gi = i0 + tid;
    const bool ok = gi < p.Nq;
    const T* qrow = qbase + (int64_t)gi * p.sq.n;
    const float* frow = p.r > 0 ? p.freqs + (int64_t)(qoff + gi) * p.sfn : nullptr;
    uint8_t* Qt = Qs + (tid >> 7) * (TQ * KD * 2) + (tid & 127) * 16;
#pragma unroll 2
    for (int c = 0; c < DC; ++c) {
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (ok) raw = *reinterpret_cast<const uint4*>(qrow + c * 8);
      if (c < RC) {
        const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t oc[4] = {0, 0, 0, 0}, os[4] = {0, 0, 0, 0};
        if (ok) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 x = unpack2<T>(rw[e]);
            float s0, c0, s1, c1;
            sincosf(frow[c * 8 + 2 * e] - biasr[c * 8 + 2 * e], &s0, &c0);
            sincosf(frow[c * 8 + 2 * e + 1] - biasr[c * 8 + 2 * e + 1], &s1, &c1);
            const float a0 = softplus_f(x.x), a1 = softplus_f(x.y);
            oc[e] = pack2<T>(a0 * c0, a1 * c1);
            os[e] = pack2<T>(a0 * s0, a1 * s1);
          }
        }
        *reinterpret_cast<uint4*>(Qt + c * (TQ * 16)) = make_uint4(oc[0], oc[1], oc[2], oc[3]);
        *reinterpret_cast<uint4*>(Qt + (DC + c) * (TQ * 16)) = make_uint4(os[0], os[1], os[2], os[3]);
      } else {
        *reinterpret_cast<uint4*>(Qt + c * (TQ * 16)) = raw;
      }
    }
  }

  // key range and tile activity
  int n_end = p.Nk;
  if (p.causal) n_end = min(n_end, min(i0 + 2 * TQ, p.Nq));
  const int T_tiles = (n_end + TK - 1) / TK;
  const bool has_rows1 = i0 + TQ < p.Nq;
  const int tile = warp >> 2;                     // which 128-row tile this thread's row is in
  const int row = i0 + tid;                       // global query row of this thread
  const bool tile_has_rows = tile == 0 || has_rows1;

  stage_keys<D, T>(p, kbase, vbase, maskb, 0, Ks, Vs, kbits, tid);
  fence_async_smem();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  // TMEM columns: scores S[buf][tile] at (buf*2 + tile)*64 (P aliases the first 32), outputs at 256 + tile*128
  const uint32_t idesc_s = instr_desc(TcFmt<T>::fmt, TQ, TK, false, false);
  const uint32_t idesc_o = instr_desc(TcFmt<T>::fmt, TQ, D, false, true);
  const uint32_t qs_addr = smem_u32(Qs), ks_addr = smem_u32(Ks), vs_addr = smem_u32(Vs);

  auto issue_s = [&](int jt) {  // S(jt) for both tiles into score buffer jt & 1
    const int buf = jt & 1, n0 = jt * TK;
    for (int t = 0; t < 2; ++t) {
      if (t == 1 && !has_rows1) continue;
      if (p.causal && n0 > i0 + t * TQ + TQ - 1) continue;
      const uint32_t d = tmem + (buf * 2 + t) * 64;
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const uint64_t ad = smem_desc(qs_addr + t * (TQ * KD * 2) + ks * 2 * (TQ * 16), TQ * 16, 128);
        const uint64_t bd = smem_desc(ks_addr + buf * (TK * KD * 2) + ks * 2 * (TK * 16), TK * 16, 128);
        mma_ss(d, ad, bd, idesc_s, ks > 0);
      }
    }
    mma_commit(&bars[buf]);
  };
  if (tid == 0) issue_s(0);

  bool failed = false;
  float m_run = -CUDART_INF_F, l_run = 0.f;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;

  for (int j = 0; j < T_tiles; ++j) {
    const int buf = j & 1, n0 = j * TK;
    if (j + 1 < T_tiles) {
      // V buffer 1-buf was read by PV(j-1); K' buffer 1-buf by S(j-1), which softmax(j-1) waited for
      if (j >= 1 && !failed) failed = !mbar_wait(&bars[2 + ((j - 1) & 1)], ((j - 1) >> 1) & 1, WAIT_LIMIT);
      stage_keys<D, T>(p, kbase, vbase, maskb, n0 + TK, Ks + (1 - buf) * (TK * KD * 2), Vs + (1 - buf) * (TK * D * 2),
                       kbits + (1 - buf) * 2, tid);
      fence_async_smem();
      fence_before_sync();
      __syncthreads();
      if (tid == 0) {
        fence_after_sync();
        issue_s(j + 1);
      }
    }
    const bool active = tile_has_rows && (!p.causal || n0 <= i0 + tile * TQ + TQ - 1);
    if (active) {
      if (!failed) failed = !mbar_wait(&bars[buf], (j >> 1) & 1, WAIT_LIMIT);
      fence_after_sync();
      const uint32_t s_addr = tmem + lane_base + (buf * 2 + tile) * 64;
      uint32_t sv[64];
      {
        uint32_t a[32], c[32];
        tmem_ld32(s_addr, a);
        tmem_ld32(s_addr + 32, c);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) sv[i] = a[i], sv[32 + i] = c[i];
      }
      // visibility of the 64 keys of this tile for this row
      uint64_t vis = ((uint64_t)kbits[buf * 2 + 1] << 32) | kbits[buf * 2];
      if (p.causal) {
        const int lim = row - n0;  // columns <= lim are visible
        vis &= lim >= 63 ? ~0ull : (lim < 0 ? 0ull : ((2ull << lim) - 1ull));
      }
      const bool all_vis = __all_sync(0xffffffffu, vis == ~0ull);
      float mx = -CUDART_INF_F;
      if (all_vis) {
#pragma unroll
        for (int i = 0; i < 64; ++i) mx = fmaxf(mx, __uint_as_float(sv[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if ((vis >> i) & 1ull) mx = fmaxf(mx, __uint_as_float(sv[i]));
      }
      const float m_new = fmaxf(m_run, mx * p.scale_log2);
      // keep a stale maximum while it is within 2^8 of the true one: P stays below 256 and the
      // output accumulator needs no rescale on most steps
      const bool need = m_new > m_run + 8.f;  // true on the first finite maximum (m_run = -inf)
      float alpha = 1.f;
      if (need) {
        alpha = ex2_approx(m_run - m_new);  // exp2(-inf) = 0
        l_run *= alpha;
        m_run = m_new;
      }
      if (j > 0 && __any_sync(0xffffffffu, need)) {
        // O was last written by PV(j-1): complete, since its barrier was waited for above or here
        if (!failed) failed = !mbar_wait(&bars[2 + ((j - 1) & 1)], ((j - 1) >> 1) & 1, WAIT_LIMIT);
        fence_after_sync();
        const uint32_t o_addr = tmem + lane_base + 256 + tile * 128;
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t ov[32];
          tmem_ld32(o_addr + c0, ov);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tmem_st32(o_addr + c0, ov);
        }
        tmem_st_wait();
      }
      const float m_use = m_run == -CUDART_INF_F ? 0.f : m_run;
      uint32_t pk[32];
      float lsum = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float p0 = ex2_approx(__uint_as_float(sv[2 * i]) * p.scale_log2 - m_use);
        float p1 = ex2_approx(__uint_as_float(sv[2 * i + 1]) * p.scale_log2 - m_use);
        if (!all_vis) {
          p0 = ((vis >> (2 * i)) & 1ull) ? p0 : 0.f;
          p1 = ((vis >> (2 * i + 1)) & 1ull) ? p1 : 0.f;
        }
        lsum += p0 + p1;
        pk[i] = pack2<T>(p0, p1);
      }
      l_run += lsum;
      tmem_st32(s_addr, pk);
      tmem_st_wait();
    }
    fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      fence_after_sync();
      for (int t = 0; t < 2; ++t) {
        if (t == 1 && !has_rows1) continue;
        if (p.causal && n0 > i0 + t * TQ + TQ - 1) continue;
        const uint32_t d = tmem + 256 + t * 128;
        const uint32_t a = tmem + (buf * 2 + t) * 64;
        for (int ks = 0; ks < TK / 16; ++ks) {
          const uint64_t bd = smem_desc(vs_addr + buf * (TK * D * 2) + ks * 2 * 128, 128, TK * 16);
          mma_ts(d, a + ks * 8, bd, idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
        }
      }
      mma_commit(&bars[2 + buf]);
    }
  }

  // ---- epilogue: O / l, LSE -----------------------------------------------------------------------
  {
    const int jl = T_tiles - 1;
    if (!failed) failed = !mbar_wait(&bars[2 + (jl & 1)], (jl >> 1) & 1, WAIT_LIMIT);
    fence_after_sync();
    if (tile_has_rows) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const uint32_t o_addr = tmem + lane_base + 256 + tile * 128;
      T* orow = (T*)p.o + b * p.so.b + h * p.so.h + (int64_t)row * p.so.n;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t ov[32];
        tmem_ld32(o_addr + c0, ov);
        tmem_ld_wait();
        if (row < p.Nq) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack2<T>(__uint_as_float(ov[i]) * inv, __uint_as_float(ov[i + 1]) * inv);
            w.y = pack2<T>(__uint_as_float(ov[i + 2]) * inv, __uint_as_float(ov[i + 3]) * inv);
            w.z = pack2<T>(__uint_as_float(ov[i + 4]) * inv, __uint_as_float(ov[i + 5]) * inv);
            w.w = pack2<T>(__uint_as_float(ov[i + 6]) * inv, __uint_as_float(ov[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c0 + i) = w;
          }
        }
      }
      if (row < p.Nq)
        p.lse[(int64_t)u * p.Nq + row] = l_run > 0.f ? m_run * 0.6931471805599453f + logf(l_run) : -CUDART_INF_F;
    }
  }
  if (failed) atomicOr(&g_tc_status, 1u);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  (void)lane;
}

// ---- host side ---------------------------------------------------------------------------------
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static bool stride_ok(const PopeStride3& s) { return s.b % 8 == 0 && s.h % 8 == 0 && s.n % 8 == 0; }

bool attn_fwd_tc_supported(const PopeAttnArgs& a) {
  const PopeShape& s = a.shape;
  if (s.dtype != POPE_BF16 && s.dtype != POPE_F16) return false;
  if (s.d != 64 && s.d != 96 && s.d != 128) return false;
  if (s.r % 16 != 0) return false;
  if (s.Nq < 64) return false;  // short query blocks take the key-split path
  if (s.r > 0 && (a.embed.sf.b != 0 || a.embed.sf.h != 0)) return false;  // one phase table for all units
  if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || !aligned16(a.out)) return false;
  if (!stride_ok(a.sq) || !stride_ok(a.sk) || !stride_ok(a.sv) || !stride_ok(a.so)) return false;
  return true;
}

size_t attn_fwd_tc_workspace(const PopeAttnArgs& a) {
  return (size_t)a.shape.Nk * a.shape.r * sizeof(__half2) + 16;
}

template <int D, typename T>
static cudaError_t launch_fwd_tc(const PopeAttnArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  TcFwdP p = {};
  p.H = s.H, p.Hk = s.Hk, p.Nq = s.Nq, p.Nk = s.Nk, p.r = s.r, p.causal = a.causal;
  p.scale_log2 = a.softmax_scale * 1.4426950408889634f;
  p.q = a.q, p.k = a.k, p.v = a.v, p.o = a.out, p.lse = a.lse;
  p.sq = a.sq, p.sk = a.sk, p.sv = a.sv, p.so = a.so;
  p.freqs = a.embed.freqs, p.sfn = a.embed.sf.n, p.bias = a.embed.bias, p.bias_sh = a.embed.bias_stride_h;
  p.table = reinterpret_cast<const __half2*>(a.workspace);
  p.mask = a.mask, p.msb = a.mask_stride_b, p.msn = a.mask_stride_n;
  if (s.r > 0) {
    const int64_t n = (int64_t)s.Nk * s.r;
    (void)n;
    cudaError_t e = launch_trig_table(a.embed.freqs, a.embed.sf.n, s.Nk, s.r, reinterpret_cast<__half2*>(a.workspace), st);
    if (e != cudaSuccess) return e;
  }
  const int KD = s.d + s.r;
  size_t smem = (size_t)2 * TQ * KD * 2 + 2 * TK * KD * 2 + 2 * TK * D * 2 + 4 * 8 + 4 * 4 + 16;
  // every CTA allocates all 512 TMEM columns: ask for more than half of the SM's shared memory so
  // that two CTAs are never co-resident
  if (smem < 120 * 1024) smem = 120 * 1024;
  cudaError_t e = cudaFuncSetAttribute(attn_fwd_tc_kernel<D, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid((s.Nq + 2 * TQ - 1) / (2 * TQ), s.B * s.H);
  attn_fwd_tc_kernel<D, T><<<grid, 256, smem, st>>>(p);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t fwd_tc_d(const PopeAttnArgs& a, cudaStream_t st) {
  switch (a.shape.d) {
    case 64: return launch_fwd_tc<64, T>(a, st);
    case 96: return launch_fwd_tc<96, T>(a, st);
    default: return launch_fwd_tc<128, T>(a, st);
  }
}

cudaError_t attn_fwd_tc(const PopeAttnArgs& a, cudaStream_t st) {
  return a.shape.dtype == POPE_BF16 ? fwd_tc_d<__nv_bfloat16>(a, st) : fwd_tc_d<__half>(a, st);
}

// ---- forward with library-owned scratch ------------------------------------------------------------
// The phase table of the forward kernel normally sits in a workspace the caller allocates.  Some
// callers cannot allocate device memory at the point where they need attention: code running
// under a framework that forbids allocator calls inside a region (a serving loop with a frozen
// memory plan, a real-time thread, a plugin whose host hands it fixed input/output buffers
// only).  For them the table lives in this fixed array, which every GPU that loads the library
// carries until the process exits.
constexpr size_t kStaticScratchBytes = POPE_B200_NOALLOC_MAX_SCRATCH;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Host code cannot use g_static_scratch as a pointer: the name is only a handle for the runtime.
// The device address is looked up once per device, with that device current.
static cudaError_t static_scratch_address(void** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static void* addr[kMaxDevices] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return e;
    addr[dev] = ptr;
  }
  *out = addr[dev];
  return cudaSuccess;
}

}  // namespace pope

extern "C" int pope_b200_attn_fwd_noalloc(const PopeAttnArgs* args, void* stream) {
  using namespace pope;
  if (!args || args->struct_bytes != sizeof(PopeAttnArgs)) return POPE_ERR_BAD_ARG;
  const PopeShape& s = args->shape;
  if (s.B <= 0 || s.H <= 0 || s.Hk <= 0 || s.Nq <= 0 || s.Nk <= 0 || s.d <= 0 || s.r < 0) return POPE_ERR_BAD_ARG;
  if (s.H % s.Hk != 0 || s.Nq > s.Nk || s.r > s.d || (int64_t)s.B * s.H > 65535) return POPE_ERR_BAD_ARG;
  if (!args->q || !args->k || !args->v || !args->out || !args->lse) return POPE_ERR_BAD_ARG;
  if (s.r > 0 && (!args->embed.freqs || !args->embed.bias)) return POPE_ERR_BAD_ARG;
  if (!attn_fwd_tc_supported(*args)) return POPE_ERR_UNSUPPORTED;
  if (attn_fwd_tc_workspace(*args) > kStaticScratchBytes) return POPE_ERR_TOO_LARGE;
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
    return POPE_ERR_CUDA;
  if (major != 10) return POPE_ERR_ARCH;
  void* scratch = nullptr;
  if (static_scratch_address(&scratch) != cudaSuccess) return POPE_ERR_CUDA;
  PopeAttnArgs local = *args;
  local.workspace = scratch;              // the kernel must get the looked-up address, never the symbol
  local.workspace_bytes = kStaticScratchBytes;
  return attn_fwd_tc(local, static_cast<cudaStream_t>(stream)) == cudaSuccess ? POPE_OK : POPE_ERR_CUDA;
}
