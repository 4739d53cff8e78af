// PoPE flash-attention backward on the Blackwell tensor cores (tcgen05 + TMEM), sm_100a only.
//
// Two kernels, no atomics on dq / dk / dv (deterministic):
//   dq kernel   : a CTA keeps 128 query rows resident (Q' expanded exactly once, dO) and
//                 streams 64-key tiles:   S = Q' K'^T, dP = dO V^T  ->  dS  ->  dQ' += dS K'
//   dkdv kernel : a CTA keeps 128 key rows resident (K' expanded exactly once, V) and streams
//                 64-query tiles: S^T = K' Q'^T, dP^T = V dO^T -> P^T, dS^T ->
//                 dV += P^T dO,  dK' += dS^T Q'
// with P = exp(S*scale - lse), dS = P (dP - delta) scale
// (PoPE_pytorch/triton_pope_flash_attn.py:190-199) and the chain rule through the transform in
// the epilogue (:202-210).  Accumulators live in TMEM (dq: 64+64+32+KD columns; dkdv:
// 64+64+D+KD = 512 columns at d = r = 128); the streamed operand is expanded in registers from
// the raw rows and a (cos, sin) phase table, the per-head phase bias being folded into whichever
// operand is resident.  A streamed tile in shared memory serves two MMAs: as the K-major B
// operand of the score product and, re-described as MN-major, as the B operand of the gradient
// product -- the 8x16-byte core-matrix layout is symmetric under that exchange.
#include <cstdio>

#include "kernels.h"
#include "tc_common.cuh"

namespace pope {

// Optional phase timers of one CTA (compile with -DPOPE_DBG_PHASES): clock64 deltas per phase, printed at the end.
#ifdef POPE_DBG_PHASES
#define PH_DECL long long _t0 = clock64(), _t1; long long _acc[8] = {}
#define PH(i) do { _t1 = clock64(); _acc[i] += _t1 - _t0; _t0 = _t1; } while (0)
#define PH_PRINT(tag, n) do { if (blockIdx.x == 7 && blockIdx.y == 3) printf("%s tiles %d: %lld %lld %lld %lld %lld %lld %lld %lld\n", tag, n, _acc[0] / (n), _acc[1] / (n), _acc[2] / (n), _acc[3] / (n), _acc[4] / (n), _acc[5] / (n), _acc[6] / (n), _acc[7] / (n)); } while (0)
#else
#define PH_DECL
#define PH(i)
#define PH_PRINT(tag, n)
#endif

struct TcBwdP {
  int H, Hk, Nq, Nk, r, causal;
  float scale, scale_log2;
  const void *q, *k, *v, *dout;
  void *dq, *dk, *dv;
  Strides sq, sk, sv, sdo, sdq, sdk, sdv, sdf;
  const float *freqs, *bias, *lse, *delta;
  int64_t sfn, bias_sh, dbias_sh;
  const void* table;   // cos / sin tables in the dtype of q, k, v
  const uint8_t* kimg;   // expanded K' image tiles, (B * Hk) units (no phase bias)
  const uint8_t* qimg;   // expanded Q' image tiles, (B * H) units (no phase bias)
  const uint8_t* vimg;   // V re-laid as image tiles, (B * Hk) units
  const uint8_t* gimg;   // dO re-laid as image tiles, (B * H) units
  const float* rowstat;  // per 64-query tile of every (batch, head): 64 x lse * log2(e) (+inf for empty rows), 64 x delta
  const uint8_t* mask;
  int64_t msb, msn;
  float *dfreqs, *dbias;
  unsigned int* status;
};

constexpr int BQ = 128;  // resident rows per CTA
constexpr int BT = 64;   // streamed rows per step

// ================================================================================================
// dq
// ================================================================================================
// Warp roles of both backward kernels (10 warps, 320 threads)
constexpr int BWD_E_WARPS = 8;     // warps 0-7 : elementwise work (P, dS) and the epilogue; build the resident operands
constexpr int BWD_L_WARP = 8;      // warp 8    : one lane issues the bulk / tensor copies of the streamed tiles
constexpr int BWD_M_WARP = 9;      // warp 9    : one lane issues every MMA; owns the TMEM allocation
constexpr int BWD_THREADS = 32 * (BWD_M_WARP + 1);
constexpr int BCS = BT * 16;       // bytes of one 16-byte chunk column of a streamed tile

// mbarrier slots shared by both backward kernels
enum { BB_FULL = 0,      // [2] streamed tile j has landed in buffer j & 1 (transaction bytes of all its copies)
       BB_SCORES = 2,    // tcgen05.commit: the two score products of the current tile are in TMEM
       BB_ACC = 3,       // [2] tcgen05.commit: the accumulation step of tile j has finished (slot j & 1; a waiter
                         //     may lag two tiles behind, which a single barrier's phase parity cannot express)
       BB_CONSUMED = 5,  // 8 warps: scores copied to registers, the score columns may be overwritten
       BB_GRAD = 6,      // 8 warps: dS (and P) of the current tile are written
       BB_RESIDENT = 7,  // 8 warps: the resident operands are in shared memory
       BB_COUNT = 8 };

__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

template <int D, typename T>
__global__ void __launch_bounds__(BWD_THREADS, 1) attn_bwd_dq_tc_kernel(TcBwdP p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int KD = D + p.r, KSTEPS = KD >> 4;
  uint8_t* Qs = smem;                          // [KD/8][128][16 B]  resident Q'
  uint8_t* Gs = Qs + BQ * KD * 2;              // [D/8][128][16 B]   resident dO
  const int KBUF = (KD / 8) * BCS, VBUF = (D / 8) * BCS;  // one streamed buffer
  uint8_t* Ks = Gs + BQ * D * 2;               // 2 x [KD/8][64][16 B]  (one K' image tile each)
  uint8_t* Vs = Ks + 2 * KBUF;                 // 2 x [D/8][64][16 B]   (one V image tile each)
  uint64_t* bars = reinterpret_cast<uint64_t*>(Vs + 2 * VBUF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BB_COUNT + 1);
  float* bias_cb = reinterpret_cast<float*>(tmem_slot + 4);
  float* bias_sb = bias_cb + 128;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int u = blockIdx.y, b = u / p.H, h = u % p.H, hk = h % p.Hk;
  const int i0 = (gridDim.x - 1 - blockIdx.x) * BQ;
  const int qoff = p.Nk - p.Nq;
  const T* qbase = (const T*)p.q + b * p.sq.b + h * p.sq.h;
  const float* biasr = p.r > 0 ? p.bias + hk * p.bias_sh : nullptr;
  const T* tab = static_cast<const T*>(p.table);

  if (warp == BWD_M_WARP) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&bars[BB_FULL], 1), mbar_init(&bars[BB_FULL + 1], 1);
    mbar_init(&bars[BB_SCORES], 1), mbar_init(&bars[BB_ACC], 1), mbar_init(&bars[BB_ACC + 1], 1);
    mbar_init(&bars[BB_CONSUMED], BWD_E_WARPS), mbar_init(&bars[BB_GRAD], BWD_E_WARPS);
    mbar_init(&bars[BB_RESIDENT], BWD_E_WARPS);
    mbar_init_fence();
  }
  int n_end = p.Nk;
  if (p.causal) n_end = min(n_end, min(i0 + BQ, p.Nq));
  const int T_tiles = (n_end + BT - 1) / BT;
  // Key tiles are visited in an order rotated per unit, which spreads the CTAs resident at one time over
  // different image tiles.
  const int rot = (u * 5 + blockIdx.x * 3) % T_tiles;
  auto tile_start = [&](int j) { int t = j + rot; if (t >= T_tiles) t -= T_tiles; return t * BT; };
  bool failed = false;
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  // TMEM columns: S [0,64), dP [64,128), dS (bf16 pairs) [128,160), dQ' [256, 256+KD)

  if (warp == BWD_L_WARP) {
    // =============================== copies: K' and V image tiles ================================
    if (lane == 0) {
      const uint8_t* kimg = p.kimg + (int64_t)(b * p.Hk + hk) * (int64_t)image_tiles(p.Nk) * KBUF;
      const uint8_t* vimg = p.vimg + (int64_t)(b * p.Hk + hk) * (int64_t)image_tiles(p.Nk) * VBUF;
      for (int j = 0; j < T_tiles; ++j) {
        const int buf = j & 1, n0 = tile_start(j);
        // buffer j & 1 was last read by the accumulation step of tile j-2 (its score products finished earlier)
        if (j >= 2 && !failed) failed = !mbar_wait(&bars[BB_ACC + buf], ((j - 2) >> 1) & 1, WAIT_LIMIT);
        if (failed) break;
        mbar_expect_tx(&bars[BB_FULL + buf], KBUF + VBUF);
        bulk_load(Ks + buf * KBUF, kimg + (int64_t)(n0 / BT) * KBUF, KBUF, &bars[BB_FULL + buf]);
        bulk_load(Vs + buf * VBUF, vimg + (int64_t)(n0 / BT) * VBUF, VBUF, &bars[BB_FULL + buf]);
      }
      if (failed) atomicOr(p.status, 1u);
    }
    __syncwarp();
  } else if (warp == BWD_M_WARP) {
    // =============================== MMA issue ===================================================
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc(TcFmt<T>::fmt, BQ, BT, false, false);
      const uint32_t idesc_q = instr_desc(TcFmt<T>::fmt, BQ, KD, false, true);
      const uint32_t qs_addr = smem_u32(Qs), gs_addr = smem_u32(Gs), ks_addr = smem_u32(Ks), vs_addr = smem_u32(Vs);
      auto issue_scores = [&](int jt) {
        const int buf = jt & 1;
        uint64_t ad = smem_desc(qs_addr, BQ * 16, 128), bd = smem_desc(ks_addr + buf * KBUF, BCS, 128);
#ifndef POPE_DBG_NO_SCORES
        for (int ks = 0; ks < KSTEPS; ++ks) {
          mma_ss(tmem, ad, bd, idesc_s, ks > 0);
          ad += (2 * BQ * 16) >> 4, bd += (2 * BCS) >> 4;
        }
        ad = smem_desc(gs_addr, BQ * 16, 128), bd = smem_desc(vs_addr + buf * VBUF, BCS, 128);
        for (int ks = 0; ks < D / 16; ++ks) {
          mma_ss(tmem + 64, ad, bd, idesc_s, ks > 0);
          ad += (2 * BQ * 16) >> 4, bd += (2 * BCS) >> 4;
        }
#endif
        mma_commit(&bars[BB_SCORES]);
      };
      if (!mbar_wait(&bars[BB_RESIDENT], 0, WAIT_LIMIT)) failed = true;
      if (!mbar_wait(&bars[BB_FULL], 0, WAIT_LIMIT)) failed = true;
      fence_after_sync();
      issue_scores(0);
      PH_DECL;
      for (int j = 0; j < T_tiles; ++j) {
        const int buf = j & 1;
        if (j + 1 < T_tiles) {
          if (!failed) failed = !mbar_wait(&bars[BB_FULL + (1 - buf)], ((j + 1) >> 1) & 1, WAIT_LIMIT);
          PH(0);
          if (!failed) failed = !mbar_wait(&bars[BB_CONSUMED], j & 1, WAIT_LIMIT);
          PH(1);
          fence_after_sync();
          issue_scores(j + 1);
          PH(2);
        }
        if (!failed) failed = !mbar_wait(&bars[BB_GRAD], j & 1, WAIT_LIMIT);
        PH(3);
        fence_after_sync();
        uint64_t bd = smem_desc(ks_addr + buf * KBUF, 128, BCS);
#ifndef POPE_DBG_NO_ACC
#pragma unroll
        for (int ks = 0; ks < BT / 16; ++ks) {
          mma_ts(tmem + 256, tmem + 128 + ks * 8, bd, idesc_q, (j > 0 || ks > 0) ? 1u : 0u);
          bd += (2 * 128) >> 4;
        }
#endif
        mma_commit(&bars[BB_ACC + buf]);
        PH(4);
      }
      PH_PRINT("dq mma [wait full, wait consumed, issue scores, wait grad, issue acc]", T_tiles);
      if (failed) atomicOr(p.status, 1u);
    }
    __syncwarp();
  }
  if (warp >= BWD_E_WARPS) {
    fence_before_sync();
    __syncthreads();
    if (warp == BWD_M_WARP) tmem_dealloc(tmem, 512);
    return;
  }

  // =============================== elementwise warps ================================================
  {
    const T* gbase = (const T*)p.dout + b * p.sdo.b + h * p.sdo.h;
    load_bias_trig(biasr, p.r, -1.f, bias_cb, bias_sb, tid);
    asm volatile("bar.sync 1, 256;" ::: "memory");
    stage_xform<D, BQ, T, true>(qbase, p.sq.n, i0, p.Nq, tab, p.Nk, qoff, p.r, bias_cb, bias_sb, Qs, tid);
    stage_plain<D, BQ, T>(gbase, p.sdo.n, i0, p.Nq, Gs, tid);
    fence_async_smem();
    warp_arrive(&bars[BB_RESIDENT], lane);
  }
  const int row = tid & 127, half = tid >> 7;           // thread = (query row, 32-key half)
  const int gi = i0 + row;
  const uint8_t* maskb = p.mask ? p.mask + b * p.msb : nullptr;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const float lse2 = gi < p.Nq ? p.lse[(int64_t)u * p.Nq + gi] * LOG2E : -CUDART_INF_F;
  const float lse_use = lse2 == -CUDART_INF_F ? 0.f : lse2;
  const float dlt = gi < p.Nq ? p.delta[(int64_t)u * p.Nq + gi] : 0.f;

  PH_DECL;
  for (int j = 0; j < T_tiles; ++j) {
    const int buf = j & 1, n0 = tile_start(j);
    // key visibility of this thread's 32-key half (key-padding mask, ragged end): the same for every row
    uint32_t vis = 0xffffffffu;
    if (maskb || n0 + BT > p.Nk) {
      const int jk = n0 + half * 32 + lane;
      vis = __ballot_sync(0xffffffffu, jk < p.Nk && (!maskb || maskb[(int64_t)jk * p.msn] != 0));
    }
    if (!failed) failed = !mbar_wait(&bars[BB_SCORES], j & 1, WAIT_LIMIT);
    fence_after_sync();
    PH(0);
#ifdef POPE_DBG_NO_ELEM
    if (p.Nq > 0) {
      fence_before_sync();
      warp_arrive(&bars[BB_CONSUMED], lane);
      if (j >= 1 && !failed) failed = !mbar_wait(&bars[BB_ACC + (1 - buf)], ((j - 1) >> 1) & 1, WAIT_LIMIT);
      warp_arrive(&bars[BB_GRAD], lane);
      continue;
    }
#endif
    if (p.causal) {
      const int lim = gi - (n0 + half * 32);  // columns <= lim visible
      vis &= lim >= 31 ? 0xffffffffu : (lim < 0 ? 0u : ((2u << lim) - 1u));
    }
    if (lse2 == -CUDART_INF_F) vis = 0u;
    const bool all_vis = __all_sync(0xffffffffu, vis == 0xffffffffu);   // interior tile: no masking work
    uint32_t pk[16];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {   // 16 key columns at a time keeps the register footprint small
      uint32_t sv[16], dv[16];
      tmem_ld16(tmem + lane_base + half * 32 + hh * 16, sv);
      tmem_ld16(tmem + lane_base + 64 + half * 32 + hh * 16, dv);
      tmem_ld_wait();
      if (hh == 1) {   // every score of this tile is in registers: the next score products may overwrite them
        fence_before_sync();
        warp_arrive(&bars[BB_CONSUMED], lane);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float p0 = ex2_approx(fmaf(__uint_as_float(sv[2 * e]), p.scale_log2, -lse_use));
        float p1 = ex2_approx(fmaf(__uint_as_float(sv[2 * e + 1]), p.scale_log2, -lse_use));
        if (!all_vis) {
          p0 = ((vis >> (hh * 16 + 2 * e)) & 1u) ? p0 : 0.f;
          p1 = ((vis >> (hh * 16 + 2 * e + 1)) & 1u) ? p1 : 0.f;
        }
        const float d0 = p0 * (__uint_as_float(dv[2 * e]) - dlt) * p.scale;
        const float d1 = p1 * (__uint_as_float(dv[2 * e + 1]) - dlt) * p.scale;
        pk[hh * 8 + e] = pack2<T>(d0, d1);
      }
    }
    PH(1);
    // the dS columns were read by the accumulation step of tile j-1
    if (j >= 1 && !failed) failed = !mbar_wait(&bars[BB_ACC + (1 - buf)], ((j - 1) >> 1) & 1, WAIT_LIMIT);
    PH(2);
    tmem_st16(tmem + lane_base + 128 + half * 16, pk);
    tmem_st_wait();
    fence_before_sync();
    warp_arrive(&bars[BB_GRAD], lane);
    PH(3);
  }
  if (tid == 0) PH_PRINT("dq elem [wait scores, ld+math, wait acc, st+arrive]", T_tiles);

  // ---- epilogue: dq = (dQc cos + dQs sin) sigmoid(q), dphase = a (dQs cos - dQc sin) ---------------
  if (!failed) failed = !mbar_wait(&bars[BB_ACC + ((T_tiles - 1) & 1)], ((T_tiles - 1) >> 1) & 1, WAIT_LIMIT);
  fence_after_sync();
  {
    constexpr int HW = D / 2;  // features handled by this thread: [half*HW, half*HW + HW)
    const uint32_t acc = tmem + lane_base + 256;
    const T* qrow = qbase + (int64_t)gi * p.sq.n;
    T* dqrow = (T*)p.dq + b * p.sdq.b + h * p.sdq.h + (int64_t)gi * p.sdq.n;
    const float* frow = p.r > 0 ? p.freqs + (int64_t)(qoff + gi) * p.sfn : nullptr;
    float* dfrow = p.dfreqs ? p.dfreqs + b * p.sdf.b + h * p.sdf.h + (int64_t)(qoff + gi) * p.sdf.n : nullptr;
#pragma unroll
    for (int c0 = 0; c0 < HW; c0 += 16) {
      const int cbase = half * HW + c0;
      uint32_t gc[16], gs[16];
      tmem_ld16(acc + cbase, gc);
      const bool rot = cbase < p.r;  // r is a multiple of 16: the 16-wide group is rotated as a whole
      if (rot) tmem_ld16(acc + D + cbase, gs);
      tmem_ld_wait();
      if (gi < p.Nq) {
        uint32_t outw[8];
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          float g0 = __uint_as_float(gc[e]), g1 = __uint_as_float(gc[e + 1]);
          if (rot) {
            const uint32_t qw = *reinterpret_cast<const uint32_t*>(qrow + cbase + e);
            const float2 x = unpack2<T>(qw);
            float s0, c0f, s1, c1f;
            sincosf(frow[cbase + e] - biasr[cbase + e], &s0, &c0f);
            sincosf(frow[cbase + e + 1] - biasr[cbase + e + 1], &s1, &c1f);
            const float h0 = __uint_as_float(gs[e]), h1 = __uint_as_float(gs[e + 1]);
            if (dfrow) {
              atomicAdd(dfrow + cbase + e, softplus_f(x.x) * (h0 * c0f - g0 * s0));
              atomicAdd(dfrow + cbase + e + 1, softplus_f(x.y) * (h1 * c1f - g1 * s1));
            }
            g0 = (g0 * c0f + h0 * s0) * sigmoid_f(x.x);
            g1 = (g1 * c1f + h1 * s1) * sigmoid_f(x.y);
          }
          outw[e >> 1] = pack2<T>(g0, g1);
        }
        *reinterpret_cast<uint4*>(dqrow + cbase) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
        *reinterpret_cast<uint4*>(dqrow + cbase + 8) = make_uint4(outw[4], outw[5], outw[6], outw[7]);
      }
    }
  }
  if (failed) atomicOr(p.status, 1u);
  fence_before_sync();
  __syncthreads();   // the issuing warp frees the tensor memory after this barrier
}

}  // namespace pope

#include "tc_attn_bwd_dkdv.inl"
