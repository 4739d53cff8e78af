// PoPE flash-attention backward on the Blackwell tensor cores (tcgen05 + TMEM), sm_100a only.
//
// Two kernels, no atomics on dq / dk / dv (deterministic):
//   dq kernel   : a CTA keeps 128 query rows resident (Q' in shared memory, dO in TMEM) and streams 64-key
//                 tiles through three stages:   S = Q' K'^T, dP = dO V^T  ->  dS  ->  dQ' += dS K'
//   dkdv kernel : a CTA keeps 128 key rows resident (K', V) and streams 64-query tiles:
//                 S^T = K' Q'^T -> P^T, then dP^T = V dO^T (same TMEM columns) -> dS^T;
//                 dV += P^T dO,  dK' += dS^T Q'  with P^T / dS^T read from TMEM
// with P = exp(S*scale - lse), dS = P (dP - delta) scale
// (PoPE_pytorch/triton_pope_flash_attn.py:190-199) and the chain rule through the transform in
// the epilogue (:202-210).  Every operand tile -- expanded Q' and K', re-laid V and dO -- comes from the images
// that a pre-pass builds once per call (tc_expand.cu) and reaches shared memory by cp.async.bulk; the per-head
// phase bias of the keys is part of the K' images.  A streamed tile in shared memory serves two MMAs: as the
// K-major B operand of the score product and, re-described as MN-major, as the B operand of the gradient
// product -- the 8x16-byte core-matrix layout is symmetric under that exchange.
#include <cstring>
#include <mutex>
#include <type_traits>

#include "kernels.h"
#include "tc_common.cuh"

namespace pope {

struct TcBwdP {
  int H, Hk, Nq, Nk, r, causal;
  float scale, scale_log2;
  const void *q, *k, *v, *dout;
  void *dq, *dk, *dv;
  Strides sq, sk, sv, sdo, sdq, sdk, sdv, sdf;
  const float *freqs, *bias, *lse, *delta;
  int64_t sfn, bias_sh, dbias_sh;
  const uint8_t* kimg;   // expanded K' image tiles, (B * Hk) units (no phase bias)
  const uint8_t* qimg;   // expanded Q' image tiles, (B * H) units (no phase bias)
  const uint8_t* vimg;   // V re-laid as image tiles, (B * Hk) units
  const uint8_t* gimg;   // dO re-laid as image tiles, (B * H) units
  const float* rowstat;  // per 64-query tile of every (batch, head): 64 x lse * log2(e) (+inf for empty rows), 64 x delta
  const uint8_t* mask;
  int64_t msb, msn;
  float *dfreqs, *dbias;
  unsigned int* status;
  int img_maps;          // 1: the resident 128-row operand arrives by one tensor-map copy of its image
};

constexpr int BQ = 128;  // resident rows per CTA
constexpr int BT = 64;   // streamed rows per step (= IMAGE_ROWS)
static_assert(BT == IMAGE_ROWS, "a streamed tile is one image tile");

// Warp roles of both backward kernels (11 warps, 352 threads).  Two issuing warps: a single thread spends ~55
// clocks per MMA instruction, so the accumulation MMAs of tile j are issued by a second thread while the first
// is still issuing the score products of tile j+1 (the tensor pipe is idle about half of that time).
constexpr int BWD_E_WARPS = 8;     // warps 0-7 : elementwise work (P, dS) and the epilogue
constexpr int BWD_L_WARP = 8;      // warp 8    : issues the bulk copies of the resident and the streamed tiles
constexpr int BWD_M_WARP = 9;      // warp 9    : one lane issues the score products; owns the TMEM allocation
constexpr int BWD_A_WARP = 10;     // warp 10   : one lane issues the accumulation products
constexpr int BWD_THREADS = 32 * (BWD_A_WARP + 1);
constexpr int BCS = BT * 16;       // bytes of one 16-byte chunk column of a streamed tile

// mbarrier slots shared by both backward kernels; a streamed tile j lives in stage j % NST
enum { BB_FULL = 0,      // [3] streamed tile j has landed in its stage (transaction bytes of all its copies)
       BB_ACC = 3,       // [3] tcgen05.commit: the accumulation step of tile j has finished; its stage is free
       BB_SCORES = 6,    // tcgen05.commit: the two score products of the current tile are in TMEM
       BB_CONSUMED = 7,  // 8 warps: scores copied to registers, the score columns may be overwritten
       BB_GRAD = 8,      // 8 warps: dS (and P) of the current tile are written
       BB_RESIDENT = 9,  // the resident operands are in place (copies' transaction bytes, plus the warps that wrote TMEM)
       BB_ISSUED = 10,   // [2] the score products of tile j have been ISSUED (slot j & 1): what is issued after this
                         //     executes behind them in the tensor pipe
       BB_DPDONE = 12,   // tcgen05.commit: dP of the current tile is in TMEM (dq kernel: issued by the second warp)
       BB_CONS_DP = 13,  // 8 warps: dP copied to registers (dq kernel: BB_CONSUMED then covers S alone)
       BB_COUNT = 14 };

__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

// ================================================================================================
// dq: three stages of (K' tile, V tile); Q' resident in shared memory, dO resident in TMEM
// ================================================================================================
constexpr int DQ_NST = 3;

// VW: V tiles come straight from the caller's V as tensor-map boxes of 64 features (128-byte rows, 128-byte swizzled,
// read through swizzled K-major descriptors) and dO rows straight from the caller's dO; otherwise both come from the
// re-laid image tiles of the pre-pass (head widths that are no multiple of 64, strides a tensor map cannot describe).
template <int D, typename T, bool VW>
__global__ void __launch_bounds__(BWD_THREADS, 1) attn_bwd_dq_tc_kernel(TcBwdP p, const __grid_constant__ CUtensorMap tmap_v,
                                                                        const __grid_constant__ CUtensorMap tmap_qimg) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzled tiles sit on 1 KB boundaries
  const int KD = D + p.r, KSTEPS = KD >> 4;
  const int KBUF = (KD / 8) * BCS;             // one K' image tile
  constexpr int VBUF = (D / 8) * BCS;          // one V image tile
  uint8_t* Qs = smem;                          // [KD/8][128][16 B]  resident Q'
  uint8_t* Ks = Qs + BQ * KD * 2;              // DQ_NST x [KD/8][64][16 B]
  uint8_t* Vs = Ks + DQ_NST * KBUF;            // DQ_NST x [D/8][64][16 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(Vs + DQ_NST * VBUF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BB_COUNT + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int u = blockIdx.y, b = u / p.H, h = u % p.H, hk = h % p.Hk;
  const int i0 = (gridDim.x - 1 - blockIdx.x) * BQ;
  const int qoff = p.Nk - p.Nq;

  if (warp == BWD_M_WARP) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    for (int i = 0; i < DQ_NST; ++i) mbar_init(&bars[BB_FULL + i], 1), mbar_init(&bars[BB_ACC + i], 1);
    mbar_init(&bars[BB_SCORES], 1);
    mbar_init(&bars[BB_CONSUMED], BWD_E_WARPS), mbar_init(&bars[BB_GRAD], BWD_E_WARPS);
    mbar_init(&bars[BB_CONS_DP], BWD_E_WARPS);
    mbar_init(&bars[BB_RESIDENT], 1 + BWD_E_WARPS);
    mbar_init(&bars[BB_ISSUED], 1), mbar_init(&bars[BB_ISSUED + 1], 1);
    mbar_init(&bars[BB_DPDONE], 1);
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
  // TMEM columns: S [0,64), dP [64,128), dS (16-bit pairs) [128,160), dO (16-bit pairs) [160,160+D/2), dQ' [256,256+KD)
  constexpr uint32_t TC_S = 0, TC_DP = 64, TC_DS = 128, TC_DO = 160, TC_DQ = 256;

  if (warp == BWD_L_WARP) {
    // =============================== copies: resident Q', then K' and V image tiles ===============
    {
      const uint8_t* qimg = p.qimg + ((int64_t)u * (int64_t)image_tiles(p.Nq) + i0 / BT) * KBUF;
      if (lane == 0) mbar_expect_tx(&bars[BB_RESIDENT], BQ * KD * 2);
      __syncwarp();
      // one tensor-map copy of (1 KB, 2 image tiles, all chunks) when the image has a map, else 2 x KD / 8 copies of 1 KB
      if (p.img_maps) {
        if (lane == 0) tma_load_4d(Qs, &tmap_qimg, &bars[BB_RESIDENT], 0, (int)((int64_t)u * (int64_t)image_tiles(p.Nq) + i0 / BT), 0, 0);
      } else {
        copy_resident_tiles(Qs, qimg, KD / 8, &bars[BB_RESIDENT], lane);
      }
    }
    if (lane == 0) {
      const int64_t ktiles = (int64_t)image_tiles(p.Nk);
      const uint8_t* kimg = p.kimg + (int64_t)(b * p.Hk + hk) * ktiles * KBUF;
      const uint8_t* vimg = p.vimg + (int64_t)(b * p.Hk + hk) * ktiles * VBUF;
      for (int j = 0; j < T_tiles; ++j) {
        const int st = j % DQ_NST, n0 = tile_start(j);
        // the stage was last read by the accumulation step of tile j - NST
        if (j >= DQ_NST && !failed) failed = !mbar_wait(&bars[BB_ACC + st], ((j - DQ_NST) / DQ_NST) & 1, WAIT_LIMIT);
        if (failed) { drain_copies(&bars[BB_FULL], DQ_NST, j - DQ_NST, j); break; }
        mbar_expect_tx(&bars[BB_FULL + st], KBUF + VBUF);
        bulk_load(Ks + st * KBUF, kimg + (int64_t)(n0 / BT) * KBUF, KBUF, &bars[BB_FULL + st]);
        if (VW) {
#pragma unroll
          for (int c = 0; c < D / 64; ++c) tma_load_4d(Vs + st * VBUF + c * (BT * 128), &tmap_v, &bars[BB_FULL + st], c * 64, n0, hk, b);
        } else {
          bulk_load(Vs + st * VBUF, vimg + (int64_t)(n0 / BT) * VBUF, VBUF, &bars[BB_FULL + st]);
        }
      }
      if (failed) atomicOr(p.status, 1u);
    }
    __syncwarp();
  } else if (warp == BWD_M_WARP) {
    // =============================== MMA issue: S = Q' K'^T ======================================
    // The two score products of a tile are issued by the two issuing warps at the same time (16 + 8 instructions at
    // ~55 clk each from one thread were the longest link of the score -> elementwise -> score chain).
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc(TcFmt<T>::fmt, BQ, BT, false, false);
      const uint32_t qs_addr = smem_u32(Qs), ks_addr = smem_u32(Ks);
      const uint64_t qd = smem_desc(qs_addr, BQ * 16, 128);
      if (!mbar_wait(&bars[BB_RESIDENT], 0, WAIT_LIMIT)) failed = true;
      for (int j = 0; j < T_tiles && !failed; ++j) {
        const int st = j % DQ_NST;
        failed = !mbar_wait(&bars[BB_FULL + st], (j / DQ_NST) & 1, WAIT_LIMIT);
        // the elementwise warps have copied the previous tile's scores out of TMEM
        if (j >= 1 && !failed) failed = !mbar_wait(&bars[BB_CONSUMED], (j - 1) & 1, WAIT_LIMIT);
        fence_after_sync();
        const uint64_t kd = smem_desc(ks_addr + st * KBUF, BCS, 128);
        uint32_t alo = desc_lo(qd), blo = desc_lo(kd);
        mma_ss_lh(tmem + TC_S, alo, desc_hi(qd), blo, desc_hi(kd), idesc_s, 0u);
#pragma unroll 4
        for (int ks = 1; ks < KSTEPS; ++ks) {
          alo += (2 * BQ * 16) >> 4, blo += (2 * BCS) >> 4;
          mma_ss_lh(tmem + TC_S, alo, desc_hi(qd), blo, desc_hi(kd), idesc_s, 1u);
        }
        mma_commit(&bars[BB_SCORES]);
        mbar_arrive(&bars[BB_ISSUED + (j & 1)]);
      }
      if (failed) atomicOr(p.status, 1u);
    }
    __syncwarp();
  } else if (warp == BWD_A_WARP) {
    // =============================== MMA issue: dP = dO V^T, dQ' += dS K' ========================
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc(TcFmt<T>::fmt, BQ, BT, false, false);
      const uint32_t idesc_q = instr_desc(TcFmt<T>::fmt, BQ, KD, false, true);
      const uint32_t ks_addr = smem_u32(Ks), vs_addr = smem_u32(Vs);
      if (!mbar_wait(&bars[BB_RESIDENT], 0, WAIT_LIMIT)) failed = true;   // dO is in TMEM
      for (int j = 0; j <= T_tiles && !failed; ++j) {
        if (j < T_tiles) {   // dP(j): dO from TMEM, the V tile from shared memory
          const int st = j % DQ_NST;
          failed = !mbar_wait(&bars[BB_FULL + st], (j / DQ_NST) & 1, WAIT_LIMIT);
          if (j >= 1 && !failed) failed = !mbar_wait(&bars[BB_CONS_DP], (j - 1) & 1, WAIT_LIMIT);
          fence_after_sync();
          // B = V tile, K-major: image: chunk columns BCS apart; boxes: 64-feature blocks of 64 x 128 bytes, 32 bytes per step
          const uint64_t vd = VW ? smem_desc_sw128(vs_addr + st * VBUF, 16, 1024) : smem_desc(vs_addr + st * VBUF, BCS, 128);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t koff = VW ? (uint32_t)(((ks >> 2) * (BT * 128) + (ks & 3) * 32) >> 4) : (uint32_t)(ks * ((2 * BCS) >> 4));
            mma_ts_lh(tmem + TC_DP, tmem + TC_DO + ks * 8, desc_lo(vd) + koff, desc_hi(vd), idesc_s, ks > 0);
          }
          mma_commit(&bars[BB_DPDONE]);
        }
        if (j >= 1) {   // dQ' += dS K'(j-1): dS from TMEM; the K' tile re-described as an MN-major B operand
          const int jp = j - 1, st = jp % DQ_NST;
          if (!failed) failed = !mbar_wait(&bars[BB_GRAD], jp & 1, WAIT_LIMIT);
          // Let the score product of tile j enter the pipe first: it heads the critical score -> elementwise -> score
          // chain, and this accumulation then runs in the gap while its results are copied out of TMEM.
          if (j < T_tiles && !failed) failed = !mbar_wait(&bars[BB_ISSUED + (j & 1)], (j >> 1) & 1, WAIT_LIMIT);
          fence_after_sync();
          const uint64_t bd = smem_desc(ks_addr + st * KBUF, 128, BCS);
#pragma unroll
          for (int ks = 0; ks < BT / 16; ++ks)
            mma_ts_lh(tmem + TC_DQ, tmem + TC_DS + ks * 8, desc_lo(bd) + ks * ((2 * 128) >> 4), desc_hi(bd), idesc_q,
                      (jp > 0 || ks > 0) ? 1u : 0u);
          mma_commit(&bars[BB_ACC + st]);   // every score product of this tile finished before its dS existed
        }
      }
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
  const int row = tid & 127, half = tid >> 7;           // thread = (query row, 32-key half)
  const int gi = i0 + row;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const uint8_t* maskb = p.mask ? p.mask + b * p.msb : nullptr;
  {
    // dO rows into TMEM, the A operand of dP = dO V^T: 16 columns (32 features) per step, the two threads
    // of a row take alternate steps.  Read from the dO IMAGE ([chunk][row][16 B] per 64-row tile; rows past Nq are
    // zero there): for a fixed chunk the 32 lanes of a warp (32 consecutive rows) read 512 contiguous bytes, where
    // the row-major dO itself would be touched in 32 different lines per load.
    const uint8_t* gtile = p.gimg + ((int64_t)u * (int64_t)image_tiles(p.Nq) + i0 / BT + (row >> 6)) * VBUF + (row & 63) * 16;
    // (VW: the row itself; a warp-wide 16-byte load then touches 32 rows, which costs this one-time 32 KB read little)
    const T* grow_ = static_cast<const T*>(p.dout) + b * p.sdo.b + h * p.sdo.h + (int64_t)gi * p.sdo.n;
#pragma unroll
    for (int g = 0; g < D / 32; ++g) {
      if ((g & 1) != half) continue;
      uint32_t w[16];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        uint4 v4 = make_uint4(0, 0, 0, 0);
        if (!VW) v4 = __ldg(reinterpret_cast<const uint4*>(gtile + (g * 4 + q4) * BCS));
        else if (gi < p.Nq) v4 = __ldg(reinterpret_cast<const uint4*>(grow_ + (g * 4 + q4) * 8));
        w[q4 * 4] = v4.x, w[q4 * 4 + 1] = v4.y, w[q4 * 4 + 2] = v4.z, w[q4 * 4 + 3] = v4.w;
      }
      tmem_st16(tmem + lane_base + TC_DO + g * 16, w);
    }
    tmem_st_wait();
    fence_before_sync();
    warp_arrive(&bars[BB_RESIDENT], lane);
  }
  const float lse2 = gi < p.Nq ? p.lse[(int64_t)u * p.Nq + gi] * LOG2E : -CUDART_INF_F;
  const float lse_use = lse2 == -CUDART_INF_F ? 0.f : lse2;
  const float dlt = gi < p.Nq ? p.delta[(int64_t)u * p.Nq + gi] : 0.f;
  for (int j = 0; j < T_tiles; ++j) {
    const int n0 = tile_start(j);
    // key visibility of this thread's 32-key half (key-padding mask, ragged end): the same for every row
    uint32_t vis = 0xffffffffu;
    if (maskb || n0 + BT > p.Nk) {
      const int jk = n0 + half * 32 + lane;
      vis = __ballot_sync(0xffffffffu, jk < p.Nk && (!maskb || maskb[(int64_t)jk * p.msn] != 0));
    }
    if (p.causal) {
      const int lim = gi - (n0 + half * 32);  // columns <= lim visible
      vis &= lim >= 31 ? 0xffffffffu : (lim < 0 ? 0u : ((2u << lim) - 1u));
    }
    if (lse2 == -CUDART_INF_F) vis = 0u;
    const bool all_vis = __all_sync(0xffffffffu, vis == 0xffffffffu);   // interior tile: no masking work
    // S first: the next S = Q' K'^T (16 instructions, the long product) starts as soon as these columns are free; dP
    // (its own columns, its own barrier) follows
    if (!failed) failed = !mbar_wait(&bars[BB_SCORES], j & 1, WAIT_LIMIT);
    fence_after_sync();
    uint32_t sv[32], dv[32];
    tmem_ld32(tmem + lane_base + TC_S + half * 32, sv);
    tmem_ld_wait();
    fence_before_sync();
    warp_arrive(&bars[BB_CONSUMED], lane);
    if (!failed) failed = !mbar_wait(&bars[BB_DPDONE], j & 1, WAIT_LIMIT);
    fence_after_sync();
    tmem_ld32(tmem + lane_base + TC_DP + half * 32, dv);
    tmem_ld_wait();
    fence_before_sync();
    warp_arrive(&bars[BB_CONS_DP], lane);
    uint32_t pk[16];
    // two copies of the loop: interior tiles (the common case) carry no masking arithmetic at all
    auto elementwise = [&](auto masked) {
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        float p0 = ex2_approx(fmaf(__uint_as_float(sv[2 * e]), p.scale_log2, -lse_use));
        float p1 = ex2_approx(fmaf(__uint_as_float(sv[2 * e + 1]), p.scale_log2, -lse_use));
        if (decltype(masked)::value) {
          p0 = ((vis >> (2 * e)) & 1u) ? p0 : 0.f;
          p1 = ((vis >> (2 * e + 1)) & 1u) ? p1 : 0.f;
        }
        const float d0 = p0 * (__uint_as_float(dv[2 * e]) - dlt) * p.scale;
        const float d1 = p1 * (__uint_as_float(dv[2 * e + 1]) - dlt) * p.scale;
        pk[e] = pack2<T>(d0, d1);
      }
    };
    if (all_vis) elementwise(std::false_type());
    else elementwise(std::true_type());
    // the dS columns were read by the accumulation step of tile j-1
    if (j >= 1 && !failed) failed = !mbar_wait(&bars[BB_ACC + (j - 1) % DQ_NST], ((j - 1) / DQ_NST) & 1, WAIT_LIMIT);
    tmem_st16(tmem + lane_base + TC_DS + half * 16, pk);
    tmem_st_wait();
    fence_before_sync();
    warp_arrive(&bars[BB_GRAD], lane);
  }
  // ---- epilogue: dq = (dQc cos + dQs sin) sigmoid(q), dphase = a (dQs cos - dQc sin) ---------------
  // Everything the chain rule needs is in the resident Q' tile: with qc = a cos f, qs = a sin f (a = softplus(q)),
  //   a = sqrt(qc^2 + qs^2),  sigmoid(q) = 1 - exp(-a),  dq = (dQc qc + dQs qs) / a * sigmoid(q),
  //   dphase = a (dQs cos f - dQc sin f) = dQs qc - dQc qs,
  // so the epilogue reads neither q nor the phase tables from global memory.  The 16-bit rounding of Q' costs cos f a
  // relative 2^-8 sin^2 f at most.  A thread works on its own row (TMEM hands it that row, and the Q' tile is read
  // conflict-free by rows); the dq rows then go through a row-major staging tile behind Q' (the dead stages) so that
  // they leave in fully coalesced 16-byte pieces.  (Transposing the fp32 accumulator through shared memory first and
  // running the chain rule on row-major groups took 8600 clocks of an 11 000-clock epilogue.)
  if (!failed) failed = !mbar_wait(&bars[BB_ACC + (T_tiles - 1) % DQ_NST], ((T_tiles - 1) / DQ_NST) & 1, WAIT_LIMIT);
  fence_after_sync();
  asm volatile("bar.sync 1, 256;" ::: "memory");   // every MMA is done: the stages are dead
  constexpr int OSTR = D * 2 + 16;                 // bytes of a staged output row (16 bytes of padding: conflict-free)
  uint8_t* dq_stage = Ks;
  {
    constexpr int HW = D / 2;
    const uint32_t acc = tmem + lane_base + TC_DQ;
    float* dfrow = p.dfreqs ? p.dfreqs + b * p.sdf.b + h * p.sdf.h + (int64_t)(qoff + gi) * p.sdf.n : nullptr;
    const bool live = gi < p.Nq;
#pragma unroll
    for (int c0 = 0; c0 < HW; c0 += 16) {
      const int cbase = half * HW + c0;
      uint32_t gc[16], gs[16];
      const bool rotd = cbase < p.r;   // r is a multiple of 16: the 16-wide group is rotated as a whole
      tmem_ld16(acc + cbase, gc);
      if (rotd) tmem_ld16(acc + D + cbase, gs);
      tmem_ld_wait();
      uint32_t wq[8];
      if (rotd) {
        uint32_t cw[8], sw[8];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint4 qcw = *reinterpret_cast<const uint4*>(Qs + (cbase / 8 + i) * (BQ * 16) + row * 16);
          const uint4 qsw = *reinterpret_cast<const uint4*>(Qs + (D / 8 + cbase / 8 + i) * (BQ * 16) + row * 16);
          cw[4 * i] = qcw.x, cw[4 * i + 1] = qcw.y, cw[4 * i + 2] = qcw.z, cw[4 * i + 3] = qcw.w;
          sw[4 * i] = qsw.x, sw[4 * i + 1] = qsw.y, sw[4 * i + 2] = qsw.z, sw[4 * i + 3] = qsw.w;
        }
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const float2 qc = unpack2<T>(cw[e >> 1]), qs = unpack2<T>(sw[e >> 1]);
          const float g0 = __uint_as_float(gc[e]), g1 = __uint_as_float(gc[e + 1]);
          const float h0 = __uint_as_float(gs[e]), h1 = __uint_as_float(gs[e + 1]);
          const float m0 = qc.x * qc.x + qs.x * qs.x, m1 = qc.y * qc.y + qs.y * qs.y;   // a^2
          const float r0 = m0 > 0.f ? rsqrtf(m0) : 0.f, r1 = m1 > 0.f ? rsqrtf(m1) : 0.f;
          const float sg0 = 1.f - ex2_approx(-m0 * r0 * LOG2E), sg1 = 1.f - ex2_approx(-m1 * r1 * LOG2E);
          if (dfrow && live) {
            atomicAdd(dfrow + cbase + e, h0 * qc.x - g0 * qs.x);
            atomicAdd(dfrow + cbase + e + 1, h1 * qc.y - g1 * qs.y);
          }
          wq[e >> 1] = pack2<T>((g0 * qc.x + h0 * qs.x) * r0 * sg0, (g1 * qc.y + h1 * qs.y) * r1 * sg1);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 16; e += 2) wq[e >> 1] = pack2<T>(__uint_as_float(gc[e]), __uint_as_float(gc[e + 1]));
      }
      *reinterpret_cast<uint4*>(dq_stage + row * OSTR + cbase * 2) = make_uint4(wq[0], wq[1], wq[2], wq[3]);
      *reinterpret_cast<uint4*>(dq_stage + row * OSTR + cbase * 2 + 16) = make_uint4(wq[4], wq[5], wq[6], wq[7]);
    }
  }
  asm volatile("bar.sync 1, 256;" ::: "memory");
  {
    constexpr int GPR = D / 8;   // 16-byte groups per row
    T* dqbase = (T*)p.dq + b * p.sdq.b + h * p.sdq.h;
    for (int idx = tid; idx < BQ * GPR; idx += 256) {
      const int rr = idx / GPR, g = idx - rr * GPR;
      if (i0 + rr < p.Nq)
        *reinterpret_cast<uint4*>(dqbase + (int64_t)(i0 + rr) * p.sdq.n + g * 8) = *reinterpret_cast<const uint4*>(dq_stage + rr * OSTR + g * 16);
    }
  }
  if (failed) atomicOr(p.status, 1u);
  fence_before_sync();
  __syncthreads();   // the issuing warp frees the tensor memory after this barrier
}

}  // namespace pope

#include "tc_attn_bwd_dkdv.inl"
