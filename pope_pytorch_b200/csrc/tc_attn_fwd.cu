// PoPE flash-attention forward on the Blackwell tensor cores (tcgen05 + TMEM), sm_100a only.
//
// One CTA owns 256 query rows (two 128-row MMA tiles) of one (batch, head) unit and sweeps the keys 64 at a
// time.  The expanded operands Q' and K' = [a cos | pass | a sin] come from the operand images that a pre-pass
// builds once per call (tc_expand.cu), so the main loop contains no transform work:
//   loader warp   : Q' (resident, 2 x 2 image tiles) and one K' image tile per step by cp.async.bulk; the V tile
//                   of the step by cp.async.bulk.tensor boxes straight from the caller's strided V
//   score warp    : one lane issues tcgen05.mma  S_t = Q'_t K'^T  into TMEM (t = 0, 1)
//   softmax warps : every thread owns one query row: it pulls its 64 scores out of TMEM, applies the causal /
//                   key-padding masks, keeps the running max and sum, and writes P (16-bit) back into TMEM over
//                   the scores
//   PV warp       : one lane issues  O_t += P_t V  with P read straight from TMEM
// All hand-offs are mbarriers (copy completion by transaction bytes, MMA completion by tcgen05.commit).
//
// The per-head phase bias of the keys is part of the K' images.
//
// Semantics follow PoPE_pytorch/triton_pope_flash_attn.py:23-117 (top-left causal mask,
// bottom-right positions, mask True = keep, zero output and -inf LSE for empty rows).
#include <cstring>
#include <mutex>
#include <type_traits>

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

cudaError_t tc_clear_status() {
  const unsigned int zero = 0;
  return cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(zero));
}

// cuTensorMapEncodeTiled, fetched once through the runtime's driver entry point (the library links no libcuda)
typedef CUresult (*TmapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TmapEncodeFn tmap_encoder() {
  static TmapEncodeFn encode = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      encode = reinterpret_cast<TmapEncodeFn>(fn);
  });
  return encode;
}

// (feature, row, head, batch) view of a strided tensor.  A size-1 axis may come with any stride: it gets a valid
// dummy (multiple of 16 bytes, increasing); an axis with more entries must come with a usable stride.
static bool tmap_4d(CUtensorMap* out, CUtensorMapDataType dt, int esz, const void* base, int cols, int rows, int heads,
                    int batch, int64_t sn, int64_t sh, int64_t sb, int box_cols, int box_rows, CUtensorMapSwizzle swz) {
  TmapEncodeFn encode = tmap_encoder();
  if (!encode) return false;
  cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)heads, (cuuint64_t)batch};
  int64_t st[3] = {sn, sh, sb};
  if ((rows > 1 && st[0] < cols) || (heads > 1 && st[1] <= 0) || (batch > 1 && st[2] <= 0)) return false;
  if (rows == 1) st[0] = (cols + 15) / 16 * 16;
  if (heads == 1) st[1] = st[0] * rows;
  if (batch == 1) st[2] = st[1] * heads;
  cuuint64_t strides[3] = {(cuuint64_t)st[0] * esz, (cuuint64_t)st[1] * esz, (cuuint64_t)st[2] * esz};
  for (int i = 0; i < 3; ++i)
    if (strides[i] % 16 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return false;
  cuuint32_t box[4] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1, 1}, estr[4] = {1, 1, 1, 1};
  return encode(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_chunk_tmap(CUtensorMap* out, const void* base, bool is_bf16, int d, int rows, int heads, int batch, int64_t sn,
                     int64_t sh, int64_t sb, int box_rows) {
  return tmap_4d(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, d, rows, heads,
                 batch, sn, sh, sb, 8, box_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
}

// 16-bit rows cut into boxes of 64 features (128 bytes) x box_rows rows, 128-byte swizzled
static bool make_wide_tmap(CUtensorMap* out, const void* base, bool is_bf16, int d, int rows, int heads, int batch, int64_t sn,
                           int64_t sh, int64_t sb, int box_rows) {
  return tmap_4d(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, d, rows, heads,
                 batch, sn, sh, sb, 64, box_rows, CU_TENSOR_MAP_SWIZZLE_128B);
}

bool make_load_tmap_f32(CUtensorMap* out, const void* base, int cols, int rows, int heads, int batch, int64_t sn, int64_t sh,
                        int64_t sb, int box_rows) {
  return tmap_4d(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, cols, rows, heads, batch, sn, sh, sb, 32, box_rows,
                 CU_TENSOR_MAP_SWIZZLE_128B);
}

bool make_store_tmap(CUtensorMap* out, const void* base, int dtype, int cols, int rows, int heads, int batch, int64_t sn,
                     int64_t sh, int64_t sb, int box_rows) {
  const int esz = dtype == POPE_F32 ? 4 : 2;
  const CUtensorMapDataType dt = dtype == POPE_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == POPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return tmap_4d(out, dt, esz, base, cols, rows, heads, batch, sn, sh, sb, 128 / esz, box_rows, CU_TENSOR_MAP_SWIZZLE_128B);
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
  const uint8_t* qimg; // expanded Q' image tiles, (B * H) units
  const uint8_t* kimg; // expanded K' image tiles (phase bias folded in), (B * Hk) units
  const uint8_t* mask;
  int64_t msb, msn;
};

constexpr int TQ = 128;   // rows per MMA tile
constexpr int TK = 64;    // keys per step (= IMAGE_ROWS)
static_assert(TK == IMAGE_ROWS, "a streamed K' tile is one image tile");

// Warp roles of the forward kernel (12 warps, 384 threads).  Three issuing warps: a single thread spends ~55 clocks
// per 128x64x16 MMA instruction against 32 clocks of tensor time, so the score products of the two row tiles are
// issued by two threads in parallel (16 instructions each per key tile) and O += P V of tile j by a third.
constexpr int FWD_SOFTMAX_WARPS = 8;               // warps 0-7 : one query row per thread (two 128-row tiles)
constexpr int FWD_LOAD_WARP = FWD_SOFTMAX_WARPS;   // warp 8    : one lane issues every bulk / tensor copy
constexpr int FWD_MMA_WARP = FWD_LOAD_WARP + 1;    // warp 9    : one lane issues S_0 = Q'_0 K'^T; owns the TMEM allocation
constexpr int FWD_PV_WARP = FWD_MMA_WARP + 1;      // warp 10   : one lane issues O += P V
constexpr int FWD_MMA1_WARP = FWD_PV_WARP + 1;     // warp 11   : one lane issues S_1 = Q'_1 K'^T
constexpr int FWD_THREADS = 32 * (FWD_MMA1_WARP + 1);

// mbarrier slots
enum {
  B_KFULL = 0,   // [2] K' image tile landed (transaction bytes)
  B_VFULL = 2,   // [2] V tile landed (transaction bytes)
  B_KFREE = 4,   // [2] both score products of a key tile have completed (one commit per issuing thread): its K' buffer
                 //     may be refilled
  B_PVDONE = 6,  // [2] O += P V of both row tiles done (tcgen05.commit)
  B_PFULL = 8,   // [buf][row tile] probabilities written to TMEM (4 softmax warps)
  B_QFULL = 12,  // the resident Q' tiles are in shared memory
  B_SFULL = 13,  // [buf][row tile] scores of one row tile written to TMEM (tcgen05.commit)
  B_ODONE = 17,  // [row tile] the last O += P V of that row tile has completed: one phase per barrier, so the epilogue's
                 //     wait cannot alias with a later completion (B_PVDONE of a buffer completes again two steps later
                 //     for the other row tile when the causal mask ends tile 0 early)
  B_COUNT = 19
};

template <int D, typename T>
__global__ void __launch_bounds__(FWD_THREADS, 1) attn_fwd_tc_kernel(TcFwdP p, const __grid_constant__ CUtensorMap tmap_v) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int KD = D + p.r, KSTEPS = KD >> 4;
  constexpr int CS = TK * 16;                       // bytes of one 16-byte chunk column of a streamed tile
  const int KBUF = (KD / 8) * CS;                   // one K' tile = one image tile
  constexpr int VBUF = (D / 8) * CS;
  uint8_t* Qs = smem;                               // 2 tiles x [KD/8 chunks][128 rows][16 B]
  uint8_t* Ks = Qs + 2 * TQ * KD * 2;               // 2 bufs  x [KD/8 chunks][64 keys][16 B]
  uint8_t* Vs = Ks + 2 * KBUF;                      // 2 bufs  x [D/8 chunks][64 keys][16 B]; 128-byte aligned (KD % 16 == 0)
  uint64_t* bars = reinterpret_cast<uint64_t*>(Vs + 2 * VBUF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int u = blockIdx.y, b = u / p.H, h = u % p.H, hk = h % p.Hk;
  const int i0 = (gridDim.x - 1 - blockIdx.x) * (2 * TQ);  // heavy (late) row blocks first

  int n_end = p.Nk;
  if (p.causal) n_end = min(n_end, min(i0 + 2 * TQ, p.Nq));
  const int T_tiles = (n_end + TK - 1) / TK;
  const bool has_rows1 = i0 + TQ < p.Nq;
  // number of key tiles tile t takes part in (under the causal mask tile 0 stops 128 keys earlier)
  const int T0 = p.causal ? min(T_tiles, (min(n_end, i0 + TQ) + TK - 1) / TK) : T_tiles;
  const int T1 = has_rows1 ? T_tiles : 0;

  if (warp == FWD_MMA_WARP) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[B_KFULL + i], 1), mbar_init(&bars[B_VFULL + i], 1);
      mbar_init(&bars[B_KFREE + i], 2), mbar_init(&bars[B_PVDONE + i], 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&bars[B_PFULL + i], 4), mbar_init(&bars[B_SFULL + i], 1);
    mbar_init(&bars[B_QFULL], 1);
    mbar_init(&bars[B_ODONE], 1), mbar_init(&bars[B_ODONE + 1], 1);
    mbar_init_fence();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  bool failed = false;

  if (warp == FWD_LOAD_WARP) {
    // =============================== copies ==================================================
    // K'(j) is one contiguous image tile; V(j) arrives as D/8 boxes of 64 keys x 16 bytes, each landing on its
    // chunk column.  A buffer is refilled as soon as the MMA that read it has completed.
    // the two resident Q' tiles: four image tiles, one 1 KB copy per chunk column and 64 rows
    {
      const uint8_t* qimg = p.qimg + ((int64_t)u * (int64_t)image_tiles(p.Nq) + i0 / IMAGE_ROWS) * KBUF;
      if (lane == 0) mbar_expect_tx(&bars[B_QFULL], 2 * TQ * KD * 2);
      __syncwarp();
      copy_resident_tiles(Qs, qimg, KD / 8, &bars[B_QFULL], lane);
      copy_resident_tiles(Qs + TQ * KD * 2, qimg + 2 * KBUF, KD / 8, &bars[B_QFULL], lane);
    }
    // K' tiles and V tiles are streamed by two lanes on their own: a K' buffer is free as soon as the score products
    // that read it have completed, a V buffer only after O += P V two steps later, and one lane waiting for the latter
    // would hold back the K' copy that the next score product is waiting for.
    if (lane == 0) {
      const uint8_t* kimg = p.kimg + (int64_t)(b * p.Hk + hk) * (int64_t)image_tiles(p.Nk) * KBUF;
      int j = 0;
      for (; j < T_tiles; ++j) {
        const int buf = j & 1;
        if (j >= 2 && !failed) failed = !mbar_wait(&bars[B_KFREE + buf], ((j - 2) >> 1) & 1, WAIT_LIMIT);
        if (failed) break;
        mbar_expect_tx(&bars[B_KFULL + buf], KBUF);
        bulk_load(Ks + buf * KBUF, kimg + (int64_t)j * KBUF, KBUF, &bars[B_KFULL + buf]);
      }
      if (failed) drain_copies(&bars[B_KFULL], 2, j - 2, j), drain_copies(&bars[B_QFULL], 1, 0, 1);
    } else if (lane == 1) {
      int j = 0;
      for (; j < T_tiles; ++j) {
        const int buf = j & 1, n0 = j * TK;
        if (j >= 2 && !failed) failed = !mbar_wait(&bars[B_PVDONE + buf], ((j - 2) >> 1) & 1, WAIT_LIMIT);
        if (failed) { drain_copies(&bars[B_VFULL], 2, j - 2, j); break; }
        mbar_expect_tx(&bars[B_VFULL + buf], VBUF);
#pragma unroll
        for (int c = 0; c < D / 8; ++c) tma_load_4d(Vs + buf * VBUF + c * CS, &tmap_v, &bars[B_VFULL + buf], c * 8, n0, hk, b);
      }
    }
    __syncwarp();
  } else if (warp == FWD_MMA_WARP || warp == FWD_MMA1_WARP) {
    // =============================== MMA issue: S_t = Q'_t K'^T, one thread per row tile ==========
    if (lane == 0) {
      const int t = warp == FWD_MMA_WARP ? 0 : 1;
      const int T_t = t == 0 ? T0 : T1;
      const uint32_t idesc_s = instr_desc(TcFmt<T>::fmt, TQ, TK, false, false);
      const uint32_t qs_addr = smem_u32(Qs), ks_addr = smem_u32(Ks);
      const uint64_t ad = smem_desc(qs_addr + t * (TQ * KD * 2), TQ * 16, 128);
      if (!mbar_wait(&bars[B_QFULL], 0, WAIT_LIMIT)) failed = true;
      for (int j = 0; j < T_tiles && !failed; ++j) {
        const int buf = j & 1;
        // (also paces a thread whose row tile is finished: it arrives on KFREE of tile j only after the tile has landed,
        // i.e. after the phase of tile j - 2 has completed)
        failed = !mbar_wait(&bars[B_KFULL + buf], (j >> 1) & 1, WAIT_LIMIT);
        if (j < T_t) {
          // score buffer j & 1 still holds P(j-2) until PV(j-2) has read it
          if (j >= 2 && !failed) failed = !mbar_wait(&bars[B_PVDONE + buf], ((j - 2) >> 1) & 1, WAIT_LIMIT);
          fence_after_sync();
          const uint32_t d = tmem + (buf * 2 + t) * 64;
          const uint64_t bd = smem_desc(ks_addr + buf * KBUF, CS, 128);
          uint32_t alo = desc_lo(ad), blo = desc_lo(bd);
          mma_ss_lh(d, alo, desc_hi(ad), blo, desc_hi(bd), idesc_s, 0u);
#pragma unroll 4
          for (int ks = 1; ks < KSTEPS; ++ks) {
            alo += (2 * TQ * 16) >> 4, blo += (2 * CS) >> 4;
            mma_ss_lh(d, alo, desc_hi(ad), blo, desc_hi(bd), idesc_s, 1u);
          }
          mma_commit(&bars[B_SFULL + buf * 2 + t]);   // this row tile's softmax may start
        }
        // one arrival per issuing thread and key tile, also for tiles this row tile does not take part in (the commit
        // then completes at once): the K' buffer is free when both have arrived
        mma_commit(&bars[B_KFREE + buf]);
      }
    }
    __syncwarp();
  } else if (warp == FWD_PV_WARP) {
    // =============================== MMA issue: O += P V =======================================
    if (lane == 0) {
      const uint32_t idesc_o = instr_desc(TcFmt<T>::fmt, TQ, D, false, true);
      const uint32_t vs_addr = smem_u32(Vs);
      for (int j = 0; j < T_tiles && !failed; ++j) {
        const int buf = j & 1;
        failed = !mbar_wait(&bars[B_VFULL + buf], (j >> 1) & 1, WAIT_LIMIT);
        for (int t = 0; t < 2; ++t) {
          if (j >= (t == 0 ? T0 : T1)) continue;
          if (!failed) failed = !mbar_wait(&bars[B_PFULL + buf * 2 + t], (j >> 1) & 1, WAIT_LIMIT);
          fence_after_sync();
          const uint32_t d = tmem + 256 + t * 128;
          const uint32_t a = tmem + (buf * 2 + t) * 64;
          const uint64_t bd = smem_desc(vs_addr + buf * VBUF, 128, CS);
#pragma unroll
          for (int ks = 0; ks < TK / 16; ++ks)
            mma_ts_lh(d, a + ks * 8, desc_lo(bd) + ks * ((2 * 128) >> 4), desc_hi(bd), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
          if (j == (t == 0 ? T0 : T1) - 1) mma_commit(&bars[B_ODONE + t]);
        }
        mma_commit(&bars[B_PVDONE + buf]);
      }
    }
    __syncwarp();
  } else {
    // =============================== softmax ==================================================
    const uint8_t* maskb = p.mask ? p.mask + b * p.msb : nullptr;

    const int tile = warp >> 2;
    const int row = i0 + tid;
    const int T_mine = tile == 0 ? T0 : T1;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    float m_run = -CUDART_INF_F, l_run = 0.f;

    for (int j = 0; j < T_mine; ++j) {
      const int buf = j & 1, n0 = j * TK;
      // key visibility of this tile (key-padding mask, ragged end): one bit per key, the same for every row
      uint64_t vis = ~0ull;
      if (maskb || n0 + TK > p.Nk) {
        const int j0 = n0 + lane, j1 = j0 + 32;
        const bool ok0 = j0 < p.Nk && (!maskb || maskb[(int64_t)j0 * p.msn] != 0);
        const bool ok1 = j1 < p.Nk && (!maskb || maskb[(int64_t)j1 * p.msn] != 0);
        vis = ((uint64_t)__ballot_sync(0xffffffffu, ok1) << 32) | __ballot_sync(0xffffffffu, ok0);
      }
      if (p.causal) {
        const int lim = row - n0;  // columns <= lim are visible
        vis &= lim >= 63 ? ~0ull : (lim < 0 ? 0ull : ((2ull << lim) - 1ull));
      }
      const bool all_vis = __all_sync(0xffffffffu, vis == ~0ull);
      if (!failed) failed = !mbar_wait(&bars[B_SFULL + buf * 2 + tile], (j >> 1) & 1, WAIT_LIMIT);
      fence_after_sync();
      const uint32_t s_addr = tmem + lane_base + (buf * 2 + tile) * 64;
      uint32_t s0[32], s1[32];
      tmem_ld32(s_addr, s0);
      tmem_ld32(s_addr + 32, s1);
      tmem_ld_wait();
      // row maximum (four independent chains)
      float m4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
      if (all_vis) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], __uint_as_float(s0[i]), __uint_as_float(s0[i + 1]));
          m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], __uint_as_float(s1[i]), __uint_as_float(s1[i + 1]));
        }
      } else {
        const uint32_t v0 = (uint32_t)vis, v1 = (uint32_t)(vis >> 32);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if ((v0 >> i) & 1u) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(s0[i]));
          if ((v1 >> i) & 1u) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(s1[i]));
        }
      }
      const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
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
        // O was last written by PV(j-1)
        if (!failed) failed = !mbar_wait(&bars[B_PVDONE + (1 - buf)], ((j - 1) >> 1) & 1, WAIT_LIMIT);
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
      // P = 2^(s*c - m), written over the scores (16 packed columns per 32 scores)
      const float m_use = m_run == -CUDART_INF_F ? 0.f : m_run;
      float ls4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[32];
      // two copies of the loop: interior tiles (the common case) carry no masking arithmetic at all
      auto exponentials = [&](auto masked) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const uint32_t vh = (uint32_t)(vis >> (32 * hh));
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const uint32_t x0 = hh ? s1[2 * i] : s0[2 * i], x1 = hh ? s1[2 * i + 1] : s0[2 * i + 1];
            float p0 = ex2_approx(fmaf(__uint_as_float(x0), p.scale_log2, -m_use));
            float p1 = ex2_approx(fmaf(__uint_as_float(x1), p.scale_log2, -m_use));
            if (decltype(masked)::value) {
              p0 = ((vh >> (2 * i)) & 1u) ? p0 : 0.f;
              p1 = ((vh >> (2 * i + 1)) & 1u) ? p1 : 0.f;
            }
            ls4[i & 3] += p0 + p1;
            pk[hh * 16 + i] = pack2<T>(p0, p1);
          }
        }
      };
      if (all_vis) exponentials(std::false_type());
      else exponentials(std::true_type());
      l_run += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
      tmem_st32(s_addr, pk);
      tmem_st_wait();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B_PFULL + buf * 2 + tile]);
    }

    // ---- epilogue: O / l, LSE ---------------------------------------------------------------------
    if (T_mine > 0) {
      if (!failed) failed = !mbar_wait(&bars[B_ODONE + tile], 0, WAIT_LIMIT);
      fence_after_sync();
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
        p.lse[(int64_t)u * p.Nq + row] = l_run > 0.f ? m_run * LN2 + logf(l_run) : -CUDART_INF_F;
    }
  }
  if (failed) atomicOr(&g_tc_status, 1u);
  fence_before_sync();
  __syncthreads();
  if (warp == FWD_MMA_WARP) tmem_dealloc(tmem, 512);
}

}  // namespace pope

#include "tc_attn_fwd2.inl"

namespace pope {

// ---- host side ---------------------------------------------------------------------------------
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static bool stride_ok(const PopeStride3& s) { return s.b % 8 == 0 && s.h % 8 == 0 && s.n % 8 == 0; }

bool attn_fwd_tc_supported(const PopeAttnArgs& a) {
  const PopeShape& s = a.shape;
  if (s.dtype != POPE_BF16 && s.dtype != POPE_F16) return false;
  if (s.d != 64 && s.d != 96 && s.d != 128) return false;
  if (s.r % 16 != 0) return false;
  if (s.Nq < 64) return false;  // short query blocks take the key-split path
  // a phase table with a head axis (b, h, n, r) serves queries and keys alike only when both have the same heads
  if (s.r > 0 && a.embed.sf.h != 0 && s.H != s.Hk) return false;
  if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || !aligned16(a.out)) return false;
  if (!stride_ok(a.sq) || !stride_ok(a.sk) || !stride_ok(a.sv) || !stride_ok(a.so)) return false;
  // V is read by TMA boxes over (feature, row, head, batch): an axis with more than one entry needs a real, positive
  // stride (a V expanded over heads or batch, stride 0, or overlapping rows go to the exact family instead)
  if ((s.Hk > 1 && a.sv.h <= 0) || (s.B > 1 && a.sv.b <= 0) || (s.Nk > 1 && a.sv.n < s.d)) return false;
  return true;
}

// workspace: [fp32 and fp16 cos / sin tables][K' image tiles of all (batch, key head) units][Q' image tiles of all (batch, head) units]
static size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }

size_t attn_fwd_tc_workspace(const PopeAttnArgs& a) {
  const PopeShape& s = a.shape;
  return trig_tables_bytes(s.Nk, s.r, table_slices(a.embed, s.B, s.H)) + up256(image_bytes(s.B * s.Hk, s.Nk, s.d + s.r)) +
         image_bytes(s.B * s.H, s.Nq, s.d + s.r);
}

template <int D, typename T>
static cudaError_t launch_fwd_tc(const PopeAttnArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  const int KD = s.d + s.r;
  const bool bf16 = s.dtype == POPE_BF16;
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  const int slices = table_slices(a.embed, s.B, s.H), tab_heads = table_heads(a.embed, s.H), by_batch = a.embed.sf.b != 0;
  const TrigTables tt = trig_tables_at(ws, s.Nk, s.r, slices);
  uint8_t* kimg = ws + trig_tables_bytes(s.Nk, s.r, slices);
  uint8_t* qimg = kimg + up256(image_bytes(s.B * s.Hk, s.Nk, KD));
  TcFwdP p = {};
  p.H = s.H, p.Hk = s.Hk, p.Nq = s.Nq, p.Nk = s.Nk, p.r = s.r, p.causal = a.causal;
  p.scale_log2 = a.softmax_scale * LOG2E;
  p.q = a.q, p.k = a.k, p.v = a.v, p.o = a.out, p.lse = a.lse;
  p.sq = a.sq, p.sk = a.sk, p.sv = a.sv, p.so = a.so;
  p.freqs = a.embed.freqs, p.sfn = a.embed.sf.n, p.bias = a.embed.bias, p.bias_sh = a.embed.bias_stride_h;
  p.qimg = qimg, p.kimg = kimg;
  p.mask = a.mask, p.msb = a.mask_stride_b, p.msn = a.mask_stride_n;
  cudaError_t e;
  if (s.r > 0 && (e = launch_trig_tables(a.embed, s.Nk, s.r, nullptr, nullptr, tt.ch, tt.sh, st, slices, tab_heads)) != cudaSuccess) return e;
  ExpandJobs jobs;
  jobs.job[0] = expand_job(a.k, a.sk, s.B, s.Hk, s.Nk, s.r, 0, a.embed.bias, a.embed.bias_stride_h, kimg, s.Nk, by_batch, tab_heads);
  jobs.job[1] = expand_job(a.q, a.sq, s.B, s.H, s.Nq, s.r, s.Nk - s.Nq, nullptr, 0, qimg, s.Nk, by_batch, tab_heads);
#ifndef POPE_FWD_V1
  jobs.job[0].tile128 = 1;   // the kernel streams K' 128 keys at a time
#endif
  if ((e = launch_expand_images(jobs, 2, s.d, bf16, tt.ch, tt.sh, st)) != cudaSuccess) return e;
#ifndef POPE_FWD_V1
  return launch_fwd2_kernel<D, T>(a, p, st);
#endif
  CUtensorMap tmap_v;
  if (!make_chunk_tmap(&tmap_v, a.v, bf16, s.d, s.Nk, s.Hk, s.B, a.sv.n, a.sv.h, a.sv.b, TK)) return cudaErrorNotSupported;
  size_t smem = (size_t)2 * TQ * KD * 2 + 2 * (size_t)TK * KD * 2 + 2 * (size_t)TK * D * 2 + (B_COUNT + 1) * 8 + 16;
  // every CTA allocates all 512 TMEM columns: ask for more than half of the SM's shared memory so
  // that two CTAs are never co-resident
  if (smem < 120 * 1024) smem = 120 * 1024;
  if ((e = ensure_max_smem<attn_fwd_tc_kernel<D, T>>()) != cudaSuccess) return e;
  dim3 grid((s.Nq + 2 * TQ - 1) / (2 * TQ), s.B * s.H);
  attn_fwd_tc_kernel<D, T><<<grid, FWD_THREADS, smem, st>>>(p, tmap_v);
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
  if (s.H % s.Hk != 0 || s.Nq > s.Nk || s.r > s.d) return POPE_ERR_BAD_ARG;
  if (s.dtype != POPE_F32 && s.dtype != POPE_BF16 && s.dtype != POPE_F16) return POPE_ERR_BAD_ARG;
  if ((int64_t)s.B * s.H > 65535) return POPE_ERR_UNSUPPORTED;
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
  if (attn_fwd_tc(local, static_cast<cudaStream_t>(stream)) != cudaSuccess) return POPE_ERR_CUDA;
  note_last_path("tcgen05");
  return POPE_OK;
}
