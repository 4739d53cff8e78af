// PoPE flash-attention forward on the Blackwell tensor cores (tcgen05 + TMEM), sm_100a only.
//
// One CTA owns 128 query rows of one (batch, head) unit and sweeps the keys 128 at a time.
//   Q' = [a cos | pass | a sin] of its rows is expanded by the CTA itself, from q and the fp16 phase tables, straight
//        into TENSOR memory ((d + r) / 2 columns): it is the TMEM-side A operand of every score product and never
//        exists in global or shared memory
//   K' comes from the operand images that a pre-pass builds once per call (tc_expand.cu, 128-row tiles, the per-head
//        phase bias of the keys folded in): every CTA of a unit re-reads it, so it is expanded once, not per CTA
//   loader warps  : one K' image tile per step by one cp.async.bulk; the V tile of the step by cp.async.bulk.tensor
//                   boxes (128-byte swizzled rows) straight from the caller's strided V
//   score warp    : one lane issues  S = Q' K'^T  (128x128x16 products, A from tensor memory) into one of two buffers
//   softmax warps : two threads per query row: each pulls its 64 scores out of TMEM, applies the causal / key-padding
//                   masks, keeps the running max (row maxima exchanged through shared memory) and sum, and writes P
//                   (16-bit) back into TMEM over the scores
//   PV warp       : one lane issues  O += P V  with P read straight from TMEM
// All hand-offs are mbarriers (copy completion by transaction bytes, MMA completion by tcgen05.commit).
// Tensor memory: Q' [0, 128), S / P double-buffered [128, 384), O [384, 512); shared memory holds nothing but two
// stages of (K' tile, V tile).  An earlier version kept two 128-row Q' tiles in SHARED memory and swept 64 keys per
// step: its 128x64x16 score products read 6 KB of operands for 32 clocks of tensor time, and shared-memory bandwidth
// set its pace (0.535 ms against 0.49 ms at B=4, H=16, N=4096, d=r=128).
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
                    int batch, int64_t sn, int64_t sh, int64_t sb, int box_cols, int box_rows, CUtensorMapSwizzle swz,
                    CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
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
  return encode(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, promo,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_chunk_tmap(CUtensorMap* out, const void* base, bool is_bf16, int d, int rows, int heads, int batch, int64_t sn,
                     int64_t sh, int64_t sb, int box_rows) {
  return tmap_4d(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, d, rows, heads,
                 batch, sn, sh, sb, 8, box_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
}

// 16-bit rows cut into boxes of 64 features (128 bytes) x box_rows rows, 128-byte swizzled
bool make_wide_tmap(CUtensorMap* out, const void* base, bool is_bf16, int d, int rows, int heads, int batch, int64_t sn,
                           int64_t sh, int64_t sb, int box_rows) {
  return tmap_4d(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, d, rows, heads,
                 batch, sn, sh, sb, 64, box_rows, CU_TENSOR_MAP_SWIZZLE_128B);
}

// An operand image ([tile][chunk][64 rows x 16 B]) seen as (1 KB run, tile, chunk): a box of (1 KB, 2 tiles, all chunks)
// lands in shared memory as [chunk][128 rows][16 B], i.e. a resident 128-row operand arrives by ONE copy.
bool make_image_tmap(CUtensorMap* out, const void* img, int64_t ntiles, int chunks) {
  TmapEncodeFn encode = tmap_encoder();
  if (!encode || (reinterpret_cast<uintptr_t>(img) & 15) != 0 || chunks < 1 || chunks > 256 || ntiles < 2) return false;
  cuuint64_t dims[4] = {128, (cuuint64_t)ntiles, (cuuint64_t)chunks, 1};                    // 128 x 8 bytes = one 1 KB run
  cuuint64_t strides[3] = {(cuuint64_t)chunks * 1024, 1024, (cuuint64_t)ntiles * chunks * 1024};
  cuuint32_t box[4] = {128, 2, (cuuint32_t)chunks, 1}, estr[4] = {1, 1, 1, 1};
  return encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT64, 4, const_cast<void*>(img), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_load_tmap_f32(CUtensorMap* out, const void* base, int cols, int rows, int heads, int batch, int64_t sn, int64_t sh,
                        int64_t sb, int box_rows) {
  // (a tile row is 2 or 4 neighbouring boxes of 128 bytes: 256-byte promotion fetches the neighbour along; -0.8 % on the
  // similarity backward)
  return tmap_4d(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, cols, rows, heads, batch, sn, sh, sb, 32, box_rows,
                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
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
  const uint8_t* kimg; // expanded K' image tiles (phase bias folded in), (B * Hk) units
  const __half *ch, *sh;         // fp16 cos / sin phase tables, [slice][Nk][r]
  int64_t tab_slice_stride;      // elements per table slice (Nk * r)
  int tab_by_batch, tab_heads;   // slice of a unit: (tab_by_batch ? batch : 0) * tab_heads + head % tab_heads
  const uint8_t* mask;
  int64_t msb, msn;
};

constexpr int TQ = 128;   // rows per MMA tile

constexpr int FW_TK = 128;                         // keys per step
constexpr int FW_NPR = 2;                          // softmax threads per query row (2 or 4; 4 measured the same), 128 / FW_NPR scores each
constexpr int FW_SM_WARPS = 4 * FW_NPR;            // softmax warps
constexpr int FW_KLOAD_WARP = FW_SM_WARPS;         // one lane issues the K' copies (one 128-row image tile per step)
constexpr int FW_S_WARP = FW_SM_WARPS + 1;         // one lane issues S = Q' K'^T; owns the TMEM allocation
constexpr int FW_PV_WARP = FW_SM_WARPS + 2;        // one lane issues O += P V
constexpr int FW_VLOAD_WARP = FW_SM_WARPS + 3;     // one lane issues the V boxes
constexpr int FW_THREADS = 32 * (FW_VLOAD_WARP + 1);
constexpr uint32_t FW_TS = 128, FW_TO = 384;       // first TMEM column of the S / P buffers and of O (Q' starts at 0)

constexpr int FW_VST = 2;                          // V stages (up to 3; a third one changed nothing measurable)
enum {
  FW_KFULL = 0,    // [2] K' tile landed (transaction bytes)
  FW_KFREE = 2,    // [2] tcgen05.commit: S(j) has completed, its K' buffer may be refilled
  FW_PVDONE = 4,   // [2] tcgen05.commit: O += P V of tile j has completed: S / P buffer j & 1 is free
  FW_SFULL = 6,    // [2] tcgen05.commit: the scores of tile j are in TMEM
  FW_PFULL = 8,    // [2] the softmax warps: the probabilities of tile j are in TMEM
  FW_QFULL = 10,   // the softmax warps: Q' is in TMEM
  FW_ODONE = 11,   // tcgen05.commit: the last O += P V has completed
  FW_VFULL = 12,   // [3] V tile landed in stage j % FW_VST (transaction bytes)
  FW_VFREE = 15,   // [3] tcgen05.commit: O += P V of tile j has completed: V stage j % FW_VST is free
  FW_COUNT = 18
};

template <int D, typename T>
__global__ void __launch_bounds__(FW_THREADS, 1) attn_fwd_tc_kernel(TcFwdP p, const __grid_constant__ CUtensorMap tmap_v) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzled tiles sit on 1 KB boundaries
  // V tiles: D a multiple of 64 -> boxes of 64 features (128-byte rows, 128-byte swizzled); else 16-byte chunk columns
  constexpr bool VWIDE = D % 64 == 0;
  const int KD = D + p.r, KSTEPS = KD >> 4;
  const int KBUF = FW_TK * KD * 2;                  // one K' stage: [KD/8 chunks][128 keys][16 B]
  constexpr int VBUF = FW_TK * D * 2;               // one V stage:  [D/8 chunks][128 keys][16 B]
  constexpr int CSV = FW_TK * 16;                   // chunk stride of both
  uint8_t* Ks = smem;
  uint8_t* Vs = Ks + 2 * KBUF;
  float* xch = reinterpret_cast<float*>(Vs + FW_VST * VBUF);       // [2 step parities][FW_NPR parts][128 rows] row maxima
  float* lxch = xch;                                                 // [FW_NPR parts][128 rows] row sums (epilogue: xch is dead)
  uint64_t* bars = reinterpret_cast<uint64_t*>(xch + 2 * FW_NPR * TQ);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + FW_COUNT + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int u = blockIdx.y, b = u / p.H, h = u % p.H, hk = h % p.Hk;
  const int i0 = (gridDim.x - 1 - blockIdx.x) * TQ;  // heavy (late) row blocks first
  int n_end = p.Nk;
  if (p.causal) n_end = min(n_end, min(i0 + TQ, p.Nq));
  const int T_tiles = (n_end + FW_TK - 1) / FW_TK;

  if (warp == FW_S_WARP) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[FW_KFULL + i], 1);
      mbar_init(&bars[FW_KFREE + i], 1), mbar_init(&bars[FW_PVDONE + i], 1);
      mbar_init(&bars[FW_SFULL + i], 1), mbar_init(&bars[FW_PFULL + i], FW_SM_WARPS);
    }
    for (int i = 0; i < FW_VST; ++i) mbar_init(&bars[FW_VFULL + i], 1), mbar_init(&bars[FW_VFREE + i], 1);
    mbar_init(&bars[FW_QFULL], FW_SM_WARPS);
    mbar_init(&bars[FW_ODONE], 1);
    mbar_init_fence();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  bool failed = false;

  if (warp == FW_KLOAD_WARP) {
    // =============================== copies: K' ==================================================
    // a 128-key stage is one 128-row image tile (the pre-pass interleaves pairs of its 64-row tiles): one bulk copy.
    // (Assembled from 2 x KD / 8 copies of 1 KB the stage took longer to arrive than the whole step should last.)
    if (lane == 0) {
      pdl_wait();   // the image pre-pass has completed
      const uint8_t* kimg = p.kimg + (int64_t)(b * p.Hk + hk) * (int64_t)(image_tiles(p.Nk) / 2) * KBUF;
      int j = 0;
      for (; j < T_tiles; ++j) {
        const int buf = j & 1;
        if (j >= 2 && !failed) failed = !mbar_wait(&bars[FW_KFREE + buf], ((j - 2) >> 1) & 1, WAIT_LIMIT);
        if (failed) break;
        mbar_expect_tx(&bars[FW_KFULL + buf], KBUF);
        bulk_load(Ks + buf * KBUF, kimg + (int64_t)j * KBUF, KBUF, &bars[FW_KFULL + buf]);
      }
      if (failed) drain_copies(&bars[FW_KFULL], 2, j - 2, j);
    }
    __syncwarp();
  } else if (warp == FW_VLOAD_WARP) {
    // =============================== copies: V ===================================================
    if (lane == 0) {
      int j = 0;
      for (; j < T_tiles; ++j) {
        const int buf = j % FW_VST, n0 = j * FW_TK;
        if (j >= FW_VST && !failed) failed = !mbar_wait(&bars[FW_VFREE + buf], ((j - FW_VST) / FW_VST) & 1, WAIT_LIMIT);
        if (failed) { drain_copies(&bars[FW_VFULL], FW_VST, j - FW_VST, j); break; }
        mbar_expect_tx(&bars[FW_VFULL + buf], VBUF);
        if (VWIDE) {
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(Vs + buf * VBUF + c * (FW_TK * 128), &tmap_v, &bars[FW_VFULL + buf], c * 64, n0, hk, b);
        } else {
#pragma unroll
          for (int c = 0; c < D / 8; ++c) tma_load_4d(Vs + buf * VBUF + c * CSV, &tmap_v, &bars[FW_VFULL + buf], c * 8, n0, hk, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == FW_S_WARP) {
    // =============================== MMA issue: S = Q' K'^T ======================================
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc(TcFmt<T>::fmt, TQ, FW_TK, false, false);
      const uint32_t ks_addr = smem_u32(Ks);
      if (!mbar_wait(&bars[FW_QFULL], 0, WAIT_LIMIT)) failed = true;
      for (int j = 0; j < T_tiles && !failed; ++j) {
        const int buf = j & 1;
        failed = !mbar_wait(&bars[FW_KFULL + buf], (j >> 1) & 1, WAIT_LIMIT);
        // score buffer j & 1 still holds P(j-2) until PV(j-2) has read it
        if (j >= 2 && !failed) failed = !mbar_wait(&bars[FW_PVDONE + buf], ((j - 2) >> 1) & 1, WAIT_LIMIT);
        if (failed) break;
        fence_after_sync();
        const uint32_t d = tmem + FW_TS + buf * FW_TK;
        const uint64_t bd = smem_desc(ks_addr + buf * KBUF, CSV, 128);
        uint32_t blo = desc_lo(bd), at = tmem;
#pragma unroll 4
        for (int ks = 0; ks < KSTEPS; ++ks) {
          mma_ts_lh(d, at, blo, desc_hi(bd), idesc_s, ks > 0 ? 1u : 0u);
          at += 8, blo += (2 * CSV) >> 4;
        }
        mma_commit(&bars[FW_SFULL + buf]);
        mma_commit(&bars[FW_KFREE + buf]);
      }
    }
    __syncwarp();
  } else if (warp == FW_PV_WARP) {
    // =============================== MMA issue: O += P V =========================================
    if (lane == 0) {
      const uint32_t idesc_o = instr_desc(TcFmt<T>::fmt, TQ, D, false, true);
      const uint32_t vs_addr = smem_u32(Vs);
      for (int j = 0; j < T_tiles && !failed; ++j) {
        const int buf = j & 1;
        failed = !mbar_wait(&bars[FW_VFULL + j % FW_VST], (j / FW_VST) & 1, WAIT_LIMIT);
        if (!failed) failed = !mbar_wait(&bars[FW_PFULL + buf], (j >> 1) & 1, WAIT_LIMIT);
        if (failed) break;
        fence_after_sync();
        const uint32_t a = tmem + FW_TS + buf * FW_TK;
        // B = V, MN-major: wide boxes: 64-feature blocks 16 KB apart, 8-key groups 1 KB apart, 2 KB per 16 keys;
        // chunk columns: 8-feature chunks CSV apart, 8-key groups 128 bytes apart, 256 bytes per 16 keys
        const uint32_t vaddr = vs_addr + (j % FW_VST) * VBUF;
        const uint64_t bd = VWIDE ? smem_desc_sw128(vaddr, FW_TK * 128, 1024) : smem_desc(vaddr, 128, CSV);
        constexpr uint32_t kstep = VWIDE ? (2048 >> 4) : ((2 * 128) >> 4);
        constexpr int CPT = FW_TK / FW_NPR;   // P of keys [CPT t, CPT t + CPT) sits in the first CPT / 2 columns of part t
#pragma unroll
        for (int ks = 0; ks < FW_TK / 16; ++ks)
          mma_ts_lh(tmem + FW_TO, a + (ks * 16 / CPT) * CPT + (ks * 16 % CPT) / 2, desc_lo(bd) + ks * kstep, desc_hi(bd), idesc_o,
                    (j > 0 || ks > 0) ? 1u : 0u);
        if (j == T_tiles - 1) mma_commit(&bars[FW_ODONE]);
        mma_commit(&bars[FW_PVDONE + buf]);
        mma_commit(&bars[FW_VFREE + j % FW_VST]);
      }
    }
    __syncwarp();
  } else {
    // =============================== softmax: FW_NPR threads per query row =======================
    const uint8_t* maskb = p.mask ? p.mask + b * p.msb : nullptr;
    constexpr int CPT = FW_TK / FW_NPR;              // score columns per thread (64 or 32)
    constexpr int OC = FW_NPR == 4 ? 32 : D / 2;     // output columns per thread ...
    const int rloc = tid & 127, part = tid >> 7;
    const bool o_active = part * OC < D;             // ... of the threads that own any
    const int row = i0 + rloc;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const int row_bar = 1 + (warp & 3);   // named barrier of the FW_NPR warps that share 32 rows
    auto row_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(row_bar), "n"(32 * FW_NPR) : "memory"); };
    pdl_wait();   // the phase tables read below come from the kernels before this one
    {
      // Q' = [a cos f | pass | a sin f] of this CTA's rows, expanded HERE from q and the fp16 phase tables and written
      // straight into tensor memory (lane = row, 4 columns per 8-feature chunk): the resident operand never exists in
      // global memory.  The threads of a row share its 16-byte groups; rows past Nq are zero.
      constexpr int DC = D >> 3;
      const int RC = p.r >> 3;
      const bool live = row < p.Nq;
      const T* qrow = static_cast<const T*>(p.q) + b * p.sq.b + h * p.sq.h + (int64_t)row * p.sq.n;
      const int64_t trow = p.tab_slice_stride * ((p.tab_by_batch ? b : 0) * p.tab_heads + h % p.tab_heads) +
                           (int64_t)(p.Nk - p.Nq + row) * p.r;   // bottom-right positions
      // (a compact loop on purpose: unrolled into groups of chunks with their loads up front, this prologue came out
      // 14-30 us slower per forward -- its code displaces the main loop's in the instruction cache)
      for (int c = part; c < DC; c += FW_NPR) {
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (live) raw = __ldg(reinterpret_cast<const uint4*>(qrow + c * 8));
        if (c < RC) {
          uint4 cq = make_uint4(0, 0, 0, 0), sq = cq;
          if (live) {
            cq = __ldg(reinterpret_cast<const uint4*>(p.ch + trow + c * 8));
            sq = __ldg(reinterpret_cast<const uint4*>(p.sh + trow + c * 8));
          }
          const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w}, cw[4] = {cq.x, cq.y, cq.z, cq.w}, sw[4] = {sq.x, sq.y, sq.z, sq.w};
          uint32_t o1[4], o2[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 xv = unpack2<T>(rw[e]), cv = unpack2<__half>(cw[e]), sv2 = unpack2<__half>(sw[e]);
            const float a0 = live ? softplus_fast(xv.x) : 0.f, a1 = live ? softplus_fast(xv.y) : 0.f;
            o1[e] = pack2<T>(a0 * cv.x, a1 * cv.y);
            o2[e] = pack2<T>(a0 * sv2.x, a1 * sv2.y);
          }
          tmem_st4(tmem + lane_base + c * 4, o1[0], o1[1], o1[2], o1[3]);
          tmem_st4(tmem + lane_base + (DC + c) * 4, o2[0], o2[1], o2[2], o2[3]);
        } else {
          tmem_st4(tmem + lane_base + c * 4, raw.x, raw.y, raw.z, raw.w);
        }
      }
      tmem_st_wait();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[FW_QFULL]);
    }
    float m_run = -CUDART_INF_F, l_run = 0.f;

    for (int j = 0; j < T_tiles; ++j) {
      const int buf = j & 1, n0 = j * FW_TK + part * CPT;   // first key of this thread's columns
      // key visibility of this thread's columns (key-padding mask, ragged end): one bit per key, the same for every row
      uint64_t vis = ~0ull;
      if (maskb || n0 + CPT > p.Nk) {
        const int j0 = n0 + lane, j1 = j0 + 32;
        const bool ok0 = j0 < p.Nk && (!maskb || maskb[(int64_t)j0 * p.msn] != 0);
        const bool ok1 = CPT == 32 || (j1 < p.Nk && (!maskb || maskb[(int64_t)j1 * p.msn] != 0));
        vis = ((uint64_t)__ballot_sync(0xffffffffu, ok1) << 32) | __ballot_sync(0xffffffffu, ok0);
      }
      if (p.causal) {
        const int lim = row - n0;  // columns <= lim are visible
        vis &= lim >= 63 ? ~0ull : (lim < 0 ? 0ull : ((2ull << lim) - 1ull));
      }
      if (CPT == 32) vis |= 0xffffffff00000000ull;
      const bool all_vis = __all_sync(0xffffffffu, vis == ~0ull);
      if (!failed) failed = !mbar_wait(&bars[FW_SFULL + buf], (j >> 1) & 1, WAIT_LIMIT);
      fence_after_sync();
      const uint32_t s_addr = tmem + lane_base + FW_TS + buf * FW_TK + part * CPT;
      uint32_t sv[CPT / 32][32];
#pragma unroll
      for (int q = 0; q < CPT / 32; ++q) tmem_ld32(s_addr + q * 32, sv[q]);
      tmem_ld_wait();
      // maximum of this thread's scores (four independent chains), then of the row
      float m4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
      if (all_vis) {
#pragma unroll
        for (int q = 0; q < CPT / 32; ++q)
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], __uint_as_float(sv[q][i]), __uint_as_float(sv[q][i + 1]));
      } else {
#pragma unroll
        for (int q = 0; q < CPT / 32; ++q) {
          const uint32_t vq = (uint32_t)(vis >> (32 * q));
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if ((vq >> i) & 1u) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(sv[q][i]));
        }
      }
      float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      xch[(buf * FW_NPR + part) * TQ + rloc] = mx;
      row_sync();
#pragma unroll
      for (int t = 0; t < FW_NPR; ++t) mx = fmaxf(mx, xch[(buf * FW_NPR + t) * TQ + rloc]);
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
        // O was last written by PV(j-1); the threads of a row rescale OC of its columns each
        if (!failed) failed = !mbar_wait(&bars[FW_PVDONE + (1 - buf)], ((j - 1) >> 1) & 1, WAIT_LIMIT);
        fence_after_sync();
        if (o_active) {
          const uint32_t o_addr = tmem + lane_base + FW_TO + part * OC;
#pragma unroll
          for (int c0 = 0; c0 < OC; c0 += 16) {
            uint32_t ov[16];
            tmem_ld16(o_addr + c0, ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st16(o_addr + c0, ov);
          }
          tmem_st_wait();
        }
      }
      // P = 2^(s*c - m), written over this thread's scores (CPT / 2 packed columns for its CPT scores)
      const float m_use = m_run == -CUDART_INF_F ? 0.f : m_run;
      float ls4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[CPT / 32][16];
      auto exponentials = [&](auto masked) {
#pragma unroll
        for (int q = 0; q < CPT / 32; ++q) {
          const uint32_t vq = (uint32_t)(vis >> (32 * q));
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float p0 = ex2_approx(fmaf(__uint_as_float(sv[q][2 * i]), p.scale_log2, -m_use));
            float p1 = ex2_approx(fmaf(__uint_as_float(sv[q][2 * i + 1]), p.scale_log2, -m_use));
            if (decltype(masked)::value) {
              p0 = ((vq >> (2 * i)) & 1u) ? p0 : 0.f;
              p1 = ((vq >> (2 * i + 1)) & 1u) ? p1 : 0.f;
            }
            ls4[i & 3] += p0 + p1;
            pk[q][i] = pack2<T>(p0, p1);
          }
        }
      };
      if (all_vis) exponentials(std::false_type());
      else exponentials(std::true_type());
      l_run += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
#pragma unroll
      for (int q = 0; q < CPT / 32; ++q) tmem_st16(s_addr + q * 16, pk[q]);
      tmem_st_wait();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[FW_PFULL + buf]);
    }

    // ---- epilogue: O / l, LSE ---------------------------------------------------------------------
    row_sync();   // (every thread of the row is past its last look at the row maxima)
    lxch[part * TQ + rloc] = l_run;
    row_sync();
    float l_tot = 0.f;
#pragma unroll
    for (int t = 0; t < FW_NPR; ++t) l_tot += lxch[t * TQ + rloc];
    if (T_tiles > 0 && !failed) failed = !mbar_wait(&bars[FW_ODONE], 0, WAIT_LIMIT);
    fence_after_sync();
    const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
    if (o_active) {
      const uint32_t o_addr = tmem + lane_base + FW_TO + part * OC;
      T* orow = (T*)p.o + b * p.so.b + h * p.so.h + (int64_t)row * p.so.n + part * OC;
#pragma unroll
      for (int c0 = 0; c0 < OC; c0 += 16) {
        uint32_t ov[16];
        tmem_ld16(o_addr + c0, ov);
        tmem_ld_wait();
        if (row < p.Nq) {
#pragma unroll
          for (int i = 0; i < 16; i += 8) {
            uint4 w;
            w.x = pack2<T>(__uint_as_float(ov[i]) * inv, __uint_as_float(ov[i + 1]) * inv);
            w.y = pack2<T>(__uint_as_float(ov[i + 2]) * inv, __uint_as_float(ov[i + 3]) * inv);
            w.z = pack2<T>(__uint_as_float(ov[i + 4]) * inv, __uint_as_float(ov[i + 5]) * inv);
            w.w = pack2<T>(__uint_as_float(ov[i + 6]) * inv, __uint_as_float(ov[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c0 + i) = w;
          }
        }
      }
    }
    if (part == 0 && row < p.Nq) p.lse[(int64_t)u * p.Nq + row] = l_tot > 0.f ? m_run * LN2 + logf(l_tot) : -CUDART_INF_F;
  }
  if (failed) atomicOr(&g_tc_status, 1u);
  fence_before_sync();
  __syncthreads();
  if (warp == FW_S_WARP) tmem_dealloc(tmem, 512);
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
  // a phase table with a head axis (b, h, n, r) serves queries and keys alike only when both have the same heads
  if (s.r > 0 && a.embed.sf.h != 0 && s.H != s.Hk) return false;
  if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || !aligned16(a.out)) return false;
  if (!stride_ok(a.sq) || !stride_ok(a.sk) || !stride_ok(a.sv) || !stride_ok(a.so)) return false;
  // V is read by TMA boxes over (feature, row, head, batch): an axis with more than one entry needs a real, positive
  // stride (a V expanded over heads or batch, stride 0, or overlapping rows go to the exact family instead)
  if ((s.Hk > 1 && a.sv.h <= 0) || (s.B > 1 && a.sv.b <= 0) || (s.Nk > 1 && a.sv.n < s.d)) return false;
  return true;
}

// workspace: [fp16 cos / sin tables][K' image tiles of all (batch, key head) units]
static size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }

size_t attn_fwd_tc_workspace(const PopeAttnArgs& a) {
  const PopeShape& s = a.shape;
  return trig_tables_bytes(s.Nk, s.r, table_slices(a.embed, s.B, s.H)) + up256(image_bytes(s.B * s.Hk, s.Nk, s.d + s.r));
}

template <int D, typename T>
static cudaError_t launch_fwd_tc(const PopeAttnArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  const bool bf16 = s.dtype == POPE_BF16;
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  const int slices = table_slices(a.embed, s.B, s.H), tab_heads = table_heads(a.embed, s.H), by_batch = a.embed.sf.b != 0;
  const TrigTables tt = trig_tables_at(ws, s.Nk, s.r, slices);
  uint8_t* kimg = ws + trig_tables_bytes(s.Nk, s.r, slices);
  TcFwdP p = {};
  p.H = s.H, p.Hk = s.Hk, p.Nq = s.Nq, p.Nk = s.Nk, p.r = s.r, p.causal = a.causal;
  p.scale_log2 = a.softmax_scale * LOG2E;
  p.q = a.q, p.k = a.k, p.v = a.v, p.o = a.out, p.lse = a.lse;
  p.sq = a.sq, p.sk = a.sk, p.sv = a.sv, p.so = a.so;
  p.freqs = a.embed.freqs, p.sfn = a.embed.sf.n, p.bias = a.embed.bias, p.bias_sh = a.embed.bias_stride_h;
  p.kimg = kimg;
  p.ch = static_cast<const __half*>(tt.ch), p.sh = static_cast<const __half*>(tt.sh);
  p.tab_slice_stride = (int64_t)s.Nk * s.r, p.tab_by_batch = by_batch, p.tab_heads = tab_heads;
  p.mask = a.mask, p.msb = a.mask_stride_b, p.msn = a.mask_stride_n;
  // all host-side preparation first, then the three launches back to back (what the host does between two launches is
  // time the GPU spends idle on small problems)
  const int KD = s.d + s.r;
  CUtensorMap tmap_v;
  const bool tm_ok = D % 64 == 0 ? make_wide_tmap(&tmap_v, a.v, bf16, s.d, s.Nk, s.Hk, s.B, a.sv.n, a.sv.h, a.sv.b, FW_TK)
                                 : make_chunk_tmap(&tmap_v, a.v, bf16, s.d, s.Nk, s.Hk, s.B, a.sv.n, a.sv.h, a.sv.b, FW_TK);
  if (!tm_ok) return cudaErrorNotSupported;
  size_t smem = 2 * (size_t)FW_TK * KD * 2 + FW_VST * (size_t)FW_TK * D * 2 + 2 * FW_NPR * TQ * sizeof(float) + (FW_COUNT + 1) * 8 + 16 + 1024;
  // every CTA allocates all 512 TMEM columns: keep two CTAs from sharing an SM
  if (smem < 120 * 1024) smem = 120 * 1024;
  cudaError_t e = ensure_max_smem<attn_fwd_tc_kernel<D, T>>();
  if (e != cudaSuccess) return e;
  // K' (phase bias folded in) as 128-row image tiles: the kernel streams it 128 keys at a time; Q' is expanded in the kernel
  ExpandJobs jobs;
  jobs.job[0] = expand_job(a.k, a.sk, s.B, s.Hk, s.Nk, s.r, 0, a.embed.bias, a.embed.bias_stride_h, kimg, s.Nk, by_batch, tab_heads);
  jobs.job[0].tile128 = 1;
  if (s.r > 0 && (e = launch_trig_tables(a.embed, s.Nk, s.r, nullptr, nullptr, tt.ch, tt.sh, st, slices, tab_heads)) != cudaSuccess) return e;
  // tables -> images -> attention: the second and third kernel start as programmatic dependents of the one before (each
  // waits for it before its first read of that kernel's output); the first launch of the chain is an ordinary one
  if ((e = launch_expand_images(jobs, 1, s.d, bf16, tt.ch, tt.sh, st, s.r > 0)) != cudaSuccess) return e;
  dim3 grid((s.Nq + TQ - 1) / TQ, s.B * s.H);
  return launch_dependent(attn_fwd_tc_kernel<D, T>, grid, dim3(FW_THREADS), smem, st, p, tmap_v);
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
