// Fused PoPE similarity  sim = q' k'^T  on the Blackwell tensor cores (tcgen05 + TMEM), sm_100a only.
//
// The kernel is bound by the store of the Nq x Nk output; the contraction only has to keep up.  fp32
// inputs must come out at fp32 accuracy (1e-4 of max|sim|), which one bf16 product misses by an order of
// magnitude, so every expanded operand element x is split into two bf16 numbers  x = hi + lo  and the
// product is accumulated as  hi*hi' + hi*lo' + lo*hi'  (the dropped lo*lo' term is below 2^-17 relative).
// bf16 / fp16 inputs take the single-product path.
//
// Work list = all 128-key tiles of all row blocks of all (batch, head) units, flattened with the key tile
// fastest; the grid is one CTA per SM and CTA i takes the i-th contiguous slice of the list, so every SM
// gets the same number of tiles (within one) and re-expands a row block at most twice.  A row block is 256
// query rows (two MMA tiles) where shared memory allows, else 128.
//   * Expanding operands inside the main loop made the kernel transform-bound: about 3000 clocks of softplus /
//     split work per key tile, serialised with the MMA chains through the one key buffer that fits, against the
//     5700 clocks which the 128 KB of output of a tile need at an SM's share of the HBM write rate (measured:
//     2.4 TB/s); and the once-per-row-block expansion of Q' still cost 12000 clocks each time it ran (large unrolled
//     code that is cold in the instruction cache).  ONE pre-pass launch therefore expands every Q and K tile once into
//     the caller's workspace, (hi | lo) in the byte order the tensor core reads, with the reference's own phase
//     arithmetic (query phase f, key phase fl(f + b), accurate sincosf), and the main kernel brings a tile in with a
//     single cp.async.bulk.
//   * loader warp: the Q' tiles of a row block, and K' tile t + 1 while the MMA chains of tile t run;
//     issuing warp: the chains of a tile into one of two TMEM buffers;
//     8 worker warps: TMEM -> registers -> the warp's own 128-byte-swizzled staging tile -> global memory with one
//     tensor-map store of 32 rows x 128 bytes per warp and pass (full lines; the copy engine clips ragged edges).
//
// Reference semantics: PoPE_pytorch/triton_pope.py:28-83, PoPE_pytorch/attention.py:30-47.
#include <algorithm>
#include <cstring>
#include <type_traits>

#include "kernels.h"
#include "tc_common.cuh"

namespace pope {

struct TcSimP {
  int H, Hk, Nq, Nk, d, r;
  int ktiles, rblocks;       // 128-key tiles per unit, row blocks (MT x 128 rows) per unit
  int64_t total_tiles;       // units x rblocks x ktiles: the flattened work list cut into one contiguous range per CTA
  int use_tma;               // 1: tiles leave through the swizzled staging tiles and tensor-map stores
  void* sim;
  Strides ss;
  const uint8_t* qimg;       // expanded Q' tiles, [unit = b * H + h][row tile][hi | lo][chunk][128 rows][16 B]
  const uint8_t* kimg;       // expanded K' tiles, [unit = b * Hk + hk][key tile][...]
  unsigned int* status;
};

constexpr int SIM_M = 128;         // rows of one MMA tile
constexpr int SIM_N = 128;         // keys per step
constexpr int SIM_WORKERS = 8;     // warps 0-7: draining of the accumulators
constexpr int SIM_MMA_WARP = 8;    // one lane issues the MMA chains; owns the TMEM allocation
constexpr int SIM_LOAD_WARP = 9;   // one lane issues the K' tile copies
constexpr int SIM_THREADS = 320;

// ch / sh (may be null): the same tables rounded to fp16 (cos and sin lie in [-1, 1]: 2^-12 absolute error), read by
// the operand-image pre-pass, whose result is rounded to 8 or 11 bits anyway.
// grid.y = table slice (batch entry x head of a batched caller table)
__global__ void pope_trig_table_f32_kernel(PhaseSrc src, int n, int r, float* ctab, float* stab, __half* ch, __half* sh) {
  pdl_trigger();   // the kernel behind this one may set itself up; it waits for this grid before it reads the tables
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)n * r) return;
  const int pos = idx / r, c = idx % r, slice = blockIdx.y;
  if (!src.pos) src.freqs += (slice / src.tab_heads) * src.sfb + (slice % src.tab_heads) * src.sfh;
  float sn, cs;
  sincosf(src.at(pos, c), &sn, &cs);
  idx += (int64_t)slice * n * r;
  if (ctab) stab[idx] = sn, ctab[idx] = cs;
  if (ch) ch[idx] = __float2half_rn(cs), sh[idx] = __float2half_rn(sn);
}

cudaError_t launch_trig_tables(const PopeEmbed& e, int n, int r, float* ctab, float* stab, void* ch, void* sh, cudaStream_t st,
                               int slices, int tab_heads) {
  const int64_t total = (int64_t)n * r;
  PhaseSrc src = phase_src(e);
  src.tab_heads = tab_heads;
  pope_trig_table_f32_kernel<<<dim3((unsigned)((total + 255) / 256), (unsigned)slices), 256, 0, st>>>(
      src, n, r, ctab, stab, static_cast<__half*>(ch), static_cast<__half*>(sh));
  return cudaGetLastError();
}
cudaError_t launch_trig_table_f32(const PopeEmbed& e, int n, int r, float* ctab, float* stab, cudaStream_t st) {
  return launch_trig_tables(e, n, r, ctab, stab, nullptr, nullptr, st);
}

template <typename T> struct Load8;
template <> struct Load8<float> {
  static __device__ __forceinline__ void run(const float* p, float (&x)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x, x[1] = a.y, x[2] = a.z, x[3] = a.w, x[4] = b.x, x[5] = b.y, x[6] = b.z, x[7] = b.w;
  }
};
template <> struct Load8<__nv_bfloat16> {
  static __device__ __forceinline__ void run(const __nv_bfloat16* p, float (&x)[8]) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 v = unpack2<__nv_bfloat16>(w[e]);
      x[2 * e] = v.x, x[2 * e + 1] = v.y;
    }
  }
};
template <> struct Load8<__half> {
  static __device__ __forceinline__ void run(const __half* p, float (&x)[8]) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 v = unpack2<__half>(w[e]);
      x[2 * e] = v.x, x[2 * e + 1] = v.y;
    }
  }
};

// write 8 fp32 values as one 16-byte bf16 chunk (hi) and, when SPLIT, the residual chunk (lo)
template <bool SPLIT>
__device__ __forceinline__ void put_chunk(uint8_t* hi_dst, uint8_t* lo_dst, const float (&v)[8]) {
  uint32_t h[4], l[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __nv_bfloat162 hh = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
    h[e] = *reinterpret_cast<const uint32_t*>(&hh);
    if (SPLIT) {
      const float2 back = unpack2<__nv_bfloat16>(h[e]);
      const __nv_bfloat162 ll = __floats2bfloat162_rn(v[2 * e] - back.x, v[2 * e + 1] - back.y);
      l[e] = *reinterpret_cast<const uint32_t*>(&ll);
    }
  }
  *reinterpret_cast<uint4*>(hi_dst) = make_uint4(h[0], h[1], h[2], h[3]);
  if (SPLIT) *reinterpret_cast<uint4*>(lo_dst) = make_uint4(l[0], l[1], l[2], l[3]);
}


constexpr int SIM_CSK = SIM_N * 16;        // K' chunk stride: a tile arrives by one bulk copy, exactly as the pre-pass wrote it
constexpr int SIM_CSQ = SIM_M * 16;        // Q' chunk stride
constexpr int SIM_STG_WARP = 32 * 128;     // staging tile of one worker warp: 32 rows x 128 bytes, 128-byte swizzled

// ---- pre-pass: expanded operand tiles ------------------------------------------------------------------------------
// grid.x = (query rows + key rows) / 32 (each rounded up to whole tiles), grid.y = max(B * H, B * Hk) units.  A block
// expands 32 rows (small blocks keep the pre-pass of a small problem short) of one unit into the tile image
// [hi | lo][chunk][tile_rows rows][16 B]; tile_rows is 128 for the forward kernel and 64 for the backward kernel, whose
// steps consume 64 rows of the swept operand.  Expanded columns: d cos/pass columns, then r sin columns.  Phases as the reference
// computes them (PoPE_pytorch/pope.py:56-79): query row i uses freqs[Nk - Nq + i], key row j uses fl(freqs[j] + bias[hk]);
// range-reduced sin / cos (1e-6 absolute) and softplus through ex2 / lg2 (2^-22 relative): far inside the 1e-5 the split
// product needs.
// The 8-feature chunks of the 32 rows are numbered row-major and thread t takes chunks t, t + 256, ...: a warp's loads
// cover whole rows.  Rows past the end of the operand become zeros.
template <typename T, bool SPLIT>
__global__ void __launch_bounds__(256) sim_prepass_kernel(const T* __restrict__ q, Strides sq, const T* __restrict__ k, Strides sk,
                                                          PhaseSrc src,
                                                          const float* __restrict__ bias, int64_t bias_sh, int B, int H, int Hk, int Nq,
                                                          int Nk, int d, int r, int qtiles, int ktiles, int tile_rows,
                                                          uint8_t* __restrict__ qimg, uint8_t* __restrict__ kimg) {
  const int tid = threadIdx.x, u = blockIdx.y;
  pdl_trigger();   // the similarity kernel behind this one may set itself up; it waits for this grid before it reads the images
  const int bpt = tile_rows / 32;   // blocks per tile
  const bool is_q = (int)blockIdx.x < bpt * qtiles;
  const int blk = is_q ? blockIdx.x : blockIdx.x - bpt * qtiles, tile = blk / bpt, quarter = blk % bpt;
  const int heads = is_q ? H : Hk, rows = is_q ? Nq : Nk, tiles = is_q ? qtiles : ktiles;
  const int b = u / heads, h = u % heads;
  if (b >= B) return;   // grid.y covers the larger of the two unit counts
  const int DC = d >> 3, RC = r >> 3, KC = DC + RC;
  const Strides sx = is_q ? sq : sk;
  const T* base = (is_q ? q : k) + (int64_t)b * sx.b + (int64_t)h * sx.h;
  const int pos0 = is_q ? Nk - Nq : 0;
  const float* brow = is_q ? nullptr : bias + (int64_t)h * bias_sh;
  const int csb = tile_rows * 16;
  uint8_t* img = (is_q ? qimg : kimg) + ((int64_t)u * tiles + tile) * ((int64_t)KC * (SPLIT ? 2 : 1) * csb);
  for (int f = tid; f < 32 * DC; f += 256) {
    const int row = quarter * 32 + f / DC, c = f % DC, j = tile * tile_rows + row;
    const bool ok = j < rows;
    uint8_t* dst = img + row * 16;
    float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (ok) Load8<T>::run(base + (int64_t)j * sx.n + c * 8, x);
    if (c < RC) {
      float vc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, vs[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (ok) {
        float fr[8];
        if (src.pos) {
#pragma unroll
          for (int e = 0; e < 8; ++e) fr[e] = src.at(pos0 + j, c * 8 + e);
        } else {
          Load8<float>::run(src.freqs + (int64_t)(pos0 + j) * src.sfn + c * 8, fr);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float sn, cs;
          sincos_reduced(brow ? fr[e] + brow[c * 8 + e] : fr[e], &sn, &cs);
          const float a = softplus_fast(x[e]);
          vc[e] = a * cs, vs[e] = a * sn;
        }
      }
      put_chunk<SPLIT>(dst + c * csb, dst + (KC + c) * csb, vc);
      put_chunk<SPLIT>(dst + (DC + c) * csb, dst + (KC + DC + c) * csb, vs);
    } else {
      put_chunk<SPLIT>(dst + c * csb, dst + (KC + c) * csb, x);
    }
  }
}

// shared-memory plan, the same arithmetic on host and device
struct SimSmem {
  int opq, opk, q_off, k_off, stg_off, misc_off, total;
};
__host__ __device__ inline SimSmem sim_smem_plan(int kd, int r, bool split, int mt, int nkb) {
  SimSmem m;
  const int kc = kd >> 3, parts = split ? 2 : 1;
  m.opq = kc * parts * SIM_CSQ;            // one 128-row Q' tile
  m.opk = kc * parts * SIM_CSK;            // the K' tile
  m.q_off = 0;
  m.k_off = mt * m.opq;
  m.stg_off = (m.k_off + nkb * m.opk + 1023) & ~1023; // swizzled tiles must sit on 1024-byte boundaries
  m.misc_off = m.stg_off + SIM_WORKERS * SIM_STG_WARP; // barriers, TMEM slot
  m.total = m.misc_off + 128 + 1024;                  // + slack to put the base on a 1024-byte boundary at run time
  return m;
}

// mbarrier slots
enum { SB_MMADONE = 0,   // [2] tcgen05.commit: the chains of tile t (slot t & 1) have completed: its K' buffer is free again
       SB_KFULL = 2,     // [2] the K' tile has landed in buffer t % NKB (transaction bytes)
       SB_TFREE = 4,     // [2] 8 worker warps: TMEM buffer b has been drained
       SB_QFULL = 6,     // the Q' tiles of the row block have landed (transaction bytes)
       SB_COUNT = 7 };

// MT row tiles per block, NKB key buffers (2: the copy of tile t + 1 overlaps the chains of tile t)
template <typename T, bool SPLIT, int MT, int NKB>
__global__ void __launch_bounds__(SIM_THREADS, 1) sim_fwd_tc_kernel(TcSimP p, const __grid_constant__ CUtensorMap tmap_out) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int KD = p.d + p.r, KC = KD >> 3, KSTEPS = KD >> 4;
  const SimSmem L = sim_smem_plan(KD, p.r, SPLIT, MT, NKB);
  uint8_t* base = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);
  uint8_t* Qs = base + L.q_off;
  uint8_t* Kb = base + L.k_off;
  uint8_t* Stg = base + L.stg_off;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + L.misc_off);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + SB_COUNT + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr uint32_t TCOLS = MT * SIM_N * 2;     // two buffers of MT accumulator tiles
  if (warp == SIM_MMA_WARP) {
    tmem_alloc(tmem_slot, TCOLS);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&bars[SB_MMADONE], 1), mbar_init(&bars[SB_MMADONE + 1], 1);
    mbar_init(&bars[SB_KFULL], 1), mbar_init(&bars[SB_KFULL + 1], 1);
    mbar_init(&bars[SB_TFREE], SIM_WORKERS), mbar_init(&bars[SB_TFREE + 1], SIM_WORKERS);
    mbar_init(&bars[SB_QFULL], 1);
    mbar_init_fence();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  bool failed = false;

  // this CTA's slice of the flattened (unit, row block, key tile) list; tile t of the slice is list entry g_begin + t
  const int64_t g_begin = p.total_tiles * blockIdx.x / gridDim.x, g_end = p.total_tiles * (blockIdx.x + 1) / gridDim.x;
  const int ntiles = (int)(g_end - g_begin);
  const int opk_bytes = L.opk;
  // a row block starts at the first tile of the slice and wherever the key-tile index wraps to 0
  auto key_tile = [&](int t) { return (int)((g_begin + t) % p.ktiles); };
  auto starts_block = [&](int t) { return t == 0 || key_tile(t) == 0; };

  if (warp == SIM_LOAD_WARP) {
    // =============================== copies: one K' tile per step ==============================
    if (lane == 0) {
      pdl_wait();   // the image pre-pass has completed (this thread is the only reader of its output)
      int t = 0;
      for (; t < ntiles && !failed; ++t) {
        const int64_t g = g_begin + t, rbg = g / p.ktiles;
        const int kt = (int)(g - rbg * p.ktiles), u = (int)(rbg / p.rblocks), b = u / p.H, hk = (u % p.H) % p.Hk;
        if (starts_block(t)) {
          // every chain that read the previous Q' tiles has completed once the chains of tile t - 1 have (commits are
          // in issue order)
          if (t >= 1) failed = !mbar_wait(&bars[SB_MMADONE + ((t - 1) & 1)], ((t - 1) >> 1) & 1, WAIT_LIMIT);
          if (failed) break;
          const int rb = (int)(rbg - (int64_t)u * p.rblocks), qtiles = (p.Nq + SIM_M - 1) / SIM_M;
          const int nq = min(MT, qtiles - rb * MT);
          mbar_expect_tx(&bars[SB_QFULL], nq * L.opq);
          for (int mt = 0; mt < nq; ++mt)
            bulk_load(Qs + mt * L.opq, p.qimg + ((int64_t)u * qtiles + rb * MT + mt) * L.opq, L.opq, &bars[SB_QFULL]);
        }
        // key buffer t % NKB was last read by the chains of tile t - NKB
        if (t >= NKB) failed = !mbar_wait(&bars[SB_MMADONE + ((t - NKB) & 1)], ((t - NKB) >> 1) & 1, WAIT_LIMIT);
        if (failed) break;
        uint64_t* full = &bars[SB_KFULL + (t % NKB)];
        mbar_expect_tx(full, opk_bytes);
        bulk_load(Kb + (t % NKB) * opk_bytes, p.kimg + ((int64_t)(b * p.Hk + hk) * p.ktiles + kt) * opk_bytes, opk_bytes, full);
      }
      if (failed) {   // let the copies in flight land before the CTA may leave (the Q' tiles: whichever phase is pending)
        drain_copies(&bars[SB_KFULL], NKB, t - NKB, t);
        mbar_wait(&bars[SB_QFULL], 0, 1u << 11), mbar_wait(&bars[SB_QFULL], 1, 1u << 11);
        atomicOr(p.status, 1u);
      }
    }
    __syncwarp();
  } else if (warp == SIM_MMA_WARP) {
    // =============================== MMA issue ====================================================
    if (lane == 0) {
      const uint32_t idesc = instr_desc(FMT_BF16, SIM_M, SIM_N, false, false);
      const uint32_t q_addr = smem_u32(Qs), k_addr = smem_u32(Kb);
      int blocks_seen = 0;
      for (int t = 0; t < ntiles && !failed; ++t) {
        if (starts_block(t)) {
          failed = !mbar_wait(&bars[SB_QFULL], blocks_seen & 1, WAIT_LIMIT);
          ++blocks_seen;
        }
        if (!failed) failed = !mbar_wait(&bars[SB_KFULL + (t % NKB)], (t / NKB) & 1, WAIT_LIMIT);
        // TMEM buffer t & 1 was last used by tile t - 2
        if (t >= 2 && !failed) failed = !mbar_wait(&bars[SB_TFREE + (t & 1)], ((t - 2) >> 1) & 1, WAIT_LIMIT);
        if (failed) break;
        fence_after_sync();
        constexpr int chains = SPLIT ? 3 : 1;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint32_t d = tmem + (t & 1) * (MT * SIM_N) + mt * SIM_N;
          uint32_t acc = 0;
#pragma unroll
          for (int ch = 0; ch < chains; ++ch) {
            // chain 0: hi x hi, chain 1: hi x lo, chain 2: lo x hi
            const uint64_t ad = smem_desc(q_addr + mt * L.opq + (ch == 2 ? KC * SIM_CSQ : 0), SIM_CSQ, 128);
            const uint64_t bd = smem_desc(k_addr + (t % NKB) * opk_bytes + (ch == 1 ? KC * SIM_CSK : 0), SIM_CSK, 128);
            uint32_t alo = desc_lo(ad), blo = desc_lo(bd);
#pragma unroll 4
            for (int ks = 0; ks < KSTEPS; ++ks) {
              mma_ss_lh(d, alo, desc_hi(ad), blo, desc_hi(bd), idesc, acc);
              acc = 1;
              alo += (2 * SIM_CSQ) >> 4, blo += (2 * SIM_CSK) >> 4;
            }
          }
        }
        mma_commit(&bars[SB_MMADONE + (t & 1)]);
      }
      if (failed) atomicOr(p.status, 1u);
    }
    __syncwarp();
  } else {
    // =============================== workers ======================================================
    const int row = tid & 127, grp = (tid >> 7) & 1;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    // Every warp drains its own 32 accumulator rows through its own staging tile and its own tensor-map stores: eight
    // independent streams keep the copy engine busy, and their hand-offs are warp-level only.
    uint8_t* stg = Stg + warp * SIM_STG_WARP;
    constexpr int PIECE = 128 / (int)sizeof(T);    // output columns per staged row: 128 bytes
    constexpr int NPIECE = SIM_N / PIECE;
    using T16 = typename std::conditional<sizeof(T) == 4, __nv_bfloat16, T>::type;
    for (int t = 0; t < ntiles; ++t) {
      const int64_t g = g_begin + t, rbg = g / p.ktiles;
      const int kt = (int)(g - rbg * p.ktiles), u = (int)(rbg / p.rblocks), rb = (int)(rbg - (int64_t)u * p.rblocks);
      const int b = u / p.H, h = u % p.H;
      const int i0 = rb * (MT * SIM_M);
      const uint32_t buf = t & 1;
      if (!failed) failed = !mbar_wait(&bars[SB_MMADONE + buf], (t >> 1) & 1, WAIT_LIMIT);
      fence_after_sync();
      const int tile0 = kt * SIM_N;
      // MT = 2: group g drains row tile g, all column pieces; MT = 1: the groups take alternate pieces of the one tile
      const int mt = MT == 2 ? grp : 0;
      const int gi = i0 + mt * SIM_M + row;
      const uint32_t acc = tmem + lane_base + buf * (MT * SIM_N) + mt * SIM_N;
      for (int pc = (MT == 2 ? 0 : grp); pc < NPIECE; pc += (MT == 2 ? 1 : 2)) {
        uint32_t w[32];
        if (sizeof(T) == 4) {
          tmem_ld32(acc + pc * PIECE, w);
          tmem_ld_wait();
        } else {
          uint32_t v0[32], v1[32];
          tmem_ld32(acc + pc * PIECE, v0);
          tmem_ld32(acc + pc * PIECE + 32, v1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            w[i] = pack2<T16>(__uint_as_float(v0[2 * i]), __uint_as_float(v0[2 * i + 1]));
            w[16 + i] = pack2<T16>(__uint_as_float(v1[2 * i]), __uint_as_float(v1[2 * i + 1]));
          }
        }
        const int c0 = tile0 + pc * PIECE;
        if (p.use_tma) {
          // the previous store of this warp must have finished reading the staging tile
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
          // 128-byte swizzle: 16-byte chunk c of row R sits at chunk position c ^ (R % 8)
          uint8_t* dst = stg + lane * 128;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<uint4*>(dst + ((i ^ (lane & 7)) << 4)) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_4d(&tmap_out, stg, c0, i0 + mt * SIM_M + (warp & 3) * 32, h, b);
            tma_store_commit();
          }
        } else if (gi < p.Nq) {
          T* dstg = (T*)p.sim + b * p.ss.b + h * p.ss.h + (int64_t)gi * p.ss.n + c0;
          const T* wv = reinterpret_cast<const T*>(w);
          for (int i = 0; i < PIECE; ++i)
            if (c0 + i < p.Nk) dstg[i] = wv[i];
        }
      }
      // this warp's lanes of TMEM buffer `buf` are in registers / on their way out
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[SB_TFREE + buf]);
    }
    if (lane == 0) tma_store_wait_all<0>();
    if (failed && lane == 0) atomicOr(p.status, 1u);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == SIM_MMA_WARP) tmem_dealloc(tmem, TCOLS);
}

// ---- host side ---------------------------------------------------------------------------------
bool sim_fwd_tc_supported(const PopeSimArgs& a) {
  const PopeShape& s = a.shape;
  if (s.d % 8 != 0 || s.r % 8 != 0 || (s.d + s.r) % 16 != 0) return false;
  if (sim_smem_plan(s.d + s.r, s.r, s.dtype == POPE_F32, 1, 1).total > kMaxDynamicSmem) return false;
  if (s.r > 0 && (a.embed.sf.b != 0 || a.embed.sf.h != 0)) return false;
  if (s.r > 256) return false;
  const int esz = s.dtype == POPE_F32 ? 4 : 2;
  const int align_elems = 16 / esz;
  auto ok = [&](const void* ptr, const PopeStride3& st) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && st.b % align_elems == 0 && st.h % align_elems == 0 &&
           st.n % align_elems == 0;
  };
  if (!ok(a.q, a.sq) || !ok(a.k, a.sk)) return false;
  if (s.r > 0 && ((reinterpret_cast<uintptr_t>(a.embed.freqs) & 15) != 0 || a.embed.sf.n % 4 != 0)) return false;
  return true;
}

// workspace: [Q' tile images of all (batch, head) units][K' tile images of all (batch, key head) units]
static size_t sim_tile_bytes(const PopeShape& s) { return (size_t)((s.d + s.r) / 8) * (s.dtype == POPE_F32 ? 2 : 1) * SIM_CSK; }
static size_t sim_qimg_bytes(const PopeShape& s) {
  return ((size_t)s.B * s.H * ((s.Nq + SIM_M - 1) / SIM_M) * sim_tile_bytes(s) + 255) & ~(size_t)255;
}
static size_t sim_kimg_bytes(const PopeShape& s) { return (size_t)s.B * s.Hk * ((s.Nk + SIM_N - 1) / SIM_N) * sim_tile_bytes(s); }
size_t sim_fwd_tc_workspace(const PopeSimArgs& a) { return sim_qimg_bytes(a.shape) + sim_kimg_bytes(a.shape); }
// the same images serve the backward (tc_sim_bwd.cu): total bytes, and the offset of the K' images
size_t sim_fwd_tc_image_bytes(const PopeShape& s, size_t* q_bytes) {
  if (q_bytes) *q_bytes = sim_qimg_bytes(s);
  return sim_qimg_bytes(s) + sim_kimg_bytes(s);
}

cudaError_t sim_launch_prepass(const PopeShape& s, const PopeEmbed& e, const void* q, const PopeStride3& sq, const void* k,
                               const PopeStride3& sk, uint8_t* qimg, uint8_t* kimg, int tile_rows, cudaStream_t st) {
  const int qtiles = (s.Nq + tile_rows - 1) / tile_rows, ktiles = (s.Nk + tile_rows - 1) / tile_rows;
  const dim3 grid((tile_rows / 32) * (qtiles + ktiles), s.B * s.H);
  switch (s.dtype) {
    case POPE_F32:
      sim_prepass_kernel<float, true><<<grid, 256, 0, st>>>(static_cast<const float*>(q), Strides(sq), static_cast<const float*>(k),
                                                            Strides(sk), phase_src(e), e.bias, e.bias_stride_h, s.B, s.H, s.Hk,
                                                            s.Nq, s.Nk, s.d, s.r, qtiles, ktiles, tile_rows, qimg, kimg);
      break;
    case POPE_BF16:
      sim_prepass_kernel<__nv_bfloat16, false><<<grid, 256, 0, st>>>(
          static_cast<const __nv_bfloat16*>(q), Strides(sq), static_cast<const __nv_bfloat16*>(k), Strides(sk), phase_src(e), e.bias,
          e.bias_stride_h, s.B, s.H, s.Hk, s.Nq, s.Nk, s.d, s.r, qtiles, ktiles, tile_rows, qimg, kimg);
      break;
    default:
      sim_prepass_kernel<__half, false><<<grid, 256, 0, st>>>(static_cast<const __half*>(q), Strides(sq), static_cast<const __half*>(k),
                                                              Strides(sk), phase_src(e), e.bias, e.bias_stride_h, s.B, s.H, s.Hk,
                                                              s.Nq, s.Nk, s.d, s.r, qtiles, ktiles, tile_rows, qimg, kimg);
  }
  return cudaGetLastError();
}

template <typename T, bool SPLIT, int MT, int NKB>
static cudaError_t launch_sim_tc(const PopeSimArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  TcSimP p = {};
  p.H = s.H, p.Hk = s.Hk, p.Nq = s.Nq, p.Nk = s.Nk, p.d = s.d, p.r = s.r;
  p.sim = a.sim, p.ss = a.ss;
  uint8_t* qimg = static_cast<uint8_t*>(a.workspace);
  uint8_t* kimg = qimg + sim_qimg_bytes(s);
  p.qimg = qimg, p.kimg = kimg;
  p.status = tc_status_ptr();
  if (!p.status) return cudaErrorInvalidSymbol;
  const int qtiles = (s.Nq + SIM_M - 1) / SIM_M;
  p.ktiles = (s.Nk + SIM_N - 1) / SIM_N;
  p.rblocks = (qtiles + MT - 1) / MT;
  p.total_tiles = (int64_t)s.B * s.H * p.rblocks * p.ktiles;
  // (all host-side preparation first, then the two launches back to back: what the host does between them is time
  // the GPU spends idle on small problems)
  CUtensorMap tmap;
  memset(&tmap, 0, sizeof(tmap));
  p.use_tma = make_store_tmap(&tmap, a.sim, s.dtype, s.Nk, s.Nq, s.H, s.B, a.ss.n, a.ss.h, a.ss.b, 32) ? 1 : 0;
  const SimSmem L = sim_smem_plan(s.d + s.r, s.r, SPLIT, MT, NKB);
  // keep one CTA per SM: TMEM columns are allocated per CTA
  const size_t smem = L.total < 120 * 1024 ? 120 * 1024 : L.total;
  cudaError_t e;
  if ((e = ensure_max_smem<sim_fwd_tc_kernel<T, SPLIT, MT, NKB>>()) != cudaSuccess) return e;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0, n = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    sms = n;
  }
  const unsigned grid = (unsigned)std::min<int64_t>(sms, p.total_tiles);
  if ((e = sim_launch_prepass(s, a.embed, a.q, a.sq, a.k, a.sk, qimg, kimg, SIM_M, st)) != cudaSuccess) return e;
  // (launched as a programmatic dependent of the pre-pass: 25.6 -> 22.4 us at (1, 8, 1024, 64))
  return launch_dependent(sim_fwd_tc_kernel<T, SPLIT, MT, NKB>, dim3(grid), dim3(SIM_THREADS), smem, st, p, tmap);
}

template <typename T, bool SPLIT>
static cudaError_t launch_sim_mt(const PopeSimArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  auto fits = [&](int mt, int nkb) { return sim_smem_plan(s.d + s.r, s.r, SPLIT, mt, nkb).total <= kMaxDynamicSmem; };
  // Two key buffers first (the copy of the next tile overlaps the MMA chains), then two row tiles per block (half the
  // K' traffic) when the problem is large enough that every SM still gets whole blocks.
  const int64_t blocks2 = (int64_t)s.B * s.H * ((s.Nq + 2 * SIM_M - 1) / (2 * SIM_M));
  const bool want2 = s.Nq > SIM_M && blocks2 * ((s.Nk + SIM_N - 1) / SIM_N) >= 8 * 148;
  if (want2 && fits(2, 2)) return launch_sim_tc<T, SPLIT, 2, 2>(a, st);
  if (fits(1, 2)) return launch_sim_tc<T, SPLIT, 1, 2>(a, st);
  if (want2 && fits(2, 1)) return launch_sim_tc<T, SPLIT, 2, 1>(a, st);
  return launch_sim_tc<T, SPLIT, 1, 1>(a, st);
}

cudaError_t sim_fwd_tc(const PopeSimArgs& a, cudaStream_t st) {
  switch (a.shape.dtype) {
    case POPE_F32: return launch_sim_mt<float, true>(a, st);
    case POPE_BF16: return launch_sim_mt<__nv_bfloat16, false>(a, st);
    default: return launch_sim_mt<__half, false>(a, st);
  }
}

}  // namespace pope
