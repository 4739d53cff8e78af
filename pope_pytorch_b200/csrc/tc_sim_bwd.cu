// Backward of the fused PoPE similarity on the Blackwell tensor cores (tcgen05 + TMEM), sm_100a only, fp32 inputs.
//
//   sim = Q' K'^T   =>   dQ' = G K',   dK' = G^T Q'   (G = d sim, fp32, Nq x Nk per (batch, head))
// followed by the chain rule through the transform (PoPE_pytorch/triton_pope.py:129-151, 174-194, 246-256):
//   dx = (dXc cos + dXs sin) sigmoid(x),  dphase = a (dXs cos - dXc sin)  -> dfreqs, and dbias on the key side.
//
// The work is one read of G per side (bytes = 4 Nq Nk per unit and side), so the kernel is built around that stream.
// ONE launch runs both sides: a query-side CTA keeps 128 query rows and their 128 x (d + r) accumulator resident and
// sweeps the keys 64 at a time; a key-side CTA keeps 128 key rows resident and sweeps the query rows of all grouped
// query heads.  The CTAs of a head run in the same wave and sweep in opposite directions from their diagonal block, so
// the second read of every block of G is served by L2 (DRAM traffic 1.2 x G instead of 2 x).  Per step
//   loader warps  : two, one thread of each streaming on its own: the 32 KB tile of G by tensor-map copies (boxes of 32
//                   fp32 columns, 128-byte swizzled; rows and columns past the end arrive as zeros), and the matching 64-row
//                   tile of the OTHER operand's expanded image (hi | lo, built by the pre-pass in the forward kernel's
//                   file with 64-row tiles) by one bulk copy
//   8 worker warps: a thread per row pulls its 32 values out of the staging tile, splits each into two bf16 numbers
//                   G = hi + lo and writes them as 16-byte chunks of 8 keys; that one layout serves both sides -- as the
//                   K-major A operand of G K' and, re-described as MN-major, as the A operand of G^T Q'
//   issuing warps : two, taking the even and the odd steps: three MMA chains per step, hi*hi' + hi*lo' + lo*hi' (fp32
//                   accuracy from bf16 products, as in the forward), accumulating in TMEM over the whole sweep
// and the epilogue applies the chain rule with accurate sincosf / softplus on the rows it owns.
#include <algorithm>
#include <cstring>

#include "kernels.h"
#include "tc_common.cuh"

namespace pope {

constexpr int SBW_THREADS = 384;     // 8 worker warps, two MMA-issuing warps (even / odd steps), two loader warps
constexpr int SBW_MMA_WARP = 8, SBW_LOAD_WARP = 9, SBW_MMA2_WARP = 10, SBW_IMG_WARP = 11;
constexpr int SBW_STG = 32 * 1024;   // one staged G tile (fp32) and one converted G tile (hi | lo bf16)
constexpr int SBW_GST = 3;           // staging buffers of G: two tiles in flight while one is converted
constexpr int SBW_CS_HALF = 64 * 16; // chunk stride of a 64-row operand image tile

struct TcSimBwdP {
  int H, Hk, Nq, Nk, d, r;
  int qtiles, ktiles;                  // 64-row image tiles per unit
  const void *q, *k;
  Strides sq, sk;
  void *dq, *dk;
  Strides sdq, sdk;
  const float* freqs;
  Strides sf;
  const float* bias;
  int64_t bias_sh;
  float* dfreqs;
  Strides sdf;
  float* dbias;
  int64_t dbias_sh;
  const uint8_t *qimg, *kimg;          // expanded tiles [unit][tile][hi | lo][chunk][64 rows][16 B]
  unsigned int* status;
};

enum { WB_GFULL = 0,     // [3] the G tile of step s has landed in staging buffer s % 3 (transaction bytes)
       WB_GFREE = 3,     // [3] 8 worker warps: staging buffer s % 3 has been read
       WB_CONV = 6,      // [2] 8 worker warps: the converted tile of step s is in buffer s & 1
       WB_IFULL = 8,     // [2] the operand tile of step s has landed in buffer s & 1 (transaction bytes)
       WB_DONE = 10,     // [2] tcgen05.commit: the chains of step s have completed: both buffers s & 1 are free
       WB_HEAD = 12,     // the first instruction of step 0 (the one that overwrites the accumulator) has been issued
       WB_COUNT = 13 };

// One side of the backward for one CTA: resident block `blk` (128 rows) of unit `u` (batch x query heads on the query
// side, batch x key heads on the key side).
template <typename T, bool KEY_SIDE>
__device__ __forceinline__ void sim_bwd_side(const TcSimBwdP& p, const CUtensorMap* tmap_g, int blk, int u) {
  static_assert(sizeof(T) == 4, "the tensor-core similarity backward serves fp32");
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int KD = p.d + p.r, KC = KD >> 3;
  const int img_bytes = 2 * KC * SBW_CS_HALF;           // one (hi | lo) half tile of 64 rows
  uint8_t* Gstg = smem;                                  // 3 x 32 KB, 128-byte swizzled boxes
  uint8_t* Gbf = smem + SBW_GST * SBW_STG;               // 2 x [hi | lo][chunk of 8 keys][rows][16 B]
  uint8_t* Img = smem + (SBW_GST + 2) * SBW_STG;         // 2 x [hi | lo][chunk of 8 features][64 rows][16 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(Img + 2 * img_bytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + WB_COUNT + 1);

  constexpr int GROWS = KEY_SIDE ? 64 : 128;             // rows (query rows) of a G step tile
  constexpr int GBOX = KEY_SIDE ? 4 : 2;                 // boxes of 32 key columns per step tile
  constexpr int GCS = GROWS * 16;                        // chunk stride of the converted tile
  constexpr int GPART = GBOX * 4 * GCS;                  // bytes of its hi part (16 KB)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int heads_out = KEY_SIDE ? p.Hk : p.H;
  const int b = u / heads_out, ho = u % heads_out, hk = KEY_SIDE ? ho : ho % p.Hk;
  const int groups = KEY_SIDE ? p.H / p.Hk : 1;
  const int blk0 = blk * 128;                            // first resident row (query row or key row)
  const int inner = KEY_SIDE ? p.Nq : p.Nk;              // swept length per head
  const int steps_per_head = (inner + 63) / 64;
  const int S = steps_per_head * groups;

  if (warp == SBW_MMA_WARP) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    for (int i = 0; i < SBW_GST; ++i) mbar_init(&bars[WB_GFULL + i], 1), mbar_init(&bars[WB_GFREE + i], 8);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[WB_CONV + i], 8), mbar_init(&bars[WB_IFULL + i], 1), mbar_init(&bars[WB_DONE + i], 1);
    }
    mbar_init(&bars[WB_HEAD], 1);
    mbar_init_fence();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  bool failed = false;

  if (warp == SBW_LOAD_WARP || warp == SBW_IMG_WARP) {
    // =============================== copies =====================================================
    // Swept rows m0 .. m0 + 63 of step s.  The sweep starts at the CTA's own diagonal block and the two sides walk in
    // opposite directions: query block i reads key step (2 i + t) and key block j reads query step (2 j + 1 - t) at time
    // t, so the two CTAs that share a 128 x 128 block of G read it within the same two steps, and whichever comes
    // second finds it in L2 (both sides of a head are in flight together: see the launch).
    auto swept = [&](int s, int& hq) {
      const int g = s / steps_per_head, t = s - g * steps_per_head;
      int st = KEY_SIDE ? (2 * blk + 1 - t) % steps_per_head : (2 * blk + t) % steps_per_head;
      if (st < 0) st += steps_per_head;
      hq = KEY_SIDE ? g * p.Hk + hk : ho;   // query head of this G tile
      return st * 64;
    };
    // Two threads stream on their own: the G tiles (three staging buffers, freed as soon as the workers have read them)
    // and the operand image tiles (two buffers, freed by the MMAs two steps later); one thread doing both would hold
    // back the next G copy while it waits for an image buffer.  They sit in DIFFERENT warps: as two lanes of one warp
    // the one parked in its barrier wait kept the other from running (its copy went out ~900 clocks after the barrier
    // it was waiting for had completed).
    if (warp == SBW_LOAD_WARP && lane == 0) {
      int s = 0;
      for (; s < S; ++s) {
        int hq;
        const int m0 = swept(s, hq), gst = s % SBW_GST;
        if (s >= SBW_GST) failed = !mbar_wait(&bars[WB_GFREE + gst], ((s - SBW_GST) / SBW_GST) & 1, WAIT_LIMIT);
        if (failed) break;
        mbar_expect_tx(&bars[WB_GFULL + gst], SBW_STG);
        const int col0 = KEY_SIDE ? blk0 : m0, row0 = KEY_SIDE ? m0 : blk0;
#pragma unroll
        for (int bx = 0; bx < GBOX; ++bx)
          tma_load_4d(Gstg + gst * SBW_STG + bx * (GROWS * 128), tmap_g, &bars[WB_GFULL + gst], col0 + bx * 32, row0, hq, b);
      }
      // a wait gave up: let the copies in flight land before the CTA may leave
      if (failed) drain_copies(&bars[WB_GFULL], SBW_GST, s - SBW_GST, s);
    } else if (warp == SBW_IMG_WARP && lane == 0) {
      pdl_wait();   // the image pre-pass has completed (the G copies of the other loader do not depend on it)
      int s = 0;
      for (; s < S; ++s) {
        int hq;
        const int m0 = swept(s, hq), buf = s & 1;
        if (s >= 2) failed = !mbar_wait(&bars[WB_DONE + buf], ((s - 2) >> 1) & 1, WAIT_LIMIT);
        if (failed) break;
        const uint8_t* tile = KEY_SIDE ? p.qimg + ((int64_t)(b * p.H + hq) * p.qtiles + m0 / 64) * (int64_t)img_bytes
                                       : p.kimg + ((int64_t)(b * p.Hk + hk) * p.ktiles + m0 / 64) * (int64_t)img_bytes;
        mbar_expect_tx(&bars[WB_IFULL + buf], img_bytes);
        bulk_load(Img + buf * img_bytes, tile, img_bytes, &bars[WB_IFULL + buf]);
      }
      if (failed) drain_copies(&bars[WB_IFULL], 2, s - 2, s);
    }
    failed = __any_sync(0xffffffffu, failed);
    if (failed && lane == 0) atomicOr(p.status, 1u);
  } else if (warp == SBW_MMA_WARP || warp == SBW_MMA2_WARP) {
    // =============================== MMA issue ====================================================
    // Two issuing threads take the even and the odd steps.  Around the 12 instructions of a step (about 630 clocks of
    // issue) one thread spends as long again on its waits, fences and commits, and it alone set the pace of the loop;
    // alternating, each has two steps' time for one step's work.  Every instruction accumulates into the same columns
    // except the first of step 0, so the odd thread starts once that one has been issued.
    if (lane == 0) {
      const int first = warp == SBW_MMA_WARP ? 0 : 1;
      if (first == 1 && S > 1) failed = !mbar_wait(&bars[WB_HEAD], 0, WAIT_LIMIT);
      // query side: A = G (K-major: 128 query rows x 16 keys per step); key side: A = G^T (MN-major: 128 keys x 16 query rows)
      const uint32_t idesc = instr_desc(FMT_BF16, 128, KD, KEY_SIDE, true);
      const uint32_t g_addr = smem_u32(Gbf), i_addr = smem_u32(Img);
      for (int s = first; s < S && !failed; s += 2) {
        const int buf = s & 1;
        failed = !mbar_wait(&bars[WB_CONV + buf], (s >> 1) & 1, WAIT_LIMIT);
        if (!failed) failed = !mbar_wait(&bars[WB_IFULL + buf], (s >> 1) & 1, WAIT_LIMIT);
        if (failed) break;
        fence_after_sync();
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) {
          // chain 0: hi x hi, chain 1: hi x lo, chain 2: lo x hi
          const uint32_t ga = g_addr + buf * SBW_STG + (ch == 2 ? GPART : 0);
          const uint32_t ia = i_addr + buf * img_bytes + (ch == 1 ? KC * SBW_CS_HALF : 0);
          const uint64_t ad = KEY_SIDE ? smem_desc(ga, 128, GCS) : smem_desc(ga, GCS, 128);
          const uint64_t bd = smem_desc(ia, 128, SBW_CS_HALF);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {   // 16 swept rows per instruction
            const uint32_t astep = KEY_SIDE ? ks * ((2 * 128) >> 4) : ks * ((2 * GCS) >> 4);
            mma_ss_lh(tmem, desc_lo(ad) + astep, desc_hi(ad), desc_lo(bd) + ks * ((2 * 128) >> 4), desc_hi(bd), idesc,
                      (s > 0 || ch > 0 || ks > 0) ? 1u : 0u);
            if (s == 0 && ch == 0 && ks == 0) mbar_arrive(&bars[WB_HEAD]);
          }
        }
        mma_commit(&bars[WB_DONE + buf]);
      }
      if (failed) atomicOr(p.status, 1u);
    }
    __syncwarp();
  } else {
    // =============================== workers: split G, then the chain rule ========================
    const int grow = tid % GROWS, gbox = tid / GROWS;      // row of the G step tile, box of 32 key columns
    for (int s = 0; s < S; ++s) {
      const int buf = s & 1, gst = s % SBW_GST;
      if (!failed) failed = !mbar_wait(&bars[WB_GFULL + gst], (s / SBW_GST) & 1, WAIT_LIMIT);
      // the row's 128 bytes of its box; 16-byte chunk c sits at chunk position c ^ (row % 8)
      const uint8_t* src = Gstg + gst * SBW_STG + gbox * (GROWS * 128) + grow * 128;
      uint4 v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = *reinterpret_cast<const uint4*>(src + ((i ^ (grow & 7)) << 4));
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[WB_GFREE + gst]);
      // the converted buffer was last read by the chains of step s - 2
      if (s >= 2 && !failed) failed = !mbar_wait(&bars[WB_DONE + buf], ((s - 2) >> 1) & 1, WAIT_LIMIT);
      uint8_t* dst = Gbf + buf * SBW_STG + (gbox * 4) * GCS + grow * 16;
#pragma unroll
      for (int c = 0; c < 4; ++c) {   // 8 keys per chunk
        const float x[8] = {__uint_as_float(v[2 * c].x),     __uint_as_float(v[2 * c].y),     __uint_as_float(v[2 * c].z),
                            __uint_as_float(v[2 * c].w),     __uint_as_float(v[2 * c + 1].x), __uint_as_float(v[2 * c + 1].y),
                            __uint_as_float(v[2 * c + 1].z), __uint_as_float(v[2 * c + 1].w)};
        uint32_t h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const __nv_bfloat162 hh = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
          h[e] = *reinterpret_cast<const uint32_t*>(&hh);
          const float2 back = unpack2<__nv_bfloat16>(h[e]);
          const __nv_bfloat162 ll = __floats2bfloat162_rn(x[2 * e] - back.x, x[2 * e + 1] - back.y);
          l[e] = *reinterpret_cast<const uint32_t*>(&ll);
        }
        *reinterpret_cast<uint4*>(dst + c * GCS) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(dst + c * GCS + GPART) = make_uint4(l[0], l[1], l[2], l[3]);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[WB_CONV + buf]);
    }
    // ---- epilogue -----------------------------------------------------------------------------------
    // TMEM hands every thread one ROW of the accumulator, but x, the phase table and the outputs are row-major in
    // global memory: the accumulator goes through the (now dead) staging buffers first, and the chain rule runs with
    // consecutive threads on consecutive 8-feature groups of a row, so that every global access is contiguous.
    if (S > 0 && !failed) failed = !mbar_wait(&bars[WB_DONE + ((S - 1) & 1)], ((S - 1) >> 1) & 1, WAIT_LIMIT);
    if (S > 1 && !failed) failed = !mbar_wait(&bars[WB_DONE + ((S - 2) & 1)], ((S - 2) >> 1) & 1, WAIT_LIMIT);   // the other issuing thread's last step
    fence_after_sync();
    const int ASTR = KD * 4 + 16;                       // bytes of a staged fp32 row (padded: conflict-free 16-byte stores)
    uint8_t* accs = Gstg;                               // 128 x ASTR <= 96 KB for KD <= 188; larger KD spill into Gbf (dead too)
    float* dbias_s = reinterpret_cast<float*>(Img);     // [r] column sums of the key-phase gradient of this CTA
    {
      const int row = tid & 127, grp = tid >> 7;
      const uint32_t acc = tmem + ((uint32_t)((warp & 3) * 32) << 16);
      for (int cg = grp; cg * 16 < KD; cg += 2) {
        uint32_t w[16];
        if (S > 0) {
          tmem_ld16(acc + cg * 16, w);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) w[e] = 0u;
        }
        uint4* dst = reinterpret_cast<uint4*>(accs + row * ASTR + cg * 64);
#pragma unroll
        for (int e = 0; e < 4; ++e) dst[e] = make_uint4(w[4 * e], w[4 * e + 1], w[4 * e + 2], w[4 * e + 3]);
      }
      for (int c = tid; c < p.r; c += 256) dbias_s[c] = 0.f;
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    {
      const int R = KEY_SIDE ? p.Nk : p.Nq, DG = p.d >> 3;
      const Strides sx = KEY_SIDE ? p.sk : p.sq, sdx = KEY_SIDE ? p.sdk : p.sdq;
      const T* xbase = static_cast<const T*>(KEY_SIDE ? p.k : p.q) + b * sx.b + ho * sx.h;
      T* dbase = static_cast<T*>(KEY_SIDE ? p.dk : p.dq) + b * sdx.b + ho * sdx.h;
      const float* brow = (KEY_SIDE && p.r > 0) ? p.bias + hk * p.bias_sh : nullptr;
      for (int idx = tid; idx < 128 * DG; idx += 256) {   // 128 * DG is a multiple of 256: every thread makes the same trips
        const int row = idx / DG, g8 = idx - row * DG, c0 = g8 * 8, gr = blk0 + row;
        const bool live = gr < R;
        const bool rot = c0 < p.r;   // r is a multiple of 16: an 8-wide group is rotated as a whole
        const float* arow = reinterpret_cast<const float*>(accs + row * ASTR);
        float gc[8], x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, dx[8], dph[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        *reinterpret_cast<float4*>(gc) = *reinterpret_cast<const float4*>(arow + c0);
        *reinterpret_cast<float4*>(gc + 4) = *reinterpret_cast<const float4*>(arow + c0 + 4);
        if (live) {
          *reinterpret_cast<float4*>(x) = *reinterpret_cast<const float4*>(xbase + (int64_t)gr * sx.n + c0);
          *reinterpret_cast<float4*>(x + 4) = *reinterpret_cast<const float4*>(xbase + (int64_t)gr * sx.n + c0 + 4);
        }
        if (live && rot) {
          const int pos = KEY_SIDE ? gr : p.Nk - p.Nq + gr;
          float gs[8], f[8];
          *reinterpret_cast<float4*>(gs) = *reinterpret_cast<const float4*>(arow + p.d + c0);
          *reinterpret_cast<float4*>(gs + 4) = *reinterpret_cast<const float4*>(arow + p.d + c0 + 4);
          const float* frow = p.freqs + b * p.sf.b + ho * p.sf.h + (int64_t)pos * p.sf.n + c0;
          *reinterpret_cast<float4*>(f) = *reinterpret_cast<const float4*>(frow);
          *reinterpret_cast<float4*>(f + 4) = *reinterpret_cast<const float4*>(frow + 4);
          float* dfrow = p.dfreqs ? p.dfreqs + b * p.sdf.b + ho * p.sdf.h + (int64_t)pos * p.sdf.n + c0 : nullptr;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float sn, cs;
            sincos_reduced(brow ? f[e] + brow[c0 + e] : f[e], &sn, &cs);
            // ex2 / lg2 approximations: 2^-22 relative, far inside the gradient tolerance (rtol 1e-3)
            const float t = ex2_approx(-fabsf(x[e]) * LOG2E);                     // exp(-|x|)
            const float a = fmaxf(x[e], 0.f) + lg2_approx(1.f + t) * LN2;         // softplus(x)
            const float sg = (x[e] >= 0.f ? 1.f : t) / (1.f + t);                 // sigmoid(x)
            dx[e] = (gc[e] * cs + gs[e] * sn) * sg;
            dph[e] = a * (gs[e] * cs - gc[e] * sn);
            if (dfrow) atomicAdd(dfrow + e, dph[e]);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) dx[e] = gc[e];
        }
        if (KEY_SIDE && p.dbias) {
          // column sums of the key-phase gradient: when the feature groups divide the warp evenly, the lanes that hold the
          // same group (other rows) are summed by shuffles first and one lane per group touches shared memory
          if (32 % DG == 0) {
#pragma unroll
            for (int e = 0; e < 8; ++e)
              for (int off = DG; off < 32; off <<= 1) dph[e] += __shfl_xor_sync(0xffffffffu, dph[e], off);
            if (lane < DG && rot) {
#pragma unroll
              for (int e = 0; e < 8; ++e) atomicAdd(dbias_s + c0 + e, dph[e]);
            }
          } else if (live && rot) {
#pragma unroll
            for (int e = 0; e < 8; ++e) atomicAdd(dbias_s + c0 + e, dph[e]);
          }
        }
        if (live) {
          float* drow = reinterpret_cast<float*>(dbase + (int64_t)gr * sdx.n + c0);
          *reinterpret_cast<float4*>(drow) = *reinterpret_cast<const float4*>(dx);
          *reinterpret_cast<float4*>(drow + 4) = *reinterpret_cast<const float4*>(dx + 4);
        }
      }
    }
    if (KEY_SIDE && p.dbias) {
      asm volatile("bar.sync 1, 256;" ::: "memory");
      for (int c = tid; c < p.r; c += 256) atomicAdd(p.dbias + hk * p.dbias_sh + c, dbias_s[c]);
    }
    if (failed && lane == 0) atomicOr(p.status, 1u);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == SBW_MMA_WARP) tmem_dealloc(tmem, 256);
}

// Both sides in ONE launch, 1-D grid.  Blocks are numbered so that the CTAs of one (batch, key head) group are
// neighbours -- its query-side CTAs (all grouped query heads) and its key-side CTAs, alternating when both sides have
// the same number of blocks -- because the block scheduler hands out blocks in index order: the two CTAs that read the
// same block of G then run in the same wave, and with the opposite sweep directions above the second read of every
// block comes out of L2 instead of HBM.
template <typename T>
__global__ void __launch_bounds__(SBW_THREADS, 1) sim_bwd_tc_kernel(TcSimBwdP p, const __grid_constant__ CUtensorMap tmap_q,
                                                                     const __grid_constant__ CUtensorMap tmap_k) {
  const int qblocks = (p.Nq + 127) / 128, kblocks = (p.Nk + 127) / 128, groups = p.H / p.Hk;
  const int nq = groups * qblocks, per = nq + kblocks;
  const int grp = blockIdx.x / per, w = blockIdx.x - grp * per;   // grp = batch * Hk + key head
  const int b = grp / p.Hk, hk = grp - b * p.Hk;
  bool key_side;
  int blk, head = 0;
  if (nq == kblocks) {        // one query head per key head, square: q0 k0 q1 k1 ...
    key_side = (w & 1) != 0, blk = w >> 1;
  } else if (w < nq) {
    key_side = false, head = w / qblocks, blk = w - head * qblocks;
  } else {
    key_side = true, blk = w - nq;
  }
  if (key_side) sim_bwd_side<T, true>(p, &tmap_k, blk, b * p.Hk + hk);
  else sim_bwd_side<T, false>(p, &tmap_q, blk, b * p.H + head * p.Hk + hk);
}

// ---- host side ---------------------------------------------------------------------------------
size_t sim_fwd_tc_image_bytes(const PopeShape& s, size_t* q_bytes);   // tc_sim_fwd.cu: sizes of the Q' / K' tile images
cudaError_t sim_launch_prepass(const PopeShape& s, const PopeEmbed& e, const void* q, const PopeStride3& sq, const void* k,
                               const PopeStride3& sk, uint8_t* qimg, uint8_t* kimg, int tile_rows, cudaStream_t st);

bool sim_bwd_tc_supported(const PopeSimBwdArgs& a) {
  const PopeShape& s = a.shape;
  if (s.dtype != POPE_F32) return false;
  if (s.d % 16 != 0 || s.r % 8 != 0 || (s.d + s.r) % 16 != 0 || s.d + s.r > 256) return false;
  if (s.r > 0 && (a.embed.sf.b != 0 || a.embed.sf.h != 0)) return false;
  if (a.dfreqs && (a.sdf.b != 0 || a.sdf.h != 0)) return false;
  auto ok = [&](const void* ptr, const PopeStride3& st) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && st.b % 4 == 0 && st.h % 4 == 0 && st.n % 4 == 0;
  };
  if (!ok(a.q, a.sq) || !ok(a.k, a.sk) || !ok(a.dsim, a.sds)) return false;
  if (s.Nk > 1 && a.sds.n < s.Nk) return false;
  if (s.r > 0 && ((reinterpret_cast<uintptr_t>(a.embed.freqs) & 15) != 0 || a.embed.sf.n % 4 != 0)) return false;
  const size_t smem = (SBW_GST + 2) * (size_t)SBW_STG + 2 * (size_t)(2 * ((s.d + s.r) / 8) * SBW_CS_HALF) + (WB_COUNT + 1) * 8 + 16 + 1024;
  return smem <= (size_t)kMaxDynamicSmem;
}

size_t sim_bwd_tc_workspace(const PopeSimBwdArgs& a) { return sim_fwd_tc_image_bytes(a.shape, nullptr); }

bool make_load_tmap_f32(CUtensorMap* out, const void* base, int cols, int rows, int heads, int batch, int64_t sn, int64_t sh,
                        int64_t sb, int box_rows);

cudaError_t sim_bwd_tc(const PopeSimBwdArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  size_t q_bytes = 0;
  sim_fwd_tc_image_bytes(s, &q_bytes);
  uint8_t* qimg = static_cast<uint8_t*>(a.workspace);
  uint8_t* kimg = qimg + q_bytes;
  cudaError_t e;
  TcSimBwdP p = {};
  p.H = s.H, p.Hk = s.Hk, p.Nq = s.Nq, p.Nk = s.Nk, p.d = s.d, p.r = s.r;
  p.qtiles = (s.Nq + 63) / 64, p.ktiles = (s.Nk + 63) / 64;
  p.q = a.q, p.k = a.k, p.sq = Strides(a.sq), p.sk = Strides(a.sk);
  p.dq = a.dq, p.dk = a.dk, p.sdq = Strides(a.sdq), p.sdk = Strides(a.sdk);
  p.freqs = a.embed.freqs, p.sf = Strides(a.embed.sf), p.bias = a.embed.bias, p.bias_sh = a.embed.bias_stride_h;
  p.dfreqs = s.r > 0 ? a.dfreqs : nullptr, p.sdf = Strides(a.sdf);
  p.dbias = s.r > 0 ? a.dbias : nullptr, p.dbias_sh = a.dbias_stride_h;
  p.qimg = qimg, p.kimg = kimg;
  p.status = tc_status_ptr();
  if (!p.status) return cudaErrorInvalidSymbol;
  CUtensorMap tmap_q, tmap_k;   // the same tensor, boxes of 128 rows (query side) and of 64 rows (key side)
  memset(&tmap_q, 0, sizeof(tmap_q)), memset(&tmap_k, 0, sizeof(tmap_k));
  if (!make_load_tmap_f32(&tmap_q, a.dsim, s.Nk, s.Nq, s.H, s.B, a.sds.n, a.sds.h, a.sds.b, 128) ||
      !make_load_tmap_f32(&tmap_k, a.dsim, s.Nk, s.Nq, s.H, s.B, a.sds.n, a.sds.h, a.sds.b, 64))
    return cudaErrorNotSupported;
  const int KC = (s.d + s.r) / 8;
  size_t smem = (SBW_GST + 2) * (size_t)SBW_STG + 2 * (size_t)(2 * KC * SBW_CS_HALF) + (WB_COUNT + 1) * 8 + 16 + 1024;
  if (smem < 120 * 1024) smem = 120 * 1024;   // one CTA per SM: the TMEM columns are allocated per CTA
  if ((e = ensure_max_smem<sim_bwd_tc_kernel<float>>()) != cudaSuccess) return e;
  const int groups = s.H / s.Hk;
  const unsigned grid = (unsigned)(s.B * s.Hk) * (unsigned)(groups * ((s.Nq + 127) / 128) + (s.Nk + 127) / 128);
  // (the host-side preparation is done: the two launches go out back to back)
  if ((e = sim_launch_prepass(s, a.embed, a.q, a.sq, a.k, a.sk, qimg, kimg, 64, st)) != cudaSuccess) return e;
  return launch_dependent(sim_bwd_tc_kernel<float>, dim3(grid), dim3(SBW_THREADS), smem, st, p, tmap_q, tmap_k);
}

}  // namespace pope
