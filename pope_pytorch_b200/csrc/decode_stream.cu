// Single-token decode of PoPE attention for 16-bit inputs (sm_100a): one query row per (batch, head) unit against a
// long key / value range.  The work is one pass over K and V (HBM-bound: bytes = K + V), so the kernel is built around
// the copy engine:
//
//   loader warp    : streams tiles of keys through a ring of shared-memory stages with cp.async.bulk (K rows, V rows,
//                    and the fp16 cos / sin rows of the position phase table), completion by mbarrier transaction bytes
//   8 worker warps : LPK lanes share one key; every lane transforms 8-feature chunks of the key straight out of shared
//                    memory (softplus magnitude, table phase) and multiplies them with the query's pre-rotated polar
//                    coordinates, a short shuffle reduction gives the score; every warp keeps its own running
//                    (max, sum, output) over its keys, so no block-wide barrier sits in the loop
//
// With q' = (a_q cos fq, a_q sin fq) and k' = (a_k cos(fk + b), a_k sin(fk + b)) the score term of a rotated feature
// is a_q a_k cos(fq - fk - b) = a_k (Qc cos fk + Qs sin fk), Qc = a_q cos(fq - b), Qs = a_q sin(fq - b): the head's bias
// is folded into the query once per CTA and the key side needs only the bias-free table shared by all units.
// Key ranges are split over CTAs; each CTA writes a partial (o, max, sum) that the split combine merges.
//
// Semantics: PoPE_pytorch/triton_pope_flash_attn.py:52-57,73-80 (transform), :89-91 (mask, True = keep), :96-117
// (softmax, empty rows); the query sits at the LAST table row (PoPE_pytorch/pope.py:64).
//
// Paged cache: the same kernel with K and V in fixed-size pages ([page][key head][page_size][d], page_size a multiple of
// the 64-key tile, so a tile never straddles pages): the page indices of the CTA's key range are read into shared
// memory once, the loader takes each tile's address from them, and every sequence has its own length (the query sits
// at its last cached position).  kv_append_kernel writes new rows into the pages.
#include <algorithm>

#include "kernels.h"
#include "tc_common.cuh"

namespace pope {


struct DecodeStreamP {
  int H, Hk, Nk, r, nsplit, split_len, nstages, HDP;
  int k_rows_contiguous, v_rows_contiguous;
  float scale_log2;
  const void *q, *k, *v;
  Strides sq, sk, sv;
  const float *freqs, *bias;
  int64_t sfn, bias_sh;
  const __half *ch, *sh;     // fp16 cos / sin of freqs, [Nk][r]
  const uint8_t* mask;
  int64_t msb, msn;
  float *part_o, *part_ml;
  unsigned int* status;
  // paged cache (page_table != nullptr): k / v point at the page pools, sk.h / sv.h = page_size * d, sk.n = sv.n = d
  const int32_t* page_table;
  const int32_t* seq_lens;
  int page_size, max_pages, num_pages, npg_smem;
  int64_t page_stride;       // elements per page
};

template <typename T> __device__ __forceinline__ void unpack8(const uint4& w, float (&x)[8]) {
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 v = unpack2<T>(u[e]);
    x[2 * e] = v.x, x[2 * e + 1] = v.y;
  }
}

// D: head dim (64, 96, 128); LPK: lanes per key (4 or 8); KPL: keys per lane and tile; NW: worker warps (+ 1 loader
// warp); MINB: CTAs per SM the register allocation must allow.  A tile is NW * KPL * 32 / LPK keys.
template <typename T, int D, int LPK, int KPL, int NW, int MINB>
__global__ void __launch_bounds__(32 * (NW + 1), MINB) attn_decode_stream_kernel(DecodeStreamP p) {
  constexpr int DS_WORKERS = NW;
  constexpr int KPW = 32 / LPK;                 // keys per warp and pass
  constexpr int TILE = DS_WORKERS * KPW * KPL;  // keys per tile
  constexpr int NCH = D / 8;                    // 16-byte chunks per key row
  constexpr int NI = NCH / LPK;                 // chunks per lane
  static_assert(NCH % LPK == 0, "chunks must divide over the lanes of a key");
  constexpr int FPL = 4;                        // output features per lane in the P V step
  constexpr int OLANES = D / FPL;               // lanes that own output features
  constexpr bool SWZ = (LPK == 4) && (D % 64 == 0);   // see the bank note below

  extern __shared__ __align__(128) uint8_t smem[];
  const int r = p.r, RC = r >> 3;
  const int kbytes = TILE * D * 2, tbytes = TILE * r * 2;
  const int stage_bytes = 2 * kbytes + 2 * tbytes;
  float* qcs = reinterpret_cast<float*>(smem + (size_t)p.nstages * stage_bytes);   // [D] Qc / pass-through q, then [D] Qs
  float* red_o = qcs + 2 * D;                                                       // [DS_WORKERS][D]
  float* red_ml = red_o + DS_WORKERS * D;                                           // [DS_WORKERS][2]
  uint64_t* full = reinterpret_cast<uint64_t*>(red_ml + 2 * DS_WORKERS);            // [nstages] tile landed
  uint64_t* empty = full + p.nstages;                                               // [nstages] all workers done with it
  int* pages_s = reinterpret_cast<int*>(empty + p.nstages);                         // [npg_smem] pages of this CTA's key range

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int u = blockIdx.y, b = u / p.H, h = u % p.H, hk = h % p.Hk;
  const T* kbase = (const T*)p.k + b * p.sk.b + hk * p.sk.h;
  const T* vbase = (const T*)p.v + b * p.sv.b + hk * p.sv.h;
  // keys of this sequence (paged cache: its own length, at most the bound the split was planned for)
  const int nk = p.seq_lens ? max(0, min(p.seq_lens[b], p.Nk)) : p.Nk;
  const int kb = blockIdx.x * p.split_len, ke = min(nk, kb + p.split_len);
  const int T_tiles = ke > kb ? (ke - kb + TILE - 1) / TILE : 0;

  if (tid == 0) {
    for (int s = 0; s < p.nstages; ++s) mbar_init(&full[s], 1), mbar_init(&empty[s], DS_WORKERS);
    mbar_init_fence();
  }
  // the query's polar coordinates with the key-side bias folded in (exact transform: one row per CTA)
  if (tid < D) {
    const T* qrow = (const T*)p.q + b * p.sq.b + h * p.sq.h;
    const float x = to_f32<T>(qrow[tid]);
    float c = x, s = 0.f;
    if (tid < r) {
      float sn, cs;
      sincosf(p.freqs[(int64_t)(max(nk, 1) - 1) * p.sfn + tid] - p.bias[hk * p.bias_sh + tid], &sn, &cs);
      const float a = softplus_f(x);
      c = a * cs, s = a * sn;
    }
    qcs[tid] = c, qcs[D + tid] = s;
  }
  if (p.page_table) {
    // page indices of [kb, ke); an index outside the pool is never dereferenced (clamped, status bit 1)
    for (int i = tid; i < p.npg_smem; i += blockDim.x) {
      const int lp = kb / p.page_size + i;
      int pg = 0;
      if ((int64_t)lp * p.page_size < ke) {
        pg = lp < p.max_pages ? p.page_table[(int64_t)b * p.max_pages + lp] : -1;   // a length past the table's reach
        if (pg < 0 || pg >= p.num_pages) pg = 0, atomicOr(p.status, 2u);
      }
      pages_s[i] = pg;
    }
  }
  __syncthreads();
  bool failed = false;

  if (w == DS_WORKERS) {
    // =============================== loader =====================================================
    pdl_trigger();   // the split combine behind this kernel may set itself up
    pdl_wait();      // the fp16 phase table (the kernel before this one) is complete
    for (int jt = 0; jt < T_tiles && !failed; ++jt) {
      const int s = jt % p.nstages, key0 = kb + jt * TILE, n = min(TILE, ke - key0);
      uint8_t* st = smem + (size_t)s * stage_bytes;
      if (jt >= p.nstages) failed = !mbar_wait(&empty[s], ((jt / p.nstages) - 1) & 1, WAIT_LIMIT);
      if (failed) { drain_copies(full, p.nstages, jt - p.nstages, jt); break; }
      if (lane == 0) mbar_expect_tx(&full[s], (uint32_t)(2 * n * D * 2 + 2 * n * r * 2));
      __syncwarp();
      const T *kt = kbase + (int64_t)key0 * p.sk.n, *vt = vbase + (int64_t)key0 * p.sv.n;
      if (p.page_table) {   // the tile lies inside one page
        const int64_t off = (int64_t)pages_s[key0 / p.page_size - kb / p.page_size] * p.page_stride + (int64_t)hk * p.sk.h +
                            (int64_t)(key0 % p.page_size) * p.sk.n;
        kt = (const T*)p.k + off, vt = (const T*)p.v + off;
      }
      if (p.k_rows_contiguous) {
        if (lane == 0) bulk_load(st, kt, n * D * 2, &full[s]);
      } else {
        for (int i = lane; i < n; i += 32) bulk_load(st + i * D * 2, kt + (int64_t)i * p.sk.n, D * 2, &full[s]);
      }
      if (p.v_rows_contiguous) {
        if (lane == 1) bulk_load(st + kbytes, vt, n * D * 2, &full[s]);
      } else {
        for (int i = lane; i < n; i += 32) bulk_load(st + kbytes + i * D * 2, vt + (int64_t)i * p.sv.n, D * 2, &full[s]);
      }
      if (r > 0) {
        if (lane == 2) bulk_load(st + 2 * kbytes, p.ch + (int64_t)key0 * r, n * r * 2, &full[s]);
        if (lane == 3) bulk_load(st + 2 * kbytes + tbytes, p.sh + (int64_t)key0 * r, n * r * 2, &full[s]);
      }
    }
    if (failed && lane == 0) atomicOr(p.status, 1u);
    return;   // nothing below is a block-wide barrier; the workers finish on their own
  }

  // =============================== workers ======================================================
  const int kw = lane / LPK, t = lane % LPK;        // key of the warp's group, lane within the key
  const int krow0 = w * KPW * KPL + kw;             // first row of the tile this lane works on; the others KPW apart
  // Bank note: with 4 lanes per key a quarter-warp covers two keys; when the row stride is a multiple of 128 bytes
  // both rows start on the same bank, so odd rows walk their chunk groups in the swapped order (i ^ 1).
  const int swz = SWZ ? (krow0 & 1) : 0;            // KPW is even for LPK = 4: all rows of a lane share the parity
  // this lane's slice of the query, in the order it visits its chunks
  float qc[NI][8], qs[NI][8];
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int c = t + LPK * (i ^ swz);
#pragma unroll
    for (int e = 0; e < 8; ++e) qc[i][e] = qcs[c * 8 + e], qs[i][e] = qcs[D + c * 8 + e];
  }
  const uint8_t* maskb = p.mask ? p.mask + b * p.msb : nullptr;
  float mrun = -CUDART_INF_F, lrun = 0.f, o[FPL] = {0.f, 0.f, 0.f, 0.f};

  for (int jt = 0; jt < T_tiles; ++jt) {
    const int s = jt % p.nstages, key0 = kb + jt * TILE;
    const uint8_t* st = smem + (size_t)s * stage_bytes;
    if (!failed) failed = !mbar_wait(&full[s], (jt / p.nstages) & 1, WAIT_LIMIT);
    if (failed) break;
    float part[KPL];
    bool valid[KPL];
#pragma unroll
    for (int kq = 0; kq < KPL; ++kq) {
      const int krow = krow0 + kq * KPW, key = key0 + krow;
      valid[kq] = key < ke && (!maskb || maskb[(int64_t)key * p.msn] != 0);
      part[kq] = 0.f;
      if (key < ke) {
        const uint8_t* krow_p = st + krow * (D * 2);
        const uint8_t* crow_p = st + 2 * kbytes + krow * (r * 2);
        const uint8_t* srow_p = crow_p + tbytes;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          const int c = t + LPK * (i ^ swz);
          float x[8];
          unpack8<T>(*reinterpret_cast<const uint4*>(krow_p + c * 16), x);
          if (c < RC) {
            float co[8], si[8];
            unpack8<__half>(*reinterpret_cast<const uint4*>(crow_p + c * 16), co);
            unpack8<__half>(*reinterpret_cast<const uint4*>(srow_p + c * 16), si);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float a = softplus_fast(x[e]);
              part[kq] = fmaf(a, fmaf(qc[i][e], co[e], qs[i][e] * si[e]), part[kq]);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) part[kq] = fmaf(qc[i][e], x[e], part[kq]);
          }
        }
      }
    }
    float sc[KPL], mloc = -CUDART_INF_F;
#pragma unroll
    for (int kq = 0; kq < KPL; ++kq) {
#pragma unroll
      for (int off = 1; off < LPK; off <<= 1) part[kq] += __shfl_xor_sync(0xffffffffu, part[kq], off);
      sc[kq] = valid[kq] ? part[kq] * p.scale_log2 : -CUDART_INF_F;     // log2 units
      mloc = fmaxf(mloc, sc[kq]);
    }
    const float mnew = fmaxf(mrun, warp_max(mloc));
    if (mnew != -CUDART_INF_F) {   // warp-uniform
      const float alpha = ex2_approx(mrun - mnew);    // exp2(-inf) = 0 on the first visible tile
      float pj[KPL], psum = 0.f;
#pragma unroll
      for (int kq = 0; kq < KPL; ++kq) pj[kq] = ex2_approx(sc[kq] - mnew), psum += pj[kq];   // 0 for masked keys
      lrun = lrun * alpha + warp_sum(t == 0 ? psum : 0.f);
      mrun = mnew;
#pragma unroll
      for (int e = 0; e < FPL; ++e) o[e] *= alpha;
      const uint8_t* vt = st + kbytes + (w * KPW * KPL) * (D * 2) + lane * (FPL * 2);
#pragma unroll
      for (int kq = 0; kq < KPL; ++kq)
#pragma unroll
        for (int kk = 0; kk < KPW; ++kk) {
          const float pk = __shfl_sync(0xffffffffu, pj[kq], kk * LPK);
          if (pk != 0.f && lane < OLANES) {   // masked / out-of-range rows may hold stale bytes: never touch them
            const uint2 vv = *reinterpret_cast<const uint2*>(vt + (kq * KPW + kk) * (D * 2));
            const float2 v01 = unpack2<T>(vv.x), v23 = unpack2<T>(vv.y);
            o[0] = fmaf(pk, v01.x, o[0]), o[1] = fmaf(pk, v01.y, o[1]);
            o[2] = fmaf(pk, v23.x, o[2]), o[3] = fmaf(pk, v23.y, o[3]);
          }
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }
  if (failed && lane == 0) atomicOr(p.status, 1u);

  // merge the worker warps of the CTA, then hand the partial to the cross-split combine (natural-log units)
  if (lane < OLANES) {
#pragma unroll
    for (int e = 0; e < FPL; ++e) red_o[w * D + lane * FPL + e] = o[e];
  }
  if (lane == 0) red_ml[2 * w] = mrun, red_ml[2 * w + 1] = lrun;
  asm volatile("bar.sync 1, %0;" ::"n"(32 * DS_WORKERS) : "memory");
  float M = -CUDART_INF_F;
#pragma unroll
  for (int ww = 0; ww < DS_WORKERS; ++ww) M = fmaxf(M, red_ml[2 * ww]);
  const int64_t slot = (int64_t)u * p.nsplit + blockIdx.x;     // one query row per unit
  for (int c = tid; c < p.HDP; c += 32 * DS_WORKERS) {
    float acc = 0.f;
    if (c < D) {
#pragma unroll
      for (int ww = 0; ww < DS_WORKERS; ++ww)
        acc += red_ml[2 * ww] == -CUDART_INF_F ? 0.f : red_o[ww * D + c] * ex2_approx(red_ml[2 * ww] - M);
    }
    p.part_o[slot * p.HDP + c] = acc;
  }
  if (tid == 0) {
    float L = 0.f;
#pragma unroll
    for (int ww = 0; ww < DS_WORKERS; ++ww)
      L += red_ml[2 * ww] == -CUDART_INF_F ? 0.f : red_ml[2 * ww + 1] * ex2_approx(red_ml[2 * ww] - M);
    p.part_ml[slot * 2] = M * LN2, p.part_ml[slot * 2 + 1] = L;
  }
}

// ---- host side -----------------------------------------------------------------------------------
bool decode_stream_supported(const PopeAttnArgs& a) {
  const PopeShape& s = a.shape;
  if (s.Nq != 1 || a.causal || s.Nk < 1024) return false;
  if (s.dtype != POPE_BF16 && s.dtype != POPE_F16) return false;
  if (s.d != 64 && s.d != 96 && s.d != 128) return false;
  if (s.r % 8 != 0) return false;
  if (s.r > 0 && (a.embed.sf.b != 0 || a.embed.sf.h != 0)) return false;
  auto ok = [&](const void* ptr, const PopeStride3& st) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && st.b % 8 == 0 && st.h % 8 == 0 && st.n % 8 == 0;
  };
  if (!ok(a.k, a.sk) || !ok(a.v, a.sv)) return false;
  if ((s.Nk > 1 && (a.sk.n < s.d || a.sv.n < s.d))) return false;
  return true;
}

static int decode_tile(int) { return 64; }   // keys per tile of every instantiation below (8 warps x 32 / LPK x KPL)   // keys per tile: 4 lanes per key at d = 96, else 8

// Split the keys so that the grid fills whole waves of one CTA pair per SM; every split keeps at least 8 tiles.
static void decode_stream_plan(const PopeShape& s, int& nsplit, int& split_len) {
  const int tile = decode_tile(s.d);
  const int64_t units = (int64_t)s.B * s.H;
  const int slots = 2 * 148;
  const int max_split = std::max(1, s.Nk / (8 * tile));
  int best = 1;
  double best_eff = 0.0;
  for (int n = 1; n <= max_split && n <= 64; ++n) {
    const int64_t ctas = units * n;
    const double eff = (double)ctas / (double)(((ctas + slots - 1) / slots) * slots);
    if (eff > best_eff + 1e-9) best = n, best_eff = eff;
    if (eff >= 0.95 && ctas >= 2 * slots) break;
  }
  nsplit = best;
  split_len = ((s.Nk + nsplit - 1) / nsplit + tile - 1) / tile * tile;
  nsplit = (s.Nk + split_len - 1) / split_len;
}

static size_t decode_partials_bytes(const PopeShape& s, int nsplit) {
  const int HDP = simt_dch(s.d) * 32;
  return ((size_t)s.B * s.H * nsplit * (HDP + 2) * sizeof(float) + 255) / 256 * 256;
}

size_t decode_stream_workspace(const PopeAttnArgs& a) {
  int ns, sl;
  decode_stream_plan(a.shape, ns, sl);
  return decode_partials_bytes(a.shape, ns) + (((size_t)a.shape.Nk * a.shape.r * 4 + 255) & ~(size_t)255);
}

cudaError_t launch_split_combine(const PopeAttnArgs& a, int nsplit, float* part_o, float* part_ml, cudaStream_t st);

template <typename T, int D, int LPK, int KPL, int NW, int MINB>
static cudaError_t launch_decode_stream(const PopeAttnArgs& a, cudaStream_t st, const PopePagedKV* kv) {
  constexpr int DS_WORKERS = NW, DS_THREADS = 32 * (NW + 1);
  const PopeShape& s = a.shape;
  DecodeStreamP p = {};
  p.H = s.H, p.Hk = s.Hk, p.Nk = s.Nk, p.r = s.r;
  decode_stream_plan(s, p.nsplit, p.split_len);
  p.HDP = simt_dch(s.d) * 32;
  p.scale_log2 = a.softmax_scale * LOG2E;
  p.q = a.q, p.k = a.k, p.v = a.v, p.sq = a.sq, p.sk = a.sk, p.sv = a.sv;
  p.k_rows_contiguous = a.sk.n == s.d, p.v_rows_contiguous = a.sv.n == s.d;
  p.freqs = a.embed.freqs, p.bias = a.embed.bias, p.sfn = a.embed.sf.n, p.bias_sh = a.embed.bias_stride_h;
  p.mask = a.mask, p.msb = a.mask_stride_b, p.msn = a.mask_stride_n;
  if (kv) {
    p.page_table = kv->page_table, p.seq_lens = kv->seq_lens;
    p.page_size = kv->page_size, p.max_pages = kv->max_pages_per_seq, p.num_pages = kv->num_pages;
    p.page_stride = (int64_t)s.Hk * kv->page_size * s.d;
    p.npg_smem = p.split_len / kv->page_size + 2;
  }
  const size_t slots = (size_t)s.B * s.H * p.nsplit;
  p.part_o = static_cast<float*>(a.workspace);
  p.part_ml = p.part_o + slots * p.HDP;
  __half* ch = reinterpret_cast<__half*>(static_cast<uint8_t*>(a.workspace) + decode_partials_bytes(s, p.nsplit));
  __half* sh = ch + (size_t)s.Nk * s.r;
  p.ch = ch, p.sh = sh;
  p.status = tc_status_ptr();
  if (!p.status) return cudaErrorInvalidSymbol;
  cudaError_t e;
  if (s.r > 0 && (e = launch_trig_tables(a.embed, s.Nk, s.r, nullptr, nullptr, ch, sh, st)) != cudaSuccess) return e;
  constexpr int TILE = DS_WORKERS * KPL * 32 / LPK;
  const size_t stage = (size_t)TILE * (2 * D * 2 + 2 * s.r * 2);
  const size_t fixed = (2 * D + DS_WORKERS * D + 2 * DS_WORKERS) * sizeof(float) + 2 * 8 * 8 + 64 + (size_t)p.npg_smem * sizeof(int);
  // two CTAs per SM: the ring of each takes what half of the shared memory leaves, at most 3 stages
  // Measured on B200 (8 x 32 x 32768 x 128, r = 64): two keys per lane and two resident CTAs per SM reach 4.67 TB/s;
  // a deeper ring in one CTA per SM is slower (2.06 ms against 0.92 ms): the workers, not the copies, need the overlap.
  int nst = (int)((110 * 1024 - fixed) / stage);
  if (nst < 2) nst = (int)((kMaxDynamicSmem - 1024 - fixed) / stage);   // wide rotations (r = d = 128): one CTA per SM
  nst = nst > 3 ? 3 : nst;
  if (nst < 2) return cudaErrorInvalidValue;
  p.nstages = nst;
  const size_t smem = nst * stage + fixed;
  if ((e = ensure_max_smem<attn_decode_stream_kernel<T, D, LPK, KPL, NW, MINB>>()) != cudaSuccess) return e;
  // behind the table kernel the decode kernel starts as its programmatic dependent (its loader waits for the table);
  // without rotated features it is the first launch of the call and an ordinary one
  if (s.r > 0) {
    e = launch_dependent(attn_decode_stream_kernel<T, D, LPK, KPL, NW, MINB>, dim3(p.nsplit, s.B * s.H), dim3(DS_THREADS), smem, st, p);
  } else {
    attn_decode_stream_kernel<T, D, LPK, KPL, NW, MINB><<<dim3(p.nsplit, s.B * s.H), DS_THREADS, smem, st>>>(p);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return e;
  return launch_split_combine(a, p.nsplit, p.part_o, p.part_ml, st);
}

template <typename T>
static cudaError_t decode_stream_d(const PopeAttnArgs& a, cudaStream_t st, const PopePagedKV* kv) {
  switch (a.shape.d) {
    case 64: return launch_decode_stream<T, 64, 8, 2, 8, 1>(a, st, kv);
    case 96: return launch_decode_stream<T, 96, 4, 1, 8, 1>(a, st, kv);
    default: return launch_decode_stream<T, 128, 8, 2, 8, 1>(a, st, kv);
  }
}

cudaError_t decode_stream(const PopeAttnArgs& a, cudaStream_t st) {
  return a.shape.dtype == POPE_BF16 ? decode_stream_d<__nv_bfloat16>(a, st, nullptr) : decode_stream_d<__half>(a, st, nullptr);
}

// ---- paged cache ---------------------------------------------------------------------------------
// The paged call as the contiguous call sees it: K / V = the page pools, head stride inside a page, rows contiguous.
static PopeAttnArgs paged_as_attn(const PopePagedDecodeArgs& g, float* lse) {
  PopeAttnArgs a = {};
  a.struct_bytes = sizeof(PopeAttnArgs);
  a.causal = 0, a.softmax_scale = g.softmax_scale;
  a.shape = g.shape, a.embed = g.embed;
  a.q = g.q, a.sq = g.sq, a.out = g.out, a.so = g.so, a.lse = lse;
  a.k = g.kv.k_pages, a.v = g.kv.v_pages;
  a.sk.b = 0, a.sk.h = (int64_t)g.kv.page_size * g.shape.d, a.sk.n = g.shape.d;
  a.sv = a.sk;
  a.workspace = g.workspace, a.workspace_bytes = g.workspace_bytes;
  return a;
}

static size_t paged_lse_bytes(const PopeShape& s) { return ((size_t)s.B * s.H * sizeof(float) + 255) & ~(size_t)255; }

bool decode_paged_supported(const PopePagedDecodeArgs& g) {
  const PopeShape& s = g.shape;
  if (s.Nq != 1 || (s.dtype != POPE_BF16 && s.dtype != POPE_F16)) return false;
  if (s.d != 64 && s.d != 96 && s.d != 128) return false;
  if (s.r % 8 != 0) return false;
  if (s.r > 0 && (g.embed.sf.b != 0 || g.embed.sf.h != 0)) return false;
  if (g.kv.page_size < 64 || g.kv.page_size % 64 != 0) return false;
  return true;
}

size_t decode_paged_workspace(const PopePagedDecodeArgs& g) {
  return decode_stream_workspace(paged_as_attn(g, nullptr)) + paged_lse_bytes(g.shape);
}

cudaError_t decode_paged(const PopePagedDecodeArgs& g, cudaStream_t st) {
  // the row statistics of the split combine go to the caller's lse or, without one, to the end of the workspace
  float* lse = g.lse;
  if (!lse) lse = reinterpret_cast<float*>(static_cast<uint8_t*>(g.workspace) + decode_stream_workspace(paged_as_attn(g, nullptr)));
  const PopeAttnArgs a = paged_as_attn(g, lse);
  return g.shape.dtype == POPE_BF16 ? decode_stream_d<__nv_bfloat16>(a, st, &g.kv) : decode_stream_d<__half>(a, st, &g.kv);
}

struct KvAppendP {
  int Hk, d, n_new, page_size, max_pages, num_pages;
  int64_t page_stride;
  const void *k, *v;
  Strides sk, sv;
  void *k_pages, *v_pages;
  const int32_t* page_table;
  int32_t* seq_lens;
  unsigned int* status;
};

// One thread per 16 bytes of a new row of k and of v.  A position past the table or a page index outside the pool is
// skipped and reported through status bit 1.
template <typename T>
__global__ void __launch_bounds__(256) kv_append_kernel(KvAppendP p) {
  const int cpr = p.d >> 3;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= p.n_new * cpr) return;
  const int i = idx / cpr, c = idx - i * cpr, hk = blockIdx.y, b = blockIdx.z;
  const int pos = p.seq_lens[b] + i, lp = pos / p.page_size;
  if (pos < 0 || lp >= p.max_pages) { atomicOr(p.status, 2u); return; }
  const int pg = p.page_table[(int64_t)b * p.max_pages + lp];
  if (pg < 0 || pg >= p.num_pages) { atomicOr(p.status, 2u); return; }
  const int64_t dst = (int64_t)pg * p.page_stride + ((int64_t)hk * p.page_size + pos % p.page_size) * p.d + c * 8;
  const T* krow = static_cast<const T*>(p.k) + b * p.sk.b + hk * p.sk.h + (int64_t)i * p.sk.n + c * 8;
  const T* vrow = static_cast<const T*>(p.v) + b * p.sv.b + hk * p.sv.h + (int64_t)i * p.sv.n + c * 8;
  *reinterpret_cast<uint4*>(static_cast<T*>(p.k_pages) + dst) = __ldg(reinterpret_cast<const uint4*>(krow));
  *reinterpret_cast<uint4*>(static_cast<T*>(p.v_pages) + dst) = __ldg(reinterpret_cast<const uint4*>(vrow));
}

__global__ void kv_advance_kernel(int32_t* seq_lens, int B, int n_new) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) seq_lens[b] += n_new;
}

cudaError_t kv_append(const PopeKvAppendArgs& g, cudaStream_t st) {
  KvAppendP p = {};
  p.Hk = g.Hk, p.d = g.d, p.n_new = g.n_new;
  p.page_size = g.kv.page_size, p.max_pages = g.kv.max_pages_per_seq, p.num_pages = g.kv.num_pages;
  p.page_stride = (int64_t)g.Hk * g.kv.page_size * g.d;
  p.k = g.k, p.v = g.v, p.sk = Strides(g.sk), p.sv = Strides(g.sv);
  p.k_pages = g.kv.k_pages, p.v_pages = g.kv.v_pages, p.page_table = g.kv.page_table, p.seq_lens = g.kv.seq_lens;
  p.status = tc_status_ptr();
  if (!p.status) return cudaErrorInvalidSymbol;
  const dim3 grid((unsigned)((g.n_new * (g.d / 8) + 255) / 256), (unsigned)g.Hk, (unsigned)g.B);
  // (both 16-bit types move as raw 16-byte groups)
  kv_append_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (g.advance) {
    kv_advance_kernel<<<(g.B + 255) / 256, 256, 0, st>>>(g.kv.seq_lens, g.B, g.n_new);
    e = cudaGetLastError();
  }
  return e;
}

}  // namespace pope
