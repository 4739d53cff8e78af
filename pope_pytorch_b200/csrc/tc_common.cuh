// Helpers shared by the tensor-core (tcgen05) attention kernels: operand formats, packing,
// fast device math and the per-position (cos, sin) phase table.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include <cuda.h>   // CUtensorMap (types only; the encoder is fetched through the runtime's driver entry point)

#include "common.cuh"
#include "tc05.cuh"

namespace pope {

using namespace tc;

// device address of the sticky status word (bit 0 = a bounded wait gave up) on the current device
unsigned int* tc_status_ptr();

constexpr uint32_t WAIT_LIMIT = 1u << 17;   // parked tries of up to 10 us each
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

template <typename T> struct TcFmt;
template <> struct TcFmt<__nv_bfloat16> { static constexpr uint32_t fmt = FMT_BF16; };
template <> struct TcFmt<__half> { static constexpr uint32_t fmt = FMT_F16; };

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t u);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) {
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// softplus with ONE special-function op: t = 2^(-|x| log2 e), log1p(t) = t * q(t) with a degree-5
// polynomial q (relative error 1.8e-5 on (0, 1]); the operand is rounded to 8 or 11 bits afterwards.
__device__ __forceinline__ float softplus_poly(float x) {
  const float t = ex2_approx(-fabsf(x) * LOG2E);
  float q = fmaf(t, -0.023689253f, 0.10028721f);
  q = fmaf(t, q, -0.20866966f);
  q = fmaf(t, q, 0.32441181f);
  q = fmaf(t, q, -0.49918786f);
  q = fmaf(t, q, 0.99998188f);
  return fmaf(t, q, fmaxf(x, 0.f));
}

template <typename T> __device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b);
template <> __device__ __forceinline__ uint32_t mul2<__nv_bfloat16>(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t mul2<__half>(uint32_t a, uint32_t b) {
  __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

// Phase tables built once per call in the workspace: cos(freqs[pos][c]) and sin(freqs[pos][c]) as two
// half arrays [n][r], the sine array following the cosine array.
// Tensor map of a (batch, head, row, feature) operand for box loads of `box_rows` rows x 8 features (one
// 16-byte chunk column of the operand layout).  Returns false when the driver's encoder is unavailable or
// rejects the geometry; callers then stage that operand with ordinary loads.
bool make_chunk_tmap(CUtensorMap* out, const void* base, bool is_bf16, int d, int rows, int heads, int batch, int64_t sn,
                     int64_t sh, int64_t sb, int box_rows);

// `as_bf16` selects bf16 instead of fp16 entries (the forward multiplies in the operand dtype).
cudaError_t launch_trig_table(const float* freqs, int64_t sfn, int n, int r, void* table, bool as_bf16, cudaStream_t st);
inline size_t trig_table_bytes(int n, int r) { return (size_t)n * r * 2 * sizeof(__half) + 16; }

// Expanded-operand images (see tc_expand.cu): 64-row tiles [chunk][row][16 B], contiguous per (unit, tile).
constexpr int IMAGE_ROWS = 64;
__host__ __device__ inline size_t image_tiles(int rows) { return (size_t)(rows + IMAGE_ROWS - 1) / IMAGE_ROWS; }
inline size_t image_bytes(int units, int rows, int kd) { return (size_t)units * image_tiles(rows) * IMAGE_ROWS * kd * 2; }
// `table` = the 16-bit cos / sin table in the operand dtype ([tab_n][r] twice); row j of the operand takes table
// row pos0 + j.
cudaError_t launch_expand_images(const void* x, const PopeStride3& sx, int batch, int heads, int rows, int d, int r,
                                 bool is_bf16, const void* table, int tab_n, int pos0, void* img, cudaStream_t st);

// cos / sin of the per-head phase bias into shared memory (r floats each); `sign` = -1 folds the bias
// into a query-side phase (f - b), +1 into a key-side phase (f + b).  Call before a __syncthreads().
__device__ __forceinline__ void load_bias_trig(const float* bias, int r, float sign, float* cb, float* sb, int tid) {
  for (int c = tid; c < r; c += 256) {
    float s, co;
    sincosf(sign * bias[c], &s, &co);
    cb[c] = co, sb[c] = s;
  }
}

// Work split of the staging helpers: the 16-byte chunks of a ROWS x D tile are numbered row-major and a
// warp takes 32 consecutive ones per pass, so every global request covers 512 contiguous bytes of a row
// pair (requests spread over 8 rows ran at a third of that rate).  In shared memory chunk c of a
// streamed 64-row tile starts at c * (64*16 + 16): the 16 bytes of padding put the lanes of a pass,
// which hold consecutive chunks of one row, on distinct banks.
template <int ROWS> struct ChunkStride { static constexpr int v = ROWS == 64 ? 64 * 16 + 16 : ROWS * 16; };
constexpr int CS64 = ChunkStride<64>::v;
constexpr int CS128 = ChunkStride<128>::v;

template <int ROWS, int DC>
__device__ __forceinline__ void stage_coords(int wt, int lane, int& row, int& c) {
  const int f = wt * 32 + lane;
  row = f / DC;
  c = f - row * DC;
}

// Expand ROWS rows (row0 .. row0+ROWS) of a (rows, D) operand into the K-major operand layout
// (chunk-major storage: chunk*ROWS*16 + row*16 bytes): chunks [0, D/8) hold a*cos(phase) for rotated
// features and the raw feature otherwise, chunks [D/8, D/8 + r/8) hold a*sin(phase).  phase = table
// row (pos0 + row), rotated by the shared-memory bias trig when BIAS.  Rows >= nrows are zero-filled.
// All global loads of a batch are issued before any of its arithmetic.  256 threads.
struct NoHook {
  __device__ __forceinline__ void operator()() const {}
};

// NW warps share the work; `warp` is this warp's index among them (0 .. NW-1).  `before_store` runs once,
// after the first batch of loads has been issued and before anything is written to `buf` (the place to
// wait for the buffer to become free without delaying the loads).
template <int D, int ROWS, typename T, bool BIAS, int NW = 8, typename Hook = NoHook, typename TT = __half>
__device__ __forceinline__ void stage_xform_w(const T* base, int64_t sn, int row0, int nrows, const TT* tab,
                                              int tab_n, int pos0, int r, const float* cb, const float* sb, uint8_t* buf,
                                              int warp, int lane, Hook before_store = Hook()) {
  constexpr int DC = D / 8, NT = (ROWS * DC / 32) / NW, BATCH = NT > 4 ? NT / 2 : NT;
  static_assert(NT * NW * 32 == ROWS * DC && NT % BATCH == 0, "work does not split evenly");
  const int RC = r >> 3;
  const TT* tab_s = tab + (int64_t)tab_n * r;
#pragma unroll
  for (int b0 = 0; b0 < NT; b0 += BATCH) {
    uint4 raw[BATCH], tc[BATCH], ts[BATCH];
#pragma unroll
    for (int it = 0; it < BATCH; ++it) {
      int row, c;
      stage_coords<ROWS, DC>(warp + NW * (b0 + it), lane, row, c);
      const int j = row0 + row;
      raw[it] = tc[it] = ts[it] = make_uint4(0, 0, 0, 0);
#ifdef POPE_DBG_NOLOAD
      if (false) {
#else
      if (j < nrows) {
#endif
        raw[it] = *reinterpret_cast<const uint4*>(base + (int64_t)j * sn + c * 8);
        if (c < RC) {
          tc[it] = *reinterpret_cast<const uint4*>(tab + (int64_t)(pos0 + j) * r + c * 8);
          ts[it] = *reinterpret_cast<const uint4*>(tab_s + (int64_t)(pos0 + j) * r + c * 8);
        }
      }
    }
    if (b0 == 0) before_store();
#pragma unroll
    for (int it = 0; it < BATCH; ++it) {
      int row, c;
      stage_coords<ROWS, DC>(warp + NW * (b0 + it), lane, row, c);
      if (c < RC) {
        const uint32_t rw[4] = {raw[it].x, raw[it].y, raw[it].z, raw[it].w};
        const uint32_t cw[4] = {tc[it].x, tc[it].y, tc[it].z, tc[it].w};
        const uint32_t sw[4] = {ts[it].x, ts[it].y, ts[it].z, ts[it].w};
        uint32_t oc[4], os[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = unpack2<T>(rw[e]);
          if (BIAS) {   // resident operand, built once per CTA: fp32 products with the bias rotation
            float2 co = unpack2<TT>(cw[e]);
            float2 si = unpack2<TT>(sw[e]);
            const float2 b_c = *reinterpret_cast<const float2*>(cb + c * 8 + 2 * e);
            const float2 b_s = *reinterpret_cast<const float2*>(sb + c * 8 + 2 * e);
            const float2 c2 = make_float2(co.x * b_c.x - si.x * b_s.x, co.y * b_c.y - si.y * b_s.y);
            si = make_float2(si.x * b_c.x + co.x * b_s.x, si.y * b_c.y + co.y * b_s.y);
            co = c2;
            const float a0 = softplus_fast(x.x), a1 = softplus_fast(x.y);
            oc[e] = pack2<T>(a0 * co.x, a1 * co.y);   // zero rows: softplus(0) * table 0 = 0
            os[e] = pack2<T>(a0 * si.x, a1 * si.y);
          } else {      // streamed operand: packed 16-bit products, table already in the operand dtype
            static_assert(BIAS || sizeof(TT) == sizeof(T), "streamed tiles multiply in the operand dtype");
            const uint32_t a2 = pack2<T>(softplus_fast(x.x), softplus_fast(x.y));
            oc[e] = mul2<T>(a2, cw[e]);
            os[e] = mul2<T>(a2, sw[e]);
          }
        }
        *reinterpret_cast<uint4*>(buf + c * ChunkStride<ROWS>::v + row * 16) = make_uint4(oc[0], oc[1], oc[2], oc[3]);
        *reinterpret_cast<uint4*>(buf + (DC + c) * ChunkStride<ROWS>::v + row * 16) = make_uint4(os[0], os[1], os[2], os[3]);
      } else {
        *reinterpret_cast<uint4*>(buf + c * ChunkStride<ROWS>::v + row * 16) = raw[it];
      }
    }
  }
}

// Pull one streamed tile towards L2 ahead of use.  Every CTA of a (batch, head) unit walks the same tiles at
// about the same time, so without this each tile's first touch is an HBM miss that all of them wait on.
// 256 producer threads: thread t covers row t % 64 of array t / 64 (X rows, Y rows, cos rows, sin rows);
// a row is D (or r) 2-byte elements.
template <int D, typename T>
__device__ __forceinline__ void prefetch_tile_l2(const T* xbase, int64_t xsn, const T* ybase, int64_t ysn, int row0,
                                                 int nrows, const T* tab, int tab_n, int pos0, int r, int ptid) {
  const int row = row0 + (ptid & 63), which = ptid >> 6;
  if (row >= nrows) return;
  const char* ptr;
  int bytes;
  if (which == 0) ptr = reinterpret_cast<const char*>(xbase + (int64_t)row * xsn), bytes = D * 2;
  else if (which == 1) ptr = reinterpret_cast<const char*>(ybase + (int64_t)row * ysn), bytes = D * 2;
  else ptr = reinterpret_cast<const char*>(tab + (int64_t)(which - 2) * tab_n * r + (int64_t)(pos0 + row) * r), bytes = r * 2;
  for (int o = 0; o < bytes; o += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr + o));
}

// ---- streaming producer: a register window of K-tile tasks kept in flight across tiles ---------------
struct XTask {
  uint4 raw, tc, ts;
};

// load the inputs of one 8-row x 4-chunk warp task (no shared-memory traffic)
template <int D, int ROWS, typename T>
__device__ __forceinline__ void xtask_load(XTask& t, const T* base, int64_t sn, int row0, int nrows, const T* tab,
                                           const T* tab_s, int pos0, int r, int wt, int lane) {
  constexpr int DC = D / 8;
  int row, c;
  stage_coords<ROWS, DC>(wt, lane, row, c);
  const int j = row0 + row;
  t.raw = t.tc = t.ts = make_uint4(0, 0, 0, 0);
#ifdef POPE_DBG_NOLOAD
  t.raw = make_uint4(j, c, wt, lane); t.tc = t.raw; t.ts = t.raw;
  if (false) {
#else
  if (j < nrows) {
#endif
    t.raw = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)j * sn + c * 8));
    if (c < (r >> 3)) {
      t.tc = __ldg(reinterpret_cast<const uint4*>(tab + (int64_t)(pos0 + j) * r + c * 8));
      t.ts = __ldg(reinterpret_cast<const uint4*>(tab_s + (int64_t)(pos0 + j) * r + c * 8));
    }
  }
}

// Expand one task and write it into the operand buffer.  The table holds cos / sin in the operand dtype
// and the products are packed 16-bit multiplies: no 16 -> 32-bit conversion of the table.
template <int D, int ROWS, typename T>
__device__ __forceinline__ void xtask_store_packed(const XTask& t, int r, uint8_t* buf, int wt, int lane) {
  constexpr int DC = D / 8;
  int row, c;
  stage_coords<ROWS, DC>(wt, lane, row, c);
  if (c < (r >> 3)) {
    const uint32_t rw[4] = {t.raw.x, t.raw.y, t.raw.z, t.raw.w};
    const uint32_t cw[4] = {t.tc.x, t.tc.y, t.tc.z, t.tc.w};
    const uint32_t sw[4] = {t.ts.x, t.ts.y, t.ts.z, t.ts.w};
    uint32_t oc[4], os[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
#ifdef POPE_DBG_NOMATH
      oc[e] = rw[e] ^ cw[e];
      os[e] = rw[e] ^ sw[e];
#else
      const float2 x = unpack2<T>(rw[e]);
      const uint32_t a2 = pack2<T>(softplus_fast(x.x), softplus_fast(x.y));
      oc[e] = mul2<T>(a2, cw[e]);
      os[e] = mul2<T>(a2, sw[e]);
#endif
    }
#ifdef POPE_DBG_NOSTORE
    if ((oc[0] ^ oc[1] ^ oc[2] ^ oc[3] ^ os[0] ^ os[1] ^ os[2] ^ os[3]) == 0x12345u)
#endif
    {
    *reinterpret_cast<uint4*>(buf + c * ChunkStride<ROWS>::v + row * 16) = make_uint4(oc[0], oc[1], oc[2], oc[3]);
    *reinterpret_cast<uint4*>(buf + (DC + c) * ChunkStride<ROWS>::v + row * 16) = make_uint4(os[0], os[1], os[2], os[3]);
    }
  } else {
    *reinterpret_cast<uint4*>(buf + c * ChunkStride<ROWS>::v + row * 16) = t.raw;
  }
}

// 256-thread form used where all of a CTA's first eight warps stage together
template <int D, int ROWS, typename T, bool BIAS, typename TT>
__device__ __forceinline__ void stage_xform(const T* base, int64_t sn, int row0, int nrows, const TT* tab, int tab_n,
                                            int pos0, int r, const float* cb, const float* sb, uint8_t* buf, int tid) {
  stage_xform_w<D, ROWS, T, BIAS, 8, NoHook, TT>(base, sn, row0, nrows, tab, tab_n, pos0, r, cb, sb, buf, tid >> 5,
                                                   tid & 31);
}

// Copy ROWS rows of a (rows, D) operand unchanged into the same chunk-major layout.
template <int D, int ROWS, typename T, int NW = 8, typename Hook = NoHook>
__device__ __forceinline__ void stage_plain_w(const T* base, int64_t sn, int row0, int nrows, uint8_t* buf, int warp,
                                              int lane, Hook before_store = Hook()) {
  constexpr int DC = D / 8, NT = (ROWS * DC / 32) / NW;
  uint4 raw[NT];
#pragma unroll
  for (int it = 0; it < NT; ++it) {
    int row, c;
    stage_coords<ROWS, DC>(warp + NW * it, lane, row, c);
    const int j = row0 + row;
    raw[it] = make_uint4(0, 0, 0, 0);
    if (j < nrows) raw[it] = *reinterpret_cast<const uint4*>(base + (int64_t)j * sn + c * 8);
  }
  before_store();
#pragma unroll
  for (int it = 0; it < NT; ++it) {
    int row, c;
    stage_coords<ROWS, DC>(warp + NW * it, lane, row, c);
    *reinterpret_cast<uint4*>(buf + c * ChunkStride<ROWS>::v + row * 16) = raw[it];
  }
}
template <int D, int ROWS, typename T>
__device__ __forceinline__ void stage_plain(const T* base, int64_t sn, int row0, int nrows, uint8_t* buf, int tid) {
  stage_plain_w<D, ROWS, T, 8>(base, sn, row0, nrows, buf, tid >> 5, tid & 31);
}

}  // namespace pope
