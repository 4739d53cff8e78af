// Helpers shared by the tensor-core (tcgen05) attention kernels: operand formats, packing,
// fast device math and the per-position (cos, sin) phase table.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include <atomic>
#include <cstdio>
#include <utility>

#include <cuda.h>   // CUtensorMap (types only; the encoder is fetched through the runtime's driver entry point)

#include "common.cuh"
#include "tc05.cuh"

namespace pope {

using namespace tc;

// Opt a kernel into the full 227 KB of dynamic shared memory once per (kernel instantiation, device) instead of
// on every launch.  `Kernel` is the kernel function itself (a template VALUE parameter: instantiations share one
// function-pointer type), so every instantiation gets its own flag word, one bit per device.
constexpr int kMaxDynamicSmem = 227 * 1024;
template <auto Kernel>
inline cudaError_t ensure_max_smem() {
  static std::atomic<uint64_t> done{0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && ((done.load(std::memory_order_acquire) >> dev) & 1ull)) return cudaSuccess;
  e = cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem);
  if (e == cudaSuccess && dev >= 0 && dev < 64) done.fetch_or(1ull << dev, std::memory_order_release);
  return e;
}

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

// Tensor map of a (batch, head, row, feature) operand for box loads of `box_rows` rows x 8 features (one
// 16-byte chunk column of the operand layout).  Returns false when the driver's encoder is unavailable or
// rejects the geometry; callers then stage that operand with ordinary loads.
bool make_chunk_tmap(CUtensorMap* out, const void* base, bool is_bf16, int d, int rows, int heads, int batch, int64_t sn,
                     int64_t sh, int64_t sb, int box_rows);
// Tensor map of a (batch, head, row, column) OUTPUT for tiled stores out of a 128-byte-swizzled staging tile: boxes of
// `box_rows` rows x 128 bytes (32 fp32 or 64 16-bit columns); rows / columns beyond the tensor are clipped by the
// copy engine.  dtype is a PopeDtype.  Returns false when the geometry breaks the 16-byte stride / base rules.
bool make_store_tmap(CUtensorMap* out, const void* base, int dtype, int cols, int rows, int heads, int batch, int64_t sn,
                     int64_t sh, int64_t sb, int box_rows);

// Expanded-operand images (see tc_expand.cu): 64-row tiles [chunk][row][16 B], contiguous per (unit, tile).
// Every unit is padded with zero rows to a multiple of 256 rows (4 tiles), so that a CTA which keeps 128 or 256
// rows resident can always copy whole tiles.
constexpr int IMAGE_ROWS = 64;
__host__ __device__ inline size_t image_tiles(int rows) { return (size_t)((rows + 255) / 256) * 4; }
inline size_t image_bytes(int units, int rows, int kd) { return (size_t)units * image_tiles(rows) * IMAGE_ROWS * kd * 2; }
// One operand to expand: `rows` rows of `units` = batch x heads (batch, head) slices of x, the first r of its d
// features rotated by table row pos0 + j (r = 0: a pure re-layout).  bias (may be null) = per-head phase offset
// added to the table phase, head index = unit % heads.  The image goes to img.
struct ExpandJob {
  const void* x;
  PopeStride3 sx;
  int units, heads, rows, r, pos0;
  int tab_rows, tab_by_batch, tab_heads;   // table slice of a unit: (tab_by_batch ? batch : 0) * tab_heads + head % tab_heads
  const float* bias;
  int64_t bias_sh;
  void* img;
  int tile128;   // 1: pairs of 64-row tiles are interleaved into 128-row tiles [chunk][128 rows][16 B] (one bulk copy per 128-key stage)
};
struct ExpandJobs { ExpandJob job[4]; };
inline ExpandJob expand_job(const void* x, const PopeStride3& sx, int batch, int heads, int rows, int r, int pos0,
                            const float* bias, int64_t bias_sh, void* img, int tab_rows = 0, int tab_by_batch = 0,
                            int tab_heads = 1) {
  ExpandJob j;
  j.x = x, j.sx = sx, j.units = batch * heads, j.heads = heads, j.rows = rows, j.r = r, j.pos0 = pos0;
  j.tab_rows = tab_rows, j.tab_by_batch = tab_by_batch, j.tab_heads = tab_heads;
  j.bias = r > 0 ? bias : nullptr, j.bias_sh = bias_sh, j.img = img, j.tile128 = 0;
  return j;
}
// 16-bit (feature, row, head, batch) view cut into boxes of 64 features (128-byte rows) x box_rows rows, 128-byte swizzled
bool make_wide_tmap(CUtensorMap* out, const void* base, bool is_bf16, int d, int rows, int heads, int batch, int64_t sn,
                    int64_t sh, int64_t sb, int box_rows);
// an operand image as (1 KB run, tile, chunk): box = (1 KB, 2 tiles, all chunks) = one resident 128-row operand
bool make_image_tmap(CUtensorMap* out, const void* img, int64_t ntiles, int chunks);
// ch / sh = fp16 cos / sin of the phase table, [positions][r].  All jobs share d and the dtype; one launch.
// `dependent`: launch it as a programmatic dependent of the kernel before it on the stream (only when that kernel is one
// of this library's: the kernel waits for it before its first read)
cudaError_t launch_expand_images(const ExpandJobs& jobs, int njobs, int d, bool is_bf16, const void* ch, const void* sh,
                                 cudaStream_t st, bool dependent = false);

// Launch `kernel` so that its CTAs may start while the previous kernel on `st` still runs (programmatic stream
// serialization); the kernel calls pdl_wait() before it reads what that kernel wrote.  Use it only behind a kernel of
// this library that was itself ordered after everything earlier on the stream.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
// fp32 cos / sin of freqs[pos][c] into ctab / stab ([n][r] each); launch_trig_tables also writes fp16 copies (ch, sh).
// Where a phase comes from: the caller's table, or (factored form) position x inverse frequency, one fp32 multiply.
struct PhaseSrc {
  const float* freqs;
  int64_t sfn, sfb, sfh;   // row stride; batch / head strides of a batched table (0 = that axis is broadcast)
  int tab_heads;           // table slices per batch entry: the head count when the table has a head axis, else 1
  const float* pos;
  int64_t spos;
  const float* inv;
  const int32_t* axis;
  __device__ __forceinline__ float at(int64_t row, int c) const {
    if (pos) return __fmul_rn(pos[row * spos + (axis ? axis[c] : 0)], inv[c]);
    return freqs[row * sfn + c];
  }
};
inline PhaseSrc phase_src(const PopeEmbed& e) {
  PhaseSrc s;
  s.freqs = e.freqs, s.sfn = e.sf.n, s.sfb = e.sf.b, s.sfh = e.sf.h, s.tab_heads = 1;
  const bool factored = e.positions && e.inv_freqs && e.sf.b == 0 && e.sf.h == 0;
  s.pos = factored ? e.positions : nullptr, s.spos = e.pos_stride_n, s.inv = e.inv_freqs, s.axis = e.axis_of;
  return s;
}
cudaError_t launch_trig_table_f32(const PopeEmbed& e, int n, int r, float* ctab, float* stab, cudaStream_t st);
// `slices` tables of n x r entries, slice = batch index x tab_heads + head index of a batched caller table (1 slice for a
// plain (n, r) table); every output pointer may be null
cudaError_t launch_trig_tables(const PopeEmbed& e, int n, int r, float* ctab, float* stab, void* ch, void* sh, cudaStream_t st,
                               int slices = 1, int tab_heads = 1);
// slices of the phase table an attention call needs: one per batch entry and / or head that the caller's table tells apart
inline int table_heads(const PopeEmbed& e, int heads) { return e.sf.h != 0 ? heads : 1; }
inline int table_slices(const PopeEmbed& e, int batch, int heads) { return (e.sf.b != 0 ? batch : 1) * table_heads(e, heads); }
// Table block of the attention workspace: [cos fp16][sin fp16], slices * n * r entries each (cos and sin lie in [-1, 1]:
// 2^-12 absolute error, and the operand the image pre-pass builds from them is rounded to 8 or 11 bits anyway).
struct TrigTables {
  void *ch, *sh;
};
inline size_t trig_tables_bytes(int n, int r, int slices = 1) { return ((size_t)slices * n * r * 4 + 255) & ~(size_t)255; }
inline TrigTables trig_tables_at(void* base, int n, int r, int slices = 1) {
  TrigTables t;
  t.ch = base, t.sh = static_cast<uint8_t*>(base) + (size_t)slices * n * r * 2;
  return t;
}

// A resident 128-row operand [chunk][128 rows][16 B] out of two consecutive image tiles: 2 x `chunks` bulk copies
// of 1 KB, issued by the lanes of one warp after one of them has posted 2 * chunks * 1024 transaction bytes on `bar`.
__device__ __forceinline__ void copy_resident_tiles(uint8_t* dst, const uint8_t* img_tile0, int chunks, uint64_t* bar, int lane) {
  for (int i = lane; i < 2 * chunks; i += 32) {
    const int c = i >> 1, hlf = i & 1;
    bulk_load(dst + c * 2048 + hlf * 1024, img_tile0 + ((size_t)hlf * chunks + c) * 1024, 1024, bar);
  }
}

// Chunk stride used where THREADS store 16-byte groups of a 64-row tile in row-major group order (the image
// pre-pass): 16 bytes of padding per chunk column put the lanes of a warp, which hold consecutive chunks of one
// row, on distinct banks.  Tiles written by the copy engine are unpadded.
constexpr int CS64 = 64 * 16 + 16;

}  // namespace pope
