// Operand images for the tensor-core attention kernels (sm_100a).
//
// The attention kernels multiply EXPANDED operands X' = [a cos(f) | pass-through | a sin(f)], a = softplus(x)
// (PoPE_pytorch/pope.py:52-84), of width d + r.  A streamed operand is re-read by every CTA that sweeps it
// (Nq / 256 times in the forward), so expanding it inside those CTAs repeats the softplus and the products
// that many times.  This pre-pass expands each operand ONCE per call into the caller's workspace, already cut
// into 64-row tiles in the byte order the tensor core reads from shared memory:
//
//     image[unit][tile][chunk c = 0 .. (d+r)/8)[row 0..64)[8 features]      (16 bytes per innermost group)
//
// so that a tile reaches shared memory as one contiguous bulk copy, and a 128-row resident operand as
// (d+r)/8 copies of 1 KB per 64 rows.  Rows past the end of the operand are zero, and every unit is padded to a
// multiple of 256 rows.  The per-head phase offset (the learned bias of the keys, PoPE_pytorch/pope.py:75-79)
// is folded into the key images; query images carry the bare table phase.
#include <algorithm>

#include "kernels.h"
#include "tc_common.cuh"

namespace pope {

// grid (tiles / 4, units, jobs), 256 threads; dynamic shared memory (d+r)/8 * CS64 bytes + 2 r floats.  One launch
// builds the images of up to four operands (blockIdx.z picks the job); CTAs outside a job's tile / unit range leave.
// A CTA builds EXPAND_TPC consecutive tiles of one unit.  A thread keeps the same 16-byte feature group (chunk) for
// every row it touches, so whether it rotates at all, and the cos / sin of the head's phase offset for its eight
// features, are fixed for its lifetime (registers instead of 16 shared-memory loads per group); the raw rows of the
// next tile are requested before the current tile is worked on.
constexpr int EXPAND_TPC = 4;
template <typename T, int D>
__global__ void __launch_bounds__(256, 3) expand_image_kernel(ExpandJobs jobs, const __half* __restrict__ ctab,
                                                            const __half* __restrict__ stab) {
  // (ctab / stab are advanced to the unit's table slice below)
  extern __shared__ __align__(16) uint8_t stage[];
  pdl_trigger();   // the attention kernel behind this one may set itself up
  pdl_wait();      // the phase tables (the kernel before this one) are complete
  const ExpandJob& jb = jobs.job[blockIdx.z];
  const int tid = threadIdx.x, u = blockIdx.y;
  const int tiles = (int)image_tiles(jb.rows);   // a multiple of EXPAND_TPC
  const int tile0 = blockIdx.x * EXPAND_TPC;
  if (tile0 >= tiles || u >= jb.units) return;
  const int r = jb.r, rows = jb.rows;
  constexpr int DC = D >> 3;
  constexpr int RPP = 256 / DC;                          // rows per pass of the 256 threads
  constexpr int NIT = (IMAGE_ROWS + RPP - 1) / RPP;      // passes per tile
  const int RC = r >> 3, KC = DC + RC;
  const int c = tid % DC, row0 = tid / DC;
  const bool active = row0 < RPP, rotated = c < RC;
  float* bias_c = reinterpret_cast<float*>(stage + KC * CS64);   // cos / sin of this head's phase offset
  float* bias_s = bias_c + r;
  const Strides sx(jb.sx);
  const T* base = static_cast<const T*>(jb.x) + (int64_t)(u / jb.heads) * sx.b + (int64_t)(u % jb.heads) * sx.h + c * 8;
  const float* bias = jb.bias;
  {   // this unit's slice of the phase tables (a batched caller table has one slice per batch entry and / or head)
    const int64_t slice = (int64_t)(jb.tab_by_batch ? u / jb.heads : 0) * jb.tab_heads + (u % jb.heads) % jb.tab_heads;
    ctab += slice * jb.tab_rows * r + c * 8, stab += slice * jb.tab_rows * r + c * 8;
  }
  float cb[8], sb[8];
  if (bias) {
    for (int i = tid; i < r; i += 256) sincosf(bias[(int64_t)(u % jb.heads) * jb.bias_sh + i], &bias_s[i], &bias_c[i]);
    __syncthreads();
    if (rotated) {
#pragma unroll
      for (int e = 0; e < 8; ++e) cb[e] = bias_c[c * 8 + e], sb[e] = bias_s[c * 8 + e];
    }
  }
  auto load_raw = [&](int tile, uint4 (&raw)[NIT]) {
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int row = row0 + it * RPP, jrow = tile * IMAGE_ROWS + row;
      raw[it] = make_uint4(0, 0, 0, 0);
      if (active && row < IMAGE_ROWS && jrow < rows) raw[it] = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)jrow * sx.n));
    }
  };
  for (int tt = 0; tt < EXPAND_TPC; ++tt) {
    const int tile = tile0 + tt;
    uint4 raw[NIT];
    load_raw(tile, raw);
    // phase 1: 16-byte groups in row-major order (a warp reads 512 contiguous bytes of a row pair); the
    // padded chunk stride keeps the shared-memory stores of a warp on distinct banks.
    if (rotated) {
      uint4 cq[NIT], sq[NIT];
#pragma unroll
      for (int it = 0; it < NIT; ++it) {
        const int row = row0 + it * RPP, jrow = tile * IMAGE_ROWS + row;
        cq[it] = sq[it] = make_uint4(0, 0, 0, 0);
        if (active && row < IMAGE_ROWS && jrow < rows) {
          cq[it] = __ldg(reinterpret_cast<const uint4*>(ctab + (int64_t)(jb.pos0 + jrow) * r));
          sq[it] = __ldg(reinterpret_cast<const uint4*>(stab + (int64_t)(jb.pos0 + jrow) * r));
        }
      }
#pragma unroll
      for (int it = 0; it < NIT; ++it) {
        const int row = row0 + it * RPP;
        if (!active || row >= IMAGE_ROWS) continue;
        // (rows past the end carry zero raw words and zero table words: softplus(0) * 0 = 0)
        const uint32_t cw[4] = {cq[it].x, cq[it].y, cq[it].z, cq[it].w}, sw[4] = {sq[it].x, sq[it].y, sq[it].z, sq[it].w};
        const uint32_t rw[4] = {raw[it].x, raw[it].y, raw[it].z, raw[it].w};
        uint32_t o1[4], o2[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 cv = unpack2<__half>(cw[e]), sv = unpack2<__half>(sw[e]);
          if (bias) {   // cos(f + b), sin(f + b)
            const float c0 = cv.x * cb[2 * e] - sv.x * sb[2 * e], s0 = sv.x * cb[2 * e] + cv.x * sb[2 * e];
            const float c1 = cv.y * cb[2 * e + 1] - sv.y * sb[2 * e + 1], s1 = sv.y * cb[2 * e + 1] + cv.y * sb[2 * e + 1];
            cv = make_float2(c0, c1), sv = make_float2(s0, s1);
          }
          const float2 xv = unpack2<T>(rw[e]);
          const float a0 = softplus_fast(xv.x), a1 = softplus_fast(xv.y);
          o1[e] = pack2<T>(a0 * cv.x, a1 * cv.y);
          o2[e] = pack2<T>(a0 * sv.x, a1 * sv.y);
        }
        *reinterpret_cast<uint4*>(stage + c * CS64 + row * 16) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
        *reinterpret_cast<uint4*>(stage + (DC + c) * CS64 + row * 16) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
      }
    } else {
#pragma unroll
      for (int it = 0; it < NIT; ++it) {
        const int row = row0 + it * RPP;
        if (active && row < IMAGE_ROWS) *reinterpret_cast<uint4*>(stage + c * CS64 + row * 16) = raw[it];
      }
    }
    __syncthreads();
    // phase 2: the image leaves in its own byte order, 16 bytes per thread, fully coalesced
    if (jb.tile128) {   // tile 2 t and 2 t + 1 share one 128-row tile: chunk stride 2 KB, this tile's rows in one half of it
      uint8_t* out = static_cast<uint8_t*>(jb.img) + (((int64_t)u * tiles + tile) >> 1) * ((int64_t)2 * IMAGE_ROWS * KC * 16) +
                     (tile & 1) * (IMAGE_ROWS * 16);
      for (int g = tid; g < IMAGE_ROWS * KC; g += 256) {
        const int cc = g / IMAGE_ROWS, row = g - cc * IMAGE_ROWS;
        *reinterpret_cast<uint4*>(out + cc * (2 * IMAGE_ROWS * 16) + row * 16) = *reinterpret_cast<const uint4*>(stage + cc * CS64 + row * 16);
      }
    } else {
      uint4* out = reinterpret_cast<uint4*>(static_cast<uint8_t*>(jb.img) + ((int64_t)u * tiles + tile) * ((int64_t)IMAGE_ROWS * KC * 16));
      for (int g = tid; g < IMAGE_ROWS * KC; g += 256) {
        const int cc = g / IMAGE_ROWS, row = g - cc * IMAGE_ROWS;
        out[g] = *reinterpret_cast<const uint4*>(stage + cc * CS64 + row * 16);
      }
    }
    if (tt + 1 < EXPAND_TPC) __syncthreads();   // the stage is rewritten by the next tile
  }
}

template <typename T>
static cudaError_t launch_expand_t(const ExpandJobs& jobs, int njobs, int d, const __half* ctab, const __half* stab,
                                   cudaStream_t st, bool dependent) {
  int tiles = 0, units = 0, rmax = 0;
  for (int i = 0; i < njobs; ++i) {
    tiles = std::max(tiles, (int)image_tiles(jobs.job[i].rows));
    units = std::max(units, jobs.job[i].units);
    rmax = std::max(rmax, jobs.job[i].r);
  }
  const dim3 grid((unsigned)(tiles / EXPAND_TPC), (unsigned)units, (unsigned)njobs);
  const size_t smem = (size_t)((d + rmax) / 8) * CS64 + 2 * (size_t)rmax * sizeof(float);
  if (dependent) {
    switch (d) {
      case 64: return launch_dependent(expand_image_kernel<T, 64>, grid, dim3(256), smem, st, jobs, ctab, stab);
      case 96: return launch_dependent(expand_image_kernel<T, 96>, grid, dim3(256), smem, st, jobs, ctab, stab);
      case 128: return launch_dependent(expand_image_kernel<T, 128>, grid, dim3(256), smem, st, jobs, ctab, stab);
      default: return cudaErrorInvalidValue;
    }
  }
  switch (d) {
    case 64: expand_image_kernel<T, 64><<<grid, 256, smem, st>>>(jobs, ctab, stab); break;
    case 96: expand_image_kernel<T, 96><<<grid, 256, smem, st>>>(jobs, ctab, stab); break;
    case 128: expand_image_kernel<T, 128><<<grid, 256, smem, st>>>(jobs, ctab, stab); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_expand_images(const ExpandJobs& jobs, int njobs, int d, bool is_bf16, const void* ch, const void* sh,
                                 cudaStream_t st, bool dependent) {
  if (njobs < 1 || njobs > 4) return cudaErrorInvalidValue;
  const __half* ctab = static_cast<const __half*>(ch);
  const __half* stab = static_cast<const __half*>(sh);
  return is_bf16 ? launch_expand_t<__nv_bfloat16>(jobs, njobs, d, ctab, stab, st, dependent)
                 : launch_expand_t<__half>(jobs, njobs, d, ctab, stab, st, dependent);
}

}  // namespace pope
