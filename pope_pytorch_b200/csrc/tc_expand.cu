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
// (d+r)/8 copies of 1 KB per 64 rows.  Rows past the end of the operand are zero.  The per-head phase
// bias is NOT part of an image: the kernels fold it into whichever operand they keep resident.
#include "kernels.h"
#include "tc_common.cuh"

namespace pope {

// grid (tiles, units), 256 threads; dynamic shared memory (d+r)/8 * CS64 bytes
template <typename T>
__global__ void __launch_bounds__(256) expand_image_kernel(const T* __restrict__ x, Strides sx, int heads, int rows, int d,
                                                            int r, const T* __restrict__ tab, int tab_n, int pos0,
                                                            uint8_t* __restrict__ img) {
  extern __shared__ __align__(16) uint8_t stage[];
  const int tid = threadIdx.x, tile = blockIdx.x, u = blockIdx.y;
  const int DC = d >> 3, RC = r >> 3, KC = DC + RC;
  const T* base = x + (int64_t)(u / heads) * sx.b + (int64_t)(u % heads) * sx.h;
  const T* tab_s = tab + (int64_t)tab_n * r;
  // phase 1: 16-byte groups in row-major order (a warp reads 512 contiguous bytes of a row pair); the
  // padded chunk stride keeps the shared-memory stores of a warp on distinct banks
  for (int f = tid; f < IMAGE_ROWS * DC; f += 256) {
    const int row = f / DC, c = f - row * DC, j = tile * IMAGE_ROWS + row;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (j < rows) raw = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)j * sx.n + c * 8));
    if (c < RC) {
      uint4 oc = make_uint4(0, 0, 0, 0), os = oc;
      if (j < rows) {
        const uint4 tc = __ldg(reinterpret_cast<const uint4*>(tab + (int64_t)(pos0 + j) * r + c * 8));
        const uint4 ts = __ldg(reinterpret_cast<const uint4*>(tab_s + (int64_t)(pos0 + j) * r + c * 8));
        const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w}, cw[4] = {tc.x, tc.y, tc.z, tc.w}, sw[4] = {ts.x, ts.y, ts.z, ts.w};
        uint32_t o1[4], o2[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 xv = unpack2<T>(rw[e]), co = unpack2<T>(cw[e]), si = unpack2<T>(sw[e]);
          const float a0 = softplus_fast(xv.x), a1 = softplus_fast(xv.y);
          o1[e] = pack2<T>(a0 * co.x, a1 * co.y);
          o2[e] = pack2<T>(a0 * si.x, a1 * si.y);
        }
        oc = make_uint4(o1[0], o1[1], o1[2], o1[3]), os = make_uint4(o2[0], o2[1], o2[2], o2[3]);
      }
      *reinterpret_cast<uint4*>(stage + c * CS64 + row * 16) = oc;
      *reinterpret_cast<uint4*>(stage + (DC + c) * CS64 + row * 16) = os;
    } else {
      *reinterpret_cast<uint4*>(stage + c * CS64 + row * 16) = raw;
    }
  }
  __syncthreads();
  // phase 2: the image leaves in its own byte order, 16 bytes per thread, fully coalesced
  uint4* out = reinterpret_cast<uint4*>(img + ((int64_t)u * gridDim.x + tile) * ((int64_t)IMAGE_ROWS * KC * 16));
  for (int g = tid; g < IMAGE_ROWS * KC; g += 256) {
    const int c = g / IMAGE_ROWS, row = g - c * IMAGE_ROWS;
    out[g] = *reinterpret_cast<const uint4*>(stage + c * CS64 + row * 16);
  }
}

cudaError_t launch_expand_images(const void* x, const PopeStride3& sx, int batch, int heads, int rows, int d, int r,
                                 bool is_bf16, const void* table, int tab_n, int pos0, void* img, cudaStream_t st) {
  const dim3 grid((unsigned)image_tiles(rows), (unsigned)(batch * heads));
  const size_t smem = (size_t)((d + r) / 8) * CS64;
  if (is_bf16)
    expand_image_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>(static_cast<const __nv_bfloat16*>(x), Strides(sx), heads, rows,
                                                                 d, r, static_cast<const __nv_bfloat16*>(table), tab_n, pos0,
                                                                 static_cast<uint8_t*>(img));
  else
    expand_image_kernel<__half><<<grid, 256, smem, st>>>(static_cast<const __half*>(x), Strides(sx), heads, rows, d, r,
                                                          static_cast<const __half*>(table), tab_n, pos0,
                                                          static_cast<uint8_t*>(img));
  return cudaGetLastError();
}

}  // namespace pope
