// Fused PoPE similarity  sim = q' k'^T  on the Blackwell tensor cores (tcgen05 + TMEM), sm_100a only.
//
// The kernel is bound by the store of the Nq x Nk output; the contraction only has to keep up.  fp32
// inputs must come out at fp32 accuracy (1e-4 of max|sim|), which one bf16 product misses by an order of
// magnitude, so every expanded operand element x is split into two bf16 numbers  x = hi + lo  and the
// product is accumulated as  hi*hi' + hi*lo' + lo*hi'  (the dropped lo*lo' term is below 2^-17 relative).
// bf16 / fp16 inputs take the single-product path.
//
// A CTA owns 128 query rows and a range of key tiles (the key range is split so that small problems still
// fill the machine).  Q' (hi | lo) is expanded once into shared memory; per 128-key tile the eight worker
// warps expand K' (hi | lo), a ninth warp issues the MMA chains into one of two 128-column TMEM buffers,
// and the workers stream the previous tile out of TMEM with 16-byte stores, a row per thread.
// Phases come from fp32 (cos f, sin f) tables built once per call in the workspace; the per-head bias is
// rotated in at fp32 (cos(f + b) = cos f cos b - sin f sin b).  Nothing expanded goes to global memory.
//
// Reference semantics: PoPE_pytorch/triton_pope.py:28-83, PoPE_pytorch/attention.py:30-47.
#include "kernels.h"
#include "tc_common.cuh"

namespace pope {

struct TcSimP {
  int H, Hk, Nq, Nk, d, r;
  int keys_per_cta;          // multiple of 128
  int use_stg;               // 1: full fp32 tiles leave through the shared-memory staging tile and bulk stores
  const void *q, *k;
  void* sim;
  Strides sq, sk, ss;
  const float *ctab, *stab;  // [Nk][r] cos / sin of freqs
  const float* bias;
  int64_t bias_sh;
  unsigned int* status;
};

constexpr int SIM_M = 128;   // query rows per CTA
constexpr int SIM_N = 128;   // keys per step
constexpr int SIM_THREADS = 288;
constexpr int SIM_STG_ROW = 256 + 16;             // staging row: 64 fp32 columns + padding (conflict-free 16-byte stores)
constexpr int SIM_STG = SIM_M * SIM_STG_ROW;      // bytes of the output staging tile

// ch / sh (may be null): the same tables rounded to fp16 (cos and sin lie in [-1, 1]: 2^-12 absolute error), read by
// the operand-image pre-pass, whose result is rounded to 8 or 11 bits anyway.
__global__ void pope_trig_table_f32_kernel(const float* freqs, int64_t sfn, int n, int r, float* ctab, float* stab,
                                           __half* ch, __half* sh) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)n * r) return;
  const int pos = idx / r, c = idx % r;
  float sn, cs;
  sincosf(freqs[pos * sfn + c], &sn, &cs);
  if (ctab) stab[idx] = sn, ctab[idx] = cs;
  if (ch) ch[idx] = __float2half_rn(cs), sh[idx] = __float2half_rn(sn);
}

cudaError_t launch_trig_tables(const float* freqs, int64_t sfn, int n, int r, float* ctab, float* stab, void* ch, void* sh,
                               cudaStream_t st) {
  const int64_t total = (int64_t)n * r;
  pope_trig_table_f32_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(freqs, sfn, n, r, ctab, stab,
                                                                               static_cast<__half*>(ch), static_cast<__half*>(sh));
  return cudaGetLastError();
}
cudaError_t launch_trig_table_f32(const float* freqs, int64_t sfn, int n, int r, float* ctab, float* stab, cudaStream_t st) {
  return launch_trig_tables(freqs, sfn, n, r, ctab, stab, nullptr, nullptr, st);
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

constexpr int SIM_CS = SIM_M * 16 + 16;   // chunk stride in shared memory (padded: consecutive chunks of a row hit distinct banks)

// Expand 128 rows into chunk-major K-major storage: chunk c of the hi part at c*SIM_CS + row*16, the lo part KC
// chunks later.  Expanded columns: d cos/pass columns, then r sin columns.  The 8-feature chunks of the tile
// are numbered row-major and thread t takes chunks t, t + 256, ...: a warp's loads cover whole rows.
// phase = table row (pos0 + row), rotated by (cb, sb) when given.
template <typename T, bool SPLIT>
__device__ __forceinline__ void sim_stage(const T* base, int64_t sn, int row0, int nrows, const float* ctab,
                                          const float* stab, int pos0, int d, int r, const float* cb, const float* sb,
                                          uint8_t* buf, int tid) {
  const int DC = d >> 3, RC = r >> 3, KC = DC + RC;
  for (int f = tid; f < SIM_M * DC; f += 256) {
    const int row = f / DC, c = f - row * DC, j = row0 + row;
    const bool ok = j < nrows;
    uint8_t* dst = buf + row * 16;
    float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (ok) Load8<T>::run(base + (int64_t)j * sn + c * 8, x);
    if (c < RC) {
      float vc[8], vs[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) vc[e] = 0.f, vs[e] = 0.f;
      if (ok) {
        float co[8], si[8];
        Load8<float>::run(ctab + (int64_t)(pos0 + j) * r + c * 8, co);
        Load8<float>::run(stab + (int64_t)(pos0 + j) * r + c * 8, si);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float cs = co[e], sn_ = si[e];
          if (cb) {
            const float bc = cb[c * 8 + e], bs = sb[c * 8 + e];
            const float c2 = cs * bc - sn_ * bs;
            sn_ = sn_ * bc + cs * bs;
            cs = c2;
          }
          // ex2.approx / lg2.approx keep 2^-22: far inside the 1e-5 the split product needs, at a sixth of
          // the instructions of expf + log1pf
          const float a = softplus_fast(x[e]);
          vc[e] = a * cs, vs[e] = a * sn_;
        }
      }
      put_chunk<SPLIT>(dst + c * SIM_CS, dst + (KC + c) * SIM_CS, vc);
      put_chunk<SPLIT>(dst + (DC + c) * SIM_CS, dst + (KC + DC + c) * SIM_CS, vs);
    } else {
      put_chunk<SPLIT>(dst + c * SIM_CS, dst + (KC + c) * SIM_CS, x);
    }
  }
}

template <typename T, bool SPLIT>
__global__ void __launch_bounds__(SIM_THREADS, 1) sim_fwd_tc_kernel(TcSimP p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int KD = p.d + p.r, KC = KD >> 3, KSTEPS = KD >> 4;
  const int OPB = KC * SIM_CS * (SPLIT ? 2 : 1);         // bytes of one expanded 128-row operand (hi | lo)
  const int STGB = p.use_stg ? SIM_STG : 0;
  const int NKB = (3 * OPB + STGB + 4096 <= 227 * 1024) ? 2 : 1;  // double-buffer the key tile when it fits
  uint8_t* Qs = smem;
  uint8_t* Kb = Qs + OPB;
  uint8_t* Stg = Kb + NKB * OPB;                                  // output staging for the bulk stores
  uint64_t* bars = reinterpret_cast<uint64_t*>(Stg + STGB);       // [2] MMA chains of tile j done (slot j & 1)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  float* cb = reinterpret_cast<float*>(tmem_slot + 4);
  float* sb = cb + 256;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool issuer = warp == 8;
  const int u = blockIdx.z, b = u / p.H, h = u % p.H, hk = h % p.Hk;
  const int i0 = blockIdx.y * SIM_M;
  const int key0 = blockIdx.x * p.keys_per_cta, key1 = min(p.Nk, key0 + p.keys_per_cta);
  const int T_tiles = (key1 - key0 + SIM_N - 1) / SIM_N;
  const int qoff = p.Nk - p.Nq;
  const T* qbase = (const T*)p.q + b * p.sq.b + h * p.sq.h;
  const T* kbase = (const T*)p.k + b * p.sk.b + hk * p.sk.h;

  if (issuer) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&bars[0], 1), mbar_init(&bars[1], 1);
    mbar_init_fence();
  }
  if (!issuer) {
    for (int c = tid; c < p.r; c += 256) sincosf(p.bias[hk * p.bias_sh + c], &sb[c], &cb[c]);
    asm volatile("bar.sync 1, 256;" ::: "memory");
    sim_stage<T, SPLIT>(qbase, p.sq.n, i0, p.Nq, p.ctab, p.stab, qoff, p.d, p.r, nullptr, nullptr, Qs, tid);
    sim_stage<T, SPLIT>(kbase, p.sk.n, key0, key1, p.ctab, p.stab, 0, p.d, p.r, cb, sb, Kb, tid);
    fence_async_smem();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t idesc = instr_desc(FMT_BF16, SIM_M, SIM_N, false, false);
  const uint32_t q_addr = smem_u32(Qs), k_addr = smem_u32(Kb);
  bool failed = false;

  auto issue = [&](int jt) {   // the MMA chains of key tile jt into TMEM buffer jt & 1
    const uint32_t d = tmem + (jt & 1) * SIM_N;
    const uint32_t kb = k_addr + (jt % NKB) * OPB;
    const int chains = SPLIT ? 3 : 1;
    uint32_t acc = 0;
    for (int ch = 0; ch < chains; ++ch) {
      // chain 0: hi x hi, chain 1: hi x lo, chain 2: lo x hi
      uint64_t ad = smem_desc(q_addr + (ch == 2 ? KC * SIM_CS : 0), SIM_CS, 128);
      uint64_t bd = smem_desc(kb + (ch == 1 ? KC * SIM_CS : 0), SIM_CS, 128);
      for (int ks = 0; ks < KSTEPS; ++ks) {
        mma_ss(d, ad, bd, idesc, acc);
        acc = 1;
        ad += (2 * SIM_CS) >> 4, bd += (2 * SIM_CS) >> 4;
      }
    }
    mma_commit(&bars[jt & 1]);
  };
  if (issuer && lane == 0) issue(0);

  const int row = tid & 127, half = (tid >> 7) & 1;
  const int gi = i0 + row;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  T* srow = (T*)p.sim + b * p.ss.b + h * p.ss.h + (int64_t)gi * p.ss.n;

  for (int j = 0; j < T_tiles; ++j) {
    if (j + 1 < T_tiles) {
      if (!issuer) {
        // a single key buffer is still being read by the chains of tile j
        if (NKB == 1 && !failed) failed = !mbar_wait(&bars[j & 1], (j >> 1) & 1, WAIT_LIMIT);
        sim_stage<T, SPLIT>(kbase, p.sk.n, key0 + (j + 1) * SIM_N, key1, p.ctab, p.stab, 0, p.d, p.r, cb, sb,
                            Kb + ((j + 1) % NKB) * OPB, tid);
        fence_async_smem();
      }
      fence_before_sync();
      __syncthreads();   // also: every worker has drained TMEM buffer (j+1) & 1 (tile j-1)
      if (issuer && lane == 0) {
        fence_after_sync();
        issue(j + 1);
      }
    }
    if (!issuer) {
      if (!failed) failed = !mbar_wait(&bars[j & 1], (j >> 1) & 1, WAIT_LIMIT);
      fence_after_sync();
      const int tile0 = key0 + j * SIM_N;
      // Full fp32 tiles leave through shared memory: each pass moves 64 contiguous columns of every row
      // (the two thread halves hold its two 32-column pieces) as one 256-byte bulk store per row, so the
      // output is written in full lines instead of 16-byte pieces scattered over 32 rows per instruction.
      const bool bulk = sizeof(T) == 4 && p.use_stg && tile0 + SIM_N <= key1;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t v[32];
        const int piece = bulk ? hh * 2 + half : half * 2 + hh;   // which 32-column piece of the tile
        tmem_ld32(tmem + lane_base + (j & 1) * SIM_N + piece * 32, v);
        tmem_ld_wait();
        const int c0 = tile0 + piece * 32;
        if (bulk) {
          // the previous pass's bulk stores must have finished reading the staging tile
          if (tid < SIM_M) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          asm volatile("bar.sync 1, 256;" ::: "memory");
          uint8_t* dst = Stg + row * SIM_STG_ROW + half * 128;
#pragma unroll
          for (int i = 0; i < 32; i += 4) *reinterpret_cast<uint4*>(dst + i * 4) = make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
          fence_async_smem();
          asm volatile("bar.sync 1, 256;" ::: "memory");
          if (tid < SIM_M && gi < p.Nq) {
            const float* gdst = reinterpret_cast<const float*>(srow) + tile0 + hh * 64;
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 256;" ::"l"(gdst),
                         "r"(smem_u32(Stg + row * SIM_STG_ROW))
                         : "memory");
          }
          if (tid < SIM_M) asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          continue;
        }
        if (gi < p.Nq) {
          if (sizeof(T) == 4) {
            float* dst = reinterpret_cast<float*>(srow) + c0;
            if (c0 + 32 <= key1) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) *reinterpret_cast<uint4*>(dst + i) = make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            } else {
              for (int i = 0; i < 32; ++i)
                if (c0 + i < key1) dst[i] = __uint_as_float(v[i]);
            }
          } else {
            T* dst = srow + c0;
            if (c0 + 32 <= key1) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 w;
                w.x = pack2<T>(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                w.y = pack2<T>(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                w.z = pack2<T>(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
                w.w = pack2<T>(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
                *reinterpret_cast<uint4*>(dst + i) = w;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (c0 + i < key1) dst[i] = from_f32<T>(__uint_as_float(v[i]));
            }
          }
        }
      }
    }
  }
  if (!issuer && tid < SIM_M) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  if (failed) atomicOr(p.status, 1u);
  fence_before_sync();
  __syncthreads();
  if (issuer) tmem_dealloc(tmem, 256);
}

// ---- host side ---------------------------------------------------------------------------------
bool sim_fwd_tc_supported(const PopeSimArgs& a) {
  const PopeShape& s = a.shape;
  if (s.d % 8 != 0 || s.r % 8 != 0 || (s.d + s.r) % 16 != 0) return false;
  const int kd = s.d + s.r;
  const size_t opb = (size_t)(kd / 8) * SIM_CS * (s.dtype == POPE_F32 ? 2 : 1);
  if (2 * opb + 4096 > 227 * 1024) return false;
  if (s.r > 0 && (a.embed.sf.b != 0 || a.embed.sf.h != 0)) return false;
  if (s.r > 256) return false;
  const int esz = s.dtype == POPE_F32 ? 4 : 2;
  const int align_elems = 16 / esz;
  auto ok = [&](const void* ptr, const PopeStride3& st) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && st.b % align_elems == 0 && st.h % align_elems == 0 &&
           st.n % align_elems == 0;
  };
  if (!ok(a.q, a.sq) || !ok(a.k, a.sk) || !ok(a.sim, a.ss)) return false;
  return true;
}

size_t sim_fwd_tc_workspace(const PopeSimArgs& a) {
  return (size_t)a.shape.Nk * a.shape.r * 2 * sizeof(float) + 16;
}

template <typename T, bool SPLIT>
static cudaError_t launch_sim_tc(const PopeSimArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  TcSimP p = {};
  p.H = s.H, p.Hk = s.Hk, p.Nq = s.Nq, p.Nk = s.Nk, p.d = s.d, p.r = s.r;
  p.q = a.q, p.k = a.k, p.sim = a.sim, p.sq = a.sq, p.sk = a.sk, p.ss = a.ss;
  float* ctab = reinterpret_cast<float*>(a.workspace);
  float* stab = ctab + (size_t)s.Nk * s.r;
  p.ctab = ctab, p.stab = stab, p.bias = a.embed.bias, p.bias_sh = a.embed.bias_stride_h;
  p.status = tc_status_ptr();
  if (!p.status) return cudaErrorInvalidSymbol;
  if (s.r > 0) {
    const int64_t n = (int64_t)s.Nk * s.r;
    pope_trig_table_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a.embed.freqs, a.embed.sf.n, s.Nk, s.r, ctab, stab, nullptr, nullptr);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  // split the keys until about two waves of CTAs exist (each CTA re-expands its 128 query rows)
  const int qblocks = (s.Nq + SIM_M - 1) / SIM_M;
  const int ktiles = (s.Nk + SIM_N - 1) / SIM_N;
  const int64_t base_ctas = (int64_t)qblocks * s.B * s.H;
  int splits = (int)((2 * 148 + base_ctas - 1) / base_ctas);
  if (splits > ktiles) splits = ktiles;
  if (splits < 1) splits = 1;
  const int tiles_per_cta = (ktiles + splits - 1) / splits;
  p.keys_per_cta = tiles_per_cta * SIM_N;
  splits = (ktiles + tiles_per_cta - 1) / tiles_per_cta;
  const int kd = s.d + s.r;
  const size_t opb = (size_t)(kd / 8) * SIM_CS * (SPLIT ? 2 : 1);
  p.use_stg = (SPLIT && 2 * opb + SIM_STG + 4096 <= 227 * 1024) ? 1 : 0;
  const size_t stgb = p.use_stg ? SIM_STG : 0;
  const int nkb = (3 * opb + stgb + 4096 <= 227 * 1024) ? 2 : 1;
  size_t smem = opb * (1 + nkb) + stgb + 2 * 8 + 16 + 2 * 256 * 4 + 64;
  if (smem < 120 * 1024) smem = 120 * 1024;   // keep one CTA per SM: TMEM columns are allocated per CTA
  cudaError_t e = cudaFuncSetAttribute(sim_fwd_tc_kernel<T, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid(splits, qblocks, s.B * s.H);
  sim_fwd_tc_kernel<T, SPLIT><<<grid, SIM_THREADS, smem, st>>>(p);
  return cudaGetLastError();
}

cudaError_t sim_fwd_tc(const PopeSimArgs& a, cudaStream_t st) {
  switch (a.shape.dtype) {
    case POPE_F32: return launch_sim_tc<float, true>(a, st);
    case POPE_BF16: return launch_sim_tc<__nv_bfloat16, false>(a, st);
    default: return launch_sim_tc<__half, false>(a, st);
  }
}

}  // namespace pope
