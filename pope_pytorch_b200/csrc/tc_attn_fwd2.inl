// Forward kernel with the resident Q' tile in TENSOR memory (included by tc_attn_fwd.cu).
//
// The kernel above is bound by shared-memory bandwidth: a 128x64x16 score product with both operands in shared memory
// reads 6 KB for 32 clocks of tensor time.  Here a CTA owns ONE 128-row tile whose expanded Q' sits in tensor memory
// ((d + r) / 2 columns) as the A operand of every score product, and the keys come 128 at a time:
//     S = Q' K'^T : 128x128x16 products, A from tensor memory, B = the K' tile in shared memory (4 KB per 64 clocks)
//     O += P V    : 128 x d x 16 products, A = P written over S in tensor memory, B = the V tile
// Tensor memory: Q' [0, 128), S / P double-buffered [128, 384), O [384, 512).  Shared memory holds nothing but two
// stages of (K' tile, V tile).  Two softmax threads share a query row (64 of the 128 scores each; they exchange their
// row maxima through shared memory), so that the softmax keeps the thread count it had for two row tiles.
namespace pope {

constexpr int F2_TK = 128;                         // keys per step
constexpr int F2_KLOAD_WARP = 8;                   // warp 8  : one lane issues the K' copies (one 128-row image tile per step)
constexpr int F2_S_WARP = 9;                       // warp 9  : one lane issues S = Q' K'^T; owns the TMEM allocation
constexpr int F2_PV_WARP = 10;                     // warp 10 : one lane issues O += P V
constexpr int F2_VLOAD_WARP = 11;                  // warp 11 : one lane issues the V boxes
constexpr int F2_THREADS = 32 * (F2_VLOAD_WARP + 1);
constexpr uint32_t F2_TS = 128, F2_TO = 384;       // first TMEM column of the S / P buffers and of O (Q' starts at 0)

#ifndef F2_VST_N
#define F2_VST_N 2
#endif
constexpr int F2_VST = F2_VST_N;                   // V stages (a V tile arrives as 16-byte-wide boxes and takes its time)
enum {
  F2_KFULL = 0,    // [2] K' tile landed (transaction bytes)
  F2_KFREE = 2,    // [2] tcgen05.commit: S(j) has completed, its K' buffer may be refilled
  F2_PVDONE = 4,   // [2] tcgen05.commit: O += P V of tile j has completed: S / P buffer j & 1 is free
  F2_SFULL = 6,    // [2] tcgen05.commit: the scores of tile j are in TMEM
  F2_PFULL = 8,    // [2] 8 softmax warps: the probabilities of tile j are in TMEM
  F2_QFULL = 10,   // 8 softmax warps: Q' is in TMEM
  F2_ODONE = 11,   // tcgen05.commit: the last O += P V has completed
  F2_VFULL = 12,   // [3] V tile landed in stage j % F2_VST (transaction bytes)
  F2_VFREE = 15,   // [3] tcgen05.commit: O += P V of tile j has completed: V stage j % F2_VST is free
  F2_COUNT = 18
};

template <int D, typename T>
__global__ void __launch_bounds__(F2_THREADS, 1) attn_fwd2_tc_kernel(TcFwdP p, const __grid_constant__ CUtensorMap tmap_v) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzled tiles sit on 1 KB boundaries
  // V tiles: D a multiple of 64 -> boxes of 64 features (128-byte rows, 128-byte swizzled); else 16-byte chunk columns
  constexpr bool VWIDE = D % 64 == 0;
  const int KD = D + p.r, KC = KD >> 3, KSTEPS = KD >> 4;
  const int KBUF = F2_TK * KD * 2;                  // one K' stage: [KD/8 chunks][128 keys][16 B]
  constexpr int VBUF = F2_TK * D * 2;               // one V stage:  [D/8 chunks][128 keys][16 B]
  constexpr int CSV = F2_TK * 16;                   // chunk stride of both
  uint8_t* Ks = smem;
  uint8_t* Vs = Ks + 2 * KBUF;
  float* xch = reinterpret_cast<float*>(Vs + F2_VST * VBUF);       // [2 step parities][2 halves][128 rows] row maxima
  float* lxch = xch;                                                 // [2 halves][128 rows] row sums (epilogue: xch is dead)
  uint64_t* bars = reinterpret_cast<uint64_t*>(xch + 2 * 2 * TQ);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + F2_COUNT + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int u = blockIdx.y, b = u / p.H, h = u % p.H, hk = h % p.Hk;
  const int i0 = (gridDim.x - 1 - blockIdx.x) * TQ;  // heavy (late) row blocks first
  int n_end = p.Nk;
  if (p.causal) n_end = min(n_end, min(i0 + TQ, p.Nq));
  const int T_tiles = (n_end + F2_TK - 1) / F2_TK;

  if (warp == F2_S_WARP) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[F2_KFULL + i], 1);
      mbar_init(&bars[F2_KFREE + i], 1), mbar_init(&bars[F2_PVDONE + i], 1);
      mbar_init(&bars[F2_SFULL + i], 1), mbar_init(&bars[F2_PFULL + i], FWD_SOFTMAX_WARPS);
    }
    for (int i = 0; i < F2_VST; ++i) mbar_init(&bars[F2_VFULL + i], 1), mbar_init(&bars[F2_VFREE + i], 1);
    mbar_init(&bars[F2_QFULL], FWD_SOFTMAX_WARPS);
    mbar_init(&bars[F2_ODONE], 1);
    mbar_init_fence();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  bool failed = false;

  if (warp == F2_KLOAD_WARP) {
    // =============================== copies: K' ==================================================
    // a 128-key stage is one 128-row image tile (the pre-pass interleaves pairs of its 64-row tiles): one bulk copy.
    // (Assembled from 2 x KD / 8 copies of 1 KB the stage took longer to arrive than the whole step should last.)
    if (lane == 0) {
      const uint8_t* kimg = p.kimg + (int64_t)(b * p.Hk + hk) * (int64_t)(image_tiles(p.Nk) / 2) * KBUF;
      int j = 0;
      for (; j < T_tiles; ++j) {
        const int buf = j & 1;
        if (j >= 2 && !failed) failed = !mbar_wait(&bars[F2_KFREE + buf], ((j - 2) >> 1) & 1, WAIT_LIMIT);
        if (failed) break;
#ifdef F2_EXP_NO_K
        if (j >= 2) { mbar_arrive(&bars[F2_KFULL + buf]); continue; }
#endif
        mbar_expect_tx(&bars[F2_KFULL + buf], KBUF);
        bulk_load(Ks + buf * KBUF, kimg + (int64_t)j * KBUF, KBUF, &bars[F2_KFULL + buf]);
      }
      if (failed) drain_copies(&bars[F2_KFULL], 2, j - 2, j);
    }
    __syncwarp();
  } else if (warp == F2_VLOAD_WARP) {
    // =============================== copies: V ===================================================
    if (lane == 0) {
      int j = 0;
      for (; j < T_tiles; ++j) {
        const int buf = j % F2_VST, n0 = j * F2_TK;
        if (j >= F2_VST && !failed) failed = !mbar_wait(&bars[F2_VFREE + buf], ((j - F2_VST) / F2_VST) & 1, WAIT_LIMIT);
        if (failed) { drain_copies(&bars[F2_VFULL], F2_VST, j - F2_VST, j); break; }
#ifdef F2_EXP_NO_V
        if (j >= 2) { mbar_arrive(&bars[F2_VFULL + buf]); continue; }
#endif
        mbar_expect_tx(&bars[F2_VFULL + buf], VBUF);
        if (VWIDE) {
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(Vs + buf * VBUF + c * (F2_TK * 128), &tmap_v, &bars[F2_VFULL + buf], c * 64, n0, hk, b);
        } else {
#pragma unroll
          for (int c = 0; c < D / 8; ++c) tma_load_4d(Vs + buf * VBUF + c * CSV, &tmap_v, &bars[F2_VFULL + buf], c * 8, n0, hk, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == F2_S_WARP) {
    // =============================== MMA issue: S = Q' K'^T ======================================
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc(TcFmt<T>::fmt, TQ, F2_TK, false, false);
      const uint32_t ks_addr = smem_u32(Ks);
      if (!mbar_wait(&bars[F2_QFULL], 0, WAIT_LIMIT)) failed = true;
      for (int j = 0; j < T_tiles && !failed; ++j) {
        const int buf = j & 1;
        failed = !mbar_wait(&bars[F2_KFULL + buf], (j >> 1) & 1, WAIT_LIMIT);
        // score buffer j & 1 still holds P(j-2) until PV(j-2) has read it
        if (j >= 2 && !failed) failed = !mbar_wait(&bars[F2_PVDONE + buf], ((j - 2) >> 1) & 1, WAIT_LIMIT);
        if (failed) break;
        fence_after_sync();
        const uint32_t d = tmem + F2_TS + buf * F2_TK;
        const uint64_t bd = smem_desc(ks_addr + buf * KBUF, CSV, 128);
        uint32_t blo = desc_lo(bd), at = tmem;
#pragma unroll 4
        for (int ks = 0; ks < KSTEPS; ++ks) {
          mma_ts_lh(d, at, blo, desc_hi(bd), idesc_s, ks > 0 ? 1u : 0u);
          at += 8, blo += (2 * CSV) >> 4;
        }
        mma_commit(&bars[F2_SFULL + buf]);
        mma_commit(&bars[F2_KFREE + buf]);
      }
    }
    __syncwarp();
  } else if (warp == F2_PV_WARP) {
    // =============================== MMA issue: O += P V =========================================
    if (lane == 0) {
      const uint32_t idesc_o = instr_desc(TcFmt<T>::fmt, TQ, D, false, true);
      const uint32_t vs_addr = smem_u32(Vs);
      for (int j = 0; j < T_tiles && !failed; ++j) {
        const int buf = j & 1;
        failed = !mbar_wait(&bars[F2_VFULL + j % F2_VST], (j / F2_VST) & 1, WAIT_LIMIT);
        if (!failed) failed = !mbar_wait(&bars[F2_PFULL + buf], (j >> 1) & 1, WAIT_LIMIT);
        if (failed) break;
        fence_after_sync();
        const uint32_t a = tmem + F2_TS + buf * F2_TK;
        // B = V, MN-major: wide boxes: 64-feature blocks 16 KB apart, 8-key groups 1 KB apart, 2 KB per 16 keys;
        // chunk columns: 8-feature chunks CSV apart, 8-key groups 128 bytes apart, 256 bytes per 16 keys
        const uint32_t vaddr = vs_addr + (j % F2_VST) * VBUF;
        const uint64_t bd = VWIDE ? smem_desc_sw128(vaddr, F2_TK * 128, 1024) : smem_desc(vaddr, 128, CSV);
        constexpr uint32_t kstep = VWIDE ? (2048 >> 4) : ((2 * 128) >> 4);
#pragma unroll
        for (int ks = 0; ks < F2_TK / 16; ++ks)   // P of keys [64 h, 64 h + 64) sits in the first 32 columns of half h
          mma_ts_lh(tmem + F2_TO, a + (ks >> 2) * 64 + (ks & 3) * 8, desc_lo(bd) + ks * kstep, desc_hi(bd), idesc_o,
                    (j > 0 || ks > 0) ? 1u : 0u);
        if (j == T_tiles - 1) mma_commit(&bars[F2_ODONE]);
        mma_commit(&bars[F2_PVDONE + buf]);
        mma_commit(&bars[F2_VFREE + j % F2_VST]);
      }
    }
    __syncwarp();
  } else {
    // =============================== softmax: two threads per query row ===========================
    const uint8_t* maskb = p.mask ? p.mask + b * p.msb : nullptr;
    const int rloc = tid & 127, half = tid >> 7;
    const int row = i0 + rloc;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const int pair_bar = 1 + (warp & 3);   // named barrier of the two warps that share 32 rows
    {
      // Q' into tensor memory: lane = row, 4 columns per 8-feature chunk; the two threads of a row take half of the
      // chunks each.  Read from the Q' image (for one chunk the lanes of a warp read 512 contiguous bytes).
      const int64_t QIMG = (int64_t)IMAGE_ROWS * KD * 2;
      const uint8_t* img = p.qimg + ((int64_t)u * (int64_t)image_tiles(p.Nq) + i0 / IMAGE_ROWS + (rloc >> 6)) * QIMG + (rloc & 63) * 16;
      for (int c = half; c < KC; c += 2) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(img + (int64_t)c * (IMAGE_ROWS * 16)));
        tmem_st4(tmem + lane_base + c * 4, v.x, v.y, v.z, v.w);
      }
      tmem_st_wait();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[F2_QFULL]);
    }
    float m_run = -CUDART_INF_F, l_run = 0.f;

    for (int j = 0; j < T_tiles; ++j) {
      const int buf = j & 1, n0 = j * F2_TK + half * 64;   // first key of this thread's 64 columns
      // key visibility of this half tile (key-padding mask, ragged end): one bit per key, the same for every row
      uint64_t vis = ~0ull;
      if (maskb || n0 + 64 > p.Nk) {
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
      if (!failed) failed = !mbar_wait(&bars[F2_SFULL + buf], (j >> 1) & 1, WAIT_LIMIT);
      fence_after_sync();
      const uint32_t s_addr = tmem + lane_base + F2_TS + buf * F2_TK + half * 64;
      uint32_t s0[32], s1[32];
      tmem_ld32(s_addr, s0);
      tmem_ld32(s_addr + 32, s1);
      tmem_ld_wait();
      // maximum of this thread's 64 scores (four independent chains), then of the row
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
      float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      xch[(buf * 2 + half) * TQ + rloc] = mx;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      mx = fmaxf(mx, xch[(buf * 2 + (1 - half)) * TQ + rloc]);
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
        // O was last written by PV(j-1); each of the two threads of a row rescales half of its columns
        if (!failed) failed = !mbar_wait(&bars[F2_PVDONE + (1 - buf)], ((j - 1) >> 1) & 1, WAIT_LIMIT);
        fence_after_sync();
        const uint32_t o_addr = tmem + lane_base + F2_TO + half * (D / 2);
#pragma unroll
        for (int c0 = 0; c0 < D / 2; c0 += 16) {
          uint32_t ov[16];
          tmem_ld16(o_addr + c0, ov);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tmem_st16(o_addr + c0, ov);
        }
        tmem_st_wait();
      }
      // P = 2^(s*c - m), written over this thread's scores (32 packed columns for its 64 scores)
      const float m_use = m_run == -CUDART_INF_F ? 0.f : m_run;
      float ls4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[32];
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
      if (lane == 0) mbar_arrive(&bars[F2_PFULL + buf]);
    }

    // ---- epilogue: O / l, LSE ---------------------------------------------------------------------
    lxch[half * TQ + rloc] = l_run;
    asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
    const float l_tot = l_run + lxch[(1 - half) * TQ + rloc];
    if (T_tiles > 0 && !failed) failed = !mbar_wait(&bars[F2_ODONE], 0, WAIT_LIMIT);
    fence_after_sync();
    const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
    const uint32_t o_addr = tmem + lane_base + F2_TO + half * (D / 2);
    T* orow = (T*)p.o + b * p.so.b + h * p.so.h + (int64_t)row * p.so.n + half * (D / 2);
#pragma unroll
    for (int c0 = 0; c0 < D / 2; c0 += 16) {
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
    if (half == 0 && row < p.Nq) p.lse[(int64_t)u * p.Nq + row] = l_tot > 0.f ? m_run * LN2 + logf(l_tot) : -CUDART_INF_F;
  }
  if (failed) atomicOr(&g_tc_status, 1u);
  fence_before_sync();
  __syncthreads();
  if (warp == F2_S_WARP) tmem_dealloc(tmem, 512);
}

template <int D, typename T>
static cudaError_t launch_fwd2_kernel(const PopeAttnArgs& a, const TcFwdP& p, cudaStream_t st) {
  const PopeShape& s = a.shape;
  const int KD = s.d + s.r;
  CUtensorMap tmap_v;
  const bool tm_ok = D % 64 == 0 ? make_wide_tmap(&tmap_v, a.v, s.dtype == POPE_BF16, s.d, s.Nk, s.Hk, s.B, a.sv.n, a.sv.h, a.sv.b, F2_TK)
                                 : make_chunk_tmap(&tmap_v, a.v, s.dtype == POPE_BF16, s.d, s.Nk, s.Hk, s.B, a.sv.n, a.sv.h, a.sv.b, F2_TK);
  if (!tm_ok) return cudaErrorNotSupported;
  size_t smem = 2 * (size_t)F2_TK * KD * 2 + F2_VST * (size_t)F2_TK * D * 2 + 4 * TQ * sizeof(float) + (F2_COUNT + 1) * 8 + 16 + 1024;
  // every CTA allocates all 512 TMEM columns: keep two CTAs from sharing an SM
  if (smem < 120 * 1024) smem = 120 * 1024;
  cudaError_t e = ensure_max_smem<attn_fwd2_tc_kernel<D, T>>();
  if (e != cudaSuccess) return e;
  dim3 grid((s.Nq + TQ - 1) / TQ, s.B * s.H);
  attn_fwd2_tc_kernel<D, T><<<grid, F2_THREADS, smem, st>>>(p, tmap_v);
  return cudaGetLastError();
}

}  // namespace pope
