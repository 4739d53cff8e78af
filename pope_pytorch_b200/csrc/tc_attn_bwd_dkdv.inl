// dk / dv kernel and the host-side launch of the tensor-core backward (included by tc_attn_bwd.cu).
namespace pope {

// mbarrier slots of the dk/dv kernel.  Q' tiles have three stages and dO tiles two: that is what fits beside the
// resident K' and V once P^T and dS^T live in TMEM, and the Q' tile is the one whose copy is needed first.
enum { KB_QFULL = 0,     // [3] Q' tile j (and its lse / delta rows) has landed in stage j % 3
       KB_GFULL = 3,     // [2] dO tile j has landed in stage j % 2
       KB_ACCQ = 5,      // [3] tcgen05.commit: dK' += dS^T Q' of tile j finished (slot j % 3): its Q' stage and the dS^T
                         //     columns are free
       KB_ACCG = 8,      // [2] tcgen05.commit: dV += P^T dO of tile j finished (slot j % 2): its dO stage and the P^T
                         //     columns are free
       KB_SDONE = 10,    // tcgen05.commit: S^T of the current tile is in TMEM
       KB_DPDONE = 11,   // tcgen05.commit: dP^T of the current tile is in TMEM (same columns as S^T)
       KB_CONS_S = 12,   // 8 warps: S^T copied to registers, dP^T may overwrite it
       KB_CONS_DP = 13,  // 8 warps: dP^T copied to registers, the next S^T may overwrite it
       KB_GRAD = 14,     // 8 warps: P^T and dS^T of the current tile are written to TMEM
       KB_RESIDENT = 15, // the resident K' and V tiles have landed
       KB_ISS_S = 16,    // [2] S^T of tile j has been ISSUED (slot j & 1): what another thread issues after this executes
                         //     behind it in the tensor pipe
       KB_ISS_DP = 18,   // [2] the same for dP^T of tile j
       KB_COUNT = 20 };
constexpr int KQ_NST = 3, KG_NST = 2;

template <int D, typename T, bool VW>
__global__ void __launch_bounds__(BWD_THREADS, 1) attn_bwd_dkdv_tc_kernel(TcBwdP p, const __grid_constant__ CUtensorMap tmap_v,
                                                                          const __grid_constant__ CUtensorMap tmap_g,
                                                                          const __grid_constant__ CUtensorMap tmap_kimg) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzled tiles sit on 1 KB boundaries
  const int KD = D + p.r, KSTEPS = KD >> 4;
  uint8_t* Ks = smem;                          // [KD/8][128][16 B]  resident K' (phase fk + bias)
  uint8_t* Vs = Ks + BQ * KD * 2;              // [D/8][128][16 B]   resident V
  const int KBUF = (KD / 8) * BCS, VBUF = (D / 8) * BCS;  // one streamed buffer
  uint8_t* Qb = Vs + BQ * D * 2;               // 3 x [KD/8][64][16 B] streamed Q'
  uint8_t* Gb = Qb + KQ_NST * KBUF;            // 2 x [D/8][64][16 B]  streamed dO
  float* rowstat = reinterpret_cast<float*>(Gb + KG_NST * VBUF);  // 3 x (64 lse*log2e, 64 delta), with the Q' stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(rowstat + KQ_NST * 128);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + KB_COUNT + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int u = blockIdx.y, b = u / p.Hk, hk = u % p.Hk;
  const int j0 = blockIdx.x * BQ;
  const int groups = p.H / p.Hk;

  if (warp == BWD_M_WARP) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    for (int i = 0; i < KQ_NST; ++i) mbar_init(&bars[KB_QFULL + i], 1), mbar_init(&bars[KB_ACCQ + i], 1);
    for (int i = 0; i < KG_NST; ++i) mbar_init(&bars[KB_GFULL + i], 1), mbar_init(&bars[KB_ACCG + i], 1);
    mbar_init(&bars[KB_SDONE], 1), mbar_init(&bars[KB_DPDONE], 1);
    mbar_init(&bars[KB_CONS_S], BWD_E_WARPS), mbar_init(&bars[KB_CONS_DP], BWD_E_WARPS), mbar_init(&bars[KB_GRAD], BWD_E_WARPS);
    mbar_init(&bars[KB_RESIDENT], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&bars[KB_ISS_S + i], 1), mbar_init(&bars[KB_ISS_DP + i], 1);
    mbar_init_fence();
  }
  // query tiles: under the causal mask rows i < j0 see none of this CTA's keys
  const int m_begin = p.causal ? (j0 / BT) * BT : 0;
  const int tiles_per_group = m_begin < p.Nq ? (p.Nq - m_begin + BT - 1) / BT : 0;
  const int T_tiles = tiles_per_group * groups;
  // tile j -> (query head of the group, first query row); rotated per CTA like the dq kernel's key order
  const int rot = tiles_per_group > 0 ? (u * 5 + blockIdx.x * 3) % tiles_per_group : 0;
  auto tile_head = [&](int j) { return (j / tiles_per_group) * p.Hk + hk; };
  auto tile_start = [&](int j) {
    int t = j % tiles_per_group + rot;
    if (t >= tiles_per_group) t -= tiles_per_group;
    return m_begin + t * BT;
  };
  bool failed = false;
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  // TMEM columns: S^T, then dP^T [0,64); P^T (16-bit pairs) [64,96); dS^T (16-bit pairs) [96,128); dV [128,128+D);
  // dK' [256,256+KD).  S^T and dP^T share their columns: dP^T is issued once the elementwise warps hold S^T in
  // registers, which frees 64 columns for P^T / dS^T as TMEM-resident A operands of the accumulation products.
  constexpr uint32_t TK_SD = 0, TK_P = 64, TK_DS = 96, TK_DV = 128, TK_DK = 256;

  if (warp == BWD_L_WARP) {
    // =============================== copies: resident K' / V, then Q' and dO image tiles ==========
    {   // resident K' (phase bias folded in) and V: two image tiles each, one 1 KB copy per chunk column and 64 rows
      const int64_t t0 = (int64_t)u * (int64_t)image_tiles(p.Nk) + j0 / BT;
      if (T_tiles > 0) {   // (a CTA without any visible query row would leave with these copies in flight)
        if (lane == 0) mbar_expect_tx(&bars[KB_RESIDENT], BQ * KD * 2 + BQ * D * 2);
        __syncwarp();
        if (p.img_maps) {
          if (lane == 31) tma_load_4d(Ks, &tmap_kimg, &bars[KB_RESIDENT], 0, (int)t0, 0, 0);
        } else {
          copy_resident_tiles(Ks, p.kimg + t0 * KBUF, KD / 8, &bars[KB_RESIDENT], lane);
        }
        if (!VW) copy_resident_tiles(Vs, p.vimg + t0 * VBUF, D / 8, &bars[KB_RESIDENT], lane);
        else if (lane < D / 64) tma_load_4d(Vs + lane * (BQ * 128), &tmap_v, &bars[KB_RESIDENT], lane * 64, j0, hk, b);
      }
    }
    if (lane == 0) {
      const int64_t qtiles = (int64_t)image_tiles(p.Nq);
      for (int j = 0; j < T_tiles; ++j) {
        const int sq = j % KQ_NST, sg = j % KG_NST, m0 = tile_start(j), h = tile_head(j);
        const int64_t t = (int64_t)(b * p.H + h) * qtiles + m0 / BT;
        if (j >= KQ_NST && !failed) failed = !mbar_wait(&bars[KB_ACCQ + sq], ((j - KQ_NST) / KQ_NST) & 1, WAIT_LIMIT);
        if (failed) { drain_copies(&bars[KB_QFULL], KQ_NST, j - KQ_NST, j), drain_copies(&bars[KB_GFULL], KG_NST, j - KG_NST, j); break; }
        mbar_expect_tx(&bars[KB_QFULL + sq], KBUF + 2 * BT * 4);
        bulk_load(Qb + sq * KBUF, p.qimg + t * KBUF, KBUF, &bars[KB_QFULL + sq]);
        bulk_load(rowstat + sq * 128, p.rowstat + t * 128, 2 * BT * 4, &bars[KB_QFULL + sq]);
        if (j >= KG_NST && !failed) failed = !mbar_wait(&bars[KB_ACCG + sg], ((j - KG_NST) / KG_NST) & 1, WAIT_LIMIT);
        if (failed) { drain_copies(&bars[KB_QFULL], KQ_NST, j + 1 - KQ_NST, j + 1), drain_copies(&bars[KB_GFULL], KG_NST, j - KG_NST, j); break; }
        mbar_expect_tx(&bars[KB_GFULL + sg], VBUF);
        if (VW) {
#pragma unroll
          for (int c = 0; c < D / 64; ++c) tma_load_4d(Gb + sg * VBUF + c * (BT * 128), &tmap_g, &bars[KB_GFULL + sg], c * 64, m0, h, b);
        } else {
          bulk_load(Gb + sg * VBUF, p.gimg + t * VBUF, VBUF, &bars[KB_GFULL + sg]);
        }
      }
      if (failed) atomicOr(p.status, 1u);
    }
    __syncwarp();
  } else if (warp == BWD_M_WARP) {
    // =============================== MMA issue: the score chain  S^T(j), dP^T(j) =================
    // Two issuing threads.  One thread that issued everything was busy all the time (about 2200 clocks of issue and
    // 1000 clocks of barrier checks per tile of 3400) and the elementwise warps waited for it.  This thread issues the
    // critical chain S^T(j) -> dP^T(j); the second one issues the accumulation products of tile j - 1, each only after
    // it has seen the ISSUED barrier of the score product behind which it should run in the tensor pipe, which keeps the
    // order  S^T(j) | dV(j-1) | dP^T(j) | dK'(j-1)  (issued freely from a second thread, the accumulation products ran
    // ahead of S^T(j) and delayed the chain).
    if (lane == 0 && T_tiles > 0) {
      const uint32_t idesc_s = instr_desc(TcFmt<T>::fmt, BQ, BT, false, false);
      const uint32_t ks_addr = smem_u32(Ks), vs_addr = smem_u32(Vs), qb_addr = smem_u32(Qb), gb_addr = smem_u32(Gb);
      // V and the dO tiles: image layout (chunk columns) or 128-byte swizzled boxes (64-feature blocks, 32 bytes per k-step)
      const uint64_t ka = smem_desc(ks_addr, BQ * 16, 128);
      const uint64_t va = VW ? smem_desc_sw128(vs_addr, 16, 1024) : smem_desc(vs_addr, BQ * 16, 128);
      if (!mbar_wait(&bars[KB_RESIDENT], 0, WAIT_LIMIT)) failed = true;
      for (int j = 0; j < T_tiles && !failed; ++j) {
        const int sq = j % KQ_NST, sg = j % KG_NST;
        failed = !mbar_wait(&bars[KB_QFULL + sq], (j / KQ_NST) & 1, WAIT_LIMIT);
        // the elementwise warps hold dP^T of the previous tile in registers
        if (j >= 1 && !failed) failed = !mbar_wait(&bars[KB_CONS_DP], (j - 1) & 1, WAIT_LIMIT);
        fence_after_sync();
        {
          const uint64_t qb = smem_desc(qb_addr + sq * KBUF, BCS, 128);
          uint32_t alo = desc_lo(ka), blo = desc_lo(qb);
          mma_ss_lh(tmem + TK_SD, alo, desc_hi(ka), blo, desc_hi(qb), idesc_s, 0u);
#pragma unroll 4
          for (int ks = 1; ks < KSTEPS; ++ks) {
            alo += (2 * BQ * 16) >> 4, blo += (2 * BCS) >> 4;
            mma_ss_lh(tmem + TK_SD, alo, desc_hi(ka), blo, desc_hi(qb), idesc_s, 1u);
          }
          mma_commit(&bars[KB_SDONE]);
          mbar_arrive(&bars[KB_ISS_S + (j & 1)]);
        }
        if (!failed) failed = !mbar_wait(&bars[KB_GFULL + sg], (j / KG_NST) & 1, WAIT_LIMIT);
        // ... and S^T of this tile
        if (!failed) failed = !mbar_wait(&bars[KB_CONS_S], j & 1, WAIT_LIMIT);
        fence_after_sync();
        {
          const uint64_t gb = VW ? smem_desc_sw128(gb_addr + sg * VBUF, 16, 1024) : smem_desc(gb_addr + sg * VBUF, BCS, 128);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t aoff = VW ? (uint32_t)(((ks >> 2) * (BQ * 128) + (ks & 3) * 32) >> 4) : (uint32_t)(ks * ((2 * BQ * 16) >> 4));
            const uint32_t boff = VW ? (uint32_t)(((ks >> 2) * (BT * 128) + (ks & 3) * 32) >> 4) : (uint32_t)(ks * ((2 * BCS) >> 4));
            mma_ss_lh(tmem + TK_SD, desc_lo(va) + aoff, desc_hi(va), desc_lo(gb) + boff, desc_hi(gb), idesc_s, ks > 0);
          }
          mma_commit(&bars[KB_DPDONE]);
          mbar_arrive(&bars[KB_ISS_DP + (j & 1)]);
        }
      }
      if (failed) atomicOr(p.status, 1u);
    }
    __syncwarp();
  } else if (warp == BWD_A_WARP) {
    // =============================== MMA issue: the accumulation products  dV(j-1), dK'(j-1) =====
    if (lane == 0 && T_tiles > 0) {
      const uint32_t idesc_v = instr_desc(TcFmt<T>::fmt, BQ, D, false, true);
      const uint32_t idesc_k = instr_desc(TcFmt<T>::fmt, BQ, KD, false, true);
      const uint32_t qb_addr = smem_u32(Qb), gb_addr = smem_u32(Gb);
      for (int j = 1; j <= T_tiles && !failed; ++j) {
        const int pq = (j - 1) % KQ_NST, pg = (j - 1) % KG_NST;
        // dV += P^T dO of tile j-1 (P^T from TMEM; the dO tile re-described as an MN-major B operand)
        failed = !mbar_wait(&bars[KB_GRAD], (j - 1) & 1, WAIT_LIMIT);
        if (j < T_tiles && !failed) failed = !mbar_wait(&bars[KB_ISS_S + (j & 1)], (j >> 1) & 1, WAIT_LIMIT);
        fence_after_sync();
        {
          // the dO tile re-described as an MN-major B operand (boxes: 64-feature blocks 8 KB apart, 8-row groups 1 KB
          // apart, 2 KB per 16 query rows)
          const uint64_t gd = VW ? smem_desc_sw128(gb_addr + pg * VBUF, BT * 128, 1024) : smem_desc(gb_addr + pg * VBUF, 128, BCS);
          constexpr uint32_t gstep = VW ? (2048 >> 4) : ((2 * 128) >> 4);
#pragma unroll
          for (int ks = 0; ks < BT / 16; ++ks)
            mma_ts_lh(tmem + TK_DV, tmem + TK_P + ks * 8, desc_lo(gd) + ks * gstep, desc_hi(gd), idesc_v,
                      (j > 1 || ks > 0) ? 1u : 0u);
          mma_commit(&bars[KB_ACCG + pg]);
        }
        // dK' += dS^T Q' of tile j-1
        if (j < T_tiles && !failed) failed = !mbar_wait(&bars[KB_ISS_DP + (j & 1)], (j >> 1) & 1, WAIT_LIMIT);
        {
          const uint64_t qd = smem_desc(qb_addr + pq * KBUF, 128, BCS);
#pragma unroll
          for (int ks = 0; ks < BT / 16; ++ks)
            mma_ts_lh(tmem + TK_DK, tmem + TK_DS + ks * 8, desc_lo(qd) + ks * ((2 * 128) >> 4), desc_hi(qd), idesc_k,
                      (j > 1 || ks > 0) ? 1u : 0u);
          mma_commit(&bars[KB_ACCQ + pq]);
        }
      }
      if (failed) atomicOr(p.status, 1u);
    }
    __syncwarp();
  }
  if (warp >= BWD_E_WARPS) {
    fence_before_sync();
    __syncthreads();
    if (warp == BWD_M_WARP) tmem_dealloc(tmem, 512);
    return;
  }

  // =============================== elementwise warps ================================================
  const uint8_t* maskb = p.mask ? p.mask + b * p.msb : nullptr;

  const int row = tid & 127, half = tid >> 7;          // thread = (key row, 32-query half)
  const int gj = j0 + row;
  const bool key_ok = gj < p.Nk && (!maskb || maskb[(int64_t)gj * p.msn] != 0);
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  for (int j = 0; j < T_tiles; ++j) {
    const int sq = j % KQ_NST;
    const int m0 = tile_start(j);
    if (!failed) failed = !mbar_wait(&bars[KB_QFULL + sq], (j / KQ_NST) & 1, WAIT_LIMIT);   // orders the lse / delta read
    if (!failed) failed = !mbar_wait(&bars[KB_SDONE], j & 1, WAIT_LIMIT);
    fence_after_sync();
    const float* st = rowstat + sq * 128 + half * 32;
    // interior tile for this warp: every key row valid and (causal) every key at or before every query column;
    // out-of-range queries and rows without any visible key carry lse = +inf, which makes P exactly 0
    const int gj_hi = j0 + (warp & 3) * 32 + 31, gi_lo = m0 + half * 32;
    const bool interior = __all_sync(0xffffffffu, key_ok) && (!p.causal || gj_hi <= gi_lo);
    uint32_t sv[32];
    tmem_ld32(tmem + lane_base + TK_SD + half * 32, sv);
    tmem_ld_wait();
    // S^T of this tile is in registers: dP^T may overwrite it
    fence_before_sync();
    warp_arrive(&bars[KB_CONS_S], lane);
    uint32_t pw[16];   // P^T of this thread's 32 query columns, packed in pairs; the fp32 values stay in sv
    // two copies of the loop: interior tiles (the common case) carry no masking arithmetic at all
    auto probabilities = [&](auto masked) {
#pragma unroll
      for (int c4 = 0; c4 < 8; ++c4) {
        const float4 l4 = *reinterpret_cast<const float4*>(st + c4 * 4);
        const float l2v[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int cl = c4 * 4 + t;   // query column within the thread's half
          float pr = ex2_approx(fmaf(__uint_as_float(sv[cl]), p.scale_log2, -l2v[t]));
          if (decltype(masked)::value) pr = (key_ok && (!p.causal || gj <= gi_lo + cl)) ? pr : 0.f;
          sv[cl] = __float_as_uint(pr);
        }
        pw[c4 * 2] = pack2<T>(__uint_as_float(sv[c4 * 4]), __uint_as_float(sv[c4 * 4 + 1]));
        pw[c4 * 2 + 1] = pack2<T>(__uint_as_float(sv[c4 * 4 + 2]), __uint_as_float(sv[c4 * 4 + 3]));
      }
    };
    if (interior) probabilities(std::false_type());
    else probabilities(std::true_type());
    // dP^T first: the next S^T waits for these columns, and that wait heads the longest chain of the step; P^T is
    // stored after it (its consumer, dV of this tile, is issued only once dS^T is stored as well).  Storing P^T before
    // this load cost 2.5 % of the backward; loading dP^T before or in the middle of the probability arithmetic is
    // slower again (dP^T is not complete any earlier).
    if (!failed) failed = !mbar_wait(&bars[KB_DPDONE], j & 1, WAIT_LIMIT);
    fence_after_sync();
    uint32_t dv[32];
    tmem_ld32(tmem + lane_base + TK_SD + half * 32, dv);
    tmem_ld_wait();
    // dP^T of this tile is in registers: the next S^T may overwrite it
    fence_before_sync();
    warp_arrive(&bars[KB_CONS_DP], lane);
    // the P^T columns were read by dV += P^T dO of tile j-1
    if (j >= 1 && !failed) failed = !mbar_wait(&bars[KB_ACCG + (j - 1) % KG_NST], ((j - 1) / KG_NST) & 1, WAIT_LIMIT);
    tmem_st16(tmem + lane_base + TK_P + half * 16, pw);
    uint32_t dw[16];
#pragma unroll
    for (int c4 = 0; c4 < 8; ++c4) {
      const float4 d4 = *reinterpret_cast<const float4*>(st + 64 + c4 * 4);
      const float dlv[4] = {d4.x, d4.y, d4.z, d4.w};
      float ds[4];
#pragma unroll
      for (int t = 0; t < 4; ++t)
        ds[t] = __uint_as_float(sv[c4 * 4 + t]) * (__uint_as_float(dv[c4 * 4 + t]) - dlv[t]) * p.scale;
      dw[c4 * 2] = pack2<T>(ds[0], ds[1]);
      dw[c4 * 2 + 1] = pack2<T>(ds[2], ds[3]);
    }
    // the dS^T columns were read by dK' += dS^T Q' of tile j-1
    if (j >= 1 && !failed) failed = !mbar_wait(&bars[KB_ACCQ + (j - 1) % KQ_NST], ((j - 1) / KQ_NST) & 1, WAIT_LIMIT);
    tmem_st16(tmem + lane_base + TK_DS + half * 16, dw);
    tmem_st_wait();
    fence_before_sync();
    warp_arrive(&bars[KB_GRAD], lane);
  }

  // ---- epilogue ---------------------------------------------------------------------------------
  if (T_tiles > 0 && !failed)
    failed = !mbar_wait(&bars[KB_ACCG + (T_tiles - 1) % KG_NST], ((T_tiles - 1) / KG_NST) & 1, WAIT_LIMIT) ||
             !mbar_wait(&bars[KB_ACCQ + (T_tiles - 1) % KQ_NST], ((T_tiles - 1) / KQ_NST) & 1, WAIT_LIMIT);
  fence_after_sync();
  asm volatile("bar.sync 1, 256;" ::: "memory");   // every MMA is done: the streamed buffers can be reused
  // Everything below reuses dead shared memory behind the resident K' tile (V and the streamed buffers): row-major
  // staging tiles of dk and dv, so that both leave in fully coalesced 16-byte pieces, and the per-row key-phase
  // gradients (feature-major, [r][128 rows] fp32) for the bias gradient.
  // Everything the chain rule needs is in the resident K' tile: with kc = a cos(f + b), ks = a sin(f + b)
  // (a = softplus(k)),   a = sqrt(kc^2 + ks^2),  sigmoid(k) = 1 - exp(-a),
  //   dk = (dKc kc + dKs ks) / a * sigmoid(k),   dphase = a (dKs cos - dKc sin) = dKs kc - dKc ks,
  // so the epilogue reads neither k nor the phase tables from global memory.  The 16-bit rounding of K' costs the
  // cosine a relative 2^-8 sin^2 at most.  Rows past Nk are zero in the image and produce zeros.
  constexpr int OSTR = D * 2 + 16;             // bytes of a staged output row (16 bytes of padding: conflict-free)
  uint8_t* dk_stage = Vs;
  uint8_t* dv_stage = Vs + BQ * OSTR;
  float* dmat = reinterpret_cast<float*>(Vs + 2 * BQ * OSTR);   // [128 rows][r + 1]: a thread writes its row, the column sums
  const int DSTR = p.r + 1;                                     // read along a row; the odd stride keeps both off bank conflicts
  {
    constexpr int HW = D / 2;
    const uint32_t accv = tmem + lane_base + TK_DV, acck = tmem + lane_base + TK_DK;
    float* dfrow = p.dfreqs ? p.dfreqs + b * p.sdf.b + hk * p.sdf.h + (int64_t)gj * p.sdf.n : nullptr;
    const bool live = gj < p.Nk;
#pragma unroll
    for (int c0 = 0; c0 < HW; c0 += 16) {
      const int cbase = half * HW + c0;
      uint32_t gv[16], gc[16], gs[16];
      const bool rot = cbase < p.r && T_tiles > 0;
      if (T_tiles > 0) {
        tmem_ld16(accv + cbase, gv);
        tmem_ld16(acck + cbase, gc);
        if (rot) tmem_ld16(acck + D + cbase, gs);
        tmem_ld_wait();
      } else {   // no visible query row: zero gradients (the resident tiles were never loaded)
#pragma unroll
        for (int e = 0; e < 16; ++e) gv[e] = gc[e] = gs[e] = 0u;
      }
      uint32_t wv[8], wk[8];
#pragma unroll
      for (int e = 0; e < 16; e += 2) wv[e >> 1] = pack2<T>(__uint_as_float(gv[e]), __uint_as_float(gv[e + 1]));
      if (rot) {
        uint32_t cw[8], sw[8];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint4 kcw = *reinterpret_cast<const uint4*>(Ks + (cbase / 8 + i) * (BQ * 16) + row * 16);
          const uint4 ksw = *reinterpret_cast<const uint4*>(Ks + (D / 8 + cbase / 8 + i) * (BQ * 16) + row * 16);
          cw[4 * i] = kcw.x, cw[4 * i + 1] = kcw.y, cw[4 * i + 2] = kcw.z, cw[4 * i + 3] = kcw.w;
          sw[4 * i] = ksw.x, sw[4 * i + 1] = ksw.y, sw[4 * i + 2] = ksw.z, sw[4 * i + 3] = ksw.w;
        }
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const float2 kc = unpack2<T>(cw[e >> 1]), ks = unpack2<T>(sw[e >> 1]);
          const float g0 = __uint_as_float(gc[e]), g1 = __uint_as_float(gc[e + 1]);
          const float h0 = __uint_as_float(gs[e]), h1 = __uint_as_float(gs[e + 1]);
          const float m0 = kc.x * kc.x + ks.x * ks.x, m1 = kc.y * kc.y + ks.y * ks.y;   // a^2
          const float r0 = m0 > 0.f ? rsqrtf(m0) : 0.f, r1 = m1 > 0.f ? rsqrtf(m1) : 0.f;
          const float sg0 = 1.f - ex2_approx(-m0 * r0 * LOG2E), sg1 = 1.f - ex2_approx(-m1 * r1 * LOG2E);
          const float d0 = h0 * kc.x - g0 * ks.x, d1 = h1 * kc.y - g1 * ks.y;
          if (dfrow && live) atomicAdd(dfrow + cbase + e, d0), atomicAdd(dfrow + cbase + e + 1, d1);
          if (p.dbias) dmat[row * DSTR + cbase + e] = d0, dmat[row * DSTR + cbase + e + 1] = d1;
          wk[e >> 1] = pack2<T>((g0 * kc.x + h0 * ks.x) * r0 * sg0, (g1 * kc.y + h1 * ks.y) * r1 * sg1);
        }
      } else {
        if (p.dbias && cbase < p.r) {
#pragma unroll
          for (int e = 0; e < 16; ++e) dmat[row * DSTR + cbase + e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < 16; e += 2) wk[e >> 1] = pack2<T>(__uint_as_float(gc[e]), __uint_as_float(gc[e + 1]));
      }
      *reinterpret_cast<uint4*>(dv_stage + row * OSTR + cbase * 2) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
      *reinterpret_cast<uint4*>(dv_stage + row * OSTR + cbase * 2 + 16) = make_uint4(wv[4], wv[5], wv[6], wv[7]);
      *reinterpret_cast<uint4*>(dk_stage + row * OSTR + cbase * 2) = make_uint4(wk[0], wk[1], wk[2], wk[3]);
      *reinterpret_cast<uint4*>(dk_stage + row * OSTR + cbase * 2 + 16) = make_uint4(wk[4], wk[5], wk[6], wk[7]);
    }
  }
  asm volatile("bar.sync 1, 256;" ::: "memory");
  {
    // dk / dv rows leave 16 bytes per thread: consecutive threads cover one 2 D-byte row after the other
    constexpr int GPR = D / 8;   // 16-byte groups per row
    T* dkbase = (T*)p.dk + b * p.sdk.b + hk * p.sdk.h;
    T* dvbase = (T*)p.dv + b * p.sdv.b + hk * p.sdv.h;
    for (int idx = tid; idx < BQ * GPR; idx += 256) {
      const int rr = idx / GPR, g = idx - rr * GPR;
      if (j0 + rr < p.Nk) {
        *reinterpret_cast<uint4*>(dkbase + (int64_t)(j0 + rr) * p.sdk.n + g * 8) = *reinterpret_cast<const uint4*>(dk_stage + rr * OSTR + g * 16);
        *reinterpret_cast<uint4*>(dvbase + (int64_t)(j0 + rr) * p.sdv.n + g * 8) = *reinterpret_cast<const uint4*>(dv_stage + rr * OSTR + g * 16);
      }
    }
    if (p.dbias) {
      // column sums of the key-phase gradient: a thread per (feature, half of the rows), four running sums
      // (one warp per feature with a shuffle reduction took 4800 clocks of this epilogue; this takes a sixth)
      const int c = tid & 127, r0 = (tid >> 7) * (BQ / 2);
      if (c < p.r) {
        const float* col = dmat + r0 * DSTR + c;
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int rr = 0; rr < BQ / 2; rr += 4) {
          s4[0] += col[rr * DSTR], s4[1] += col[(rr + 1) * DSTR], s4[2] += col[(rr + 2) * DSTR], s4[3] += col[(rr + 3) * DSTR];
        }
        atomicAdd(p.dbias + hk * p.dbias_sh + c, (s4[0] + s4[1]) + (s4[2] + s4[3]));
      }
    }
  }
  if (failed) atomicOr(p.status, 1u);
  fence_before_sync();
  __syncthreads();   // the issuing warp frees the tensor memory after this barrier
}

// ---- host side -----------------------------------------------------------------------------------
static bool bwd_aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; }
static bool bwd_stride_ok(const PopeStride3& s) { return s.b % 8 == 0 && s.h % 8 == 0 && s.n % 8 == 0; }

bool attn_bwd_tc_supported(const PopeAttnBwdArgs& a) {
  const PopeShape& s = a.shape;
  if (s.dtype != POPE_BF16 && s.dtype != POPE_F16) return false;
  if (s.d != 64 && s.d != 96 && s.d != 128) return false;
  if (s.r % 16 != 0) return false;
  if (s.Nq < 64) return false;
  // a phase table with a head axis (b, h, n, r) serves queries and keys alike only when both have the same heads
  if (s.r > 0 && a.embed.sf.h != 0 && s.H != s.Hk) return false;
  if (a.dfreqs && a.sdf.h != 0 && s.H != s.Hk) return false;
  const void* ptrs[] = {a.q, a.k, a.v, a.out, a.dout, a.dq, a.dk, a.dv};
  for (const void* ptr : ptrs)
    if (!bwd_aligned16(ptr)) return false;
  const PopeStride3 strides[] = {a.sq, a.sk, a.sv, a.so, a.sdo, a.sdq, a.sdk, a.sdv};
  for (const PopeStride3& st : strides)
    if (!bwd_stride_ok(st)) return false;
  return true;
}

// Row statistics of the backward in one pass over out and dout: delta[u, i] = <out_i, dout_i>
// (PoPE_pytorch/triton_pope_flash_attn.py:119-130) as a plain (B*H, Nq) array for the dq kernel, and, in the order
// the dk/dv kernel consumes them, [unit][64-query tile][64 x lse * log2(e) | 64 x delta], padded to whole tiles so
// that one aligned 512-byte bulk copy brings a tile's rows.  Empty rows (lse = -inf) and rows past Nq carry +inf,
// which makes their probabilities exactly 0.  grid (tiles, units), 256 threads: four threads per row.
template <typename T>
__global__ void __launch_bounds__(256) bwd_rowstat_kernel(const T* __restrict__ out, Strides so, const T* __restrict__ dout,
                                                           Strides sdo, const float* __restrict__ lse, int H, int Nq, int d,
                                                           float* __restrict__ delta, float* __restrict__ rowstat) {
  const int tile = blockIdx.x, u = blockIdx.y, b = u / H, h = u % H;
  const int t = threadIdx.x >> 2, part = threadIdx.x & 3, i = tile * BT + t;
  float acc = 0.f;
  if (i < Nq) {
    const T* o = out + b * so.b + h * so.h + (int64_t)i * so.n;
    const T* g = dout + b * sdo.b + h * sdo.h + (int64_t)i * sdo.n;
    for (int c = part * 8; c < d; c += 32) {
      const uint4 ov = __ldg(reinterpret_cast<const uint4*>(o + c)), gv = __ldg(reinterpret_cast<const uint4*>(g + c));
      const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x = unpack2<T>(ow[e]), y = unpack2<T>(gw[e]);
        acc = fmaf(x.x, y.x, fmaf(x.y, y.y, acc));
      }
    }
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  if (part == 0) {
    const float l = i < Nq ? lse[(int64_t)u * Nq + i] : -CUDART_INF_F;
    float* rs = rowstat + ((int64_t)u * gridDim.x + tile) * (2 * BT);
    rs[t] = l == -CUDART_INF_F ? CUDART_INF_F : l * LOG2E;
    rs[BT + t] = i < Nq ? acc : 0.f;
    if (i < Nq) delta[(int64_t)u * Nq + i] = acc;
  }
}

// workspace: [delta][fp32 and fp16 cos / sin tables][K' images][Q' images][V images][dO images][row statistics], each
// rounded up to 256 bytes
static size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }
static size_t delta_bytes(const PopeShape& s) { return up256((size_t)s.B * s.H * s.Nq * sizeof(float)); }
static size_t bwd_table_bytes(const PopeShape& s, const PopeEmbed& e) { return trig_tables_bytes(s.Nk, s.r, table_slices(e, s.B, s.H)); }
static size_t rowstat_bytes(const PopeShape& s) { return up256((size_t)s.B * s.H * image_tiles(s.Nq) * 2 * BT * sizeof(float)); }

size_t attn_bwd_tc_workspace(const PopeAttnBwdArgs& a) {
  const PopeShape& s = a.shape;
  return delta_bytes(s) + bwd_table_bytes(s, a.embed) + up256(image_bytes(s.B * s.Hk, s.Nk, s.d + s.r)) +
         up256(image_bytes(s.B * s.H, s.Nq, s.d + s.r)) + up256(image_bytes(s.B * s.Hk, s.Nk, s.d)) +
         up256(image_bytes(s.B * s.H, s.Nq, s.d)) + rowstat_bytes(s);
}

// Side streams and fork / join events of the backward: a small pool per device, created on first use and kept for
// the life of the process.  A call borrows one slot for the time it ENQUEUES its work (the slot's mutex is never held
// while the GPU runs), so host threads that call the backward at the same time on one device do not wait for each
// other; when every slot is taken, or none could be created, both kernels simply run on the caller's stream.
struct BwdFork {
  cudaStream_t side = nullptr;
  cudaEvent_t begin = nullptr, stats = nullptr, ready = nullptr, done = nullptr;
  std::mutex busy;
  int state = 0;   // 0 = not tried, 1 = usable, -1 = unavailable
};
constexpr int kForkSlots = 4;
static BwdFork* bwd_fork_pool() {
  constexpr int kMaxDevices = 64;
  static BwdFork forks[kMaxDevices][kForkSlots];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  return forks[dev];
}
// Borrowed slot with the fork open: the destructor joins the side stream back into the caller's stream on EVERY
// path out of the launch function, error returns included, so the caller's stream always orders after whatever
// was enqueued on the side stream.
class ForkGuard {
 public:
  explicit ForkGuard(cudaStream_t st) : st_(st) {
    BwdFork* pool = bwd_fork_pool();
    for (int i = 0; pool && i < kForkSlots && !fk_; ++i) {
      std::unique_lock<std::mutex> lk(pool[i].busy, std::try_to_lock);
      if (!lk.owns_lock()) continue;
      BwdFork& f = pool[i];
      if (f.state == 0) {
        const bool ok = cudaStreamCreateWithFlags(&f.side, cudaStreamNonBlocking) == cudaSuccess &&
                        cudaEventCreateWithFlags(&f.begin, cudaEventDisableTiming) == cudaSuccess &&
                        cudaEventCreateWithFlags(&f.stats, cudaEventDisableTiming) == cudaSuccess &&
                        cudaEventCreateWithFlags(&f.ready, cudaEventDisableTiming) == cudaSuccess &&
                        cudaEventCreateWithFlags(&f.done, cudaEventDisableTiming) == cudaSuccess;
        f.state = ok ? 1 : -1;
      }
      if (f.state != 1) continue;
      if (cudaEventRecord(f.begin, st) != cudaSuccess || cudaStreamWaitEvent(f.side, f.begin, 0) != cudaSuccess) continue;
      fk_ = &f, lock_ = std::move(lk);
    }
  }
  ~ForkGuard() { join(); }
  bool forked() const { return fk_ != nullptr; }
  BwdFork* operator->() const { return fk_; }
  cudaStream_t side() const { return fk_ ? fk_->side : st_; }
  cudaError_t join() {
    if (!fk_) return cudaSuccess;
    cudaError_t e = cudaEventRecord(fk_->done, fk_->side);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(st_, fk_->done, 0);
    fk_ = nullptr;
    lock_.unlock();
    return e;
  }
 private:
  cudaStream_t st_;
  BwdFork* fk_ = nullptr;
  std::unique_lock<std::mutex> lock_;
};

template <int D, typename T, bool VW>
static cudaError_t launch_bwd_kernels(const TcBwdP& p, const PopeShape& s, size_t smem_q, size_t smem_k, const CUtensorMap& tv64,
                                      const CUtensorMap& tv128, const CUtensorMap& tg64, const CUtensorMap& tqi,
                                      const CUtensorMap& tki, cudaStream_t st, cudaStream_t sk) {
  cudaError_t e;
  if ((e = ensure_max_smem<attn_bwd_dq_tc_kernel<D, T, VW>>()) != cudaSuccess) return e;
  if ((e = ensure_max_smem<attn_bwd_dkdv_tc_kernel<D, T, VW>>()) != cudaSuccess) return e;
  attn_bwd_dq_tc_kernel<D, T, VW><<<dim3((s.Nq + BQ - 1) / BQ, s.B * s.H), BWD_THREADS, smem_q, st>>>(p, tv64, tqi);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  attn_bwd_dkdv_tc_kernel<D, T, VW><<<dim3((s.Nk + BQ - 1) / BQ, s.B * s.Hk), BWD_THREADS, smem_k, sk>>>(p, tv128, tg64, tki);
  return cudaGetLastError();
}

template <int D, typename T>
static cudaError_t launch_bwd_tc(const PopeAttnBwdArgs& a, cudaStream_t st) {
  const PopeShape& s = a.shape;
  const int KD = s.d + s.r;
  const bool bf16 = s.dtype == POPE_BF16;
  uint8_t* ws = reinterpret_cast<uint8_t*>(a.workspace);
  float* delta = reinterpret_cast<float*>(ws);
  const int slices = table_slices(a.embed, s.B, s.H), tab_heads = table_heads(a.embed, s.H), by_batch = a.embed.sf.b != 0;
  const TrigTables tt = trig_tables_at(ws + delta_bytes(s), s.Nk, s.r, slices);
  uint8_t* kimg = ws + delta_bytes(s) + bwd_table_bytes(s, a.embed);
  uint8_t* qimg = kimg + up256(image_bytes(s.B * s.Hk, s.Nk, KD));
  uint8_t* vimg = qimg + up256(image_bytes(s.B * s.H, s.Nq, KD));
  uint8_t* gimg = vimg + up256(image_bytes(s.B * s.Hk, s.Nk, s.d));
  float* rowstat = reinterpret_cast<float*>(gimg + up256(image_bytes(s.B * s.H, s.Nq, s.d)));
  cudaError_t e;
  // V and dO straight from the caller's tensors (tensor-map boxes of 64 features) when the head width is a multiple of
  // 64 and the tensors can be described; else re-laid image tiles from the pre-pass
  CUtensorMap tv64, tv128, tg64;
  memset(&tv64, 0, sizeof(tv64)), memset(&tv128, 0, sizeof(tv128)), memset(&tg64, 0, sizeof(tg64));
  const bool wide = D % 64 == 0 && make_wide_tmap(&tv64, a.v, bf16, s.d, s.Nk, s.Hk, s.B, a.sv.n, a.sv.h, a.sv.b, BT) &&
                    make_wide_tmap(&tv128, a.v, bf16, s.d, s.Nk, s.Hk, s.B, a.sv.n, a.sv.h, a.sv.b, BQ) &&
                    make_wide_tmap(&tg64, a.dout, bf16, s.d, s.Nq, s.H, s.B, a.sdo.n, a.sdo.h, a.sdo.b, BT);
  // Two independent strands run on two streams: a library-owned side stream forks from the caller's stream, takes the
  // row statistics while the caller's stream builds tables and images, and later the dk/dv kernel while the caller's
  // stream runs the dq kernel (its CTAs fill the SMs which the dq kernel's last partial wave leaves idle); the
  // caller's stream waits for it at the end.
  ForkGuard fk(st);
  const bool fork = fk.forked();
  cudaStream_t sk = fk.side();
  bwd_rowstat_kernel<T><<<dim3((unsigned)image_tiles(s.Nq), s.B * s.H), 256, 0, sk>>>(
      static_cast<const T*>(a.out), Strides(a.so), static_cast<const T*>(a.dout), Strides(a.sdo), a.lse, s.H, s.Nq, s.d, delta,
      rowstat);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  if (fork && (e = cudaEventRecord(fk->stats, sk)) != cudaSuccess) return e;
  if (s.r > 0 && (e = launch_trig_tables(a.embed, s.Nk, s.r, nullptr, nullptr, tt.ch, tt.sh, st, slices, tab_heads)) != cudaSuccess) return e;
  // K' (phase bias folded in), Q', and -- unless the kernels read them directly -- V / dO as the same tiles without
  // rotated features (a pure re-layout)
  ExpandJobs jobs;
  jobs.job[0] = expand_job(a.k, a.sk, s.B, s.Hk, s.Nk, s.r, 0, a.embed.bias, a.embed.bias_stride_h, kimg, s.Nk, by_batch, tab_heads);
  jobs.job[1] = expand_job(a.q, a.sq, s.B, s.H, s.Nq, s.r, s.Nk - s.Nq, nullptr, 0, qimg, s.Nk, by_batch, tab_heads);
  jobs.job[2] = expand_job(a.v, a.sv, s.B, s.Hk, s.Nk, 0, 0, nullptr, 0, vimg);
  jobs.job[3] = expand_job(a.dout, a.sdo, s.B, s.H, s.Nq, 0, 0, nullptr, 0, gimg);
  if ((e = launch_expand_images(jobs, wide ? 2 : 4, s.d, bf16, tt.ch, tt.sh, st, s.r > 0)) != cudaSuccess) return e;
  TcBwdP p = {};
  p.H = s.H, p.Hk = s.Hk, p.Nq = s.Nq, p.Nk = s.Nk, p.r = s.r, p.causal = a.causal;
  p.scale = a.softmax_scale, p.scale_log2 = a.softmax_scale * LOG2E;
  p.q = a.q, p.k = a.k, p.v = a.v, p.dout = a.dout, p.dq = a.dq, p.dk = a.dk, p.dv = a.dv;
  p.sq = a.sq, p.sk = a.sk, p.sv = a.sv, p.sdo = a.sdo, p.sdq = a.sdq, p.sdk = a.sdk, p.sdv = a.sdv, p.sdf = a.sdf;
  p.freqs = a.embed.freqs, p.bias = a.embed.bias, p.lse = a.lse, p.delta = delta;
  p.sfn = a.embed.sf.n, p.bias_sh = a.embed.bias_stride_h, p.dbias_sh = a.dbias_stride_h;
  p.kimg = kimg, p.qimg = qimg, p.vimg = vimg, p.gimg = gimg, p.rowstat = rowstat;
  p.mask = a.mask, p.msb = a.mask_stride_b, p.msn = a.mask_stride_n;
  p.dfreqs = s.r > 0 ? a.dfreqs : nullptr, p.dbias = s.r > 0 ? a.dbias : nullptr;
  p.status = tc_status_ptr();
  if (!p.status) return cudaErrorInvalidSymbol;
  CUtensorMap tqi, tki;
  memset(&tqi, 0, sizeof(tqi)), memset(&tki, 0, sizeof(tki));
  p.img_maps = make_image_tmap(&tqi, qimg, (int64_t)s.B * s.H * (int64_t)image_tiles(s.Nq), KD / 8) &&
               make_image_tmap(&tki, kimg, (int64_t)s.B * s.Hk * (int64_t)image_tiles(s.Nk), KD / 8);
  const size_t stage = (size_t)BT * KD * 2 + (size_t)BT * D * 2;
  size_t smem_q = (size_t)BQ * KD * 2 + DQ_NST * stage + (BB_COUNT + 1) * 8 + 16 + 1024;
  size_t smem_k = (size_t)BQ * KD * 2 + BQ * D * 2 + KQ_NST * (size_t)BT * KD * 2 + KG_NST * (size_t)BT * D * 2 + KQ_NST * 512 +
                  (KB_COUNT + 1) * 8 + 16 + 1024;   // 232.2 KB at d = r = 128 (1 KB of it to put the base on a 1 KB boundary)
  // every CTA allocates all 512 TMEM columns: keep two CTAs from sharing an SM
  if (smem_q < 120 * 1024) smem_q = 120 * 1024;
  if (smem_k < 120 * 1024) smem_k = 120 * 1024;
  if (fork) {   // images -> side stream (dk/dv); row statistics -> caller's stream (dq reads delta)
    if ((e = cudaEventRecord(fk->ready, st)) != cudaSuccess) return e;
    if ((e = cudaStreamWaitEvent(fk->side, fk->ready, 0)) != cudaSuccess) return e;
    if ((e = cudaStreamWaitEvent(st, fk->stats, 0)) != cudaSuccess) return e;
  }
  e = wide ? launch_bwd_kernels<D, T, (D % 64 == 0)>(p, s, smem_q, smem_k, tv64, tv128, tg64, tqi, tki, st, sk)
           : launch_bwd_kernels<D, T, false>(p, s, smem_q, smem_k, tv64, tv128, tg64, tqi, tki, st, sk);
  if (e != cudaSuccess) return e;
  return fk.join();
}

template <typename T>
static cudaError_t bwd_tc_d(const PopeAttnBwdArgs& a, cudaStream_t st) {
  switch (a.shape.d) {
    case 64: return launch_bwd_tc<64, T>(a, st);
    case 96: return launch_bwd_tc<96, T>(a, st);
    default: return launch_bwd_tc<128, T>(a, st);
  }
}

cudaError_t attn_bwd_tc(const PopeAttnBwdArgs& a, cudaStream_t st) {
  return a.shape.dtype == POPE_BF16 ? bwd_tc_d<__nv_bfloat16>(a, st) : bwd_tc_d<__half>(a, st);
}

}  // namespace pope
