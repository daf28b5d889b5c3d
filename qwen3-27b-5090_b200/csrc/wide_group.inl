// The grouped launch for 33..128 tokens (part of umma_gemm.cu, after skinny_group.inl): the same persistent walk over
// a device-side list of whole weight tiles, with the roles of the many-row GEMM - the tokens (one tile of 128) on the
// MMA's M side, 256 weight rows per tile on its N side, one CTA per SM.
//
// Why a second form: with the tokens on the N side a stage brings 16 KiB of weights AND 16 KiB of activations into the
// SM at 128 tokens, twice the weight bytes, and the stream stops at what an SM can ingest from L2 (58 % of the HBM
// peak over the 64-layer sweep). A 256-row weight tile shares one activation tile: 1.5 bytes into the SM per weight
// byte instead of 2 (1.25 instead of 1.5 at 64 tokens: rows past M are not read), and 4 x 36 KiB of weights in flight
// per SM as in the few-token configuration. Measured over the sweep: 83 % at 128 tokens, 91 % at 64 (tokens on N: 88 %),
// 93 % at 32 (tokens on N: 101 %) - hence the planner takes this form from 33 tokens (Q27_GROUP_WIDE_ABOVE_M moves that).
// Whole tiles only (Q27B_GROUP_WHOLE_TILES): every output is one accumulation chain over all of K, bit-identical to the
// many-row GEMM. No partial tiles, no sums, no workspace use.

__global__ void __launch_bounds__((Cfg<256, 4, 1, false>::kThreads), 1) wide_group_kernel(const __grid_constant__ GroupLaunch g) {
  constexpr int STAGES = 4;
  using C = Cfg<256, STAGES, 1, false>;
  static_assert(C::kQAtoms == 2 && C::kAccBufs == 1 && C::kEpiWarps == 16, "128 tokens x 256 weight rows, one accumulator");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::kStageBytes + C::kXchgBytes);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, sfr0 = empty0 + 8 * STAGES, afull = sfr0 + 8 * STAGES,
                 aempty = afull + 16;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile uint32_t* abort_flag = tmem_holder + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i0 = __ldg(g.cta_first + blockIdx.x), i1 = __ldg(g.cta_first + blockIdx.x + 1);
  const uint32_t smem_base = smem_u32(smem);

  auto sf_bytes_of = [&](const GroupUnits& k) { return uint32_t(min(4, k.ksteps - 4 * k.c)) * 512; };
  auto load_w = [&](const GroupUnits& k, int stage) {  // 256 weight rows and their two runs of scale atoms: read once
    const uint32_t sbase = smem_base + stage * C::kStageBytes, bar = full0 + 8 * stage;
    tma_load_2d(sbase + C::kOffQ, &g.probs[k.prob].tmap_w, k.c * 128, k.tile * 256, bar, kEvictFirst);
    const uint8_t* sf = k.w_sf_tile + int64_t(4 * k.c) * 512;
    bulk_load(sbase + C::kOffSfQ, sf, sf_bytes_of(k), bar, kEvictFirst);
    bulk_load(sbase + C::kOffSfQ + C::kSfBytes, sf + int64_t(k.ksteps) * 512, sf_bytes_of(k), bar, kEvictFirst);
  };
  auto load_a = [&](const GroupUnits& k, int stage) {  // the token tile: re-read for every weight tile, kept in L2
    const uint32_t sbase = smem_base + stage * C::kStageBytes, bar = full0 + 8 * stage;
    tma_load_2d(sbase, &g.probs[k.prob].tmap_a, k.c * 128, 0, bar, kEvictLast);
    bulk_load(sbase + C::kOffSfP, k.a_sf + int64_t(4 * k.c) * 512, sf_bytes_of(k), bar, kEvictLast);
  };
  uint32_t armed = 0;
  int npre = 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) mbar_init(full0 + 8 * s, 1), mbar_init(empty0 + 8 * s, 1), mbar_init(sfr0 + 8 * s, 4);
    mbar_init(afull, 1), mbar_init(aempty, C::kEpiWarps);
    *abort_flag = 0;
    mbar_init_fence();
    for (GroupUnits k(g, i0, i1); k.valid && npre < STAGES; k.advance(), npre++) {  // weights first, before the wait
      mbar_arrive_expect_tx(full0 + 8 * npre, C::kPBytes + C::kQBytes + 3 * sf_bytes_of(k));
      armed |= 1u << npre;
      load_w(k, npre);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t last_parity = 0;
      pdl_wait();
      GroupUnits k(g, i0, i1);
      for (int s = 0; s < npre; s++, k.advance()) load_a(k, s);
      int stage = npre % STAGES;
      uint32_t phase = npre == STAGES ? 1 : 0;
      bool ok = true;
      int cur_prob = -1;
      for (; k.valid; k.advance()) {
        if (k.prob != cur_prob) {
          cur_prob = k.prob;
          prefetch_tensormap(&g.probs[cur_prob].tmap_w);
          prefetch_tensormap(&g.probs[cur_prob].tmap_a);
        }
        if (!mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1, abort_flag, &g_status, kStatusEmptyWaitTimeout)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(full0 + 8 * stage, C::kPBytes + C::kQBytes + 3 * sf_bytes_of(k));
        last_parity = (last_parity & ~(1u << stage)) | (phase << stage);
        load_w(k, stage);
        load_a(k, stage);
        if (++stage == STAGES) stage = 0, phase ^= 1;
      }
      pdl_trigger();
      if (!ok) {
        for (int s = 0; s < STAGES; s++)
          if (armed >> s & 1) {
            bool landed = false;
            const long long t0 = clock64();
            for (uint32_t i = 0; i < kMaxPolls && !landed; i++) {
              landed = mbar_try_wait(full0 + 8 * s, last_parity >> s & 1);
              if ((i & 63u) == 63u && clock64() - t0 > kMaxWaitCycles) break;
            }
            if (!landed) atomicCAS(&g_status, 0u, uint32_t(kStatusDrainTimeout));
          }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_nvfp4(256);
      int stage = 0, ntiles = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = i0; ok && i < i1; i++, ntiles++) {
        const int4 w0 = ldg16(g.items + i), w1 = ldg16(reinterpret_cast<const int4*>(g.items + i) + 1);
        const int c0 = w0.z, c1 = w0.w, ksteps = w1.w;
        if (!mbar_wait_bounded(aempty, (ntiles & 1) ^ 1, abort_flag, &g_status, kStatusAccumFreeTimeout)) break;
        tc_fence_after_sync();
        uint32_t accumulate = 0;
        for (int c = c0; c < c1; c++) {
          if (!mbar_wait_bounded(sfr0 + 8 * stage, phase, abort_flag, &g_status, kStatusFullWaitTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const int nsteps = min(4, ksteps - 4 * c);
          const uint32_t sbase = smem_base + stage * C::kStageBytes;
          const uint64_t desc_p = umma_desc_k_sw128(sbase), desc_q = umma_desc_k_sw128(sbase + C::kOffQ);
          const uint32_t sf_col = tmem_base + C::kSfCol0 + C::kSfCols * stage;
          for (int ks = 0; ks < nsteps; ks++) {
            umma_nvfp4(tmem_base, desc_p + 2 * ks, desc_q + 2 * ks, idesc, sf_col + 4 * ks, sf_col + 16 + 8 * ks, accumulate);
            accumulate = 1;
          }
          umma_commit(empty0 + 8 * stage);
          if (++stage == STAGES) stage = 0, phase ^= 1;
        }
        if (ok) umma_commit(afull);
      }
      if (ok && ntiles > 0) mbar_wait_bounded(aempty, (ntiles - 1) & 1, abort_flag, &g_status, kStatusAccumFreeTimeout, 64);
    }
  } else if (warp >= C::kFeederWarp0) {
    // ------------------------------------------------------------------------------------------ scales -> tensor memory
    // (as in skinny_group_kernel: tcgen05.cp by one thread of each of four warps; three atoms each - the tokens' atom of
    //  MMA step j and the atoms of both blocks of 128 weight rows of that step)
    if (lane == 0) {
      const int j = warp - C::kFeederWarp0;
      const int units = __ldg(g.cta_units + blockIdx.x);
      const uint64_t atom0 = umma_desc_sf_atom(smem_base + C::kOffSfP);  // atoms 0..3: tokens; 4..7, 8..11: weight rows 0..127, 128..255
      int stage = 0;
      uint32_t phase = 0;
      for (int u = 0; u < units; u++) {
        if (!mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag, &g_status, kStatusFullWaitTimeout, 32)) break;
        const uint64_t d0 = atom0 + uint64_t(stage) * (C::kStageBytes >> 4);
        const uint32_t t0 = tmem_base + C::kSfCol0 + C::kSfCols * stage;
        tmem_cp_sf_atom(t0 + 4 * j, d0 + uint64_t(j) * (512 >> 4));
        tmem_cp_sf_atom(t0 + 16 + 8 * j, d0 + uint64_t(4 + j) * (512 >> 4));
        tmem_cp_sf_atom(t0 + 20 + 8 * j, d0 + uint64_t(8 + j) * (512 >> 4));
        umma_commit(sfr0 + 8 * stage);
        if (++stage == STAGES) stage = 0, phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------------------------------ epilogue (16 warps)
    // lane = token, column = output channel. Every warp pulls its share of the accumulator into registers at once and
    // hands the accumulator back before it does any arithmetic or stores.
    const int quarter = warp & 3, sub = (warp - 2) >> 2, m = quarter * 32 + lane;
    const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16);
    const bool valid = m < g.M;
    int ntiles = 0;
    for (int i = i0; i < i1; i++, ntiles++) {
      const int4 w0 = ldg16(g.items + i);
      const int q_row0 = w0.y * 256;
      GemmParams p = {};
      const GroupProblemDev* q = g.probs + w0.x;
      p.M = g.M, p.d = q->d, p.c = q->c, p.alpha = q->alpha, p.alpha_up = q->alpha_up, p.beta = q->beta, p.N = q->N;
      const int epi = q->epi;
      if (!warp_wait(afull, ntiles & 1, abort_flag, &g_status, kStatusAccumWaitTimeout, 64)) break;
      tc_fence_after_sync();
      if (epi == kEpiGluBf16) {
        float gt[2][16], up[2][16];  // 8 units of 16 outputs: 4 gate units per 128-row block, the up values 64 columns on
#pragma unroll
        for (int j = 0; j < 2; j++) {
          const int un = sub + 4 * j, c0 = (un >> 2) * 128 + (un & 3) * 16;
          tmem_ld16(taddr + c0, gt[j]);
          tmem_ld16(taddr + 64 + c0, up[j]);
        }
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(aempty);
#pragma unroll
        for (int j = 0; j < 2; j++) {
          const int un = sub + 4 * j;
          emit_many<kEpiGluBf16>(p, m, valid, q_row0, (un >> 2) * 128 + (un & 3) * 16, gt[j], up[j]);
        }
      } else {
        float v[4][16];  // 16 units of 16 outputs
#pragma unroll
        for (int j = 0; j < 4; j++) tmem_ld16(taddr + (sub + 4 * j) * 16, v[j]);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(aempty);
#pragma unroll
        for (int j = 0; j < 4; j++) {
          if (epi == kEpiBf16) emit_many<kEpiBf16>(p, m, valid, q_row0, (sub + 4 * j) * 16, v[j], v[j]);
          else emit_many<kEpiF32>(p, m, valid, q_row0, (sub + 4 * j) * 16, v[j], v[j]);
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

int launch_wide_group(const GroupLaunch& gl, int ctas, cudaStream_t s) {
  using C = Cfg<256, 4, 1, false>;
  static bool done[64] = {};
  int dev = 0;
  Q27B_CUDA(cudaGetDevice(&dev));
  if (!(dev < 64 && done[dev])) {
    Q27B_CUDA(cudaFuncSetAttribute(wide_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    if (dev < 64) done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas), cfg.blockDim = dim3(C::kThreads), cfg.dynamicSmemBytes = C::kSmemBytes, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = pdl_enabled() ? 1 : 0;
  Q27B_CUDA(cudaLaunchKernelEx(&cfg, wide_group_kernel, gl));
  return 0;
}
