// The grouped weight-streaming GEMM (part of umma_gemm.cu, which provides the tile configuration, the epilogue
// helpers and the status word): ONE persistent launch computes a whole list of skinny GEMMs D_p = alpha_p A_p W_p^T.
//
// Why: on this GPU a decode GEMM needs 2-4 us of HBM time, while a launch costs 7-9 us around it (ring fill, tail,
// hand-over to the next launch). Here every CTA walks a device-side list of pieces {problem, weight tile, K range}
// (group_plan.h) and its TMA producer keeps the shared-memory ring full ACROSS problem boundaries: the weights of
// problem p + 1 are already in flight while the last stages of problem p are multiplied, its cut tiles summed and
// its epilogue stored. Ring fill and tail are paid once per group.
//
// Each problem keeps the K split of its stand-alone launch and a cut tile is summed in ascending K order whatever
// the order in which its pieces arrive, so the results are bit-identical to q27b_skinny_fp4 / _bf16 / _glu_bf16
// called problem by problem, for every M. Which CTA sums a tile is fixed by the plan (see the epilogue).
//
// The table (header, problems with their two tensor maps, per-CTA piece lists) is built once on the host
// (q27b_skinny_group_build) and lives in device memory the caller owns; a launch only passes pointers, so it can
// be captured into a CUDA graph. No multicast, no peer memory, every wait bounded.

struct alignas(128) GroupProblemDev {
  CUtensorMap tmap_w;  // weight codes [N][K/2]: boxes of 128 rows x 128 bytes
  CUtensorMap tmap_a;  // activation codes [M][K/2]: boxes of NB rows x 128 bytes
  void* d;
  const float* c;
  AlphaSeg alpha;
  float alpha_up, beta;
  int N, epi;
};
static_assert(sizeof(GroupProblemDev) == 384, "GroupProblemDev layout");

constexpr uint32_t kGroupMagic = 0x51324742u;  // "Q2GB"
struct GroupHeader {  // the first 128 bytes of the table
  uint32_t magic;
  int M, nb, n_problems, n_ctas, n_items, counters, sms;
  int64_t slots, off_problems, off_cta_first, off_cta_units, off_items, table_bytes, ws_bytes;
  int imbalance_permille;  // stages of the busiest CTA over the mean, in thousandths (1000 = perfectly even)
  int pad32;
  int64_t pad[4];
};
static_assert(sizeof(GroupHeader) == 128, "GroupHeader layout");

struct GroupLaunch {
  const GroupProblemDev* probs;
  const int* cta_first;  // pieces of CTA g: [cta_first[g], cta_first[g + 1])
  const int* cta_units;  // stages CTA g streams
  const GroupItem* items;
  int M;
  int* counters;         // one per cut tile, zero between launches
  float* partials;       // [slots][M][128]
  // Gather fused into the epilogue (several GPUs): every output store is repeated into the peers' memory, and the
  // last CTA to finish tells every peer that this GPU's block of the outputs has been written.
  PeerCopies peers;          // n = 0: single GPU
  int32_t* signals;          // this GPU's signal block (kSignalWords words; see GatherWait)
  int32_t* peer_signals[7];  // the peers' signal blocks, in their memory
  int my_slot;               // the word of a signal block this GPU counts its finished launches in (its rank)
#ifdef Q27B_TRACE
  unsigned long long* trace;  // [cta][16]: per-role busy / waiting times in ns (null: off)
#endif
};

#ifdef Q27B_TRACE
#define GTRACE_DECL(name) unsigned long long name = 0
#define GTRACE_T0(t) const unsigned long long t = gtime()
#define GTRACE_ADD(acc, t) acc += gtime() - t
#define GTRACE_INC(acc) acc += 1
#define GTRACE_PUT(slot, v)                                                     \
  do {                                                                          \
    if (g.trace) g.trace[size_t(blockIdx.x) * 16 + (slot)] = (v);               \
  } while (0)
#else
#define GTRACE_DECL(name)
#define GTRACE_T0(t)
#define GTRACE_ADD(acc, t)
#define GTRACE_INC(acc)
#define GTRACE_PUT(slot, v)
#endif

constexpr int kSignalStep = 8, kSignalDone = 9, kSignalWords = 16;  // layout of a signal block (see GatherWait)
__device__ __forceinline__ int4 ldg16(const void* p) { return __ldg(reinterpret_cast<const int4*>(p)); }
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
constexpr int kSumBatch = 4;  // partial tiles whose loads are in flight together when a cut tile is summed

// Tile configuration of the grouped kernel: the stage layout of the stand-alone weight-streaming kernel, but as
// many accumulator buffers as tensor memory holds beside the scale columns (8 at 16 tokens, 4 at 32, 2 at 64, 1 at
// 128). A piece of a cut tile is only 2-4 stages long while its epilogue (partial tile out, arrival counted, now and
// then the sum of a whole tile) takes as long as streaming it: with many buffers the MMAs run several pieces ahead
// and the epilogue catches up during the long uncut tiles instead of stalling the stream.
template <int NB, int STAGES>
struct GroupCfg {
  using C = Cfg<NB, STAGES, 2, true>;
  static constexpr int kAccBufs = (C::kTmemCols - C::kSfCols * STAGES) / NB < 8 ? (C::kTmemCols - C::kSfCols * STAGES) / NB : 8;
  static constexpr int kSfCol0 = kAccBufs * NB;
  static constexpr int kXchgBytes = 8 * 64 * 4 + 16 * 16;      // SiLU*mul exchange between the gate and the up warps + the queue of tiles to sum
  static constexpr int kNumBars = 3 * STAGES + 2 * kAccBufs;
  // Fused gather at up to 16 tokens: a finished tile (16 tokens x 128 channels, at most fp32) is laid out token-major
  // in shared memory and leaves as 16-byte pieces of whole token rows (see flush_staged_tile)
  static constexpr int kStageOutBytes = NB == 16 ? 16 * 128 * 4 : 0;
  static constexpr int kStageOutOff = STAGES * C::kStageBytes + kXchgBytes + (kNumBars * 8 + 16 + 15) / 16 * 16;
  static constexpr int kSmemBytes = kStageOutOff + kStageOutBytes + 1024;
  static_assert(kAccBufs >= 1 && kSfCol0 + C::kSfCols * STAGES <= C::kTmemCols, "tensor memory budget");
  static_assert(2 * (kSmemBytes + 1024) <= 228 * 1024, "shared memory budget");
};

// The stages (units of 128 weight rows x 256 K-elements) of this CTA in the order it streams them. The record of
// the next piece is requested while the current one is being streamed, so that moving on never waits for memory.
struct GroupUnits {
  const GroupItem* items;
  int i, i1;
  int prob, tile, c, c1, ksteps;
  const uint8_t *w_sf_tile, *a_sf;
  int4 n0, n1, n2;  // words 0..2 of piece i + 1
  bool valid;
  __device__ __forceinline__ void fetch_next() {
    if (i + 1 < i1) {
      const int4* r = reinterpret_cast<const int4*>(items + i + 1);
      n0 = __ldg(r), n1 = __ldg(r + 1), n2 = __ldg(r + 2);
    }
  }
  __device__ __forceinline__ void adopt() {
    prob = n0.x, tile = n0.y, c = n0.z, c1 = n0.w, ksteps = n1.w;
    w_sf_tile = reinterpret_cast<const uint8_t*>((uint64_t(uint32_t(n2.y)) << 32) | uint32_t(n2.x));
    a_sf = reinterpret_cast<const uint8_t*>((uint64_t(uint32_t(n2.w)) << 32) | uint32_t(n2.z));
  }
  __device__ __forceinline__ GroupUnits(const GroupLaunch& g, int first, int last) : items(g.items), i(first - 1), i1(last) {
    valid = first < last;
    if (valid) {
      fetch_next();
      i = first;
      adopt();
      fetch_next();
    }
  }
  __device__ __forceinline__ void advance() {
    if (++c < c1) return;
    if (++i < i1) {
      adopt();
      fetch_next();
    } else {
      valid = false;
    }
  }
};

// Fused gather, few tokens: with the tokens on the MMA's N side a thread holds ONE channel of every token, and stores
// straight from registers are 2-byte pieces, 64 contiguous bytes per warp instruction - once per destination GPU. At
// eight GPUs the epilogue then issues 128 such stores per thread and tile and the NVLink packets are small. Instead the
// finished values go token-major into shared memory (stage_swapped: the arithmetic of store_swapped, bit for bit) and
// leave as 16-byte pieces of whole token rows, a quarter of the store instructions and rows of 128-512 contiguous bytes.
template <int kEpi>
__device__ __forceinline__ void stage_swapped(const GemmParams& p, const float (&v)[8], int m0, int tile, int row, float* xchg,
                                              uint8_t* stage_out) {
  if constexpr (kEpi == kEpiGluBf16) {
    if (row >= 64) {
#pragma unroll
      for (int j = 0; j < 8; j++) xchg[j * 64 + row - 64] = v[j];
    }
    epi_bar();
    if (row < 64) {
      const float ag = p.alpha.alpha[0], au = p.alpha_up;
      uint16_t* d = reinterpret_cast<uint16_t*>(stage_out) + row;
#pragma unroll
      for (int j = 0; j < 8; j++)
        if (m0 + j < p.M) d[(m0 + j) * 64] = bf16_bits(silu_mul(__fmul_rn(ag, v[j]), __fmul_rn(au, xchg[j * 64 + row])));
    }
    epi_bar();
  } else {
    const int n = tile * 128 + row;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int m = m0 + j;
      if (m < p.M) {
        const float out = finish_f32(p, v[j], m, n);
        if constexpr (kEpi == kEpiF32) reinterpret_cast<float*>(stage_out)[m * 128 + row] = out;
        else reinterpret_cast<uint16_t*>(stage_out)[m * 128 + row] = bf16_bits(out);
      }
    }
  }
}
// The staged tile to this GPU's memory and to every peer's: thread t moves 16-byte pieces t, t + 128, ... of the M token
// rows (128, 256 or 512 bytes each). Called by the four epilogue warps together.
template <int kEpi>
__device__ __forceinline__ void flush_staged_tile(const GemmParams& p, int tile, const uint8_t* stage_out, const PeerCopies& peers) {
  constexpr int kRowBytes = kEpi == kEpiF32 ? 512 : kEpi == kEpiBf16 ? 256 : 128, kPieces = kRowBytes / 16;
  const int64_t ld = kEpi == kEpiF32 ? int64_t(p.N) * 4 : kEpi == kEpiBf16 ? int64_t(p.N) * 2 : int64_t(p.N);  // bytes between token rows
  epi_bar();  // the tile is staged
  char* d0 = static_cast<char*>(p.d) + int64_t(tile) * kRowBytes;
  for (int i = threadIdx.x - 64; i < p.M * kPieces; i += 128) {
    const int m = i / kPieces, piece = i % kPieces;
    const uint4 val = *reinterpret_cast<const uint4*>(stage_out + m * kRowBytes + piece * 16);
    char* d = d0 + m * ld + piece * 16;
    *reinterpret_cast<uint4*>(d) = val;
    for (int j = 0; j < peers.n; j++) *reinterpret_cast<uint4*>(d + peers.delta[j]) = val;
  }
  epi_bar();  // ... and may be overwritten by the next tile
}

template <int NB, int STAGES>
__global__ void __launch_bounds__((Cfg<NB, STAGES, 2, true>::kThreads), 2) skinny_group_kernel(const __grid_constant__ GroupLaunch g) {
  using C = Cfg<NB, STAGES, 2, true>;
  using G = GroupCfg<NB, STAGES>;
  static_assert(C::kQAtoms == 1, "the tokens of a group fit one 128-row block");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* xchg = reinterpret_cast<float*>(smem + STAGES * C::kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::kStageBytes + G::kXchgBytes);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, sfr0 = empty0 + 8 * STAGES,
                 afull0 = sfr0 + 8 * STAGES, aempty0 = afull0 + 8 * G::kAccBufs;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + G::kNumBars);
  volatile uint32_t* abort_flag = tmem_holder + 1;
  volatile uint32_t* last_flag = tmem_holder + 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i0 = __ldg(g.cta_first + blockIdx.x), i1 = __ldg(g.cta_first + blockIdx.x + 1);
  const uint32_t smem_base = smem_u32(smem);

  auto stage_bytes = [&](const GroupUnits& k) { return uint32_t(C::kPBytes + C::kQBytes + 2 * min(4, k.ksteps - 4 * k.c) * 512); };
  auto load_w = [&](const GroupUnits& k, int stage) {  // weights: read once, evict first
    const uint32_t sbase = smem_base + stage * C::kStageBytes, bar = full0 + 8 * stage;
    tma_load_2d(sbase, &g.probs[k.prob].tmap_w, k.c * 128, k.tile * 128, bar, kEvictFirst);
    bulk_load(sbase + C::kOffSfP, k.w_sf_tile + int64_t(4 * k.c) * 512, min(4, k.ksteps - 4 * k.c) * 512, bar, kEvictFirst);
  };
  auto load_a = [&](const GroupUnits& k, int stage) {  // activations: re-read by every CTA, keep them in L2
    const uint32_t sbase = smem_base + stage * C::kStageBytes, bar = full0 + 8 * stage;
    tma_load_2d(sbase + C::kOffQ, &g.probs[k.prob].tmap_a, k.c * 128, 0, bar, kEvictLast);
    bulk_load(sbase + C::kOffSfQ, k.a_sf + int64_t(4 * k.c) * 512, min(4, k.ksteps - 4 * k.c) * 512, bar, kEvictLast);
  };
  uint32_t armed = 0;  // (producer lane) stages with a copy possibly in flight
  int npre = 0;        // (producer lane) stages filled before the steady state

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) mbar_init(full0 + 8 * s, 1), mbar_init(empty0 + 8 * s, 1), mbar_init(sfr0 + 8 * s, 4);
    for (int b = 0; b < G::kAccBufs; b++) mbar_init(afull0 + 8 * b, 1), mbar_init(aempty0 + 8 * b, C::kEpiWarps);
    *abort_flag = 0;
    mbar_init_fence();
    // The stream starts at once: the ring is filled with weights (which no kernel of this stream produces) while the
    // rest of the CTA sets up and before the preceding kernel is known to have finished.
    for (GroupUnits k(g, i0, i1); k.valid && npre < STAGES; k.advance(), npre++) {
      mbar_arrive_expect_tx(full0 + 8 * npre, stage_bytes(k));
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
      pdl_wait();  // the activations may come from the preceding kernel
      GroupUnits k(g, i0, i1);
      for (int s = 0; s < npre; s++, k.advance()) load_a(k, s);
      int stage = npre % STAGES;
      uint32_t phase = npre == STAGES ? 1 : 0;
      bool ok = true;
      int cur_prob = -1;
      GTRACE_DECL(t_wait_empty);
      GTRACE_PUT(0, gtime());
      for (; k.valid; k.advance()) {
        if (k.prob != cur_prob) {  // descriptors of a problem this CTA has not touched yet
          cur_prob = k.prob;
          prefetch_tensormap(&g.probs[cur_prob].tmap_w);
          prefetch_tensormap(&g.probs[cur_prob].tmap_a);
        }
        GTRACE_T0(t0);
        if (!mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1, abort_flag, &g_status, kStatusEmptyWaitTimeout)) {
          ok = false;
          break;
        }
        GTRACE_ADD(t_wait_empty, t0);
        mbar_arrive_expect_tx(full0 + 8 * stage, stage_bytes(k));
        last_parity = (last_parity & ~(1u << stage)) | (phase << stage);
        load_w(k, stage);
        load_a(k, stage);
        if (++stage == STAGES) stage = 0, phase ^= 1;
      }
      GTRACE_PUT(1, gtime());
      GTRACE_PUT(2, t_wait_empty);
      pdl_trigger();  // everything this CTA reads from HBM has been requested
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
      constexpr uint32_t idesc = umma_idesc_nvfp4(NB);
      int stage = 0, nseg = 0;
      uint32_t phase = 0;
      bool ok = true;
      GTRACE_DECL(t_wait_acc);
      GTRACE_DECL(t_wait_stage);
      for (int i = i0; ok && i < i1; i++) {
        const int4 w0 = ldg16(g.items + i), w1 = ldg16(reinterpret_cast<const int4*>(g.items + i) + 1);
        const int c0 = w0.z, c1 = w0.w, ksteps = w1.w, n = i - i0;
        const int buf = n % G::kAccBufs, use = n / G::kAccBufs;
        GTRACE_T0(ta);
        if (!mbar_wait_bounded(aempty0 + 8 * buf, (use & 1) ^ 1, abort_flag, &g_status, kStatusAccumFreeTimeout)) break;
        GTRACE_ADD(t_wait_acc, ta);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * NB;
        uint32_t accumulate = 0;
        for (int c = c0; c < c1; c++) {
          GTRACE_T0(ts);
          if (!mbar_wait_bounded(sfr0 + 8 * stage, phase, abort_flag, &g_status, kStatusFullWaitTimeout)) {
            ok = false;
            break;
          }
          GTRACE_ADD(t_wait_stage, ts);
          tc_fence_after_sync();
          const int nsteps = min(4, ksteps - 4 * c);
          const uint32_t sbase = smem_base + stage * C::kStageBytes;
          const uint64_t desc_p = umma_desc_k_sw128(sbase), desc_q = umma_desc_k_sw128(sbase + C::kOffQ);
          const uint32_t sf_col = tmem_base + G::kSfCol0 + C::kSfCols * stage;
          for (int ks = 0; ks < nsteps; ks++) {
            umma_nvfp4(d_tmem, desc_p + 2 * ks, desc_q + 2 * ks, idesc, sf_col + 4 * ks, sf_col + 16 + 4 * ks, accumulate);
            accumulate = 1;
          }
          umma_commit(empty0 + 8 * stage);
          if (++stage == STAGES) stage = 0, phase ^= 1;
        }
        if (ok) umma_commit(afull0 + 8 * buf);
        nseg = n + 1;
      }
      GTRACE_PUT(3, t_wait_acc);
      GTRACE_PUT(4, t_wait_stage);
      GTRACE_PUT(5, gtime());
      for (int j = nseg - 1; ok && j >= 0 && j >= nseg - G::kAccBufs; j--)
        ok = mbar_wait_bounded(aempty0 + 8 * (j % G::kAccBufs), (j / G::kAccBufs) & 1, abort_flag, &g_status,
                               kStatusAccumFreeTimeout, 64);
    }
  } else if (warp >= C::kFeederWarp0) {
    // ------------------------------------------------------------------------------------------ scales -> tensor memory
    // One thread of each of the four warps copies two of a landed stage's eight scale atoms (four of the weight rows,
    // four of the tokens) shared memory -> tensor memory with tcgen05.cp (a 512-byte atom becomes 4 columns, replicated
    // to the four lane quarters as the MMA expects) and commits: the commit arrives on the barrier the MMA issuer waits
    // on once the copies have completed. (On the MMA-issuing thread itself these copies cost ~90 cycles each and capped
    // the stream; through registers - four warps, tcgen05.st - they cost 16 KiB of shared-memory reads per stage.)
    if (lane == 0) {
      const int j = warp - C::kFeederWarp0;  // 0..3: MMA step whose atoms this thread copies
      const int units = __ldg(g.cta_units + blockIdx.x);
      const uint64_t atom0 = umma_desc_sf_atom(smem_base + C::kOffSfP);  // atoms 0..3: weight rows, 4..7: tokens
      int stage = 0;
      uint32_t phase = 0;
      for (int u = 0; u < units; u++) {
        if (!mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag, &g_status, kStatusFullWaitTimeout, 32)) break;
        const uint64_t d0 = atom0 + uint64_t(stage) * (C::kStageBytes >> 4);
        const uint32_t t0 = tmem_base + G::kSfCol0 + C::kSfCols * stage;
        tmem_cp_sf_atom(t0 + 4 * j, d0 + uint64_t(j) * (512 >> 4));
        tmem_cp_sf_atom(t0 + 16 + 4 * j, d0 + uint64_t(4 + j) * (512 >> 4));
        umma_commit(sfr0 + 8 * stage);
        if (++stage == STAGES) stage = 0, phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------------------------------ epilogue
    // A piece that is a whole tile is finished here. A piece of a CUT tile leaves its partial sums in the workspace and
    // counts its arrival (fire and forget). One piece of every cut tile is marked by the planner: its CTA sums the tile,
    // in ascending K order whatever the order of arrival. It does not wait for the other pieces: the tile goes into a
    // short queue, and before each later piece the CTA looks once whether the oldest queued tile is complete; what is
    // still queued when the CTA has no pieces left is waited for (bounded). The sums are thus dealt out by the plan,
    // evenly - with "whoever arrives last sums" the CTAs that fall behind collect the sums and fall further behind.
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // weight row of the tile = output channel
    const int M = g.M;
    constexpr int kQueue = 16;
    int4* queue = reinterpret_cast<int4*>(xchg + 8 * 64);  // {first slot, pieces | problem << 16, counter, tile}
    uint8_t* stage_out = smem + G::kStageOutOff;           // (16-token configuration only)
    int head = 0, queued = 0, polls = 0;
    bool ok = true;
    GTRACE_DECL(t_wait_mma);
    GTRACE_DECL(t_reduce);
    GTRACE_DECL(n_reduce);
    // The epilogue's view of a problem, read when a tile is finished (once per whole tile or summed tile; the
    // record sits in L1 / L2) rather than carried in registers across pieces.
    auto load_problem = [&](int prob, GemmParams& dst, int& e) {
      const GroupProblemDev* q = g.probs + prob;
      dst.M = M, dst.d = q->d, dst.c = q->c, dst.alpha = q->alpha, dst.alpha_up = q->alpha_up, dst.beta = q->beta, dst.N = q->N;
      dst.wscale = nullptr, e = q->epi;
    };
    auto store = [&](const GemmParams& q, int e, const float(&v)[8], int m0, int tile) {
      if (e == kEpiGluBf16) store_swapped<kEpiGluBf16>(q, v, m0, tile, row, xchg, g.peers);
      else if (e == kEpiBf16) store_swapped<kEpiBf16>(q, v, m0, tile, row, xchg, g.peers);
      else store_swapped<kEpiF32>(q, v, m0, tile, row, xchg, g.peers);
    };
    // Has every piece of the oldest queued tile arrived? One thread reads the counter; `wait`: keep reading (bounded).
    auto oldest_complete = [&](bool wait) -> bool {
      volatile uint32_t* flag = last_flag + (polls++ & 1);
      if (threadIdx.x == 64) {
        const int4 e = queue[head % kQueue];
        const int want = e.y & 0xffff;
        bool done = ld_acquire_gpu(g.counters + e.z) == want;
        if (!done && wait) {
          const long long t0 = clock64();
          for (uint32_t it = 0; !done && it < kMaxPolls; it++) {
            __nanosleep(200);
            done = ld_acquire_gpu(g.counters + e.z) == want;
            if ((it & 63u) == 63u && (*abort_flag || clock64() - t0 > kMaxWaitCycles)) break;
          }
          if (!done) {
            *abort_flag = 1u;
            atomicCAS(&g_status, 0u, uint32_t(kStatusTileWaitTimeout));
          }
        }
        *flag = done;
      }
      epi_bar();
      return *flag != 0;
    };
    // Sums the pieces of the oldest queued tile in ascending K order and finishes the tile.
    auto sum_oldest = [&]() {
      const int4 e = queue[head % kQueue];
      head++, queued--;
      const int slot0 = e.x, nparts = e.y & 0xffff, prob = e.y >> 16, counter = e.z, tile = e.w;
      GemmParams pr;
      int sum_epi;
      load_problem(prob, pr, sum_epi);
      GTRACE_T0(tr);
      if (pr.M <= 2) {
        // one or two tokens (plain decode): up to eight pieces in flight, one round trip
        float v[8] = {};
        for (int q0 = 0; q0 < nparts; q0 += 8) {
          float x[8][2];
#pragma unroll
          for (int q = 0; q < 8; q++) {
            if (q0 + q < nparts) {
              const float* part = g.partials + int64_t(slot0 + q0 + q) * pr.M * 128 + row;
              x[q][0] = __ldcg(part);
              x[q][1] = pr.M > 1 ? __ldcg(part + 128) : 0.f;
            }
          }
#pragma unroll
          for (int q = 0; q < 8; q++) {
            if (q0 + q < nparts) {
              v[0] = (q0 + q == 0) ? x[q][0] : __fadd_rn(v[0], x[q][0]);
              v[1] = (q0 + q == 0) ? x[q][1] : __fadd_rn(v[1], x[q][1]);
            }
          }
        }
        store(pr, sum_epi, v, 0, tile);
      } else {
        for (int m0 = 0; m0 < pr.M; m0 += 8) {
          float v[8];
          for (int q0 = 0; q0 < nparts; q0 += kSumBatch) {  // kSumBatch pieces in flight at a time
            float x[kSumBatch][8];
#pragma unroll
            for (int q = 0; q < kSumBatch; q++) {
              if (q0 + q < nparts) {
                const float* part = g.partials + (int64_t(slot0 + q0 + q) * pr.M + m0) * 128 + row;
#pragma unroll
                for (int j = 0; j < 8; j++) x[q][j] = m0 + j < pr.M ? __ldcg(part + j * 128) : 0.f;
              }
            }
#pragma unroll
            for (int q = 0; q < kSumBatch; q++) {
              if (q0 + q < nparts) {
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = (q0 + q == 0) ? x[q][j] : __fadd_rn(v[j], x[q][j]);
              }
            }
          }
          store(pr, sum_epi, v, m0, tile);
        }
      }
      if (threadIdx.x == 64) g.counters[counter] = 0;  // the counters are zero again when the kernel ends
      GTRACE_ADD(t_reduce, tr);
      GTRACE_INC(n_reduce);
    };

    for (int i = i0; ok && i < i1; i++) {
      const int4 w0 = ldg16(g.items + i), w1 = ldg16(reinterpret_cast<const int4*>(g.items + i) + 1),
                 w3 = ldg16(reinterpret_cast<const int4*>(g.items + i) + 3);
      const int prob = w0.x, tile = w0.y, slot = w1.x, nparts = w1.y, slot0 = w1.z, counter = w3.x, sums = w3.y;
      if (queued > 0) {  // one look per piece; the queue only blocks when it is full
        if (oldest_complete(queued == kQueue)) sum_oldest();
        else if (queued == kQueue) break;  // (timed out: the status word says so)
      }
      const int n = i - i0, buf = n % G::kAccBufs;
      GTRACE_T0(tw);
      if (!warp_wait(afull0 + 8 * buf, (n / G::kAccBufs) & 1, abort_flag, &g_status, kStatusAccumWaitTimeout, 128)) {
        ok = false;
        break;
      }
      GTRACE_ADD(t_wait_mma, tw);
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * NB;
      if (slot < 0) {
        GemmParams p;
        int epi;
        load_problem(prob, p, epi);
        const bool staged = G::kStageOutBytes > 0 && g.peers.n > 0;  // (uniform over the CTA)
        for (int m0 = 0; m0 < M; m0 += 8) {
          float v[8];
          tmem_ld8(taddr + m0, v);
          tmem_ld_wait();
          if (!staged) store(p, epi, v, m0, tile);
          else if (epi == kEpiGluBf16) stage_swapped<kEpiGluBf16>(p, v, m0, tile, row, xchg, stage_out);
          else if (epi == kEpiBf16) stage_swapped<kEpiBf16>(p, v, m0, tile, row, xchg, stage_out);
          else stage_swapped<kEpiF32>(p, v, m0, tile, row, xchg, stage_out);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(aempty0 + 8 * buf);
        if (staged) {
          if (epi == kEpiGluBf16) flush_staged_tile<kEpiGluBf16>(p, tile, stage_out, g.peers);
          else if (epi == kEpiBf16) flush_staged_tile<kEpiBf16>(p, tile, stage_out, g.peers);
          else flush_staged_tile<kEpiF32>(p, tile, stage_out, g.peers);
        }
        continue;
      }
      for (int m0 = 0; m0 < M; m0 += 16) {
        float* part = g.partials + (int64_t(slot) * M + m0) * 128 + row;
        if (M - m0 > 8) {
          float v[16];
          tmem_ld16(taddr + m0, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; j++)
            if (m0 + j < M) __stcg(part + j * 128, v[j]);
        } else {
          float v[8];
          tmem_ld8(taddr + m0, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; j++)
            if (m0 + j < M) __stcg(part + j * 128, v[j]);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(aempty0 + 8 * buf);
      epi_bar();  // every partial sum of this CTA is written ...
      if (threadIdx.x == 64) {
        __threadfence();  // ... and published device-wide before the arrival is counted
        atomicAdd(g.counters + counter, 1);
        if (sums) queue[(head + queued) % kQueue] = make_int4(slot0, nparts | (prob << 16), counter, tile);
      }
      if (sums) queued++;
    }
    while (ok && queued > 0) {  // what is still queued: wait for the other pieces (bounded)
      if (!oldest_complete(true)) break;
      sum_oldest();
    }
    if (threadIdx.x == 64) {
      GTRACE_PUT(6, t_wait_mma);
      GTRACE_PUT(7, t_reduce);
      GTRACE_PUT(8, n_reduce);
      GTRACE_PUT(9, gtime());
      GTRACE_PUT(10, (unsigned long long)(i1 - i0));
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
  if (g.peers.n > 0 && threadIdx.x == 0) {
    // every store of this CTA (local and into the peers) is ordered before the count; the CTA that counts last
    // orders all of them before it raises this GPU's word in every peer's signal block
    __threadfence_system();
    if (atomicAdd(g.signals + kSignalDone, 1) == int(gridDim.x) - 1) {
      g.signals[kSignalDone] = 0;
      __threadfence_system();
      for (int j = 0; j < g.peers.n; j++) atomicAdd_system(g.peer_signals[j] + g.my_slot, 1);
    }
  }
}

// The other half of the fused gather: a one-warp kernel, enqueued behind the grouped launch, that returns once every
// peer has raised its word in this GPU's signal block for this step, i.e. once the peers' blocks of the outputs have
// arrived in this GPU's memory. Words 0..7: launches finished by the GPU with that slot (written by the peers);
// kSignalStep: steps waited for so far (this kernel); kSignalDone: CTAs of the running launch that have finished.
// The wait is bounded; when it runs out the status word is set (8) and the kernel ends.
struct GatherWait {
  int32_t* signals;
  int n;
  int slot[7];
};
__global__ void group_gather_wait_kernel(const GatherWait w) {
  const int lane = threadIdx.x;
  // Launched as a programmatic dependent of the grouped launch: it may start while that launch's last CTAs finish and
  // watches the peers' words meanwhile. It ends - and only thereby releases its own successor - after the launch before
  // it has completed (griddepcontrol.wait below): "this kernel is done" keeps meaning "every GPU's block of the outputs
  // is in place". (The step word it reads at its start was written by the previous wait kernel, which has ended by
  // then: between two wait kernels lies a launch that passed its own griddepcontrol.wait before releasing this one.)
  const int step = w.signals[kSignalStep] + 1;
  bool ok = true;
  if (lane < w.n) {
    const volatile int32_t* word = w.signals + w.slot[lane];
    const long long t0 = clock64();
    ok = false;
    for (uint32_t it = 0; it < kMaxPolls; it++) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
      if (v - step >= 0) {
        ok = true;
        break;
      }
      __nanosleep(100);
      if ((it & 63u) == 63u && clock64() - t0 > kMaxWaitCycles) break;
    }
    if (!ok) atomicCAS(&g_status, 0u, uint32_t(kStatusPeerWaitTimeout));
  }
  __syncwarp();
  pdl_wait();
  if (lane == 0) w.signals[kSignalStep] = step;  // (no early release: the next kernel starts when this one has ended)
}

// ------------------------------------------------------------------------------------------------ host side

constexpr int kGroupMaxProblems = 4096;

int group_tokens_tile(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128; }

int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

int check_group_problem(int i, const q27b_group_problem& q) {
  Q27B_REQUIRE(q.N > 0 && q.N % 128 == 0, "skinny_group: problem %d: N must be a positive multiple of 128 (N = %d)", i, q.N);
  Q27B_REQUIRE(q.K > 0 && q.K % 64 == 0, "skinny_group: problem %d: K must be a positive multiple of 64 (K = %d)", i, q.K);
  Q27B_REQUIRE(q.epilogue >= 0 && q.epilogue <= 2, "skinny_group: problem %d: epilogue must be 0 (fp32), 1 (bf16) or 2 (SiLU*mul -> bf16)", i);
  Q27B_REQUIRE(q.alpha_count >= 1 && q.alpha_count <= 4, "skinny_group: problem %d: 1..4 alpha segments", i);
  Q27B_REQUIRE(q.epilogue == 0 || !q.c, "skinny_group: problem %d: a residual needs the fp32 epilogue", i);
  return 0;
}

template <int NB, int STAGES>
int launch_group(const GroupLaunch& gl, int ctas, cudaStream_t s) {
  using C = Cfg<NB, STAGES, 2, true>;
  auto kernel = skinny_group_kernel<NB, STAGES>;
  static bool done[64] = {};
  int dev = 0;
  Q27B_CUDA(cudaGetDevice(&dev));
  if (!(dev < 64 && done[dev])) {
    Q27B_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GroupCfg<NB, STAGES>::kSmemBytes));
    if (dev < 64) done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas), cfg.blockDim = dim3(C::kThreads), cfg.dynamicSmemBytes = GroupCfg<NB, STAGES>::kSmemBytes, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = pdl_enabled() ? 1 : 0;
  Q27B_CUDA(cudaLaunchKernelEx(&cfg, kernel, gl));
  return 0;
}
