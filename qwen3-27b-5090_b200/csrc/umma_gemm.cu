// NVFP4 x NVFP4 GEMM on the sm_100a tensor cores: tcgen05.mma kind::mxf4nvf4 (E2M1 operands, one UE4M3 scale per
// 16 K-elements, fp32 accumulators in tensor memory), operands and scale atoms brought in by TMA through a
// multi-stage shared-memory ring. One persistent, warp-specialised kernel serves both regimes:
//
//  * weight streaming (1 <= M <= 128, "skinny"): the roles of the operands are swapped — a 128-row weight tile is
//    the MMA's M side, the (padded) tokens are its N side — so one instruction consumes 4 KiB of weights whatever
//    the token count, and the kernel is bound by HBM. The K range of the whole weight matrix is cut into
//    pieces for two CTAs per SM (layout.h: contiguous unit ranges, or every tile in s equal K-parts, whichever a
//    cost model prefers; the split never depends on M). A tile that is cut is summed in ascending K order
//    whatever the order of arrival: up to 8 tokens by whichever of its CTAs arrives last, above by a small
//    fix-up kernel doing the same sums on the whole GPU (deterministic; no CTA ever waits for another).
//  * many rows (prefill): 128 tokens x 128 or 256 output channels per tile, tiles walked token-tile fastest so
//    that the CTAs running together share weight tiles through L2; the accumulator goes back to the MMA issuer
//    as soon as the epilogue warps hold it in registers. umma_gemm2_kernel runs the same on CTA pairs.
//
// Warp roles (320 threads): warp 0 = TMA producer (one lane), warp 1 = tensor-memory owner and MMA issuer (one
// lane), warps 2..5 = epilogue (tcgen05.ld -> alpha / residual / SiLU*mul -> fp32 or bf16 stores), one lane of each
// of warps 6..9 = scale copier (tcgen05.cp of a landed stage's scale atoms shared memory -> tensor memory, then a
// commit onto the barrier the MMA issuer waits on; measured here: a tcgen05.cp of one 512-byte atom costs its
// issuing thread ~90 cycles and an MMA ~140 whatever its N, so eight copies per stage on the MMA-issuing thread
// capped the stream at about half of HBM speed, and moving the atoms through registers with four whole warps cost
// shared-memory bandwidth and power).
// No multicast load, no peer memory in the loads. Every wait is bounded (ptx_sm100.cuh); a timeout is reported through a status word.
//
// Replaces, behind the same launcher contracts: skinny_fp4 (engine/src/skinny.cu:154-549), gemm_fp4 /
// gemm_fp4_bf16 (engine/src/gemm_mma.cu:463-626) and the gate | up SiLU*mul epilogue (gemm_mma.cu:350-399,
// kernels.cu:319-339) of the reference.
#include <cuda.h>
#include <dlfcn.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <type_traits>
#include <vector>

#include "../../include/q27b200/capi.h"
#include "common.cuh"
#include "group_plan.h"
#include "layout.h"
#include "ptx_sm100.cuh"
#include "quad_abi.h"
#include "quant_block.cuh"

namespace q27b {

__device__ uint32_t g_status;  // first bounded-wait timeout code since the last clear (0 = none)

#ifdef Q27B_TRACE
unsigned long long* g_trace = nullptr;  // device buffer for in-kernel time stamps (q27b_trace_set; -DQ27B_TRACE builds only)
#endif

namespace {

enum Epi : int { kEpiF32 = 0, kEpiBf16 = 1, kEpiGluBf16 = 2, kEpiGluFp4 = 3 };
constexpr bool epi_is_glu(int e) { return e == kEpiGluBf16 || e == kEpiGluFp4; }

// warp 0: TMA producer, 1: MMA issuer, then the epilogue warps (4, or 16 where a big tile is drained by one CTA
// alone), then 4 scale feeders
constexpr int kCounterBytes = 16384;  // per-tile arrival counters at the head of the workspace (4096 tiles)
constexpr int kMaxParts = 500;        // unit ranges that may share one tile (never more than there are ranges)

struct GemmParams {
  int M, N, K;          // tokens, weight rows (2 I for gate | up), reduction length
  int ksteps;           // K / 64 (MMA steps; also scale atoms per 128 rows)
  int chunks;           // ceil(ksteps / 4) pipeline stages over K
  const uint8_t* sf_p;  // scale atoms of the MMA's M-side operand
  const uint8_t* sf_q;  // scale atoms of the MMA's N-side operand
  AlphaSeg alpha;       // per output channel (gate alpha for the SiLU*mul epilogue)
  float alpha_up;
  const float* c;       // residual (may alias d) or null
  const float* wscale;  // optional per-output-channel scale [N] (weights quantised at load with channel scales)
  const float* ascale;  // with it: per-token scale [M] (dynamically quantised activations)
  float beta;
  void* d;              // fp32 or bf16 output; NVFP4 epilogue: E2M1 codes [M][N / 4]
  uint8_t* d_sf;        // NVFP4 epilogue: swizzled scales of the output, [M rows][N / 32 blocks]
  float out_gs;         // NVFP4 epilogue: 1 / (tensor scale of the output)
  int* counters;        // weight streaming: arrivals per cut tile (zero between calls)
  float* partials;      // weight streaming: per-CTA partial tiles [2 * grid][M][128]
  SkinnyPlan plan;      // weight streaming
  int m_tiles, items;   // many rows
  int n_tile;           // many rows: weight rows per tile (128 or 256)
  int ext_reduce;       // weight streaming: cut tiles are summed by skinny_fixup_kernel, not by the last CTA to arrive
  // many rows, gather fused into the epilogue (several GPUs; see q27b_group_peers): bf16 stores are repeated into the
  // peers' memory, and the last CTA of the launch raises this GPU's word in every peer's signal block
  int n_peers;
  long long peer_delta[7];
  int32_t* signals;
  int32_t* peer_signals[7];
  int my_slot;
#ifdef Q27B_TRACE
  unsigned long long* trace;  // [cta][4][64] globaltimer samples (null: off)
#endif
};

// CTAS = CTAs of this configuration that fit on one SM (2: half the shared and tensor memory each, so that the
// epilogue of one CTA overlaps the stream of the other and a CTA of the next launch can move in as soon as one of
// this launch leaves).
template <int NB, int STAGES, int CTAS, bool SWAP>
struct Cfg {
  static_assert(NB % 16 == 0 && NB >= 16 && NB <= 256 && (NB <= 128 || !SWAP), "N-side tile: 16..128 rows (256: many rows)");
  static_assert(CTAS == 1 || CTAS == 2, "one or two CTAs per SM");
  static constexpr int kQAtoms = (NB + 127) / 128;  // 128-row blocks of the N-side tile (scale atoms per MMA step)
  static constexpr int kPBytes = 128 * 128;  // 128 rows x 256 E2M1
  static constexpr int kQBytes = NB * 128;
  static constexpr int kSfBytes = 4 * 512;   // 4 MMA steps x one 512-byte atom (per 128-row block)
  static constexpr int kStageBytes = kPBytes + kQBytes + (1 + kQAtoms) * kSfBytes;
  static constexpr int kOffQ = kPBytes, kOffSfP = kPBytes + kQBytes, kOffSfQ = kOffSfP + kSfBytes;
  static constexpr int kSfCols = 16 + 16 * kQAtoms;  // tensor-memory columns of one stage's scales
  // Cut tiles may be summed inside the kernel only by the 16-token configuration (few tokens); the others always
  // leave that to the fix-up kernel and do not carry the list of partial tiles.
  static constexpr bool kInKernelReduce = SWAP && NB == 16;
  static constexpr int kXchgBytes = SWAP ? 8 * 64 * 4 + (kInKernelReduce ? 2048 : 0) : 0;  // SiLU*mul exchange between the gate and the up warps (+ cut-tile info)
  static constexpr int kNumBars = 3 * STAGES + 4;
  static constexpr int kBarBytes = kNumBars * 8 + 16;
  static constexpr int kSmemBytes = STAGES * kStageBytes + kXchgBytes + kBarBytes + 1024;  // + alignment slack
  static constexpr int kTmemCols = 512 / CTAS;
  // accumulators: two buffers when tensor memory allows (the epilogue of one piece overlaps the MMAs of the next),
  // else one (two CTAs per SM overlap each other instead); scales: kSfCols columns per stage after them
  static constexpr int kAccBufs = 2 * NB + kSfCols * STAGES <= kTmemCols ? 2 : 1;
  static constexpr int kSfCol0 = kAccBufs * NB;
  static constexpr int kRangesPerCta = 1;  // unit ranges of the work split per CTA
  // Epilogue warps: four per quarter of the tensor-memory lanes where one CTA per SM drains a 128 x 256 tile alone:
  // together they pull the whole accumulator into registers at once and hand it back to the MMA issuer before
  // doing any arithmetic or stores. Else one per quarter.
  static constexpr int kEpiWarps = (!SWAP && CTAS == 1) ? 16 : 4;
  static constexpr int kFeederWarp0 = 2 + kEpiWarps;
  static constexpr int kThreads = (kFeederWarp0 + 4) * 32;
  static_assert(kStageBytes % 1024 == 0, "stage tiles must stay 1024-byte aligned");
  static_assert(kSfCol0 + kSfCols * STAGES <= kTmemCols, "tensor memory budget");
  static_assert(CTAS * (kSmemBytes + 1024) <= 228 * 1024, "shared memory budget");
};

struct Work {
  int p_row0, q_row0;  // first row of the M-side / N-side tile
  int c0, c1;          // chunk range
  int slot;            // partial slot or -1 (finish in place)
  int tile;
};

// The pieces of work of this CTA, in the order every role walks them. Weight streaming: a CTA takes kRanges
// consecutive unit ranges of the work split.
template <bool kSwap, int kRanges>
struct WorkIter {
  const GemmParams& p;
  int64_t u;
  int item, range, range_end;
  __device__ explicit WorkIter(const GemmParams& p_) : p(p_) {
    if constexpr (kSwap) {
      u = -1, range = blockIdx.x * kRanges;
      range_end = min(range + kRanges, p.plan.grid);
    } else {
      item = blockIdx.x;
    }
  }
  __device__ bool next(Work& w) {
    if constexpr (kSwap) {
      Segment s;
      while (range < range_end) {
        if (next_segment(p.plan, range, u, s)) {
          w.p_row0 = s.tile * 128, w.q_row0 = 0, w.c0 = s.c0, w.c1 = s.c1, w.slot = s.slot, w.tile = s.tile;
          return true;
        }
        range++, u = -1;
      }
      return false;
    } else {
      if (item >= p.items) return false;
      const int mi = item % p.m_tiles, ni = item / p.m_tiles;
      w.p_row0 = mi * 128, w.q_row0 = ni * p.n_tile, w.c0 = 0, w.c1 = p.chunks, w.slot = -1, w.tile = ni;
      item += gridDim.x;
      return true;
    }
  }
};

// The same walk chunk by chunk (one chunk = one pipeline stage).
template <bool kSwap, int kRanges>
struct ChunkIter {
  WorkIter<kSwap, kRanges> it;
  Work w;
  int c;
  bool valid;
  __device__ explicit ChunkIter(const GemmParams& p) : it(p) {
    valid = it.next(w);
    c = valid ? w.c0 : 0;
  }
  __device__ void advance() {
    if (++c < w.c1) return;
    valid = it.next(w);
    c = valid ? w.c0 : 0;
  }
};

// In-kernel time stamps for performance work exist only in builds made with -DQ27B_TRACE (make TRACE=1), as the
// reference compiles its trace points in only under -DQ27_TRACE (engine/src/launch.cuh:17-44): the product kernels
// carry neither the pointer nor the checks.
#ifdef Q27B_TRACE
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define TRACE(kind, idx)                                                                                  \
  do {                                                                                                    \
    if (p.trace && (idx) < 64) p.trace[(size_t(blockIdx.x) * 4 + (kind)) * 64 + (idx)] = gtime();         \
  } while (0)
#define TRACE_DECL(name) unsigned long long name = 0
#define TRACE_INC(name) name++
#define TRACE_T0(t) const unsigned long long t = gtime()
#define TRACE_C0(c) const long long c = clock64()
#define TRACE_CPUT(idx, c) TRACE_PUT(idx, (unsigned long long)(clock64() - c))
#define TRACE_CADD(acc, c) acc += (unsigned long long)(clock64() - c)
#define TRACE_ADD(acc, t) acc += gtime() - t
#define TRACE_PUT(idx, v)                                                           \
  do {                                                                              \
    if (p.trace) p.trace[(size_t(blockIdx.x) * 4 + 3) * 64 + (idx)] = (v);          \
  } while (0)
#else
#define TRACE(kind, idx) \
  do {                   \
  } while (0)
#define TRACE_DECL(name)
#define TRACE_INC(name)
#define TRACE_T0(t)
#define TRACE_C0(c)
#define TRACE_CPUT(idx, c)
#define TRACE_CADD(acc, c)
#define TRACE_ADD(acc, t)
#define TRACE_PUT(idx, v)
#endif

// silu(g) * u with the fast exponential and reciprocal (the reference's fused epilogue uses the same pair,
// engine/src/gemm_mma.cu:362-378): no division slow path, and 1 / (1 + inf) = 0 for very negative gates.
__device__ __forceinline__ float silu_mul(float g, float u) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.44269504f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
  return g * r * u;
}

__device__ __forceinline__ uint16_t bf16_bits(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }

// Final value of output (m, n) from the accumulated dot product, with the reference's explicit roundings
// (engine/src/skinny.cu:452-458) so that a tile finished in place and a tile summed from partials agree bit for bit.
__device__ __forceinline__ float finish_f32(const GemmParams& p, float acc, int m, int n) {
  float out = __fmul_rn(alpha_of(p.alpha, n), acc);
  if (p.wscale) out = __fmul_rn(out, __fmul_rn(p.wscale[n], p.ascale[m]));
  if (p.c) out = __fmaf_rn(p.beta, p.c[int64_t(m) * p.N + n], out);
  return out;
}

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Copies of an output in other GPUs' memory: a store to local address x is repeated at x + delta[j] for j < n (plain
// stores through peer-mapped pointers). NoPeers: none, and the loops below vanish at compile time.
struct NoPeers {
  static constexpr int n = 0;
  long long delta[1];
};
struct PeerCopies {
  int n;
  long long delta[7];
};
template <typename T, typename Peers>
__device__ __forceinline__ void store_out(T* ptr, T val, const Peers& peers) {
  *ptr = val;
  for (int j = 0; j < peers.n; j++) *reinterpret_cast<T*>(reinterpret_cast<char*>(ptr) + peers.delta[j]) = val;
}

// Weight streaming: the epilogue of 8 tokens (m0 .. m0 + 7) of one weight row per thread (row = tile row 0..127).
template <int kEpi, typename Peers = NoPeers>
__device__ __forceinline__ void store_swapped(const GemmParams& p, const float (&v)[8], int m0, int tile, int row,
                                              float* xchg, const Peers& peers = Peers()) {
  if constexpr (kEpi == kEpiGluBf16) {
    // rows 0..63 of the tile are gate rows, 64..127 the up rows of the same 64 outputs
    if (row >= 64) {
#pragma unroll
      for (int j = 0; j < 8; j++) xchg[j * 64 + row - 64] = v[j];
    }
    epi_bar();
    if (row < 64) {
      const float ag = p.alpha.alpha[0], au = p.alpha_up;
      uint16_t* d = static_cast<uint16_t*>(p.d) + int64_t(tile) * 64 + row;
#pragma unroll
      for (int j = 0; j < 8; j++)
        if (m0 + j < p.M)
          store_out(d + int64_t(m0 + j) * (p.N / 2), bf16_bits(silu_mul(__fmul_rn(ag, v[j]), __fmul_rn(au, xchg[j * 64 + row]))), peers);
    }
    epi_bar();
  } else {
    const int n = tile * 128 + row;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int m = m0 + j;
      if (m < p.M) {
        const float out = finish_f32(p, v[j], m, n);
        if constexpr (kEpi == kEpiF32) store_out(static_cast<float*>(p.d) + int64_t(m) * p.N + n, out, peers);
        else store_out(static_cast<uint16_t*>(p.d) + int64_t(m) * p.N + n, bf16_bits(out), peers);
      }
    }
  }
}

// Many rows: stores 16 finished outputs of one token (tile columns c0 .. c0 + 15 of the tile starting at weight row
// q_row0; for the SiLU*mul epilogue g / u are 16 gate values and the up values of the same outputs: every 128
// weight rows are 64 gate rows followed by the up rows of the same 64 outputs).
template <int kEpi>
__device__ __forceinline__ void emit_many(const GemmParams& p, int m, bool valid, int q_row0, int c0, const float* g,
                                          const float* u) {
  if (!valid) return;
  if constexpr (kEpi == kEpiGluFp4) {
    // silu(gate) * up in fp32 (never rounded to bf16), then the activation quantiser's block arithmetic: the 16
    // outputs are one NVFP4 block of the next GEMM's activation (engine/src/gemm_mma.cu:350-399).
    const float ag = p.alpha.alpha[0], au = p.alpha_up;
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; j++) v[j] = silu_mul(__fmul_rn(ag, g[j]), __fmul_rn(au, u[j]));
    uint32_t lo, hi;
    uint8_t sfq;
    quant_block16_codes(v, p.out_gs, lo, hi, sfq);
    const int I = p.N / 2, o0 = (q_row0 + c0) / 2 + (c0 & 63) / 2;  // first of the 16 output channels
    *reinterpret_cast<uint2*>(static_cast<uint8_t*>(p.d) + int64_t(m) * (I / 2) + o0 / 2) = make_uint2(lo, hi);
    p.d_sf[sf_offset(m, o0 / 16, I / 16)] = sfq;
  } else if constexpr (kEpi == kEpiGluBf16) {
    const float ag = p.alpha.alpha[0], au = p.alpha_up;
    uint32_t pk[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const uint32_t lo = bf16_bits(silu_mul(__fmul_rn(ag, g[2 * j]), __fmul_rn(au, u[2 * j])));
      const uint32_t hi = bf16_bits(silu_mul(__fmul_rn(ag, g[2 * j + 1]), __fmul_rn(au, u[2 * j + 1])));
      pk[j] = lo | (hi << 16);
    }
    uint4* d = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.d) + int64_t(m) * (p.N / 2) + (q_row0 + c0) / 2 + (c0 & 63) / 2);
    d[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    d[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);

  } else {
    const int n0 = q_row0 + c0;
    float out[16];
#pragma unroll
    for (int j = 0; j < 16; j++) out[j] = finish_f32(p, g[j], m, n0 + j);
    if constexpr (kEpi == kEpiF32) {
      float4* d = reinterpret_cast<float4*>(static_cast<float*>(p.d) + int64_t(m) * p.N + n0);
#pragma unroll
      for (int j = 0; j < 4; j++) d[j] = make_float4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
    } else {
      uint32_t pk[8];
#pragma unroll
      for (int j = 0; j < 8; j++) pk[j] = uint32_t(bf16_bits(out[2 * j])) | (uint32_t(bf16_bits(out[2 * j + 1])) << 16);
      uint4* d = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.d) + int64_t(m) * p.N + n0);
      d[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      d[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
    }
  }
}

template <int NB, int STAGES, int CTAS, bool kSwap, int kEpi>
__global__ void __launch_bounds__((Cfg<NB, STAGES, CTAS, kSwap>::kThreads), CTAS) umma_gemm_kernel(const __grid_constant__ CUtensorMap tmap_p,
                                                                const __grid_constant__ CUtensorMap tmap_q,
                                                                const __grid_constant__ GemmParams p) {
  using C = Cfg<NB, STAGES, CTAS, kSwap>;
  using Chunks = ChunkIter<kSwap, C::kRangesPerCta>;
  using Works = WorkIter<kSwap, C::kRangesPerCta>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* xchg = reinterpret_cast<float*>(smem + STAGES * C::kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::kStageBytes + C::kXchgBytes);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, sfr0 = empty0 + 8 * STAGES,
                 afull0 = sfr0 + 8 * STAGES, aempty0 = afull0 + 16;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile uint32_t* abort_flag = tmem_holder + 1;
  volatile uint32_t* last_flag = tmem_holder + 2;
  volatile int* seg_info = reinterpret_cast<volatile int*>(xchg) + 8 * 64;  // [0] parts of a cut tile, [1..] their slots
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const uint32_t smem_base = smem_u32(smem);
  // Weights are read once (evict first); the activations are re-read by every CTA (keep them in L2).
  const uint64_t hint_w = kEvictFirst, hint_a = kEvictLast;
  const uint64_t hint_p = kSwap ? hint_w : hint_a, hint_q = kSwap ? hint_a : hint_w;
  auto stage_bytes = [&](int c) { return uint32_t(C::kPBytes + C::kQBytes + (1 + C::kQAtoms) * min(4, p.ksteps - 4 * c) * 512); };
  auto load_p = [&](const Chunks& k, int stage) {
    const uint32_t sbase = smem_base + stage * C::kStageBytes, bar = full0 + 8 * stage;
    tma_load_2d(sbase, &tmap_p, k.c * 128, k.w.p_row0, bar, hint_p);
    bulk_load(sbase + C::kOffSfP, p.sf_p + (int64_t(k.w.p_row0 / 128) * p.ksteps + 4 * k.c) * 512,
              min(4, p.ksteps - 4 * k.c) * 512, bar, hint_p);
  };
  auto load_q = [&](const Chunks& k, int stage) {
    const uint32_t sbase = smem_base + stage * C::kStageBytes, bar = full0 + 8 * stage;
    tma_load_2d(sbase + C::kOffQ, &tmap_q, k.c * 128, k.w.q_row0, bar, hint_q);
#pragma unroll
    for (int rb = 0; rb < C::kQAtoms; rb++)  // one run of atoms per 128-row block
      bulk_load(sbase + C::kOffSfQ + rb * C::kSfBytes, p.sf_q + (int64_t(k.w.q_row0 / 128 + rb) * p.ksteps + 4 * k.c) * 512,
                min(4, p.ksteps - 4 * k.c) * 512, bar, hint_q);
  };
  uint32_t armed = 0;  // (producer lane) stages with a copy possibly in flight
  int npre = 0;        // (producer lane) stages filled before the steady state

  if (threadIdx.x == 0) {
    TRACE(3, 0);
    prefetch_tensormap(&tmap_p);
    prefetch_tensormap(&tmap_q);
    for (int s = 0; s < STAGES; s++) mbar_init(full0 + 8 * s, 1), mbar_init(empty0 + 8 * s, 1), mbar_init(sfr0 + 8 * s, 4);
    for (int b = 0; b < 2; b++) mbar_init(afull0 + 8 * b, 1), mbar_init(aempty0 + 8 * b, C::kEpiWarps);
    *abort_flag = 0;
    mbar_init_fence();
    // The stream starts at once, while the rest of the CTA is still setting up: fill the ring with the operand
    // that does not depend on the preceding kernel (the weights when streaming).
    for (Chunks k(p); k.valid && npre < STAGES; k.advance(), npre++) {
      mbar_arrive_expect_tx(full0 + 8 * npre, stage_bytes(k.c));
      armed |= 1u << npre;
      TRACE(0, npre);
      if constexpr (kSwap) load_p(k, npre); else load_q(k, npre);
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
      // 1. (done above) the ring holds the first weights, 2. wait for the preceding kernel, 3. add the operand it
      //    produced, 4. steady state.
      uint32_t last_parity = 0;  // the phase each stage was last armed for
      pdl_wait();
      TRACE(3, 2);
      Chunks k(p);
      for (int s = 0; s < npre; s++, k.advance()) {
        if constexpr (kSwap) load_q(k, s); else load_p(k, s);
      }
      int stage = npre % STAGES, tk = npre;
      uint32_t phase = npre == STAGES ? 1 : 0;
      bool ok = true;
      for (; k.valid; k.advance()) {
        if (!mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1, abort_flag, &g_status, kStatusEmptyWaitTimeout)) {
          ok = false;
          break;
        }
        TRACE(0, tk);
        tk++;
        mbar_arrive_expect_tx(full0 + 8 * stage, stage_bytes(k.c));
        last_parity = (last_parity & ~(1u << stage)) | (phase << stage);
        load_p(k, stage);
        load_q(k, stage);
        if (++stage == STAGES) stage = 0, phase ^= 1;
      }
      // Everything this CTA reads from HBM has been requested: kernels queued behind this one may be scheduled
      // (once every CTA says so). They wait for this grid to finish before touching what it reads or writes; what
      // they may do at once, as SMs free up, is set up and pull their own weights into shared memory.
      pdl_trigger();
      if (!ok) {
        // Unwinding: let every copy that was started land before the CTA gives its shared memory back.
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
      Works it(p);
      Work w;
      int stage = 0, tk = 0, nseg = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; ok && it.next(w); i++) {
        const int buf = i % C::kAccBufs, use = i / C::kAccBufs;
        if (!mbar_wait_bounded(aempty0 + 8 * buf, (use & 1) ^ 1, abort_flag, &g_status, kStatusAccumFreeTimeout))
          break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * NB;
        uint32_t accumulate = 0;
        for (int c = w.c0; c < w.c1; c++) {
          // the scale feeders arrive here once the stage has landed and its scales are in tensor memory
          if (!mbar_wait_bounded(sfr0 + 8 * stage, phase, abort_flag, &g_status, kStatusFullWaitTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          TRACE(1, tk);
          const int nsteps = min(4, p.ksteps - 4 * c);
          const uint32_t sbase = smem_base + stage * C::kStageBytes;
          const uint64_t desc_p = umma_desc_k_sw128(sbase), desc_q = umma_desc_k_sw128(sbase + C::kOffQ);
          const uint32_t sf_col = tmem_base + C::kSfCol0 + C::kSfCols * stage;
          for (int ks = 0; ks < nsteps; ks++) {
            // 64 E2M1 = 32 bytes further along K inside the 128-byte swizzle span: +2 in 16-byte address units
            umma_nvfp4(d_tmem, desc_p + 2 * ks, desc_q + 2 * ks, idesc, sf_col + 4 * ks,
                       sf_col + 16 + 4 * C::kQAtoms * ks, accumulate);
            accumulate = 1;
          }
          umma_commit(empty0 + 8 * stage);  // the stage is free once these MMAs have read it
          TRACE(2, tk);
          tk++;
          if (++stage == STAGES) stage = 0, phase ^= 1;
        }
        if (ok) umma_commit(afull0 + 8 * buf);
        nseg = i + 1;
      }
      // Tensor memory is freed by this warp: not before the epilogue has read the last accumulators.
      for (int j = nseg - 1; ok && j >= 0 && j >= nseg - C::kAccBufs; j--)
        ok = mbar_wait_bounded(aempty0 + 8 * (j % C::kAccBufs), (j / C::kAccBufs) & 1, abort_flag, &g_status,
                               kStatusAccumFreeTimeout, 64);
    }
  } else if (warp >= C::kFeederWarp0) {
    // ------------------------------------------------------------------------------------------ scales -> tensor memory
    // One thread of each of the four warps copies its share of a landed stage's scale atoms shared memory -> tensor
    // memory with tcgen05.cp (a 512-byte atom becomes 4 columns, replicated to the four lane quarters as the MMA
    // expects): thread j the atoms of MMA step j - one of the M-side operand, one per 128-row block of the N side -
    // and commits; the commit arrives on the barrier the MMA issuer waits on once the copies have completed. (On the
    // MMA-issuing thread itself these copies cost ~90 cycles each and capped the stream; through registers - four warps,
    // tcgen05.st - they cost 16-24 KiB of shared-memory reads per stage and measurably more power.)
    if (lane == 0) {
      const int j = warp - C::kFeederWarp0;
      const uint64_t atom0 = umma_desc_sf_atom(smem_base + C::kOffSfP);  // atoms 0..3: M side; 4..7 (8..11): N side
      int stage = 0;
      uint32_t phase = 0;
      for (Chunks k(p); k.valid; k.advance()) {
        if (!mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag, &g_status, kStatusFullWaitTimeout, 32)) break;
        const uint64_t d0 = atom0 + uint64_t(stage) * (C::kStageBytes >> 4);
        const uint32_t t0 = tmem_base + C::kSfCol0 + C::kSfCols * stage;
        tmem_cp_sf_atom(t0 + 4 * j, d0 + uint64_t(j) * (512 >> 4));
#pragma unroll
        for (int b = 0; b < C::kQAtoms; b++)
          tmem_cp_sf_atom(t0 + 16 + 4 * C::kQAtoms * j + 4 * b, d0 + uint64_t(4 + 4 * b + j) * (512 >> 4));
        umma_commit(sfr0 + 8 * stage);
        if (++stage == STAGES) stage = 0, phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // the 32 tensor-memory lanes this warp may read
    const int row = quarter * 32 + lane;
    Works it(p);
    Work w;
    for (int i = 0; it.next(w); i++) {
      const int buf = i % C::kAccBufs;
      if constexpr (kSwap) {
        if (C::kInKernelReduce && w.slot >= 0 && !p.ext_reduce && threadIdx.x == 64) {  // the partial tiles this cut tile is summed from
          const TileParts t = tile_parts(p.plan, w.tile);
          seg_info[0] = t.n;
          for (int q = 0; q < t.n && q < kMaxParts; q++) seg_info[1 + q] = part_slot(p.plan, t, q);
        }
      }
      if (!warp_wait(afull0 + 8 * buf, (i / C::kAccBufs) & 1, abort_flag, &g_status, kStatusAccumWaitTimeout, 128)) break;
      tc_fence_after_sync();
      if (threadIdx.x == 64 && i < 4) TRACE(3, 4 + i);
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * NB;
      if constexpr (kSwap) {
        // lane = weight row (output channel), column = token
        if (w.slot < 0) {
          for (int m0 = 0; m0 < p.M; m0 += 8) {
            float v[8];
            tmem_ld8(taddr + m0, v);
            tmem_ld_wait();
            store_swapped<kEpi>(p, v, m0, w.tile, row, xchg);
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(aempty0 + 8 * buf);
        } else {
          // A tile cut by a range boundary: leave the partial sums, count the arrival; whoever arrives last sums
          // all partial tiles in ascending K order (whatever the order of arrival) and finishes the tile.
          for (int m0 = 0; m0 < p.M; m0 += 8) {
            float v[8];
            tmem_ld8(taddr + m0, v);
            tmem_ld_wait();
            float* part = p.partials + (int64_t(w.slot) * p.M + m0) * 128 + row;
#pragma unroll
            for (int j = 0; j < 8; j++)
              if (m0 + j < p.M) __stcg(part + j * 128, v[j]);
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(aempty0 + 8 * buf);
          if (!C::kInKernelReduce || p.ext_reduce) continue;  // (uniform) a separate kernel sums the partial tiles
          epi_bar();  // every partial of this CTA is written (and seg_info is visible) ...
          if (threadIdx.x == 64) {
            __threadfence();  // ... and published device-wide before the arrival is counted
            *last_flag = atomicAdd(p.counters + w.tile, 1) == seg_info[0] - 1;
          }
          epi_bar();
          if (*last_flag) {
            __threadfence();
            const int nparts = seg_info[0];
            // (not compiled into the SiLU*mul instantiation: gate | up weights are wide enough not to be cut, and
            //  the extra registers cost that kernel, the one the streaming rate is measured on, 1 % of its speed)
            constexpr bool kFewTokensPath = kEpi != kEpiGluBf16;
            if (kFewTokensPath && p.M <= 2) {
              // one or two tokens (plain decode): eight partial tiles in flight, one round trip for up to 8 parts
              float v[8] = {};
              for (int q0 = 0; q0 < nparts; q0 += 8) {
                float x[8][2];
#pragma unroll
                for (int q = 0; q < 8; q++) {
                  if (q0 + q < nparts) {
                    const float* part = p.partials + int64_t(seg_info[1 + q0 + q]) * p.M * 128 + row;
                    x[q][0] = __ldcg(part);
                    x[q][1] = p.M > 1 ? __ldcg(part + 128) : 0.f;
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
              store_swapped<kEpi>(p, v, 0, w.tile, row, xchg);
            }
            for (int m0 = 0; (!kFewTokensPath || p.M > 2) && m0 < p.M; m0 += 8) {
              float v[8];
              for (int q0 = 0; q0 < nparts; q0 += 4) {  // four partial tiles in flight at a time
                float x[4][8];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                  if (q0 + q < nparts) {
                    const float* part = p.partials + (int64_t(seg_info[1 + q0 + q]) * p.M + m0) * 128 + row;
#pragma unroll
                    for (int j = 0; j < 8; j++) x[q][j] = m0 + j < p.M ? __ldcg(part + j * 128) : 0.f;
                  }
                }
#pragma unroll
                for (int q = 0; q < 4; q++) {
                  if (q0 + q < nparts) {
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j] = (q0 + q == 0) ? x[q][j] : __fadd_rn(v[j], x[q][j]);
                  }
                }
              }
              store_swapped<kEpi>(p, v, m0, w.tile, row, xchg);
            }
            if (threadIdx.x == 64) p.counters[w.tile] = 0;  // the counters are zero again when the kernel ends
            epi_bar();  // seg_info may be rewritten for the next piece only after everyone has used it
          }
        }
      } else {
        // lane = token, column = output channel
        const int m = w.p_row0 + row;
        const bool valid = m < p.M;
        constexpr bool kGlu = epi_is_glu(kEpi);
        auto emit = [&](int c0, const float* g, const float* u) { emit_many<kEpi>(p, m, valid, w.q_row0, c0, g, u); };
        // first column of the u-th unit of 16 outputs: plain 16 u; SiLU*mul: 4 gate units per 128-row block
        auto unit_col = [&](int u) { return kGlu ? (u >> 2) * 128 + (u & 3) * 16 : u * 16; };
        constexpr int kUnits = kGlu ? NB / 32 : NB / 16;
        if constexpr (C::kEpiWarps == 16) {
          // Pull this warp's share of the accumulator into registers in one go, give the accumulator back, then
          // do the arithmetic and the stores while the MMAs of the next tile already run.
          constexpr int kMine = kUnits / 4;
          const int sub = (warp - 2) >> 2;
          float g[kMine][16], u[kGlu ? kMine : 1][16];
#pragma unroll
          for (int j = 0; j < kMine; j++) {
            const int c0 = unit_col(sub + 4 * j);
            tmem_ld16(taddr + c0, g[j]);
            if constexpr (kGlu) tmem_ld16(taddr + 64 + c0, u[j]);
          }
          tmem_ld_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(aempty0 + 8 * buf);
#pragma unroll
          for (int j = 0; j < kMine; j++) emit(unit_col(sub + 4 * j), g[j], u[kGlu ? j : 0]);
        } else {
#pragma unroll 1
          for (int un = 0; un < kUnits; un++) {
            const int c0 = unit_col(un);
            float g[16], u[16];
            tmem_ld16(taddr + c0, g);
            if constexpr (kGlu) tmem_ld16(taddr + 64 + c0, u);
            tmem_ld_wait();
            emit(c0, g, u);
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(aempty0 + 8 * buf);
        }
      }
      if (threadIdx.x == 64 && i < 4) TRACE(3, 8 + i);
    }
  }

  // Teardown: every role is done (or gave up); tensor memory goes back before the CTA exits. The lanes that
  // skipped their warp's single-lane role wait for that lane here: a CTA-wide barrier counts a warp as arrived as
  // soon as any of its lanes arrives, so a warp must reach it converged.
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) TRACE(3, 12);
  if (threadIdx.x == 32) TRACE(3, 13);
  if (threadIdx.x == 64) TRACE(3, 14);
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Many rows on CTA pairs: a cluster of two CTAs on neighbouring SMs computes a 256-token x 256-channel tile with
// tcgen05.mma.cta_group::2. Each CTA loads its own 128 tokens, HALF of the 256 weight rows (the instruction reads
// the other half from the partner's shared memory), its own activation scales and the scales of all 256 weight
// rows: 38 KiB per SM per 256 K-elements for the flops that cost a lone CTA 54 KiB. The kernel with one CTA per
// tile is bound by what an SM can pull from L2 (~48 bytes per clock measured), so this is the way to more flops.
// Rank 0 of the pair issues the MMAs and owns the barriers that gather both CTAs; no load is multicast.
template <int STAGES>
struct Cfg2 {
  static constexpr int kPBytes = 128 * 128, kQBytes = 128 * 128, kSfBytes = 4 * 512;
  static constexpr int kStageBytes = kPBytes + kQBytes + 3 * kSfBytes;  // + scales: own tokens, 2 x 128 weight rows
  static constexpr int kOffQ = kPBytes, kOffSfP = kPBytes + kQBytes, kOffSfQ = kOffSfP + kSfBytes;
  static constexpr int kSfCols = 48;
  static constexpr int kNumBars = 4 * STAGES + 2;  // per slot: landed, free, scales in tensor memory, partner landed; + accumulator full / free
  static constexpr int kOutOff = STAGES * kStageBytes + (kNumBars * 8 + 16 + 15) / 16 * 16;  // staging of an output tile
  static constexpr int kOutBytes = 128 * 256;  // 128 tokens x 128 bf16 outputs (SiLU*mul epilogue)
  static constexpr int kSmemBytes = kOutOff + kOutBytes + 1024;
  static constexpr int kTmemCols = 512, kSfCol0 = 256;
  static constexpr int kEpiWarps = 16, kFeederWarp0 = 2 + kEpiWarps, kThreads = (kFeederWarp0 + 4) * 32;
  static_assert(kStageBytes % 1024 == 0, "stage tiles must stay 1024-byte aligned");
  static_assert(kSfCol0 + kSfCols * STAGES <= kTmemCols, "tensor memory budget");
  static_assert(kSmemBytes + 1024 <= 228 * 1024, "shared memory budget");
};

template <int STAGES, int kEpi>
__global__ void __launch_bounds__(Cfg2<STAGES>::kThreads, 1) umma_gemm2_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                                              const __grid_constant__ CUtensorMap tmap_w,
                                                                              const __grid_constant__ GemmParams p) {
  using C = Cfg2<STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::kStageBytes);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, sfr0 = empty0 + 8 * STAGES, pfull0 = sfr0 + 8 * STAGES,
                 afull = pfull0 + 8 * STAGES, aempty = afull + 8;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile uint32_t* abort_flag = tmem_holder + 1;
  volatile uint32_t* epi_ok = tmem_holder + 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: leader
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int m_pairs = (p.M + 255) / 256, items = m_pairs * (p.N / 256);
  const int m_blocks = (p.M + 127) / 128;
  const uint32_t smem_base = smem_u32(smem);

  if (threadIdx.x == 0) {
    TRACE(3, 0);
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_w);
    for (int s = 0; s < STAGES; s++)
      mbar_init(full0 + 8 * s, 1), mbar_init(empty0 + 8 * s, 1), mbar_init(sfr0 + 8 * s, 4), mbar_init(pfull0 + 8 * s, 1);
    mbar_init(afull, 1), mbar_init(aempty, 2 * C::kEpiWarps);
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc_2sm(smem_u32(tmem_holder), C::kTmemCols);
    tmem_relinquish_2sm();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0, tk = 0;
      uint32_t phase = 0, armed = 0, last_parity = 0;
      bool ok = true, waited = false;
      // (the time between a slot coming free and its loads being issued is part of every slot's round trip: per tile the
      //  source pointers are set up once and only stepped per stage)
      for (int item = pair; ok && item < items; item += npairs) {
        const int m0 = (item % m_pairs) * 256 + int(rank) * 128, n0 = (item / m_pairs) * 256;
        const bool sfa_valid = m0 / 128 < m_blocks;  // the partner half of the last token tile may not exist
        const uint8_t* sfq = p.sf_q + int64_t(n0 / 128) * p.ksteps * 512;  // scale atoms of weight rows n0 .. n0 + 127
        const uint8_t* sfp = p.sf_p + int64_t(m0 / 128) * p.ksteps * 512;  // scale atoms of this CTA's tokens
        const int64_t sfq_block = int64_t(p.ksteps) * 512;                 // ... and of the next 128 weight rows
        const int wrow = n0 + int(rank) * 128;
        for (int c = 0; c < p.chunks; c++, sfq += 2048, sfp += 2048) {
          if (!mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1, abort_flag, &g_status, kStatusEmptyWaitTimeout)) {
            ok = false;
            break;
          }
          const uint32_t sf_bytes = uint32_t(min(4, p.ksteps - 4 * c)) * 512;
          const uint32_t sbase = smem_base + stage * C::kStageBytes, bar = full0 + 8 * stage;
          TRACE(0, tk);
          tk++;
          mbar_arrive_expect_tx(bar, C::kPBytes + C::kQBytes + (sfa_valid ? 3 : 2) * sf_bytes);
          armed |= 1u << stage;
          last_parity = (last_parity & ~(1u << stage)) | (phase << stage);
          tma_load_2d(sbase + C::kOffQ, &tmap_w, c * 128, wrow, bar, kEvictNormal);
          bulk_load(sbase + C::kOffSfQ, sfq, sf_bytes, bar, kEvictNormal);
          bulk_load(sbase + C::kOffSfQ + C::kSfBytes, sfq + sfq_block, sf_bytes, bar, kEvictNormal);
          if (!waited) pdl_wait(), waited = true;  // the activations come from the preceding kernel
          tma_load_2d(sbase, &tmap_a, c * 128, m0, bar, kEvictLast);
          if (sfa_valid) bulk_load(sbase + C::kOffSfP, sfp, sf_bytes, bar, kEvictLast);
          if (++stage == STAGES) stage = 0, phase ^= 1;
        }
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
    // ------------------------------------------------------------------------------------------ MMA issuer (leader)
    if (lane == 0 && rank == 0) {
      // This one thread feeds the tensor cores of both SMs, nothing queues behind a tcgen05.mma, and every instruction
      // the thread executes between two MMAs is time the tensor pipe idles. Cycle counts of this thread, per stage of
      // four MMAs (512 cycles at the pipe's rate): fence + MMAs + commit 416, the (always successful) wait for the stage
      // 111, the accumulator 64 - and 380 in the loop around them when that loop dispatched every stage through a
      // switch on the ring slot. So the K loop is straight-line code over one lap of the ring, every shared-memory
      // address, descriptor offset, tensor-memory column and barrier a compile-time constant; it is entered at the slot
      // the ring stands at (one switch per TILE, whose first stage overwrites the accumulator and is an instantiation
      // of its own), and after each stage a single counter says whether the tile is complete.
      static_assert(STAGES == 5, "the issue loop is written out for a ring of five slots");
      constexpr uint32_t idesc = umma_idesc_nvfp4_2sm(256);
      int slot = 0, ntiles = 0;  // slot: where the ring stands (the slot of the next stage)
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t desc_a0 = umma_desc_k_sw128(smem_base), desc_b0 = umma_desc_k_sw128(smem_base + C::kOffQ);
      const uint32_t sf_col0 = tmem_base + C::kSfCol0;
      const int tail_steps = p.ksteps - 4 * (p.chunks - 1);  // MMA steps of a tile's last stage: 4 unless K % 256
      TRACE_DECL(w_stage);
      TRACE_DECL(w_acc);
      TRACE_T0(t_begin);
      TRACE_C0(c_begin);
      TRACE_DECL(w_issue);
      auto stage_body = [&](auto stage_c, auto first_c, bool last) -> bool {
        constexpr int S = decltype(stage_c)::value;
        constexpr bool kFirst = decltype(first_c)::value;
        // four arrivals: the commits of the threads that copied this stage's scales into tensor memory, each after
        // both CTAs' copies of the stage had landed
        TRACE_C0(c_s);
        if (!mbar_wait_bounded(sfr0 + 8 * S, phase, abort_flag, &g_status, kStatusFullWaitTimeout)) return false;
        TRACE_CADD(w_stage, c_s);  // cycles in the wait for the stage (data landed, scales in tensor memory)
        TRACE_C0(c_i);
        tc_fence_after_sync();
        constexpr uint64_t kStageDesc = uint64_t(S) * (C::kStageBytes >> 4);  // the stage's offset in 16-byte units
        const uint64_t da = desc_a0 + kStageDesc, db = desc_b0 + kStageDesc;
        const uint32_t sf = sf_col0 + C::kSfCols * S;
        if (!last || tail_steps == 4) {
          umma_nvfp4_2sm_imm<!kFirst>(tmem_base, da, db, idesc, sf, sf + 16);
          umma_nvfp4_2sm_imm<true>(tmem_base, da + 2, db + 2, idesc, sf + 4, sf + 24);
          umma_nvfp4_2sm_imm<true>(tmem_base, da + 4, db + 4, idesc, sf + 8, sf + 32);
          umma_nvfp4_2sm_imm<true>(tmem_base, da + 6, db + 6, idesc, sf + 12, sf + 40);
        } else {
          for (int ks = 0; ks < tail_steps; ks++)
            umma_nvfp4_2sm(tmem_base, da + 2 * ks, db + 2 * ks, idesc, sf + 4 * ks, sf + 16 + 8 * ks, (kFirst && ks == 0) ? 0u : 1u);
        }
        umma_commit_2sm(empty0 + 8 * S);  // frees the stage in both CTAs
        TRACE_CADD(w_issue, c_i);  // cycles from the fence to after the commit: the stage's MMAs
        return true;
      };
      using std::integral_constant;
      // One stage in slot S; leaves the K loop when the thread gave up or the tile is complete.
#define Q27B_ISSUE_STAGE(S, FIRST)                                                        \
  {                                                                                       \
    if (!stage_body(integral_constant<int, S>(), FIRST(), remaining == 1)) {              \
      ok = false;                                                                         \
      goto issue_done;                                                                    \
    }                                                                                     \
    if (S == STAGES - 1) phase ^= 1;                                                      \
    if (--remaining == 0) {                                                               \
      slot = (S + 1) % STAGES;                                                            \
      goto tile_done;                                                                     \
    }                                                                                     \
  }
      for (int item = pair; item < items; item += npairs, ntiles++) {
        // both CTAs' epilogues have read the accumulators of the previous tile
        TRACE_C0(c_e);
        if (!mbar_wait_bounded(aempty, (ntiles & 1) ^ 1, abort_flag, &g_status, kStatusAccumFreeTimeout, 0, true)) {
          ok = false;
          break;
        }
        TRACE_CADD(w_acc, c_e);
        tc_fence_after_sync();
        {
          int remaining = p.chunks;
          switch (slot) {  // the tile's first stage, in whatever slot the ring stands at; then on into the lap
            case 0: Q27B_ISSUE_STAGE(0, std::true_type) goto lap1;
            case 1: Q27B_ISSUE_STAGE(1, std::true_type) goto lap2;
            case 2: Q27B_ISSUE_STAGE(2, std::true_type) goto lap3;
            case 3: Q27B_ISSUE_STAGE(3, std::true_type) goto lap4;
            default: Q27B_ISSUE_STAGE(4, std::true_type) goto lap0;
          }
          for (;;) {
          lap0:
            Q27B_ISSUE_STAGE(0, std::false_type)
          lap1:
            Q27B_ISSUE_STAGE(1, std::false_type)
          lap2:
            Q27B_ISSUE_STAGE(2, std::false_type)
          lap3:
            Q27B_ISSUE_STAGE(3, std::false_type)
          lap4:
            Q27B_ISSUE_STAGE(4, std::false_type)
          }
        }
      tile_done:
        umma_commit_2sm(afull);
      }
    issue_done:
#undef Q27B_ISSUE_STAGE
      TRACE_PUT(58, w_stage);
      TRACE_PUT(59, w_acc);
      TRACE_PUT(60, gtime() - t_begin);
      TRACE_PUT(61, (unsigned long long)ntiles);
      TRACE_CPUT(62, c_begin);  // with 60: the SM clock this kernel really ran at
      TRACE_PUT(63, w_issue);    // 58, 59, 63: cycles waiting for stages / for the accumulator / issuing; 62: all cycles
      if (ok && ntiles > 0) mbar_wait_bounded(aempty, (ntiles - 1) & 1, abort_flag, &g_status, kStatusAccumFreeTimeout, 64, true);
    }
  } else if (warp >= C::kFeederWarp0) {
    // ------------------------------------------------------------------------------------------ scales -> tensor memory
    // Four threads of the LEADER copy the scale atoms of a landed stage into tensor memory with tcgen05.cp: one
    // instruction moves a 512-byte atom of each CTA of the pair from that CTA's shared memory into that CTA's tensor
    // memory (4 columns, replicated to the four lane quarters as the MMA expects). Three atoms per thread and stage, then
    // a commit that arrives on the barrier the MMA issuer waits on. The partner's only part is to say when its copy of
    // the stage has landed. (Before: four warps in each CTA moved the atoms shared memory -> registers -> tcgen05.st,
    // 24 KiB of shared-memory reads per CTA and stage; timing runs with those copies left out were 4 % faster cold and
    // 11 % faster once the power cap had acted.)
    if (lane == 0) {
      const int j = warp - C::kFeederWarp0;  // 0..3
      int stage = 0, tkf = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (rank != 0) {
        if (j == 0) {
          for (int item = pair; ok && item < items; item += npairs)
            for (int c = 0; c < p.chunks; c++) {
              if (!mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag, &g_status, kStatusFullWaitTimeout)) {
                ok = false;
                break;
              }
              mbar_arrive_remote(pfull0 + 8 * stage, 0);
              if (++stage == STAGES) stage = 0, phase ^= 1;
            }
        }
      } else {
        const uint64_t atom0 = umma_desc_sf_atom(smem_base + C::kOffSfP);  // atoms 0..3: tokens; 4..7, 8..11: the two blocks of weight rows
        for (int item = pair; ok && item < items; item += npairs)
          for (int c = 0; c < p.chunks; c++) {
            if (!mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag, &g_status, kStatusFullWaitTimeout) ||
                !mbar_wait_bounded(pfull0 + 8 * stage, phase, abort_flag, &g_status, kStatusFullWaitTimeout, 0, true)) {
              ok = false;
              break;
            }
            if (j == 0 && tkf >= 24 && tkf < 44) TRACE(3, 16 + 2 * (tkf - 24));
            const uint64_t d0 = atom0 + uint64_t(stage) * (C::kStageBytes >> 4);
            const uint32_t t0 = tmem_base + C::kSfCol0 + C::kSfCols * stage;
            // thread j: the token atom of MMA step j, and the weight atoms of step j for both blocks of 128 rows
            tmem_cp_sf_atom_2sm(t0 + 4 * j, d0 + uint64_t(j) * (512 >> 4));
            tmem_cp_sf_atom_2sm(t0 + 16 + 8 * j, d0 + uint64_t(4 + j) * (512 >> 4));
            tmem_cp_sf_atom_2sm(t0 + 20 + 8 * j, d0 + uint64_t(8 + j) * (512 >> 4));
            umma_commit_2sm_local(sfr0 + 8 * stage);
            if (j == 0 && tkf >= 24 && tkf < 44) TRACE(3, 17 + 2 * (tkf - 24));
            tkf++;
            if (++stage == STAGES) stage = 0, phase ^= 1;
          }
      }
    }
  } else {
    // ------------------------------------------------------------------------------------------ epilogue
    const int quarter = warp & 3, sub = (warp - 2) >> 2, row = quarter * 32 + lane;
    const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16);
    constexpr bool kGlu = epi_is_glu(kEpi);
    constexpr int kUnits = kGlu ? 8 : 16, kMine = kUnits / 4;
    int ntiles = 0;
    for (int item = pair; item < items; item += npairs, ntiles++) {
      const int m = (item % m_pairs) * 256 + int(rank) * 128 + row, n0 = (item / m_pairs) * 256;
      // One warp watches the accumulator barrier closely; the other fifteen sleep in a hardware barrier until it has
      // seen the MMAs complete (sixteen polling warps would either poll rarely or crowd the shared-memory pipe).
      if (warp == 2) {
        const bool done = warp_wait(afull, ntiles & 1, abort_flag, &g_status, kStatusAccumWaitTimeout, 20);
        if (lane == 0) *epi_ok = done;
      }
      asm volatile("bar.sync 2, %0;" ::"r"(C::kEpiWarps * 32) : "memory");
      if (!*epi_ok) break;
      mbar_wait_bounded(afull, ntiles & 1, abort_flag, &g_status, kStatusAccumWaitTimeout);  // (every thread observes the phase itself)
      tc_fence_after_sync();
      if (warp == 2 && lane == 0 && ntiles < 4) TRACE(3, 4 + ntiles);
      float g[kMine][16], u[kGlu ? kMine : 1][16];
#pragma unroll
      for (int j = 0; j < kMine; j++) {
        const int un = sub + 4 * j, c0 = kGlu ? (un >> 2) * 128 + (un & 3) * 16 : un * 16;
        tmem_ld16(taddr + c0, g[j]);
        if constexpr (kGlu) tmem_ld16(taddr + 64 + c0, u[j]);
      }
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(aempty);
        else mbar_arrive_remote(aempty, 0);
      }
      if (warp == 2 && lane == 0 && ntiles < 4) TRACE(3, 8 + ntiles);
      if constexpr (kEpi == kEpiGluBf16) {
        // The CTA's 128 tokens x 128 outputs go through shared memory so that global memory (this GPU's and, with the
        // fused gather, the peers') is written in whole 256-byte rows: a lane holds one token, so direct stores would
        // be 32-byte pieces of 32 different rows per instruction - 1.4 x the bytes in local DRAM traffic, and far worse
        // as NVLink packets. 16-byte chunks are XOR-swizzled by the row so that neither side has bank conflicts.
        uint8_t* stage_out = smem + C::kOutOff;
        const float ag = p.alpha.alpha[0], au = p.alpha_up;
        asm volatile("bar.sync 3, %0;" ::"r"(C::kEpiWarps * 32) : "memory");  // the previous tile has left the staging area
#pragma unroll
        for (int j = 0; j < kMine; j++) {
          const int un = sub + 4 * j, chunk0 = (un >> 2) * 8 + (un & 3) * 2;  // first of the unit's two 16-byte chunks
          uint32_t pk[8];
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const uint32_t lo = bf16_bits(silu_mul(__fmul_rn(ag, g[j][2 * i]), __fmul_rn(au, u[j][2 * i])));
            const uint32_t hi = bf16_bits(silu_mul(__fmul_rn(ag, g[j][2 * i + 1]), __fmul_rn(au, u[j][2 * i + 1])));
            pk[i] = lo | (hi << 16);
          }
          uint4* r = reinterpret_cast<uint4*>(stage_out + row * 256);
          r[chunk0 ^ (row & 15)] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          r[(chunk0 + 1) ^ (row & 15)] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
        asm volatile("bar.sync 3, %0;" ::"r"(C::kEpiWarps * 32) : "memory");
        const int m_base = (item % m_pairs) * 256 + int(rank) * 128, chunk = lane & 15;
        uint16_t* out0 = static_cast<uint16_t*>(p.d) + n0 / 2 + chunk * 8;
#pragma unroll
        for (int it = 0; it < 4; it++) {  // a warp copies 8 rows, two per instruction: 2 x 256 contiguous bytes
          const int r = (warp - 2) * 8 + it * 2 + (lane >> 4), mr = m_base + r;
          if (mr < p.M) {
            const uint4 v = reinterpret_cast<const uint4*>(stage_out + r * 256)[chunk ^ (r & 15)];
            uint4* dst = reinterpret_cast<uint4*>(out0 + int64_t(mr) * (p.N / 2));
            *dst = v;
            for (int q = 0; q < p.n_peers; q++) *reinterpret_cast<uint4*>(reinterpret_cast<char*>(dst) + p.peer_delta[q]) = v;
          }
        }
      } else if constexpr (kEpi == kEpiBf16 || kEpi == kEpiF32) {
        // The same whole-row stores for the plain epilogues: the CTA's 128 tokens x 256 channels leave in passes of
        // 256 bytes per token (bf16: two passes of 128 channels; fp32: four of 64), staged as above. The residual of
        // the fp32 epilogue is added on the way out, where a warp reads it in whole rows too: the same
        // fma(beta, c, alpha * acc) as finish_f32, so the bits do not depend on which path stored them.
        uint8_t* stage_out = smem + C::kOutOff;
        constexpr int kPasses = kEpi == kEpiBf16 ? 2 : 4, kPerPass = kMine / kPasses, kPassCols = 256 / kPasses;
        const int m_base = (item % m_pairs) * 256 + int(rank) * 128, chunk = lane & 15;
#pragma unroll
        for (int ps = 0; ps < kPasses; ps++) {
          asm volatile("bar.sync 3, %0;" ::"r"(C::kEpiWarps * 32) : "memory");  // the previous pass has left the staging area
#pragma unroll
          for (int jj = 0; jj < kPerPass; jj++) {
            const int j = ps * kPerPass + jj, un = sub + 4 * j, col = un * 16, n = n0 + col;
            uint4* r = reinterpret_cast<uint4*>(stage_out + row * 256);
            float out[16];
#pragma unroll
            for (int i = 0; i < 16; i++) {
              out[i] = __fmul_rn(alpha_of(p.alpha, n + i), g[j][i]);
              if (p.wscale) out[i] = __fmul_rn(out[i], __fmul_rn(p.wscale[n + i], p.ascale[min(m, p.M - 1)]));
            }
            if constexpr (kEpi == kEpiBf16) {
              const int chunk0 = (col - ps * kPassCols) / 8;
              uint32_t pk[8];
#pragma unroll
              for (int i = 0; i < 8; i++) pk[i] = uint32_t(bf16_bits(out[2 * i])) | (uint32_t(bf16_bits(out[2 * i + 1])) << 16);
              r[chunk0 ^ (row & 15)] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              r[(chunk0 + 1) ^ (row & 15)] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            } else {
              const int chunk0 = (col - ps * kPassCols) / 4;
#pragma unroll
              for (int i = 0; i < 4; i++)
                r[(chunk0 + i) ^ (row & 15)] = make_uint4(__float_as_uint(out[4 * i]), __float_as_uint(out[4 * i + 1]),
                                                          __float_as_uint(out[4 * i + 2]), __float_as_uint(out[4 * i + 3]));
            }
          }
          asm volatile("bar.sync 3, %0;" ::"r"(C::kEpiWarps * 32) : "memory");
          constexpr int kElem = kEpi == kEpiBf16 ? 2 : 4;
          char* out0 = static_cast<char*>(p.d) + (int64_t(n0) + ps * kPassCols) * kElem + chunk * 16;
#pragma unroll
          for (int it = 0; it < 4; it++) {  // a warp copies 8 rows, two per instruction: 2 x 256 contiguous bytes
            const int rr = (warp - 2) * 8 + it * 2 + (lane >> 4), mr = m_base + rr;
            if (mr < p.M) {
              uint4 v = reinterpret_cast<const uint4*>(stage_out + rr * 256)[chunk ^ (rr & 15)];
              const int64_t off = int64_t(mr) * p.N * kElem;
              if constexpr (kEpi == kEpiF32) {
                if (p.c) {
                  const float4 c = *reinterpret_cast<const float4*>(reinterpret_cast<const char*>(p.c) + (out0 - static_cast<char*>(p.d)) + off);
                  v.x = __float_as_uint(__fmaf_rn(p.beta, c.x, __uint_as_float(v.x)));
                  v.y = __float_as_uint(__fmaf_rn(p.beta, c.y, __uint_as_float(v.y)));
                  v.z = __float_as_uint(__fmaf_rn(p.beta, c.z, __uint_as_float(v.z)));
                  v.w = __float_as_uint(__fmaf_rn(p.beta, c.w, __uint_as_float(v.w)));
                }
              }
              *reinterpret_cast<uint4*>(out0 + off) = v;
            }
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < kMine; j++) {
          const int un = sub + 4 * j, c0 = kGlu ? (un >> 2) * 128 + (un & 3) * 16 : un * 16;
          emit_many<kEpi>(p, m, m < p.M, n0, c0, g[j], u[kGlu ? j : 0]);
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // nothing of either CTA goes away while the other may still signal it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_2sm(tmem_base, C::kTmemCols);
  }
  if (p.n_peers > 0 && threadIdx.x == 0) {
    // every store of this CTA (local and into the peers) is ordered before the count; the CTA that counts last orders
    // all of them before it raises this GPU's word in every peer's signal block (words as in skinny_group.inl)
    __threadfence_system();
    if (atomicAdd(p.signals + 9, 1) == int(gridDim.x) - 1) {
      p.signals[9] = 0;
      __threadfence_system();
      for (int j = 0; j < p.n_peers; j++) atomicAdd_system(p.peer_signals[j] + p.my_slot, 1);
    }
  }
}

// Self-test of the bounded waits: one thread waits on a barrier that nothing ever arrives at, with a short budget;
// the wait must give up by itself, raise the status word and let the kernel end normally.
__global__ void wait_timeout_probe_kernel(long long max_cycles) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    mbar_init_fence();
    mbar_wait_bounded(smem_u32(&bar), 0, &abort_flag, &g_status, kStatusProbeTimeout, 64, false, max_cycles);
  }
}

// Sums the partial tiles of every cut weight tile in ascending K order and applies the epilogue: the same
// arithmetic as the in-kernel reduction, spread over the whole GPU. Used when there are many tokens (the in-kernel
// reduction leaves a cut tile to the one CTA that arrives last). Block = (tile, group of 8 tokens), thread = row.
template <int kEpi>
__global__ void __launch_bounds__(128) skinny_fixup_kernel(const __grid_constant__ GemmParams p) {
  pdl_trigger();
  const int tile = blockIdx.x, row = threadIdx.x;
  const TileParts t = tile_parts(p.plan, tile);
  if (t.n == 1) return;  // finished in place by its only owner
  __shared__ float xchg[8 * 64];
  const int m0 = blockIdx.y * 8;
  pdl_wait();
  float v[8];
  for (int q0 = 0; q0 < t.n; q0 += 8) {  // eight partial tiles in flight at a time, summed in ascending K order
    float x[8][8];
#pragma unroll
    for (int q = 0; q < 8; q++) {
      if (q0 + q < t.n) {
        const float* part = p.partials + (int64_t(part_slot(p.plan, t, q0 + q)) * p.M + m0) * 128 + row;
#pragma unroll
        for (int j = 0; j < 8; j++) x[q][j] = m0 + j < p.M ? __ldcg(part + j * 128) : 0.f;
      }
    }
#pragma unroll
    for (int q = 0; q < 8; q++) {
      if (q0 + q < t.n) {
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = (q0 + q == 0) ? x[q][j] : __fadd_rn(v[j], x[q][j]);
      }
    }
  }
  if constexpr (kEpi == kEpiGluBf16) {
    if (row >= 64) {
#pragma unroll
      for (int j = 0; j < 8; j++) xchg[j * 64 + row - 64] = v[j];
    }
    __syncthreads();
    if (row < 64) {
      const float ag = p.alpha.alpha[0], au = p.alpha_up;
      uint16_t* d = static_cast<uint16_t*>(p.d) + int64_t(tile) * 64 + row;
#pragma unroll
      for (int j = 0; j < 8; j++)
        if (m0 + j < p.M)
          d[int64_t(m0 + j) * (p.N / 2)] = bf16_bits(silu_mul(__fmul_rn(ag, v[j]), __fmul_rn(au, xchg[j * 64 + row])));
    }
  } else {
    const int n = tile * 128 + row;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int m = m0 + j;
      if (m < p.M) {
        const float out = finish_f32(p, v[j], m, n);
        if constexpr (kEpi == kEpiF32) static_cast<float*>(p.d)[int64_t(m) * p.N + n] = out;
        else static_cast<uint16_t*>(p.d)[int64_t(m) * p.N + n] = bf16_bits(out);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ host side

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &f, 12000, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// Rows of K/2 packed bytes, loaded as boxes of 128 bytes x box_rows with the 128-byte swizzle; rows past `rows`
// read as zero.
int make_operand_map(CUtensorMap* map, const uint8_t* base, int rows, int K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  Q27B_REQUIRE(fn, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {cuuint64_t(K / 2), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(K / 2)};
  const cuuint32_t box[2] = {128u, cuuint32_t(box_rows)};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  Q27B_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed (%d) for rows=%d K=%d box_rows=%d", int(r), rows, K,
               box_rows);
  return 0;
}

template <typename Kern>
int launch_gemm(Kern kernel, int grid, int threads, int smem, cudaStream_t s, const CUtensorMap& mp,
                const CUtensorMap& mq, const GemmParams& p, bool pdl) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(threads), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
  Q27B_CUDA(cudaLaunchKernelEx(&cfg, kernel, mp, mq, p));
  return 0;
}

// One-time opt-in to large dynamic shared memory, per kernel instantiation and per device.
template <int NB, int STAGES, int CTAS, bool kSwap, int kEpi>
int ensure_smem() {
  static bool done[64] = {};  // one array per instantiation
  int dev = 0;
  Q27B_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && done[dev]) return 0;
  Q27B_CUDA(cudaFuncSetAttribute(umma_gemm_kernel<NB, STAGES, CTAS, kSwap, kEpi>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<NB, STAGES, CTAS, kSwap>::kSmemBytes));
  if (dev < 64) done[dev] = true;
  return 0;
}

template <int NB, int STAGES, int CTAS, int kEpi>
int run_skinny(const uint8_t* a, const uint8_t* w, GemmParams& p, cudaStream_t s) {
  using C = Cfg<NB, STAGES, CTAS, true>;
  auto kernel = umma_gemm_kernel<NB, STAGES, CTAS, true, kEpi>;
  if (int rc = ensure_smem<NB, STAGES, CTAS, true, kEpi>()) return rc;
  CUtensorMap mp, mq;
  if (int rc = make_operand_map(&mp, w, p.N, p.K, 128)) return rc;
  if (int rc = make_operand_map(&mq, a, p.M, p.K, NB)) return rc;
  const int grid = (p.plan.grid + C::kRangesPerCta - 1) / C::kRangesPerCta;
  if (int rc = launch_gemm(kernel, grid, C::kThreads, C::kSmemBytes, s, mp, mq, p, true)) return rc;
  if (p.ext_reduce) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.plan.tiles, (p.M + 7) / 8), cfg.blockDim = dim3(128), cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = pdl_enabled() ? 1 : 0;
    Q27B_CUDA(cudaLaunchKernelEx(&cfg, skinny_fixup_kernel<kEpi>, p));
  }
  return 0;
}

template <int kEpi>
int skinny_dispatch(const uint8_t* a, const uint8_t* w, GemmParams& p, cudaStream_t s) {
  if (p.M <= 16) return run_skinny<16, 4, 2, kEpi>(a, w, p, s);
  if (p.M <= 32) return run_skinny<32, 4, 2, kEpi>(a, w, p, s);
  if (p.M <= 64) return run_skinny<64, 3, 2, kEpi>(a, w, p, s);
  return run_skinny<128, 3, 2, kEpi>(a, w, p, s);
}

int check_operands(const char* what, int M, int N, int K, const void* a, const void* a_sf, const void* w,
                   const void* w_sf, const void* d) {
  Q27B_REQUIRE(N > 0 && N % 128 == 0, "%s: N must be a positive multiple of 128 (N = %d)", what, N);
  Q27B_REQUIRE(K > 0 && K % 64 == 0, "%s: K must be a positive multiple of 64 (K = %d)", what, K);
  Q27B_REQUIRE(a && a_sf && w && w_sf && d, "%s: null pointer", what);
  Q27B_REQUIRE(aligned16(a) && aligned16(a_sf) && aligned16(w) && aligned16(w_sf) && aligned16(d),
               "%s: operands, scales and output must be 16-byte aligned", what);
  (void)M;
  return 0;
}

int many_common(int kEpi, int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                const uint8_t* w_sf, float alpha, float alpha_up, const float* c, float beta, void* d, cudaStream_t s,
                uint8_t* d_sf, float out_scale, const q27b_group_peers* peers = nullptr);

int skinny_common(int kEpi, int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                  const uint8_t* w_sf, const AlphaSeg& alpha, float alpha_up, const float* c, float beta, void* d,
                  void* ws, size_t ws_bytes, cudaStream_t s, const float* wscale = nullptr, const float* ascale = nullptr) {
  Q27B_REQUIRE(M >= 1 && M <= 128, "skinny_fp4: M must be 1..128 (M = %d)", M);
  if (int rc = check_operands("skinny_fp4", M, N, K, a, a_sf, w, w_sf, d)) return rc;
  Q27B_REQUIRE(alpha.count >= 1 && alpha.count <= 4, "skinny_fp4: 1..4 alpha segments");
  const int sms = sm_count();
  Q27B_REQUIRE(sms > 0, "skinny_fp4: no CUDA device");
  // More than 32 tokens on a weight with about one 256-row tile per SM or more (gate | up, lm_head): the many-row
  // tiles of 128 tokens x 256 weight rows stream it faster (22.7 against 25.7 us at 64 tokens, 23.7 against 33.4 at
  // 128 for gate | up). Neither kernel splits K on such a weight, both accumulate a dot product over the same
  // 64-element steps in the same order, and their results are bit-identical (asserted by the tests), so a token's
  // row still does not depend on M.
  if (M > 32 && !wscale && alpha.count == 1 && N % 256 == 0 && K % 128 == 0 && N / 256 >= 3 * sms / 4 &&
      !plan_cuts_tiles(choose_skinny_plan(N, K, 2 * sms)))
    return many_common(kEpi, M, N, K, a, a_sf, w, w_sf, alpha.alpha[0], alpha_up, c, beta, d, s, nullptr, 1.f);
  GemmParams p = {};
  p.M = M, p.N = N, p.K = K, p.ksteps = K / 64, p.chunks = (p.ksteps + 3) / 4;
  p.sf_p = w_sf, p.sf_q = a_sf, p.alpha = alpha, p.alpha_up = alpha_up, p.c = c, p.beta = beta, p.d = d;
  p.wscale = wscale, p.ascale = ascale;
  // Two CTA slots per SM whatever M: the split depends on the weight's shape only, so a token's result is the
  // same whatever M it is computed with (the reference's invariant for its M <= 64 path, engine/src/skinny.cu:142-147).
  p.plan = choose_skinny_plan(N, K, 2 * sms);
  // Cut tiles: up to 8 tokens the last CTA to arrive sums them inside the kernel; above, a second small kernel
  // does it across the whole GPU (measured cross-over on B200; Q27_SKINNY_EXT_REDUCE_M moves it, as the reference's
  // switch of the same name does, engine/src/skinny.cu:494-521). Both ways add the parts in ascending K order.
  p.ext_reduce = plan_cuts_tiles(p.plan) && M > env_int("Q27_SKINNY_EXT_REDUCE_M", 8, 0, 16);
  Q27B_REQUIRE(p.plan.grid <= kMaxParts, "skinny_fp4: more than %d CTAs", kMaxParts);
  Q27B_REQUIRE(p.plan.tiles * 4 <= kCounterBytes, "skinny_fp4: N too large (%d rows, at most %d)", N, kCounterBytes / 4 * 128);
  const size_t need = size_t(kCounterBytes + skinny_workspace_bytes(M, p.plan));
  Q27B_REQUIRE(ws && aligned16(ws) && ws_bytes >= need, "skinny_fp4: workspace too small (%zu bytes, need %zu)", ws_bytes,
               need);
  p.counters = static_cast<int*>(ws);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + kCounterBytes);
#ifdef Q27B_TRACE
  p.trace = g_trace;
#endif
  switch (kEpi) {
    case kEpiF32: return skinny_dispatch<kEpiF32>(a, w, p, s);
    case kEpiBf16: return skinny_dispatch<kEpiBf16>(a, w, p, s);
    default: return skinny_dispatch<kEpiGluBf16>(a, w, p, s);
  }
}

template <int NB, int STAGES, int CTAS, int kEpi>
int run_many_cfg(const uint8_t* a, const uint8_t* w, GemmParams& p, cudaStream_t s) {
  using C = Cfg<NB, STAGES, CTAS, false>;
  auto kernel = umma_gemm_kernel<NB, STAGES, CTAS, false, kEpi>;
  if (int rc = ensure_smem<NB, STAGES, CTAS, false, kEpi>()) return rc;
  p.n_tile = NB, p.items = p.m_tiles * (p.N / NB);
  CUtensorMap mp, mq;
  if (int rc = make_operand_map(&mp, a, p.M, p.K, 128)) return rc;
  if (int rc = make_operand_map(&mq, w, p.N, p.K, NB)) return rc;
  const int slots = CTAS * sm_count();
  return launch_gemm(kernel, p.items < slots ? p.items : slots, C::kThreads, C::kSmemBytes, s, mp, mq, p, true);
}

template <int kEpi, int STAGES = 5>
int run_many_pairs(const uint8_t* a, const uint8_t* w, GemmParams& p, cudaStream_t s) {
  using C = Cfg2<STAGES>;
  auto kernel = umma_gemm2_kernel<STAGES, kEpi>;
  static bool done[64] = {};
  int dev = 0;
  Q27B_CUDA(cudaGetDevice(&dev));
  if (!(dev < 64 && done[dev])) {
    Q27B_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    if (dev < 64) done[dev] = true;
  }
  CUtensorMap ma, mw;
  if (int rc = make_operand_map(&ma, a, p.M, p.K, 128)) return rc;
  if (int rc = make_operand_map(&mw, w, p.N, p.K, 128)) return rc;
  const int items = ((p.M + 255) / 256) * (p.N / 256), pairs = std::min(items, sm_count() / 2);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs), cfg.blockDim = dim3(C::kThreads), cfg.dynamicSmemBytes = C::kSmemBytes, cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = pdl_enabled() ? 2 : 1;
  Q27B_CUDA(cudaLaunchKernelEx(&cfg, kernel, ma, mw, p));
  return 0;
}

// The optional libq27b200_quad.so (quad_gemm.cu: clusters of four CTAs that share their weight tile), looked for once
// beside this library. It is a single-GPU accelerator: a process that does not find it runs the pair kernel.
struct QuadLib {
  QuadGemmFn gemm = nullptr;
  QuadErrorFn error = nullptr;
};
const QuadLib& quad_lib() {
  static const QuadLib lib = [] {
    QuadLib l;
    Dl_info info;
    if (!dladdr(reinterpret_cast<const void*>(&q27b_device_status), &info) || !info.dli_fname) return l;
    std::string path = info.dli_fname;
    const size_t slash = path.rfind('/');
    path = (slash == std::string::npos ? std::string(".") : path.substr(0, slash)) + "/libq27b200_quad.so";
    if (void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL)) {
      l.gemm = reinterpret_cast<QuadGemmFn>(dlsym(h, "q27b_quad_gemm"));
      l.error = reinterpret_cast<QuadErrorFn>(dlsym(h, "q27b_quad_last_error"));
      if (!l.gemm || !l.error) l = QuadLib();
    }
    return l;
  }();
  return lib;
}

template <int kEpi>
int run_many_quad(const uint8_t* a, const uint8_t* w, const GemmParams& p, cudaStream_t s) {
  const QuadLib& lib = quad_lib();
  QuadParams qp = {};
  qp.M = p.M, qp.N = p.N, qp.K = p.K, qp.ksteps = p.ksteps, qp.chunks = p.chunks, qp.sf_p = p.sf_p, qp.sf_q = p.sf_q;
  qp.alpha = p.alpha.alpha[0], qp.alpha_up = p.alpha_up, qp.c = p.c, qp.beta = p.beta, qp.d = p.d, qp.epi = kEpi;
  qp.status = device_status_ptr();
  Q27B_REQUIRE(qp.status, "gemm_fp4: no device status word");
  CUtensorMap ma, mw;
  if (int rc = make_operand_map(&ma, a, p.M, p.K, 128)) return rc;
  if (int rc = make_operand_map(&mw, w, p.N, p.K, 64)) return rc;
  if (lib.gemm(&ma, &mw, &qp, s)) return fail("%s", lib.error());
  return 0;
}

// Which many-row kernel runs (read at every launch): Q27B_MANY=quad|pairs|wide|narrow forces one, else the best that
// the shape allows.
template <int kEpi>
int run_many(const uint8_t* a, const uint8_t* w, GemmParams& p, cudaStream_t s) {
  const char* e = getenv("Q27B_MANY");
  const bool force_wide = e && !strcmp(e, "wide"), force_narrow = e && !strcmp(e, "narrow");
  const bool force_quad = e && !strcmp(e, "quad"), free_choice = !e || !*e;
  if constexpr (kEpi == kEpiF32 || kEpi == kEpiBf16 || kEpi == kEpiGluBf16) {
    // Clusters of four (two pairs sharing their weight tile, delivered once per cluster): 29 % fewer bytes from L2 per flop.
    const bool fits = p.M > 128 && ((p.M + 255) / 256) % 2 == 0 && p.N % 256 == 0 && p.K % 256 == 0 && !p.n_peers && !p.wscale &&
                      p.alpha.count == 1;
    Q27B_REQUIRE(!force_quad || (fits && quad_lib().gemm), "gemm_fp4: Q27B_MANY=quad, but %s",
                 fits ? "libq27b200_quad.so is not beside this library" : "the shape does not fit (M > 128 in an even number of 256-token tiles, N and K multiples of 256)");
    // Opt-in: measured on this pool it is no faster than the pair kernel (both run into the board's power cap, not
    // into L2 bandwidth), and clusters of four leave SMs unused where a GPC's SM count is not a multiple of four.
    (void)free_choice;
    if (force_quad) return run_many_quad<kEpi>(a, w, p, s);
  } else {
    Q27B_REQUIRE(!force_quad, "gemm_fp4: Q27B_MANY=quad has no NVFP4 epilogue");
  }
  // CTA pairs, 256 x 256 tiles: least L2 traffic per flop. One CTA per 128 x 256 tile where there is less than one
  // pair tile per SM pair to go round. 128 x 128 tiles on two CTAs per SM when the weight rows do not divide by 256.
  if (p.N % 256 == 0 && p.M > 128 && !force_wide && !force_narrow) return run_many_pairs<kEpi>(a, w, p, s);
  if (p.N % 256 == 0 && !force_narrow) return run_many_cfg<256, 4, 1, kEpi>(a, w, p, s);
  return run_many_cfg<128, 3, 2, kEpi>(a, w, p, s);
}

int many_common(int kEpi, int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                const uint8_t* w_sf, float alpha, float alpha_up, const float* c, float beta, void* d, cudaStream_t s,
                uint8_t* d_sf, float out_scale, const q27b_group_peers* peers) {
  Q27B_REQUIRE(M >= 0, "gemm_fp4: M must not be negative");
  if (M == 0) return 0;
  if (int rc = check_operands("gemm_fp4", M, N, K, a, a_sf, w, w_sf, d)) return rc;
  Q27B_REQUIRE(K % 128 == 0, "gemm_fp4: K must be a multiple of 128 (K = %d)", K);
  Q27B_REQUIRE(sm_count() > 0, "gemm_fp4: no CUDA device");
  GemmParams p = {};
  p.M = M, p.N = N, p.K = K, p.ksteps = K / 64, p.chunks = (p.ksteps + 3) / 4;
  p.sf_p = a_sf, p.sf_q = w_sf, p.alpha.count = 1, p.alpha.alpha[0] = alpha, p.alpha_up = alpha_up;
  p.c = (c && beta != 0.f) ? c : nullptr, p.beta = beta, p.d = d;
  p.m_tiles = (M + 127) / 128;
  p.d_sf = d_sf, p.out_gs = 1.f / out_scale;  // (IEEE division, as the quantiser kernels compute it)
  if (peers) {
    Q27B_REQUIRE(kEpi == kEpiGluBf16 && N % 256 == 0 && M > 128, "gemm_fp4 gather: the SiLU*mul bf16 GEMM on CTA pairs only (M > 128, 2 I a multiple of 256)");
    const char* force = getenv("Q27B_MANY");
    Q27B_REQUIRE(!force || !*force || !strcmp(force, "pairs"), "gemm_fp4 gather: Q27B_MANY forces a kernel without the fused gather");
    p.n_peers = peers->n_peers, p.signals = peers->signals, p.my_slot = peers->my_slot;
    for (int j = 0; j < peers->n_peers; j++) p.peer_delta[j] = peers->out_delta[j], p.peer_signals[j] = peers->peer_signals[j];
  }
#ifdef Q27B_TRACE
  p.trace = g_trace;
#endif
  switch (kEpi) {
    case kEpiF32: return run_many<kEpiF32>(a, w, p, s);
    case kEpiBf16: return run_many<kEpiBf16>(a, w, p, s);
    case kEpiGluFp4: return run_many<kEpiGluFp4>(a, w, p, s);
    default: return run_many<kEpiGluBf16>(a, w, p, s);
  }
}

#include "skinny_group.inl"
#include "wide_group.inl"

AlphaSeg make_alpha(int count, const int* begin, const float* alpha) {
  AlphaSeg a = {};
  a.count = count;
  for (int i = 0; i < 4; i++) a.begin[i] = i < count ? begin[i] : 0, a.alpha[i] = i < count ? alpha[i] : 1.f;
  return a;
}

}  // namespace

uint32_t* device_status_ptr() {
  static uint32_t* ptr[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status) != cudaSuccess) return nullptr;
    ptr[dev] = static_cast<uint32_t*>(p);
  }
  return ptr[dev];
}

int sm_count() {
  static int sms[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev >= 64) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
  }
  if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
  return sms[dev];
}

}  // namespace q27b

using namespace q27b;

extern "C" {

int q27b_skinny_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w, const uint8_t* w_sf,
                    int alpha_count, const int* alpha_begin, const float* alpha, const float* c, float beta, float* d,
                    void* ws, size_t ws_bytes, void* stream) {
  Q27B_REQUIRE(alpha_count >= 1 && alpha_count <= 4 && alpha_begin && alpha, "skinny_fp4: 1..4 alpha segments");
  return skinny_common(kEpiF32, M, N, K, a, a_sf, w, w_sf, make_alpha(alpha_count, alpha_begin, alpha), 1.f,
                       (c && beta != 0.f) ? c : nullptr, beta, d, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}
int q27b_skinny_fp4_bf16(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                         const uint8_t* w_sf, int alpha_count, const int* alpha_begin, const float* alpha, void* d,
                         void* ws, size_t ws_bytes, void* stream) {
  Q27B_REQUIRE(alpha_count >= 1 && alpha_count <= 4 && alpha_begin && alpha, "skinny_fp4_bf16: 1..4 alpha segments");
  return skinny_common(kEpiBf16, M, N, K, a, a_sf, w, w_sf, make_alpha(alpha_count, alpha_begin, alpha), 1.f, nullptr,
                       0.f, d, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}
int q27b_skinny_fp4_glu_bf16(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                             const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, void* d, void* ws,
                             size_t ws_bytes, void* stream) {
  Q27B_REQUIRE(I > 0 && I % 64 == 0, "skinny_fp4_glu_bf16: I must be a positive multiple of 64 (I = %d)", I);
  const int zero = 0;
  return skinny_common(kEpiGluBf16, M, 2 * I, K, a, a_sf, gate_up, gate_up_sf, make_alpha(1, &zero, &alpha_gate),
                       alpha_up, nullptr, 0.f, d, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}
int q27b_skinny_fp4_scaled(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const float* ascale,
                           const uint8_t* w, const uint8_t* w_sf, const float* wscale, float* d, void* ws,
                           size_t ws_bytes, void* stream) {
  Q27B_REQUIRE(ascale && wscale, "skinny_fp4_scaled: null scale pointer");
  const int zero = 0;
  const float one = 1.f;
  return skinny_common(kEpiF32, M, N, K, a, a_sf, w, w_sf, make_alpha(1, &zero, &one), 1.f, nullptr, 0.f, d, ws, ws_bytes,
                       static_cast<cudaStream_t>(stream), wscale, ascale);
}
int64_t q27b_skinny_workspace_bytes(int M, int N, int K) {
  const int sms = sm_count();
  if (sms <= 0 || N <= 0 || K <= 0 || M <= 0) return -1;
  return kCounterBytes + skinny_workspace_bytes(M, choose_skinny_plan(N, K, 2 * sms));
}

int q27b_gemm_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
                  float alpha, const float* c, float beta, float* d, void* stream) {
  return many_common(kEpiF32, M, N, K, a, a_sf, b, b_sf, alpha, 1.f, c, beta, d, static_cast<cudaStream_t>(stream), nullptr, 1.f);
}
int q27b_gemm_fp4_bf16(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b,
                       const uint8_t* b_sf, float alpha, void* d, void* stream) {
  return many_common(kEpiBf16, M, N, K, a, a_sf, b, b_sf, alpha, 1.f, nullptr, 0.f, d, static_cast<cudaStream_t>(stream),
                     nullptr, 1.f);
}
int q27b_gemm_fp4_glu_bf16(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                           const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, void* d, void* stream) {
  Q27B_REQUIRE(I > 0 && I % 64 == 0, "gemm_fp4_glu_bf16: I must be a positive multiple of 64 (I = %d)", I);
  return many_common(kEpiGluBf16, M, 2 * I, K, a, a_sf, gate_up, gate_up_sf, alpha_gate, alpha_up, nullptr, 0.f, d,
                     static_cast<cudaStream_t>(stream), nullptr, 1.f);
}
int q27b_gemm_fp4_glu_bf16_gather(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                                  const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, void* d,
                                  const q27b_group_peers* peers, void* stream) {
  Q27B_REQUIRE(I > 0 && I % 64 == 0, "gemm_fp4_glu_bf16_gather: I must be a positive multiple of 64 (I = %d)", I);
  Q27B_REQUIRE(peers && peers->n_peers >= 1 && peers->n_peers <= 7 && peers->signals && peers->my_slot >= 0 && peers->my_slot < 8,
               "gemm_fp4_glu_bf16_gather: 1..7 peers, a signal block and a slot 0..7");
  for (int j = 0; j < peers->n_peers; j++)
    Q27B_REQUIRE(peers->peer_signals[j] && peers->out_delta[j] % 16 == 0, "gemm_fp4_glu_bf16_gather: peer %d: null signal block or misaligned delta", j);
  return many_common(kEpiGluBf16, M, 2 * I, K, a, a_sf, gate_up, gate_up_sf, alpha_gate, alpha_up, nullptr, 0.f, d,
                     static_cast<cudaStream_t>(stream), nullptr, 1.f, peers);
}
int q27b_gemm_fp4_glu(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                      const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, float out_scale, uint8_t* q,
                      uint8_t* q_sf, void* stream) {
  Q27B_REQUIRE(I > 0 && I % 64 == 0, "gemm_fp4_glu: I must be a positive multiple of 64 (I = %d)", I);
  Q27B_REQUIRE(q_sf && aligned16(q_sf), "gemm_fp4_glu: the output scales must be a 16-byte aligned device buffer");
  Q27B_REQUIRE(out_scale > 0.f, "gemm_fp4_glu: out_scale must be positive");
  return many_common(kEpiGluFp4, M, 2 * I, K, a, a_sf, gate_up, gate_up_sf, alpha_gate, alpha_up, nullptr, 0.f, q,
                     static_cast<cudaStream_t>(stream), q_sf, out_scale);
}

int q27b_trace_set(void* buf) {
#ifdef Q27B_TRACE
  g_trace = static_cast<unsigned long long*>(buf);
  return 0;
#else
  Q27B_REQUIRE(!buf, "trace_set: this library was built without the trace points (build with make TRACE=1)");
  return 0;
#endif
}

// ---- the grouped weight-streaming GEMM ------------------------------------------------------------------------------

int q27b_skinny_group_build(int M, int n_problems, const q27b_group_problem* problems, int flags, void* table_host,
                            size_t table_cap, size_t* table_bytes, size_t* ws_bytes) {
  Q27B_REQUIRE((flags & ~(Q27B_GROUP_WHOLE_TILES | Q27B_GROUP_TOKENS_ON_N)) == 0, "skinny_group: unknown flags 0x%x", flags);
  Q27B_REQUIRE(M >= 1 && M <= 128, "skinny_group: M must be 1..128 (M = %d)", M);
  Q27B_REQUIRE(n_problems >= 1 && n_problems <= kGroupMaxProblems && problems, "skinny_group: 1..%d problems", kGroupMaxProblems);
  const int sms = sm_count();
  Q27B_REQUIRE(sms > 0, "skinny_group: no CUDA device");
  std::vector<GroupShape> shapes(n_problems);
  for (int i = 0; i < n_problems; i++) {
    if (int rc = check_group_problem(i, problems[i])) return rc;
    shapes[i] = {problems[i].N, problems[i].K};
  }
  // 33..128 tokens, whole tiles, every weight a multiple of 256 rows: the many-row roles (tokens on the MMA's M side,
  // 256 weight rows per tile, one CTA per SM) bring fewer activation bytes into the SM per weight byte (wide_group.inl)
  bool wide = (flags & Q27B_GROUP_WHOLE_TILES) && !(flags & Q27B_GROUP_TOKENS_ON_N) && M > env_int("Q27_GROUP_WIDE_ABOVE_M", 32, 0, 128);
  for (int i = 0; wide && i < n_problems; i++) wide = problems[i].N % 256 == 0;
  const GroupSchedule sch = wide ? schedule_group(shapes.data(), n_problems, sms, true, false, 256)
                                 : schedule_group(shapes.data(), n_problems, 2 * sms, (flags & Q27B_GROUP_WHOLE_TILES) != 0);
  const int ctas = int(sch.cta_units.size());
  GroupHeader h = {};
  h.magic = kGroupMagic, h.M = M, h.nb = wide ? 256 : group_tokens_tile(M), h.n_problems = n_problems, h.n_ctas = ctas;
  h.n_items = int(sch.items.size()), h.counters = sch.counters, h.sms = sms, h.slots = sch.slots;
  h.imbalance_permille = int(sch.imbalance() * 1000.0 + 0.5);
  h.off_problems = sizeof(GroupHeader);
  h.off_cta_first = h.off_problems + int64_t(n_problems) * sizeof(GroupProblemDev);
  h.off_cta_units = align_up(h.off_cta_first + int64_t(ctas + 1) * 4, 16);
  h.off_items = align_up(h.off_cta_units + int64_t(ctas) * 4, 128);
  h.table_bytes = h.off_items + int64_t(h.n_items) * sizeof(GroupItem);
  h.ws_bytes = align_up(int64_t(sch.counters) * 4, 256) + sch.slots * M * 512;
  if (table_bytes) *table_bytes = size_t(h.table_bytes);
  if (ws_bytes) *ws_bytes = size_t(h.ws_bytes);
  if (!table_host) return 0;  // size query
  Q27B_REQUIRE(table_cap >= size_t(h.table_bytes), "skinny_group: table buffer too small (%zu bytes, need %lld)", table_cap,
               (long long)h.table_bytes);
  uint8_t* base = static_cast<uint8_t*>(table_host);
  memset(base, 0, size_t(h.table_bytes));
  memcpy(base, &h, sizeof h);
  for (int i = 0; i < n_problems; i++) {
    const q27b_group_problem& q = problems[i];
    Q27B_REQUIRE(q.a && q.a_sf && q.w && q.w_sf && q.d, "skinny_group: problem %d: null pointer", i);
    Q27B_REQUIRE(aligned16(q.a) && aligned16(q.a_sf) && aligned16(q.w) && aligned16(q.w_sf) && aligned16(q.d) && aligned16(q.c),
                 "skinny_group: problem %d: operands, scales, residual and output must be 16-byte aligned", i);
    GroupProblemDev d = {};
    if (int rc = make_operand_map(&d.tmap_w, q.w, q.N, q.K, wide ? 256 : 128)) return rc;
    if (int rc = make_operand_map(&d.tmap_a, q.a, M, q.K, wide ? 128 : h.nb)) return rc;
    d.d = q.d, d.c = (q.c && q.beta != 0.f) ? q.c : nullptr, d.beta = q.beta;
    d.alpha = make_alpha(q.alpha_count, q.alpha_begin, q.alpha), d.alpha_up = q.alpha_up;
    d.N = q.N, d.epi = q.epilogue == 2 ? kEpiGluBf16 : q.epilogue == 1 ? kEpiBf16 : kEpiF32;
    memcpy(base + h.off_problems + int64_t(i) * sizeof d, &d, sizeof d);
  }
  memcpy(base + h.off_cta_first, sch.cta_first.data(), size_t(ctas + 1) * 4);
  int* units = reinterpret_cast<int*>(base + h.off_cta_units);
  for (int g = 0; g < ctas; g++) units[g] = int(sch.cta_units[g]);
  GroupItem* items = reinterpret_cast<GroupItem*>(base + h.off_items);
  for (int i = 0; i < h.n_items; i++) {
    GroupItem it = sch.items[i];
    const q27b_group_problem& q = problems[it.prob];
    it.w_sf_tile = q.w_sf + int64_t(it.tile) * (wide ? 2 : 1) * it.ksteps * 512;
    it.a_sf = q.a_sf;
    items[i] = it;
  }
  return 0;
}

static int group_launch(const void* table_host, const void* table_dev, void* ws, size_t ws_bytes, const q27b_group_peers* peers,
                        void* stream);

int q27b_skinny_fp4_group(const void* table_host, const void* table_dev, void* ws, size_t ws_bytes, void* stream) {
  return group_launch(table_host, table_dev, ws, ws_bytes, nullptr, stream);
}
int q27b_skinny_fp4_group_gather(const void* table_host, const void* table_dev, void* ws, size_t ws_bytes,
                                 const q27b_group_peers* peers, void* stream) {
  Q27B_REQUIRE(peers && peers->n_peers >= 1 && peers->n_peers <= 7, "skinny_group_gather: 1..7 peers");
  Q27B_REQUIRE(peers->signals, "skinny_group_gather: null signal block");
  for (int j = 0; j < peers->n_peers; j++)
    Q27B_REQUIRE(peers->peer_signals[j] && peers->out_delta[j] % 16 == 0, "skinny_group_gather: peer %d: null signal block or misaligned delta", j);
  Q27B_REQUIRE(peers->my_slot >= 0 && peers->my_slot < 8, "skinny_group_gather: my_slot must be 0..7");
  return group_launch(table_host, table_dev, ws, ws_bytes, peers, stream);
}
int q27b_group_gather_wait(int32_t* signals, int n_peers, const int* peer_slots, void* stream) {
  Q27B_REQUIRE(signals && n_peers >= 1 && n_peers <= 7 && peer_slots, "group_gather_wait: bad arguments");
  GatherWait w = {};
  w.signals = signals, w.n = n_peers;
  for (int j = 0; j < n_peers; j++) {
    Q27B_REQUIRE(peer_slots[j] >= 0 && peer_slots[j] < 8, "group_gather_wait: slots are 0..7");
    w.slot[j] = peer_slots[j];
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1), cfg.blockDim = dim3(32), cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = pdl_enabled() ? 1 : 0;
  Q27B_CUDA(cudaLaunchKernelEx(&cfg, group_gather_wait_kernel, w));
  return 0;
}

static int group_launch(const void* table_host, const void* table_dev, void* ws, size_t ws_bytes, const q27b_group_peers* peers,
                        void* stream) {
  Q27B_REQUIRE(table_host && table_dev, "skinny_group: null table");
  GroupHeader h;
  memcpy(&h, table_host, sizeof h);
  Q27B_REQUIRE(h.magic == kGroupMagic, "skinny_group: table_host does not hold a table made by q27b_skinny_group_build");
  Q27B_REQUIRE((reinterpret_cast<uintptr_t>(table_dev) & 127u) == 0, "skinny_group: the device copy of the table must be 128-byte aligned");
  Q27B_REQUIRE(h.sms == sm_count(), "skinny_group: the table was built for a device with %d multiprocessors", h.sms);
  Q27B_REQUIRE(ws && aligned16(ws) && ws_bytes >= size_t(h.ws_bytes), "skinny_group: workspace too small (%zu bytes, need %lld)",
               ws_bytes, (long long)h.ws_bytes);
  const uint8_t* base = static_cast<const uint8_t*>(table_dev);
  GroupLaunch gl = {};
  gl.probs = reinterpret_cast<const GroupProblemDev*>(base + h.off_problems);
  gl.cta_first = reinterpret_cast<const int*>(base + h.off_cta_first);
  gl.cta_units = reinterpret_cast<const int*>(base + h.off_cta_units);
  gl.items = reinterpret_cast<const GroupItem*>(base + h.off_items);
  gl.M = h.M;
  gl.counters = static_cast<int*>(ws);
  gl.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + align_up(int64_t(h.counters) * 4, 256));
#ifdef Q27B_TRACE
  gl.trace = g_trace;
#endif
  if (peers) {
    gl.peers.n = peers->n_peers;
    gl.signals = peers->signals, gl.my_slot = peers->my_slot;
    for (int j = 0; j < peers->n_peers; j++) gl.peers.delta[j] = peers->out_delta[j], gl.peer_signals[j] = peers->peer_signals[j];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (h.nb) {
    case 16: return launch_group<16, 4>(gl, h.n_ctas, s);
    case 32: return launch_group<32, 4>(gl, h.n_ctas, s);
    case 64: return launch_group<64, 3>(gl, h.n_ctas, s);
    case 128: return launch_group<128, 3>(gl, h.n_ctas, s);
    default:
      Q27B_REQUIRE(!peers, "skinny_group_gather: a table planned with 256-row tiles has no fused gather; build it with Q27B_GROUP_TOKENS_ON_N");
      return launch_wide_group(gl, h.n_ctas, s);
  }
}

// ---- the entry point that allocates nothing ---------------------------------------------------------------------
//
// Some callers of this library cannot hand over a workspace: code running where device allocation is forbidden or
// already frozen (a serving process that planned all of its memory up front and has none left to give, a plug-in
// loaded into such a process). For them the scratch of the
// weight-streaming GEMM lives in the library image itself.
constexpr int kStaticMaxM = 16;  // decode and speculative-verify batches
constexpr size_t kStaticScratchBytes = kCounterBytes + size_t(2) * kMaxParts * kStaticMaxM * 128 * 4;  // 7.8 MiB
static __device__ __align__(256) uint8_t g_static_scratch[kStaticScratchBytes];

// Device address of the array above on the current device; resolved (and the counters cleared) on the first call
// per device. In host code the array's name is only a handle for cudaGetSymbolAddress, never a pointer to pass on.
// A wait that ran out inside a kernel can leave arrival counters non-zero; q27b_device_status sets `dirty` for the
// device when it reports such a status, and the next call clears the counters again before its kernel.
static void* g_static_ptr[64] = {};
static bool g_static_dirty[64] = {};
static int static_scratch(void** out, cudaStream_t stream) {
  int dev = 0;
  Q27B_CUDA(cudaGetDevice(&dev));
  Q27B_REQUIRE(dev >= 0 && dev < 64, "skinny_fp4_static: device index %d out of range", dev);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    Q27B_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    g_static_ptr[dev] = p;
    g_static_dirty[dev] = true;  // (a module's globals start at zero; clearing once also covers a reload)
  }
  if (g_static_dirty[dev]) {
    // on the caller's stream, so that it is ordered before the kernel whatever kind of stream that is
    Q27B_CUDA(cudaMemsetAsync(g_static_ptr[dev], 0, kCounterBytes, stream));
    g_static_dirty[dev] = false;
  }
  *out = g_static_ptr[dev];
  return 0;
}

int q27b_skinny_fp4_static(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                           const uint8_t* w_sf, int alpha_count, const int* alpha_begin, const float* alpha,
                           const float* c, float beta, float* d, void* stream) {
  Q27B_REQUIRE(M >= 1 && M <= kStaticMaxM, "skinny_fp4_static: M must be 1..%d (M = %d); larger batches need q27b_skinny_fp4 "
               "with a caller-provided workspace", kStaticMaxM, M);
  Q27B_REQUIRE(alpha_count >= 1 && alpha_count <= 4 && alpha_begin && alpha, "skinny_fp4_static: 1..4 alpha segments");
  void* ws = nullptr;
  if (int rc = static_scratch(&ws, static_cast<cudaStream_t>(stream))) return rc;
  return skinny_common(kEpiF32, M, N, K, a, a_sf, w, w_sf, make_alpha(alpha_count, alpha_begin, alpha), 1.f,
                       (c && beta != 0.f) ? c : nullptr, beta, d, ws, kStaticScratchBytes, static_cast<cudaStream_t>(stream));
}

// Launches the bounded-wait self-test: a wait that cannot succeed, limited to `budget_us` microseconds (at most
// 100 ms); afterwards q27b_device_status reports 6 and the device is as usable as before.
int q27b_probe_wait_timeout(int budget_us, void* stream) {
  Q27B_REQUIRE(budget_us >= 1 && budget_us <= 100000, "probe_wait_timeout: budget must be 1..100000 us");
  wait_timeout_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(2000ll * budget_us);  // ~2 GHz
  Q27B_CUDA(cudaGetLastError());
  return 0;
}

// Reads and clears the device status word (0 = no bounded wait ran out since the last call). Synchronises.
int q27b_quad_available(void) { return quad_lib().gemm != nullptr; }

int q27b_device_status(uint32_t* status) {
  Q27B_REQUIRE(status, "device_status: null pointer");
  Q27B_CUDA(cudaDeviceSynchronize());
  Q27B_CUDA(cudaMemcpyFromSymbol(status, g_status, sizeof(uint32_t)));
  const uint32_t zero = 0;
  Q27B_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(uint32_t)));
  if (*status != 0) {
    // a kernel gave up half-way: arrival counters may be non-zero. The library's own scratch is cleared by the next
    // q27b_skinny_fp4_static call; a caller-owned workspace must be re-zeroed by the caller (its first 16 KiB).
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) g_static_dirty[dev] = true;
  }
  return 0;
}

}  // extern "C"
