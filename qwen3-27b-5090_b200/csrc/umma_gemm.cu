// NVFP4 x NVFP4 GEMM on the sm_100a tensor cores: tcgen05.mma kind::mxf4nvf4 (E2M1 operands, one UE4M3 scale per
// 16 K-elements, fp32 accumulators in tensor memory), operands and scale atoms brought in by TMA through a
// multi-stage shared-memory ring. One persistent, warp-specialised kernel serves both regimes:
//
//  * weight streaming (1 <= M <= 128, "skinny"): the roles of the operands are swapped — a 128-row weight tile is
//    the MMA's M side, the (padded) tokens are its N side — so one instruction consumes 4 KiB of weights whatever
//    the token count, and the kernel is bound by HBM. The K range of the whole weight matrix is cut into
//    equal contiguous unit ranges, one per SM (layout.h); tiles cut by a range boundary are finished by
//    a small fix-up kernel that sums the partial tiles in ascending K order (deterministic, independent of M).
//  * many rows (prefill): 128 tokens x 128 output channels per tile, tiles walked token-tile fastest so that the
//    CTAs running together share weight tiles through L2; accumulators double-buffered in tensor memory so the
//    epilogue of one tile overlaps the MMAs of the next.
//
// Warp roles (192 threads): warp 0 = TMA producer (one lane), warp 1 = tensor-memory owner and MMA issuer (one
// lane), warps 2..5 = epilogue (tcgen05.ld -> alpha / residual / SiLU*mul -> fp32 or bf16 stores).
// No multicast, no peer memory. Every wait is bounded (ptx_sm100.cuh); a timeout is reported through a status word.
//
// Replaces, behind the same launcher contracts: skinny_fp4 (engine/src/skinny.cu:154-549), gemm_fp4 /
// gemm_fp4_bf16 (engine/src/gemm_mma.cu:463-626) and the gate | up SiLU*mul epilogue (gemm_mma.cu:350-399,
// kernels.cu:319-339) of the reference.
#include <cuda.h>

#include "common.cuh"
#include "layout.h"
#include "ptx_sm100.cuh"

namespace q27b {

__device__ uint32_t g_status;  // first bounded-wait timeout code since the last clear (0 = none)

namespace {

enum Epi : int { kEpiF32 = 0, kEpiBf16 = 1, kEpiGluBf16 = 2 };

struct GemmParams {
  int M, N, K;          // tokens, weight rows (2 I for gate | up), reduction length
  int ksteps;           // K / 64 (MMA steps; also scale atoms per 128 rows)
  int chunks;           // ceil(ksteps / 4) pipeline stages over K
  const uint8_t* sf_p;  // scale atoms of the MMA's M-side operand
  const uint8_t* sf_q;  // scale atoms of the MMA's N-side operand
  AlphaSeg alpha;       // per output channel (gate alpha for the SiLU*mul epilogue)
  float alpha_up;
  const float* c;       // residual (may alias d) or null
  float beta;
  void* d;              // fp32 or bf16 output
  float* partials;      // weight streaming: per-CTA partial tiles [2 * grid][M][128]
  SkinnyPlan plan;      // weight streaming
  int m_tiles, items;   // many rows
};

template <int NB, int STAGES>
struct Cfg {
  static_assert(NB % 16 == 0 && NB >= 16 && NB <= 128, "N-side tile: 16..128 rows");
  static constexpr int kPBytes = 128 * 128;  // 128 rows x 256 E2M1
  static constexpr int kQBytes = NB * 128;
  static constexpr int kSfBytes = 4 * 512;   // 4 MMA steps x one 512-byte atom
  static constexpr int kStageBytes = kPBytes + kQBytes + 2 * kSfBytes;
  static constexpr int kOffQ = kPBytes, kOffSfP = kPBytes + kQBytes, kOffSfQ = kOffSfP + kSfBytes;
  static constexpr int kXchgBytes = 8 * 64 * 4;  // SiLU*mul exchange between the gate and the up warps
  static constexpr int kBarBytes = (2 * STAGES + 4) * 8 + 16;
  static constexpr int kSmemBytes = STAGES * kStageBytes + kXchgBytes + kBarBytes + 1024;  // + alignment slack
  static constexpr int kTmemCols = 512;
  static constexpr int kSfCol0 = 256;  // accumulators: columns [0, 2 NB); scales: 32 columns per stage from here
  static_assert(kStageBytes % 1024 == 0, "stage tiles must stay 1024-byte aligned");
  static_assert(kSfCol0 + 32 * STAGES <= kTmemCols && 2 * NB <= kSfCol0, "tensor memory budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

struct Work {
  int p_row0, q_row0;  // first row of the M-side / N-side tile
  int c0, c1;          // chunk range
  int slot;            // partial slot or -1 (finish in place)
  int tile;
};

template <bool kSwap>
struct WorkIter {
  const GemmParams& p;
  int64_t u;
  int item;
  __device__ explicit WorkIter(const GemmParams& p_) : p(p_) {
    if constexpr (kSwap) u = unit_begin(p.plan, blockIdx.x);
    else item = blockIdx.x;
  }
  __device__ bool next(Work& w) {
    if constexpr (kSwap) {
      Segment s;
      if (!next_segment(p.plan, blockIdx.x, u, s)) return false;
      w.p_row0 = s.tile * 128, w.q_row0 = 0, w.c0 = s.c0, w.c1 = s.c1, w.slot = s.slot, w.tile = s.tile;
      return true;
    } else {
      if (item >= p.items) return false;
      const int mi = item % p.m_tiles, ni = item / p.m_tiles;
      w.p_row0 = mi * 128, w.q_row0 = ni * 128, w.c0 = 0, w.c1 = p.chunks, w.slot = -1, w.tile = ni;
      item += gridDim.x;
      return true;
    }
  }
};

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.f + __expf(-g)) * u; }

__device__ __forceinline__ uint16_t bf16_bits(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }

// Final value of output (m, n) from the accumulated dot product, with the reference's explicit roundings
// (engine/src/skinny.cu:452-458) so that the in-place path and the fix-up path agree bit for bit.
__device__ __forceinline__ float finish_f32(const GemmParams& p, float acc, int m, int n) {
  float out = __fmul_rn(alpha_of(p.alpha, n), acc);
  if (p.c) out = __fmaf_rn(p.beta, p.c[int64_t(m) * p.N + n], out);
  return out;
}

template <int NB, int STAGES, bool kSwap, int kEpi>
__global__ void __launch_bounds__(192, 1) umma_gemm_kernel(const __grid_constant__ CUtensorMap tmap_p,
                                                           const __grid_constant__ CUtensorMap tmap_q,
                                                           const __grid_constant__ GemmParams p) {
  using C = Cfg<NB, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* xchg = reinterpret_cast<float*>(smem + STAGES * C::kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::kStageBytes + C::kXchgBytes);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, afull0 = empty0 + 8 * STAGES,
                 aempty0 = afull0 + 16;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = tmem_holder + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_p);
    prefetch_tensormap(&tmap_q);
    for (int s = 0; s < STAGES; s++) mbar_init(full0 + 8 * s, 1), mbar_init(empty0 + 8 * s, 1);
    for (int b = 0; b < 2; b++) mbar_init(afull0 + 8 * b, 1), mbar_init(aempty0 + 8 * b, 4);
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t smem_base = smem_u32(smem);

  if (warp == 0) {
    // ------------------------------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // Weights are read once (evict first); the activations are re-read by every CTA (keep them in L2).
      const uint64_t hint_p = kSwap ? kEvictFirst : kEvictLast, hint_q = kSwap ? kEvictLast : kEvictNormal;
      WorkIter<kSwap> it(p);
      Work w;
      int stage = 0;
      uint32_t phase = 0, armed = 0;  // armed: bit s set once stage s has a copy that may still be in flight
      uint32_t last_parity = 0;       // bit s: parity of the full-barrier phase stage s was last armed for
      bool ok = true;
      pdl_wait();  // the N-side operand of the weight-streaming call is produced by the preceding kernel
      while (ok && it.next(w)) {
        for (int c = w.c0; c < w.c1; c++) {
          if (!mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1, abort_flag, &g_status, kStatusEmptyWaitTimeout)) {
            ok = false;
            break;
          }
          const int nsteps = min(4, p.ksteps - 4 * c);
          const uint32_t sbase = smem_base + stage * C::kStageBytes, bar = full0 + 8 * stage;
          mbar_arrive_expect_tx(bar, C::kPBytes + C::kQBytes + 2 * nsteps * 512);
          armed |= 1u << stage;
          last_parity = (last_parity & ~(1u << stage)) | (phase << stage);
          tma_load_2d(sbase, &tmap_p, c * 128, w.p_row0, bar, hint_p);
          tma_load_2d(sbase + C::kOffQ, &tmap_q, c * 128, w.q_row0, bar, hint_q);
          bulk_load(sbase + C::kOffSfP, p.sf_p + (int64_t(w.p_row0 / 128) * p.ksteps + 4 * c) * 512, nsteps * 512, bar,
                    hint_p);
          bulk_load(sbase + C::kOffSfQ, p.sf_q + (int64_t(w.q_row0 / 128) * p.ksteps + 4 * c) * 512, nsteps * 512, bar,
                    hint_q);
          if (++stage == STAGES) stage = 0, phase ^= 1;
        }
      }
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
      WorkIter<kSwap> it(p);
      Work w;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; ok && it.next(w); i++) {
        const int buf = i & 1;
        if (!mbar_wait_bounded(aempty0 + 8 * buf, ((i >> 1) & 1) ^ 1, abort_flag, &g_status, kStatusAccumFreeTimeout))
          break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * NB;
        uint32_t accumulate = 0;
        for (int c = w.c0; c < w.c1; c++) {
          if (!mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag, &g_status, kStatusFullWaitTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const int nsteps = min(4, p.ksteps - 4 * c);
          const uint32_t sbase = smem_base + stage * C::kStageBytes;
          const uint64_t desc_p = umma_desc_k_sw128(sbase), desc_q = umma_desc_k_sw128(sbase + C::kOffQ);
          const uint32_t sf_col = tmem_base + C::kSfCol0 + 32 * stage;
          for (int ks = 0; ks < nsteps; ks++) {
            tmem_cp_sf_atom(sf_col + 4 * ks, umma_desc_sf_atom(sbase + C::kOffSfP + 512 * ks));
            tmem_cp_sf_atom(sf_col + 16 + 4 * ks, umma_desc_sf_atom(sbase + C::kOffSfQ + 512 * ks));
            // 64 E2M1 = 32 bytes further along K inside the 128-byte swizzle span: +2 in 16-byte address units
            umma_nvfp4(d_tmem, desc_p + 2 * ks, desc_q + 2 * ks, idesc, sf_col + 4 * ks, sf_col + 16 + 4 * ks,
                       accumulate);
            accumulate = 1;
          }
          umma_commit(empty0 + 8 * stage);  // the stage is free once these MMAs have read it
          if (++stage == STAGES) stage = 0, phase ^= 1;
        }
        if (ok) umma_commit(afull0 + 8 * buf);
      }
    }
  } else {
    // ------------------------------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // the 32 tensor-memory lanes this warp may read
    const int row = quarter * 32 + lane;
    WorkIter<kSwap> it(p);
    Work w;
    for (int i = 0; it.next(w); i++) {
      const int buf = i & 1;
      if (!mbar_wait_bounded(afull0 + 8 * buf, (i >> 1) & 1, abort_flag, &g_status, kStatusAccumWaitTimeout)) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * NB;
      if constexpr (kSwap) {
        // lane = weight row (output channel), column = token
        const int n = w.p_row0 + row;
        for (int m0 = 0; m0 < p.M; m0 += 8) {
          float v[8];
          tmem_ld8(taddr + m0, v);
          tmem_ld_wait();
          if (w.slot >= 0) {
            float* part = p.partials + (int64_t(w.slot) * p.M + m0) * 128 + row;
#pragma unroll
            for (int j = 0; j < 8; j++)
              if (m0 + j < p.M) part[j * 128] = v[j];
          } else if constexpr (kEpi == kEpiGluBf16) {
            // rows 0..63 of the tile are gate rows, 64..127 the up rows of the same 64 outputs
            if (quarter >= 2) {
#pragma unroll
              for (int j = 0; j < 8; j++) xchg[j * 64 + row - 64] = v[j];
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (quarter < 2) {
              const float ag = p.alpha.alpha[0], au = p.alpha_up;
              uint16_t* d = static_cast<uint16_t*>(p.d) + int64_t(w.tile) * 64 + row;
#pragma unroll
              for (int j = 0; j < 8; j++)
                if (m0 + j < p.M)
                  d[int64_t(m0 + j) * (p.N / 2)] = bf16_bits(silu_mul(__fmul_rn(ag, v[j]), __fmul_rn(au, xchg[j * 64 + row])));
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          } else {
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
      } else {
        // lane = token, column = output channel
        const int m = w.p_row0 + row;
        const bool valid = m < p.M;
#pragma unroll 1
        for (int c0 = 0; c0 < NB; c0 += 16) {
          if constexpr (kEpi == kEpiGluBf16) {
            if (c0 >= 64) break;
            float g[16], u[16];
            tmem_ld16(taddr + c0, g);
            tmem_ld16(taddr + 64 + c0, u);
            tmem_ld_wait();
            if (valid) {
              const float ag = p.alpha.alpha[0], au = p.alpha_up;
              uint32_t pk[8];
#pragma unroll
              for (int j = 0; j < 8; j++) {
                const uint32_t lo = bf16_bits(silu_mul(__fmul_rn(ag, g[2 * j]), __fmul_rn(au, u[2 * j])));
                const uint32_t hi = bf16_bits(silu_mul(__fmul_rn(ag, g[2 * j + 1]), __fmul_rn(au, u[2 * j + 1])));
                pk[j] = lo | (hi << 16);
              }
              uint4* d = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.d) + int64_t(m) * (p.N / 2) + w.tile * 64 + c0);
              d[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              d[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
          } else {
            float v[16];
            tmem_ld16(taddr + c0, v);
            tmem_ld_wait();
            if (valid) {
              const int n0 = w.q_row0 + c0;
              float out[16];
#pragma unroll
              for (int j = 0; j < 16; j++) out[j] = finish_f32(p, v[j], m, n0 + j);
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
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(aempty0 + 8 * buf);
    }
  }

  // Teardown: every role is done (or gave up); tensor memory goes back before the CTA exits.
  pdl_trigger();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// Sums the partial tiles of every weight tile that was cut by a CTA range boundary, in ascending K order, and
// applies the epilogue. Block = (tile, group of 8 tokens), thread = row of the tile.
template <int kEpi>
__global__ void __launch_bounds__(128) skinny_fixup_kernel(const __grid_constant__ GemmParams p) {
  pdl_trigger();
  const int tile = blockIdx.x, row = threadIdx.x;
  const int64_t ubeg = int64_t(tile) * p.plan.chunks;
  const int g0 = unit_owner(p.plan, ubeg), g1 = unit_owner(p.plan, ubeg + p.plan.chunks - 1);
  if (g0 == g1) return;  // finished in place by its only owner
  pdl_wait();
  __shared__ float up_s[8][64];
  const int m0 = blockIdx.y * 8;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; j++) acc[j] = 0.f;
  for (int g = g0; g <= g1; g++) {
    const int slot = 2 * g + (unit_begin(p.plan, g) >= ubeg ? 0 : 1);
    const float* part = p.partials + (int64_t(slot) * p.M + m0) * 128 + row;
#pragma unroll
    for (int j = 0; j < 8; j++)
      if (m0 + j < p.M) acc[j] = g == g0 ? __ldcg(part + j * 128) : __fadd_rn(acc[j], __ldcg(part + j * 128));
  }
  const int n = tile * 128 + row;
  if constexpr (kEpi == kEpiGluBf16) {
    if (row >= 64) {
#pragma unroll
      for (int j = 0; j < 8; j++) up_s[j][row - 64] = acc[j];
    }
    __syncthreads();
    if (row < 64) {
      uint16_t* d = static_cast<uint16_t*>(p.d) + int64_t(tile) * 64 + row;
#pragma unroll
      for (int j = 0; j < 8; j++)
        if (m0 + j < p.M)
          d[int64_t(m0 + j) * (p.N / 2)] =
              bf16_bits(silu_mul(__fmul_rn(p.alpha.alpha[0], acc[j]), __fmul_rn(p.alpha_up, up_s[j][row])));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int m = m0 + j;
      if (m < p.M) {
        const float out = finish_f32(p, acc[j], m, n);
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
int launch_gemm(Kern kernel, int grid, int smem, cudaStream_t s, const CUtensorMap& mp, const CUtensorMap& mq,
                const GemmParams& p, bool pdl) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(192), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = pdl ? 1 : 0;
  Q27B_CUDA(cudaLaunchKernelEx(&cfg, kernel, mp, mq, p));
  return 0;
}

// One-time opt-in to large dynamic shared memory, per kernel instantiation and per device.
template <int NB, int STAGES, bool kSwap, int kEpi>
int ensure_smem() {
  static bool done[64] = {};  // one array per instantiation
  int dev = 0;
  Q27B_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && done[dev]) return 0;
  Q27B_CUDA(cudaFuncSetAttribute(umma_gemm_kernel<NB, STAGES, kSwap, kEpi>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<NB, STAGES>::kSmemBytes));
  if (dev < 64) done[dev] = true;
  return 0;
}

template <int NB, int STAGES, int kEpi>
int run_skinny(const uint8_t* a, const uint8_t* w, GemmParams& p, cudaStream_t s) {
  using C = Cfg<NB, STAGES>;
  auto kernel = umma_gemm_kernel<NB, STAGES, true, kEpi>;
  if (int rc = ensure_smem<NB, STAGES, true, kEpi>()) return rc;
  CUtensorMap mp, mq;
  if (int rc = make_operand_map(&mp, w, p.N, p.K, 128)) return rc;
  if (int rc = make_operand_map(&mq, a, p.M, p.K, NB)) return rc;
  if (int rc = launch_gemm(kernel, p.plan.grid, C::kSmemBytes, s, mp, mq, p, true)) return rc;
  // Any tile cut by a range boundary? (Only when the unit ranges do not coincide with tile boundaries.)
  bool cut = false;
  for (int g = 1; g < p.plan.grid && !cut; g++) cut = unit_begin(p.plan, g) % p.plan.chunks != 0;
  if (cut) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.plan.tiles, (p.M + 7) / 8), cfg.blockDim = dim3(128), cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    Q27B_CUDA(cudaLaunchKernelEx(&cfg, skinny_fixup_kernel<kEpi>, p));
  }
  return 0;
}

template <int kEpi>
int skinny_dispatch(const uint8_t* a, const uint8_t* w, GemmParams& p, cudaStream_t s) {
  if (p.M <= 16) return run_skinny<16, 8, kEpi>(a, w, p, s);
  if (p.M <= 32) return run_skinny<32, 8, kEpi>(a, w, p, s);
  if (p.M <= 64) return run_skinny<64, 7, kEpi>(a, w, p, s);
  return run_skinny<128, 6, kEpi>(a, w, p, s);
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

int skinny_common(int kEpi, int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                  const uint8_t* w_sf, const AlphaSeg& alpha, float alpha_up, const float* c, float beta, void* d,
                  void* ws, size_t ws_bytes, cudaStream_t s) {
  Q27B_REQUIRE(M >= 1 && M <= 128, "skinny_fp4: M must be 1..128 (M = %d)", M);
  if (int rc = check_operands("skinny_fp4", M, N, K, a, a_sf, w, w_sf, d)) return rc;
  Q27B_REQUIRE(alpha.count >= 1 && alpha.count <= 4, "skinny_fp4: 1..4 alpha segments");
  const int sms = sm_count();
  Q27B_REQUIRE(sms > 0, "skinny_fp4: no CUDA device");
  GemmParams p = {};
  p.M = M, p.N = N, p.K = K, p.ksteps = K / 64, p.chunks = (p.ksteps + 3) / 4;
  p.sf_p = w_sf, p.sf_q = a_sf, p.alpha = alpha, p.alpha_up = alpha_up, p.c = c, p.beta = beta, p.d = d;
  p.plan = make_skinny_plan(N, K, sms);
  const size_t need = size_t(skinny_workspace_bytes(M, p.plan.grid));
  Q27B_REQUIRE(ws && aligned16(ws) && ws_bytes >= need, "skinny_fp4: workspace too small (%zu bytes, need %zu)", ws_bytes,
               need);
  p.partials = static_cast<float*>(ws);
  switch (kEpi) {
    case kEpiF32: return skinny_dispatch<kEpiF32>(a, w, p, s);
    case kEpiBf16: return skinny_dispatch<kEpiBf16>(a, w, p, s);
    default: return skinny_dispatch<kEpiGluBf16>(a, w, p, s);
  }
}

template <int kEpi>
int run_many(const uint8_t* a, const uint8_t* w, GemmParams& p, cudaStream_t s) {
  constexpr int NB = 128, STAGES = 6;
  using C = Cfg<NB, STAGES>;
  auto kernel = umma_gemm_kernel<NB, STAGES, false, kEpi>;
  if (int rc = ensure_smem<NB, STAGES, false, kEpi>()) return rc;
  CUtensorMap mp, mq;
  if (int rc = make_operand_map(&mp, a, p.M, p.K, 128)) return rc;
  if (int rc = make_operand_map(&mq, w, p.N, p.K, NB)) return rc;
  const int sms = sm_count();
  return launch_gemm(kernel, p.items < sms ? p.items : sms, C::kSmemBytes, s, mp, mq, p, true);
}

int many_common(int kEpi, int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                const uint8_t* w_sf, float alpha, float alpha_up, const float* c, float beta, void* d, cudaStream_t s) {
  Q27B_REQUIRE(M >= 0, "gemm_fp4: M must not be negative");
  if (M == 0) return 0;
  if (int rc = check_operands("gemm_fp4", M, N, K, a, a_sf, w, w_sf, d)) return rc;
  Q27B_REQUIRE(K % 128 == 0, "gemm_fp4: K must be a multiple of 128 (K = %d)", K);
  Q27B_REQUIRE(sm_count() > 0, "gemm_fp4: no CUDA device");
  GemmParams p = {};
  p.M = M, p.N = N, p.K = K, p.ksteps = K / 64, p.chunks = (p.ksteps + 3) / 4;
  p.sf_p = a_sf, p.sf_q = w_sf, p.alpha.count = 1, p.alpha.alpha[0] = alpha, p.alpha_up = alpha_up;
  p.c = (c && beta != 0.f) ? c : nullptr, p.beta = beta, p.d = d;
  p.m_tiles = (M + 127) / 128, p.items = p.m_tiles * (N / 128);
  switch (kEpi) {
    case kEpiF32: return run_many<kEpiF32>(a, w, p, s);
    case kEpiBf16: return run_many<kEpiBf16>(a, w, p, s);
    default: return run_many<kEpiGluBf16>(a, w, p, s);
  }
}

AlphaSeg make_alpha(int count, const int* begin, const float* alpha) {
  AlphaSeg a = {};
  a.count = count;
  for (int i = 0; i < 4; i++) a.begin[i] = i < count ? begin[i] : 0, a.alpha[i] = i < count ? alpha[i] : 1.f;
  return a;
}

}  // namespace

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
int64_t q27b_skinny_workspace_bytes(int M, int N, int K) {
  const int sms = sm_count();
  if (sms <= 0 || N <= 0 || K <= 0 || M <= 0) return -1;
  return skinny_workspace_bytes(M, make_skinny_plan(N, K, sms).grid);
}

int q27b_gemm_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
                  float alpha, const float* c, float beta, float* d, void* stream) {
  return many_common(kEpiF32, M, N, K, a, a_sf, b, b_sf, alpha, 1.f, c, beta, d, static_cast<cudaStream_t>(stream));
}
int q27b_gemm_fp4_bf16(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b,
                       const uint8_t* b_sf, float alpha, void* d, void* stream) {
  return many_common(kEpiBf16, M, N, K, a, a_sf, b, b_sf, alpha, 1.f, nullptr, 0.f, d, static_cast<cudaStream_t>(stream));
}
int q27b_gemm_fp4_glu_bf16(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                           const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, void* d, void* stream) {
  Q27B_REQUIRE(I > 0 && I % 64 == 0, "gemm_fp4_glu_bf16: I must be a positive multiple of 64 (I = %d)", I);
  return many_common(kEpiGluBf16, M, 2 * I, K, a, a_sf, gate_up, gate_up_sf, alpha_gate, alpha_up, nullptr, 0.f, d,
                     static_cast<cudaStream_t>(stream));
}

// Reads and clears the device status word (0 = no bounded wait ran out since the last call). Synchronises.
int q27b_device_status(uint32_t* status) {
  Q27B_REQUIRE(status, "device_status: null pointer");
  Q27B_CUDA(cudaDeviceSynchronize());
  Q27B_CUDA(cudaMemcpyFromSymbol(status, g_status, sizeof(uint32_t)));
  const uint32_t zero = 0;
  Q27B_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(uint32_t)));
  return 0;
}

}  // extern "C"
