// libq27b200_quad.so: the many-row GEMM on clusters of FOUR CTAs - two CTA pairs that work on neighbouring token tiles
// of the same 256 weight rows and share those weight rows: every 64-row slice of the weight tile and every quarter of
// its scale atoms is fetched from L2 ONCE per cluster and delivered to the shared memory of every CTA that needs it by
// TMA multicast. A CTA then pulls 27 KiB per 256 K-elements out of L2 instead of 38 KiB, and L2 -> SM delivery is what
// bounds the pair kernel (at the rate the tensor pipe sustains on random operands the 148 SMs would need 15.8 TB/s).
//
// An OPTIONAL library for single-GPU processes, built from this file alone: libq27b200.so opens it if it lies beside it
// and routes eligible shapes here (see run_many in umma_gemm.cu); without it the pair kernel runs. Every load reads
// this GPU's own memory: the operands are the caller's local weights and activations, nothing here takes a peer
// pointer. Same arithmetic as the pair kernel: every output element is one accumulation chain over K in 64-element
// steps of the same instruction, and the epilogues are the same code: bit-identical results.
//
// Replaces, for these shapes: gemm_fp4 / gemm_fp4_bf16 (engine/src/gemm_mma.cu:463-626) and the gate | up SiLU*mul
// epilogue (gemm_mma.cu:350-399) of the reference.
#include <cuda.h>

#include <algorithm>
#include <cstdint>

#include "common.cuh"
#include "ptx_sm100.cuh"
#include "quad_abi.h"

namespace q27b {
namespace {

enum Epi : int { kEpiF32 = 0, kEpiBf16 = 1, kEpiGluBf16 = 2 };

__device__ __forceinline__ float silu_mul(float g, float u) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.44269504f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
  return g * r * u;
}
__device__ __forceinline__ uint16_t bf16_bits(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }

// 2-D tiled load delivered to the same shared-memory offset (and signalled on the barrier at the same offset) in every
// CTA of the cluster whose bit is set in `mask`. x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d_to(uint32_t smem_dst, const void* tmap, int x, int y, uint32_t bar, uint16_t mask,
                                               uint64_t hint) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.multicast::cluster.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5, %6;"
      ::"r"(smem_dst), "l"(tmap), "r"(bar), "r"(x), "r"(y), "h"(mask), "l"(hint)
      : "memory");
}
// Flat copy global -> shared of every CTA in `mask`; addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load_to(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar, uint16_t mask,
                                             uint64_t hint) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.multicast::cluster.L2::cache_hint [%0], [%1], %2, [%3], %4, %5;"
      ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar), "h"(mask), "l"(hint)
      : "memory");
}
// Arrives on the barrier at this offset in every CTA of `mask` once this thread's tcgen05 operations so far are done.
__device__ __forceinline__ void umma_commit_to(uint32_t bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(mask)
      : "memory");
}

template <int STAGES>
struct CfgQ {
  static constexpr int kPBytes = 128 * 128, kQBytes = 128 * 128, kSfBytes = 4 * 512;
  static constexpr int kStageBytes = kPBytes + kQBytes + 3 * kSfBytes;  // own tokens, half the weight rows, scales of tokens + 256 weight rows
  static constexpr int kOffQ = kPBytes, kOffSfP = kPBytes + kQBytes, kOffSfQ = kOffSfP + kSfBytes;
  static constexpr int kSfCols = 48;
  static constexpr int kNumBars = 3 * STAGES + 2;
  static constexpr int kOutOff = STAGES * kStageBytes + (kNumBars * 8 + 16 + 15) / 16 * 16;
  static constexpr int kOutBytes = 128 * 256;
  static constexpr int kSmemBytes = kOutOff + kOutBytes + 1024;
  static constexpr int kTmemCols = 512, kSfCol0 = 256;
  static constexpr int kEpiWarps = 16, kFeederWarp0 = 2 + kEpiWarps, kThreads = (kFeederWarp0 + 4) * 32;
  static_assert(kStageBytes % 1024 == 0, "stage tiles must stay 1024-byte aligned");
  static_assert(kSfCol0 + kSfCols * STAGES <= kTmemCols, "tensor memory budget");
  static_assert(kSmemBytes + 1024 <= 228 * 1024, "shared memory budget");
};

// Cluster rank r: pair q = r >> 1 (token tile 2 j + q of the cluster's two), half h = r & 1 within the pair (tokens
// h * 128 .. of the pair's 256, weight rows h * 128 .. of the tile's 256). Ranks 0 and 2 lead their pairs.
template <int STAGES, int kEpi>
__global__ void __launch_bounds__(CfgQ<STAGES>::kThreads, 1) quad_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                                             const __grid_constant__ CUtensorMap tmap_w64,
                                                                             const __grid_constant__ QuadParams p) {
  using C = CfgQ<STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::kStageBytes);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, sfr0 = empty0 + 8 * STAGES, afull = sfr0 + 8 * STAGES,
                 aempty = afull + 8;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile uint32_t* abort_flag = tmem_holder + 1;
  volatile uint32_t* epi_ok = tmem_holder + 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank(), q = rank >> 1, h = rank & 1, leader = rank & 2u;
  const int cluster = blockIdx.x >> 2, nclusters = gridDim.x >> 2;
  const int m_pairs = (p.M + 255) / 256, m_duos = m_pairs / 2, items = m_duos * (p.N / 256);  // (m_pairs is even)
  const int m_blocks = (p.M + 127) / 128;
  const uint32_t smem_base = smem_u32(smem);
  uint32_t* status = p.status;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_w64);
    // a slot is free once BOTH pairs have read it: each CTA's slot is also written by loads of the other pair's CTAs
    for (int s = 0; s < STAGES; s++) mbar_init(full0 + 8 * s, 1), mbar_init(empty0 + 8 * s, 2), mbar_init(sfr0 + 8 * s, 8);
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
  cluster_sync_all();  // every CTA's barriers exist before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, armed = 0, last_parity = 0;
      bool ok = true, waited = false;
      const uint16_t same_half = uint16_t((1u << h) | (1u << (h + 2)));  // the CTAs that hold this half of the weight rows
      for (int item = cluster; ok && item < items; item += nclusters) {
        const int m0 = ((item % m_duos) * 2 + int(q)) * 256 + int(h) * 128, n0 = (item / m_duos) * 256;
        const bool sfa_valid = m0 / 128 < m_blocks;
        // this CTA's quarter of the weight tile's scale atoms: row block `q`, MMA steps 2 h and 2 h + 1 of the stage
        const uint8_t* sfq = p.sf_q + (int64_t(n0 / 128) + q) * p.ksteps * 512 + h * 1024;
        const uint8_t* sfp = p.sf_p + int64_t(m0 / 128) * p.ksteps * 512;
        const int wrow = n0 + int(h) * 128 + int(q) * 64;  // this CTA's 64-row slice of half h
        for (int c = 0; c < p.chunks; c++, sfq += 2048, sfp += 2048) {
          if (!mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1, abort_flag, status, kStatusEmptyWaitTimeout, 0, true)) {
            ok = false;
            break;
          }
          const uint32_t sbase = smem_base + stage * C::kStageBytes, bar = full0 + 8 * stage;
          // bytes that land in THIS CTA's slot, whoever issues them: own tokens (+ their scales), both slices of the
          // weight half, all four quarters of the weight scales
          mbar_arrive_expect_tx(bar, C::kPBytes + C::kQBytes + (sfa_valid ? 3 : 2) * C::kSfBytes);
          armed |= 1u << stage;
          last_parity = (last_parity & ~(1u << stage)) | (phase << stage);
          tma_load_2d_to(sbase + C::kOffQ + q * 8192, &tmap_w64, c * 128, wrow, bar, same_half, kEvictNormal);
          bulk_load_to(sbase + C::kOffSfQ + q * C::kSfBytes + h * 1024, sfq, 1024, bar, uint16_t(0xF), kEvictNormal);
          if (!waited) pdl_wait(), waited = true;  // the activations come from the preceding kernel
          tma_load_2d(sbase, &tmap_a, c * 128, m0, bar, kEvictLast);
          if (sfa_valid) bulk_load(sbase + C::kOffSfP, sfp, C::kSfBytes, bar, kEvictLast);
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
            if (!landed) atomicCAS(status, 0u, uint32_t(kStatusDrainTimeout));
          }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------------------ MMA issuer (pair leaders)
    if (lane == 0 && h == 0) {
      constexpr uint32_t idesc = umma_idesc_nvfp4_2sm(256);
      const uint16_t my_pair = uint16_t(3u << leader);
      int stage = 0, ntiles = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t desc_a0 = umma_desc_k_sw128(smem_base), desc_b0 = umma_desc_k_sw128(smem_base + C::kOffQ);
      const uint32_t sf_col0 = tmem_base + C::kSfCol0;
      auto issue_stage = [&](auto stage_c, auto first_c) -> bool {
        constexpr int S = decltype(stage_c)::value;
        constexpr bool kFirst = decltype(first_c)::value;
        if (!mbar_wait_bounded(sfr0 + 8 * S, phase, abort_flag, status, kStatusFullWaitTimeout, 0, true)) return false;
        tc_fence_after_sync();
        constexpr uint64_t kStageDesc = uint64_t(S) * (C::kStageBytes >> 4);
        const uint64_t da = desc_a0 + kStageDesc, db = desc_b0 + kStageDesc;
        const uint32_t sf = sf_col0 + C::kSfCols * S;
        umma_nvfp4_2sm_imm<!kFirst>(tmem_base, da, db, idesc, sf, sf + 16);
        umma_nvfp4_2sm_imm<true>(tmem_base, da + 2, db + 2, idesc, sf + 4, sf + 24);
        umma_nvfp4_2sm_imm<true>(tmem_base, da + 4, db + 4, idesc, sf + 8, sf + 32);
        umma_nvfp4_2sm_imm<true>(tmem_base, da + 6, db + 6, idesc, sf + 12, sf + 40);
        umma_commit_to(empty0 + 8 * S, uint16_t(0xF));  // one of the two arrivals that free the slot in all four CTAs
        return true;
      };
      auto issue = [&](auto first_c) -> bool {
        bool r;
        switch (stage) {
          case 0: r = issue_stage(std::integral_constant<int, 0>(), first_c); break;
          case 1: r = issue_stage(std::integral_constant<int, 1 % STAGES>(), first_c); break;
          case 2: r = issue_stage(std::integral_constant<int, 2 % STAGES>(), first_c); break;
          case 3: r = issue_stage(std::integral_constant<int, 3 % STAGES>(), first_c); break;
          case 4: r = issue_stage(std::integral_constant<int, 4 % STAGES>(), first_c); break;
          default: r = issue_stage(std::integral_constant<int, 5 % STAGES>(), first_c); break;
        }
        if (++stage == STAGES) stage = 0, phase ^= 1;
        return r;
      };
      static_assert(STAGES <= 6, "one case per ring slot");
      for (int item = cluster; ok && item < items; item += nclusters, ntiles++) {
        if (!mbar_wait_bounded(aempty, (ntiles & 1) ^ 1, abort_flag, status, kStatusAccumFreeTimeout, 0, true)) break;
        tc_fence_after_sync();
        ok = issue(std::true_type());
        for (int c = 1; ok && c < p.chunks; c++) ok = issue(std::false_type());
        if (ok) umma_commit_to(afull, my_pair);
      }
      if (ok && ntiles > 0) mbar_wait_bounded(aempty, (ntiles - 1) & 1, abort_flag, status, kStatusAccumFreeTimeout, 64, true);
    }
  } else if (warp >= C::kFeederWarp0) {
    // ------------------------------------------------------------------------------------------ scale feeders
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int item = cluster; ok && item < items; item += nclusters) {
      for (int c = 0; c < p.chunks; c++) {
        if (!warp_wait(full0 + 8 * stage, phase, abort_flag, status, kStatusFullWaitTimeout, 32)) {
          ok = false;
          break;
        }
        const uint8_t* sb = smem + stage * C::kStageBytes;
        const uint4* sfp = reinterpret_cast<const uint4*>(sb + C::kOffSfP) + lane;
        const uint4* sfq = reinterpret_cast<const uint4*>(sb + C::kOffSfQ) + lane;
        const uint32_t taddr = tmem_base + lane_base + C::kSfCol0 + C::kSfCols * stage;
        uint4 a[4];
#pragma unroll
        for (int ks = 0; ks < 4; ks++) a[ks] = sfp[32 * ks];
        tmem_st16(taddr, a);
#pragma unroll
        for (int hh = 0; hh < 2; hh++) {
#pragma unroll
          for (int ks = 0; ks < 2; ks++) a[2 * ks] = sfq[32 * (2 * hh + ks)], a[2 * ks + 1] = sfq[32 * (4 + 2 * hh + ks)];
          tmem_st16(taddr + 16 + 16 * hh, a);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (h == 0) mbar_arrive(sfr0 + 8 * stage);
          else mbar_arrive_remote(sfr0 + 8 * stage, leader);
        }
        if (++stage == STAGES) stage = 0, phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------------------------------ epilogue
    // (the pair kernel's: the accumulator into registers, handed back at once, outputs staged in shared memory and
    //  written as whole 256-byte rows)
    const int quarter = warp & 3, sub = (warp - 2) >> 2, row = quarter * 32 + lane;
    const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16);
    constexpr bool kGlu = kEpi == kEpiGluBf16;
    constexpr int kUnits = kGlu ? 8 : 16, kMine = kUnits / 4;
    uint8_t* stage_out = smem + C::kOutOff;
    int ntiles = 0;
    for (int item = cluster; item < items; item += nclusters, ntiles++) {
      const int m_base = ((item % m_duos) * 2 + int(q)) * 256 + int(h) * 128, n0 = (item / m_duos) * 256;
      if (warp == 2) {
        const bool done = warp_wait(afull, ntiles & 1, abort_flag, status, kStatusAccumWaitTimeout, 20);
        if (lane == 0) *epi_ok = done;
      }
      asm volatile("bar.sync 2, %0;" ::"r"(C::kEpiWarps * 32) : "memory");
      if (!*epi_ok) break;
      mbar_wait_bounded(afull, ntiles & 1, abort_flag, status, kStatusAccumWaitTimeout);
      tc_fence_after_sync();
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
        if (h == 0) mbar_arrive(aempty);
        else mbar_arrive_remote(aempty, leader);
      }
      const int chunk = lane & 15;
      if constexpr (kGlu) {
        const float ag = p.alpha, au = p.alpha_up;
        asm volatile("bar.sync 3, %0;" ::"r"(C::kEpiWarps * 32) : "memory");
#pragma unroll
        for (int j = 0; j < kMine; j++) {
          const int un = sub + 4 * j, chunk0 = (un >> 2) * 8 + (un & 3) * 2;
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
        uint16_t* out0 = static_cast<uint16_t*>(p.d) + n0 / 2 + chunk * 8;
#pragma unroll
        for (int it = 0; it < 4; it++) {
          const int r = (warp - 2) * 8 + it * 2 + (lane >> 4), mr = m_base + r;
          if (mr < p.M)
            *reinterpret_cast<uint4*>(out0 + int64_t(mr) * (p.N / 2)) = reinterpret_cast<const uint4*>(stage_out + r * 256)[chunk ^ (r & 15)];
        }
      } else {
        constexpr int kPasses = kEpi == kEpiBf16 ? 2 : 4, kPerPass = kMine / kPasses, kPassCols = 256 / kPasses;
        constexpr int kElem = kEpi == kEpiBf16 ? 2 : 4;
#pragma unroll
        for (int ps = 0; ps < kPasses; ps++) {
          asm volatile("bar.sync 3, %0;" ::"r"(C::kEpiWarps * 32) : "memory");
#pragma unroll
          for (int jj = 0; jj < kPerPass; jj++) {
            const int j = ps * kPerPass + jj, col = (sub + 4 * j) * 16;
            uint4* r = reinterpret_cast<uint4*>(stage_out + row * 256);
            float out[16];
#pragma unroll
            for (int i = 0; i < 16; i++) out[i] = __fmul_rn(p.alpha, g[j][i]);
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
          char* out0 = static_cast<char*>(p.d) + (int64_t(n0) + ps * kPassCols) * kElem + chunk * 16;
#pragma unroll
          for (int it = 0; it < 4; it++) {
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
      }
    }
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // nothing of any CTA goes away while another may still signal it or write into it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_2sm(tmem_base, C::kTmemCols);
  }
}

template <int kEpi, int STAGES = 5>
int run_quad(const CUtensorMap& ma, const CUtensorMap& mw64, const QuadParams& p, cudaStream_t s) {
  using C = CfgQ<STAGES>;
  auto kernel = quad_gemm_kernel<STAGES, kEpi>;
  static int max_clusters[64] = {};  // per device: clusters of four that can be resident at once (0: not asked yet)
  int dev = 0;
  Q27B_CUDA(cudaGetDevice(&dev));
  Q27B_REQUIRE(dev < 64, "quad_gemm: device index %d", dev);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(C::kThreads), cfg.dynamicSmemBytes = C::kSmemBytes, cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 4, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  if (!max_clusters[dev]) {
    Q27B_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    int sms = 0, n = 0;
    Q27B_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    cfg.gridDim = dim3(sms / 4 * 4);
    Q27B_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
    Q27B_REQUIRE(n > 0, "quad_gemm: no cluster of four fits this device");
    max_clusters[dev] = std::min(n, sms / 4);
  }
  const int items = ((p.M + 255) / 256 / 2) * (p.N / 256), clusters = std::min(items, max_clusters[dev]);
  cfg.gridDim = dim3(4 * clusters);
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  Q27B_CUDA(cudaLaunchKernelEx(&cfg, kernel, ma, mw64, p));
  return 0;
}

}  // namespace
}  // namespace q27b

using namespace q27b;

extern "C" int q27b_quad_gemm(const void* tmap_a, const void* tmap_w64, const QuadParams* p, void* stream) {
  Q27B_REQUIRE(tmap_a && tmap_w64 && p && p->status, "quad_gemm: null argument");
  Q27B_REQUIRE(p->M > 128 && ((p->M + 255) / 256) % 2 == 0 && p->N % 256 == 0 && p->K % 256 == 0,
               "quad_gemm: M > 128 with an even number of 256-token tiles, N and K multiples of 256 (M = %d, N = %d, K = %d)", p->M, p->N, p->K);
  const CUtensorMap& ma = *static_cast<const CUtensorMap*>(tmap_a);
  const CUtensorMap& mw = *static_cast<const CUtensorMap*>(tmap_w64);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (p->epi) {
    case kEpiF32: return run_quad<kEpiF32>(ma, mw, *p, s);
    case kEpiBf16: return run_quad<kEpiBf16>(ma, mw, *p, s);
    case kEpiGluBf16: return run_quad<kEpiGluBf16>(ma, mw, *p, s);
    default: return fail("quad_gemm: epilogue %d is not built here", p->epi);
  }
}

// fail() / last_error() of this library (libq27b200.so has its own; the caller copies the message over)
namespace q27b {
std::string& last_error() {
  thread_local std::string e;
  return e;
}
int fail(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  last_error() = buf;
  return -1;
}
}  // namespace q27b

extern "C" const char* q27b_quad_last_error() { return q27b::last_error().c_str(); }
