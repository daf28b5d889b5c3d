// Activation -> NVFP4 quantisers and the scale-factor relayout.
//
// Numerics follow the reference's definition bit for bit (reference/qwen27b/quant.py:58-67; device twin
// engine/src/kernels.cu:99-113): per 16 consecutive K elements
//   gs = 1 / input_scale;  sf = e4m3_satfinite(gs * amax / 6);  inv = sf != 0 ? gs / sf : 0;
//   code = rne_e2m1(x * inv)   (ties to the even code, saturating at +-6)
// with every operation a separate IEEE fp32 operation (no contraction, no fast-math). Codes are packed two per
// byte, even column in the low nibble; scales go to the swizzled 128 x 4 atom layout (layout.h).
//
// Thread mapping, shared by every kernel here: one lane per 16-element block, consecutive lanes on consecutive
// blocks of a row. A warp therefore reads 1 KiB (bf16) or 2 KiB (fp32) of contiguous input and writes 256 contiguous
// bytes of codes; the four lanes of a quad hold the four k-blocks of ONE 32-bit word of the swizzled scale layout
// (same row, kb % 4 = 0..3), so their scale bytes are gathered with two shuffles and stored once per quad instead
// of as four scattered byte stores. Several activations can be quantised by one launch (a job per grid row):
// a decode layer quantises three small activations, and a launch costs more than the work.
//
// Programmatic dependent launch: every kernel here waits for its predecessor FIRST and releases its successor
// only then. A successor (a GEMM that prefetches weights before its own wait) can thus never run ahead of anything
// but the kernel directly before it.
#include <algorithm>

#include "../../include/q27b200/capi.h"
#include "common.cuh"
#include "layout.h"
#include "ptx_sm100.cuh"
#include "quant_block.cuh"

namespace q27b {
namespace {

constexpr int kThreads = 256;

// 16 consecutive elements of a row as fp32.
__device__ __forceinline__ void load16(const float* p, float* v) {
  const float4* s = reinterpret_cast<const float4*>(p);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const float4 t = s[j];
    v[4 * j] = t.x, v[4 * j + 1] = t.y, v[4 * j + 2] = t.z, v[4 * j + 3] = t.w;
  }
}
__device__ __forceinline__ void load16(const __nv_bfloat16* p, float* v) {
  const uint4* s = reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int j = 0; j < 2; j++) {
    const uint4 t = s[j];
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
      // bf16 -> fp32 is exact: the 16 bits become the high half
      v[8 * j + 2 * k] = __uint_as_float(w[k] << 16);
      v[8 * j + 2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
    }
  }
}

// Stores block (m, kb) of an [M][K] activation: its 8 bytes of codes, and - once per quad of lanes - the 32-bit scale
// word of k-blocks kb .. kb + 3. Called by all 32 lanes of a warp (`active` false for lanes past the end; K / 16 is a
// multiple of 4, so a quad is active or idle as a whole).
__device__ __forceinline__ void store_block(bool active, int m, int kb, int K, uint32_t lo, uint32_t hi, uint8_t sfq,
                                            uint8_t* q, uint8_t* sf) {
  if (active) *reinterpret_cast<uint2*>(q + int64_t(m) * (K / 2) + kb * 8) = make_uint2(lo, hi);
  uint32_t word = uint32_t(sfq) << (8 * (kb & 3));
  word |= __shfl_xor_sync(0xffffffffu, word, 1);
  word |= __shfl_xor_sync(0xffffffffu, word, 2);
  if (active && (kb & 3) == 0) *reinterpret_cast<uint32_t*>(sf + sf_offset(m, kb, K / 16)) = word;
}

__device__ __forceinline__ void quant_store(bool active, const float* v, float input_scale, int m, int kb, int K,
                                            uint8_t* q, uint8_t* sf) {
  uint32_t lo = 0, hi = 0;
  uint8_t sfq = 0;
  if (active) quant_block16_codes(v, __fdiv_rn(1.f, input_scale), lo, hi, sfq);
  store_block(active, m, kb, K, lo, hi, sfq, q, sf);
}

// ---- activation quantiser: a list of jobs per launch ----------------------------------------------------------------

using QuantJob = q27b_quant_job;
struct QuantJobs4 {
  QuantJob job[4];
};

// grid = (blocks of the largest job, jobs). kTable: the jobs are read from device memory, else from the launch
// parameters (up to four).
template <bool kTable>
__global__ void __launch_bounds__(kThreads) quant_fp4_jobs_kernel(const __grid_constant__ QuantJobs4 inl,
                                                                  const QuantJob* __restrict__ table) {
  pdl_wait();
  pdl_trigger();
  QuantJob j;
  if constexpr (kTable) j = table[blockIdx.y]; else j = inl.job[blockIdx.y];
  const int kblocks = j.K / 16;
  const int64_t idx = int64_t(blockIdx.x) * kThreads + threadIdx.x;
  if (int64_t(blockIdx.x) * kThreads >= int64_t(j.M) * kblocks) return;  // (whole CTA: this job is smaller than the grid)
  const bool active = idx < int64_t(j.M) * kblocks;
  const int m = active ? int(idx / kblocks) : 0, kb = active ? int(idx % kblocks) : int(threadIdx.x & 3);
  float v[16];
  if (active) {
    if (j.bf16) load16(static_cast<const __nv_bfloat16*>(j.x) + int64_t(m) * j.K + kb * 16, v);
    else load16(static_cast<const float*>(j.x) + int64_t(m) * j.K + kb * 16, v);
  }
  quant_store(active, v, j.input_scale, m, kb, j.K, j.q, j.sf);
}

// ---- silu(gate) * up, then the block quantiser ------------------------------------------------------------------------
// kGlu: `gate` is the [T][2 I] output of the interleaved gate | up weights (the up value 64 columns after its gate)
// and the alphas are applied here.
template <typename E, bool kGlu>
__global__ void __launch_bounds__(kThreads) silu_mul_quant_fp4_kernel(const E* __restrict__ gate,
                                                                      const E* __restrict__ up, int64_t ld, int T,
                                                                      int I, float input_scale, uint8_t* q,
                                                                      uint8_t* sf, float alpha_gate, float alpha_up) {
  pdl_wait();
  pdl_trigger();
  const int kblocks = I / 16;
  const int64_t idx = int64_t(blockIdx.x) * kThreads + threadIdx.x;
  const bool active = idx < int64_t(T) * kblocks;
  const int t = active ? int(idx / kblocks) : 0, kb = active ? int(idx % kblocks) : int(threadIdx.x & 3);
  float g[16], u[16];
  if (active) {
    const int64_t col = kGlu ? glu_row(int64_t(kb) * 16, 0) : int64_t(kb) * 16;
    load16(gate + t * ld + col, g);
    load16((kGlu ? gate + 64 : up) + t * ld + col, u);
#pragma unroll
    for (int j = 0; j < 16; j++) {
      if (kGlu) g[j] = __fmul_rn(g[j], alpha_gate), u[j] = __fmul_rn(u[j], alpha_up);
      g[j] = __fmul_rn(__fdiv_rn(g[j], __fadd_rn(1.f, expf(-g[j]))), u[j]);
    }
  }
  quant_store(active, g, input_scale, t, kb, I, q, sf);
}

// ---- RMSNorm(1 + w) fused with the quantiser ----------------------------------------------------------------------
// One CTA per token, one lane per 16 elements of the hidden state (D / 16 threads, a multiple of 32). Replaces
// rmsnorm_quant_kernel (engine/src/kernels.cu:211-262) for its NVFP4 and plain outputs. The sum of squares is formed
// in a fixed order with separate IEEE operations (each lane its 16 squares in order, a butterfly over the warp, the
// warps' sums in order) and 1 / sqrt is the IEEE square root and division, so the CPU restatement follows it bit for
// bit; the quantised copy is exactly the quantisation of the fp32 result.
__global__ void __launch_bounds__(1024) rmsnorm_quant_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                             int D, float eps, float* __restrict__ out, float input_scale,
                                                             uint8_t* q, uint8_t* sf, __nv_bfloat16* cap, int cap_ld,
                                                             float* rstd) {
  __shared__ float warp_sum[32];
  const int t = blockIdx.x, kb = threadIdx.x;
  float wv[16];
  load16(w + kb * 16, wv);  // the norm weights do not come from the preceding kernel
  pdl_wait();
  pdl_trigger();
  float v[16];
  load16(x + int64_t(t) * D + kb * 16, v);
  if (cap) {  // a bf16 copy of the input rows (the residual stream)
    uint32_t pk[8];
#pragma unroll
    for (int j = 0; j < 8; j++)
      pk[j] = uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(v[2 * j]))) |
              (uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(v[2 * j + 1]))) << 16);
    uint4* o = reinterpret_cast<uint4*>(cap + int64_t(t) * cap_ld + kb * 16);
    o[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    o[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 16; j++) ss = __fadd_rn(ss, __fmul_rn(v[j], v[j]));
  for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
  for (int i = 0; i < int(blockDim.x >> 5); i++) total = __fadd_rn(total, warp_sum[i]);
  const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, float(D)), eps)));
  if (rstd && kb == 0) rstd[t] = r;
#pragma unroll
  for (int j = 0; j < 16; j++) v[j] = __fmul_rn(__fmul_rn(v[j], r), __fadd_rn(1.f, wv[j]));
  if (out) {
    float4* o = reinterpret_cast<float4*>(out + int64_t(t) * D + kb * 16);
#pragma unroll
    for (int j = 0; j < 4; j++) o[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  }
  if (q) quant_store(true, v, input_scale, t, kb, D, q, sf);
}

__global__ void __launch_bounds__(kThreads) swizzle_sf_kernel(const uint8_t* __restrict__ src, int rows, int kblocks,
                                                              uint8_t* __restrict__ dst, int glu_half) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= int64_t(rows) * kblocks) return;
  const int r = int(i / kblocks), kb = int(i % kblocks);
  dst[sf_offset(glu_half < 0 ? r : glu_row(r, glu_half), kb, kblocks)] = src[i];
}

unsigned blocks_for(int64_t n) { return unsigned((n + kThreads - 1) / kThreads); }

template <typename... Args, typename... Act>
int launch_pdl(void (*kernel)(Args...), dim3 grid, int threads, cudaStream_t s, Act... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = dim3(threads), cfg.dynamicSmemBytes = 0, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = pdl_enabled() ? 1 : 0;
  Q27B_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<Args>(args)...));
  return 0;
}

// Dynamic per-token quantisation: one CTA per row; the row's tensor scale is amax(row) / (6 * 448) (1 for an
// all-zero row), written to ascale[row], and every block of the row is quantised with it as quant_fp4 does. The
// GEMM multiplies it back in per token (skinny_fp4_scaled). (The rule of the reference's draft model,
// engine/src/draft.cu:70-111: row_scale, act_row, quant_block16.)
template <typename E>
__global__ void __launch_bounds__(kThreads) quant_fp4_dynamic_kernel(const E* __restrict__ x, int M, int K,
                                                                     uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                                     float* __restrict__ ascale) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[kThreads / 32];
  const int m = blockIdx.x, kblocks = K / 16;
  const E* row = x + int64_t(m) * K;
  float am = 0.f;
  for (int kb = threadIdx.x; kb < kblocks; kb += kThreads) {
    float v[16];
    load16(row + kb * 16, v);
#pragma unroll
    for (int j = 0; j < 16; j++) am = fmaxf(am, fabsf(v[j]));
  }
  for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = am;
  __syncthreads();
  am = red[0];
#pragma unroll
  for (int i = 1; i < kThreads / 32; i++) am = fmaxf(am, red[i]);
  const float rs = am > 0.f ? __fdiv_rn(am, 6.f * 448.f) : 1.f;
  if (threadIdx.x == 0) ascale[m] = rs;
  for (int kb0 = 0; kb0 < kblocks; kb0 += kThreads) {  // whole warps stay in the loop: the scale store shuffles
    const int kb = kb0 + threadIdx.x;
    const bool active = kb < kblocks;
    float v[16];
    if (active) load16(row + kb * 16, v);
    quant_store(active, v, rs, m, active ? kb : int(threadIdx.x & 3), K, q, sf);
  }
}

// The load-time weight quantiser: one lane per 16-element block of a bf16 weight matrix. The block's E4M3 scale
// code is searched around the code of amax / 6 for the smallest squared error of the block, the candidates in a
// fixed order (the code itself, so that it stays on a tie, then 1..4 below, then 1..8 above, each clamped to
// 1..126) and the first best kept; value = global * scale * e2m1. Codes go out row-major, scales straight into
// the swizzled atoms. (Replaces quant_fp4_weight_kernel, engine/src/kernels.cu:167-206; the candidate order and
// every operation being a separate IEEE fp32 operation are what the CPU restatement follows bit for bit.)
__constant__ float kE2m1Magnitude[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
__device__ __forceinline__ float e2m1_value(uint32_t code) {
  const float m = kE2m1Magnitude[code & 7];
  return (code & 8) ? -m : m;
}
// Squared error of the block when quantised with scale code `code`.
__device__ __forceinline__ float block_error(const float (&v)[16], int code, float global) {
  const float step = __fmul_rn(e4m3_to_float(__nv_fp8_storage_t(code)), global), inv = __fdiv_rn(1.f, step);
  float err = 0.f;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const uint32_t pair = e2m1x2(__fmul_rn(v[2 * j], inv), __fmul_rn(v[2 * j + 1], inv));
    const float d0 = __fsub_rn(v[2 * j], __fmul_rn(e2m1_value(pair & 15), step));
    const float d1 = __fsub_rn(v[2 * j + 1], __fmul_rn(e2m1_value(pair >> 4), step));
    err = __fadd_rn(err, __fadd_rn(__fmul_rn(d0, d0), __fmul_rn(d1, d1)));
  }
  return err;
}
__global__ void __launch_bounds__(kThreads) quant_fp4_weight_kernel(const __nv_bfloat16* __restrict__ w, int M, int K,
                                                                    float global, uint8_t* __restrict__ q,
                                                                    uint8_t* __restrict__ sf) {
  const int kblocks = K / 16;
  const int64_t idx = int64_t(blockIdx.x) * kThreads + threadIdx.x;
  const bool active = idx < int64_t(M) * kblocks;
  const int m = active ? int(idx / kblocks) : 0, kb = active ? int(idx % kblocks) : int(threadIdx.x & 3);
  float v[16];
  uint32_t lo = 0, hi = 0;
  int chosen = 0;
  if (active) {
    load16(w + int64_t(m) * K + kb * 16, v);
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(v[j]));
    const int centre = __nv_cvt_float_to_fp8(__fdiv_rn(__fdiv_rn(amax, 6.f), global), __NV_SATFINITE, __NV_E4M3);
    chosen = centre;
    if (amax > 0.f) {
      float least = INFINITY;
      auto consider = [&](int code) {
        code = min(max(code, 1), 126);
        const float err = block_error(v, code, global);
        if (err < least) least = err, chosen = code;
      };
      consider(centre);
#pragma unroll 1
      for (int below = 1; below <= 4; below++) consider(centre - below);
#pragma unroll 1
      for (int above = 1; above <= 8; above++) consider(centre + above);
    }
    const float scale = e4m3_to_float(__nv_fp8_storage_t(chosen));
    const float inv = scale != 0.f ? __fdiv_rn(1.f, __fmul_rn(scale, global)) : 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      lo |= e2m1x2(__fmul_rn(v[2 * j], inv), __fmul_rn(v[2 * j + 1], inv)) << (8 * j);
      hi |= e2m1x2(__fmul_rn(v[8 + 2 * j], inv), __fmul_rn(v[9 + 2 * j], inv)) << (8 * j);
    }
  }
  store_block(active, m, kb, K, lo, hi, uint8_t(chosen), q, sf);
}

int check_job(const QuantJob& j) {
  Q27B_REQUIRE(j.M >= 0 && j.K > 0 && j.K % 64 == 0, "quant_fp4: K must be a positive multiple of 64 (K = %d)", j.K);
  if (j.M == 0) return 0;
  Q27B_REQUIRE(j.x && j.q && j.sf, "quant_fp4: null pointer");
  Q27B_REQUIRE(aligned16(j.x) && (reinterpret_cast<uintptr_t>(j.q) & 7u) == 0 && (reinterpret_cast<uintptr_t>(j.sf) & 3u) == 0,
               "quant_fp4: x must be 16-byte, q 8-byte and sf 4-byte aligned");
  Q27B_REQUIRE(j.input_scale > 0.f, "quant_fp4: input_scale must be positive");
  return 0;
}

int quant_jobs(const QuantJob* host, const QuantJob* dev, int n, cudaStream_t s) {
  Q27B_REQUIRE(n >= 1 && host, "quant_fp4_batch: at least one job");
  Q27B_REQUIRE(dev || n <= 4, "quant_fp4_batch: more than four jobs need a device copy of the job list");
  Q27B_REQUIRE(n <= 65535, "quant_fp4_batch: at most 65535 jobs");
  int64_t most = 0;
  for (int i = 0; i < n; i++) {
    if (int rc = check_job(host[i])) return rc;
    most = std::max<int64_t>(most, int64_t(host[i].M) * (host[i].K / 16));
  }
  if (most == 0) return 0;
  QuantJobs4 inl = {};
  if (!dev)
    for (int i = 0; i < n; i++) inl.job[i] = host[i];
  const dim3 grid(blocks_for(most), unsigned(n));
  if (dev) return launch_pdl(quant_fp4_jobs_kernel<true>, grid, kThreads, s, inl, dev);
  return launch_pdl(quant_fp4_jobs_kernel<false>, grid, kThreads, s, inl, dev);
}

int quant_one(const void* x, bool bf16, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, cudaStream_t s) {
  QuantJob j = {};
  j.x = x, j.q = q, j.sf = sf, j.M = M, j.K = K, j.input_scale = input_scale, j.bf16 = bf16 ? 1 : 0;
  if (M == 0) return check_job(j);
  return quant_jobs(&j, nullptr, 1, s);
}

template <typename E>
int quant_dynamic_impl(const E* x, int M, int K, uint8_t* q, uint8_t* sf, float* ascale, cudaStream_t s) {
  Q27B_REQUIRE(M >= 0 && K > 0 && K % 64 == 0, "quant_fp4_dynamic: K must be a positive multiple of 64 (K = %d)", K);
  if (M == 0) return 0;
  Q27B_REQUIRE(x && q && sf && ascale, "quant_fp4_dynamic: null pointer");
  Q27B_REQUIRE(aligned16(x) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0, "quant_fp4_dynamic: x must be 16-byte and q 8-byte aligned");
  return launch_pdl(quant_fp4_dynamic_kernel<E>, dim3(unsigned(M)), kThreads, s, x, M, K, q, sf, ascale);
}

template <typename E, bool kGlu>
int silu_impl(const E* gate, const E* up, int64_t ld, int T, int I, float input_scale, uint8_t* q, uint8_t* sf,
              float ag, float au, cudaStream_t s) {
  Q27B_REQUIRE(T >= 0 && I > 0 && I % 64 == 0, "silu_mul_quant_fp4: I must be a positive multiple of 64 (I = %d)", I);
  if (T == 0) return 0;
  Q27B_REQUIRE(gate && (kGlu || up) && q && sf, "silu_mul_quant_fp4: null pointer");
  Q27B_REQUIRE(aligned16(gate) && (kGlu || aligned16(up)) && (ld * sizeof(E)) % 16 == 0,
               "silu_mul_quant_fp4: gate / up rows must be 16-byte aligned");
  Q27B_REQUIRE(input_scale > 0.f, "silu_mul_quant_fp4: input_scale must be positive");
  return launch_pdl(silu_mul_quant_fp4_kernel<E, kGlu>, dim3(blocks_for(int64_t(T) * (I / 16))), kThreads, s, gate, up, ld,
                    T, I, input_scale, q, sf, ag, au);
}

}  // namespace
}  // namespace q27b

using namespace q27b;

extern "C" {

int q27b_quant_fp4(const float* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, void* stream) {
  return quant_one(x, false, M, K, input_scale, q, sf, static_cast<cudaStream_t>(stream));
}
int q27b_quant_fp4_bf16(const void* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, void* stream) {
  return quant_one(x, true, M, K, input_scale, q, sf, static_cast<cudaStream_t>(stream));
}
int q27b_quant_fp4_batch(const q27b_quant_job* jobs_host, const q27b_quant_job* jobs_dev, int n, void* stream) {
  return quant_jobs(jobs_host, jobs_dev, n, static_cast<cudaStream_t>(stream));
}
int q27b_rmsnorm_quant_fp4(const float* x, const void* w, int T, int D, float eps, float* out, float input_scale, uint8_t* q,
                           uint8_t* sf, void* cap, int cap_ld, float* rstd, void* stream) {
  Q27B_REQUIRE(T >= 0 && D > 0 && D % 512 == 0 && D <= 16384, "rmsnorm_quant: D must be a multiple of 512 up to 16384 (D = %d)", D);
  if (T == 0) return 0;
  Q27B_REQUIRE(x && w, "rmsnorm_quant: null pointer");
  Q27B_REQUIRE(aligned16(x) && aligned16(w) && aligned16(out) && aligned16(cap) && (cap_ld * 2) % 16 == 0,
               "rmsnorm_quant: x, w, out and cap rows must be 16-byte aligned");
  Q27B_REQUIRE(!q || (sf && input_scale > 0.f && (reinterpret_cast<uintptr_t>(q) & 7u) == 0 && (reinterpret_cast<uintptr_t>(sf) & 3u) == 0),
               "rmsnorm_quant: the NVFP4 output needs q (8-byte aligned), sf (4-byte aligned) and a positive input_scale");
  Q27B_REQUIRE(eps >= 0.f, "rmsnorm_quant: eps must not be negative");
  return launch_pdl(rmsnorm_quant_kernel, dim3(unsigned(T)), D / 16, static_cast<cudaStream_t>(stream), x,
                    static_cast<const __nv_bfloat16*>(w), D, eps, out, input_scale, q, sf, static_cast<__nv_bfloat16*>(cap),
                    cap_ld, rstd);
}
int q27b_quant_fp4_dynamic(const float* x, int M, int K, uint8_t* q, uint8_t* sf, float* ascale, void* stream) {
  return quant_dynamic_impl(x, M, K, q, sf, ascale, static_cast<cudaStream_t>(stream));
}
int q27b_quant_fp4_dynamic_bf16(const void* x, int M, int K, uint8_t* q, uint8_t* sf, float* ascale, void* stream) {
  return quant_dynamic_impl(static_cast<const __nv_bfloat16*>(x), M, K, q, sf, ascale, static_cast<cudaStream_t>(stream));
}
int q27b_quant_fp4_weight(const void* w, int M, int K, float global, uint8_t* q, uint8_t* sf, void* stream) {
  Q27B_REQUIRE(M >= 0 && K > 0 && K % 64 == 0, "quant_fp4_weight: K must be a positive multiple of 64 (K = %d)", K);
  if (M == 0) return 0;
  Q27B_REQUIRE(w && q && sf, "quant_fp4_weight: null pointer");
  Q27B_REQUIRE(aligned16(w) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0 && (reinterpret_cast<uintptr_t>(sf) & 3u) == 0,
               "quant_fp4_weight: w must be 16-byte, q 8-byte and sf 4-byte aligned");
  Q27B_REQUIRE(global > 0.f, "quant_fp4_weight: the tensor scale must be positive");
  quant_fp4_weight_kernel<<<blocks_for(int64_t(M) * (K / 16)), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(w), M, K, global, q, sf);
  Q27B_CUDA(cudaGetLastError());
  return 0;
}
int q27b_silu_mul_quant_fp4(const float* gate, const float* up, int64_t ld, int T, int I, float input_scale,
                            uint8_t* q, uint8_t* sf, void* stream) {
  return silu_impl<float, false>(gate, up, ld, T, I, input_scale, q, sf, 1.f, 1.f, static_cast<cudaStream_t>(stream));
}
int q27b_silu_mul_quant_fp4_bf16(const void* gate, const void* up, int64_t ld, int T, int I, float input_scale,
                                 uint8_t* q, uint8_t* sf, void* stream) {
  return silu_impl<__nv_bfloat16, false>(static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up),
                                         ld, T, I, input_scale, q, sf, 1.f, 1.f, static_cast<cudaStream_t>(stream));
}
int q27b_silu_mul_quant_fp4_glu(const float* gu, int T, int I, float alpha_gate, float alpha_up, float input_scale,
                                uint8_t* q, uint8_t* sf, void* stream) {
  return silu_impl<float, true>(gu, nullptr, int64_t(2) * I, T, I, input_scale, q, sf, alpha_gate, alpha_up,
                                static_cast<cudaStream_t>(stream));
}
int q27b_silu_mul_quant_fp4_glu_bf16(const void* gu, int T, int I, float alpha_gate, float alpha_up,
                                     float input_scale, uint8_t* q, uint8_t* sf, void* stream) {
  return silu_impl<__nv_bfloat16, true>(static_cast<const __nv_bfloat16*>(gu), nullptr, int64_t(2) * I, T, I,
                                        input_scale, q, sf, alpha_gate, alpha_up, static_cast<cudaStream_t>(stream));
}
int q27b_swizzle_sf(const uint8_t* src, int rows, int kblocks, uint8_t* dst, int glu_half, void* stream) {
  Q27B_REQUIRE(rows >= 0 && kblocks >= 0 && glu_half >= -1 && glu_half <= 1, "swizzle_sf: bad arguments");
  if (rows == 0 || kblocks == 0) return 0;
  Q27B_REQUIRE(src && dst, "swizzle_sf: null pointer");
  swizzle_sf_kernel<<<blocks_for(int64_t(rows) * kblocks), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      src, rows, kblocks, dst, glu_half);
  Q27B_CUDA(cudaGetLastError());
  return 0;
}
int64_t q27b_sf_bytes(int64_t rows, int64_t kblocks) { return sf_bytes(rows, kblocks); }
int64_t q27b_sf_offset(int64_t row, int64_t kb, int64_t kblocks) { return sf_offset(row, kb, kblocks); }
int64_t q27b_glu_row(int64_t r, int half) { return glu_row(r, half); }

}  // extern "C"
