// Activation -> NVFP4 quantisers and the scale-factor relayout.
//
// Numerics follow the reference's definition bit for bit (reference/qwen27b/quant.py:58-67; device twin
// engine/src/kernels.cu:99-113): per 16 consecutive K elements
//   gs = 1 / input_scale;  sf = e4m3_satfinite(gs * amax / 6);  inv = sf != 0 ? gs / sf : 0;
//   code = rne_e2m1(x * inv)   (ties to the even code, saturating at +-6)
// with every operation a separate IEEE fp32 operation (no contraction, no fast-math). Codes are packed two per
// byte, even column in the low nibble; scales go to the swizzled 128 x 4 atom layout (layout.h).
#include "common.cuh"
#include "layout.h"
#include "ptx_sm100.cuh"
#include "quant_block.cuh"

namespace q27b {
namespace {

constexpr int kThreads = 256;

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

template <typename E>
__global__ void __launch_bounds__(kThreads) quant_fp4_kernel(const E* __restrict__ x, int M, int K,
                                                             float input_scale, uint8_t* __restrict__ q,
                                                             uint8_t* __restrict__ sf) {
  pdl_trigger();  // dependents may begin their prologue; they wait for this grid before reading q / sf
  pdl_wait();
  const int kblocks = K / 16;
  const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= int64_t(M) * kblocks) return;
  const int m = int(idx / kblocks), kb = int(idx % kblocks);
  float v[16];
  load16(x + int64_t(m) * K + kb * 16, v);
  quant_block16(v, input_scale, m, kb, K, q, sf);
}

// silu(gate) * up, then the block quantiser; one thread per 16 outputs. kGlu: `gate` is the [T][2 I] output of
// the interleaved gate | up weights (the up value 64 columns after its gate) and the alphas are applied here.
template <typename E, bool kGlu>
__global__ void __launch_bounds__(kThreads) silu_mul_quant_fp4_kernel(const E* __restrict__ gate,
                                                                      const E* __restrict__ up, int64_t ld, int T,
                                                                      int I, float input_scale, uint8_t* q,
                                                                      uint8_t* sf, float alpha_gate, float alpha_up) {
  pdl_trigger();
  pdl_wait();
  const int kblocks = I / 16;
  const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= int64_t(T) * kblocks) return;
  const int t = int(idx / kblocks), kb = int(idx % kblocks);
  const int64_t col = kGlu ? glu_row(int64_t(kb) * 16, 0) : int64_t(kb) * 16;
  float g[16], u[16];
  load16(gate + t * ld + col, g);
  load16((kGlu ? gate + 64 : up) + t * ld + col, u);
#pragma unroll
  for (int j = 0; j < 16; j++) {
    if (kGlu) g[j] = __fmul_rn(g[j], alpha_gate), u[j] = __fmul_rn(u[j], alpha_up);
    g[j] = __fmul_rn(__fdiv_rn(g[j], __fadd_rn(1.f, expf(-g[j]))), u[j]);
  }
  quant_block16(g, input_scale, t, kb, I, q, sf);
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
int launch_pdl(void (*kernel)(Args...), unsigned grid, cudaStream_t s, Act... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = 0, cfg.stream = s;
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
  pdl_trigger();
  pdl_wait();
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
  for (int kb = threadIdx.x; kb < kblocks; kb += kThreads) {
    float v[16];
    load16(row + kb * 16, v);
    quant_block16(v, rs, m, kb, K, q, sf);
  }
}

template <typename E>
int quant_dynamic_impl(const E* x, int M, int K, uint8_t* q, uint8_t* sf, float* ascale, cudaStream_t s);

// The load-time weight quantiser: one thread per 16-element block of a bf16 weight matrix; the block's E4M3 scale
// code is searched around the code of amax / 6 (the code itself first, so it stays on a tie, then 4 below and 8
// above, clamped to 1..126) for the smallest squared error of the block; value = global * scale * e2m1. Codes go
// out row-major, scales straight into the swizzled atoms. (Replaces quant_fp4_weight_kernel,
// engine/src/kernels.cu:167-206. Every operation is a separate IEEE fp32 operation so that the CPU restatement
// can follow it bit for bit.)
__constant__ float kE2m1Magnitude[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
__device__ __forceinline__ float e2m1_value(uint32_t code) {
  const float m = kE2m1Magnitude[code & 7];
  return (code & 8) ? -m : m;
}
__global__ void __launch_bounds__(kThreads) quant_fp4_weight_kernel(const __nv_bfloat16* __restrict__ w, int M, int K,
                                                                    float global, uint8_t* __restrict__ q,
                                                                    uint8_t* __restrict__ sf) {
  const int kblocks = K / 16;
  const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= int64_t(M) * kblocks) return;
  const int m = int(idx / kblocks), kb = int(idx % kblocks);
  float v[16];
  load16(w + int64_t(m) * K + kb * 16, v);
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(v[j]));
  const int c0 = __nv_cvt_float_to_fp8(__fdiv_rn(__fdiv_rn(amax, 6.f), global), __NV_SATFINITE, __NV_E4M3);
  int best = c0;
  if (amax > 0.f) {
    float best_err = INFINITY;
#pragma unroll 1
    for (int t = 0; t < 13; t++) {
      const int c = min(max(c0 + (t <= 4 ? -t : t - 4), 1), 126);
      const float s = __fmul_rn(e4m3_to_float(__nv_fp8_storage_t(c)), global), inv = __fdiv_rn(1.f, s);
      float err = 0.f;
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const uint32_t p = e2m1x2(__fmul_rn(v[2 * j], inv), __fmul_rn(v[2 * j + 1], inv));
        const float a = __fsub_rn(v[2 * j], __fmul_rn(e2m1_value(p & 15), s));
        const float b = __fsub_rn(v[2 * j + 1], __fmul_rn(e2m1_value(p >> 4), s));
        err = __fadd_rn(err, __fadd_rn(__fmul_rn(a, a), __fmul_rn(b, b)));
      }
      if (err < best_err) best_err = err, best = c;
    }
  }
  const float sff = e4m3_to_float(__nv_fp8_storage_t(best));
  const float inv = sff != 0.f ? __fdiv_rn(1.f, __fmul_rn(sff, global)) : 0.f;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    lo |= e2m1x2(__fmul_rn(v[2 * j], inv), __fmul_rn(v[2 * j + 1], inv)) << (8 * j);
    hi |= e2m1x2(__fmul_rn(v[8 + 2 * j], inv), __fmul_rn(v[9 + 2 * j], inv)) << (8 * j);
  }
  *reinterpret_cast<uint2*>(q + int64_t(m) * (K / 2) + kb * 8) = make_uint2(lo, hi);
  sf[sf_offset(m, kb, kblocks)] = uint8_t(best);
}

template <typename E>
int quant_impl(const E* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, cudaStream_t s) {
  Q27B_REQUIRE(M >= 0 && K > 0 && K % 64 == 0, "quant_fp4: K must be a positive multiple of 64 (K = %d)", K);
  if (M == 0) return 0;
  Q27B_REQUIRE(x && q && sf, "quant_fp4: null pointer");
  Q27B_REQUIRE(aligned16(x) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0, "quant_fp4: x must be 16-byte and q 8-byte aligned");
  Q27B_REQUIRE(input_scale > 0.f, "quant_fp4: input_scale must be positive");
  return launch_pdl(quant_fp4_kernel<E>, blocks_for(int64_t(M) * (K / 16)), s, x, M, K, input_scale, q, sf);
}

template <typename E>
int quant_dynamic_impl(const E* x, int M, int K, uint8_t* q, uint8_t* sf, float* ascale, cudaStream_t s) {
  Q27B_REQUIRE(M >= 0 && K > 0 && K % 64 == 0, "quant_fp4_dynamic: K must be a positive multiple of 64 (K = %d)", K);
  if (M == 0) return 0;
  Q27B_REQUIRE(x && q && sf && ascale, "quant_fp4_dynamic: null pointer");
  Q27B_REQUIRE(aligned16(x) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0, "quant_fp4_dynamic: x must be 16-byte and q 8-byte aligned");
  return launch_pdl(quant_fp4_dynamic_kernel<E>, unsigned(M), s, x, M, K, q, sf, ascale);
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
  return launch_pdl(silu_mul_quant_fp4_kernel<E, kGlu>, blocks_for(int64_t(T) * (I / 16)), s, gate, up, ld, T, I,
                    input_scale, q, sf, ag, au);
}

}  // namespace
}  // namespace q27b

using namespace q27b;

extern "C" {

int q27b_quant_fp4(const float* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, void* stream) {
  return quant_impl(x, M, K, input_scale, q, sf, static_cast<cudaStream_t>(stream));
}
int q27b_quant_fp4_bf16(const void* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, void* stream) {
  return quant_impl(static_cast<const __nv_bfloat16*>(x), M, K, input_scale, q, sf, static_cast<cudaStream_t>(stream));
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
  Q27B_REQUIRE(aligned16(w) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0, "quant_fp4_weight: w must be 16-byte and q 8-byte aligned");
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
