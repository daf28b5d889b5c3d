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
  cfg.attrs = attr, cfg.numAttrs = 1;
  Q27B_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<Args>(args)...));
  return 0;
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
