// C++ launchers of the NVFP4 GEMM path with the signatures of the reference engine's kernel header
// (engine/src/kernels.h): same names, namespace, argument order and meaning, so the engine's callers
// (Model::gemm_q, Model::mlp, the draft model) compile against this header unchanged. Each launcher forwards to
// the C ABI (capi.h) and, like the reference's Q27_CHECK / Q27_CUDA (engine/src/check.h:6-13,
// engine/src/common.h:27-33), throws std::runtime_error on a failed precondition or CUDA error.
// All launches are asynchronous on the caller's stream; nothing allocates.
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace q27 {

using bf16 = __nv_bfloat16;

// engine/src/kernels.h:186-199
inline int64_t glu_row(int64_t r, int half) { return (r / 64) * 128 + half * 64 + r % 64; }
inline int64_t gate_glu_offset(int64_t c) { return glu_row(c, 0); }
inline int64_t sf_offset(int64_t row, int64_t kb, int64_t kblocks) {
  const int64_t katoms = (kblocks + 3) / 4;
  return ((row / 128) * katoms + kb / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 + (kb % 4);
}
inline int64_t sf_bytes(int64_t rows, int64_t kblocks) { return ((rows + 127) / 128) * 128 * ((kblocks + 3) / 4) * 4; }
void swizzle_sf(const uint8_t* src, int rows, int kblocks, uint8_t* dst, cudaStream_t s, int glu_half = -1);

// engine/src/kernels.h:124-126,137-147
void quant_fp4(const float* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, cudaStream_t s);
void quant_fp4(const bf16* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, cudaStream_t s);  // new
// Dynamic per-token quantisation (the draft model's rule, engine/src/draft.cu:70-111): writes ascale[m].
void quant_fp4_dynamic(const float* x, int M, int K, uint8_t* q, uint8_t* sf, float* ascale, cudaStream_t s);
void quant_fp4_dynamic(const bf16* x, int M, int K, uint8_t* q, uint8_t* sf, float* ascale, cudaStream_t s);
// engine/src/kernels.h:104-114,131-136: the quantised copy an op writes for the next GEMM, and RMSNorm(1 + w) over the
// hidden size (5120) fused with it. Of the reference's kinds this path has kNone and kFp4; the FP8 kinds throw.
struct QuantOut {
  enum Kind : int { kNone = 0, kFp8 = 1, kFp4 = 2, kFp8Row = 3 };
  Kind kind = kNone;
  float in_scale = 1.f;
  uint8_t* q = nullptr;    // packed e2m1 [T][D/2]
  uint8_t* sf = nullptr;   // swizzled scale factors
  float* scale = nullptr;  // (kFp8Row only)
};
void rmsnorm_quant(const float* x, const bf16* w, int T, float eps, float* out, QuantOut q, cudaStream_t s,
                   bf16* cap = nullptr, int cap_ld = 0, float* rstd = nullptr);
// engine/src/kernels.h:130: the load-time weight quantiser (block scales searched for the smallest squared error)
void quant_fp4_weight(const bf16* w, int M, int K, float global, uint8_t* q, uint8_t* sf, cudaStream_t s);
void silu_mul_quant_fp4(const float* gate, const float* up, int64_t ld, int T, int I, float input_scale, uint8_t* q,
                        uint8_t* sf, cudaStream_t s);
void silu_mul_quant_fp4(const bf16* gate, const bf16* up, int64_t ld, int T, int I, float input_scale, uint8_t* q,
                        uint8_t* sf, cudaStream_t s);
void silu_mul_quant_fp4_glu(const float* gu, int T, int I, float alpha_gate, float alpha_up, float input_scale,
                            uint8_t* q, uint8_t* sf, cudaStream_t s);
void silu_mul_quant_fp4_glu(const bf16* gu, int T, int I, float alpha_gate, float alpha_up, float input_scale,
                            uint8_t* q, uint8_t* sf, cudaStream_t s);

// engine/src/kernels.h:203-209
void gemm_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
              float alpha, const float* c, float beta, float* d, cudaStream_t s);
void gemm_fp4_bf16(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
                   float alpha, bf16* d, cudaStream_t s);
// gate | up GEMM on interleaved weights, d[M][I] = bf16(silu(alpha_gate * gate) * (alpha_up * up)) (new: the bf16
// form of gemm_fp4_glu, engine/src/kernels.h:216-221).
void gemm_fp4_glu_bf16(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                       const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, bf16* d, cudaStream_t s);
// engine/src/kernels.h:216-221: the same GEMM with silu(gate) * up quantised to NVFP4 (q, q_sf: the down GEMM's
// activation, tensor scale out_scale).
void gemm_fp4_glu(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                  const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, float out_scale, uint8_t* q,
                  uint8_t* q_sf, cudaStream_t s);

// engine/src/kernels.h:228-245
struct AlphaSegments {
  static constexpr int kMax = 4;
  int count = 1;
  int begin[kMax] = {0, 0, 0, 0};
  float alpha[kMax] = {1.f, 1.f, 1.f, 1.f};
  static AlphaSegments one(float a) {
    AlphaSegments s;
    s.alpha[0] = a;
    return s;
  }
};
// 1 <= M <= 128 here (the reference: 64). The workspace needs skinny_workspace_bytes(M, N, K) bytes (within the
// reference's 32 MiB up to M = 64 on a 148-SM device, up to 38.8 MiB at M = 128) and, as in the reference, must be zeroed once
// before the first call; the kernels leave its counters at zero.
void skinny_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w, const uint8_t* w_sf,
                const AlphaSegments& alpha, const float* c, float beta, float* d, void* ws, size_t ws_bytes,
                cudaStream_t s);
// engine/src/kernels.h:255-256: d[t][n] = acc * wscale[n] * ascale[t]
void skinny_fp4_scaled(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const float* ascale, const uint8_t* w,
                       const uint8_t* w_sf, const float* wscale, float* d, void* ws, size_t ws_bytes, cudaStream_t s);
void skinny_fp4_bf16(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w, const uint8_t* w_sf,
                     const AlphaSegments& alpha, bf16* d, void* ws, size_t ws_bytes, cudaStream_t s);  // new
void skinny_fp4_glu_bf16(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                         const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, bf16* d, void* ws,
                         size_t ws_bytes, cudaStream_t s);  // new
size_t skinny_workspace_bytes(int M, int N, int K);

}  // namespace q27
