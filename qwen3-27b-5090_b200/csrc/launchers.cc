// The engine-facing C++ launchers (include/q27b200/kernels.h): thin forwards to the C ABI that turn its
// return code into the exception the engine's callers expect.
#include <stdexcept>
#include <string>

#include "../../include/q27b200/capi.h"
#include "../../include/q27b200/kernels.h"

namespace q27 {
namespace {
inline void check(int rc) {
  if (rc != 0) throw std::runtime_error(std::string("check failed: ") + q27_last_error());
}
}  // namespace

void swizzle_sf(const uint8_t* src, int rows, int kblocks, uint8_t* dst, cudaStream_t s, int glu_half) {
  check(q27b_swizzle_sf(src, rows, kblocks, dst, glu_half, s));
}
void quant_fp4(const float* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, cudaStream_t s) {
  check(q27b_quant_fp4(x, M, K, input_scale, q, sf, s));
}
void quant_fp4(const bf16* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, cudaStream_t s) {
  check(q27b_quant_fp4_bf16(x, M, K, input_scale, q, sf, s));
}
void rmsnorm_quant(const float* x, const bf16* w, int T, float eps, float* out, QuantOut q, cudaStream_t s, bf16* cap,
                   int cap_ld, float* rstd) {
  if (q.kind != QuantOut::kNone && q.kind != QuantOut::kFp4)
    throw std::runtime_error("check failed: rmsnorm_quant: only QuantOut::kNone and kFp4 are part of the NVFP4 path");
  check(q27b_rmsnorm_quant_fp4(x, w, T, 5120, eps, out, q.in_scale, q.kind == QuantOut::kFp4 ? q.q : nullptr, q.sf, cap,
                               cap_ld, rstd, s));
}
void quant_fp4_dynamic(const float* x, int M, int K, uint8_t* q, uint8_t* sf, float* ascale, cudaStream_t s) {
  check(q27b_quant_fp4_dynamic(x, M, K, q, sf, ascale, s));
}
void quant_fp4_dynamic(const bf16* x, int M, int K, uint8_t* q, uint8_t* sf, float* ascale, cudaStream_t s) {
  check(q27b_quant_fp4_dynamic_bf16(x, M, K, q, sf, ascale, s));
}
void skinny_fp4_scaled(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const float* ascale, const uint8_t* w,
                       const uint8_t* w_sf, const float* wscale, float* d, void* ws, size_t ws_bytes, cudaStream_t s) {
  check(q27b_skinny_fp4_scaled(M, N, K, a, a_sf, ascale, w, w_sf, wscale, d, ws, ws_bytes, s));
}
void quant_fp4_weight(const bf16* w, int M, int K, float global, uint8_t* q, uint8_t* sf, cudaStream_t s) {
  check(q27b_quant_fp4_weight(w, M, K, global, q, sf, s));
}
void silu_mul_quant_fp4(const float* gate, const float* up, int64_t ld, int T, int I, float input_scale, uint8_t* q,
                        uint8_t* sf, cudaStream_t s) {
  check(q27b_silu_mul_quant_fp4(gate, up, ld, T, I, input_scale, q, sf, s));
}
void silu_mul_quant_fp4(const bf16* gate, const bf16* up, int64_t ld, int T, int I, float input_scale, uint8_t* q,
                        uint8_t* sf, cudaStream_t s) {
  check(q27b_silu_mul_quant_fp4_bf16(gate, up, ld, T, I, input_scale, q, sf, s));
}
void silu_mul_quant_fp4_glu(const float* gu, int T, int I, float alpha_gate, float alpha_up, float input_scale,
                            uint8_t* q, uint8_t* sf, cudaStream_t s) {
  check(q27b_silu_mul_quant_fp4_glu(gu, T, I, alpha_gate, alpha_up, input_scale, q, sf, s));
}
void silu_mul_quant_fp4_glu(const bf16* gu, int T, int I, float alpha_gate, float alpha_up, float input_scale,
                            uint8_t* q, uint8_t* sf, cudaStream_t s) {
  check(q27b_silu_mul_quant_fp4_glu_bf16(gu, T, I, alpha_gate, alpha_up, input_scale, q, sf, s));
}
void gemm_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
              float alpha, const float* c, float beta, float* d, cudaStream_t s) {
  check(q27b_gemm_fp4(M, N, K, a, a_sf, b, b_sf, alpha, c, beta, d, s));
}
void gemm_fp4_bf16(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
                   float alpha, bf16* d, cudaStream_t s) {
  check(q27b_gemm_fp4_bf16(M, N, K, a, a_sf, b, b_sf, alpha, d, s));
}
void gemm_fp4_glu_bf16(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                       const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, bf16* d, cudaStream_t s) {
  check(q27b_gemm_fp4_glu_bf16(M, I, K, a, a_sf, gate_up, gate_up_sf, alpha_gate, alpha_up, d, s));
}
void gemm_fp4_glu(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                  const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, float out_scale, uint8_t* q,
                  uint8_t* q_sf, cudaStream_t s) {
  check(q27b_gemm_fp4_glu(M, I, K, a, a_sf, gate_up, gate_up_sf, alpha_gate, alpha_up, out_scale, q, q_sf, s));
}
void skinny_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w, const uint8_t* w_sf,
                const AlphaSegments& alpha, const float* c, float beta, float* d, void* ws, size_t ws_bytes,
                cudaStream_t s) {
  check(q27b_skinny_fp4(M, N, K, a, a_sf, w, w_sf, alpha.count, alpha.begin, alpha.alpha, c, beta, d, ws, ws_bytes, s));
}
void skinny_fp4_bf16(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w, const uint8_t* w_sf,
                     const AlphaSegments& alpha, bf16* d, void* ws, size_t ws_bytes, cudaStream_t s) {
  check(q27b_skinny_fp4_bf16(M, N, K, a, a_sf, w, w_sf, alpha.count, alpha.begin, alpha.alpha, d, ws, ws_bytes, s));
}
void skinny_fp4_glu_bf16(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                         const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, bf16* d, void* ws,
                         size_t ws_bytes, cudaStream_t s) {
  check(q27b_skinny_fp4_glu_bf16(M, I, K, a, a_sf, gate_up, gate_up_sf, alpha_gate, alpha_up, d, ws, ws_bytes, s));
}
size_t skinny_workspace_bytes(int M, int N, int K) {
  const int64_t b = q27b_skinny_workspace_bytes(M, N, K);
  if (b < 0) throw std::runtime_error("check failed: skinny_workspace_bytes: no CUDA device or bad shape");
  return size_t(b);
}

}  // namespace q27
