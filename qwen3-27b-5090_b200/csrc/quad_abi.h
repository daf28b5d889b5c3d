// What libq27b200.so passes to the optional libq27b200_quad.so (quad_gemm.cu): the many-row GEMM on clusters of four
// CTAs, for single-GPU processes. Plain data only.
#pragma once

#include <cstdint>

namespace q27b {

struct QuadParams {
  int M, N, K;          // tokens (> 128, an even number of 256-token tiles), weight rows (multiple of 256), reduction length (multiple of 256)
  int ksteps, chunks;   // K / 64, K / 256
  const uint8_t* sf_p;  // scale atoms of the activation
  const uint8_t* sf_q;  // scale atoms of the weight
  float alpha;          // gate alpha for the SiLU*mul epilogue
  float alpha_up;
  const float* c;       // fp32 epilogue: residual (may alias d) or null
  float beta;
  void* d;              // fp32 [M][N], bf16 [M][N] or, SiLU*mul, bf16 [M][N / 2]
  int epi;              // 0 fp32, 1 bf16, 2 SiLU*mul -> bf16
  uint32_t* status;     // device status word of the calling library (bounded-wait time-outs are reported there)
};

// tmap_a: CUtensorMap of the activation codes, boxes of 128 bytes x 128 rows; tmap_w64: of the weight codes, boxes of
// 128 bytes x 64 rows (both with the 128-byte swizzle). 0 on success; -1 with a message from q27b_quad_last_error().
using QuadGemmFn = int (*)(const void* tmap_a, const void* tmap_w64, const QuadParams* p, void* stream);
using QuadErrorFn = const char* (*)();

}  // namespace q27b
