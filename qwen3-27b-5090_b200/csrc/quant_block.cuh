// The NVFP4 block quantiser shared by the stand-alone quantisers and the GEMM epilogue that emits NVFP4: per 16
// consecutive elements
//   gs = 1 / input_scale;  sf = e4m3_satfinite(gs * amax / 6);  inv = sf != 0 ? gs / sf : 0;
//   code = rne_e2m1(x * inv)   (ties to the even code, saturating at +-6)
// every operation a separate IEEE fp32 operation (reference/qwen27b/quant.py:58-67; engine/src/kernels.cu:99-113).
#pragma once

#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "layout.h"

namespace q27b {

// Two values -> one byte of E2M1 codes, `even` in the low nibble.
__device__ __forceinline__ uint32_t e2m1x2(float even, float odd) {
  uint16_t r;
  asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u16.u8 %0, t;\n\t}"
      : "=h"(r)
      : "f"(odd), "f"(even));
  return r;
}

__device__ __forceinline__ float e4m3_to_float(__nv_fp8_storage_t c) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(c, __NV_E4M3)));
}

// Codes (lo: elements 0..7, hi: 8..15, four bits each, element 0 in the lowest nibble) and the E4M3 scale byte of one
// 16-element block; gs = 1 / input_scale as an IEEE division.
__device__ __forceinline__ void quant_block16_codes(const float* v, float gs, uint32_t& lo, uint32_t& hi, uint8_t& sfq) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(v[j]));
  const __nv_fp8_storage_t s8 = __nv_cvt_float_to_fp8(__fdiv_rn(__fmul_rn(gs, amax), 6.f), __NV_SATFINITE, __NV_E4M3);
  const float sff = e4m3_to_float(s8);
  const float inv = sff != 0.f ? __fdiv_rn(gs, sff) : 0.f;
  lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    lo |= e2m1x2(__fmul_rn(v[2 * j], inv), __fmul_rn(v[2 * j + 1], inv)) << (8 * j);
    hi |= e2m1x2(__fmul_rn(v[8 + 2 * j], inv), __fmul_rn(v[9 + 2 * j], inv)) << (8 * j);
  }
  sfq = s8;
}

// One 16-element block (row m, k-block kb) of an [M][K] activation: codes row-major, scale into its swizzled atom.
__device__ __forceinline__ void quant_block16(const float* v, float input_scale, int m, int kb, int K, uint8_t* q,
                                              uint8_t* sf) {
  uint32_t lo, hi;
  uint8_t sfq;
  quant_block16_codes(v, __fdiv_rn(1.f, input_scale), lo, hi, sfq);
  *reinterpret_cast<uint2*>(q + int64_t(m) * (K / 2) + kb * 8) = make_uint2(lo, hi);
  sf[sf_offset(m, kb, K / 16)] = sfq;
}

}  // namespace q27b
