// Device-side cross-check for the tests: one thread per output, every product formed exactly and accumulated in
// fp32 in ascending K order. Deliberately naive; no product entry point routes through it.
#include <cuda_fp8.h>

#include "common.cuh"
#include "layout.h"

namespace q27b {
namespace {

__device__ __forceinline__ float e2m1_value(uint32_t code) {
  const float mag[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const float v = mag[code & 7];
  return (code & 8) ? -v : v;
}
__device__ __forceinline__ float e4m3_value(uint8_t c) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(c, __NV_E4M3)));
}

__global__ void ref_gemm_fp4_kernel(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b,
                                    const uint8_t* b_sf, float alpha, float* d) {
  const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= int64_t(M) * N) return;
  const int m = int(idx / N), n = int(idx % N), kblocks = K / 16;
  float acc = 0.f;
  for (int kb = 0; kb < kblocks; kb++) {
    const float s = e4m3_value(a_sf[sf_offset(m, kb, kblocks)]) * e4m3_value(b_sf[sf_offset(n, kb, kblocks)]);
    float dot = 0.f;  // exact: at most 16 products of multiples of 0.25 below 36
    for (int j = 0; j < 8; j++) {
      const uint32_t x = a[int64_t(m) * (K / 2) + kb * 8 + j], y = b[int64_t(n) * (K / 2) + kb * 8 + j];
      dot += e2m1_value(x & 15) * e2m1_value(y & 15) + e2m1_value(x >> 4) * e2m1_value(y >> 4);
    }
    acc += dot * s;
  }
  d[idx] = alpha * acc;
}

}  // namespace
}  // namespace q27b

extern "C" int q27b_ref_gemm_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b,
                                 const uint8_t* b_sf, float alpha, float* d, void* stream) {
  using namespace q27b;
  Q27B_REQUIRE(M > 0 && N > 0 && K > 0 && K % 64 == 0, "ref_gemm_fp4: bad shape");
  Q27B_REQUIRE(a && a_sf && b && b_sf && d, "ref_gemm_fp4: null pointer");
  const int64_t n = int64_t(M) * N;
  ref_gemm_fp4_kernel<<<unsigned((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(M, N, K, a, a_sf, b, b_sf,
                                                                                              alpha, d);
  Q27B_CUDA(cudaGetLastError());
  return 0;
}
