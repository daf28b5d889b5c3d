// libq27b200_test.so: scaffolding of the test suite (include/q27b200/testing.h), linked against the product library
// but not part of it. A naive device GEMM (one thread per output, every product formed exactly and accumulated in
// fp32 in ascending K order), host-only views of the work split, and a self-test of the C++ launchers.
#include <cuda_fp8.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/q27b200/capi.h"
#include "../../include/q27b200/kernels.h"
#include "../../include/q27b200/testing.h"
#include "common.cuh"
#include "group_plan.h"
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

using namespace q27b;

extern "C" {

int q27t_ref_gemm_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
                      float alpha, float* d) {
  Q27B_REQUIRE(M > 0 && N > 0 && K > 0 && K % 64 == 0, "ref_gemm_fp4: bad shape");
  Q27B_REQUIRE(a && a_sf && b && b_sf && d, "ref_gemm_fp4: null pointer");
  Q27B_CUDA(cudaDeviceSynchronize());
  const int64_t n = int64_t(M) * N;
  ref_gemm_fp4_kernel<<<unsigned((n + 255) / 256), 256>>>(M, N, K, a, a_sf, b, b_sf, alpha, d);
  Q27B_CUDA(cudaGetLastError());
  Q27B_CUDA(cudaDeviceSynchronize());
  return 0;
}

int q27b_skinny_plan(int N, int K, int slots, int cta, int* seg, int cap, int* grid_out, int64_t* units_out,
                     int* split_out) {
  if (N <= 0 || N % 128 || K <= 0 || K % 64 || slots <= 0) return fail("skinny_plan: bad shape");
  const SkinnyPlan p = choose_skinny_plan(N, K, slots);
  if (grid_out) *grid_out = p.grid;
  if (units_out) *units_out = p.units;
  if (split_out) *split_out = p.split;
  if (cta < 0 || cta >= p.grid) return 0;
  int64_t u = -1;
  Segment s;
  int n = 0;
  while (next_segment(p, cta, u, s)) {
    if (seg && n < cap) seg[4 * n] = s.tile, seg[4 * n + 1] = s.c0, seg[4 * n + 2] = s.c1, seg[4 * n + 3] = s.slot;
    n++;
  }
  return n;
}

int q27b_skinny_tile_parts(int N, int K, int slots, int tile, int* slot, int cap) {
  const SkinnyPlan p = choose_skinny_plan(N, K, slots);
  const TileParts t = tile_parts(p, tile);
  for (int i = 0; i < t.n && i < cap; i++) slot[i] = t.n == 1 ? -1 : part_slot(p, t, i);
  return t.n;
}

int q27b_skinny_group_plan(int n, const int* N, const int* K, int slots, int whole_tiles, int rotate, int* pieces, int cap, int* ctas_out,
                           int64_t* slots_out, int* counters_out) {
  if (n <= 0 || !N || !K || slots <= 0) return fail("skinny_group_plan: bad arguments");
  std::vector<GroupShape> shapes(n);
  for (int i = 0; i < n; i++) {
    if (N[i] <= 0 || N[i] % (whole_tiles == 2 ? 256 : 128) || K[i] <= 0 || K[i] % 64) return fail("skinny_group_plan: bad shape");
    shapes[i] = {N[i], K[i]};
  }
  const GroupSchedule sch = schedule_group(shapes.data(), n, slots, whole_tiles != 0, rotate != 0, whole_tiles == 2 ? 256 : 128);
  if (ctas_out) *ctas_out = int(sch.cta_units.size());
  if (slots_out) *slots_out = sch.slots;
  if (counters_out) *counters_out = sch.counters;
  for (size_t g = 0; g + 1 < sch.cta_first.size(); g++)
    for (int i = sch.cta_first[g]; i < sch.cta_first[g + 1]; i++) {
      if (!pieces || i >= cap) continue;
      const GroupItem& it = sch.items[i];
      const int v[9] = {int(g), it.prob, it.tile, it.c0, it.c1, it.slot, it.nparts, it.slot0, it.sums};
      for (int j = 0; j < 9; j++) pieces[9 * i + j] = v[j];
    }
  return int(sch.items.size());
}

int q27t_cxx_launchers(const float* x, int M, int K, float in_scale, uint8_t* q, uint8_t* sf, int N, const uint8_t* w,
                       const uint8_t* w_sf, int nseg, const int* seg_begin, const float* seg_alpha, float* d, void* ws,
                       size_t ws_bytes, int I, const uint8_t* gate_up, const uint8_t* gate_up_sf, float alpha_gate,
                       float alpha_up, float out_scale, uint8_t* h_q, uint8_t* h_sf) {
  Q27B_REQUIRE(nseg >= 1 && nseg <= q27::AlphaSegments::kMax && seg_begin && seg_alpha, "cxx_launchers: 1..4 segments");
  cudaStream_t s = nullptr;
  Q27B_CUDA(cudaDeviceSynchronize());
  Q27B_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  int rc = 0;
  try {
    q27::AlphaSegments seg;
    seg.count = nseg;
    for (int i = 0; i < nseg; i++) seg.begin[i] = seg_begin[i], seg.alpha[i] = seg_alpha[i];
    q27::quant_fp4(x, M, K, in_scale, q, sf, s);
    q27::skinny_fp4(M, N, K, q, sf, w, w_sf, seg, nullptr, 0.f, d, ws, ws_bytes, s);
    q27::gemm_fp4_glu(M, I, K, q, sf, gate_up, gate_up_sf, alpha_gate, alpha_up, out_scale, h_q, h_sf, s);
  } catch (const std::exception& e) {
    rc = fail("cxx_launchers: %s", e.what());
  }
  const cudaError_t err = cudaStreamSynchronize(s);
  cudaStreamDestroy(s);
  if (rc == 0 && err != cudaSuccess) rc = fail("cxx_launchers: %s", cudaGetErrorString(err));
  return rc;
}

int q27t_cxx_throws(void) {
  int thrown = 0;
  try {
    q27::skinny_fp4(0, 128, 256, nullptr, nullptr, nullptr, nullptr, q27::AlphaSegments::one(1.f), nullptr, 0.f, nullptr,
                    nullptr, 0, nullptr);
  } catch (const std::runtime_error& e) {
    thrown += std::string(e.what()).rfind("check failed", 0) == 0;
  }
  try {
    q27::quant_fp4(static_cast<const float*>(nullptr), 1, 8, 1.f, nullptr, nullptr, nullptr);
  } catch (const std::runtime_error& e) {
    thrown += std::string(e.what()).rfind("check failed", 0) == 0;
  }
  return thrown == 2;
}

}  // extern "C"
