// C-ABI glue: the thread-local error message, and the synchronous one-kernel wrappers q27t_* that the tests and
// the benchmark call with raw device pointers (the protocol of the reference's test layer,
// engine/src/capi.cc:46-95,498-636: synchronise the device, launch on a private non-blocking stream, synchronise,
// return 0 / -1 with a message; Q27T_REPEAT=n additionally times n launches replayed from a CUDA graph).
#include <cstdlib>
#include <cstring>

#include "../../include/q27b200/capi.h"
#include "common.cuh"
#include "layout.h"

namespace q27b {

std::string& last_error() {
  thread_local std::string e;
  return e;
}

int fail(const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  last_error() = buf;
  return -1;
}

namespace {

float g_last_us = 0.f;

cudaStream_t test_stream() {
  static cudaStream_t s = [] {
    cudaStream_t x = nullptr;
    cudaStreamCreateWithFlags(&x, cudaStreamNonBlocking);
    return x;
  }();
  return s;
}

// What the synchronous wrappers do around one launcher call `launch` (a callable returning the library's status
// code, launching on test_stream()):
//   1. drain the device, so that the call starts from a quiet GPU and earlier failures are not blamed on it;
//   2. launch once and wait for the private stream;
//   3. when the environment asks for timing (Q27T_REPEAT=n, the reference's switch, engine/src/capi.cc:57-92): time n
//      more launches, replayed from a CUDA graph so that host launch cost stays out, into q27t_last_us();
//   4. fail if a kernel gave up on a bounded wait (device status word).
struct ReplayTimer {  // the graph of `n` launches and the two events; everything is released on scope exit
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  cudaEvent_t begin = nullptr, end = nullptr;
  ~ReplayTimer() {
    if (begin) cudaEventDestroy(begin);
    if (end) cudaEventDestroy(end);
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
  }
};

template <class Launch>
int time_replays(Launch& launch, int n) {
  ReplayTimer t;
  cudaStream_t s = test_stream();
  Q27B_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
  int status = 0;
  for (int i = 0; i < n && status == 0; i++) status = launch();
  Q27B_CUDA(cudaStreamEndCapture(s, &t.graph));  // (always ended, also after a failed launch)
  if (status != 0) return status;
  Q27B_CUDA(cudaGraphInstantiate(&t.exec, t.graph, 0));
  Q27B_CUDA(cudaEventCreate(&t.begin));
  Q27B_CUDA(cudaEventCreate(&t.end));
  Q27B_CUDA(cudaGraphLaunch(t.exec, s));  // one untimed replay first
  Q27B_CUDA(cudaEventRecord(t.begin, s));
  Q27B_CUDA(cudaGraphLaunch(t.exec, s));
  Q27B_CUDA(cudaEventRecord(t.end, s));
  Q27B_CUDA(cudaEventSynchronize(t.end));
  float ms = 0.f;
  Q27B_CUDA(cudaEventElapsedTime(&ms, t.begin, t.end));
  g_last_us = ms * 1000.f / float(n);
  return 0;
}

template <class Launch>
int kernel(Launch&& launch) {
  Q27B_CUDA(cudaDeviceSynchronize());
  if (int status = launch()) return status;
  Q27B_CUDA(cudaStreamSynchronize(test_stream()));
  const char* repeat = getenv("Q27T_REPEAT");
  if (repeat && atoi(repeat) > 0)
    if (int status = time_replays(launch, atoi(repeat))) return status;
  uint32_t waited_out = 0;
  if (int status = q27b_device_status(&waited_out)) return status;
  Q27B_REQUIRE(waited_out == 0, "a bounded wait inside a kernel ran out (device status %u)", waited_out);
  return 0;
}

}  // namespace
}  // namespace q27b

using namespace q27b;

extern "C" {

const char* q27_last_error(void) { return last_error().c_str(); }
float q27t_last_us(void) { return g_last_us; }
int64_t q27t_sf_bytes(int64_t rows, int64_t kblocks) { return sf_bytes(rows, kblocks); }

int q27t_quant_fp4(const float* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf) {
  return kernel([&] { return q27b_quant_fp4(x, M, K, input_scale, q, sf, test_stream()); });
}
int q27t_quant_fp4_dynamic(const float* x, int M, int K, uint8_t* q, uint8_t* sf, float* ascale) {
  return kernel([&] { return q27b_quant_fp4_dynamic(x, M, K, q, sf, ascale, test_stream()); });
}
int q27t_skinny_fp4_scaled(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const float* ascale,
                           const uint8_t* w, const uint8_t* w_sf, const float* wscale, float* d, void* ws,
                           size_t ws_bytes) {
  return kernel([&] {
    return q27b_skinny_fp4_scaled(M, N, K, a, a_sf, ascale, w, w_sf, wscale, d, ws, ws_bytes, test_stream());
  });
}
int q27t_quant_fp4_weight(const void* w, int M, int K, float global, uint8_t* q, uint8_t* sf) {
  return kernel([&] { return q27b_quant_fp4_weight(w, M, K, global, q, sf, test_stream()); });
}
int q27t_quant_fp4_bf16(const void* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf) {
  return kernel([&] { return q27b_quant_fp4_bf16(x, M, K, input_scale, q, sf, test_stream()); });
}
int q27t_rmsnorm_quant(const float* x, const void* w, int T, float eps, float* out, int kind, float in_scale, uint8_t* q,
                       uint8_t* sf) {
  Q27B_REQUIRE(kind == 0 || kind == 2, "rmsnorm_quant: only the plain (0) and NVFP4 (2) outputs are part of this path");
  return kernel([&] {
    return q27b_rmsnorm_quant_fp4(x, w, T, 5120, eps, out, in_scale, kind == 2 ? q : nullptr, sf, nullptr, 0, nullptr,
                                  test_stream());
  });
}
int q27t_silu_mul_quant_fp4(const float* g, const float* u, int64_t ld, int T, int I, float in_scale, uint8_t* q,
                            uint8_t* sf) {
  return kernel([&] { return q27b_silu_mul_quant_fp4(g, u, ld, T, I, in_scale, q, sf, test_stream()); });
}
int q27t_silu_mul_quant_fp4_bf16(const void* g, const void* u, int64_t ld, int T, int I, float in_scale, uint8_t* q,
                                 uint8_t* sf) {
  return kernel([&] { return q27b_silu_mul_quant_fp4_bf16(g, u, ld, T, I, in_scale, q, sf, test_stream()); });
}
int q27t_silu_mul_quant_fp4_glu(const float* gu, int T, int I, float ag, float au, float in_scale, uint8_t* q,
                                uint8_t* sf) {
  return kernel([&] { return q27b_silu_mul_quant_fp4_glu(gu, T, I, ag, au, in_scale, q, sf, test_stream()); });
}
int q27t_silu_mul_quant_fp4_glu_bf16(const void* gu, int T, int I, float ag, float au, float in_scale, uint8_t* q,
                                     uint8_t* sf) {
  return kernel([&] { return q27b_silu_mul_quant_fp4_glu_bf16(gu, T, I, ag, au, in_scale, q, sf, test_stream()); });
}
int q27t_swizzle_sf(const uint8_t* src, int rows, int kblocks, uint8_t* dst) {
  return kernel([&] { return q27b_swizzle_sf(src, rows, kblocks, dst, -1, test_stream()); });
}
int q27t_swizzle_sf_glu(const uint8_t* src, int rows, int kblocks, uint8_t* dst, int half) {
  return kernel([&] { return q27b_swizzle_sf(src, rows, kblocks, dst, half, test_stream()); });
}
int q27t_gemm_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
                  float alpha, const float* c, float beta, float* d) {
  return kernel([&] { return q27b_gemm_fp4(M, N, K, a, a_sf, b, b_sf, alpha, c, beta, d, test_stream()); });
}
int q27t_gemm_fp4_bf16(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b,
                       const uint8_t* b_sf, float alpha, void* d) {
  return kernel([&] { return q27b_gemm_fp4_bf16(M, N, K, a, a_sf, b, b_sf, alpha, d, test_stream()); });
}
int q27t_gemm_fp4_glu_bf16(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                           const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, void* d) {
  return kernel([&] {
    return q27b_gemm_fp4_glu_bf16(M, I, K, a, a_sf, gate_up, gate_up_sf, alpha_gate, alpha_up, d, test_stream());
  });
}
int q27t_gemm_fp4_glu(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                      const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, float out_scale, uint8_t* q,
                      uint8_t* q_sf) {
  return kernel([&] {
    return q27b_gemm_fp4_glu(M, I, K, a, a_sf, gate_up, gate_up_sf, alpha_gate, alpha_up, out_scale, q, q_sf, test_stream());
  });
}
int q27t_skinny_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w, const uint8_t* w_sf,
                    float alpha, const float* c, float beta, float* d, void* ws, size_t ws_bytes) {
  const int zero = 0;
  return kernel([&] {
    return q27b_skinny_fp4(M, N, K, a, a_sf, w, w_sf, 1, &zero, &alpha, c, beta, d, ws, ws_bytes, test_stream());
  });
}
int q27t_skinny_fp4_segments(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                             const uint8_t* w_sf, int count, const int* begin, const float* alpha, const float* c,
                             float beta, float* d, void* ws, size_t ws_bytes) {
  return kernel([&] {
    return q27b_skinny_fp4(M, N, K, a, a_sf, w, w_sf, count, begin, alpha, c, beta, d, ws, ws_bytes, test_stream());
  });
}
int q27t_skinny_fp4_bf16(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                         const uint8_t* w_sf, float alpha, void* d, void* ws, size_t ws_bytes) {
  const int zero = 0;
  return kernel([&] {
    return q27b_skinny_fp4_bf16(M, N, K, a, a_sf, w, w_sf, 1, &zero, &alpha, d, ws, ws_bytes, test_stream());
  });
}
int q27t_skinny_fp4_glu_bf16(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                             const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, void* d, void* ws,
                             size_t ws_bytes) {
  return kernel([&] {
    return q27b_skinny_fp4_glu_bf16(M, I, K, a, a_sf, gate_up, gate_up_sf, alpha_gate, alpha_up, d, ws, ws_bytes,
                                    test_stream());
  });
}
int q27t_skinny_fp4_static(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                           const uint8_t* w_sf, float alpha, const float* c, float beta, float* d) {
  const int zero = 0;
  return kernel([&] {
    return q27b_skinny_fp4_static(M, N, K, a, a_sf, w, w_sf, 1, &zero, &alpha, c, beta, d, test_stream());
  });
}
int q27t_skinny_fp4_group(const void* table_host, const void* table_dev, void* ws, size_t ws_bytes) {
  return kernel([&] { return q27b_skinny_fp4_group(table_host, table_dev, ws, ws_bytes, test_stream()); });
}
// Average time (us) of `iters` calls cycling through `nbuf` weight copies w_stride / sf_stride bytes apart (so
// that the weights never come from L2). many != 0: the many-row GEMM; else the weight-streaming one.
int q27t_bench_gemm(int many, int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                    const uint8_t* w_sf, int64_t w_stride, int64_t sf_stride, int nbuf, int iters, float* d, void* ws,
                    size_t ws_bytes, float* us) {
  Q27B_REQUIRE(nbuf >= 1 && iters >= 1 && us, "bench_gemm: bad arguments");
  return kernel([&]() -> int {
    const int zero = 0;
    const float one = 1.f;
    auto run = [&](int i) -> int {
      const uint8_t* wi = w + int64_t(i % nbuf) * w_stride;
      const uint8_t* si = w_sf + int64_t(i % nbuf) * sf_stride;
      if (many) return q27b_gemm_fp4(M, N, K, a, a_sf, wi, si, 1.f, nullptr, 0.f, d, test_stream());
      return q27b_skinny_fp4(M, N, K, a, a_sf, wi, si, 1, &zero, &one, nullptr, 0.f, d, ws, ws_bytes, test_stream());
    };
    for (int i = 0; i < (nbuf > iters ? nbuf : iters); i++)
      if (int rc = run(i)) return rc;
    cudaEvent_t e0, e1;
    Q27B_CUDA(cudaEventCreate(&e0));
    Q27B_CUDA(cudaEventCreate(&e1));
    Q27B_CUDA(cudaEventRecord(e0, test_stream()));
    for (int i = 0; i < iters; i++)
      if (int rc = run(i)) return rc;
    Q27B_CUDA(cudaEventRecord(e1, test_stream()));
    Q27B_CUDA(cudaEventSynchronize(e1));
    float ms = 0.f;
    Q27B_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    *us = 1000.f * ms / iters;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return 0;
  });
}

}  // extern "C"
