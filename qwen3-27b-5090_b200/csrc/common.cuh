// Error convention of the C-ABI layer and small shared types.
// Every extern "C" entry point returns 0 on success and -1 on failure, leaving a thread-local message for
// q27_last_error() (the convention of engine/src/capi.cc:19-36 in the reference). Nothing here allocates.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace q27b {

std::string& last_error();                 // thread-local
int fail(const char* fmt, ...);            // formats the message, returns -1
uint32_t* device_status_ptr();             // address of the per-device status word (resolved once per device)
int sm_count();                            // multiprocessors of the current device (cached per device)

#define Q27B_REQUIRE(cond, ...)                    \
  do {                                             \
    if (!(cond)) return ::q27b::fail(__VA_ARGS__); \
  } while (0)

#define Q27B_CUDA(call)                                                                              \
  do {                                                                                               \
    cudaError_t err_ = (call);                                                                       \
    if (err_ != cudaSuccess)                                                                         \
      return ::q27b::fail("%s failed: %s at %s:%d", #call, cudaGetErrorString(err_), __FILE__, __LINE__); \
  } while (0)

// Per-output-channel alpha of fused projections: alpha[i] applies from column begin[i] on
// (AlphaSegments, engine/src/kernels.h:228-239).
struct AlphaSeg {
  int count;
  int begin[4];
  float alpha[4];
};

__host__ __device__ inline float alpha_of(const AlphaSeg& a, int n) {
  float v = a.alpha[0];
#pragma unroll
  for (int i = 1; i < 4; i++)
    if (i < a.count && n >= a.begin[i]) v = a.alpha[i];
  return v;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Per-launch switches. They are read from the environment at EVERY launch, so that a CUDA graph captured after a
// change sees the new value (the reference reads its tunables the same way, engine/src/skinny.cu:494-521,
// engine/src/launch.cuh:15):
//   Q27_NO_PDL=1               no launch of this library carries the programmatic-dependent-launch attribute: every
//                              kernel starts only after its predecessor in the stream has completed (debugging a
//                              chain; weights written by the preceding kernel);
//   Q27_SKINNY_EXT_REDUCE_M=m  the weight-streaming GEMM sums cut tiles in its separate fix-up kernel above m
//                              tokens (0..16, default 8; above 16 tokens it always does).
inline bool env_flag(const char* name) {
  const char* e = getenv(name);
  return e && *e && !(e[0] == '0' && e[1] == 0);
}
inline int env_int(const char* name, int dflt, int lo, int hi) {
  const char* e = getenv(name);
  if (!e || !*e) return dflt;
  const int v = atoi(e);
  return v < lo ? lo : (v > hi ? hi : v);
}
inline bool pdl_enabled() { return !env_flag("Q27_NO_PDL"); }

}  // namespace q27b
