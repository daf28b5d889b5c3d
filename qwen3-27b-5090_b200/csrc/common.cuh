// Error convention of the C-ABI layer and small shared types.
// Every extern "C" entry point returns 0 on success and -1 on failure, leaving a thread-local message for
// q27_last_error() (the convention of engine/src/capi.cc:19-36 in the reference). Nothing here allocates.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <cstdio>
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

}  // namespace q27b
