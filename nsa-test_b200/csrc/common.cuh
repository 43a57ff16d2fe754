// Shared helpers for the NSA sm_100a kernels: error reporting, dtype traits, warp reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/nsa_b200.h"

namespace nsa {

// Thread-local message behind nsa_last_error().
char* error_buffer();
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);

// Optional per-kernel timing (nsa_profile_enable): records a CUDA event pair around a launch on the
// launching stream.  Costs nothing while profiling is off.
struct KernelTimer {
  KernelTimer(const char* name, cudaStream_t st);
  ~KernelTimer();
  cudaStream_t st_;
  int slot_;
};

#define NSA_REQUIRE(cond, ...)                                  \
  do {                                                          \
    if (!(cond)) return ::nsa::fail(NSA_ERR_ARG, __VA_ARGS__);  \
  } while (0)

template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float x) { *p = x; }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
};

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

constexpr int kMaxHeadDim = 256;  // generic kernels keep head_dim/32 accumulators per lane

}  // namespace nsa
