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

// gates of one (batch, head, token): sigmoid of the three logits, or their softmax (nsa/kernels.py:2446-2451)
__device__ __forceinline__ void gates3(const float* lg, int mode, float g[3]) {
  if (mode == NSA_GATE_SOFTMAX) {
    const float m = fmaxf(lg[0], fmaxf(lg[1], lg[2]));
    const float e0 = expf(lg[0] - m), e1 = expf(lg[1] - m), e2 = expf(lg[2] - m);
    const float inv = 1.f / (e0 + e1 + e2);
    g[0] = e0 * inv; g[1] = e1 * inv; g[2] = e2 * inv;
  } else {
#pragma unroll
    for (int i = 0; i < 3; ++i) g[i] = 1.f / (1.f + expf(-lg[i]));
  }
}

// Row index of (b,h,t) in the mixed output (and in its gradient): head-major [B,H,T,dv] like the branch outputs, or
// token-major [B,T,H,dv], the layout the output projection consumes without a transposing copy.
__device__ __forceinline__ int64_t mixed_row(int64_t row, int b, int h, int t, int H, int T_, int token_major) {
  return token_major ? ((int64_t)b * T_ + t) * H + h : row;
}

constexpr int kMaxHeadDim = 256;  // generic kernels keep head_dim/32 accumulators per lane

}  // namespace nsa
