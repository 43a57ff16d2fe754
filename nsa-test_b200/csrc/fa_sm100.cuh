// Tensor-core (tcgen05) attention kernels for sm_100a: parameters and host entry points.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nsa {

struct FaFwdParams {
  __nv_bfloat16* o;  // [B,H,Tq,dv] contiguous
  float *L, *M;      // [B,H,Tq] contiguous, may be null
  int B, H, G, Tq, Tk;
  int window;                // sliding window: keys (t-window, t]
  int cmp_l, cmp_d, cmp_nb;  // compressed tokens: key i visible iff i < cmp_nb and i*cmp_d + cmp_l - 1 <= t
  float scale_log2;          // softmax scale times log2(e)
};

// True when the tensor-core forward covers this shape (bf16, canonical contiguous layouts assumed).
bool fa_fwd_sm100_supported(int H, int G, int Tq, int Tk, int dk, int dv);

// q [B,H,Tq,dk], k [B,G,dk,Tk], v [B,G,Tk,dv], o [B,H,Tq,dv]: contiguous bf16.  mode = kWin or kCmp.
int fa_fwd_sm100(const void* q, const void* k, const void* v, void* o, float* L, float* M, int B, int H, int G, int Tq,
                 int Tk, int dk, int dv, int mode, int window, int cmp_l, int cmp_d, int cmp_nb, float scale,
                 cudaStream_t st);

// Number of CTAs that ever gave up on a barrier wait (0 in a healthy run); optionally reset.
int fa_fwd_sm100_timeouts(int* count, bool reset);

}  // namespace nsa
