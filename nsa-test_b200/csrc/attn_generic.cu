// Stride-generic attention kernels (fp32 math on CUDA cores) for the three NSA branches.
//
// These kernels honour arbitrary element strides and any head dim <= 256, in fp32 or bf16 storage.
// They serve the raw kernel-call contract (callers may pass any strides), fp32 I/O, and shapes the
// tensor-core kernels do not cover.  One warp owns one query row (forward, dQ) or one key row
// (dK/dV), so every reduction has a single writer and a fixed order: results are deterministic.
//
// Semantics follow the reference kernels: _nsa_sliding_window_* (nsa/kernels.py:1151-1530),
// _nsa_compression_* (nsa/kernels.py:1533-1917), _nsa_sparse_selection_* (nsa/kernels.py:594-1148):
// logits = (q*scale)·k, masked rows give O=0, L=M=-inf, L = log(sum exp(s-M)).
#include "attn_args.cuh"
#include "common.cuh"

namespace nsa {

constexpr int kWarps = 4;

// Calls f(kbeg, kend) for every contiguous run of candidate keys of query t.
template <int MODE, typename F>
__device__ __forceinline__ void for_each_segment(const AttnArgs& a, int b, int g, int t, F&& f) {
  if (MODE == kWin) {
    int beg = max(0, t - a.window + 1), end = min(t + 1, a.Tk);
    if (beg < end) f(beg, end);
  } else if (MODE == kCmp) {
    if (a.Tk > 0) f(0, a.Tk);
  } else {
    const int* row = a.indices + b * a.sidx[0] + g * a.sidx[1] + (int64_t)t * a.sidx[2];
    for (int s = 0; s < a.nslots; ++s) {
      int id = row[s * a.sidx[3]];
      if (id < 0) continue;
      int64_t beg = (int64_t)id * a.lprime;
      if (beg >= a.Tk || (a.causal && beg > t)) continue;
      bool dup = false;
      for (int s2 = 0; s2 < s; ++s2) dup |= (row[s2 * a.sidx[3]] == id);
      if (dup) continue;
      int64_t end = min(beg + a.lprime, (int64_t)a.Tk);
      if (a.causal) end = min(end, (int64_t)t + 1);
      f((int)beg, (int)end);
    }
  }
}

template <int MODE>
__device__ __forceinline__ bool key_visible(const AttnArgs& a, int key, int t) {
  return MODE == kCmp ? (a.block_ends[key] <= t) : true;
}

// ------------------------------------------------------------------------------------------------
// forward: one warp per (b,h,t)
// ------------------------------------------------------------------------------------------------
template <typename T, int MODE>
__global__ void __launch_bounds__(kWarps * 32) attn_fwd_generic(const __grid_constant__ AttnArgs a) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kWarps + warp;
  const int b = blockIdx.y / a.H, h = blockIdx.y % a.H, g = h / (a.H / a.G);
  if (t >= a.Tq) return;
  float* qs = smem + warp * a.dk;
  const T* qp = (const T*)a.q + b * a.sq[0] + h * a.sq[1] + (int64_t)t * a.sq[2];
  for (int d = lane; d < a.dk; d += 32) qs[d] = Elem<T>::ld(qp + d * a.sq[3]) * a.scale;
  __syncwarp();
  const T* kp = (const T*)a.k + b * a.sk[0] + g * a.sk[1];
  const T* vp = (const T*)a.v + b * a.sv[0] + g * a.sv[1];
  const int nv = (a.dv + 31) / 32;
  float m = -CUDART_INF_F, l = 0.f, acc[kMaxHeadDim / 32];
#pragma unroll
  for (int c = 0; c < kMaxHeadDim / 32; ++c) acc[c] = 0.f;

  for_each_segment<MODE>(a, b, g, t, [&](int kbeg, int kend) {
    for (int k0 = kbeg; k0 < kend; k0 += 32) {
      const int key = k0 + lane;
      const bool valid = key < kend && key_visible<MODE>(a, key, t);
      float s = -CUDART_INF_F;
      if (valid) {
        const T* kr = kp + (int64_t)key * a.sk[2];
        s = 0.f;
        for (int d = 0; d < a.dk; ++d) s = fmaf(qs[d], Elem<T>::ld(kr + d * a.sk[3]), s);
      }
      const float mx = warp_max(s);
      if (mx == -CUDART_INF_F) continue;
      const float mnew = fmaxf(m, mx);
      const float p = valid ? expf(s - mnew) : 0.f;
      const float alpha = expf(m - mnew);  // m = -inf -> 0
      l = l * alpha + warp_sum(p);
#pragma unroll
      for (int c = 0; c < kMaxHeadDim / 32; ++c) acc[c] *= alpha;
      for (int j = 0; j < 32; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        if (pj == 0.f) continue;
        const T* vr = vp + (int64_t)(k0 + j) * a.sv[2];
#pragma unroll
        for (int c = 0; c < kMaxHeadDim / 32; ++c)
          if (c < nv && lane + 32 * c < a.dv) acc[c] = fmaf(pj, Elem<T>::ld(vr + (lane + 32 * c) * a.sv[3]), acc[c]);
      }
      m = mnew;
    }
  });

  T* op = (T*)a.o + b * a.so[0] + h * a.so[1] + (int64_t)t * a.so[2];
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int c = 0; c < kMaxHeadDim / 32; ++c)
    if (lane + 32 * c < a.dv) Elem<T>::st(op + (lane + 32 * c) * a.so[3], acc[c] * inv);
  if (lane == 0) {
    if (a.L) a.L[b * a.sL[0] + h * a.sL[1] + (int64_t)t * a.sL[2]] = l > 0.f ? logf(l) : -CUDART_INF_F;
    if (a.M) a.M[b * a.sM[0] + h * a.sM[1] + (int64_t)t * a.sM[2]] = m;
  }
}

// ------------------------------------------------------------------------------------------------
// backward dQ: one warp per (b,h,t); P is recomputed from the saved statistics
// ------------------------------------------------------------------------------------------------
template <typename T, int MODE>
__global__ void __launch_bounds__(kWarps * 32) attn_bwd_dq_generic(const __grid_constant__ AttnArgs a) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kWarps + warp;
  const int b = blockIdx.y / a.H, h = blockIdx.y % a.H, g = h / (a.H / a.G);
  if (t >= a.Tq) return;
  float* qs = smem + warp * (a.dk + a.dv);
  float* dos = qs + a.dk;
  const T* qp = (const T*)a.q + b * a.sq[0] + h * a.sq[1] + (int64_t)t * a.sq[2];
  const T* op = (const T*)a.o_in + b * a.so[0] + h * a.so[1] + (int64_t)t * a.so[2];
  const T* dop = (const T*)a.dout + b * a.so[0] + h * a.so[1] + (int64_t)t * a.so[2];
  float dsum = 0.f;
  for (int d = lane; d < a.dk; d += 32) qs[d] = Elem<T>::ld(qp + d * a.sq[3]) * a.scale;
  for (int c = lane; c < a.dv; c += 32) {
    const float x = Elem<T>::ld(dop + c * a.so[3]);
    dos[c] = x;
    dsum = fmaf(x, Elem<T>::ld(op + c * a.so[3]), dsum);
  }
  const float D = warp_sum(dsum);
  __syncwarp();
  const float lse = a.Mc[b * a.sM[0] + h * a.sM[1] + (int64_t)t * a.sM[2]] +
                    a.Lc[b * a.sL[0] + h * a.sL[1] + (int64_t)t * a.sL[2]];
  const bool row_ok = isfinite(lse);
  const T* kp = (const T*)a.k + b * a.sk[0] + g * a.sk[1];
  const T* vp = (const T*)a.v + b * a.sv[0] + g * a.sv[1];
  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int c = 0; c < kMaxHeadDim / 32; ++c) acc[c] = 0.f;

  if (row_ok) {
    for_each_segment<MODE>(a, b, g, t, [&](int kbeg, int kend) {
      for (int k0 = kbeg; k0 < kend; k0 += 32) {
        const int key = k0 + lane;
        const bool valid = key < kend && key_visible<MODE>(a, key, t);
        float ds = 0.f;
        if (valid) {
          const T* kr = kp + (int64_t)key * a.sk[2];
          const T* vr = vp + (int64_t)key * a.sv[2];
          float s = 0.f, dp = 0.f;
          for (int d = 0; d < a.dk; ++d) s = fmaf(qs[d], Elem<T>::ld(kr + d * a.sk[3]), s);
          for (int c = 0; c < a.dv; ++c) dp = fmaf(dos[c], Elem<T>::ld(vr + c * a.sv[3]), dp);
          ds = expf(s - lse) * (dp - D);
        }
        for (int j = 0; j < 32; ++j) {
          const float dsj = __shfl_sync(0xffffffffu, ds, j);
          if (dsj == 0.f) continue;
          const T* kr = kp + (int64_t)(k0 + j) * a.sk[2];
#pragma unroll
          for (int c = 0; c < kMaxHeadDim / 32; ++c)
            if (lane + 32 * c < a.dk) acc[c] = fmaf(dsj, Elem<T>::ld(kr + (lane + 32 * c) * a.sk[3]), acc[c]);
        }
      }
    });
  }
  T* dqp = (T*)a.dq + b * a.sdq[0] + h * a.sdq[1] + (int64_t)t * a.sdq[2];
#pragma unroll
  for (int c = 0; c < kMaxHeadDim / 32; ++c)
    if (lane + 32 * c < a.dk) Elem<T>::st(dqp + (lane + 32 * c) * a.sdq[3], acc[c] * a.scale);
}

// ------------------------------------------------------------------------------------------------
// backward dK/dV: one warp per (b,g,key); heads in order, queries in order -> fixed summation order
// ------------------------------------------------------------------------------------------------
template <typename T, int MODE>
__global__ void __launch_bounds__(kWarps * 32) attn_bwd_dkv_generic(const __grid_constant__ AttnArgs a) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int key = blockIdx.x * kWarps + warp;
  const int b = blockIdx.y / a.G, g = blockIdx.y % a.G;
  if (key >= a.Tk) return;
  float* ks = smem + warp * (a.dk + a.dv);
  float* vs = ks + a.dk;
  const T* kr = (const T*)a.k + b * a.sk[0] + g * a.sk[1] + (int64_t)key * a.sk[2];
  const T* vr = (const T*)a.v + b * a.sv[0] + g * a.sv[1] + (int64_t)key * a.sv[2];
  for (int d = lane; d < a.dk; d += 32) ks[d] = Elem<T>::ld(kr + d * a.sk[3]) * a.scale;
  for (int c = lane; c < a.dv; c += 32) vs[c] = Elem<T>::ld(vr + c * a.sv[3]);
  __syncwarp();

  // query list of this key: a range [tbeg,tend) or a slice of the inverse index
  int tbeg = 0, tend = 0;
  const int* tl = nullptr;
  if (MODE == kWin) {
    tbeg = key;
    tend = min(a.Tq, key + a.window);
  } else if (MODE == kCmp) {
    tbeg = max(a.block_ends[key], 0);
    tend = a.Tq;
  } else {
    const int blk = key / a.lprime;
    const int* off = a.csr_off + (int64_t)(b * a.G + g) * (a.nblk + 1);
    tl = a.csr_t + (int64_t)(b * a.G + g) * a.Tq * a.nslots;
    tbeg = off[blk];
    tend = off[blk + 1];
  }
  float acck[kMaxHeadDim / 32], accv[kMaxHeadDim / 32];
#pragma unroll
  for (int c = 0; c < kMaxHeadDim / 32; ++c) acck[c] = accv[c] = 0.f;
  const int hpg = a.H / a.G;

  for (int hh = 0; hh < hpg; ++hh) {
    const int h = g * hpg + hh;
    const T* qb = (const T*)a.q + b * a.sq[0] + h * a.sq[1];
    const T* ob = (const T*)a.o_in + b * a.so[0] + h * a.so[1];
    const T* dob = (const T*)a.dout + b * a.so[0] + h * a.so[1];
    for (int e0 = tbeg; e0 < tend; e0 += 32) {
      const int e = e0 + lane;
      int t = -1;
      if (e < tend) {
        t = (MODE == kSlc) ? (tl[e] & 0xFFFFFF) : e;
        if (MODE == kSlc && a.causal && t < key) t = -1;
      }
      float p = 0.f, ds = 0.f;
      if (t >= 0) {
        const float lse = a.Mc[b * a.sM[0] + h * a.sM[1] + (int64_t)t * a.sM[2]] +
                          a.Lc[b * a.sL[0] + h * a.sL[1] + (int64_t)t * a.sL[2]];
        if (isfinite(lse)) {
          const T* qr = qb + (int64_t)t * a.sq[2];
          const T* orow = ob + (int64_t)t * a.so[2];
          const T* dor = dob + (int64_t)t * a.so[2];
          float s = 0.f, dp = 0.f, D = 0.f;
          for (int d = 0; d < a.dk; ++d) s = fmaf(ks[d], Elem<T>::ld(qr + d * a.sq[3]), s);
          for (int c = 0; c < a.dv; ++c) {
            const float x = Elem<T>::ld(dor + c * a.so[3]);
            dp = fmaf(x, vs[c], dp);
            D = fmaf(x, Elem<T>::ld(orow + c * a.so[3]), D);
          }
          p = expf(s - lse);
          ds = p * (dp - D);
        }
      }
      for (int j = 0; j < 32; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const float dsj = __shfl_sync(0xffffffffu, ds, j);
        const int tj = __shfl_sync(0xffffffffu, t, j);
        if (pj == 0.f && dsj == 0.f) continue;
        const T* qr = qb + (int64_t)tj * a.sq[2];
        const T* dor = dob + (int64_t)tj * a.so[2];
#pragma unroll
        for (int c = 0; c < kMaxHeadDim / 32; ++c) {
          if (lane + 32 * c < a.dk) acck[c] = fmaf(dsj, Elem<T>::ld(qr + (lane + 32 * c) * a.sq[3]), acck[c]);
          if (lane + 32 * c < a.dv) accv[c] = fmaf(pj, Elem<T>::ld(dor + (lane + 32 * c) * a.so[3]), accv[c]);
        }
      }
    }
  }
  T* dkp = (T*)a.dk_out + b * a.sdk[0] + g * a.sdk[1] + (int64_t)key * a.sdk[2];
  T* dvp = (T*)a.dv_out + b * a.sdv[0] + g * a.sdv[1] + (int64_t)key * a.sdv[2];
#pragma unroll
  for (int c = 0; c < kMaxHeadDim / 32; ++c) {
    const int i = lane + 32 * c;
    if (i < a.dk) Elem<T>::st(dkp + i * a.sdk[3], Elem<T>::ld(dkp + i * a.sdk[3]) + acck[c] * a.scale);
    if (i < a.dv) Elem<T>::st(dvp + i * a.sdv[3], Elem<T>::ld(dvp + i * a.sdv[3]) + accv[c]);
  }
}

// ------------------------------------------------------------------------------------------------
// host launchers
// ------------------------------------------------------------------------------------------------
template <typename T, int MODE>
static int launch_fwd_t(const AttnArgs& a, cudaStream_t st) {
  KernelTimer kt("attn_fwd_generic", st);
  dim3 grid((a.Tq + kWarps - 1) / kWarps, a.B * a.H);
  attn_fwd_generic<T, MODE><<<grid, kWarps * 32, kWarps * a.dk * sizeof(float), st>>>(a);
  return check_launch("attn_fwd_generic");
}
template <typename T, int MODE>
static int launch_bwd_t(const AttnArgs& a, cudaStream_t st) {
  KernelTimer kt("attn_bwd_generic", st);
  const size_t sm = kWarps * (a.dk + a.dv) * sizeof(float);
  dim3 gq((a.Tq + kWarps - 1) / kWarps, a.B * a.H);
  attn_bwd_dq_generic<T, MODE><<<gq, kWarps * 32, sm, st>>>(a);
  if (int rc = check_launch("attn_bwd_dq_generic")) return rc;
  if (a.Tk == 0) return NSA_OK;
  dim3 gk((a.Tk + kWarps - 1) / kWarps, a.B * a.G);
  attn_bwd_dkv_generic<T, MODE><<<gk, kWarps * 32, sm, st>>>(a);
  return check_launch("attn_bwd_dkv_generic");
}

int launch_attn_generic(const AttnArgs& a, int mode, int dtype, bool backward, cudaStream_t st) {
  if (a.B * a.H == 0 || a.Tq == 0) return NSA_OK;
#define NSA_DISPATCH(T)                                                                  \
  switch (mode) {                                                                        \
    case kWin: return backward ? launch_bwd_t<T, kWin>(a, st) : launch_fwd_t<T, kWin>(a, st); \
    case kCmp: return backward ? launch_bwd_t<T, kCmp>(a, st) : launch_fwd_t<T, kCmp>(a, st); \
    case kSlc: return backward ? launch_bwd_t<T, kSlc>(a, st) : launch_fwd_t<T, kSlc>(a, st); \
  }
  if (dtype == NSA_F32) {
    NSA_DISPATCH(float)
  } else if (dtype == NSA_BF16) {
    NSA_DISPATCH(__nv_bfloat16)
  }
#undef NSA_DISPATCH
  return fail(NSA_ERR_ARG, "unsupported dtype %d / mode %d", dtype, mode);
}

}  // namespace nsa
