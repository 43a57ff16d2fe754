// Branch gates and mix (Eq. 5; nsa/kernels.py:2446-2463): gates = sigmoid (or softmax over the three
// branches) of logits[b,t,3h+i], out = g0*o_cmp + g1*o_slc + g2*o_win.  HBM-bound: three reads and
// one write of [B,H,T,dv] forward; backward reads four tensors and writes three.
#include "common.cuh"

namespace nsa {

// one warp per (b,h,t) row
template <typename T>
__global__ void gate_mix_fwd_kernel(const float* __restrict__ logits, const T* __restrict__ oc, const T* __restrict__ os,
                                    const T* __restrict__ ow, T* __restrict__ out, float* __restrict__ gates, int B,
                                    int H, int T_, int dv, int mode, int out_tm) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= (int64_t)B * H * T_) return;
  const int t = row % T_, h = (row / T_) % H, b = row / ((int64_t)T_ * H);
  float g[3];
  gates3(logits + ((int64_t)b * T_ + t) * 3 * H + 3 * h, mode, g);
  if (lane < 3) gates[row * 3 + lane] = g[lane];
  const int64_t base = row * dv, obase = mixed_row(row, b, h, t, H, T_, out_tm) * dv;
  for (int c = lane; c < dv; c += 32) {
    const float x = Elem<T>::ld(oc + base + c) * g[0];
    const float y = x + Elem<T>::ld(os + base + c) * g[1];
    Elem<T>::st(out + obase + c, y + Elem<T>::ld(ow + base + c) * g[2]);
  }
}

template <typename T>
__global__ void gate_mix_bwd_kernel(const float* __restrict__ gates, const T* __restrict__ oc, const T* __restrict__ os,
                                    const T* __restrict__ ow, const T* __restrict__ dout, T* __restrict__ doc,
                                    T* __restrict__ dos, T* __restrict__ dow, float* __restrict__ dlogits, int B, int H,
                                    int T_, int dv, int mode, float* __restrict__ delta, int dout_tm) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= (int64_t)B * H * T_) return;
  const int t = row % T_, h = (row / T_) % H, b = row / ((int64_t)T_ * H);
  const float g0 = gates[row * 3], g1 = gates[row * 3 + 1], g2 = gates[row * 3 + 2];
  const int64_t base = row * dv, dbase = mixed_row(row, b, h, t, H, T_, dout_tm) * dv;
  float d0 = 0.f, d1 = 0.f, d2 = 0.f;
  for (int c = lane; c < dv; c += 32) {
    const float dy = Elem<T>::ld(dout + dbase + c);
    d0 = fmaf(dy, Elem<T>::ld(oc + base + c), d0);
    d1 = fmaf(dy, Elem<T>::ld(os + base + c), d1);
    d2 = fmaf(dy, Elem<T>::ld(ow + base + c), d2);
    Elem<T>::st(doc + base + c, dy * g0);
    Elem<T>::st(dos + base + c, dy * g1);
    Elem<T>::st(dow + base + c, dy * g2);
  }
  d0 = warp_sum(d0); d1 = warp_sum(d1); d2 = warp_sum(d2);
  if (lane == 0) {
    if (delta) {  // row sums dO_b . O_b of the three branches, dO_b = g_b dO
      const int64_t rows = (int64_t)B * H * T_;
      delta[row] = g0 * d0; delta[rows + row] = g1 * d1; delta[2 * rows + row] = g2 * d2;
    }
    float* dl = dlogits + ((int64_t)b * T_ + t) * 3 * H + 3 * h;
    if (mode == NSA_GATE_SOFTMAX) {
      const float dot = g0 * d0 + g1 * d1 + g2 * d2;
      dl[0] = g0 * (d0 - dot); dl[1] = g1 * (d1 - dot); dl[2] = g2 * (d2 - dot);
    } else {
      dl[0] = d0 * g0 * (1.f - g0); dl[1] = d1 * g1 * (1.f - g1); dl[2] = d2 * g2 * (1.f - g2);
    }
  }
}

// bf16, dv a multiple of 128: each lane owns 4 consecutive values (8-byte accesses, 256 B per warp and row segment)
__device__ __forceinline__ void unpack4(const uint2 r, float (&f)[4]) {
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ uint2 pack4(const float (&f)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  return make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}

__device__ __forceinline__ void unpack8(const uint4 r, float (&f)[8]) {
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.z));
  const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.w));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  __nv_bfloat162 c = __floats2bfloat162_rn(f[4], f[5]), d = __floats2bfloat162_rn(f[6], f[7]);
  return make_uint4(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b), *reinterpret_cast<uint32_t*>(&c),
                    *reinterpret_cast<uint32_t*>(&d));
}

// bf16, dv a multiple of 128: half a warp per (b,h,t) row, each lane owns 8 consecutive values (16-byte accesses)
__global__ void gate_mix_fwd_bf16x4_kernel(const float* __restrict__ logits, const __nv_bfloat16* __restrict__ oc,
                                           const __nv_bfloat16* __restrict__ os, const __nv_bfloat16* __restrict__ ow,
                                           __nv_bfloat16* __restrict__ out, float* __restrict__ gates, int B, int H, int T_, int dv,
                                           int mode, int out_tm) {
  const int lane = threadIdx.x & 31, hl = lane & 15;
  const int64_t row = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 2 + (lane >> 4);
  if (row >= (int64_t)B * H * T_) return;
  const int t = row % T_, h = (row / T_) % H, b = row / ((int64_t)T_ * H);
  const int64_t base = row * dv, obase = mixed_row(row, b, h, t, H, T_, out_tm) * dv;
  // the tile loads go out before the gate arithmetic
  uint4 ra = *reinterpret_cast<const uint4*>(oc + base + hl * 8);
  uint4 rs = *reinterpret_cast<const uint4*>(os + base + hl * 8);
  uint4 rw = *reinterpret_cast<const uint4*>(ow + base + hl * 8);
  float g[3];
  gates3(logits + ((int64_t)b * T_ + t) * 3 * H + 3 * h, mode, g);
  if (hl < 3) gates[row * 3 + hl] = g[hl];
  for (int c = hl * 8; c < dv; c += 128) {
    float a[8], s_[8], w[8], y[8];
    unpack8(ra, a); unpack8(rs, s_); unpack8(rw, w);
    if (c + 128 < dv) {
      ra = *reinterpret_cast<const uint4*>(oc + base + c + 128);
      rs = *reinterpret_cast<const uint4*>(os + base + c + 128);
      rw = *reinterpret_cast<const uint4*>(ow + base + c + 128);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = (a[i] * g[0] + s_[i] * g[1]) + w[i] * g[2];
    *reinterpret_cast<uint4*>(out + obase + c) = pack8(y);
  }
}

__global__ void gate_mix_bwd_bf16x4_kernel(const float* __restrict__ gates, const __nv_bfloat16* __restrict__ oc,
                                           const __nv_bfloat16* __restrict__ os, const __nv_bfloat16* __restrict__ ow,
                                           const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ doc,
                                           __nv_bfloat16* __restrict__ dos, __nv_bfloat16* __restrict__ dow, float* __restrict__ dlogits,
                                           int B, int H, int T_, int dv, int mode, float* __restrict__ delta, int dout_tm) {
  const int lane = threadIdx.x & 31, hl = lane & 15;
  int64_t row = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 2 + (lane >> 4);
  const bool live = row < (int64_t)B * H * T_;  // both halves stay for the shuffles
  if (!live) row = 0;
  const int t = row % T_, h = (row / T_) % H, b = row / ((int64_t)T_ * H);
  const float g0 = gates[row * 3], g1 = gates[row * 3 + 1], g2 = gates[row * 3 + 2];
  const int64_t base = row * dv, dbase = mixed_row(row, b, h, t, H, T_, dout_tm) * dv;
  float d0 = 0.f, d1 = 0.f, d2 = 0.f;
  for (int c = hl * 8; c < dv; c += 128) {
    float dy[8], a[8], s_[8], w[8], r0[8], r1[8], r2[8];
    const uint4 qd = *reinterpret_cast<const uint4*>(dout + dbase + c), qa = *reinterpret_cast<const uint4*>(oc + base + c);
    const uint4 qs = *reinterpret_cast<const uint4*>(os + base + c), qw = *reinterpret_cast<const uint4*>(ow + base + c);
    unpack8(qd, dy); unpack8(qa, a); unpack8(qs, s_); unpack8(qw, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      d0 = fmaf(dy[i], a[i], d0); d1 = fmaf(dy[i], s_[i], d1); d2 = fmaf(dy[i], w[i], d2);
      r0[i] = dy[i] * g0; r1[i] = dy[i] * g1; r2[i] = dy[i] * g2;
    }
    if (live) {
      *reinterpret_cast<uint4*>(doc + base + c) = pack8(r0);
      *reinterpret_cast<uint4*>(dos + base + c) = pack8(r1);
      *reinterpret_cast<uint4*>(dow + base + c) = pack8(r2);
    }
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) {  // sums inside each half-warp
    d0 += __shfl_xor_sync(0xffffffffu, d0, o);
    d1 += __shfl_xor_sync(0xffffffffu, d1, o);
    d2 += __shfl_xor_sync(0xffffffffu, d2, o);
  }
  if (hl == 0 && live) {
    if (delta) {  // row sums dO_b . O_b of the three branches, dO_b = g_b dO
      const int64_t rows = (int64_t)B * H * T_;
      delta[row] = g0 * d0; delta[rows + row] = g1 * d1; delta[2 * rows + row] = g2 * d2;
    }
    float* dl = dlogits + ((int64_t)b * T_ + t) * 3 * H + 3 * h;
    if (mode == NSA_GATE_SOFTMAX) {
      const float dot = g0 * d0 + g1 * d1 + g2 * d2;
      dl[0] = g0 * (d0 - dot); dl[1] = g1 * (d1 - dot); dl[2] = g2 * (d2 - dot);
    } else {
      dl[0] = d0 * g0 * (1.f - g0); dl[1] = d1 * g1 * (1.f - g1); dl[2] = d2 * g2 * (1.f - g2);
    }
  }
}

}  // namespace nsa

using namespace nsa;

extern "C" NSA_API int nsa_gate_mix_fwd(const float* logits, const void* o_cmp, const void* o_slc, const void* o_win, void* out,
                                float* gates_out, int B, int H, int T, int dv, int gate_mode, int dtype, int out_token_major,
                                void* stream) {
  const int out_tm = out_token_major ? 1 : 0;
  NSA_REQUIRE(logits && o_cmp && o_slc && o_win && out && gates_out, "gate_mix_fwd: null pointer");
  NSA_REQUIRE(gate_mode == NSA_GATE_SIGMOID || gate_mode == NSA_GATE_SOFTMAX, "gate_mix_fwd: bad gate mode %d", gate_mode);
  const int64_t rows = (int64_t)B * H * T;
  if (rows == 0) return NSA_OK;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  cudaStream_t st = (cudaStream_t)stream;
  KernelTimer kt("gate_mix_fwd", st);
  if (dtype == NSA_F32)
    gate_mix_fwd_kernel<float><<<grid, 256, 0, st>>>(logits, (const float*)o_cmp, (const float*)o_slc, (const float*)o_win,
                                                      (float*)out, gates_out, B, H, T, dv, gate_mode, out_tm);
  else if (dtype == NSA_BF16 && dv % 128 == 0)
    gate_mix_fwd_bf16x4_kernel<<<(unsigned)((rows + 15) / 16), 256, 0, st>>>(logits, (const __nv_bfloat16*)o_cmp, (const __nv_bfloat16*)o_slc,
                                                     (const __nv_bfloat16*)o_win, (__nv_bfloat16*)out, gates_out, B, H, T, dv, gate_mode, out_tm);
  else if (dtype == NSA_BF16)
    gate_mix_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(logits, (const __nv_bfloat16*)o_cmp,
                                                              (const __nv_bfloat16*)o_slc, (const __nv_bfloat16*)o_win,
                                                              (__nv_bfloat16*)out, gates_out, B, H, T, dv, gate_mode, out_tm);
  else
    return fail(NSA_ERR_ARG, "gate_mix_fwd: unsupported dtype %d", dtype);
  return check_launch("gate_mix_fwd");
}

extern "C" NSA_API int nsa_gate_mix_bwd_delta(const float* gates, const void* o_cmp, const void* o_slc, const void* o_win,
                                      const void* dout, void* do_cmp, void* do_slc, void* do_win, float* dlogits,
                                      float* delta, int B, int H, int T, int dv, int gate_mode, int dtype, int dout_token_major,
                                      void* stream) {
  const int dout_tm = dout_token_major ? 1 : 0;
  NSA_REQUIRE(gates && o_cmp && o_slc && o_win && dout && do_cmp && do_slc && do_win && dlogits, "gate_mix_bwd: null pointer");
  const int64_t rows = (int64_t)B * H * T;
  if (rows == 0) return NSA_OK;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  cudaStream_t st = (cudaStream_t)stream;
  KernelTimer kt("gate_mix_bwd", st);
  if (dtype == NSA_F32)
    gate_mix_bwd_kernel<float><<<grid, 256, 0, st>>>(gates, (const float*)o_cmp, (const float*)o_slc, (const float*)o_win,
                                                      (const float*)dout, (float*)do_cmp, (float*)do_slc, (float*)do_win,
                                                      dlogits, B, H, T, dv, gate_mode, delta, dout_tm);
  else if (dtype == NSA_BF16 && dv % 128 == 0)
    gate_mix_bwd_bf16x4_kernel<<<(unsigned)((rows + 15) / 16), 256, 0, st>>>(gates, (const __nv_bfloat16*)o_cmp, (const __nv_bfloat16*)o_slc,
                                                     (const __nv_bfloat16*)o_win, (const __nv_bfloat16*)dout, (__nv_bfloat16*)do_cmp,
                                                     (__nv_bfloat16*)do_slc, (__nv_bfloat16*)do_win, dlogits, B, H, T, dv, gate_mode, delta, dout_tm);
  else if (dtype == NSA_BF16)
    gate_mix_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        gates, (const __nv_bfloat16*)o_cmp, (const __nv_bfloat16*)o_slc, (const __nv_bfloat16*)o_win,
        (const __nv_bfloat16*)dout, (__nv_bfloat16*)do_cmp, (__nv_bfloat16*)do_slc, (__nv_bfloat16*)do_win, dlogits, B, H,
        T, dv, gate_mode, delta, dout_tm);
  else
    return fail(NSA_ERR_ARG, "gate_mix_bwd: unsupported dtype %d", dtype);
  return check_launch("gate_mix_bwd");
}

extern "C" NSA_API int nsa_gate_mix_bwd(const float* gates, const void* o_cmp, const void* o_slc, const void* o_win,
                                const void* dout, void* do_cmp, void* do_slc, void* do_win, float* dlogits, int B, int H,
                                int T, int dv, int gate_mode, int dtype, int dout_token_major, void* stream) {
  return nsa_gate_mix_bwd_delta(gates, o_cmp, o_slc, o_win, dout, do_cmp, do_slc, do_win, dlogits, nullptr, B, H, T, dv,
                                gate_mode, dtype, dout_token_major, stream);
}
