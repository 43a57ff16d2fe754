// Pooling half of the block-compression MLP phi (NSAAttention.compress_tokens,
// nsa/kernels.py:2119-2208): with A[t] = W1[:, :dk] k_t precomputed by a GEMM and the per-offset
// table C[j] = W1[:, dk:] pos_embed[j] + b1, block i is hbar[i] = mean_j relu(A[i*d+j] + C[j]);
// values are mean-pooled.  All of it is HBM-bound streaming work: A is read l/d times (twice for
// l=32, d=16), served from L2 for the second read.
#include "common.cuh"

namespace nsa {

template <typename T>
__global__ void phi_pool_fwd_kernel(const float* __restrict__ a, const float* __restrict__ c, const T* __restrict__ v,
                                    int64_t svz, int64_t svg, int64_t svn, int64_t svk, float* __restrict__ hbar,
                                    T* __restrict__ v_cmp, int G, int T_, int U, int dv, int l, int d, int nb,
                                    int nbp) {
  const int i = blockIdx.x, bg = blockIdx.y, b = bg / G, g = bg % G;
  const float* ab = a + ((int64_t)bg * T_ + (int64_t)i * d) * U;
  const float inv = 1.f / (float)l;
  for (int u = threadIdx.x; u < U; u += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < l; ++j) acc += fmaxf(ab[(int64_t)j * U + u] + c[j * U + u], 0.f);
    hbar[((int64_t)bg * nb + i) * U + u] = acc * inv;
  }
  const T* vb = v + b * svz + g * svg + (int64_t)i * d * svn;
  for (int x = threadIdx.x; x < dv; x += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < l; ++j) acc += Elem<T>::ld(vb + (int64_t)j * svn + x * svk);
    Elem<T>::st(v_cmp + ((int64_t)bg * nbp + i) * dv + x, acc * inv);
  }
}

// da[t,u] = sum_{blocks i holding t} [A[t,u] + C[t-i*d,u] > 0] * dhbar[i,u] / l; dv likewise without a mask.
__global__ void phi_pool_bwd_tok_kernel(const float* __restrict__ a, const float* __restrict__ c,
                                        const float* __restrict__ dhbar, const float* __restrict__ dv_cmp,
                                        float* __restrict__ da, float* __restrict__ dv, int T_, int U, int dvd,
                                        int l, int d, int nb, int nbp) {
  const int t = blockIdx.x, bg = blockIdx.y;
  const int ilo = t - l + 1 <= 0 ? 0 : (t - l + d) / d;  // ceil((t-l+1)/d)
  const int ihi = min(nb - 1, t / d);
  const float inv = 1.f / (float)l;
  for (int u = threadIdx.x; u < U; u += blockDim.x) {
    const float av = a[((int64_t)bg * T_ + t) * U + u];
    float acc = 0.f;
    for (int i = ilo; i <= ihi; ++i)
      if (av + c[(t - i * d) * U + u] > 0.f) acc += dhbar[((int64_t)bg * nb + i) * U + u];
    da[((int64_t)bg * T_ + t) * U + u] = acc * inv;
  }
  for (int x = threadIdx.x; x < dvd; x += blockDim.x) {
    float acc = 0.f;
    for (int i = ilo; i <= ihi; ++i) acc += dv_cmp[((int64_t)bg * nbp + i) * dvd + x];
    dv[((int64_t)bg * T_ + t) * dvd + x] = acc * inv;
  }
}

// dc_part[bg,j,u] = sum_i [A[i*d+j,u] + C[j,u] > 0] * dhbar[i,u] / l.  The blocks are dealt round-robin to kTabGroups
// thread groups whose sums are added in group order, so the result does not depend on scheduling.
constexpr int kTabGroups = 8, kTabLanes = 128;
__global__ void __launch_bounds__(kTabGroups * kTabLanes)
phi_pool_bwd_tab_kernel(const float* __restrict__ a, const float* __restrict__ c, const float* __restrict__ dhbar,
                        float* __restrict__ dc_part, int T_, int U, int l, int d, int nb) {
  __shared__ float part[kTabGroups][kTabLanes];
  const int j = blockIdx.x, bg = blockIdx.y;
  const int ul = threadIdx.x % kTabLanes, grp = threadIdx.x / kTabLanes;
  const float inv = 1.f / (float)l;
  for (int u0 = 0; u0 < U; u0 += kTabLanes) {
    const int u = u0 + ul;
    float acc = 0.f;
    if (u < U) {
      const float cv = c[j * U + u];
#pragma unroll 4
      for (int i = grp; i < nb; i += kTabGroups)
        if (a[((int64_t)bg * T_ + (int64_t)i * d + j) * U + u] + cv > 0.f) acc += dhbar[((int64_t)bg * nb + i) * U + u];
    }
    part[grp][ul] = acc;
    __syncthreads();
    if (grp == 0 && u < U) {
      float tot = 0.f;
#pragma unroll
      for (int g2 = 0; g2 < kTabGroups; ++g2) tot += part[g2][ul];
      dc_part[((int64_t)bg * l + j) * U + u] = tot * inv;
    }
    __syncthreads();
  }
}

}  // namespace nsa

using namespace nsa;

extern "C" NSA_API int nsa_phi_pool_fwd(const float* a, const float* c, const void* v, const int64_t* vs, float* hbar,
                                void* v_cmp, int B, int G, int T, int U, int dv, int l, int d, int n_blocks, int nbp,
                                int dtype, void* stream) {
  NSA_REQUIRE(a && c && v && vs && hbar && v_cmp, "phi_pool_fwd: null pointer");
  NSA_REQUIRE(l > 0 && d > 0 && n_blocks >= 0 && nbp >= n_blocks && (int64_t)(n_blocks - 1) * d + l <= T,
              "phi_pool_fwd: blocks (n=%d,l=%d,d=%d) exceed T=%d", n_blocks, l, d, T);
  if (n_blocks == 0 || B * G == 0) return NSA_OK;
  dim3 grid(n_blocks, B * G);
  cudaStream_t st = (cudaStream_t)stream;
  KernelTimer kt("phi_pool_fwd", st);
  if (dtype == NSA_F32)
    phi_pool_fwd_kernel<float><<<grid, 128, 0, st>>>(a, c, (const float*)v, vs[0], vs[1], vs[2], vs[3], hbar,
                                                      (float*)v_cmp, G, T, U, dv, l, d, n_blocks, nbp);
  else if (dtype == NSA_BF16)
    phi_pool_fwd_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(a, c, (const __nv_bfloat16*)v, vs[0], vs[1], vs[2],
                                                              vs[3], hbar, (__nv_bfloat16*)v_cmp, G, T, U, dv, l, d,
                                                              n_blocks, nbp);
  else
    return fail(NSA_ERR_ARG, "phi_pool_fwd: unsupported dtype %d", dtype);
  return check_launch("phi_pool_fwd");
}

extern "C" NSA_API int nsa_phi_pool_bwd(const float* a, const float* c, const float* dhbar, const float* dv_cmp, float* da,
                                float* dc_part, float* dv, int B, int G, int T, int U, int dv_dim, int l, int d,
                                int n_blocks, int nbp, void* stream) {
  NSA_REQUIRE(a && c && dhbar && dv_cmp && da && dc_part && dv, "phi_pool_bwd: null pointer");
  NSA_REQUIRE(l > 0 && d > 0 && n_blocks >= 0 && (int64_t)(n_blocks - 1) * d + l <= T, "phi_pool_bwd: bad blocks");
  if (B * G == 0 || T == 0) return NSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  KernelTimer kt("phi_pool_bwd", st);
  phi_pool_bwd_tok_kernel<<<dim3(T, B * G), 128, 0, st>>>(a, c, dhbar, dv_cmp, da, dv, T, U, dv_dim, l, d, n_blocks,
                                                          nbp);
  if (int rc = check_launch("phi_pool_bwd_tok")) return rc;
  phi_pool_bwd_tab_kernel<<<dim3(l, B * G), kTabGroups * kTabLanes, 0, st>>>(a, c, dhbar, dc_part, T, U, l, d, n_blocks);
  return check_launch("phi_pool_bwd_tab");
}
