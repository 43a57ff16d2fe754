// Selection scoring: Eq. 8 (compressed-attention probabilities) -> Eq. 9 (stencil onto selection
// blocks) -> Eq. 10 (sum over the heads of a GQA group) -> Eq. 11 (top-n with forced blocks).
//
// Semantics pinned to the reference's torch code: p_cmp (nsa/kernels.py:2316-2343, rows that see no
// compressed block use block 0 alone), derive_selection_from_compression_per_timestep
// (nsa/kernels.py:1943-1960: adds in (m outer, n inner) order from zero, n_sel from the padded block
// count), select_top_k_blocks_per_query_with_gqa (nsa/kernels.py:1986-2040: heads summed in order,
// stable descending sort so ties go to the lower block id, fixed blocks first, repeats dropped,
// -1 padding).  Nothing of size [B,H,T,n_cmp] ever reaches HBM: one CTA owns one (b,g,t).
#include <algorithm>
#include "common.cuh"
#include "fa_sm100.cuh"

namespace nsa {

constexpr int kThreads = 256;
constexpr int kMaxN = 64;

__device__ __forceinline__ float block_max(float x, float* red) {
  x = warp_max(x);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = x;
  __syncthreads();
  float r = red[0];
  for (int w = 1; w < kThreads / 32; ++w) r = fmaxf(r, red[w]);
  return r;
}
__device__ __forceinline__ float block_sum(float x, float* red) {
  x = warp_sum(x);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = x;
  __syncthreads();
  float r = red[0];
  for (int w = 1; w < kThreads / 32; ++w) r += red[w];
  return r;
}

// Stable top-k of agg[0..n_sel) (value descending, index ascending), fixed-block merge, -1 padding.
// Destroys agg.  All threads of the CTA must call it.
__device__ void topn_and_merge(float* agg, int n_sel, int t, int l_prime, int n, int n_fixed, int* top,
                               float* redv, int* redi, int32_t* out) {
  const int k_actual = min(n, n_sel);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = 0; r < k_actual; ++r) {
    float bv = -CUDART_INF_F;
    int bi = 0x7fffffff;
    for (int j = threadIdx.x; j < n_sel; j += kThreads) {
      const float v = agg[j];
      if (v > bv || (v == bv && j < bi)) { bv = v; bi = j; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { redv[warp] = bv; redi[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < kThreads / 32; ++w)
        if (redv[w] > bv || (redv[w] == bv && redi[w] < bi)) { bv = redv[w]; bi = redi[w]; }
      top[r] = bi;
      if (bi < n_sel) agg[bi] = -CUDART_INF_F;  // taken; scores are >= 0
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    int cnt = 0;
    int res[kMaxN];
    auto push = [&](int id) {
      if (cnt >= n) return;
      for (int i = 0; i < cnt; ++i)
        if (res[i] == id) return;
      res[cnt++] = id;
    };
    if (n_fixed > 0) {
      push(0);
      push(t < l_prime ? 0 : (t - l_prime) / l_prime);
      push(t / l_prime);
    }
    for (int r = 0; r < k_actual; ++r) push(top[r]);
    for (int i = 0; i < n; ++i) out[i] = i < cnt ? res[i] : -1;
  }
}

// A handful of query rows (decode): the q.k products of every head against every visible compressed block, one thread
// per block and all heads of the group in registers, so that the keys are read once per row and the work spreads over
// (blocks / 128) x (group, row) CTAs instead of one CTA per row.  Same fmaf chain over the head dimension as the row
// kernel's own loop.
template <typename T, int HPG>
__global__ void __launch_bounds__(128)
score_logits_kernel(const T* __restrict__ q, int64_t sqz, int64_t sqh, int64_t sqm, int64_t sqk, const float* __restrict__ kc,
                    const int* __restrict__ block_ends, float* __restrict__ logits, int H, int G, int T_, int dk, int nbp,
                    int q0) {
  extern __shared__ float qsm[];        // [HPG][dk]
  const int tq = blockIdx.z, bg = blockIdx.y, b = bg / G, g = bg % G;
  const int t = q0 + tq;
  for (int i = threadIdx.x; i < HPG * dk; i += 128) {
    const int hh = i / dk, d = i % dk;
    qsm[i] = Elem<T>::ld(q + b * sqz + (int64_t)(g * HPG + hh) * sqh + (int64_t)tq * sqm + d * sqk);
  }
  __syncthreads();
  const int i = blockIdx.x * 128 + threadIdx.x;
  if (i >= nbp || block_ends[i] > t) return;   // hidden blocks are never read back
  const float* kb = kc + (int64_t)bg * dk * nbp + i;
  float acc[HPG];
#pragma unroll
  for (int u = 0; u < HPG; ++u) acc[u] = 0.f;
#pragma unroll 8
  for (int d = 0; d < dk; ++d) {
    const float kv = __ldg(kb + (int64_t)d * nbp);
#pragma unroll
    for (int u = 0; u < HPG; ++u) acc[u] = fmaf(qsm[u * dk + d], kv, acc[u]);
  }
  float* dst = logits + (((int64_t)bg * T_ + tq) * HPG) * nbp + i;
#pragma unroll
  for (int u = 0; u < HPG; ++u) dst[(int64_t)u * nbp] = acc[u];
}

// HB heads share one sweep over the compressed keys (each key element is loaded once per HB heads); the softmax
// and the Eq. 9 sums then run head by head in head order, so the result does not depend on HB.
template <typename T, int HB>
__global__ void __launch_bounds__(kThreads)
score_topn_kernel(const T* __restrict__ q, int64_t sqz, int64_t sqh, int64_t sqm, int64_t sqk,
                  const float* __restrict__ kc, const int* __restrict__ block_ends, int32_t* __restrict__ out, int H,
                  int G, int T_, int dk, int nbp, int a_, int s_, int n_sel, int l_prime, int n, int n_fixed,
                  float scale, int q0, const float* __restrict__ logits) {
  extern __shared__ float sm[];
  const int tq = blockIdx.x, bg = blockIdx.y, b = bg / G, g = bg % G, hpg = H / G;
  const int t = q0 + tq;                // position of query row tq
  const int pstride = nbp + a_ + s_;
  float* qs = sm;                       // [hpg][dk]
  float* p = qs + hpg * dk;             // [HB][nbp + a_ + s_]
  float* agg = p + HB * pstride;        // [n_sel]
  float* redv = agg + n_sel;            // [8]
  int* redi = (int*)(redv + 8);         // [8]
  int* top = redi + 8;                  // [kMaxN]
  for (int i = threadIdx.x; i < hpg * dk; i += kThreads) {
    const int hh = i / dk, d = i % dk;
    qs[i] = Elem<T>::ld(q + b * sqz + (int64_t)(g * hpg + hh) * sqh + (int64_t)tq * sqm + d * sqk);
  }
  for (int j = threadIdx.x; j < n_sel; j += kThreads) agg[j] = 0.f;
  for (int u = 0; u < HB; ++u)
    for (int i = nbp + threadIdx.x; i < pstride; i += kThreads) p[u * pstride + i] = 0.f;
  __syncthreads();
  const float* kb = kc + (int64_t)bg * dk * nbp;
  for (int h0 = 0; h0 < hpg; h0 += HB) {
    // logits given: q.k products [hpg][nbp] of this (group, row) from score_logits_kernel (same sums, same order)
    const float* lrow = logits ? logits + (((int64_t)bg * T_ + tq) * hpg + h0) * nbp : nullptr;
    for (int i = threadIdx.x; i < nbp; i += kThreads) {
      float acc[HB];
#pragma unroll
      for (int u = 0; u < HB; ++u) acc[u] = 0.f;
      const bool vis = block_ends[i] <= t;
      if (vis && lrow) {
#pragma unroll
        for (int u = 0; u < HB; ++u) acc[u] = lrow[(int64_t)u * nbp + i];
      } else if (vis) {
#pragma unroll 8
        for (int d = 0; d < dk; ++d) {
          const float kv = __ldg(kb + (int64_t)d * nbp + i);
#pragma unroll
          for (int u = 0; u < HB; ++u) acc[u] = fmaf(qs[(h0 + u) * dk + d], kv, acc[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < HB; ++u) p[u * pstride + i] = vis ? acc[u] * scale : -CUDART_INF_F;
    }
    __syncthreads();
    for (int u = 0; u < HB; ++u) {
      float* ph = p + u * pstride;
      float mx = -CUDART_INF_F;
      for (int i = threadIdx.x; i < nbp; i += kThreads) mx = fmaxf(mx, ph[i]);
      mx = block_max(mx, redv);
      if (mx == -CUDART_INF_F) {  // nothing visible: block 0 alone
        for (int i = threadIdx.x; i < nbp; i += kThreads) ph[i] = i == 0 ? 1.f : 0.f;
      } else {
        float sum = 0.f;
        for (int i = threadIdx.x; i < nbp; i += kThreads) {
          const float e = expf(ph[i] - mx);  // exp(-inf) = 0 for hidden blocks
          ph[i] = e;
          sum += e;
        }
        sum = block_sum(sum, redv);
        const float inv = 1.f / sum;
        for (int i = threadIdx.x; i < nbp; i += kThreads) ph[i] *= inv;
      }
      __syncthreads();
      for (int j = threadIdx.x; j < n_sel; j += kThreads) {
        float sel = 0.f;
        for (int m = 0; m < s_; ++m)
          for (int nn = 0; nn < a_; ++nn) sel += ph[s_ * j + m + nn];  // zero padding stands for skipped terms
        agg[j] += sel;
      }
      __syncthreads();
    }
  }
  topn_and_merge(agg, n_sel, t, l_prime, n, n_fixed, top, redv, redi,
                 out + ((int64_t)bg * T_ + tq) * n);
}

__global__ void __launch_bounds__(kThreads)
topn_from_scores_kernel(const float* __restrict__ scores, int32_t* __restrict__ out, int H, int G, int T_, int n_sel,
                        int l_prime, int n, int n_fixed) {
  extern __shared__ float sm[];
  const int t = blockIdx.x, bg = blockIdx.y, b = bg / G, g = bg % G, hpg = H / G;
  float* agg = sm;
  float* redv = agg + n_sel;
  int* redi = (int*)(redv + 8);
  int* top = redi + 8;
  for (int j = threadIdx.x; j < n_sel; j += kThreads) {
    float acc = 0.f;
    for (int hh = 0; hh < hpg; ++hh)
      acc += scores[(((int64_t)b * H + g * hpg + hh) * T_ + t) * n_sel + j];
    agg[j] = acc;
  }
  __syncthreads();
  topn_and_merge(agg, n_sel, t, l_prime, n, n_fixed, top, redv, redi, out + ((int64_t)bg * T_ + t) * n);
}

}  // namespace nsa

using namespace nsa;

static bool score_tc_ok(const void* q, const int64_t* qs, int B, int H, int G, int T, int dk, int nbp, int l, int d, int l_prime,
                        int n, int n_real_blocks, int dtype, int flags) {
  if ((flags & NSA_FLAG_GENERIC) || dtype != NSA_BF16 || n_real_blocks < 0 || n_real_blocks > nbp) return false;
  if (!score_sm100_supported(H, G, T, dk, nbp, l, d, l_prime, n) || (int64_t)B * G > 65535) return false;
  const int64_t cq[4] = {(int64_t)H * T * dk, (int64_t)T * dk, dk, 1};
  for (int i = 0; i < 4; ++i)
    if (qs[i] != cq[i]) return false;
  return (reinterpret_cast<uintptr_t>(q) & 15) == 0;
}

// few query rows (decode): q.k products staged in the workspace by score_logits_kernel
static constexpr int kFewRows = 64;
static size_t few_rows_logit_bytes(int B, int H, int G, int T, int nbp) {
  if (B <= 0 || G <= 0 || T <= 0 || H % G != 0 || (int64_t)B * G * T > kFewRows) return 0;
  const int hpg = H / G;
  if (hpg != 1 && hpg != 2 && hpg != 4 && hpg != 8 && hpg != 16) return 0;
  return (size_t)B * G * T * hpg * nbp * sizeof(float);
}

extern "C" NSA_API size_t nsa_score_topn_workspace_bytes(int B, int H, int G, int T, int dk, int nbp, int l, int d, int l_prime,
                                                         int n, int dtype, int flags) {
  if (B <= 0 || G <= 0 || dtype != NSA_BF16 || (flags & NSA_FLAG_GENERIC) || !score_sm100_supported(H, G, T, dk, nbp, l, d, l_prime, n))
    return std::max<size_t>(256, few_rows_logit_bytes(B, H, G, T, nbp));
  return score_sm100_workspace_bytes(B, G, T, dk, nbp, d, l_prime);
}

extern "C" NSA_API int nsa_score_topn(const void* q, const int64_t* qs, const float* k_cmp, const int32_t* block_ends,
                              int32_t* indices_out, int B, int H, int G, int T, int dk, int nbp, int l, int d,
                              int l_prime, int n, int n_fixed, float scale, int dtype, int n_real_blocks, int q_pos0, int flags,
                              const float* cmp_lse2, void* workspace, size_t workspace_bytes, void* stream) {
  NSA_REQUIRE(q && qs && k_cmp && block_ends && indices_out, "score_topn: null pointer");
  NSA_REQUIRE(q_pos0 >= 0, "score_topn: negative query offset");
  if (timeout_flagged())
    return fail(NSA_ERR_LAUNCH, "score_topn: a tensor-core kernel gave up on a barrier wait earlier (device time-out); results "
                "since then are invalid.  nsa_device_timeouts(1) reports and clears the condition");
  if (B > 0 && T > 0 && score_tc_ok(q, qs, B, H, G, T, dk, nbp, l, d, l_prime, n, n_real_blocks, dtype, flags))
    return score_topn_sm100(q, k_cmp, indices_out, B, H, G, T, dk, nbp, l, d, l_prime, n_real_blocks, n, n_fixed, scale,
                            q_pos0, cmp_lse2, workspace, workspace_bytes, (cudaStream_t)stream);
  NSA_REQUIRE(G > 0 && H % G == 0 && d > 0 && l % d == 0 && l_prime % d == 0 && l > 0 && l_prime > 0,
              "score_topn: bad block parameters");
  NSA_REQUIRE(n > 0 && n <= kMaxN, "score_topn: n=%d outside 1..%d", n, kMaxN);
  NSA_REQUIRE(nbp > 0, "score_topn: no compressed blocks");
  if (B * G == 0 || T == 0) return NSA_OK;
  const int a_ = l / d, s_ = l_prime / d, n_sel = (nbp + s_ - 1) / s_, hpg = H / G;
  auto smem_for = [&](int hb) { return ((size_t)hpg * dk + (size_t)hb * (nbp + a_ + s_) + n_sel + 16 + kMaxN) * sizeof(float); };
  const int hb = (hpg % 4 == 0 && smem_for(4) <= 160 * 1024) ? 4 : (hpg % 2 == 0 && smem_for(2) <= 160 * 1024) ? 2 : 1;
  const size_t sm = smem_for(hb);
  if (sm > 200 * 1024) return fail(NSA_ERR_UNSUPPORTED, "score_topn: %zu bytes of shared memory needed", sm);
  if (dtype != NSA_F32 && dtype != NSA_BF16) return fail(NSA_ERR_ARG, "score_topn: unsupported dtype %d", dtype);
  cudaStream_t st = (cudaStream_t)stream;
  const int q0 = q_pos0;
  const float* logits = nullptr;
  const size_t lbytes = few_rows_logit_bytes(B, H, G, T, nbp);
  if (lbytes > 0 && workspace && workspace_bytes >= lbytes && (size_t)hpg * dk * sizeof(float) <= 48 * 1024) {
    KernelTimer ktl("score_logits", st);
    const dim3 lgrid((nbp + 127) / 128, B * G, T);
    const size_t lsm = (size_t)hpg * dk * sizeof(float);
    float* lw = (float*)workspace;
#define NSA_LOGITS(TYPE, HPG_)                                                                                       \
  score_logits_kernel<TYPE, HPG_><<<lgrid, 128, lsm, st>>>((const TYPE*)q, qs[0], qs[1], qs[2], qs[3], k_cmp, block_ends, \
                                                           lw, H, G, T, dk, nbp, q0)
#define NSA_LOGITS_T(TYPE)                                                                        \
  switch (hpg) {                                                                                  \
    case 1: NSA_LOGITS(TYPE, 1); break;                                                           \
    case 2: NSA_LOGITS(TYPE, 2); break;                                                           \
    case 4: NSA_LOGITS(TYPE, 4); break;                                                           \
    case 8: NSA_LOGITS(TYPE, 8); break;                                                           \
    default: NSA_LOGITS(TYPE, 16); break;                                                         \
  }
    if (dtype == NSA_F32) { NSA_LOGITS_T(float) } else { NSA_LOGITS_T(__nv_bfloat16) }
#undef NSA_LOGITS_T
#undef NSA_LOGITS
    if (int rc = check_launch("score_logits")) return rc;
    logits = lw;
  }
  KernelTimer kt("score_topn", st);
  dim3 grid(T, B * G);
#define NSA_SCORE_LAUNCH(TYPE, HB_)                                                                                    \
  do {                                                                                                                 \
    cudaFuncSetAttribute(score_topn_kernel<TYPE, HB_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);          \
    score_topn_kernel<TYPE, HB_><<<grid, kThreads, sm, st>>>((const TYPE*)q, qs[0], qs[1], qs[2], qs[3], k_cmp,        \
                                                             block_ends, indices_out, H, G, T, dk, nbp, a_, s_, n_sel, \
                                                             l_prime, n, n_fixed, scale, q0, logits);                  \
  } while (0)
  if (dtype == NSA_F32) {
    if (hb == 4) NSA_SCORE_LAUNCH(float, 4); else if (hb == 2) NSA_SCORE_LAUNCH(float, 2); else NSA_SCORE_LAUNCH(float, 1);
  } else {
    if (hb == 4) NSA_SCORE_LAUNCH(__nv_bfloat16, 4); else if (hb == 2) NSA_SCORE_LAUNCH(__nv_bfloat16, 2); else NSA_SCORE_LAUNCH(__nv_bfloat16, 1);
  }
#undef NSA_SCORE_LAUNCH
  return check_launch("score_topn");
}

extern "C" NSA_API int nsa_topn_from_scores(const float* scores, int32_t* indices_out, int B, int H, int G, int T, int n_sel,
                                    int l_prime, int n, int n_fixed, void* stream) {
  NSA_REQUIRE(scores && indices_out, "topn_from_scores: null pointer");
  NSA_REQUIRE(G > 0 && H % G == 0 && l_prime > 0 && n > 0 && n <= kMaxN && n_sel > 0, "topn_from_scores: bad sizes");
  if (B * G == 0 || T == 0) return NSA_OK;
  const size_t sm = ((size_t)n_sel + 16 + kMaxN) * sizeof(float);
  if (sm > 200 * 1024) return fail(NSA_ERR_UNSUPPORTED, "topn_from_scores: n_sel too large");
  cudaFuncSetAttribute(topn_from_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  topn_from_scores_kernel<<<dim3(T, B * G), kThreads, sm, (cudaStream_t)stream>>>(scores, indices_out, H, G, T, n_sel,
                                                                                 l_prime, n, n_fixed);
  return check_launch("topn_from_scores");
}

// ------------------------------------------------------------------------------------------------
// diagnostics: materialised Eq. 8 probabilities and Eq. 9 scores (the layer never needs them in HBM;
// they back the module's output_attentions=True report, nsa/kernels.py:2481-2488)
// ------------------------------------------------------------------------------------------------
namespace nsa {

template <typename T>
__global__ void __launch_bounds__(kThreads)
cmp_probs_kernel(const T* __restrict__ q, int64_t sqz, int64_t sqh, int64_t sqm, int64_t sqk,
                 const float* __restrict__ kc, const int* __restrict__ block_ends, float* __restrict__ out, int H, int G,
                 int T_, int dk, int nbp, float scale) {
  extern __shared__ float sm[];
  const int t = blockIdx.x, bh = blockIdx.y, b = bh / H, h = bh % H, g = h / (H / G);
  float* qs = sm;
  float* red = qs + dk;
  for (int d = threadIdx.x; d < dk; d += kThreads) qs[d] = Elem<T>::ld(q + b * sqz + h * sqh + (int64_t)t * sqm + d * sqk);
  __syncthreads();
  const float* kb = kc + (int64_t)(b * G + g) * dk * nbp;
  float* orow = out + ((int64_t)bh * T_ + t) * nbp;
  float mx = -CUDART_INF_F;
  for (int i = threadIdx.x; i < nbp; i += kThreads) {
    float s = -CUDART_INF_F;
    if (block_ends[i] <= t) {
      float acc = 0.f;
      for (int d = 0; d < dk; ++d) acc = fmaf(qs[d], kb[(int64_t)d * nbp + i], acc);
      s = acc * scale;
    }
    orow[i] = s;
    mx = fmaxf(mx, s);
  }
  mx = block_max(mx, red);
  if (mx == -CUDART_INF_F) {
    for (int i = threadIdx.x; i < nbp; i += kThreads) orow[i] = i == 0 ? 1.f : 0.f;
    return;
  }
  float sum = 0.f;
  for (int i = threadIdx.x; i < nbp; i += kThreads) {
    const float e = expf(orow[i] - mx);
    orow[i] = e;
    sum += e;
  }
  sum = block_sum(sum, red);
  const float inv = 1.f / sum;
  for (int i = threadIdx.x; i < nbp; i += kThreads) orow[i] *= inv;
}

__global__ void eq9_kernel(const float* __restrict__ p, float* __restrict__ out, int64_t rows, int n_cmp, int n_sel,
                           int a_, int s_) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * n_sel) return;
  const int64_t r = i / n_sel;
  const int j = i % n_sel;
  const float* pr = p + r * n_cmp;
  float sel = 0.f;
  for (int m = 0; m < s_; ++m)
    for (int nn = 0; nn < a_; ++nn) {
      const int idx = s_ * j + m + nn;
      if (idx < n_cmp) sel += pr[idx];
    }
  out[i] = sel;
}

}  // namespace nsa

extern "C" NSA_API int nsa_cmp_probs(const void* q, const int64_t* qs, const float* k_cmp, const int32_t* block_ends,
                                     float* out, int B, int H, int G, int T, int dk, int nbp, float scale, int dtype,
                                     void* stream) {
  NSA_REQUIRE(q && qs && k_cmp && block_ends && out, "cmp_probs: null pointer");
  NSA_REQUIRE(G > 0 && H % G == 0 && nbp > 0 && dk > 0 && (int64_t)B * H <= 65535, "cmp_probs: bad sizes");
  if (B == 0 || T == 0) return NSA_OK;
  const size_t sm = ((size_t)dk + 8) * sizeof(float);
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(T, B * H);
  if (dtype == NSA_F32)
    cmp_probs_kernel<float><<<grid, kThreads, sm, st>>>((const float*)q, qs[0], qs[1], qs[2], qs[3], k_cmp, block_ends, out,
                                                         H, G, T, dk, nbp, scale);
  else if (dtype == NSA_BF16)
    cmp_probs_kernel<__nv_bfloat16><<<grid, kThreads, sm, st>>>((const __nv_bfloat16*)q, qs[0], qs[1], qs[2], qs[3], k_cmp,
                                                                 block_ends, out, H, G, T, dk, nbp, scale);
  else
    return fail(NSA_ERR_ARG, "cmp_probs: unsupported dtype %d", dtype);
  return check_launch("cmp_probs");
}

extern "C" NSA_API int nsa_eq9_scores(const float* p_cmp, float* out, int64_t rows, int n_cmp, int l, int d, int l_prime,
                                      void* stream) {
  NSA_REQUIRE(p_cmp && out, "eq9_scores: null pointer");
  NSA_REQUIRE(d > 0 && l > 0 && l_prime > 0 && l % d == 0 && l_prime % d == 0 && n_cmp > 0, "eq9_scores: bad block parameters");
  const int a_ = l / d, s_ = l_prime / d, n_sel = (n_cmp + s_ - 1) / s_;
  const int64_t total = rows * n_sel;
  if (total == 0) return NSA_OK;
  eq9_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(p_cmp, out, rows, n_cmp, n_sel, a_, s_);
  return check_launch("eq9_scores");
}
