// Block-compression MLP phi (NSAAttention.compress_tokens, nsa/kernels.py:2096-2102, 2119-2208), forward and backward,
// behind the C ABI.
//
// k_cmp[i] = mean_{j<l} ( W2 relu(W1 [k_{id+j} || pos_j] + b1) + b2 ) and v_cmp[i] = mean_j v_{id+j}.  Two identities keep
// the work small: W1 [k || pos_j] = W1k k + (W1p pos_j + b1), a per-offset table C[j] added after one dense product
// A = K^T W1k^T over ALL tokens (instead of one product per (block, offset)), and mean(W2 h + b2) = W2 mean(h) + b2, so the
// second linear layer runs once per block.  The dense products are library GEMMs (cuBLAS, looked up at run time); what
// sits between them is the fused pooling kernel of phi_pool.cu and a few small elementwise kernels here.
//
// Exactness of A: A decides the compressed keys, which decide the top-n selection, so it is computed like the reference's
// fp32 linear layer.  For bf16 keys the fp32 weight is split into three bf16 terms (8 + 8 + 8 mantissa bits: hi + mid +
// lo reproduces the fp32 value exactly), and A = K hi^T + K mid^T + K lo^T on the tensor cores with fp32 accumulation
// holds the same products as the fp32 GEMM.  For fp32 keys the GEMM is a plain fp32 one (no TF32).
//
// The backward forms its key-gradient products from the activation gradient rounded to the I/O type when that is
// bf16 (the result leaves in bf16 anyway); weight gradients are fp32.
#include <cublas_v2.h>
#include <dlfcn.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace nsa {
namespace {

// ---------------------------------------------------------------------------------------------- cuBLAS at run time
struct Blas {
  void* lib = nullptr;
  cublasStatus_t (*create)(cublasHandle_t*) = nullptr;
  cublasStatus_t (*set_stream)(cublasHandle_t, cudaStream_t) = nullptr;
  cublasStatus_t (*gemm_sb)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*, const void*,
                            cudaDataType, int, long long, const void*, cudaDataType, int, long long, const void*, void*,
                            cudaDataType, int, long long, int, cublasComputeType_t, cublasGemmAlgo_t) = nullptr;
  cublasHandle_t handle[64] = {};
  std::mutex mu;
};
Blas g_blas;

int blas_handle(cublasHandle_t* out, cudaStream_t st) {
  std::lock_guard<std::mutex> lk(g_blas.mu);
  if (!g_blas.lib) {
    const char* names[] = {"libcublas.so.12", "libcublas.so.13", "libcublas.so"};
    for (const char* n : names) {
      g_blas.lib = dlopen(n, RTLD_NOW | RTLD_LOCAL);
      if (g_blas.lib) break;
    }
    if (!g_blas.lib) return fail(NSA_ERR_UNSUPPORTED, "the GEMMs of this entry point need cuBLAS (libcublas.so.12 not found: %s)", dlerror());
    g_blas.create = (decltype(g_blas.create))dlsym(g_blas.lib, "cublasCreate_v2");
    g_blas.set_stream = (decltype(g_blas.set_stream))dlsym(g_blas.lib, "cublasSetStream_v2");
    g_blas.gemm_sb = (decltype(g_blas.gemm_sb))dlsym(g_blas.lib, "cublasGemmStridedBatchedEx");
    if (!g_blas.create || !g_blas.set_stream || !g_blas.gemm_sb) {
      g_blas.lib = nullptr;
      return fail(NSA_ERR_UNSUPPORTED, "cuBLAS lacks an expected symbol");
    }
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(NSA_ERR_LAUNCH, "cannot identify the current device");
  if (!g_blas.handle[dev] && g_blas.create(&g_blas.handle[dev]) != CUBLAS_STATUS_SUCCESS)
    return fail(NSA_ERR_LAUNCH, "cublasCreate failed");
  if (g_blas.set_stream(g_blas.handle[dev], st) != CUBLAS_STATUS_SUCCESS) return fail(NSA_ERR_LAUNCH, "cublasSetStream failed");
  *out = g_blas.handle[dev];
  return NSA_OK;
}

// Column-major GEMM C(m x n) = alpha op(A) op(B) + beta C, batched with element strides; fp32 accumulation.
int gemm(cublasHandle_t h, cublasOperation_t ta, cublasOperation_t tb, int m, int n, int k, const void* A, cudaDataType at, int lda,
         long long sa, const void* Bm, cudaDataType bt, int ldb, long long sb, float beta, void* C, cudaDataType ct, int ldc,
         long long sc, int batch, const char* what) {
  if (m == 0 || n == 0 || batch == 0) return NSA_OK;
  const float alpha = 1.f;
  const cublasStatus_t s = g_blas.gemm_sb(h, ta, tb, m, n, k, &alpha, A, at, lda, sa, Bm, bt, ldb, sb, &beta, C, ct, ldc, sc, batch,
                                          CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
  if (s != CUBLAS_STATUS_SUCCESS) return fail(NSA_ERR_LAUNCH, "%s: cuBLAS GEMM failed with status %d", what, (int)s);
  return NSA_OK;
}

size_t al256(size_t x) { return (x + 255) & ~size_t(255); }

// ---------------------------------------------------------------------------------------------- small kernels
// w1 [U, dk+l] fp32 -> three bf16 terms of its first dk columns, each [U, dk]
__global__ void split3_kernel(const float* __restrict__ w1, int U, int dk, int ld, __nv_bfloat16* __restrict__ hi,
                              __nv_bfloat16* __restrict__ mid, __nv_bfloat16* __restrict__ lo) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= U * dk) return;
  const float w = w1[(int64_t)(i / dk) * ld + i % dk];
  const __nv_bfloat16 h = __float2bfloat16_rn(w);
  const float r1 = w - __bfloat162float(h);
  const __nv_bfloat16 m = __float2bfloat16_rn(r1);
  hi[i] = h;
  mid[i] = m;
  lo[i] = __float2bfloat16_rn(r1 - __bfloat162float(m));
}
// first dk columns of w1 in the I/O type, [U, dk]
template <typename T>
__global__ void w1k_cast_kernel(const float* __restrict__ w1, int U, int dk, int ld, T* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < U * dk) Elem<T>::st(out + i, w1[(int64_t)(i / dk) * ld + i % dk]);
}
// C[j,u] = b1[u] + sum_m pos[j,m] w1[u, dk+m]
__global__ void c_table_kernel(const float* __restrict__ pos, const float* __restrict__ w1, const float* __restrict__ b1, int l, int U,
                               int dk, float* __restrict__ c) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= l * U) return;
  const int j = i / U, u = i % U;
  float acc = b1 ? b1[u] : 0.f;
  for (int m = 0; m < l; ++m) acc = fmaf(pos[j * l + m], w1[(int64_t)u * (dk + l) + dk + m], acc);
  c[i] = acc;
}
// k_cmp[bg, c, i] += b2[c] for the real blocks; an optional copy in the I/O type is written alongside
template <typename T>
__global__ void kcmp_finish_kernel(float* __restrict__ k_cmp, const float* __restrict__ b2, T* __restrict__ lp, int dk, int nb, int nbp,
                                   int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int blk = i % nbp, c = (i / nbp) % dk;
  float x = k_cmp[i];
  if (blk < nb && b2) x += b2[c];
  if (blk >= nb) x = 0.f;
  k_cmp[i] = x;
  if (lp) Elem<T>::st(lp + i, x);
}
// rows [bg, i < nb] of a [BG, nbp, W] tensor of the I/O type -> fp32 [BG, nb_out, W] (rows beyond nb zero)
template <typename T>
__global__ void rows_to_f32_kernel(const T* __restrict__ in, float* __restrict__ out, int nbp, int nb, int nb_out, int W, int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = i % W, r = (i / W) % nb_out;
  const int64_t bg = i / ((int64_t)W * nb_out);
  out[i] = r < nb ? Elem<T>::ld(in + (bg * nbp + r) * W + c) : 0.f;
}
// Column sums out[c] = sum over rows of in[row, c] in a fixed order: 1024-row chunks are summed by 8 row lanes per column
// (stage 1, partial sums to scratch), the chunks then one after the other (stage 2).
constexpr int kColsumChunk = 1024;
template <typename T>
__global__ void colsum_stage1_kernel(const T* __restrict__ in, int64_t rows, int W, float* __restrict__ part) {
  __shared__ float sh[8][32];
  const int c = blockIdx.x * 32 + (threadIdx.x & 31), rl = threadIdx.x >> 5;
  const int64_t r0 = (int64_t)blockIdx.y * kColsumChunk, r1 = min(rows, r0 + kColsumChunk);
  float acc = 0.f;
  if (c < W)
    for (int64_t r = r0 + rl; r < r1; r += 8) acc += Elem<T>::ld(in + r * W + c);
  sh[rl][threadIdx.x & 31] = acc;
  __syncthreads();
  if (rl == 0 && c < W) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sh[i][threadIdx.x & 31];
    part[(int64_t)blockIdx.y * W + c] = t;
  }
}
__global__ void colsum_stage2_kernel(const float* __restrict__ part, int chunks, int W, float* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= W) return;
  float acc = 0.f;
  for (int i = 0; i < chunks; ++i) acc += part[(int64_t)i * W + c];
  out[c] = acc;
}
template <typename T>
__global__ void cast_kernel(const float* __restrict__ in, T* __restrict__ out, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) Elem<T>::st(out + i, in[i]);
}
template <typename T>
__global__ void add_into_kernel(T* __restrict__ dst, const float* __restrict__ src, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) Elem<T>::st(dst + i, Elem<T>::ld(dst + i) + src[i]);
}
// dc[j,u] = sum_bg dc_part[bg,j,u]; then db1[u] = sum_j dc, dw1[u, dk+m] = sum_j dc[j,u] pos[j,m], dpos[j,m] = sum_u dc[j,u] w1[u,dk+m]
__global__ void dc_sum_kernel(const float* __restrict__ part, int BG, int n, float* __restrict__ dc) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = 0.f;
  for (int b = 0; b < BG; ++b) acc += part[(int64_t)b * n + i];
  dc[i] = acc;
}
__global__ void table_grads_kernel(const float* __restrict__ dc, const float* __restrict__ pos, const float* __restrict__ w1, int l, int U,
                                   int dk, float* __restrict__ db1, float* __restrict__ dw1, float* __restrict__ dpos) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int ld = dk + l;
  if (i < U) {
    float acc = 0.f;
    for (int j = 0; j < l; ++j) acc += dc[j * U + i];
    db1[i] = acc;
  }
  if (i < U * l) {
    const int u = i / l, m = i % l;
    float acc = 0.f;
    for (int j = 0; j < l; ++j) acc = fmaf(dc[j * U + u], pos[j * l + m], acc);
    dw1[(int64_t)u * ld + dk + m] = acc;
  }
  if (i < l * l) {
    const int j = i / l, m = i % l;
    float acc = 0.f;
    for (int u = 0; u < U; ++u) acc = fmaf(dc[j * U + u], w1[(int64_t)u * ld + dk + m], acc);
    dpos[i] = acc;
  }
}

unsigned blocks_for(int64_t n) { return (unsigned)((n + 255) / 256); }

size_t colsum_scratch_bytes(int64_t rows, int W) { return al256((size_t)((rows + kColsumChunk - 1) / kColsumChunk) * W * sizeof(float)); }
template <typename T>
void colsum(const T* in, int64_t rows, int W, float* out, float* scratch, cudaStream_t st) {
  const int chunks = (int)((rows + kColsumChunk - 1) / kColsumChunk);
  colsum_stage1_kernel<T><<<dim3((W + 31) / 32, chunks), 256, 0, st>>>(in, rows, W, scratch);
  colsum_stage2_kernel<<<blocks_for(W), 256, 0, st>>>(scratch, chunks, W, out);
}

struct SavedLayout { size_t o_a, o_c, o_hbar, total; };
SavedLayout saved_layout(int B, int G, int T, int l, int d, int U) {
  const size_t BG = (size_t)B * G, nb = T >= l ? (size_t)(T - l) / d + 1 : 0;
  SavedLayout s;
  s.o_a = 0;
  s.o_c = al256(BG * T * U * sizeof(float));
  s.o_hbar = s.o_c + al256((size_t)l * U * sizeof(float));
  s.total = s.o_hbar + al256(BG * nb * U * sizeof(float));
  return s;
}
struct BwdLayout { size_t o_dkc, o_dhbar, o_dvc, o_da, o_dalp, o_dcpart, o_dc, o_dvt, o_w1k, o_cs, total; };
BwdLayout bwd_layout(int B, int G, int T, int dk, int dv, int l, int d, int U, int nbp, int dtype) {
  const size_t BG = (size_t)B * G, nb = T >= l ? (size_t)(T - l) / d + 1 : 0, es = dtype == NSA_BF16 ? 2 : 4;
  BwdLayout w;
  size_t o = 0;
  w.o_dkc = o;    o += al256(BG * nb * dk * sizeof(float));
  w.o_dhbar = o;  o += al256(BG * nb * U * sizeof(float));
  w.o_dvc = o;    o += al256(BG * nbp * dv * sizeof(float));
  w.o_da = o;     o += al256(BG * T * U * sizeof(float));
  w.o_dalp = o;   o += dtype == NSA_BF16 ? al256(BG * T * U * es) : 0;
  w.o_dcpart = o; o += al256(BG * l * U * sizeof(float));
  w.o_dc = o;     o += al256((size_t)l * U * sizeof(float));
  w.o_dvt = o;    o += al256(BG * T * dv * sizeof(float));
  w.o_w1k = o;    o += al256((size_t)U * dk * es);
  w.o_cs = o;     o += colsum_scratch_bytes((int64_t)BG * nb, dk);
  w.total = o;
  return w;
}

}  // namespace
}  // namespace nsa

using namespace nsa;

extern "C" NSA_API size_t nsa_cmp_phi_saved_bytes(int B, int G, int T, int l, int d, int U) {
  if (B <= 0 || G <= 0 || T <= 0 || l <= 0 || d <= 0 || U <= 0) return 256;
  return saved_layout(B, G, T, l, d, U).total;
}

extern "C" NSA_API size_t nsa_cmp_phi_workspace_bytes(int B, int G, int T, int dk, int dv, int l, int d, int U, int nbp, int dtype,
                                                      int backward) {
  if (B <= 0 || G <= 0 || T <= 0 || l <= 0 || d <= 0 || U <= 0 || dk <= 0 || dv <= 0) return 256;
  if (!backward) return al256((size_t)3 * U * dk * 2) + 256;
  return bwd_layout(B, G, T, dk, dv, l, d, U, nbp, dtype).total + 256;
}

extern "C" NSA_API int nsa_cmp_phi_fwd(const void* k, const void* v, const float* pos_embed, const float* w1, const float* b1,
                                       const float* w2, const float* b2, float* k_cmp, void* k_cmp_lp, void* v_cmp, int B, int G,
                                       int T, int dk, int dv, int l, int d, int U, int nbp, int dtype, void* saved,
                                       size_t saved_bytes, void* workspace, size_t workspace_bytes, void* stream) {
  NSA_REQUIRE(k && v && pos_embed && w1 && w2 && k_cmp && v_cmp && saved, "cmp_phi_fwd: null pointer");
  NSA_REQUIRE(B > 0 && G > 0 && dk > 0 && dv > 0 && U > 0 && l > 0 && d > 0, "cmp_phi_fwd: bad sizes");
  NSA_REQUIRE(dtype == NSA_F32 || dtype == NSA_BF16, "cmp_phi_fwd: unsupported dtype %d", dtype);
  NSA_REQUIRE(T >= l, "cmp_phi_fwd: sequence length %d shorter than one compression block (%d)", T, l);
  const int nb = (T - l) / d + 1, BG = B * G;
  NSA_REQUIRE(nbp >= nb, "cmp_phi_fwd: nbp = %d holds fewer than the %d blocks of the sequence", nbp, nb);
  const SavedLayout sl = saved_layout(B, G, T, l, d, U);
  if (saved_bytes < sl.total) return fail(NSA_ERR_WORKSPACE, "cmp_phi_fwd needs %zu bytes for the backward's inputs, got %zu", sl.total, saved_bytes);
  const size_t need = nsa_cmp_phi_workspace_bytes(B, G, T, dk, dv, l, d, U, nbp, dtype, 0);
  if (dtype == NSA_BF16 && (!workspace || workspace_bytes < need))
    return fail(NSA_ERR_WORKSPACE, "cmp_phi_fwd needs %zu workspace bytes, got %zu", need, workspace_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  cublasHandle_t h;
  if (int rc = blas_handle(&h, st)) return rc;
  float* a = (float*)((char*)saved + sl.o_a);
  float* c = (float*)((char*)saved + sl.o_c);
  float* hbar = (float*)((char*)saved + sl.o_hbar);
  const int ld1 = dk + l;
  {
    KernelTimer kt("phi_mlp_fwd", st);
    c_table_kernel<<<blocks_for((int64_t)l * U), 256, 0, st>>>(pos_embed, w1, b1, l, U, dk, c);
    // A[bg] (T x U, row-major) = K[bg]^T W1k^T; column-major: C(U x T) = op_T(W (dk x U, ld)) op_T(K (T x dk, ld T))
    if (dtype == NSA_BF16) {
      __nv_bfloat16* hi = (__nv_bfloat16*)workspace;
      __nv_bfloat16 *mid = hi + (size_t)U * dk, *lo = mid + (size_t)U * dk;
      split3_kernel<<<blocks_for((int64_t)U * dk), 256, 0, st>>>(w1, U, dk, ld1, hi, mid, lo);
      const __nv_bfloat16* terms[3] = {hi, mid, lo};
      for (int t3 = 0; t3 < 3; ++t3)
        if (int rc = gemm(h, CUBLAS_OP_T, CUBLAS_OP_T, U, T, dk, terms[t3], CUDA_R_16BF, dk, 0, k, CUDA_R_16BF, T, (long long)dk * T,
                          t3 ? 1.f : 0.f, a, CUDA_R_32F, U, (long long)T * U, BG, "cmp_phi_fwd (K W1k^T)"))
          return rc;
    } else {
      if (int rc = gemm(h, CUBLAS_OP_T, CUBLAS_OP_T, U, T, dk, w1, CUDA_R_32F, ld1, 0, k, CUDA_R_32F, T, (long long)dk * T, 0.f, a,
                        CUDA_R_32F, U, (long long)T * U, BG, "cmp_phi_fwd (K W1k^T)"))
        return rc;
    }
  }
  if (int rc = check_launch("cmp_phi_fwd")) return rc;
  const int64_t vs[4] = {(int64_t)G * T * dv, (int64_t)T * dv, dv, 1};
  if (int rc = nsa_phi_pool_fwd(a, c, v, vs, hbar, v_cmp, B, G, T, U, dv, l, d, nb, nbp, dtype, stream)) return rc;
  {
    KernelTimer kt("phi_mlp_fwd", st);
    // pooled v_cmp rows beyond nb are the caller's zero padding: cleared here so that the caller need not
    const size_t es = dtype == NSA_BF16 ? 2 : 4;
    if (nbp > nb)
      cudaMemset2DAsync((char*)v_cmp + (size_t)nb * dv * es, (size_t)nbp * dv * es, 0, (size_t)(nbp - nb) * dv * es, BG, st);
    // k_cmp[bg] (dk x nbp, row-major) = (hbar[bg] W2^T)^T; column-major: C(nb x dk, ld nbp) = op_T(hbar (U x nb)) W2 (U x dk)
    if (int rc = gemm(h, CUBLAS_OP_T, CUBLAS_OP_N, nb, dk, U, hbar, CUDA_R_32F, U, (long long)nb * U, w2, CUDA_R_32F, U, 0, 0.f, k_cmp,
                      CUDA_R_32F, nbp, (long long)dk * nbp, BG, "cmp_phi_fwd (hbar W2^T)"))
      return rc;
    const int64_t total = (int64_t)BG * dk * nbp;
    if (dtype == NSA_BF16)
      kcmp_finish_kernel<__nv_bfloat16><<<blocks_for(total), 256, 0, st>>>(k_cmp, b2, (__nv_bfloat16*)k_cmp_lp, dk, nb, nbp, total);
    else
      kcmp_finish_kernel<float><<<blocks_for(total), 256, 0, st>>>(k_cmp, b2, (float*)k_cmp_lp, dk, nb, nbp, total);
  }
  return check_launch("cmp_phi_fwd");
}

extern "C" NSA_API int nsa_cmp_phi_bwd(const void* k, const float* pos_embed, const float* w1, const float* w2, const void* dk_cmp,
                                       const void* dv_cmp, const void* saved, size_t saved_bytes, void* dk_out, void* dv_out,
                                       float* dpos, float* dw1, float* db1, float* dw2, float* db2, int B, int G, int T, int dk,
                                       int dv, int l, int d, int U, int nbp, int dtype, void* workspace, size_t workspace_bytes,
                                       void* stream) {
  NSA_REQUIRE(k && pos_embed && w1 && w2 && dk_cmp && dv_cmp && saved && dk_out && dv_out && dpos && dw1 && db1 && dw2 && db2,
              "cmp_phi_bwd: null pointer");
  NSA_REQUIRE(B > 0 && G > 0 && dk > 0 && dv > 0 && U > 0 && l > 0 && d > 0 && T >= l, "cmp_phi_bwd: bad sizes");
  NSA_REQUIRE(dtype == NSA_F32 || dtype == NSA_BF16, "cmp_phi_bwd: unsupported dtype %d", dtype);
  const int nb = (T - l) / d + 1, BG = B * G;
  NSA_REQUIRE(nbp >= nb, "cmp_phi_bwd: nbp = %d holds fewer than the %d blocks of the sequence", nbp, nb);
  const SavedLayout sl = saved_layout(B, G, T, l, d, U);
  if (saved_bytes < sl.total) return fail(NSA_ERR_WORKSPACE, "cmp_phi_bwd: the forward's saved buffer has %zu bytes, got %zu", sl.total, saved_bytes);
  const BwdLayout wl = bwd_layout(B, G, T, dk, dv, l, d, U, nbp, dtype);
  if (!workspace || workspace_bytes < wl.total)
    return fail(NSA_ERR_WORKSPACE, "cmp_phi_bwd needs %zu workspace bytes, got %zu", wl.total, workspace_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  cublasHandle_t h;
  if (int rc = blas_handle(&h, st)) return rc;
  const float* a = (const float*)((const char*)saved + sl.o_a);
  const float* c = (const float*)((const char*)saved + sl.o_c);
  const float* hbar = (const float*)((const char*)saved + sl.o_hbar);
  char* w = (char*)workspace;
  float *dkc = (float*)(w + wl.o_dkc), *dhbar = (float*)(w + wl.o_dhbar), *dvc = (float*)(w + wl.o_dvc), *da = (float*)(w + wl.o_da);
  float *dcpart = (float*)(w + wl.o_dcpart), *dc = (float*)(w + wl.o_dc), *dvt = (float*)(w + wl.o_dvt);
  const int ld1 = dk + l;
  const long long N = (long long)BG * nb;
  {
    KernelTimer kt("phi_mlp_bwd", st);
    const int64_t nk = (int64_t)BG * nb * dk, nv = (int64_t)BG * nbp * dv;
    if (dtype == NSA_BF16) {
      rows_to_f32_kernel<__nv_bfloat16><<<blocks_for(nk), 256, 0, st>>>((const __nv_bfloat16*)dk_cmp, dkc, nbp, nb, nb, dk, nk);
      rows_to_f32_kernel<__nv_bfloat16><<<blocks_for(nv), 256, 0, st>>>((const __nv_bfloat16*)dv_cmp, dvc, nbp, nb, nbp, dv, nv);
    } else {
      rows_to_f32_kernel<float><<<blocks_for(nk), 256, 0, st>>>((const float*)dk_cmp, dkc, nbp, nb, nb, dk, nk);
      rows_to_f32_kernel<float><<<blocks_for(nv), 256, 0, st>>>((const float*)dv_cmp, dvc, nbp, nb, nbp, dv, nv);
    }
    colsum<float>(dkc, N, dk, db2, (float*)(w + wl.o_cs), st);
    // dW2 (dk x U, row-major) = dkc^T hbar; column-major: C(U x dk) = hbar (U x N) op_T(dkc (dk x N))
    if (int rc = gemm(h, CUBLAS_OP_N, CUBLAS_OP_T, U, dk, (int)N, hbar, CUDA_R_32F, U, 0, dkc, CUDA_R_32F, dk, 0, 0.f, dw2, CUDA_R_32F, U, 0,
                      1, "cmp_phi_bwd (dW2)"))
      return rc;
    // dhbar (N x U, row-major) = dkc W2; column-major: C(U x N) = W2 (U x dk) dkc (dk x N)
    if (int rc = gemm(h, CUBLAS_OP_N, CUBLAS_OP_N, U, (int)N, dk, w2, CUDA_R_32F, U, 0, dkc, CUDA_R_32F, dk, 0, 0.f, dhbar, CUDA_R_32F, U, 0,
                      1, "cmp_phi_bwd (dhbar)"))
      return rc;
  }
  if (int rc = check_launch("cmp_phi_bwd")) return rc;
  if (int rc = nsa_phi_pool_bwd(a, c, dhbar, dvc, da, dcpart, dvt, B, G, T, U, dv, l, d, nb, nbp, stream)) return rc;
  {
    KernelTimer kt("phi_mlp_bwd", st);
    const int64_t na = (int64_t)BG * T * U;
    const void* da_op = da;
    const void* w1k_op = w1;
    cudaDataType ot = CUDA_R_32F;
    int ldw = ld1;
    if (dtype == NSA_BF16) {
      __nv_bfloat16* dalp = (__nv_bfloat16*)(w + wl.o_dalp);
      __nv_bfloat16* w1k = (__nv_bfloat16*)(w + wl.o_w1k);
      cast_kernel<__nv_bfloat16><<<blocks_for(na), 256, 0, st>>>(da, dalp, na);
      w1k_cast_kernel<__nv_bfloat16><<<blocks_for((int64_t)U * dk), 256, 0, st>>>(w1, U, dk, ld1, w1k);
      da_op = dalp; w1k_op = w1k; ot = CUDA_R_16BF; ldw = dk;
    }
    // dK[bg] (T x dk, row-major) += da[bg] W1k; column-major: C(dk x T) = W1k (dk x U, ld) da (U x T)
    if (int rc = gemm(h, CUBLAS_OP_N, CUBLAS_OP_N, dk, T, U, w1k_op, ot, ldw, 0, da_op, ot, U, (long long)T * U, 1.f, dk_out, ot, dk,
                      (long long)T * dk, BG, "cmp_phi_bwd (dK)"))
      return rc;
    // dW1[:, :dk] (U x dk inside rows of dk + l, row-major) = sum_bg da[bg]^T K[bg]^T; column-major: C(dk x U, ld dk+l) =
    // op_T(K[bg] (T x dk, ld T)) op_T(da[bg] (U x T)), accumulated over bg in order
    for (int bg = 0; bg < BG; ++bg) {
      const size_t es = dtype == NSA_BF16 ? 2 : 4;
      const void* kb = (const char*)k + (size_t)bg * dk * T * es;
      const void* dab = (const char*)da_op + (size_t)bg * T * U * es;
      if (int rc = gemm(h, CUBLAS_OP_T, CUBLAS_OP_T, dk, U, T, kb, ot, T, 0, dab, ot, U, 0, bg ? 1.f : 0.f, dw1, CUDA_R_32F, ld1, 0, 1,
                        "cmp_phi_bwd (dW1k)"))
        return rc;
    }
    dc_sum_kernel<<<blocks_for((int64_t)l * U), 256, 0, st>>>(dcpart, BG, l * U, dc);
    const int64_t nt = std::max<int64_t>((int64_t)U * l, (int64_t)l * l);
    table_grads_kernel<<<blocks_for(nt), 256, 0, st>>>(dc, pos_embed, w1, l, U, dk, db1, dw1, dpos);
    const int64_t nvt = (int64_t)BG * T * dv;
    if (dtype == NSA_BF16) add_into_kernel<__nv_bfloat16><<<blocks_for(nvt), 256, 0, st>>>((__nv_bfloat16*)dv_out, dvt, nvt);
    else add_into_kernel<float><<<blocks_for(nvt), 256, 0, st>>>((float*)dv_out, dvt, nvt);
  }
  return check_launch("cmp_phi_bwd");
}


// ================================================================================================================
// Branch-gate MLP (nsa/kernels.py:2105-2109): logits = W2 relu(W1 x + b1) + b2, forward and backward, on the same cuBLAS
// handle.  x [N, Dm], w1 [D2, Dm], w2 [O, D2] and the biases in `dtype`; logits [N, O] fp32 (what the gate/mix kernels
// take); the hidden activation [N, D2] in `dtype` is what the backward needs.
// ================================================================================================================
namespace nsa {
namespace {
template <typename T>
__global__ void bias_relu_kernel(T* __restrict__ h, const T* __restrict__ b, int W, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float x = Elem<T>::ld(h + i) + (b ? Elem<T>::ld(b + i % W) : 0.f);
  Elem<T>::st(h + i, x > 0.f ? x : 0.f);
}
template <typename T>
__global__ void bias_add_f32_kernel(float* __restrict__ y, const T* __restrict__ b, int W, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] += Elem<T>::ld(b + i % W);
}
template <typename T>
__global__ void relu_mask_kernel(T* __restrict__ dh, const T* __restrict__ h, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && !(Elem<T>::ld(h + i) > 0.f)) Elem<T>::st(dh + i, 0.f);
}
}  // namespace
}  // namespace nsa

extern "C" NSA_API size_t nsa_gate_mlp_workspace_bytes(int64_t N, int Dm, int D2, int O, int dtype, int backward) {
  if (N <= 0 || Dm <= 0 || D2 <= 0 || O <= 0) return 256;
  const size_t es = dtype == NSA_BF16 ? 2 : 4;
  if (!backward) return 256;
  return al256((size_t)N * O * es) + al256((size_t)N * D2 * es) + colsum_scratch_bytes(N, std::max(O, D2)) + 256;
}

extern "C" NSA_API int nsa_gate_mlp_fwd(const void* x, const void* w1, const void* b1, const void* w2, const void* b2, void* hidden,
                                        float* logits, int64_t N, int Dm, int D2, int O, int dtype, void* stream) {
  NSA_REQUIRE(x && w1 && w2 && hidden && logits, "gate_mlp_fwd: null pointer");
  NSA_REQUIRE(N >= 0 && N < (1ll << 31) && Dm > 0 && D2 > 0 && O > 0, "gate_mlp_fwd: bad sizes");
  NSA_REQUIRE(dtype == NSA_F32 || dtype == NSA_BF16, "gate_mlp_fwd: unsupported dtype %d", dtype);
  if (N == 0) return NSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  cublasHandle_t h;
  if (int rc = blas_handle(&h, st)) return rc;
  const cudaDataType t = dtype == NSA_BF16 ? CUDA_R_16BF : CUDA_R_32F;
  KernelTimer kt("gate_mlp_fwd", st);
  // hidden (N x D2, row-major) = x W1^T; column-major: C(D2 x N) = op_T(W1 (Dm x D2)) x (Dm x N)
  if (int rc = gemm(h, CUBLAS_OP_T, CUBLAS_OP_N, D2, (int)N, Dm, w1, t, Dm, 0, x, t, Dm, 0, 0.f, hidden, t, D2, 0, 1, "gate_mlp_fwd (x W1^T)")) return rc;
  const int64_t nh = N * D2, nl = N * O;
  if (dtype == NSA_BF16) bias_relu_kernel<__nv_bfloat16><<<blocks_for(nh), 256, 0, st>>>((__nv_bfloat16*)hidden, (const __nv_bfloat16*)b1, D2, nh);
  else bias_relu_kernel<float><<<blocks_for(nh), 256, 0, st>>>((float*)hidden, (const float*)b1, D2, nh);
  if (int rc = gemm(h, CUBLAS_OP_T, CUBLAS_OP_N, O, (int)N, D2, w2, t, D2, 0, hidden, t, D2, 0, 0.f, logits, CUDA_R_32F, O, 0, 1, "gate_mlp_fwd (h W2^T)")) return rc;
  if (b2) {
    if (dtype == NSA_BF16) bias_add_f32_kernel<__nv_bfloat16><<<blocks_for(nl), 256, 0, st>>>(logits, (const __nv_bfloat16*)b2, O, nl);
    else bias_add_f32_kernel<float><<<blocks_for(nl), 256, 0, st>>>(logits, (const float*)b2, O, nl);
  }
  return check_launch("gate_mlp_fwd");
}

extern "C" NSA_API int nsa_gate_mlp_bwd(const void* x, const void* w1, const void* w2, const void* hidden, const float* dlogits, void* dx,
                                        float* dw1, float* db1, float* dw2, float* db2, int64_t N, int Dm, int D2, int O, int dtype,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  NSA_REQUIRE(x && w1 && w2 && hidden && dlogits && dw1 && db1 && dw2 && db2, "gate_mlp_bwd: null pointer");
  NSA_REQUIRE(N > 0 && N < (1ll << 31) && Dm > 0 && D2 > 0 && O > 0, "gate_mlp_bwd: bad sizes");
  NSA_REQUIRE(dtype == NSA_F32 || dtype == NSA_BF16, "gate_mlp_bwd: unsupported dtype %d", dtype);
  const size_t need = nsa_gate_mlp_workspace_bytes(N, Dm, D2, O, dtype, 1);
  if (!workspace || workspace_bytes < need) return fail(NSA_ERR_WORKSPACE, "gate_mlp_bwd needs %zu workspace bytes, got %zu", need, workspace_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  cublasHandle_t h;
  if (int rc = blas_handle(&h, st)) return rc;
  const size_t es = dtype == NSA_BF16 ? 2 : 4;
  const cudaDataType t = dtype == NSA_BF16 ? CUDA_R_16BF : CUDA_R_32F;
  char* w = (char*)workspace;
  void* dl = w;                                           // dlogits in the I/O type
  void* dh = w + al256((size_t)N * O * es);               // gradient of the hidden activation
  float* cs = (float*)(w + al256((size_t)N * O * es) + al256((size_t)N * D2 * es));
  KernelTimer kt("gate_mlp_bwd", st);
  const int64_t nl = N * O, nh = N * D2;
  colsum<float>(dlogits, N, O, db2, cs, st);
  const void* dl_op = dlogits;
  if (dtype == NSA_BF16) {
    cast_kernel<__nv_bfloat16><<<blocks_for(nl), 256, 0, st>>>(dlogits, (__nv_bfloat16*)dl, nl);
    dl_op = dl;
  }
  // dW2 (O x D2, row-major) = dl^T hidden; column-major: C(D2 x O) = hidden (D2 x N) op_T(dl (O x N))
  if (int rc = gemm(h, CUBLAS_OP_N, CUBLAS_OP_T, D2, O, (int)N, hidden, t, D2, 0, dl_op, t, O, 0, 0.f, dw2, CUDA_R_32F, D2, 0, 1, "gate_mlp_bwd (dW2)")) return rc;
  // dh (N x D2) = dl W2; column-major: C(D2 x N) = W2 (D2 x O) dl (O x N)
  if (int rc = gemm(h, CUBLAS_OP_N, CUBLAS_OP_N, D2, (int)N, O, w2, t, D2, 0, dl_op, t, O, 0, 0.f, dh, t, D2, 0, 1, "gate_mlp_bwd (dh)")) return rc;
  if (dtype == NSA_BF16) {
    relu_mask_kernel<__nv_bfloat16><<<blocks_for(nh), 256, 0, st>>>((__nv_bfloat16*)dh, (const __nv_bfloat16*)hidden, nh);
    colsum<__nv_bfloat16>((const __nv_bfloat16*)dh, N, D2, db1, cs, st);
  } else {
    relu_mask_kernel<float><<<blocks_for(nh), 256, 0, st>>>((float*)dh, (const float*)hidden, nh);
    colsum<float>((const float*)dh, N, D2, db1, cs, st);
  }
  // dW1 (D2 x Dm, row-major) = dh^T x; column-major: C(Dm x D2) = x (Dm x N) op_T(dh (D2 x N))
  if (int rc = gemm(h, CUBLAS_OP_N, CUBLAS_OP_T, Dm, D2, (int)N, x, t, Dm, 0, dh, t, D2, 0, 0.f, dw1, CUDA_R_32F, Dm, 0, 1, "gate_mlp_bwd (dW1)")) return rc;
  if (dx)  // dx (N x Dm) = dh W1; column-major: C(Dm x N) = W1 (Dm x D2) dh (D2 x N)
    if (int rc = gemm(h, CUBLAS_OP_N, CUBLAS_OP_N, Dm, (int)N, D2, w1, t, Dm, 0, dh, t, D2, 0, 0.f, dx, t, Dm, 0, 1, "gate_mlp_bwd (dx)")) return rc;
  return check_launch("gate_mlp_bwd");
}
