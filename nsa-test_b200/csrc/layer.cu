// The whole NSA layer between the q/k/v projections and the output projection behind two C entry points
// (the wiring of NSAAttention.forward, nsa/kernels.py:2298-2463, and of the backward that the reference leaves to
// autograd): block compression phi -> Eq. 8-11 scoring and top-n -> compressed, sliding-window and selected-block
// attention -> gate + mix (as the epilogue of the selection branch).  Everything the calls need is in their argument
// lists; the forward leaves what the backward needs in a caller-owned context buffer.
//
// Backward order: the gate/mix backward produces the three branch gradients and the row sums dO_b . O_b in one pass;
// the compressed and the sliding-window branch write their dQ to scratch, the selection branch adds both to its own
// before the one rounding of the sum; dK/dV of the three branches and of phi are ADDED into the caller's buffers, so a
// k/v pair that feeds several branches needs no extra accumulation pass.
#include <algorithm>

#include "common.cuh"

namespace nsa {
namespace {

size_t al256(size_t x) { return (x + 255) & ~size_t(255); }
int next_pow2(int n) {
  int p = 1;
  while (p < n) p *= 2;
  return p;
}

struct Sizes {
  int nb, nbp;
  size_t es, rows, o_bytes, stat_bytes;
};
Sizes sizes_of(const nsa_layer_desc& d) {
  Sizes s;
  s.nb = d.T >= d.l ? (d.T - d.l) / d.d + 1 : 0;
  s.nbp = next_pow2(s.nb < 1 ? 1 : s.nb);
  s.es = d.dtype == NSA_BF16 ? 2 : 4;
  s.rows = (size_t)d.B * d.H * d.T;
  s.o_bytes = al256(s.rows * d.dv * s.es);
  s.stat_bytes = al256(s.rows * sizeof(float));
  return s;
}

// context buffer: pieces in the order of enum nsa_layer_ctx_piece
void ctx_layout(const nsa_layer_desc& d, size_t off[NSA_CTX_PIECES + 1]) {
  const Sizes s = sizes_of(d);
  const size_t BG = (size_t)d.B * d.G;
  size_t o = 0;
  auto put = [&](int i, size_t bytes) { off[i] = o; o += al256(bytes); };
  put(NSA_CTX_O_CMP, s.o_bytes);  put(NSA_CTX_L_CMP, s.stat_bytes);  put(NSA_CTX_M_CMP, s.stat_bytes);
  put(NSA_CTX_O_SLC, s.o_bytes);  put(NSA_CTX_L_SLC, s.stat_bytes);  put(NSA_CTX_M_SLC, s.stat_bytes);
  put(NSA_CTX_O_WIN, s.o_bytes);  put(NSA_CTX_L_WIN, s.stat_bytes);  put(NSA_CTX_M_WIN, s.stat_bytes);
  put(NSA_CTX_GATES, s.rows * 3 * sizeof(float));
  put(NSA_CTX_INDICES, BG * d.T * d.n * sizeof(int32_t));
  put(NSA_CTX_K_CMP, BG * d.dk * s.nbp * sizeof(float));
  put(NSA_CTX_K_CMP_LP, BG * d.dk * s.nbp * s.es);
  put(NSA_CTX_V_CMP, BG * s.nbp * d.dv * s.es);
  put(NSA_CTX_BLOCK_ENDS, (size_t)s.nbp * sizeof(int32_t));
  put(NSA_CTX_K_CMP_LO, BG * d.dk * s.nbp * 2);
  put(NSA_CTX_LSE2_CMP, s.stat_bytes);
  put(NSA_CTX_PHI_SAVED, s.nb > 0 ? nsa_cmp_phi_saved_bytes(d.B, d.G, d.T, d.l, d.d, d.U) : 256);
  off[NSA_CTX_PIECES] = o;
}

int check_desc(const char* who, const nsa_layer_desc* d) {
  NSA_REQUIRE(d, "%s: null descriptor", who);
  NSA_REQUIRE(d->B > 0 && d->H > 0 && d->G > 0 && d->H % d->G == 0 && d->T > 0, "%s: bad B/H/G/T", who);
  NSA_REQUIRE(d->dk > 0 && d->dv > 0 && d->U > 0, "%s: bad head dims", who);
  NSA_REQUIRE(d->l > 0 && d->d > 0 && d->l % d->d == 0 && d->l_prime > 0 && d->l_prime % d->d == 0, "%s: bad block sizes", who);
  NSA_REQUIRE(d->n > 0 && d->n_fixed >= 0 && d->window > 0, "%s: bad n / window", who);
  NSA_REQUIRE(d->dtype == NSA_F32 || d->dtype == NSA_BF16, "%s: unsupported dtype %d", who, d->dtype);
  NSA_REQUIRE(d->gate_mode == NSA_GATE_SIGMOID || d->gate_mode == NSA_GATE_SOFTMAX, "%s: bad gate mode", who);
  return NSA_OK;
}

// canonical contiguous strides of the attention entry points
void fill_strides(const nsa_layer_desc& d, int Tk, int nslots, bool backward, bool selection, int64_t* s) {
  const int64_t H = d.H, G = d.G, T = d.T, dk = d.dk, dv = d.dv;
  const int64_t q[4] = {H * T * dk, T * dk, dk, 1}, k[4] = {G * dk * Tk, dk * Tk, 1, Tk}, v[4] = {G * Tk * dv, Tk * dv, dv, 1};
  const int64_t o[4] = {H * T * dv, T * dv, dv, 1}, lm[3] = {H * T, T, 1};
  int i = 0;
  for (int j = 0; j < 4; ++j) s[i++] = q[j];
  for (int j = 0; j < 4; ++j) s[i++] = k[j];
  for (int j = 0; j < 4; ++j) s[i++] = v[j];
  for (int j = 0; j < 4; ++j) s[i++] = o[j];
  for (int j = 0; j < 3; ++j) s[i++] = lm[j];
  for (int j = 0; j < 3; ++j) s[i++] = lm[j];
  if (backward) {
    const int64_t gk[4] = {G * Tk * dk, Tk * dk, dk, 1}, gv[4] = {G * Tk * dv, Tk * dv, dv, 1};
    for (int j = 0; j < 4; ++j) s[i++] = q[j];
    for (int j = 0; j < 4; ++j) s[i++] = gk[j];
    for (int j = 0; j < 4; ++j) s[i++] = gv[j];
  }
  if (selection) {
    const int64_t ix[4] = {G * T * nslots, T * nslots, nslots, 1};
    for (int j = 0; j < 4; ++j) s[i++] = ix[j];
  }
}

__global__ void block_ends_kernel(int32_t* be, int nbp, int nb, int l, int d) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < nbp) be[i] = i < nb ? i * d + l - 1 : 999999;   // padding blocks are never visible (nsa/kernels.py:2185-2192)
}
// rows whose slots are all empty attend the block holding the query (nsa/kernels.py:199-205)
__global__ void selection_fallback_kernel(int32_t* idx, int64_t rows, int T, int n, int lprime) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  int32_t* row = idx + r * n;
  bool any = false;
  for (int s = 0; s < n; ++s) any |= row[s] >= 0;
  if (!any) row[0] = (int32_t)((r % T) / lprime);
}

struct Scratch {
  char* base;
  size_t size, used;
  void* take(size_t bytes) {
    void* p = base + used;
    used += al256(bytes);
    return used <= size ? p : nullptr;
  }
};

size_t stage_scratch_fwd(const nsa_layer_desc& d, const Sizes& s) {
  size_t m = nsa_score_topn_workspace_bytes(d.B, d.H, d.G, d.T, d.dk, s.nbp, d.l, d.d, d.l_prime, d.n, d.dtype, 0);
  m = std::max(m, nsa_slc_fwd_workspace_bytes(d.B, d.H, d.G, d.T, d.T, d.dk, d.dv, d.n, d.l_prime, d.dtype, 0));
  if (s.nb > 0) m = std::max(m, nsa_cmp_phi_workspace_bytes(d.B, d.G, d.T, d.dk, d.dv, d.l, d.d, d.U, s.nbp, d.dtype, 0));
  return al256(m);
}
size_t stage_scratch_bwd(const nsa_layer_desc& d, const Sizes& s) {
  size_t m = nsa_attn_bwd_workspace_bytes(d.B, d.H, d.G, d.T, s.nbp, d.dk, d.dv, 1, 0, 0);
  m = std::max(m, nsa_attn_bwd_workspace_bytes(d.B, d.H, d.G, d.T, d.T, d.dk, d.dv, 0, d.window, 0));
  m = std::max(m, nsa_slc_bwd_workspace_bytes(d.B, d.H, d.G, d.T, d.T, d.dk, d.dv, d.n, d.l_prime, d.dtype, 0));
  if (s.nb > 0) m = std::max(m, nsa_cmp_phi_workspace_bytes(d.B, d.G, d.T, d.dk, d.dv, d.l, d.d, d.U, s.nbp, d.dtype, 1));
  return al256(m);
}
size_t fixed_scratch_bwd(const nsa_layer_desc& d, const Sizes& s) {
  const size_t BG = (size_t)d.B * d.G;
  return 3 * s.o_bytes + 3 * s.stat_bytes + 2 * al256(s.rows * d.dk * s.es) + al256(BG * s.nbp * d.dk * s.es) +
         al256(BG * s.nbp * d.dv * s.es);
}

}  // namespace
}  // namespace nsa

using namespace nsa;

extern "C" NSA_API size_t nsa_layer_ctx_bytes(const nsa_layer_desc* d, size_t* offsets) {
  if (check_desc("layer_ctx_bytes", d)) return 0;
  size_t off[NSA_CTX_PIECES + 1];
  ctx_layout(*d, off);
  if (offsets)
    for (int i = 0; i <= NSA_CTX_PIECES; ++i) offsets[i] = off[i];
  return off[NSA_CTX_PIECES];
}

extern "C" NSA_API size_t nsa_layer_workspace_bytes(const nsa_layer_desc* d, int backward) {
  if (check_desc("layer_workspace_bytes", d)) return 0;
  const Sizes s = sizes_of(*d);
  return backward ? fixed_scratch_bwd(*d, s) + stage_scratch_bwd(*d, s) + 256 : stage_scratch_fwd(*d, s) + 256;
}

extern "C" NSA_API int nsa_layer_fwd(const nsa_layer_desc* dp, const void* q, const void* k_slc, const void* v_slc, const void* k_cmp_src,
                                     const void* v_cmp_src, const void* k_win, const void* v_win, const float* gate_logits,
                                     const float* pos_embed, const float* w1, const float* b1, const float* w2, const float* b2,
                                     const int32_t* indices_in, void* out, void* ctx, size_t ctx_bytes, void* workspace,
                                     size_t workspace_bytes, void* stream) {
  if (int rc = check_desc("layer_fwd", dp)) return rc;
  const nsa_layer_desc& d = *dp;
  NSA_REQUIRE(q && k_slc && v_slc && k_cmp_src && v_cmp_src && k_win && v_win && gate_logits && out && ctx, "layer_fwd: null pointer");
  const Sizes s = sizes_of(d);
  NSA_REQUIRE(s.nb == 0 || (pos_embed && w1 && w2), "layer_fwd: null phi parameter");
  size_t off[NSA_CTX_PIECES + 1];
  ctx_layout(d, off);
  if (ctx_bytes < off[NSA_CTX_PIECES]) return fail(NSA_ERR_WORKSPACE, "layer_fwd needs a context of %zu bytes, got %zu", off[NSA_CTX_PIECES], ctx_bytes);
  const size_t need = nsa_layer_workspace_bytes(dp, 0);
  if (!workspace || workspace_bytes < need) return fail(NSA_ERR_WORKSPACE, "layer_fwd needs %zu workspace bytes, got %zu", need, workspace_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  char* c = (char*)ctx;
  auto piece = [&](int i) { return (void*)(c + off[i]); };
  float* k_cmp = (float*)piece(NSA_CTX_K_CMP);
  int32_t* be = (int32_t*)piece(NSA_CTX_BLOCK_ENDS);
  int32_t* idx = (int32_t*)piece(NSA_CTX_INDICES);
  const size_t BG = (size_t)d.B * d.G;

  // 1. block compression (a sequence shorter than one block leaves only the never-visible padding block)
  block_ends_kernel<<<(s.nbp + 255) / 256, 256, 0, st>>>(be, s.nbp, s.nb, d.l, d.d);
  if (s.nb > 0) {
    if (int rc = nsa_cmp_phi_fwd(k_cmp_src, v_cmp_src, pos_embed, w1, b1, w2, b2, k_cmp, piece(NSA_CTX_K_CMP_LP), piece(NSA_CTX_V_CMP),
                                 d.B, d.G, d.T, d.dk, d.dv, d.l, d.d, d.U, s.nbp, d.dtype, piece(NSA_CTX_PHI_SAVED),
                                 off[NSA_CTX_PHI_SAVED + 1] - off[NSA_CTX_PHI_SAVED], workspace, workspace_bytes, stream))
      return rc;
  } else {
    cudaMemsetAsync(k_cmp, 0, BG * d.dk * s.nbp * sizeof(float), st);
    cudaMemsetAsync(piece(NSA_CTX_K_CMP_LP), 0, BG * d.dk * s.nbp * s.es, st);
    cudaMemsetAsync(piece(NSA_CTX_V_CMP), 0, BG * s.nbp * d.dv * s.es, st);
  }
  int64_t strides[26];
  // 2. compressed attention.  On the tensor-core path it takes the keys as a bf16 pair hi + lo (the fp32 keys to 16
  //    mantissa bits) and also emits the log-sum-exp of its logits, the normaliser the scoring needs: the scoring
  //    kernel then makes one sweep over the compressed keys instead of two.
  const bool exact = s.nb > 0 && nsa_cmp_attn_exact_supported(d.B, d.H, d.G, d.T, s.nbp, d.dk, d.dv, d.dtype) != 0;
  float* lse2 = exact ? (float*)piece(NSA_CTX_LSE2_CMP) : nullptr;
  void* k_lo = exact ? piece(NSA_CTX_K_CMP_LO) : nullptr;
  if (exact)
    if (int rc = nsa_split_keys_hi_lo(k_cmp, piece(NSA_CTX_K_CMP_LP), k_lo, (int64_t)BG * d.dk * s.nbp, stream)) return rc;
  fill_strides(d, s.nbp, 0, false, false, strides);
  if (int rc = nsa_cmp_attn_fwd(q, piece(NSA_CTX_K_CMP_LP), piece(NSA_CTX_V_CMP), be, piece(NSA_CTX_O_CMP), (float*)piece(NSA_CTX_L_CMP),
                                (float*)piece(NSA_CTX_M_CMP), strides, d.B, d.H, d.G, d.T, s.nbp, d.dk, d.dv, d.scale, d.dtype, d.l, d.d,
                                s.nb, 0, 0, k_lo, lse2, stream))
    return rc;
  // 3. Eq. 8-11: which blocks every query attends
  if (indices_in) {
    cudaMemcpyAsync(idx, indices_in, BG * d.T * d.n * sizeof(int32_t), cudaMemcpyDeviceToDevice, st);
  } else {
    const int64_t qs[4] = {(int64_t)d.H * d.T * d.dk, (int64_t)d.T * d.dk, d.dk, 1};
    if (int rc = nsa_score_topn(q, qs, k_cmp, be, idx, d.B, d.H, d.G, d.T, d.dk, s.nbp, d.l, d.d, d.l_prime, d.n, d.n_fixed, d.scale,
                                d.dtype, s.nb, 0, 0, lse2, workspace, workspace_bytes, stream))
      return rc;
  }
  {
    const int64_t rows = (int64_t)BG * d.T;
    selection_fallback_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(idx, rows, d.T, d.n, d.l_prime);
  }
  if (int rc = check_launch("layer_fwd")) return rc;
  // 4. sliding window
  fill_strides(d, d.T, 0, false, false, strides);
  if (int rc = nsa_sliding_fwd(q, k_win, v_win, piece(NSA_CTX_O_WIN), (float*)piece(NSA_CTX_L_WIN), (float*)piece(NSA_CTX_M_WIN), strides,
                               d.B, d.H, d.G, d.T, d.dk, d.dv, d.window, d.scale, d.dtype, 0, stream))
    return rc;
  // 5. selected-block attention with the gate + mix as its epilogue
  fill_strides(d, d.T, d.n, false, true, strides);
  return nsa_slc_fwd_mix(q, k_slc, v_slc, idx, piece(NSA_CTX_O_SLC), (float*)piece(NSA_CTX_L_SLC), (float*)piece(NSA_CTX_M_SLC), strides,
                         d.B, d.H, d.G, d.T, d.T, d.n, d.l_prime, d.dk, d.dv, d.scale, d.dtype, 0, 0, gate_logits,
                         piece(NSA_CTX_O_CMP), piece(NSA_CTX_O_WIN), out, (float*)piece(NSA_CTX_GATES), d.gate_mode,
                         d.out_token_major, workspace, workspace_bytes, stream);
}

extern "C" NSA_API int nsa_layer_bwd(const nsa_layer_desc* dp, const void* q, const void* k_slc, const void* v_slc, const void* k_cmp_src,
                                     const void* k_win, const void* v_win, const float* pos_embed, const float* w1, const float* w2,
                                     const void* ctx, size_t ctx_bytes, const void* dout, void* dq, void* dk_slc, void* dv_slc,
                                     void* dk_cmp_src, void* dv_cmp_src, void* dk_win, void* dv_win, float* dlogits, float* dpos,
                                     float* dw1, float* db1, float* dw2, float* db2, void* workspace, size_t workspace_bytes,
                                     void* stream) {
  if (int rc = check_desc("layer_bwd", dp)) return rc;
  const nsa_layer_desc& d = *dp;
  NSA_REQUIRE(q && k_slc && v_slc && k_cmp_src && k_win && v_win && ctx && dout && dq && dk_slc && dv_slc && dk_cmp_src && dv_cmp_src &&
              dk_win && dv_win && dlogits && dpos && dw1 && db1 && dw2 && db2, "layer_bwd: null pointer");
  const Sizes s = sizes_of(d);
  size_t off[NSA_CTX_PIECES + 1];
  ctx_layout(d, off);
  if (ctx_bytes < off[NSA_CTX_PIECES]) return fail(NSA_ERR_WORKSPACE, "layer_bwd: the forward's context has %zu bytes, got %zu", off[NSA_CTX_PIECES], ctx_bytes);
  const size_t need = nsa_layer_workspace_bytes(dp, 1);
  if (!workspace || workspace_bytes < need) return fail(NSA_ERR_WORKSPACE, "layer_bwd needs %zu workspace bytes, got %zu", need, workspace_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  const char* c = (const char*)ctx;
  auto piece = [&](int i) { return (const void*)(c + off[i]); };
  const size_t BG = (size_t)d.B * d.G;
  Scratch sc{(char*)workspace, workspace_bytes, 0};
  void *d_cmp = sc.take(s.o_bytes), *d_slc = sc.take(s.o_bytes), *d_win = sc.take(s.o_bytes);
  float* delta = (float*)sc.take(3 * s.stat_bytes);
  void *dq_c = sc.take(s.rows * d.dk * s.es), *dq_w = sc.take(s.rows * d.dk * s.es);
  void *dkc = sc.take(BG * s.nbp * d.dk * s.es), *dvc = sc.take(BG * s.nbp * d.dv * s.es);
  void* stage = sc.base + sc.used;
  const size_t stage_bytes = workspace_bytes - sc.used;
  // delta holds three vectors of B*H*T floats back to back (the gate/mix backward's layout), not padded ones
  const float *delta0 = delta, *delta1 = delta + s.rows, *delta2 = delta + 2 * s.rows;

  if (int rc = nsa_gate_mix_bwd_delta((const float*)piece(NSA_CTX_GATES), piece(NSA_CTX_O_CMP), piece(NSA_CTX_O_SLC), piece(NSA_CTX_O_WIN), dout,
                                      d_cmp, d_slc, d_win, dlogits, delta, d.B, d.H, d.T, d.dv, d.gate_mode, d.dtype, d.out_token_major,
                                      stream))
    return rc;
  int64_t strides[38];
  const int32_t* be = (const int32_t*)piece(NSA_CTX_BLOCK_ENDS);
  cudaMemsetAsync(dkc, 0, BG * s.nbp * d.dk * s.es, st);
  cudaMemsetAsync(dvc, 0, BG * s.nbp * d.dv * s.es, st);
  fill_strides(d, s.nbp, 0, true, false, strides);
  if (int rc = nsa_cmp_attn_bwd(q, piece(NSA_CTX_K_CMP_LP), piece(NSA_CTX_V_CMP), be, piece(NSA_CTX_O_CMP), d_cmp,
                                (const float*)piece(NSA_CTX_L_CMP), (const float*)piece(NSA_CTX_M_CMP), dq_c, dkc, dvc, strides, d.B, d.H, d.G,
                                d.T, s.nbp, d.dk, d.dv, d.scale, d.dtype, d.l, d.d, s.nb, 0, delta0, 0, stage, stage_bytes, stream))
    return rc;
  fill_strides(d, d.T, 0, true, false, strides);
  if (int rc = nsa_sliding_bwd(q, k_win, v_win, piece(NSA_CTX_O_WIN), d_win, (const float*)piece(NSA_CTX_L_WIN),
                               (const float*)piece(NSA_CTX_M_WIN), dq_w, dk_win, dv_win, strides, d.B, d.H, d.G, d.T, d.dk, d.dv, d.window,
                               d.scale, d.dtype, delta2, 0, stage, stage_bytes, stream))
    return rc;
  fill_strides(d, d.T, d.n, true, true, strides);
  if (int rc = nsa_slc_bwd(q, k_slc, v_slc, (const int32_t*)piece(NSA_CTX_INDICES), piece(NSA_CTX_O_SLC), d_slc,
                           (const float*)piece(NSA_CTX_L_SLC), (const float*)piece(NSA_CTX_M_SLC), dq, dk_slc, dv_slc, strides, d.B, d.H, d.G,
                           d.T, d.T, d.n, d.l_prime, d.dk, d.dv, d.scale, d.dtype, 0, delta1, dq_c, dq_w, 0, stage, stage_bytes, stream))
    return rc;
  if (s.nb > 0)
    return nsa_cmp_phi_bwd(k_cmp_src, pos_embed, w1, w2, dkc, dvc, piece(NSA_CTX_PHI_SAVED), off[NSA_CTX_PHI_SAVED + 1] - off[NSA_CTX_PHI_SAVED],
                           dk_cmp_src, dv_cmp_src, dpos, dw1, db1, dw2, db2, d.B, d.G, d.T, d.dk, d.dv, d.l, d.d, d.U, s.nbp, d.dtype,
                           stage, stage_bytes, stream);
  // no compression block exists: phi took no part in the forward
  cudaMemsetAsync(dpos, 0, (size_t)d.l * d.l * sizeof(float), st);
  cudaMemsetAsync(dw1, 0, (size_t)d.U * (d.dk + d.l) * sizeof(float), st);
  cudaMemsetAsync(db1, 0, (size_t)d.U * sizeof(float), st);
  cudaMemsetAsync(dw2, 0, (size_t)d.dk * d.U * sizeof(float), st);
  cudaMemsetAsync(db2, 0, (size_t)d.dk * sizeof(float), st);
  return NSA_OK;
}
