/*
 * nsa_b200.h - C ABI of the B200 (sm_100a) Native Sparse Attention kernels.
 *
 * Every entry point takes raw DEVICE pointers, explicit element strides, sizes, a dtype code and a
 * CUDA stream handle (cudaStream_t passed as void*), launches asynchronously on that stream and
 * returns 0 on success or a negative NSA_ERR_* code (nsa_last_error() then holds a message).
 * Nothing here allocates device memory unless stated; scratch memory is passed in by the caller and
 * sized by the matching *_workspace_bytes() query.  No entry point has a CPU fallback.
 *
 * Layout conventions (those of the reference project's kernel-call contract, README.md:55-101 of
 * Noumena-Network/NSA-Test):
 *   Q   [B,H,T,dk]          strides (z,h,m,k)
 *   K   [B,G,dk,T] in memory; its strides are passed in the order (z,g,n=time,k=dk)
 *   V   [B,G,T,dv]          strides (z,g,n,k)
 *   Out [B,H,T,dv]          strides (z,h,m,k); dOut uses Out's strides
 *   L,M [B,H,T] fp32        L = log(sum exp(s - M)), M = row max of the scaled logits
 *   dQ  like Q (overwritten); dK is [B,G,T,dk] (time-major!) and dV [B,G,T,dv]: both must be
 *   zero-initialised by the caller, the kernels add into them (nsa/kernels.py:1146-1148).
 * Kernels honour whatever strides they are given (tests/test_kernel_contracts.py:68-90 of the
 * reference passes wrong K strides on purpose and expects a different answer, not a fault).
 */
#ifndef NSA_B200_H
#define NSA_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define NSA_API __attribute__((visibility("default")))
#else
#define NSA_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum { NSA_F32 = 0, NSA_BF16 = 1 };
enum { NSA_GATE_SIGMOID = 0, NSA_GATE_SOFTMAX = 1 };
enum {
  NSA_OK = 0,
  NSA_ERR_ARG = -1,        /* bad size / dtype / null pointer */
  NSA_ERR_LAUNCH = -2,     /* CUDA reported a launch error */
  NSA_ERR_WORKSPACE = -3,  /* scratch buffer missing or too small */
  NSA_ERR_UNSUPPORTED = -4 /* shape outside what the requested kernel family covers */
};

/* `flags` argument of the attention and scoring entry points (testing / cross-checks): by default a call runs the
 * tensor-core (tcgen05) kernels when it qualifies (bf16, canonical contiguous layouts, supported head dims, T a
 * multiple of 128) and the stride-generic kernels otherwise; NSA_FLAG_GENERIC forces the stride-generic kernels. */
enum { NSA_FLAG_GENERIC = 1, NSA_FLAG_RECOMPUTE = 2 };

/* `q_pos0` argument (query-sharded long-context runs and incremental decoding; the reference has no counterpart, its
 * wrappers assume query row t sits at position t): position of query row 0 in the sequence.  The keys keep starting
 * at position 0.  Honoured by the bf16 tensor-core paths of nsa_cmp_attn_fwd/bwd, nsa_slc_fwd/bwd and by
 * nsa_score_topn; any other path refuses a non-zero offset with NSA_ERR_ARG.
 *
 * `row_delta` argument of the backward entry points: the row sums dO . O [B,H,T] (fp32, contiguous) when the caller
 * has them already (nsa_gate_mix_bwd_delta writes them), else NULL and the call computes them (the reference computes
 * them inside its backward kernels, nsa/kernels.py:1004-1010).  Used by the tensor-core paths.
 *
 * `dq_add0/dq_add1` of nsa_slc_bwd: dQ of the other two branches (same dtype and contiguous [B,H,T,dk] layout as dq,
 * either may be NULL); the call then writes dq = dq_selection + dq_add0 + dq_add1, summed in fp32 and rounded once (the
 * reference leaves that sum to autograd, nsa/kernels.py:2446-2463 feeds one q to all three branches).
 *
 * The library keeps no per-call state between entry points: everything a call depends on is in its argument list. */

/* Every wait inside the tensor-core kernels is bounded (about 0.15 s).  A thread block whose wait runs out tears
 * down cleanly, counts itself on the device and raises a flag in mapped host memory; blocks and launches that start
 * afterwards skip their work, and EVERY attention / scoring entry point then returns NSA_ERR_LAUNCH (tested on entry,
 * without synchronising) until the caller acknowledges with nsa_device_timeouts(1).  nsa_device_timeouts returns the
 * number of blocks that gave up on the current device (0 in a healthy run), synchronises the device, and with
 * reset != 0 clears counter and flag.  Negative = error. */
NSA_API int nsa_device_timeouts(int reset);
/* Self-test of that mechanism (no counterpart in the reference): one warp waits `limit_clocks` (1..2^24) on a barrier
 * that nothing arrives at, gives up and reports like a product kernel.  Synchronises the stream.  Afterwards
 * nsa_device_timeouts(0) reads 1 and the entry points refuse work until nsa_device_timeouts(1). */
NSA_API int nsa_selftest_wait_timeout(long long limit_clocks, void* stream);

/* Per-kernel timing for benchmarks: while enabled, every kernel launch of this library is bracketed
 * by a CUDA event pair on its stream.  nsa_profile_report() synchronises the device and writes one
 * line per kernel family, "name launches total_ms", in first-launch order.  Enabling clears old
 * records.  Leave it off in timed regions (two extra event records per launch). */
NSA_API int nsa_profile_enable(int on);
NSA_API int nsa_profile_report(char* buf, size_t buf_bytes);

/* Message for the last non-zero status returned on the calling thread. */
NSA_API const char* nsa_last_error(void);
/* Library / build identification: "nsa_b200 <version> sm_100a". */
NSA_API const char* nsa_version(void);

/* Strides block shared by the attention entry points, in elements:
 *   [0..3] q (z,h,m,k)   [4..7] k (z,g,n,k)   [8..11] v (z,g,n,k)   [12..15] out (z,h,m,k)
 *   [16..18] L (z,h,m)   [19..21] M (z,h,m)
 * backward adds [22..25] dq (z,h,m,k)  [26..29] dk (z,g,n,k)  [30..33] dv (z,g,n,k)
 * selection adds, after those of its direction, 4 strides of the index tensor (z,g,m,n).      */

/* Sliding-window attention, query t sees keys [max(0,t-window+1), t].
 * Replaces _nsa_sliding_window_fwd_kernel / _bwd_kernel (nsa/kernels.py:1151-1300, 1303-1530). */
NSA_API int nsa_sliding_fwd(const void* q, const void* k, const void* v, void* out, float* L, float* M,
                    const int64_t* strides22, int B, int H, int G, int T, int dk, int dv, int window,
                    float scale, int dtype, int flags, void* stream);
/* The backward entry points of the sliding and compression branches take scratch memory of
 * nsa_attn_bwd_workspace_bytes() bytes, used by the tensor-core kernels: per-row statistics, for the compression
 * branch per-head-chunk partial dK/dV sums that are then added in a fixed order, and the dS^T tiles (bf16, one
 * 16 KiB tile per visible (key tile, 64-query sub-tile, head)) that the key-stationary dK/dV kernel leaves for the
 * dQ kernel, so that S and dP are computed once per backward step.  With flags = NSA_FLAG_RECOMPUTE the query
 * returns the small scratch only; a backward call given that much recomputes S and dP in its dQ kernel instead
 * (same results up to the rounding of dS, several times less scratch, more time).  `window` is the sliding
 * window (ignored for the compression branch). */
NSA_API size_t nsa_attn_bwd_workspace_bytes(int B, int H, int G, int Tq, int Tk, int dk, int dv,
                                            int is_compression, int window, int flags);
NSA_API int nsa_sliding_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                    const float* L, const float* M, void* dq, void* dkey, void* dval,
                    const int64_t* strides34, int B, int H, int G, int T, int dk, int dv, int window,
                    float scale, int dtype, const float* row_delta, int flags, void* workspace,
                    size_t workspace_bytes, void* stream);

/* Sliding-window backward for callers that cannot allocate device memory.  (No counterpart in the reference
 * project: its wrappers allocate freely through torch.)
 * Some hosts of this library may not call cudaMalloc at the point where they need the backward pass: code
 * running inside a CUDA-graph capture, a runtime that handed out all device memory up front, a real-time
 * loop that must not touch the allocator.  This variant of nsa_sliding_bwd takes no workspace: its scratch
 * (two floats per (batch, head, query) row) is a device array built into the library, 8 MiB that every GPU
 * loading the library holds until the process exits.
 *   - Tensors: bf16, the canonical contiguous layouts (q [B,H,T,dk], k [B,G,dk,T], v [B,G,T,dv], out/dout
 *     [B,H,T,dv], L/M [B,H,T], dq like q, dkey [B,G,T,dk], dval [B,G,T,dv]), 16-byte aligned, shapes the
 *     tensor-core kernels cover; anything else returns NSA_ERR_UNSUPPORTED (nsa_sliding_bwd serves it, and its
 *     stride-generic kernels need no scratch anyway).
 *   - Limit: B*H*T <= 1,048,576 rows; larger calls are rejected with NSA_ERR_UNSUPPORTED and a message.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, no
 *     allocation); make that first call before any stream capture begins.
 *   - No cudaMalloc, cudaFree or other allocating routine is called.  Nothing in the scratch needs clearing
 *     between calls (each call overwrites the rows it reads).
 *   - All calls on a device share the one array: two calls whose kernels may overlap on the GPU (different
 *     streams, no dependency) race on it.  Serialise them.
 * dkey/dval are added into (zero them first), dq is overwritten, as with nsa_sliding_bwd. */
NSA_API int nsa_sliding_bwd_noalloc(const void* q, const void* k, const void* v, const void* out,
                                    const void* dout, const float* L, const float* M, void* dq, void* dkey,
                                    void* dval, int B, int H, int G, int T, int dk, int dv, int window,
                                    float scale, void* stream);

/* Attention over compressed tokens, block i visible iff block_ends[i] <= t; a row that sees no block
 * gets out = 0, L = M = -inf.  k_cmp is [B,G,dk,NB] with strides passed (z,g,n=block,k), v_cmp
 * [B,G,NB,dv]; dk_cmp is written [B,G,NB,dk].  Layout hint (forward): blocks_d > 0 asserts that
 * block_ends[i] == i*blocks_d + blocks_l - 1 for i < blocks_n and that later blocks are never
 * visible, which lets the tensor-core kernels skip tiles; blocks_d == 0 makes no assumption.
 * Replaces _nsa_compression_fwd_kernel / _bwd_kernel (nsa/kernels.py:1533-1687, 1690-1917). */
/* Exact-key form (k_cmp_lo and lse2_out both non-NULL; bf16 tensor-core path only, nsa_cmp_attn_exact_supported tells
 * for a shape, and the call needs the block layout hint, canonical layouts and L, M): k_cmp is the bf16 rounding of the
 * fp32 compressed keys and k_cmp_lo [B,G,dk,NB] the bf16 rounding of the remainder (nsa_split_keys_hi_lo makes both);
 * the logits are q (k_cmp + k_cmp_lo), i.e. those of the fp32 keys to 16 mantissa bits, and lse2_out [B,H,T] fp32
 * receives their log-sum-exp in log2 units (+inf for rows that see no block).  That is the normaliser of Eq. 8, so
 * nsa_score_topn given it as cmp_lse2 skips its own first sweep over the compressed keys. */
NSA_API int nsa_cmp_attn_exact_supported(int B, int H, int G, int T, int NB, int dk, int dv, int dtype);
NSA_API int nsa_split_keys_hi_lo(const float* x, void* hi, void* lo, int64_t n, void* stream);
NSA_API int nsa_cmp_attn_fwd(const void* q, const void* k_cmp, const void* v_cmp, const int32_t* block_ends,
                     void* out, float* L, float* M, const int64_t* strides22, int B, int H, int G,
                     int T, int NB, int dk, int dv, float scale, int dtype, int blocks_l, int blocks_d,
                     int blocks_n, int q_pos0, int flags, const void* k_cmp_lo, float* lse2_out, void* stream);
NSA_API int nsa_cmp_attn_bwd(const void* q, const void* k_cmp, const void* v_cmp, const int32_t* block_ends,
                     const void* out, const void* dout, const float* L, const float* M, void* dq,
                     void* dk_cmp, void* dv_cmp, const int64_t* strides34, int B, int H, int G, int T,
                     int NB, int dk, int dv, float scale, int dtype, int blocks_l, int blocks_d,
                     int blocks_n, int q_pos0, const float* row_delta, int flags, void* workspace,
                     size_t workspace_bytes, void* stream);

/* Selected-block attention: query t of group g sees the union of blocks indices[b,g,t,:] (ids < 0
 * and blocks starting at or beyond Tkv ignored, a repeated id counts once) intersected with
 * keys <= t.  indices is int32.
 * Replaces _nsa_sparse_selection_fwd_kernel / _bwd_kernel (nsa/kernels.py:594-833, 836-1148). */
/* The tensor-core path works key-block-major (each KV block is staged once and shared by all queries
 * and heads that selected it) and needs scratch for the inverse index and per-(query, slot) partial
 * results: nsa_slc_fwd_workspace_bytes() bytes (256 when the stride-generic kernels will run). */
NSA_API size_t nsa_slc_fwd_workspace_bytes(int B, int H, int G, int Tq, int Tkv, int dk, int dv,
                                           int n_slots, int l_prime, int dtype, int flags);
NSA_API int nsa_slc_fwd(const void* q, const void* k, const void* v, const int32_t* indices, void* out,
                float* L, float* M, const int64_t* strides26, int B, int H, int G, int Tq, int Tkv,
                int n_slots, int l_prime, int dk, int dv, float scale, int dtype, int q_pos0, int flags,
                void* workspace, size_t workspace_bytes, void* stream);
/* The same forward with the gate + mix of the layer (nsa/kernels.py:2446-2463) as its epilogue: the selection branch
 * runs last, and the kernel that merges a query's per-slot partials, holding the finished O_slc row, also writes
 * out_mixed = g0*o_cmp + g1*O_slc + g2*o_win and the gates (gates_out [B,H,Tq,3] fp32; gate_logits [B,Tq,3H] fp32;
 * o_cmp, o_win contiguous [B,H,Tq,dv] in dtype).  out_mixed is head-major [B,H,Tq,dv], or with
 * out_token_major != 0 token-major [B,Tq,H,dv], which the output projection reads without a transposing copy
 * (the reference copies: nsa/kernels.py:2466-2467).  `out` still receives O_slc (the backward needs it).  Calls
 * that run on the stride-generic kernels do the mix as a separate pass inside this entry point. */
NSA_API int nsa_slc_fwd_mix(const void* q, const void* k, const void* v, const int32_t* indices, void* out,
                    float* L, float* M, const int64_t* strides26, int B, int H, int G, int Tq, int Tkv,
                    int n_slots, int l_prime, int dk, int dv, float scale, int dtype, int q_pos0, int flags,
                    const float* gate_logits, const void* o_cmp, const void* o_win, void* out_mixed,
                    float* gates_out, int gate_mode, int out_token_major, void* workspace,
                    size_t workspace_bytes, void* stream);
/* Backward; dK/dV are reduced per key block over the queries that selected it in a fixed order (an
 * inverse index "block -> queries" is built in the workspace; the tensor-core path also keeps per-
 * (query, slot) dQ partials and per-block dK/dV partials there), so results are run-to-run identical. */
NSA_API size_t nsa_slc_bwd_workspace_bytes(int B, int H, int G, int Tq, int Tkv, int dk, int dv,
                                           int n_slots, int l_prime, int dtype, int flags);
NSA_API int nsa_slc_bwd(const void* q, const void* k, const void* v, const int32_t* indices, const void* out,
                const void* dout, const float* L, const float* M, void* dq, void* dkey, void* dval,
                const int64_t* strides38, int B, int H, int G, int Tq, int Tkv, int n_slots,
                int l_prime, int dk, int dv, float scale, int dtype, int q_pos0, const float* row_delta,
                const void* dq_add0, const void* dq_add1, int flags, void* workspace, size_t workspace_bytes,
                void* stream);

/* Block-compression MLP phi, whole (NSAAttention.compress_tokens, nsa/kernels.py:2096-2102, 2119-2208):
 *   k_cmp[i] = mean_{j<l} ( W2 relu(W1 [k_{i d + j} || pos_embed[j]] + b1) + b2 ),   v_cmp[i] = mean_{j<l} v_{i d + j}
 * for the (T - l) / d + 1 blocks of the sequence.  k [B,G,dk,T] and v [B,G,T,dv] contiguous in dtype (the layouts of
 * the attention entry points); pos_embed [l,l], w1 [U,dk+l], b1 [U], w2 [dk,U], b2 [dk] fp32 (b1, b2 may be NULL);
 * k_cmp fp32 [B,G,dk,nbp] (fp32 because it decides the top-n; blocks >= n_blocks zero), k_cmp_lp an optional copy of
 * it in dtype for nsa_cmp_attn_fwd (or NULL), v_cmp [B,G,nbp,dv] in dtype (rows >= n_blocks zero).  The first product
 * K^T W1[:, :dk]^T holds exactly the products of an fp32 GEMM also for bf16 keys (three-term bf16 split of the weight,
 * fp32 accumulation).  `saved` (nsa_cmp_phi_saved_bytes) receives what the backward needs; `workspace`
 * (nsa_cmp_phi_workspace_bytes, backward = 0 / 1) is scratch.  The dense products run on cuBLAS, which is looked up
 * when first needed (NSA_ERR_UNSUPPORTED if it cannot be loaded); a cuBLAS handle is created once per device. */
NSA_API size_t nsa_cmp_phi_saved_bytes(int B, int G, int T, int l, int d, int U);
NSA_API size_t nsa_cmp_phi_workspace_bytes(int B, int G, int T, int dk, int dv, int l, int d, int U, int nbp,
                                           int dtype, int backward);
NSA_API int nsa_cmp_phi_fwd(const void* k, const void* v, const float* pos_embed, const float* w1, const float* b1,
                    const float* w2, const float* b2, float* k_cmp, void* k_cmp_lp, void* v_cmp, int B, int G,
                    int T, int dk, int dv, int l, int d, int U, int nbp, int dtype, void* saved,
                    size_t saved_bytes, void* workspace, size_t workspace_bytes, void* stream);
/* Backward of phi.  dk_cmp [B,G,nbp,dk] and dv_cmp [B,G,nbp,dv] in dtype are the gradients of the compressed keys and
 * values as nsa_cmp_attn_bwd writes them (block-major).  dk_out [B,G,T,dk] and dv_out [B,G,T,dv] in dtype are ADDED
 * INTO, like the dK/dV of the attention entry points, so one pair of buffers can collect the gradient of a k/v that
 * feeds several branches.  dpos [l,l], dw1 [U,dk+l], db1 [U], dw2 [dk,U], db2 [dk] fp32 are overwritten. */
NSA_API int nsa_cmp_phi_bwd(const void* k, const float* pos_embed, const float* w1, const float* w2,
                    const void* dk_cmp, const void* dv_cmp, const void* saved, size_t saved_bytes, void* dk_out,
                    void* dv_out, float* dpos, float* dw1, float* db1, float* dw2, float* db2, int B, int G,
                    int T, int dk, int dv, int l, int d, int U, int nbp, int dtype, void* workspace,
                    size_t workspace_bytes, void* stream);

/* Pooling half of the block-compression MLP phi (NSAAttention.compress_tokens, nsa/kernels.py:
 * 2119-2208).  With A[t,:] = W1[:, :dk] k_t (a plain GEMM done by the caller) and the table
 * C[j,:] = W1[:, dk:] pos_embed[j] + b1, computes hbar[i,:] = mean_{j<l} relu(A[i*d+j,:] + C[j,:])
 * and v_cmp[i,:] = mean_{j<l} v[i*d+j,:] for i < n_blocks; the caller finishes with
 * k_cmp[i] = W2 hbar[i] + b2.  a [BG,T,U] fp32, c [l,U] fp32, v [B,G,T,dv] (strides z,g,n,k; dtype),
 * hbar [BG,n_blocks,U] fp32, v_cmp [B,G,nbp,dv] contiguous in dtype (rows >= n_blocks untouched). */
NSA_API int nsa_phi_pool_fwd(const float* a, const float* c, const void* v, const int64_t* v_strides4,
                     float* hbar, void* v_cmp, int B, int G, int T, int U, int dv, int l, int d,
                     int n_blocks, int nbp, int dtype, void* stream);
/* Backward of the pooling: da[t,u] = sum over blocks i holding t of [A[t,u]+C[j,u] > 0] dhbar[i,u]/l,
 * dc_part[bg,j,u] = sum_i of the same terms (the caller sums dc_part over bg), and
 * dv[t,:] = sum over blocks holding t of dv_cmp[i,:]/l (fp32 [B,G,T,dv] contiguous, overwritten);
 * dhbar [BG,n_blocks,U], dv_cmp [BG,nbp,dv] fp32. */
NSA_API int nsa_phi_pool_bwd(const float* a, const float* c, const float* dhbar, const float* dv_cmp,
                     float* da, float* dc_part, float* dv, int B, int G, int T, int U, int dv_dim,
                     int l, int d, int n_blocks, int nbp, void* stream);

/* Eq. 8 -> 9 -> 10/11 in one pass (nsa/kernels.py:2304-2343, 1920-1962, 1965-2040): softmax of
 * q k_cmp over visible blocks (fallback: block 0 alone), the (l/d x l'/d) stencil onto selection
 * blocks, the sum over the heads of each group in head order, a stable top-min(n,n_sel) (ties to the
 * lower block id), then the fixed blocks [0, max(0,(t-l')/l'), t/l'] prepended, repeats dropped,
 * cut to n and padded with -1.  q [B,H,T,dk] (dtype, strides z,h,m,k), k_cmp fp32 [B,G,dk,nbp]
 * contiguous, block_ends [nbp], indices_out int32 [B,G,T,n] contiguous.
 * n_real_blocks >= 0 asserts block_ends[i] == i*d + l - 1 for i < n_real_blocks and no later block ever
 * visible, which admits the tensor-core kernel (fp32 keys split into bf16 hi + lo parts held in the
 * workspace of nsa_score_topn_workspace_bytes() bytes); -1 makes no assumption.  cmp_lse2 (or NULL): the
 * log-sum-exp [B,H,T] of the same logits from nsa_cmp_attn_fwd's exact-key form (same q_pos0); the tensor-core kernel
 * then makes one sweep over the compressed keys instead of two (other paths ignore it and compute their own). */
NSA_API size_t nsa_score_topn_workspace_bytes(int B, int H, int G, int T, int dk, int nbp, int l, int d,
                                              int l_prime, int n, int dtype, int flags);
NSA_API int nsa_score_topn(const void* q, const int64_t* q_strides4, const float* k_cmp,
                   const int32_t* block_ends, int32_t* indices_out, int B, int H, int G, int T, int dk,
                   int nbp, int l, int d, int l_prime, int n, int n_fixed, float scale, int dtype,
                   int n_real_blocks, int q_pos0, int flags, const float* cmp_lse2, void* workspace,
                   size_t workspace_bytes, void* stream);
/* Eq. 10/11 alone on a given score tensor [B,H,T,n_sel] fp32 contiguous
 * (select_top_k_blocks_per_query_with_gqa, nsa/kernels.py:1965-2040). */
NSA_API int nsa_topn_from_scores(const float* scores, int32_t* indices_out, int B, int H, int G, int T,
                         int n_sel, int l_prime, int n, int n_fixed, void* stream);

/* Diagnostics behind the module's output_attentions=True report (nsa/kernels.py:2481-2488), never
 * on the training path: Eq. 8 probabilities materialised as out [B,H,T,nbp] fp32, and Eq. 9 applied
 * to a materialised probability tensor of `rows` rows (derive_selection_from_compression_per_timestep,
 * nsa/kernels.py:1920-1962), out [rows, ceil(n_cmp/(l'/d))] fp32. */
NSA_API int nsa_cmp_probs(const void* q, const int64_t* q_strides4, const float* k_cmp,
                          const int32_t* block_ends, float* out, int B, int H, int G, int T, int dk,
                          int nbp, float scale, int dtype, void* stream);
NSA_API int nsa_eq9_scores(const float* p_cmp, float* out, int64_t rows, int n_cmp, int l, int d,
                           int l_prime, void* stream);

/* Gate + mix (nsa/kernels.py:2446-2463): gates = sigmoid | softmax-over-3 of logits[b,t,3h+i],
 * out = g0*o_cmp + g1*o_slc + g2*o_win.  logits [B,T,3H] fp32, branch outputs [B,H,T,dv] contiguous in dtype,
 * gates_out [B,H,T,3] fp32 (saved for backward / diagnostics).  out is head-major [B,H,T,dv] or, with
 * out_token_major != 0, token-major [B,T,H,dv] (what the output projection consumes without a copy). */
NSA_API int nsa_gate_mix_fwd(const float* logits, const void* o_cmp, const void* o_slc, const void* o_win,
                     void* out, float* gates_out, int B, int H, int T, int dv, int gate_mode,
                     int dtype, int out_token_major, void* stream);
/* Backward: d_branch_i = g_i * dout (three tensors in dtype, head-major), dlogits [B,T,3H] fp32; dout is head-major
 * or (dout_token_major != 0) token-major like the forward's out. */
NSA_API int nsa_gate_mix_bwd(const float* gates, const void* o_cmp, const void* o_slc, const void* o_win,
                     const void* dout, void* do_cmp, void* do_slc, void* do_win, float* dlogits,
                     int B, int H, int T, int dv, int gate_mode, int dtype, int dout_token_major,
                     void* stream);

/* Branch-gate MLP (nsa/kernels.py:2105-2109): logits = W2 relu(W1 x + b1) + b2 for N = B*T tokens.  x [N,Dm], w1 [D2,Dm],
 * b1 [D2], w2 [O,D2], b2 [O] (O = 3H) in dtype (biases may be NULL); logits [N,O] fp32, the input of the gate/mix entry
 * points; hidden [N,D2] in dtype receives the activation the backward needs.  GEMMs on cuBLAS (see nsa_cmp_phi_fwd).
 * Backward: dlogits [N,O] fp32 -> dw1 [D2,Dm], db1 [D2], dw2 [O,D2], db2 [O] fp32 (overwritten) and, when dx != NULL, dx
 * [N,Dm] in dtype; scratch of nsa_gate_mlp_workspace_bytes(..., backward = 1) bytes. */
NSA_API size_t nsa_gate_mlp_workspace_bytes(int64_t N, int Dm, int D2, int O, int dtype, int backward);
NSA_API int nsa_gate_mlp_fwd(const void* x, const void* w1, const void* b1, const void* w2, const void* b2, void* hidden,
                     float* logits, int64_t N, int Dm, int D2, int O, int dtype, void* stream);
NSA_API int nsa_gate_mlp_bwd(const void* x, const void* w1, const void* w2, const void* hidden, const float* dlogits,
                     void* dx, float* dw1, float* db1, float* dw2, float* db2, int64_t N, int Dm, int D2, int O,
                     int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* Same, and also writes delta [3][B*H*T] (fp32): the row sums dO_b . O_b of the three branches (dO_b = g_b dO), which
 * the branch backward kernels need.  Handing them over as `row_delta` saves each backward its own pass over O and dO. */
NSA_API int nsa_gate_mix_bwd_delta(const float* gates, const void* o_cmp, const void* o_slc, const void* o_win,
                                   const void* dout, void* do_cmp, void* do_slc, void* do_win, float* dlogits,
                                   float* delta, int B, int H, int T, int dv, int gate_mode, int dtype,
                                   int dout_token_major, void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * The whole layer between the q/k/v projections and the output projection: the wiring of NSAAttention.forward
 * (nsa/kernels.py:2298-2463) and of its backward, which the reference leaves to autograd, as two calls.
 *   forward   phi -> Eq. 8-11 scoring and top-n -> compressed, sliding-window and selected-block attention ->
 *             gate + mix (epilogue of the selection branch)
 *   backward  gate/mix -> the three branches (dQ summed in fp32 and rounded once) -> phi
 * Tensors are contiguous in the layouts of the branch entry points: q [B,H,T,dk]; every k [B,G,dk,T]; every v
 * [B,G,T,dv]; gate_logits [B,T,3H] fp32; out [B,H,T,dv] or, with out_token_major, [B,T,H,dv]; phi parameters fp32 as
 * for nsa_cmp_phi_fwd.  The three branches may share one k/v pair (pass the same pointers) or have their own
 * (the module's separate projections): k_slc/v_slc feed the selection branch, k_cmp_src/v_cmp_src the compression,
 * k_win/v_win the sliding window.  indices_in (int32 [B,G,T,n], or NULL) replaces the layer's own block choice.
 * `ctx` (nsa_layer_ctx_bytes) receives what the backward needs and what diagnostics want to look at: with
 * offsets != NULL the query also writes the byte offset of every piece (enum below; NSA_CTX_PIECES + 1 values, the
 * last one the total).  `workspace` (nsa_layer_workspace_bytes) is scratch, free again when the call returns.
 * Backward: dq [B,H,T,dk] is overwritten; dk_* [B,G,T,dk] (time-major, like every dK of this library) and dv_*
 * [B,G,T,dv] are ADDED INTO (zero them first; branches that share a k/v pair share its gradient buffers);
 * dlogits [B,T,3H], dpos, dw1, db1, dw2, db2 fp32 are overwritten; dout has out's layout.
 * The query position offset of the long-context mode is not available through these two calls (the sliding-window
 * branch needs a key slice per rank); that mode composes the branch entry points. */
typedef struct nsa_layer_desc {
  int B, H, G, T, dk, dv;
  int U;                 /* hidden width of phi (rows of w1); the reference uses 2*dk */
  int l, d, l_prime, n;  /* compression block and stride, selection block, blocks per query */
  int n_fixed;           /* 3 = initial + two local blocks forced (include_fixed_in_selection), 0 = none */
  int window;
  int gate_mode;         /* NSA_GATE_SIGMOID / NSA_GATE_SOFTMAX */
  int dtype;             /* NSA_F32 / NSA_BF16, of q, k, v, out */
  int out_token_major;
  float scale;
} nsa_layer_desc;
enum nsa_layer_ctx_piece {
  NSA_CTX_O_CMP = 0, NSA_CTX_L_CMP, NSA_CTX_M_CMP, NSA_CTX_O_SLC, NSA_CTX_L_SLC, NSA_CTX_M_SLC, NSA_CTX_O_WIN, NSA_CTX_L_WIN,
  NSA_CTX_M_WIN, NSA_CTX_GATES /* [B,H,T,3] fp32 */, NSA_CTX_INDICES /* int32 [B,G,T,n], all-empty rows already replaced */,
  NSA_CTX_K_CMP /* fp32 [B,G,dk,nbp] */, NSA_CTX_K_CMP_LP, NSA_CTX_V_CMP /* [B,G,nbp,dv] */, NSA_CTX_BLOCK_ENDS /* int32 [nbp] */,
  NSA_CTX_K_CMP_LO /* bf16 remainder of the fp32 compressed keys */, NSA_CTX_LSE2_CMP /* fp32 [B,H,T], log2 units */,
  NSA_CTX_PHI_SAVED, NSA_CTX_PIECES
};
NSA_API size_t nsa_layer_ctx_bytes(const nsa_layer_desc* desc, size_t* offsets);
NSA_API size_t nsa_layer_workspace_bytes(const nsa_layer_desc* desc, int backward);
NSA_API int nsa_layer_fwd(const nsa_layer_desc* desc, const void* q, const void* k_slc, const void* v_slc,
                  const void* k_cmp_src, const void* v_cmp_src, const void* k_win, const void* v_win,
                  const float* gate_logits, const float* pos_embed, const float* w1, const float* b1,
                  const float* w2, const float* b2, const int32_t* indices_in, void* out, void* ctx,
                  size_t ctx_bytes, void* workspace, size_t workspace_bytes, void* stream);
NSA_API int nsa_layer_bwd(const nsa_layer_desc* desc, const void* q, const void* k_slc, const void* v_slc,
                  const void* k_cmp_src, const void* k_win, const void* v_win, const float* pos_embed,
                  const float* w1, const float* w2, const void* ctx, size_t ctx_bytes, const void* dout, void* dq,
                  void* dk_slc, void* dv_slc, void* dk_cmp_src, void* dv_cmp_src, void* dk_win, void* dv_win,
                  float* dlogits, float* dpos, float* dw1, float* db1, float* dw2, float* db2, void* workspace,
                  size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NSA_B200_H */
