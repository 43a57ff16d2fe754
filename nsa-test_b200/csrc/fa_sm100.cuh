// Tensor-core (tcgen05) attention kernels for sm_100a: parameters and host entry points.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

struct CUtensorMap_st;

namespace nsa {

struct FaFwdParams {
  __nv_bfloat16* o;  // [B,H,Tq,dv] contiguous
  float *L, *M;      // [B,H,Tq] contiguous, may be null
  float* lse2;       // [B,H,Tq] log-sum-exp of the scaled logits in log2 units (+inf for rows that see nothing), may be null
  int B, H, G, Tq, Tk;
  int window;                // sliding window: keys (t-window, t]
  int cmp_l, cmp_d, cmp_nb;  // compressed tokens: key i visible iff i < cmp_nb and i*cmp_d + cmp_l - 1 <= t
  float scale_log2;          // softmax scale times log2(e)
};

// True when the tensor-core forward covers this shape (bf16, canonical contiguous layouts assumed).
bool fa_fwd_sm100_supported(int H, int G, int Tq, int Tk, int dk, int dv);

// q [B,H,Tq,dk], k [B,G,dk,Tk], v [B,G,Tk,dv], o [B,H,Tq,dv]: contiguous bf16.  mode = kWin or kCmp.
// k_lo (compressed branch, or null): low-order bf16 part of the keys, S = Q (k + k_lo)^T; lse2 (or null): receives the
// log-sum-exp in log2 units.
int fa_fwd_sm100(const void* q, const void* k, const void* v, void* o, float* L, float* M, int B, int H, int G, int Tq,
                 int Tk, int dk, int dv, int mode, int window, int cmp_l, int cmp_d, int cmp_nb, float scale,
                 const void* k_lo, float* lse2, cudaStream_t st);

// Backward of the same two branches.  Adds into dk [B,G,Tk,dk] and dv [B,G,Tk,dv] (time-major, bf16),
// overwrites dq [B,H,Tq,dk].  Three launches: delta/lse preparation, a query-stationary dQ kernel and
// a key-stationary dK/dV kernel whose per-head-chunk partial sums are combined in a fixed order.
// row_delta: the row sums dO.O [B,H,Tq] (fp32) when the caller has them already, else null (computed here).
// With room behind the basic scratch for the dS^T tiles (window: the sliding window, needed to size them), the dK/dV
// kernel hands dS^T to the dQ kernel and S, dP are computed once per step; `recompute` asks for the basic scratch only
// (the dQ kernel then recomputes S and dP).  fa_bwd_sm100 picks the path from the size of the workspace it is given.
size_t fa_bwd_sm100_workspace_bytes(int B, int H, int G, int Tq, int Tk, int dk, int dv, int mode, int window, bool recompute);
int fa_bwd_sm100(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* L,
                 const float* M, void* dq, void* dk_out, void* dv_out, int B, int H, int G, int Tq, int Tk, int dk, int dv,
                 int mode, int window, int cmp_l, int cmp_d, int cmp_nb, float scale, const float* row_delta,
                 void* workspace, size_t workspace_bytes, cudaStream_t st);

// bf16 row-major [rows, cols] matrix -> tensor map with box [box_rows, 64 columns], 128-byte swizzle
int make_tmap_bf16_2d(::CUtensorMap_st* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

// head-major bf16 rows [heads_total][T][width] -> rank-5 map, box = one token's rows of `heads` consecutive heads as
// [heads/8][width/64][8][64], 128-byte swizzle; coordinates (0, 0, 0, first_head / 8, token)
int make_tmap_head_rows(::CUtensorMap_st* map, const void* base, uint64_t heads_total, uint64_t T, uint32_t heads, uint32_t width);

// Fused selection scoring (Eq. 8-11) on tensor cores; see score_sm100.cu.  k_cmp fp32 [B,G,dk,nbp] contiguous,
// q bf16 [B,H,T,dk] contiguous, compressed block i ends at i*d + l - 1 for i < nb and is never visible beyond.
bool score_sm100_supported(int H, int G, int T, int dk, int nbp, int l, int d, int lprime, int n);
size_t score_sm100_workspace_bytes(int B, int G, int T, int dk, int nbp, int d, int lprime);
// lse2 (or null): the log-sum-exp [B,H,T] (log2 units, +inf for rows without a visible block) of the scaled logits over
// the visible compressed blocks, when the caller has it from the compressed attention's forward with hi + lo keys; the
// kernel then skips its own first sweep.
int score_topn_sm100(const void* q, const float* k_cmp, int32_t* out, int B, int H, int G, int T, int dk, int nbp, int l, int d,
                     int lprime, int nb, int n, int n_fixed, float scale, int q0, const float* lse2, void* workspace,
                     size_t workspace_bytes, cudaStream_t st);

// Device address (on the current device) of the counter of CTAs that gave up on a barrier wait; the first call on a
// device sets up that device's time-out record (null on failure).
int* fa_timeout_counter();
// True once any CTA on any device has given up on a wait since the last reset (read from mapped host memory: no
// synchronisation).
bool timeout_flagged();
// One warp waits `limit_clocks` on a barrier nothing arrives at and reports the time-out like a product kernel would;
// *gave_up_dev (device int, may be null) is set to 1 when the wait ran out.
int wait_timeout_selftest(long long limit_clocks, int* gave_up_dev, cudaStream_t st);

// Number of CTAs that ever gave up on a barrier wait (0 in a healthy run); optionally reset.
int fa_fwd_sm100_timeouts(int* count, bool reset);

}  // namespace nsa
