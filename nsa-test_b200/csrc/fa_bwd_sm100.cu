// Dense-range flash-attention backward on tcgen05 tensor cores for the sliding-window and compressed
// branches (replaces _nsa_sliding_window_bwd_kernel / _nsa_compression_bwd_kernel,
// nsa/kernels.py:1303-1530, 1690-1917, for bf16 tensors in canonical layouts).
//
// The reference accumulates dK/dV with atomics from every query tile.  Here gradients are produced by
// two stationary kernels, so every output element has one writer and a fixed summation order:
//   prep   D[t] = sum_c O[t,c] dO[t,c] and lse2[t] = (M+L) log2(e)           (HBM-bound, one pass)
//   dQ     query-stationary: S = Q K^T, dP = dO V^T, dS = P*(dP-D) written to tensor memory as bf16,
//          dQ += dS K   (A operand read straight from TMEM)
//   dK/dV  key-stationary, transposed: S^T = K Q^T, dP^T = V dO^T over 64-query sub-tiles of every
//          head of the group; P^T and dS^T stay in TMEM as A operands of dV += P^T dO, dK += dS^T Q.
//          TMEM: dK 192 + dV 128 + S^T 64 + dP^T 64 columns.  Heads may be split over several CTAs
//          (compressed branch, few key tiles): partial sums go to scratch and are added in head order.
#include <algorithm>
#include <cuda.h>

#include <mutex>

#include "attn_args.cuh"
#include "common.cuh"
#include "fa_sm100.cuh"
#include "sm100_ptx.cuh"

namespace nsa {

using namespace ptx;

static int bwd_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

constexpr float kLog2e = 1.4426950408889634f;

struct FaBwdParams {
  const float *D, *lse2;  // [B,H,Tq] from the prep kernel
  __nv_bfloat16 *dq, *dk, *dv;
  float *dk_part, *dv_part;  // [hsplit, B, G, Tk, dk|dv] when hsplit > 1
  int B, H, G, Tq, Tk;
  int window, cmp_l, cmp_d, cmp_nb;
  int hsplit;
  float scale, scale_log2;
  int* timeouts;
  // dS^T tiles handed from the dK/dV kernel to the dQ kernel (null: the dQ kernel recomputes S and dP itself):
  // [B*H][Tk/128 key tiles][ds_per_j sub-tile slots][128 keys][64 queries] bf16, one 16 KiB tile per (key tile, 64-query sub-tile)
  __nv_bfloat16* ds;
  int ds_per_j;
};

// Which 64-query sub-tiles meet key tile j (keys [128 j, 128 j + 128)).  The range is widened to whole 128-query tiles
// (first sub-tile even, last odd; Tq is a multiple of 128), so that the dQ kernel, which works on 128-query tiles, finds
// either both halves of a tile written or neither.  Shared by the dK/dV kernel (writer of the dS^T tiles) and the dQ
// kernel (reader): both must agree on the set of tiles.
template <int MODE>
__host__ __device__ __forceinline__ void subtile_range(int j, int Tq, int window, int cmp_l, int cmp_d, int cmp_nb, int* qs_lo,
                                                       int* qs_hi) {
  const int n0 = j * 128;
  if (MODE == kWin) {
    *qs_lo = n0 / 64;
    const int last = n0 + 126 + window;
    *qs_hi = ((last < Tq - 1 ? last : Tq - 1) / 64) | 1;
  } else {
    const int64_t tfirst = (int64_t)n0 * cmp_d + cmp_l - 1;
    if (n0 < cmp_nb && tfirst < Tq) {
      *qs_lo = (int)((tfirst > 0 ? tfirst : 0) / 64) & ~1;   // tfirst < 0: visible from the first row on
      *qs_hi = (Tq - 1) / 64;
    } else {
      *qs_lo = 1;
      *qs_hi = 0;
    }
  }
}
// slot of sub-tile qs in key tile j's row of the dS^T scratch: the window branch stores only the sub-tiles near the
// diagonal (slot = distance from the first one), the compressed branch all of them
template <int MODE>
__host__ __device__ __forceinline__ int ds_slot(int j, int qs) { return MODE == kWin ? qs - 2 * j : qs; }
static int ds_slots_per_key_tile(int mode, int Tq, int window) { return mode == kWin ? (((126 + window) / 64) | 1) + 1 : Tq / 64; }


// ------------------------------------------------------------------------------------------------
// prep: one warp per (b,h,t)
// ------------------------------------------------------------------------------------------------
__global__ void fa_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                   const float* __restrict__ L, const float* __restrict__ M, float* __restrict__ D,
                                   float* __restrict__ lse2, int64_t rows, int dv) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float acc = 0.f;
  for (int c = lane * 2; c < dv; c += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + row * dv + c));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dout + row * dv + c));
    acc = fmaf(a.x, b.x, fmaf(a.y, b.y, acc));
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    D[row] = acc;
    const float lse = M[row] + L[row];
    lse2[row] = isfinite(lse) ? lse * kLog2e : CUDART_INF_F;  // +inf: exp2(x - inf) = 0 for rows that saw nothing
  }
}

// the row sums dO.O come from the caller: only the log-sum-exp has to be prepared
__global__ void fa_bwd_prep_given_delta_kernel(const float* __restrict__ delta, const float* __restrict__ L, const float* __restrict__ M,
                                               float* __restrict__ D, float* __restrict__ lse2, int64_t rows) {
  const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  D[row] = delta[row];
  const float lse = M[row] + L[row];
  lse2[row] = isfinite(lse) ? lse * kLog2e : CUDART_INF_F;
}

void launch_bwd_prep(const void* o, const void* dout, const float* L, const float* M, const float* delta, float* D, float* lse2,
                     int64_t rows, int dv, cudaStream_t st) {
  KernelTimer kt("bwd_prep", st);
  if (delta)
    fa_bwd_prep_given_delta_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(delta, L, M, D, lse2, rows);
  else
    fa_bwd_prep_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, L, M, D, lse2,
                                                                 rows, dv);
}

// ------------------------------------------------------------------------------------------------
// dQ kernel: 128 queries of one head per CTA
// ------------------------------------------------------------------------------------------------
template <int DK, int DV>
struct DqSmem {
  static constexpr int kQ = 128 * DK * 2, kdO = 128 * DV * 2, kK = 128 * DK * 2, kV = 128 * DV * 2;
  static constexpr int oQ = 0, odO = oQ + kQ, oK = odO + kdO, oV = oK + 2 * kK, oBar = oV + kV;
  static constexpr int kDynamic = oBar + 256 + 1024;
};
struct DqBarriers {
  uint64_t qdo_full, qdo_empty, k_full[2], k_empty[2], v_full, v_empty, sdp_full, sdp_free, ds_full, ds_free, dq_done, dq_free;
  uint32_t tmem_base;
  int abort;
};

// warps 0-3 / 4-7: compute, key columns [0,64) / [64,128) of every tile (same query rows); warp 8 TMA; warp 9 UMMA.
// TMEM: S [0,128) dP [128,256) dQ [256,256+DK) dS (bf16) [256+DK, 320+DK): S/dP of tile j+1 are produced while the
// compute warps turn tile j into dS, and dQ += dS K of tile j runs while they work on tile j+1.
template <int DK, int DV, int MODE>
__global__ void __maxnreg__(200)
fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                 const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const FaBwdParams p) {
  using SM = DqSmem<DK, DV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t *sQ = smem + SM::oQ, *sdO = smem + SM::odO, *sK = smem + SM::oK, *sV = smem + SM::oV;
  DqBarriers* bar = reinterpret_cast<DqBarriers*>(smem + SM::oBar);
  volatile int* abort = &bar->abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Work items: (query tile, batch, head), late (heavy) query tiles first, taken round robin by the CTAs of a persistent
  // grid; every role walks the same list on its own, so the loads and the first S/dP MMAs of an item overlap the dQ
  // epilogue of the one before.
  const int per_qt = p.B * p.H, nqt = p.Tq / 128, nitems = nqt * per_qt;
  // once any block has given up on a wait the device results are void: later blocks skip their work and end at once
  const bool poisoned = p.timeouts && *(volatile const int*)p.timeouts != 0;
  struct Item { int m0, b, h, g, jlo, ntiles; };
  auto item_at = [&](int it) {
    Item w;
    const int qt = nqt - 1 - it / per_qt, y = it % per_qt;
    w.m0 = qt * 128;
    w.b = y / p.H;
    w.h = y % p.H;
    w.g = w.h / (p.H / p.G);
    int jhi;
    if (MODE == kWin) {
      w.jlo = max(0, w.m0 - p.window + 1) / 128;
      jhi = min(w.m0 + 127, p.Tk - 1) / 128;
    } else {
      const int tl = w.m0 + 127;
      const int kmax = tl >= p.cmp_l - 1 ? min(p.cmp_nb - 1, (tl - p.cmp_l + 1) / p.cmp_d) : -1;
      w.jlo = 0;
      jhi = kmax >= 0 ? kmax / 128 : -1;
    }
    w.ntiles = poisoned ? 0 : jhi - w.jlo + 1;
    return w;
  };

  if (threadIdx.x == 0) {
    mbar_init(&bar->qdo_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&bar->k_full[i], 1); mbar_init(&bar->k_empty[i], 1); }
    mbar_init(&bar->v_full, 1);
    mbar_init(&bar->v_empty, 1);
    mbar_init(&bar->sdp_full, 1);
    mbar_init(&bar->sdp_free, 256);
    mbar_init(&bar->ds_full, 256);
    mbar_init(&bar->ds_free, 1);
    mbar_init(&bar->dq_done, 1);
    mbar_init(&bar->qdo_empty, 1);
    mbar_init(&bar->dq_free, 256);
    bar->abort = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 9) tmem_alloc(&bar->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  constexpr uint32_t cS = 0, cdP = 128, cdQ = 256, cdS = 256 + DK;

  if (warp == 8) {
    // TMA producer: warp-uniform loops, one elected lane issues
    bool ok = true;
    int ic = 0, kc = 0;      // items with tiles / key tiles loaded so far by this CTA (barrier phases run on)
    bool q_pending = false;
    for (int it = blockIdx.x; it < nitems && ok; it += gridDim.x) {
      const Item w = item_at(it);
      if (w.ntiles <= 0) continue;
      ok = mbar_wait_warp(&bar->qdo_empty, (ic & 1) ^ 1, abort);   // the S/dP MMAs of the item before have read Q and dO
      if (!ok) break;
      if (elect_one()) {
        mbar_arrive_expect_tx(&bar->qdo_full, SM::kQ + SM::kdO);
        const int qrow = (w.b * p.H + w.h) * p.Tq + w.m0;
        for (int c = 0; c < DK / 64; ++c) tma_load_2d(&tmQ, &bar->qdo_full, sQ + c * 16384, c * 64, qrow);
        for (int c = 0; c < DV / 64; ++c) tma_load_2d(&tmdO, &bar->qdo_full, sdO + c * 16384, c * 64, qrow);
      }
      __syncwarp();
      q_pending = true;
      for (int j = 0; j < w.ntiles && ok; ++j, ++kc) {
        const int n0 = (w.jlo + j) * 128, ks = kc & 1;
        ok = mbar_wait_warp(&bar->k_empty[ks], ((kc >> 1) & 1) ^ 1, abort);
        if (!ok) break;
        if (elect_one()) {
          mbar_arrive_expect_tx(&bar->k_full[ks], SM::kK);
          for (int hf = 0; hf < 2; ++hf)
            tma_load_2d(&tmK, &bar->k_full[ks], sK + ks * SM::kK + hf * (DK * 128), n0 + hf * 64, (w.b * p.G + w.g) * DK);
        }
        __syncwarp();
        ok = mbar_wait_warp(&bar->v_empty, (kc & 1) ^ 1, abort);
        if (!ok) {
          if (lane == 0) mbar_wait(&bar->k_full[ks], (kc >> 1) & 1, abort);
          break;
        }
        if (elect_one()) {
          mbar_arrive_expect_tx(&bar->v_full, SM::kV);
          for (int c = 0; c < DV / 64; ++c)
            tma_load_2d(&tmV, &bar->v_full, sV + c * 16384, c * 64, (w.b * p.G + w.g) * p.Tk + n0);
        }
        __syncwarp();
      }
      if (ok) { ++ic; q_pending = false; }
    }
    if (!ok && lane == 0) {
      // let copies already in flight land before the CTA gives its shared memory back
      if (q_pending) mbar_wait(&bar->qdo_full, ic & 1, abort);
      for (int c = max(0, kc - 2); c < kc; ++c) mbar_wait(&bar->k_full[c & 1], (c >> 1) & 1, abort);
      if (kc > 0) mbar_wait(&bar->v_full, (kc - 1) & 1, abort);
    }
  } else if (warp == 9) {
    // UMMA issuer: warp-uniform loops, one elected lane issues
    constexpr uint32_t idS = idesc_bf16(128, 128, 0, 1);    // Q (K-major) x K tile (MN-major: keys contiguous)
    constexpr uint32_t iddP = idesc_bf16(128, 128, 0, 0);   // dO (K-major) x V tile (K-major: dv contiguous)
    constexpr uint32_t iddQ = idesc_bf16(128, DK, 0, 0);    // dS (TMEM) x K tile read K-major (keys = K dim)
    const uint64_t dQd = smem_desc_sw128(smem_u32(sQ), 16, 1024);
    const uint64_t ddO = smem_desc_sw128(smem_u32(sdO), 16, 1024);
    const uint64_t dVd = smem_desc_sw128(smem_u32(sV), 16, 1024);
    // S and dP of the key tile with running index c (over all items of this CTA)
    auto issue_sdp = [&](int c) -> bool {
      const int ks = c & 1;
      const uint64_t dK_mn = smem_desc_sw128(smem_u32(sK + ks * SM::kK), DK * 128, 1024);
      if (!(mbar_wait_warp(&bar->k_full[ks], (c >> 1) & 1, abort) && mbar_wait_warp(&bar->v_full, c & 1, abort))) return false;
      if (c > 0 && !mbar_wait_warp(&bar->sdp_free, (c - 1) & 1, abort)) return false;  // S/dP of the tile before are in registers
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk)
          umma_ss(tmem + cS, desc_advance(dQd, (kk >> 2) * 16384 + (kk & 3) * 32), desc_advance(dK_mn, kk * 2048), idS, kk > 0);
#pragma unroll
        for (int kk = 0; kk < DV / 16; ++kk)
          umma_ss(tmem + cdP, desc_advance(ddO, (kk >> 2) * 16384 + (kk & 3) * 32),
                  desc_advance(dVd, (kk >> 2) * 16384 + (kk & 3) * 32), iddP, kk > 0);
        umma_commit(&bar->sdp_full);
        umma_commit(&bar->v_empty);
      }
      __syncwarp();
      return true;
    };
    bool ok = true;
    int ic = 0, kc = 0;      // items with tiles / key tiles consumed so far by this CTA
    for (int it = blockIdx.x; it < nitems && ok; it += gridDim.x) {
      const Item w = item_at(it);
      if (w.ntiles <= 0) continue;
      ok = mbar_wait_warp(&bar->qdo_full, ic & 1, abort) && issue_sdp(kc);
      for (int j = 0; j < w.ntiles && ok; ++j) {
        const int ks = (kc + j) & 1;
        const uint64_t dK_k = smem_desc_sw128(smem_u32(sK + ks * SM::kK), 16, 1024);
        if (j + 1 < w.ntiles) ok = issue_sdp(kc + j + 1);
        if (!ok) break;
        if (j == w.ntiles - 1) {
          // every S/dP MMA of this item has been issued: Q and dO may be replaced once they have run
          if (elect_one()) umma_commit(&bar->qdo_empty);
          __syncwarp();
        }
        ok = mbar_wait_warp(&bar->ds_full, (kc + j) & 1, abort);
        if (ok && j == 0) ok = mbar_wait_warp(&bar->dq_free, (ic & 1) ^ 1, abort);  // dQ of the item before was read out
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ts(tmem + cdQ, tmem + cdS + kk * 8, desc_advance(dK_k, (kk >> 2) * (DK * 128) + (kk & 3) * 32), iddQ,
                    (j > 0) || (kk > 0));
          umma_commit(&bar->k_empty[ks]);
          umma_commit(&bar->ds_free);
        }
        __syncwarp();
      }
      if (ok) {
        if (elect_one()) umma_commit(&bar->dq_done);
        __syncwarp();
      }
      kc += w.ntiles;
      ++ic;
    }
  } else {
    const int gsel = warp >> 2;                 // which half of the key columns this thread handles
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    int ic = 0, tc = 0;      // items with tiles / key tiles of earlier items (barrier phases run on)
    for (int it = blockIdx.x; it < nitems; it += gridDim.x) {
    const Item w = item_at(it);
    const int jlo = w.jlo, ntiles = ok ? w.ntiles : 0, t = w.m0 + r;
    const int64_t row = ((int64_t)w.b * p.H + w.h) * p.Tq + t;
    const float lse2 = p.lse2[row], Dr = p.D[row];
    for (int j = 0; j < ntiles && ok; ++j) {
      const int n0 = (jlo + j) * 128 + gsel * 64;   // first key of this thread's columns
      ok = mbar_wait(&bar->sdp_full, (tc + j) & 1, abort);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[2][32], dp[2][32], pk[32];
      tmem_ld32(tmem + lane_base + cS + gsel * 64, sv[0]);
      tmem_ld32(tmem + lane_base + cS + gsel * 64 + 32, sv[1]);
      tmem_ld32(tmem + lane_base + cdP + gsel * 64, dp[0]);
      tmem_ld32(tmem + lane_base + cdP + gsel * 64 + 32, dp[1]);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(&bar->sdp_free);
      int clo, chi;
      if (MODE == kWin) {
        chi = t - n0;
        clo = t - p.window - n0;
      } else {
        const int vis = t >= p.cmp_l - 1 ? min(p.cmp_nb - 1, (t - p.cmp_l + 1) / p.cmp_d) : -1;
        chi = vis - n0;
        clo = -0x40000000;
      }
      const bool allvis = clo < 0 && chi >= 63;
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int c0 = c * 32 + 2 * e;
          float p0 = ex2(fmaf(__uint_as_float(sv[c][2 * e]), p.scale_log2, -lse2));
          float p1 = ex2(fmaf(__uint_as_float(sv[c][2 * e + 1]), p.scale_log2, -lse2));
          if (!allvis) {
            p0 = (c0 > clo && c0 <= chi) ? p0 : 0.f;
            p1 = (c0 + 1 > clo && c0 + 1 <= chi) ? p1 : 0.f;
          }
          __nv_bfloat162 x = __floats2bfloat162_rn(p0 * (__uint_as_float(dp[c][2 * e]) - Dr), p1 * (__uint_as_float(dp[c][2 * e + 1]) - Dr));
          pk[c * 16 + e] = *reinterpret_cast<uint32_t*>(&x);
        }
      if (tc + j > 0) {  // dS of the tile before (of this item or the one before) must have been consumed by its dQ MMAs
        ok = mbar_wait(&bar->ds_free, (tc + j - 1) & 1, abort);
        if (!ok) break;
        tc_fence_after();
      }
      tmem_st32(tmem + lane_base + cdS + gsel * 32, pk);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&bar->ds_full);
    }
    if (ok && ntiles > 0) ok = mbar_wait(&bar->dq_done, ic & 1, abort);
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dst = p.dq + row * DK + gsel * (DK / 2);
      // dQ goes to registers in one go and is handed back at once: the first dQ MMA of the next item may overwrite it
      // while this warp converts and stores.
      uint32_t ov[DK / 64][32];
      if (ntiles > 0) {
#pragma unroll
        for (int c = 0; c < DK / 64; ++c) tmem_ld32(tmem + lane_base + cdQ + gsel * (DK / 2) + c * 32, ov[c]);
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(&bar->dq_free);
      } else {
#pragma unroll
        for (int c = 0; c < DK / 64; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) ov[c][e] = 0;
      }
#pragma unroll
      for (int c = 0; c < DK / 64; ++c) {
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint4 pkt;
          __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(ov[c][e]) * p.scale, __uint_as_float(ov[c][e + 1]) * p.scale);
          __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(ov[c][e + 2]) * p.scale, __uint_as_float(ov[c][e + 3]) * p.scale);
          __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(ov[c][e + 4]) * p.scale, __uint_as_float(ov[c][e + 5]) * p.scale);
          __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(ov[c][e + 6]) * p.scale, __uint_as_float(ov[c][e + 7]) * p.scale);
          pkt.x = *reinterpret_cast<uint32_t*>(&a0); pkt.y = *reinterpret_cast<uint32_t*>(&a1);
          pkt.z = *reinterpret_cast<uint32_t*>(&a2); pkt.w = *reinterpret_cast<uint32_t*>(&a3);
          *reinterpret_cast<uint4*>(dst + c * 32 + e) = pkt;
        }
      }
    }
    if (ntiles > 0) { tc += ntiles; ++ic; }
    }  // items
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && bar->abort) ptx::report_timeout(p.timeouts);
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// dQ from stored dS^T: dQ[128 queries x DK] = sum over key tiles of dS[queries x keys] K[keys x DK].
// The dK/dV kernel has left dS^T (bf16) in scratch memory as [128 keys][64 queries] tiles; here they are the A operand
// straight from shared memory (MN-major: queries contiguous), K tiles the B operand (keys contiguous), so S and dP are
// computed once per step of the backward instead of once per kernel.  HBM-bound: 32 KiB of dS^T per 6.3 MFLOP.
// 192 threads: warps 0-3 read the accumulator out (one query row per thread), warp 4 TMA, warp 5 UMMA.
// Persistent grid over (query tile, batch, head) items, late (long) query tiles first; two accumulators in TMEM, so the
// MMAs of an item run under the epilogue of the one before; dS^T tiles in a ring of four stages, K tiles in a ring of two.
// ------------------------------------------------------------------------------------------------
template <int DK>
struct DqDsSmem {
  static constexpr int kDs = 2 * 128 * 64 * 2, kK = 128 * DK * 2;
  static constexpr int kDsStages = 4, kKStages = 2;
  static constexpr int oDs = 0, oK = oDs + kDsStages * kDs, oBar = oK + kKStages * kK;
  static constexpr int kDynamic = oBar + 256 + 1024;
};
struct DqDsBarriers {
  uint64_t ds_full[4], ds_empty[4], k_full[2], k_empty[2], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort;
};

template <int DK, int MODE>
__global__ void __launch_bounds__(192, 1)
fa_bwd_dq_ds_kernel(const __grid_constant__ CUtensorMap tmDs, const __grid_constant__ CUtensorMap tmK, const FaBwdParams p) {
  using SM = DqDsSmem<DK>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t *sDs = smem + SM::oDs, *sK = smem + SM::oK;
  DqDsBarriers* bar = reinterpret_cast<DqDsBarriers*>(smem + SM::oBar);
  volatile int* abort = &bar->abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_qt = p.B * p.H, nqt = p.Tq / 128, nitems = nqt * per_qt, nkt = p.Tk / 128;
  const bool poisoned = p.timeouts && *(volatile const int*)p.timeouts != 0;
  struct Item { int qt, b, h, g, jlo, ntiles; };
  // key tiles whose widened sub-tile range holds query tile qt: a contiguous run of j ending at jhi
  auto tile_visible = [&](int j, int qt) {
    int lo, hi;
    subtile_range<MODE>(j, p.Tq, p.window, p.cmp_l, p.cmp_d, p.cmp_nb, &lo, &hi);
    return lo <= 2 * qt && 2 * qt + 1 <= hi;
  };
  auto item_at = [&](int it) {
    Item w;
    const int y = it % per_qt;
    w.qt = nqt - 1 - it / per_qt;
    w.b = y / p.H;
    w.h = y % p.H;
    w.g = w.h / (p.H / p.G);
    int jhi;
    if (MODE == kWin) {
      jhi = min(w.qt, nkt - 1);
      w.jlo = jhi;
      while (w.jlo > 0 && tile_visible(w.jlo - 1, w.qt)) --w.jlo;
      if (!tile_visible(jhi, w.qt)) jhi = w.jlo - 1;
    } else {
      // visibility is monotone: key tile j is met from its first visible query tile on
      w.jlo = 0;
      jhi = -1;
      int lo = 0, hi = nkt - 1;
      while (lo <= hi) {   // last j with tile_visible(j, qt)
        const int mid = (lo + hi) >> 1;
        if (tile_visible(mid, w.qt)) { jhi = mid; lo = mid + 1; } else hi = mid - 1;
      }
    }
    w.ntiles = poisoned ? 0 : jhi - w.jlo + 1;
    return w;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) { mbar_init(&bar->ds_full[i], 1); mbar_init(&bar->ds_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->k_full[i], 1); mbar_init(&bar->k_empty[i], 1);
      mbar_init(&bar->acc_full[i], 1); mbar_init(&bar->acc_empty[i], 128);
    }
    bar->abort = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 5) tmem_alloc(&bar->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;

  if (warp == 4) {
    // TMA producer
    bool ok = true;
    int kc = 0;   // key tiles loaded so far by this CTA (ring phases run on across items)
    for (int it = blockIdx.x; it < nitems && ok; it += gridDim.x) {
      const Item w = item_at(it);
      for (int jj = 0; jj < w.ntiles && ok; ++jj, ++kc) {
        const int j = w.jlo + jj, s = kc & 3, ks = kc & 1;
        ok = mbar_wait_warp(&bar->ds_empty[s], ((kc >> 2) & 1) ^ 1, abort);
        if (!ok) break;
        if (elect_one()) {
          const int64_t tile = (((int64_t)w.b * p.H + w.h) * nkt + j) * p.ds_per_j + ds_slot<MODE>(j, 2 * w.qt);
          mbar_arrive_expect_tx(&bar->ds_full[s], SM::kDs);
          tma_load_2d(&tmDs, &bar->ds_full[s], sDs + s * SM::kDs, 0, (int)(tile * 128));
          tma_load_2d(&tmDs, &bar->ds_full[s], sDs + s * SM::kDs + 16384, 0, (int)(tile * 128 + 128));
        }
        __syncwarp();
        ok = mbar_wait_warp(&bar->k_empty[ks], ((kc >> 1) & 1) ^ 1, abort);
        if (!ok) {
          if (lane == 0) mbar_wait(&bar->ds_full[s], (kc >> 2) & 1, abort);
          break;
        }
        if (elect_one()) {
          mbar_arrive_expect_tx(&bar->k_full[ks], SM::kK);
          for (int hf = 0; hf < 2; ++hf)
            tma_load_2d(&tmK, &bar->k_full[ks], sK + ks * SM::kK + hf * (DK * 128), j * 128 + hf * 64, (w.b * p.G + w.g) * DK);
        }
        __syncwarp();
      }
    }
    if (!ok && lane == 0) {
      // let copies already in flight land before the CTA gives its shared memory back
      for (int c = max(0, kc - 4); c < kc; ++c) mbar_wait(&bar->ds_full[c & 3], (c >> 2) & 1, abort);
      for (int c = max(0, kc - 2); c < kc; ++c) mbar_wait(&bar->k_full[c & 1], (c >> 1) & 1, abort);
    }
  } else if (warp == 5) {
    // UMMA issuer
    constexpr uint32_t idesc = idesc_bf16(128, DK, 1, 0);   // dS^T tiles as A (MN-major: queries contiguous) x K tile (K-major)
    bool ok = true;
    int ic = 0, kc = 0;
    for (int it = blockIdx.x; it < nitems && ok; it += gridDim.x) {
      const Item w = item_at(it);
      if (w.ntiles <= 0) continue;
      const int a = ic & 1;
      ok = mbar_wait_warp(&bar->acc_empty[a], ((ic >> 1) & 1) ^ 1, abort);   // the epilogue has read this accumulator out
      for (int jj = 0; jj < w.ntiles && ok; ++jj, ++kc) {
        const int s = kc & 3, ks = kc & 1;
        ok = mbar_wait_warp(&bar->ds_full[s], (kc >> 2) & 1, abort) && mbar_wait_warp(&bar->k_full[ks], (kc >> 1) & 1, abort);
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          const uint64_t dA = smem_desc_sw128(smem_u32(sDs + s * SM::kDs), 16384, 1024);
          const uint64_t dB = smem_desc_sw128(smem_u32(sK + ks * SM::kK), 16, 1024);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(tmem + a * 256, desc_advance(dA, kk * 2048), desc_advance(dB, (kk >> 2) * (DK * 128) + (kk & 3) * 32), idesc,
                    (jj > 0) || (kk > 0));
          umma_commit(&bar->ds_empty[s]);
          umma_commit(&bar->k_empty[ks]);
          if (jj == w.ntiles - 1) umma_commit(&bar->acc_full[a]);
        }
        __syncwarp();
      }
      ++ic;
    }
  } else {
    // epilogue: one query row per thread
    const int r = warp * 32 + lane;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    bool ok = true;
    int ic = 0;
    for (int it = blockIdx.x; it < nitems; it += gridDim.x) {
      const Item w = item_at(it);
      const int ntiles = ok ? w.ntiles : 0;
      const int64_t row = ((int64_t)w.b * p.H + w.h) * p.Tq + w.qt * 128 + r;
      __nv_bfloat16* dst = p.dq + row * DK;
      const int a = ic & 1;
      if (ntiles > 0) {
        ok = mbar_wait(&bar->acc_full[a], (ic >> 1) & 1, abort);
        if (ok) tc_fence_after();
      }
      if (!ok) continue;
#pragma unroll
      for (int c = 0; c < DK / 32; ++c) {
        uint32_t ov[32];
        if (ntiles > 0) {
          tmem_ld32(tmem + lane_base + a * 256 + c * 32, ov);
          tc_wait_ld();
          if (c == DK / 32 - 1) {
            tc_fence_before();
            mbar_arrive(&bar->acc_empty[a]);   // the next item but one may overwrite this accumulator
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) ov[e] = 0;
        }
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint4 pkt;
          __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(ov[e]) * p.scale, __uint_as_float(ov[e + 1]) * p.scale);
          __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(ov[e + 2]) * p.scale, __uint_as_float(ov[e + 3]) * p.scale);
          __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(ov[e + 4]) * p.scale, __uint_as_float(ov[e + 5]) * p.scale);
          __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(ov[e + 6]) * p.scale, __uint_as_float(ov[e + 7]) * p.scale);
          pkt.x = *reinterpret_cast<uint32_t*>(&a0); pkt.y = *reinterpret_cast<uint32_t*>(&a1);
          pkt.z = *reinterpret_cast<uint32_t*>(&a2); pkt.w = *reinterpret_cast<uint32_t*>(&a3);
          *reinterpret_cast<uint4*>(dst + c * 32 + e) = pkt;
        }
      }
      if (ntiles > 0) ++ic;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && bar->abort) ptx::report_timeout(p.timeouts);
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// dK/dV kernel: 128 keys per CTA, loops over (head, 64-query sub-tile); transposed tiles in TMEM.
// 384 threads: warps 0-3 / 4-7 turn the two 32-query halves of S^T, dP^T into P^T, dS^T; warp 8 TMA; warp 9 issues the
// S^T / dP^T products, warp 11 the accumulations; warp 10 stores the dS^T tiles the compute warps stage in shared memory.
// ------------------------------------------------------------------------------------------------
template <int DK, int DV>
struct DkvSmem {
  static constexpr int kK = 128 * DK * 2, kV = 128 * DV * 2, kQs = 64 * DK * 2, kdOs = 64 * DV * 2;
  static constexpr int kStage = kQs + kdOs + 1024;  // + lse2[64], D[64] (512 B, padded to keep 1024 B alignment)
  static constexpr int kStages = 3;
  static constexpr int kDsTile = 128 * 64 * 2;  // one dS^T tile on its way to global memory (128-byte-swizzled rows)
  static constexpr int oK = 0, oV = oK + kK, oStage = oV + kV, oDs = oStage + kStages * kStage, oBar = oDs + kDsTile;
  static constexpr int kDynamic = oBar + 256 + 1024;
};
struct DkvBarriers {
  uint64_t kv_full, full[3], empty[3], stp_full, st_free, pds_full, pds_free, acc_done, dst_ready, dst_free;
  uint32_t tmem_base;
  int abort;
};

template <int DK, int DV, int MODE>
__global__ void __launch_bounds__(384, 1)
fa_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                  const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                  const __grid_constant__ CUtensorMap tmDs, const FaBwdParams p) {
  using SM = DkvSmem<DK, DV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t *sK = smem + SM::oK, *sV = smem + SM::oV, *sSt = smem + SM::oStage;
  DkvBarriers* bar = reinterpret_cast<DkvBarriers*>(smem + SM::oBar);
  volatile int* abort = &bar->abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 128;
  const int hc = blockIdx.y;
  const int b = blockIdx.z / p.G, g = blockIdx.z % p.G;
  const int hpg = p.H / p.G, hper = hpg / p.hsplit;
  const int hbeg = g * hpg + hc * hper;

  // 64-query sub-tiles that can see this key tile
  int qs_lo, qs_hi;
  subtile_range<MODE>(blockIdx.x, p.Tq, p.window, p.cmp_l, p.cmp_d, p.cmp_nb, &qs_lo, &qs_hi);
  const bool poisoned = p.timeouts && *(volatile const int*)p.timeouts != 0;  // a block gave up on a wait earlier: skip
  const int nq = poisoned ? 0 : max(0, qs_hi - qs_lo + 1);
  const int n_it = nq * hper;

  if (threadIdx.x == 0) {
    mbar_init(&bar->kv_full, 1);
    for (int i = 0; i < 3; ++i) { mbar_init(&bar->full[i], 2); mbar_init(&bar->empty[i], 1); }
    mbar_init(&bar->stp_full, 1);
    mbar_init(&bar->st_free, 256);
    mbar_init(&bar->pds_full, 256);
    mbar_init(&bar->pds_free, 1);
    mbar_init(&bar->acc_done, 1);
    mbar_init(&bar->dst_ready, 256);
    mbar_init(&bar->dst_free, 1);
    bar->abort = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 9) tmem_alloc(&bar->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  // fp32 S^T / dP^T tiles and their bf16 successors P^T / dS^T have separate columns, so the next tile's
  // S^T / dP^T can be produced while this tile's P^T / dS^T are still being consumed.  The bf16 columns are laid out per
  // compute group (queries [0,32) and [32,64) of the sub-tile): P^T of the group (16 columns), then its dS^T (16).
  constexpr uint32_t cdK = 0, cdV = DK, cST = DK + DV, cdPT = DK + DV + 64, cPS = DK + DV + 128;

  if (warp == 8) {
    // producer: the whole warp takes part (lanes fill the per-query statistics), one elected lane drives TMA
    if (n_it > 0) {
      if (elect_one()) {
        mbar_arrive_expect_tx(&bar->kv_full, SM::kK + SM::kV);
        for (int hf = 0; hf < 2; ++hf) tma_load_2d(&tmK, &bar->kv_full, sK + hf * (DK * 128), n0 + hf * 64, (b * p.G + g) * DK);
        for (int c = 0; c < DV / 64; ++c) tma_load_2d(&tmV, &bar->kv_full, sV + c * 16384, c * 64, (b * p.G + g) * p.Tk + n0);
      }
      __syncwarp();
      bool ok = true;
      int issued = 0, s = 0, ph = 0, h = hbeg, qs = qs_lo;
      // A stage is held from its load to the end of the accumulations that read it, so with three stages a load's HBM
      // latency (about 3 000 cycles under load) cannot hide behind the other two.  The rows of the iterations ahead are
      // therefore started towards L2 early: the tile loads then find them there.
      constexpr int kAhead = 4;
      int h_pf = hbeg, qs_pf = qs_lo, it_pf = 0;
      auto prefetch_next = [&]() {
        if (it_pf < n_it) {
          const int row = (int)((((int64_t)b * p.H + h_pf) * p.Tq) + qs_pf * 64);
          for (int c = 0; c < DK / 64; ++c) tma_prefetch_2d(&tmQ, c * 64, row);
          for (int c = 0; c < DV / 64; ++c) tma_prefetch_2d(&tmdO, c * 64, row);
          ++it_pf;
          if (++qs_pf > qs_hi) { qs_pf = qs_lo; ++h_pf; }
        }
      };
      if (elect_one())
        for (int k = 0; k < kAhead; ++k) prefetch_next();
      __syncwarp();
      for (int it = 0; it < n_it; ++it) {
        const int tq0 = qs * 64;
        const int64_t qrow = ((int64_t)b * p.H + h) * p.Tq + tq0;
        // the statistics are fetched before the stage is free
        const float s_l0 = p.lse2[qrow + lane], s_l1 = p.lse2[qrow + 32 + lane];
        const float s_d0 = p.D[qrow + lane], s_d1 = p.D[qrow + 32 + lane];
        ok = mbar_wait_warp(&bar->empty[s], ph ^ 1, abort);
        if (!ok) break;
        uint8_t* st = sSt + s * SM::kStage;
        if (elect_one()) {
          mbar_arrive_expect_tx(&bar->full[s], SM::kQs + SM::kdOs);
          for (int c = 0; c < DK / 64; ++c) tma_load_2d(&tmQ, &bar->full[s], st + c * 8192, c * 64, (int)qrow);
          for (int c = 0; c < DV / 64; ++c) tma_load_2d(&tmdO, &bar->full[s], st + SM::kQs + c * 8192, c * 64, (int)qrow);
          prefetch_next();
        }
        float* stat = reinterpret_cast<float*>(st + SM::kQs + SM::kdOs);
        stat[lane] = s_l0;
        stat[32 + lane] = s_l1;
        stat[64 + lane] = s_d0;
        stat[96 + lane] = s_d1;
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar->full[s]);
        issued = it + 1;
        if (++s == 3) { s = 0; ph ^= 1; }
        if (++qs > qs_hi) { qs = qs_lo; ++h; }
      }
      if (!ok && lane == 0) {
        mbar_wait(&bar->kv_full, 0, abort);
        for (int it = max(0, issued - 3); it < issued; ++it) mbar_wait(&bar->full[it % 3], (it / 3) & 1, abort);
      }
    }
  } else if (warp == 9) {
    // UMMA issuer: warp-uniform loop, one elected lane issues
    if (n_it > 0) {
      constexpr uint32_t idST = idesc_bf16(128, 64, 1, 0);    // K tile as A (MN-major: keys contiguous) x Q sub-tile (K-major)
      constexpr uint32_t iddPT = idesc_bf16(128, 64, 0, 0);   // V tile as A (K-major) x dO sub-tile (K-major)
      const uint64_t dKa = smem_desc_sw128(smem_u32(sK), DK * 128, 1024);
      const uint64_t dVa = smem_desc_sw128(smem_u32(sV), 16, 1024);
      // S^T = K Q^T and dP^T = V dO^T of iteration `it`, whose stage is s (phase ph)
      auto issue_st = [&](int it, int s, int ph) -> bool {
        const uint32_t st = smem_u32(sSt + s * SM::kStage);
        const uint64_t dQk = smem_desc_sw128(st, 16, 1024), dOk = smem_desc_sw128(st + SM::kQs, 16, 1024);
        if (!mbar_wait_warp(&bar->full[s], ph, abort)) return false;
        if (it > 0 && !mbar_wait_warp(&bar->st_free, (it - 1) & 1, abort)) return false;  // fp32 tiles of it-1 are in registers
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < DK / 16; ++kk)
            umma_ss(tmem + cST, desc_advance(dKa, kk * 2048), desc_advance(dQk, (kk >> 2) * 8192 + (kk & 3) * 32), idST, kk > 0);
#pragma unroll
          for (int kk = 0; kk < DV / 16; ++kk)
            umma_ss(tmem + cdPT, desc_advance(dVa, (kk >> 2) * 16384 + (kk & 3) * 32),
                    desc_advance(dOk, (kk >> 2) * 8192 + (kk & 3) * 32), iddPT, kk > 0);
          umma_commit(&bar->stp_full);
        }
        __syncwarp();
        return true;
      };
      // every iteration's S^T / dP^T as soon as its rows have landed and the fp32 tiles of the one before are in registers
      bool ok = mbar_wait_warp(&bar->kv_full, 0, abort);
      int s = 0, ph = 0;
      for (int it = 0; it < n_it && ok; ++it) {
        ok = issue_st(it, s, ph);
        if (++s == 3) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 11) {
    // second UMMA issuer: the accumulations dV += P^T dO, dK += dS^T Q.  They read other TMEM columns than the S^T / dP^T
    // products, so the two issuers need no ordering between them and the bookkeeping of one runs under the MMAs of the other.
    if (n_it > 0) {
      constexpr uint32_t iddV = idesc_bf16(128, DV, 0, 1);    // P^T (TMEM) x dO sub-tile (MN-major: dv contiguous)
      constexpr uint32_t iddK = idesc_bf16(128, DK, 0, 1);    // dS^T (TMEM) x Q sub-tile (MN-major: dk contiguous)
      bool ok = true;
      int s = 0;
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t st = smem_u32(sSt + s * SM::kStage);
        const uint64_t dQmn = smem_desc_sw128(st, 8192, 1024), dOmn = smem_desc_sw128(st + SM::kQs, 8192, 1024);
        ok = mbar_wait_warp(&bar->pds_full, it & 1, abort);
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ts(tmem + cdV, tmem + cPS + (kk >> 1) * 32 + (kk & 1) * 8, desc_advance(dOmn, kk * 2048), iddV, (it > 0) || (kk > 0));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ts(tmem + cdK, tmem + cPS + (kk >> 1) * 32 + 16 + (kk & 1) * 8, desc_advance(dQmn, kk * 2048), iddK, (it > 0) || (kk > 0));
          umma_commit(&bar->empty[s]);   // (the S^T / dP^T products that read this stage finished before P^T existed)
          umma_commit(&bar->pds_free);
        }
        __syncwarp();
        if (++s == 3) s = 0;
      }
      if (ok) {
        if (elect_one()) umma_commit(&bar->acc_done);
        __syncwarp();
      }
    }
  } else if (warp == 10) {
    // dS^T tile stores: one tile per iteration leaves through the staging area, off the compute warps' critical path
    if (p.ds && lane == 0) {
      const uint8_t* sDs = smem + SM::oDs;
      int qs = qs_lo - 1, h = hbeg;
      for (int it = 0; it < n_it; ++it) {
        if (++qs > qs_hi) { qs = qs_lo; ++h; }
        if (!mbar_wait(&bar->dst_ready, it & 1, abort)) break;
        const int64_t tile = (((int64_t)b * p.H + h) * gridDim.x + blockIdx.x) * p.ds_per_j + ds_slot<MODE>(blockIdx.x, qs);
        tma_store_2d(&tmDs, sDs, 0, (int)(tile * 128));
        bulk_commit();
        bulk_wait_read<0>();               // the staging area may be overwritten
        mbar_arrive(&bar->dst_free);
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // every tile has landed before the block ends
    }
  } else {
    // warps 0-3 / 4-7: queries [0,32) / [32,64) of every sub-tile, the same 128 key rows
    const int gsel = warp >> 2;
    const int r = (warp & 3) * 32 + lane, key = n0 + r;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    int s = -1, ph = 0, qs = qs_lo - 1, h = hbeg;
    for (int it = 0; it < n_it && ok; ++it) {
      if (++s == 3) { s = 0; ph ^= 1; }
      if (++qs > qs_hi) { qs = qs_lo; ++h; }
      const int tq0 = qs * 64;
      ok = mbar_wait(&bar->full[s], ph, abort) && mbar_wait(&bar->stp_full, it & 1, abort);
      if (!ok) break;
      tc_fence_after();
      const float* stat = reinterpret_cast<const float*>(sSt + s * SM::kStage + SM::kQs + SM::kdOs);
      // visible columns (queries) for this key: clo <= c <= chi
      int clo, chi;
      if (MODE == kWin) {
        clo = key - tq0;
        chi = key + p.window - 1 - tq0;
      } else {
        clo = key < p.cmp_nb ? key * p.cmp_d + p.cmp_l - 1 - tq0 : 0x40000000;
        chi = 0x40000000;
      }
      const bool allvis = clo <= 0 && chi >= 63;  // this key sees all 64 queries of the sub-tile
      uint32_t sT[32], dpT[32];
      tmem_ld32(tmem + lane_base + cST + gsel * 32, sT);
      tmem_ld32(tmem + lane_base + cdPT + gsel * 32, dpT);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(&bar->st_free);   // the fp32 tiles may be overwritten by the next iteration's MMAs
      uint32_t pk[32];  // [0,16): P^T of this group's 32 queries, [16,32): dS^T
#pragma unroll
      for (int e4 = 0; e4 < 8; ++e4) {
        // the statistics of four queries per load (every lane reads the same words: a broadcast)
        const float4 lv = reinterpret_cast<const float4*>(stat)[gsel * 8 + e4];
        const float4 Dv = reinterpret_cast<const float4*>(stat + 64)[gsel * 8 + e4];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int e = 2 * e4 + hf, c0 = gsel * 32 + 2 * e;
          const float l0 = hf ? lv.z : lv.x, l1 = hf ? lv.w : lv.y, D0 = hf ? Dv.z : Dv.x, D1 = hf ? Dv.w : Dv.y;
          float p0 = ex2(fmaf(__uint_as_float(sT[2 * e]), p.scale_log2, -l0));
          float p1 = ex2(fmaf(__uint_as_float(sT[2 * e + 1]), p.scale_log2, -l1));
          if (!allvis) {
            p0 = (c0 >= clo && c0 <= chi) ? p0 : 0.f;
            p1 = (c0 + 1 >= clo && c0 + 1 <= chi) ? p1 : 0.f;
          }
          const float s0 = p0 * (__uint_as_float(dpT[2 * e]) - D0), s1 = p1 * (__uint_as_float(dpT[2 * e + 1]) - D1);
          __nv_bfloat162 x = __floats2bfloat162_rn(p0, p1), y = __floats2bfloat162_rn(s0, s1);
          pk[e] = *reinterpret_cast<uint32_t*>(&x);
          pk[16 + e] = *reinterpret_cast<uint32_t*>(&y);
        }
      }
      if (p.ds) {
        // Hand dS^T to the dQ kernel through a shared-memory tile and ONE tile store (whole 128-byte lines leave the
        // SM; per-thread 16-byte stores at a 128-byte stride cost 32 partial-line writes per warp instruction).  This
        // thread holds its key row x the 32 queries of its group: chunks gsel*4 .. gsel*4+3 of the row, placed where
        // the 128-byte swizzle of the tile store expects them.
        // Every wait is a bounded mbarrier wait (no bar.sync: a thread that gave up elsewhere must not strand the rest).
        uint8_t* sDs = smem + SM::oDs;
        if (it > 0) {  // the store of the tile before has read the staging area
          ok = mbar_wait(&bar->dst_free, (it - 1) & 1, abort);
          if (!ok) break;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int chunk = (gsel * 4 + e) ^ (r & 7);
          *reinterpret_cast<uint4*>(sDs + r * 128 + chunk * 16) = make_uint4(pk[16 + 4 * e], pk[17 + 4 * e], pk[18 + 4 * e], pk[19 + 4 * e]);
        }
        fence_proxy_async();
        mbar_arrive(&bar->dst_ready);      // warp 10 sends the tile off
      }
      // P^T / dS^T of the previous iteration must have been consumed before they are overwritten
      if (it > 0) {
        ok = mbar_wait(&bar->pds_free, (it - 1) & 1, abort);
        if (!ok) break;
        tc_fence_after();
      }
      tmem_st32(tmem + lane_base + cPS + gsel * 32, pk);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&bar->pds_full);
    }
    if (ok && n_it > 0) ok = mbar_wait(&bar->acc_done, 0, abort);
    if (ok) {
      tc_fence_after();
      const int64_t krow = ((int64_t)b * p.G + g) * p.Tk + key;
      auto flush = [&](uint32_t col0, int width, float mul, __nv_bfloat16* out_bf, float* out_part) {
        for (int c = gsel * (width / 64); c < (gsel + 1) * (width / 64); ++c) {   // each compute group flushes half of the columns
          uint32_t ov[32];
          if (n_it > 0) {
            tmem_ld32(tmem + lane_base + col0 + c * 32, ov);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) ov[e] = 0;
          }
          if (out_part) {
            float* dst = out_part + ((int64_t)hc * p.B * p.G * p.Tk + krow) * width + c * 32;
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              *reinterpret_cast<float4*>(dst + e) = make_float4(__uint_as_float(ov[e]) * mul, __uint_as_float(ov[e + 1]) * mul,
                                                                __uint_as_float(ov[e + 2]) * mul, __uint_as_float(ov[e + 3]) * mul);
          } else if (n_it > 0) {
            __nv_bfloat16* dst = out_bf + krow * width + c * 32;
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              __nv_bfloat162 cur = *reinterpret_cast<__nv_bfloat162*>(dst + e);
              const float2 f = __bfloat1622float2(cur);
              cur = __floats2bfloat162_rn(f.x + __uint_as_float(ov[e]) * mul, f.y + __uint_as_float(ov[e + 1]) * mul);
              *reinterpret_cast<__nv_bfloat162*>(dst + e) = cur;
            }
          }
        }
      };
      flush(cdK, DK, p.scale, p.dk, p.hsplit > 1 ? p.dk_part : nullptr);
      flush(cdV, DV, 1.f, p.dv, p.hsplit > 1 ? p.dv_part : nullptr);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && bar->abort) ptx::report_timeout(p.timeouts);
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// out[i] += sum_{c < hsplit} part[c][i], partial sums taken in chunk order
__global__ void dkv_reduce_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int64_t n, int hsplit) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (i >= n) return;
  float a0 = 0.f, a1 = 0.f;
  for (int c = 0; c < hsplit; ++c) {
    const float2 v = *reinterpret_cast<const float2*>(part + (int64_t)c * n + i);
    a0 += v.x;
    a1 += v.y;
  }
  const float2 cur = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(out + i));
  *reinterpret_cast<__nv_bfloat162*>(out + i) = __floats2bfloat162_rn(cur.x + a0, cur.y + a1);
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static size_t al256(size_t x) { return (x + 255) & ~size_t(255); }

static int pick_hsplit(int B, int G, int H, int Tk, int mode) {
  if (mode == kWin) return 1;
  const int hpg = H / G;
  const long ctas = (long)B * G * (Tk / 128);
  int hs = 1;
  while (hs < hpg && ctas * hs < 4 * 148 && hpg % (hs * 2) == 0) hs *= 2;
  return hs;
}

static size_t bwd_base_bytes(int B, int H, int G, int Tq, int Tk, int dk, int dv, int mode) {
  const int hs = pick_hsplit(B, G, H, Tk, mode);
  size_t n = 2 * al256((size_t)B * H * Tq * sizeof(float));
  if (hs > 1) n += al256((size_t)hs * B * G * Tk * dk * sizeof(float)) + al256((size_t)hs * B * G * Tk * dv * sizeof(float));
  return n;
}
// dS^T scratch handed from the dK/dV kernel to the dQ kernel; 0 when it would be unreasonably large (the dQ kernel then
// recomputes S and dP) or its row count would not fit a tensor-map coordinate
constexpr size_t kMaxDsBytes = (size_t)48 << 30;
static size_t bwd_ds_bytes(int B, int H, int Tq, int Tk, int mode, int window) {
  const size_t tiles = (size_t)B * H * (Tk / 128) * ds_slots_per_key_tile(mode, Tq, window);
  const size_t bytes = tiles * 16384;
  if (bytes > kMaxDsBytes || tiles * 128 >= ((size_t)1 << 31)) return 0;
  return bytes;
}

size_t fa_bwd_sm100_workspace_bytes(int B, int H, int G, int Tq, int Tk, int dk, int dv, int mode, int window, bool recompute) {
  const size_t base = bwd_base_bytes(B, H, G, Tq, Tk, dk, dv, mode);
  return base + (recompute ? 0 : bwd_ds_bytes(B, H, Tq, Tk, mode, window));
}

template <int DK, int DV, int MODE>
static int launch_bwd_t(const CUtensorMap& tq128, const CUtensorMap& tdo128, const CUtensorMap& tq64,
                        const CUtensorMap& tdo64, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tds,
                        const FaBwdParams& p, cudaStream_t st) {
  auto kq = fa_bwd_dq_kernel<DK, DV, MODE>;
  auto kqd = fa_bwd_dq_ds_kernel<DK, MODE>;
  auto kkv = fa_bwd_dkv_kernel<DK, DV, MODE>;
  if (cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, DqSmem<DK, DV>::kDynamic) != cudaSuccess ||
      cudaFuncSetAttribute(kqd, cudaFuncAttributeMaxDynamicSharedMemorySize, DqDsSmem<DK>::kDynamic) != cudaSuccess ||
      cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvSmem<DK, DV>::kDynamic) != cudaSuccess)
    return fail(NSA_ERR_LAUNCH, "fa_bwd: cannot reserve shared memory");
  const dim3 qgrid((unsigned)std::min((p.Tq / 128) * p.B * p.H, bwd_sm_count()));
  const dim3 kvgrid(p.Tk / 128, p.hsplit, p.B * p.G);
  if (p.ds) {
    // key-stationary kernel first: it leaves dS^T behind, from which the dQ kernel only has one product left to do
    {
      KernelTimer kt(MODE == kWin ? "fa_bwd_dkv_win" : "fa_bwd_dkv_cmp", st);
      kkv<<<kvgrid, 384, DkvSmem<DK, DV>::kDynamic, st>>>(tq64, tdo64, tk, tv, tds, p);
    }
    if (int rc = check_launch("fa_bwd_dkv_sm100")) return rc;
    KernelTimer kt(MODE == kWin ? "fa_bwd_dqds_win" : "fa_bwd_dqds_cmp", st);
    kqd<<<qgrid, 192, DqDsSmem<DK>::kDynamic, st>>>(tds, tk, p);
    return check_launch("fa_bwd_dq_ds_sm100");
  }
  {
    KernelTimer kt(MODE == kWin ? "fa_bwd_dq_win" : "fa_bwd_dq_cmp", st);
    kq<<<qgrid, 320, DqSmem<DK, DV>::kDynamic, st>>>(tq128, tdo128, tk, tv, p);
  }
  if (int rc = check_launch("fa_bwd_dq_sm100")) return rc;
  KernelTimer kt(MODE == kWin ? "fa_bwd_dkv_win" : "fa_bwd_dkv_cmp", st);
  kkv<<<kvgrid, 384, DkvSmem<DK, DV>::kDynamic, st>>>(tq64, tdo64, tk, tv, tds, p);
  return check_launch("fa_bwd_dkv_sm100");
}

int fa_bwd_sm100(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* L,
                 const float* M, void* dq, void* dk_out, void* dv_out, int B, int H, int G, int Tq, int Tk, int dk, int dv,
                 int mode, int window, int cmp_l, int cmp_d, int cmp_nb, float scale, const float* row_delta,
                 void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (!fa_fwd_sm100_supported(H, G, Tq, Tk, dk, dv)) return fail(NSA_ERR_UNSUPPORTED, "fa_bwd_sm100: unsupported shape");
  if ((int64_t)B * H > 65535) return fail(NSA_ERR_UNSUPPORTED, "fa_bwd_sm100: B*H too large");
  const size_t need = bwd_base_bytes(B, H, G, Tq, Tk, dk, dv, mode);
  if (!workspace || workspace_bytes < need)
    return fail(NSA_ERR_WORKSPACE, "attention backward needs %zu workspace bytes, got %zu", need, workspace_bytes);
  // with room for the dS^T tiles behind the basic scratch, S and dP are computed once (dK/dV kernel) instead of twice
  const size_t ds_bytes = bwd_ds_bytes(B, H, Tq, Tk, mode, window);
  const bool use_ds = ds_bytes > 0 && workspace_bytes >= need + ds_bytes;
  FaBwdParams p;
  char* w = (char*)workspace;
  p.ds = use_ds ? (__nv_bfloat16*)(w + need) : nullptr;
  p.ds_per_j = ds_slots_per_key_tile(mode, Tq, window);
  const size_t rows = (size_t)B * H * Tq;
  float* D = (float*)w;
  float* lse2 = (float*)(w + al256(rows * sizeof(float)));
  p.D = D; p.lse2 = lse2;
  p.hsplit = pick_hsplit(B, G, H, Tk, mode);
  p.dk_part = p.dv_part = nullptr;
  if (p.hsplit > 1) {
    p.dk_part = (float*)(w + 2 * al256(rows * sizeof(float)));
    p.dv_part = (float*)((char*)p.dk_part + al256((size_t)p.hsplit * B * G * Tk * dk * sizeof(float)));
  }
  p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk_out; p.dv = (__nv_bfloat16*)dv_out;
  p.B = B; p.H = H; p.G = G; p.Tq = Tq; p.Tk = Tk;
  p.window = window; p.cmp_l = cmp_l; p.cmp_d = cmp_d; p.cmp_nb = cmp_nb;
  p.scale = scale; p.scale_log2 = scale * kLog2e;
  p.timeouts = fa_timeout_counter();
  launch_bwd_prep(o, dout, L, M, row_delta, D, lse2, (int64_t)rows, dv, st);
  if (int rc = check_launch("fa_bwd_prep")) return rc;
  CUtensorMap tq128, tdo128, tq64, tdo64, tk, tv, tds;
  if (use_ds) {
    if (int rc = make_tmap_bf16_2d(&tds, p.ds, (uint64_t)(ds_bytes / 128), 64, 128)) return rc;
  } else {
    tds = CUtensorMap{};
  }
  if (int rc = make_tmap_bf16_2d(&tq128, q, (uint64_t)B * H * Tq, dk, 128)) return rc;
  if (int rc = make_tmap_bf16_2d(&tdo128, dout, (uint64_t)B * H * Tq, dv, 128)) return rc;
  if (int rc = make_tmap_bf16_2d(&tq64, q, (uint64_t)B * H * Tq, dk, 64)) return rc;
  if (int rc = make_tmap_bf16_2d(&tdo64, dout, (uint64_t)B * H * Tq, dv, 64)) return rc;
  if (int rc = make_tmap_bf16_2d(&tk, k, (uint64_t)B * G * dk, Tk, dk)) return rc;
  if (int rc = make_tmap_bf16_2d(&tv, v, (uint64_t)B * G * Tk, dv, 128)) return rc;
  int rc = NSA_ERR_UNSUPPORTED;
#define NSA_BWD_CASE(DK_, DV_)                                                                               \
  if (dk == DK_ && dv == DV_)                                                                                \
    rc = mode == kWin ? launch_bwd_t<DK_, DV_, kWin>(tq128, tdo128, tq64, tdo64, tk, tv, tds, p, st)         \
                      : launch_bwd_t<DK_, DV_, kCmp>(tq128, tdo128, tq64, tdo64, tk, tv, tds, p, st);
  NSA_BWD_CASE(192, 128)
  NSA_BWD_CASE(128, 128)
  NSA_BWD_CASE(64, 64)
#undef NSA_BWD_CASE
  if (rc) return rc == NSA_ERR_UNSUPPORTED ? fail(rc, "fa_bwd_sm100: unsupported head dims") : rc;
  if (p.hsplit > 1) {
    const int64_t nk = (int64_t)B * G * Tk * dk, nv = (int64_t)B * G * Tk * dv;
    KernelTimer kt("fa_dkv_reduce", st);
    dkv_reduce_kernel<<<(unsigned)((nk / 2 + 255) / 256), 256, 0, st>>>(p.dk_part, p.dk, nk, p.hsplit);
    dkv_reduce_kernel<<<(unsigned)((nv / 2 + 255) / 256), 256, 0, st>>>(p.dv_part, p.dv, nv, p.hsplit);
    return check_launch("dkv_reduce");
  }
  return NSA_OK;
}

// ------------------------------------------------------------------------------------------------
// Sliding-window backward for callers that cannot allocate device memory.
//
// The scratch of the sliding-window backward (per-row D = sum(O*dO) and logsumexp*log2e, two floats per
// (batch, head, query) row) lives in the file-scope device array below instead of a caller-provided
// workspace.  Every GPU that loads this library carries the array (8 MiB) until the process exits.
// ------------------------------------------------------------------------------------------------
constexpr int64_t kNoAllocMaxRows = 1 << 20;  // B*H*T rows the static scratch can hold
static __device__ __align__(256) float g_sliding_bwd_scratch[2 * kNoAllocMaxRows];

// In host code the array's name is only a stand-in; the device address has to be asked for, once per device,
// while that device is current.  Cached per device ordinal.
static int sliding_bwd_scratch_address(float** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static float* cached[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(NSA_ERR_LAUNCH, "sliding_bwd_noalloc: cannot identify the current device");
  std::lock_guard<std::mutex> lk(mu);
  if (!cached[dev]) {
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_sliding_bwd_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(NSA_ERR_LAUNCH, "sliding_bwd_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return NSA_OK;
}

}  // namespace nsa

extern "C" NSA_API int nsa_sliding_bwd_noalloc(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                               const float* L, const float* M, void* dq, void* dkey, void* dval, int B, int H,
                                               int G, int T, int dk, int dv, int window, float scale, void* stream) {
  using namespace nsa;
  NSA_REQUIRE(q && k && v && out && dout && L && M && dq && dkey && dval, "sliding_bwd_noalloc: null pointer");
  NSA_REQUIRE(B > 0 && H > 0 && G > 0 && H % G == 0 && T > 0 && window > 0, "sliding_bwd_noalloc: bad sizes");
  if (!fa_fwd_sm100_supported(H, G, T, T, dk, dv))
    return fail(NSA_ERR_UNSUPPORTED,
                "sliding_bwd_noalloc covers bf16 tensors with head dims (192,128), (128,128) or (64,64), an even number of heads per "
                "group and T a multiple of 128; other shapes run through nsa_sliding_bwd, whose stride-generic kernels need no scratch");
  const int64_t rows = (int64_t)B * H * T;
  if (rows > kNoAllocMaxRows)
    return fail(NSA_ERR_UNSUPPORTED, "sliding_bwd_noalloc: B*H*T = %lld rows exceed the built-in scratch of %lld rows; use "
                "nsa_sliding_bwd with a caller-provided workspace", (long long)rows, (long long)kNoAllocMaxRows);
  const uintptr_t all = (uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out | (uintptr_t)dout | (uintptr_t)dq |
                        (uintptr_t)dkey | (uintptr_t)dval;
  NSA_REQUIRE((all & 15) == 0, "sliding_bwd_noalloc: tensors must be 16-byte aligned");
  float* scratch = nullptr;
  if (int rc = sliding_bwd_scratch_address(&scratch)) return rc;
  // Nothing in the scratch has to start at zero: the preparation kernel overwrites every row this call reads.
  return fa_bwd_sm100(q, k, v, out, dout, L, M, dq, dkey, dval, B, H, G, T, T, dk, dv, kWin, window, 0, 0, 0, scale, nullptr, scratch,
                      sizeof(float) * 2 * kNoAllocMaxRows, (cudaStream_t)stream);
}
