// Selection scoring on tcgen05 tensor cores: Eq. 8 -> 9 -> 10/11 fused, nothing of size [B,H,T,n_cmp]
// leaves the SM (replaces the torch code of nsa/kernels.py:2304-2343, 1920-1962, 1965-2040 for bf16
// queries in the canonical layout, l = 2d, block counts that are multiples of 128).
//
// Bit-exact top-n against an fp32 oracle needs logits far more accurate than bf16 keys give, so the fp32
// compressed keys are split into bf16 hi + lo parts and every logit tile is S = Q K_hi^T + Q K_lo^T
// accumulated in fp32 by the tensor core (16 mantissa bits of K, exact bf16 Q).
// One CTA owns 128 queries of one KV group and makes two passes over (key tile, head):
//   pass A  online (max, sum) of every (query, head) row -> logsumexp
//   pass B  p = exp2(x - lse); per-key sums over the heads of the group (fp32, registers; two compute warpgroups
//           take the even and the odd heads and their sums are added once per key tile);
//           after the last head the l/d x l'/d stencil maps 128 keys to 128/(l'/d) selection-block scores,
//           which go to a [B,G,T,n_sel] scratch buffer (4 bytes per query and block: the only per-block data leaving the SM).
// A second kernel (one warp per query) takes the top n of every row (score descending, ties to the lower id), merges the
// forced blocks in, drops repeats, cuts the list to n and pads it with -1.
#include <cuda.h>

#include "attn_args.cuh"
#include "common.cuh"
#include "fa_sm100.cuh"
#include "sm100_ptx.cuh"

namespace nsa {

using namespace ptx;

constexpr int kScoreMaxN = 32;


struct ScoreParams {
  float* sel;    // [B,G,T,n_sel] selection-block scores (blocks beyond a query tile's last key tile are not written)
  int B, H, G, T, nbp;
  int l, d, lprime, nb, n_sel;
  int q0;        // position of query row 0 in the sequence (query-sharded runs; 0 otherwise)
  float scale_log2;
  int* timeouts;
  const float* lse2_ext;  // [B,H,T] log-sum-exp (log2 units) from the compressed attention's exact forward, or null (own first sweep)
};

__global__ void split_hi_lo_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo,
                                   int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = x[i];
  const __nv_bfloat16 h = __float2bfloat16_rn(v);
  hi[i] = h;
  lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
}

struct ScoreBarriers {
  uint64_t k_full, k_empty, q_full[2], q_empty[2], s_full[2], s_free[2], xchg_full, xchg_free;
  uint32_t tmem_base;
  int abort;
};

template <int DK>
__global__ void __launch_bounds__(384, 1)
score_topn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKhi,
                     const __grid_constant__ CUtensorMap tmKlo, const ScoreParams p, int hpg, int smem_state_off,
                     int smem_bar_off) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  constexpr int kK = 128 * DK * 2, kQ = 128 * DK * 2;
  uint8_t *sKhi = smem, *sKlo = smem + kK, *sQ = smem + 2 * kK;
  float* st_m = reinterpret_cast<float*>(smem + smem_state_off);  // [hpg][128]
  float* st_l = st_m + hpg * 128;                                   // [hpg][128]
  ScoreBarriers* bar = reinterpret_cast<ScoreBarriers*>(smem + smem_bar_off);
  volatile int* abort = &bar->abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = (gridDim.x - 1 - blockIdx.x) * 128;
  const int bg = blockIdx.y, b = bg / p.G, g = bg % p.G;
  const int tl = p.q0 + m0 + 127;
  const int kmax = tl >= p.l - 1 ? min(p.nb - 1, (tl - p.l + 1) / p.d) : -1;
  const int ntiles = max(1, kmax / 128 + 1);
  const int steps_per_pass = ntiles * hpg;
  const int nsteps = (p.lse2_ext ? 1 : 2) * steps_per_pass;   // with the log-sum-exp given, only the probability sweep runs

  if (threadIdx.x == 0) {
    mbar_init(&bar->k_full, 1);
    mbar_init(&bar->k_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->q_full[i], 1);
      mbar_init(&bar->q_empty[i], 1);
      mbar_init(&bar->s_full[i], 1);
      mbar_init(&bar->s_free[i], 128);
    }
    mbar_init(&bar->xchg_full, 128);
    mbar_init(&bar->xchg_free, 128);
    bar->abort = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 9) tmem_alloc(&bar->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  // three warpgroups: 0 and 1 compute (even / odd steps), 2 holds the TMA and UMMA warps.  The compute groups need
  // far more registers than the launch-time split gives them, the third group far fewer.
  if (warp >= 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");

  const bool poisoned = p.timeouts && *(volatile const int*)p.timeouts != 0;  // a block gave up on a wait earlier: skip
  if (warp >= 10 || poisoned) {
    // idle half of the third warpgroup
  } else if (warp == 8) {
    // producer: the warp walks the schedule uniformly, one elected lane issues the copies
    bool ok = true;
    int kissued = 0, qissued = 0;
    int kt = 0, hh = 0;
    for (int step = 0; step < nsteps && ok; ++step) {
      if (hh == 0) {
        const int kidx = kissued;  // K tile loads so far
        ok = mbar_wait_warp(&bar->k_empty, (kidx & 1) ^ 1, abort);
        if (!ok) break;
        if (elect_one()) {
          mbar_arrive_expect_tx(&bar->k_full, 2 * kK);
          for (int hf = 0; hf < 2; ++hf) {
            tma_load_2d(&tmKhi, &bar->k_full, sKhi + hf * (DK * 128), kt * 128 + hf * 64, bg * DK);
            tma_load_2d(&tmKlo, &bar->k_full, sKlo + hf * (DK * 128), kt * 128 + hf * 64, bg * DK);
          }
        }
        __syncwarp();
        kissued = kidx + 1;
      }
      const int s = step & 1;
      ok = mbar_wait_warp(&bar->q_empty[s], ((step >> 1) & 1) ^ 1, abort);
      if (!ok) break;
      if (elect_one()) {
        mbar_arrive_expect_tx(&bar->q_full[s], kQ);
        for (int c = 0; c < DK / 64; ++c)
          tma_load_2d(&tmQ, &bar->q_full[s], sQ + s * kQ + c * 16384, c * 64, (b * p.H + g * hpg + hh) * p.T + m0);
      }
      __syncwarp();
      qissued = step + 1;
      if (++hh == hpg) {
        hh = 0;
        if (++kt == ntiles) kt = 0;  // second pass starts over
      }
    }
    if (!ok && lane == 0) {
      if (kissued > 0) mbar_wait(&bar->k_full, (kissued - 1) & 1, abort);
      for (int st = max(0, qissued - 2); st < qissued; ++st) mbar_wait(&bar->q_full[st & 1], (st >> 1) & 1, abort);
    }
  } else if (warp == 9) {
    // UMMA issuer: warp-uniform loop, one elected lane issues
    constexpr uint32_t idS = idesc_bf16(128, 128, 0, 1);
    const uint64_t dKhi = smem_desc_sw128(smem_u32(sKhi), DK * 128, 1024);
    const uint64_t dKlo = smem_desc_sw128(smem_u32(sKlo), DK * 128, 1024);
    bool ok = true;
    int hh = 0, ktiles = 0;
    for (int step = 0; step < nsteps && ok; ++step) {
      const int s = step & 1;
      if (hh == 0) ok = mbar_wait_warp(&bar->k_full, ktiles & 1, abort);
      ok = ok && mbar_wait_warp(&bar->q_full[s], (step >> 1) & 1, abort);
      ok = ok && mbar_wait_warp(&bar->s_free[s], ((step >> 1) & 1) ^ 1, abort);
      if (!ok) break;
      tc_fence_after();
      const uint64_t dQ = smem_desc_sw128(smem_u32(sQ + s * kQ), 16, 1024);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk)
          umma_ss(tmem + s * 128, desc_advance(dQ, (kk >> 2) * 16384 + (kk & 3) * 32), desc_advance(dKhi, kk * 2048), idS, kk > 0);
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk)
          umma_ss(tmem + s * 128, desc_advance(dQ, (kk >> 2) * 16384 + (kk & 3) * 32), desc_advance(dKlo, kk * 2048), idS, 1);
        umma_commit(&bar->s_full[s]);
        umma_commit(&bar->q_empty[s]);
        if (hh == hpg - 1) umma_commit(&bar->k_empty);
      }
      __syncwarp();
      if (++hh == hpg) {
        hh = 0;
        ++ktiles;
      }
    }
  } else {
    // Group 0 takes the even steps (even heads), group 1 the odd ones; each sums the probabilities of its heads.
    // After its last head of a key tile group 1 parks its sums in TMEM columns [256,384); group 0 adds them to its
    // own, applies the stencil and feeds the top-n list, while group 1 is already on the next tile.
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int wg = warp >> 2;
    const int r = (warp & 3) * 32 + lane, t = m0 + r;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const int tp = p.q0 + t;  // position in the sequence
    const int vis = tp >= p.l - 1 ? min(p.nb - 1, (tp - p.l + 1) / p.d) : -1;  // last visible compressed block
    const int s_ = p.lprime / p.d;   // keys per selection block (a power of two on this path); l / d == 2
    const int smask = s_ - 1, sshift = 31 - __clz(s_);
    const int per_tile = 128 >> sshift;
    float* srow = p.sel + ((int64_t)bg * p.T + t) * p.n_sel;
    bool ok = true;
    for (int hh = wg; hh < hpg; hh += 2) {
      st_m[hh * 128 + r] = -CUDART_INF_F;
      st_l[hh * 128 + r] = 0.f;
    }
    float agg[128];     // pass A: scaled logits of the current tile; pass B: per-key probability sums over heads
    float cur = 0.f;    // running stencil sum of the selection block being assembled
    for (int step = 0; step < nsteps && ok; ++step) {
      const int pass = p.lse2_ext ? 1 : step / steps_per_pass, within = step % steps_per_pass, kt = within / hpg, hh = within % hpg, s = step & 1;
      if ((step & 1) != wg) continue;
      const int n0 = kt * 128;
      const int chi = vis - n0;
      if (pass == 1 && hh == wg) {
#pragma unroll
        for (int i = 0; i < 128; ++i) agg[i] = 0.f;
      }
      ok = mbar_wait(&bar->s_full[s], (step >> 1) & 1, abort);
      if (!ok) break;
      tc_fence_after();
      const bool full = chi >= 127;  // every key of this tile is visible to this row: no per-element mask
      if (pass == 0) {
        // raw logits into agg[], running maximum in scaled (log2) units
        const float m_old = st_m[hh * 128 + r];
        float raw_mx = -CUDART_INF_F;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t sv[32];
          tmem_ld32(tmem + lane_base + s * 128 + c * 32, sv);
          tc_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const float x = (full || c * 32 + e <= chi) ? __uint_as_float(sv[e]) : -CUDART_INF_F;
            agg[c * 32 + e] = x;
            raw_mx = fmaxf(raw_mx, x);
          }
        }
        tc_fence_before();
        mbar_arrive(&bar->s_free[s]);
        if (raw_mx != -CUDART_INF_F) {
          const float mx = fmaxf(m_old, raw_mx * p.scale_log2);
          float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
          for (int i = 0; i < 128; i += 2) {
            sum0 += ex2(fmaf(agg[i], p.scale_log2, -mx));
            sum1 += ex2(fmaf(agg[i + 1], p.scale_log2, -mx));
          }
          st_l[hh * 128 + r] = st_l[hh * 128 + r] * ex2(m_old - mx) + (sum0 + sum1);  // m_old = -inf -> factor 0
          st_m[hh * 128 + r] = mx;
        }
      } else {
        float lse2;
        if (p.lse2_ext) {
          lse2 = p.lse2_ext[((int64_t)b * p.H + g * hpg + hh) * p.T + t];
        } else {
          const float m_h = st_m[hh * 128 + r], l_h = st_l[hh * 128 + r];
          lse2 = l_h > 0.f ? m_h + log2f(l_h) : CUDART_INF_F;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t sv[32];
          tmem_ld32(tmem + lane_base + s * 128 + c * 32, sv);
          tc_wait_ld();
          if (full) {
#pragma unroll
            for (int e = 0; e < 32; ++e) agg[c * 32 + e] += ex2(fmaf(__uint_as_float(sv[e]), p.scale_log2, -lse2));
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              agg[c * 32 + e] += (c * 32 + e <= chi) ? ex2(fmaf(__uint_as_float(sv[e]), p.scale_log2, -lse2)) : 0.f;
          }
        }
        tc_fence_before();
        mbar_arrive(&bar->s_free[s]);
        if (vis < 0 && kt == 0) agg[0] += 1.f;  // a row that sees no block puts all its mass on block 0
        if (wg == 1 && hh == hpg - 1) {
          // park this group's sums for group 0 (the previous tile's must have been picked up)
          if (kt > 0) {
            ok = mbar_wait(&bar->xchg_free, (kt - 1) & 1, abort);
            if (!ok) break;
            tc_fence_after();
          }
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t sv[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) sv[e] = __float_as_uint(agg[c * 32 + e]);
            tmem_st32(tmem + lane_base + 256 + c * 32, sv);
          }
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(&bar->xchg_full);
        }
        if (wg == 0 && hh == hpg - 2) {
          ok = mbar_wait(&bar->xchg_full, kt & 1, abort);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t sv[32];
            tmem_ld32(tmem + lane_base + 256 + c * 32, sv);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) agg[c * 32 + e] += __uint_as_float(sv[e]);
          }
          tc_fence_before();
          mbar_arrive(&bar->xchg_free);
          // Eq. 9 with l = 2d: sel[j] = sum_{m<s_} (A[s_ j + m] + A[s_ j + m + 1]), adds issued in that order.
          // Streaming over the keys: key i ends the previous block when i % s_ == 0 and otherwise enters the
          // current block twice in a row; the block that straddles the tile end is finished by the next tile.
          float* sdst = srow + (n0 >> sshift) - 1;
#pragma unroll
          for (int i = 0; i < 128; ++i) {
            const float av = agg[i];
            if ((i & smask) == 0) {
              if (kt > 0 || i > 0) sdst[i >> sshift] = cur + av;
              cur = av;
            } else {
              cur = (cur + av) + av;
            }
          }
        }
      }
    }
    // the last block's final term lies beyond every visible key: + 0
    if (ok && wg == 0) srow[ntiles * per_tile - 1] = cur;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && bar->abort) ptx::report_timeout(p.timeouts);
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// One warp per query row: top-k of the row's n_sel block scores (score descending, ties to the lower id), then the
// forced blocks first, repeats dropped, cut to n, padded with -1.  Scores of blocks past the last key tile of the
// row's query tile were never written and count as 0.  Lane i owns the ids i, i + 32, ...: PER of them in registers
// (PER * 32 >= n_sel), or the row in shared memory when PER == 0 (any n_sel).
template <int PER>
__global__ void __launch_bounds__(128)
topn_rows_kernel(const float* __restrict__ sel, int32_t* __restrict__ out, int64_t rows, int T, int n_sel, int per_tile, int l,
                 int d, int nb, int lprime, int n, int n_fixed, int q0) {
  extern __shared__ float sm_rows[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;
  if (row >= rows) return;  // warps are independent: no block-wide barrier below
  const int tloc = (int)(row % T), t = q0 + tloc;  // row of the launch, position in the sequence
  const int tl = q0 + (tloc / 128) * 128 + 127;
  const int kmax = tl >= l - 1 ? min(nb - 1, (tl - l + 1) / d) : -1;
  const int lim = min(n_sel, max(1, kmax / 128 + 1) * per_tile);
  const float* src = sel + row * n_sel;
  float* v = sm_rows + warp * n_sel;  // PER == 0 only
  float vr[PER > 0 ? PER : 1];        // PER > 0 only
  const int k_actual = min(n, n_sel);
  int mytop = -1;  // lane r keeps the r-th pick
  if (PER > 0) {
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int j = lane + 32 * i;
      vr[i] = j < lim ? src[j] : (j < n_sel ? 0.f : -CUDART_INF_F);
    }
    // Every lane keeps a sorted list of its next four candidates; the order is (score descending, id ascending).
    // A list is refilled from the lane's registers with the candidates that come after the last one it gave away.
    float b0, b1, b2, b3, last_v = CUDART_INF_F;
    int i0, i1, i2, i3, last_i = -1, cnt = 0;
    auto refill = [&]() {
      b0 = b1 = b2 = b3 = -CUDART_INF_F;
      i0 = i1 = i2 = i3 = 0x7fffffff;
      cnt = 0;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const float x = vr[i];
        const int id = lane + 32 * i;
        const bool after = x < last_v || (x == last_v && id > last_i);
        if (after && x > -CUDART_INF_F && x > b3) {  // ascending id: an equal score never displaces an earlier id
          ++cnt;
          if (x > b2) {
            b3 = b2; i3 = i2;
            if (x > b1) {
              b2 = b1; i2 = i1;
              if (x > b0) { b1 = b0; i1 = i0; b0 = x; i0 = id; }
              else { b1 = x; i1 = id; }
            } else { b2 = x; i2 = id; }
          } else { b3 = x; i3 = id; }
        }
      }
      cnt = min(cnt, 4);
    };
    refill();
    for (int r = 0; r < k_actual; ++r) {
      float wv = b0;
      int wi = i0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, wv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
        if (ov > wv || (ov == wv && oi < wi)) { wv = ov; wi = oi; }
      }
      if (lane == r) mytop = wi;
      const bool mine = (wi & 31) == lane && wi == i0;
      if (mine) {
        last_v = b0; last_i = i0;
        b0 = b1; i0 = i1; b1 = b2; i1 = i2; b2 = b3; i2 = i3; b3 = -CUDART_INF_F; i3 = 0x7fffffff;
        --cnt;
      }
      if (__any_sync(0xffffffffu, mine && cnt == 0)) {
        if (mine && cnt == 0) refill();
      }
    }
  } else {
    float bv = -CUDART_INF_F;
    int bi = 0x7fffffff;
    for (int j = lane; j < n_sel; j += 32) {
      const float x = j < lim ? src[j] : 0.f;
      v[j] = x;
      if (x > bv) { bv = x; bi = j; }
    }
    __syncwarp();
    for (int r = 0; r < k_actual; ++r) {
      float wv = bv;
      int wi = bi;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, wv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
        if (ov > wv || (ov == wv && oi < wi)) { wv = ov; wi = oi; }
      }
      if (lane == r) mytop = wi;
      if ((wi & 31) == lane) {  // the owner retires the pick and looks for its next best
        v[wi] = -CUDART_INF_F;
        bv = -CUDART_INF_F;
        bi = 0x7fffffff;
        for (int j = lane; j < n_sel; j += 32) {
          const float x = v[j];
          if (x > bv) { bv = x; bi = j; }
        }
      }
      __syncwarp();
    }
  }
  int32_t* dst = out + row * n;
  const int nf = n_fixed > 0 ? 3 : 0;
  if (nf + k_actual <= 32) {
    // lane i holds candidate i: the forced blocks, then the picks in order; a candidate equal to an earlier one is dropped
    int cand = -1;
    const int pick = __shfl_sync(0xffffffffu, mytop, (lane - nf) & 31);
    if (lane < nf) cand = lane == 0 ? 0 : (lane == 1 ? (t < lprime ? 0 : (t - lprime) / lprime) : t / lprime);
    else if (lane < nf + k_actual) cand = pick;
    const unsigned same = __match_any_sync(0xffffffffu, cand);
    const bool keep = cand >= 0 && (same & ((1u << lane) - 1u)) == 0;
    const unsigned kept = __ballot_sync(0xffffffffu, keep);
    const int pos = __popc(kept & ((1u << lane) - 1u));
    if (keep && pos < n) dst[pos] = cand;
    const int cnt = min(n, __popc(kept));
    for (int i = cnt + lane; i < n; i += 32) dst[i] = -1;
  } else {
    int res[kScoreMaxN];
    int nres = 0;
    auto push = [&](int id) {
      if (nres >= n) return;
      for (int i = 0; i < nres; ++i)
        if (res[i] == id) return;
      res[nres++] = id;
    };
    if (nf) {
      push(0);
      push(t < lprime ? 0 : (t - lprime) / lprime);
      push(t / lprime);
    }
    for (int i = 0; i < k_actual; ++i) {
      const int id = __shfl_sync(0xffffffffu, mytop, i);
      push(id);
    }
    if (lane == 0)
      for (int i = 0; i < n; ++i) dst[i] = i < nres ? res[i] : -1;
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
bool score_sm100_supported(int H, int G, int T, int dk, int nbp, int l, int d, int lprime, int n) {
  if (!(dk == 192 || dk == 128 || dk == 64) || G <= 0 || H % G != 0) return false;
  const int hpg = H / G;
  if (d <= 0 || l != 2 * d || lprime % d != 0 || hpg % 2 != 0) return false;
  const int s_ = lprime / d;
  const size_t smem = 4 * (size_t)128 * dk * 2 + 2 * (size_t)hpg * 512 + 256 + 1024;
  const size_t rows_smem = 4 * (size_t)(nbp / (s_ > 0 ? s_ : 1)) * sizeof(float);
  return smem <= 227 * 1024 && rows_smem <= 200 * 1024 && T % 128 == 0 && nbp % 128 == 0 && 128 % s_ == 0 && n >= 1 &&
         n <= kScoreMaxN;
}

static size_t al256s(size_t x) { return (x + 255) & ~size_t(255); }

// bf16 hi and lo copies of the compressed keys + the [B,G,T,n_sel] block scores
size_t score_sm100_workspace_bytes(int B, int G, int T, int dk, int nbp, int d, int lprime) {
  const size_t n_sel = (size_t)nbp / (size_t)(lprime / d);
  return 2 * al256s((size_t)B * G * dk * nbp * 2) + al256s((size_t)B * G * T * n_sel * sizeof(float));
}

template <int DK>
static int launch_score_t(const CUtensorMap& tq, const CUtensorMap& thi, const CUtensorMap& tlo, const ScoreParams& p,
                          cudaStream_t st) {
  const int hpg = p.H / p.G;
  const int tiles = 2 * 128 * DK * 2 + 2 * 128 * DK * 2;
  const int state_off = tiles, state_bytes = 2 * hpg * 128 * 4;
  const int bar_off = state_off + state_bytes;
  const int dyn = bar_off + 256 + 1024;
  if (dyn > 227 * 1024) return fail(NSA_ERR_UNSUPPORTED, "score_topn: %d bytes of shared memory needed", dyn);
  auto kern = score_topn_tc_kernel<DK>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn) != cudaSuccess)
    return fail(NSA_ERR_LAUNCH, "score_topn: cannot reserve shared memory");
  KernelTimer kt("score_topn_tc", st);
  kern<<<dim3(p.T / 128, p.B * p.G), 384, dyn, st>>>(tq, thi, tlo, p, hpg, state_off, bar_off);
  return check_launch("score_topn_tc");
}

int score_topn_sm100(const void* q, const float* k_cmp, int32_t* out, int B, int H, int G, int T, int dk, int nbp, int l, int d,
                     int lprime, int nb, int n, int n_fixed, float scale, int q0, const float* lse2, void* workspace,
                     size_t workspace_bytes, cudaStream_t st) {
  if (!score_sm100_supported(H, G, T, dk, nbp, l, d, lprime, n)) return fail(NSA_ERR_UNSUPPORTED, "score_topn_sm100: unsupported shape");
  const size_t need = score_sm100_workspace_bytes(B, G, T, dk, nbp, d, lprime);
  if (!workspace || workspace_bytes < need)
    return fail(NSA_ERR_WORKSPACE, "scoring needs %zu workspace bytes, got %zu", need, workspace_bytes);
  const size_t key_bytes = al256s((size_t)B * G * dk * nbp * 2);
  __nv_bfloat16* hi = (__nv_bfloat16*)workspace;
  __nv_bfloat16* lo = (__nv_bfloat16*)((char*)workspace + key_bytes);
  float* sel = (float*)((char*)workspace + 2 * key_bytes);
  const int64_t nk = (int64_t)B * G * dk * nbp;
  {
    KernelTimer kt("score_split_keys", st);
    split_hi_lo_kernel<<<(unsigned)((nk + 255) / 256), 256, 0, st>>>(k_cmp, hi, lo, nk);
  }
  if (int rc = check_launch("split_hi_lo")) return rc;
  CUtensorMap tq, thi, tlo;
  if (int rc = make_tmap_bf16_2d(&tq, q, (uint64_t)B * H * T, dk, 128)) return rc;
  if (int rc = make_tmap_bf16_2d(&thi, hi, (uint64_t)B * G * dk, nbp, dk)) return rc;
  if (int rc = make_tmap_bf16_2d(&tlo, lo, (uint64_t)B * G * dk, nbp, dk)) return rc;
  const int s_ = lprime / d, n_sel = nbp / s_;
  ScoreParams p;
  p.sel = sel;
  p.q0 = q0;
  p.B = B; p.H = H; p.G = G; p.T = T; p.nbp = nbp; p.l = l; p.d = d; p.lprime = lprime; p.nb = nb; p.n_sel = n_sel;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.timeouts = fa_timeout_counter();
  p.lse2_ext = lse2;
  int rc;
  if (dk == 192) rc = launch_score_t<192>(tq, thi, tlo, p, st);
  else if (dk == 128) rc = launch_score_t<128>(tq, thi, tlo, p, st);
  else rc = launch_score_t<64>(tq, thi, tlo, p, st);
  if (rc) return rc;
  const int64_t rows = (int64_t)B * G * T;
  KernelTimer kt("score_topn_rows", st);
  const unsigned grid = (unsigned)((rows + 3) / 4);
#define NSA_ROWS_CASE(PER_)                                                                                                   \
  topn_rows_kernel<PER_><<<grid, 128, 0, st>>>(sel, out, rows, T, n_sel, 128 / s_, l, d, nb, lprime, n, n_fixed, q0)
  if (n_sel <= 8 * 32) {
    NSA_ROWS_CASE(8);
  } else if (n_sel <= 16 * 32) {
    NSA_ROWS_CASE(16);
  } else if (n_sel <= 32 * 32) {
    NSA_ROWS_CASE(32);
  } else {
    const size_t sm = 4 * (size_t)n_sel * sizeof(float);
    if (cudaFuncSetAttribute(topn_rows_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm) != cudaSuccess)
      return fail(NSA_ERR_LAUNCH, "score_topn: cannot reserve shared memory for the row selection");
    topn_rows_kernel<0><<<grid, 128, sm, st>>>(sel, out, rows, T, n_sel, 128 / s_, l, d, nb, lprime, n, n_fixed, q0);
  }
#undef NSA_ROWS_CASE
  return check_launch("score_topn_rows");
}

}  // namespace nsa



// fp32 -> bf16 pair (hi = the rounded value, lo = the rounded remainder): what the exact compressed-attention forward and
// the scoring kernel take as keys
extern "C" NSA_API int nsa_split_keys_hi_lo(const float* x, void* hi, void* lo, int64_t n, void* stream) {
  NSA_REQUIRE(x && hi && lo && n >= 0, "split_keys_hi_lo: bad arguments");
  if (n == 0) return NSA_OK;
  nsa::split_hi_lo_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo, n);
  return nsa::check_launch("split_keys_hi_lo");
}
