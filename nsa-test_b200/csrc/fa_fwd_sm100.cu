// Dense-range flash-attention forward on 5th-generation tensor cores (tcgen05 + TMEM + TMA), used by
// the sliding-window branch and the compressed-token branch of NSA
// (replaces _nsa_sliding_window_fwd_kernel / _nsa_compression_fwd_kernel, nsa/kernels.py:1151-1300,
// 1533-1687, for bf16 tensors in their canonical layouts).
//
// One CTA owns 128 consecutive queries of TWO heads of the same KV group, so every K/V tile staged in
// shared memory feeds two 128-row MMA tiles.  Roles (warp-specialised, 320 threads):
//   warps 0-3 / 4-7  softmax of tile 0 / tile 1: one thread per query row, fp32 online softmax in the
//                    log2 domain, lazy rescaling of O (only when the row maximum grows by > 2^8)
//   warp 8           TMA producer: Q once, then a 2-deep ring of K tiles and a 1-deep V buffer
//   warp 9           UMMA issuer: S_i = Q_i K^T (SS form, K is MN-major in smem), O_i += P_i V
//                    (TS form: P is read straight from tensor memory where it aliases S_i)
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_i = bf16 pairs in S_i[0,64).
// Issue order PV0(j) QK0(j+1) PV1(j) QK1(j+1) keeps the tensor pipe busy while the other tile's
// softmax runs.  All waits are bounded; a timeout raises a device flag readable from the host.
#include <algorithm>
#include <cuda.h>

#include "attn_args.cuh"
#include <mutex>

#include "common.cuh"
#include "fa_sm100.cuh"
#include "sm100_ptx.cuh"

namespace nsa {

using namespace ptx;

static __device__ TimeoutRecord g_timeout_record;  // CTAs that gave up on a barrier wait (count 0 in every healthy run)

constexpr int kBM = 128;  // queries per MMA tile
constexpr int kBN = 128;  // keys per tile
constexpr int kFaThreads = 384;  // 8 softmax warps, producer, UMMA issuer, 2 idle warps completing the third warpgroup
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.f;  // log2 units

template <int DK, int DV>
struct FaSmem {
  static constexpr int kQBytes = kBM * DK * 2;
  static constexpr int kKBytes = kBN * DK * 2;
  static constexpr int kVBytes = kBN * DV * 2;
  static constexpr int kKStages = 2;
  static constexpr int oQ = 0;
  static constexpr int oK = oQ + 2 * kQBytes;
  static constexpr int oV = oK + kKStages * kKBytes;
  static constexpr int oBar = oV + kVBytes;
  static constexpr int kTotal = oBar + 256;
  static constexpr int kDynamic = kTotal + 1024;  // slack to align the base to 1024 B (swizzle atom)
};

struct FaBarriers {
  uint64_t q_full, q_empty, k_full[2], k_empty[2], v_full, v_empty, s_full[2], p_full[2], pv_done[2], o_free[2];
  uint32_t tmem_base;
  int abort;
};

// visible columns of a row inside the current key tile: clo < c <= chi
template <int MODE>
__device__ __forceinline__ void row_bounds(const FaFwdParams& p, int t, int n0, int& clo, int& chi) {
  if (MODE == kWin) {
    chi = t - n0;
    clo = t - p.window - n0;
  } else {
    const int vis = t >= p.cmp_l - 1 ? min(p.cmp_nb - 1, (t - p.cmp_l + 1) / p.cmp_d) : -1;
    chi = vis - n0;
    clo = -0x40000000;
  }
}

// EXACT (compressed branch only): the keys come as a bf16 pair hi + lo whose sum is the fp32 key to 16 mantissa bits; S =
// Q K_hi^T + Q K_lo^T, so the log-sum-exp this kernel emits (lse2, log2 units) is the one the selection scoring needs and
// that kernel can skip its own first sweep.  The two K stages then hold the hi and the lo part of ONE tile (the next
// tile's keys are fetched while the softmax warps work, once both heads' S MMAs have read the current ones).
template <int DK, int DV, int MODE, bool EXACT>
__global__ void __launch_bounds__(kFaThreads, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmKlo, const FaFwdParams p) {
  using SM = FaSmem<DK, DV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem + SM::oQ;
  uint8_t* sK = smem + SM::oK;
  uint8_t* sV = smem + SM::oV;
  FaBarriers* bar = reinterpret_cast<FaBarriers*>(smem + SM::oBar);
  volatile int* abort = &bar->abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hpg = p.H / p.G;
  // Work items: (query tile, batch, head pair), late (heavy) query tiles first; the CTAs of the persistent grid take
  // them round robin, and every role below walks the same item list on its own, so that the loads and the first
  // S MMAs of an item run while the softmax warps are still in the epilogue of the one before.
  const int pairs = p.H / 2, per_qt = p.B * pairs, nqt = p.Tq / kBM;
  const int nitems = nqt * per_qt;
  // once any block has given up on a wait the device results are void: later blocks skip their work and end at once
  const bool poisoned = *(volatile const int*)&g_timeout_record.count != 0;
  struct Item { int m0, b, h0, g, jlo, ntiles; };
  auto item_at = [&](int it) {
    Item w;
    const int qt = nqt - 1 - it / per_qt, y = it % per_qt;
    w.m0 = qt * kBM;
    w.b = y / pairs;
    w.h0 = (y % pairs) * 2;
    w.g = w.h0 / hpg;
    int jhi;
    if (MODE == kWin) {
      w.jlo = max(0, w.m0 - p.window + 1) / kBN;
      jhi = min(w.m0 + kBM - 1, p.Tk - 1) / kBN;
    } else {
      const int tl = w.m0 + kBM - 1;
      const int kmax = tl >= p.cmp_l - 1 ? min(p.cmp_nb - 1, (tl - p.cmp_l + 1) / p.cmp_d) : -1;
      w.jlo = 0;
      jhi = kmax >= 0 ? kmax / kBN : -1;
    }
    w.ntiles = poisoned ? 0 : jhi - w.jlo + 1;
    return w;
  };

  // K stage and barrier phase of the tile with running index c: two alternating stages, or (EXACT) one double-width stage
  auto kslot = [](int c) { return EXACT ? 0 : (c & 1); };
  auto kphase = [](int c) { return EXACT ? (c & 1) : ((c >> 1) & 1); };

  if (threadIdx.x == 0) {
    mbar_init(&bar->q_full, 1);
    mbar_init(&bar->q_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->o_free[i], 128);
      mbar_init(&bar->k_full[i], 1);
      mbar_init(&bar->k_empty[i], 1);
      mbar_init(&bar->s_full[i], 1);
      mbar_init(&bar->p_full[i], 128);
      mbar_init(&bar->pv_done[i], 1);
    }
    mbar_init(&bar->v_full, 1);
    mbar_init(&bar->v_empty, 1);
    bar->abort = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 9) tmem_alloc(&bar->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  // the softmax warpgroups need more registers than an even split gives them, the third warpgroup far fewer
  if (warp >= 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");

  if (warp >= 10) {
    // idle half of the third warpgroup
  } else if (warp == 8) {
    // ------------------------------------------------------------ TMA producer (warp-uniform loops, one elected lane issues)
    if (elect_one()) {
      prefetch_tensormap(&tmQ);
      prefetch_tensormap(&tmK);
      prefetch_tensormap(&tmV);
    }
    __syncwarp();
    bool ok = true;
    int ic = 0, kc = 0;        // items with tiles / key tiles loaded so far by this CTA (barrier phases run on)
    bool q_pending = false;
    for (int it = blockIdx.x; it < nitems && ok; it += gridDim.x) {
      const Item w = item_at(it);
      if (w.ntiles <= 0) continue;
      ok = mbar_wait_warp(&bar->q_empty, (ic & 1) ^ 1, abort);   // the S MMAs of the item before have read Q
      if (!ok) break;
      if (elect_one()) {
        mbar_arrive_expect_tx(&bar->q_full, 2 * SM::kQBytes);
        for (int i = 0; i < 2; ++i)
          for (int c = 0; c < DK / 64; ++c)
            tma_load_2d(&tmQ, &bar->q_full, sQ + i * SM::kQBytes + c * (kBM * 128), c * 64,
                        (w.b * p.H + w.h0 + i) * p.Tq + w.m0);
      }
      __syncwarp();
      q_pending = true;
      for (int j = 0; j < w.ntiles && ok; ++j, ++kc) {
        const int n0 = (w.jlo + j) * kBN, ks = kslot(kc);
        ok = mbar_wait_warp(&bar->k_empty[ks], kphase(kc) ^ 1, abort);
        if (!ok) break;
        if (elect_one()) {
          mbar_arrive_expect_tx(&bar->k_full[ks], EXACT ? 2 * SM::kKBytes : SM::kKBytes);
          for (int hf = 0; hf < 2; ++hf)
            tma_load_2d(&tmK, &bar->k_full[ks], sK + ks * SM::kKBytes + hf * (DK * 128), n0 + hf * 64, (w.b * p.G + w.g) * DK);
          if (EXACT)
            for (int hf = 0; hf < 2; ++hf)
              tma_load_2d(&tmKlo, &bar->k_full[ks], sK + SM::kKBytes + hf * (DK * 128), n0 + hf * 64, (w.b * p.G + w.g) * DK);
        }
        __syncwarp();
        ok = mbar_wait_warp(&bar->v_empty, (kc & 1) ^ 1, abort);
        if (!ok) {
          if (lane == 0) mbar_wait(&bar->k_full[ks], kphase(kc), abort);
          break;
        }
        if (elect_one()) {
          mbar_arrive_expect_tx(&bar->v_full, SM::kVBytes);
          for (int c = 0; c < DV / 64; ++c)
            tma_load_2d(&tmV, &bar->v_full, sV + c * (kBN * 128), c * 64, (w.b * p.G + w.g) * p.Tk + n0);
        }
        __syncwarp();
      }
      if (ok) { ++ic; q_pending = false; }
    }
    if (!ok && lane == 0) {
      // let copies already in flight land before the CTA gives its shared memory back
      if (q_pending) mbar_wait(&bar->q_full, ic & 1, abort);
      for (int c = max(0, kc - (EXACT ? 1 : 2)); c < kc; ++c) mbar_wait(&bar->k_full[kslot(c)], kphase(c), abort);
      if (kc > 0) mbar_wait(&bar->v_full, (kc - 1) & 1, abort);
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------ UMMA issuer (warp-uniform loops, one elected lane issues)
    constexpr uint32_t idQK = idesc_bf16(kBM, kBN, 0, 1);
    constexpr uint32_t idPV = idesc_bf16(kBM, DV, 0, 1);
    const uint64_t dQ0 = smem_desc_sw128(smem_u32(sQ), 16, 1024);
    const uint64_t dK0 = smem_desc_sw128(smem_u32(sK), DK * 128, 1024);
    const uint64_t dV = smem_desc_sw128(smem_u32(sV), kBN * 128, 1024);
    // issue S_i = Q_i K^T for key slot ks; called by the elected lane only
    auto issue_qk = [&](int i, int ks) {
      const uint64_t dQ = desc_advance(dQ0, i * SM::kQBytes), dK = desc_advance(dK0, ks * SM::kKBytes);
#pragma unroll
      for (int kk = 0; kk < DK / 16; ++kk)
        umma_ss(tmem + i * 128, desc_advance(dQ, (kk >> 2) * (kBM * 128) + (kk & 3) * 32), desc_advance(dK, kk * 2048), idQK,
                kk > 0);
      if (EXACT) {
        const uint64_t dKl = desc_advance(dK0, SM::kKBytes);
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk)
          umma_ss(tmem + i * 128, desc_advance(dQ, (kk >> 2) * (kBM * 128) + (kk & 3) * 32), desc_advance(dKl, kk * 2048), idQK, 1);
      }
      umma_commit(&bar->s_full[i]);
    };
    bool ok = true;
    int ic = 0, kc = 0;        // items with tiles / key tiles consumed so far by this CTA
    for (int it = blockIdx.x; it < nitems && ok; it += gridDim.x) {
      const Item w = item_at(it);
      if (w.ntiles <= 0) continue;
      ok = mbar_wait_warp(&bar->q_full, ic & 1, abort) && mbar_wait_warp(&bar->k_full[kslot(kc)], kphase(kc), abort);
      if (!ok) break;
      tc_fence_after();
      if (elect_one()) {
        issue_qk(0, kslot(kc));
        issue_qk(1, kslot(kc));
        umma_commit(&bar->k_empty[kslot(kc)]);
      }
      __syncwarp();
      for (int j = 0; j < w.ntiles && ok; ++j, ++kc) {
        const bool more = j + 1 < w.ntiles;
        if (!more) {
          // every S MMA of this item has been issued: Q may be replaced once they have run
          if (elect_one()) umma_commit(&bar->q_empty);
          __syncwarp();
        }
        ok = mbar_wait_warp(&bar->v_full, kc & 1, abort);
        for (int i = 0; i < 2 && ok; ++i) {
          ok = mbar_wait_warp(&bar->p_full[i], kc & 1, abort);
          if (ok && j == 0) ok = mbar_wait_warp(&bar->o_free[i], (ic & 1) ^ 1, abort);  // O_i of the item before was read out
          if (!ok) break;
          const int ks = kslot(kc + 1);
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < kBN / 16; ++kk)
              umma_ts(tmem + 256 + i * 128, tmem + i * 128 + kk * 8, desc_advance(dV, kk * 2048), idPV, (j > 0) || (kk > 0));
            umma_commit(&bar->pv_done[i]);
            if (i == 1) umma_commit(&bar->v_empty);
          }
          __syncwarp();
          if (more) {
            if (i == 0) {
              ok = mbar_wait_warp(&bar->k_full[ks], kphase(kc + 1), abort);
              if (!ok) break;
              tc_fence_after();
            }
            if (elect_one()) {
              issue_qk(i, ks);
              if (i == 1) umma_commit(&bar->k_empty[ks]);
            }
            __syncwarp();
          }
        }
      }
      ++ic;
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue, one row per thread
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int i = warp >> 2;                   // which MMA tile / head
    const int r = (warp & 3) * 32 + lane;      // row inside the tile == TMEM lane
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_base + i * 128;
    const uint32_t tO = tmem + lane_base + 256 + i * 128;
    bool ok = true;
    int tc = 0;                                // key tiles of earlier items (barrier phases run on)
    uint32_t sv[4][32];
    for (int it = blockIdx.x; it < nitems; it += gridDim.x) {
    const Item w = item_at(it);
    const int m0 = w.m0, b = w.b, h0 = w.h0, jlo = w.jlo, ntiles = ok ? w.ntiles : 0;
    const int t = m0 + r;
    float m_true = -CUDART_INF_F, m_ref = -CUDART_INF_F, l = 0.f;
    for (int j = 0; j < ntiles && ok; ++j) {
      const int n0 = (jlo + j) * kBN;
      ok = mbar_wait(&bar->s_full[i], (tc + j) & 1, abort);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, sv[c]);
      tc_wait_ld();
      // does this tile need element masks?
      bool full;
      if (MODE == kWin) {
        full = (n0 + kBN - 1 <= m0) && (n0 > m0 + kBM - 1 - p.window);
      } else {
        full = (n0 + kBN - 1 < p.cmp_nb) && ((n0 + kBN - 1) * p.cmp_d + p.cmp_l - 1 <= m0);
      }
      float mx = -CUDART_INF_F;
      if (full) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const float x = __uint_as_float(sv[c][e]) * p.scale_log2;
            sv[c][e] = __float_as_uint(x);
            mx = fmaxf(mx, x);
          }
      } else {
        int clo, chi;
        row_bounds<MODE>(p, t, n0, clo, chi);
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int col = c * 32 + e;
            const float x = (col > clo && col <= chi) ? __uint_as_float(sv[c][e]) * p.scale_log2 : -CUDART_INF_F;
            sv[c][e] = __float_as_uint(x);
            mx = fmaxf(mx, x);
          }
      }
      m_true = fmaxf(m_true, mx);
      // lazy rescale: move the reference maximum only when the true one ran away from it
      const bool grow = m_true > m_ref + kRescaleThreshold;  // also true on the first finite maximum
      const bool need_o = grow && m_ref != -CUDART_INF_F;
      if (__any_sync(0xffffffffu, need_o)) {
        ok = mbar_wait(&bar->pv_done[i], (tc + j - 1) & 1, abort);  // O_i must hold PV(j-1) before it is scaled
        if (!ok) break;
        tc_fence_after();
        const float f = need_o ? ex2(m_ref - m_true) : 1.f;
        l *= f;
#pragma unroll
        for (int c = 0; c < DV / 32; ++c) {
          uint32_t ov[32];
          tmem_ld32(tO + c * 32, ov);
          tc_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * f);
          tmem_st32(tO + c * 32, ov);
        }
        tc_wait_st();
      }
      if (grow) m_ref = m_true;
      const float mref_use = m_ref == -CUDART_INF_F ? 0.f : m_ref;
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int cc = c * 2 + (e >> 4), ee = (e & 15) * 2;
          const float p0 = ex2(__uint_as_float(sv[cc][ee]) - mref_use);
          const float p1 = ex2(__uint_as_float(sv[cc][ee + 1]) - mref_use);
          rs += p0 + p1;
          __nv_bfloat162 v2 = __floats2bfloat162_rn(p0, p1);  // .x (low half) = even key
          pk[e] = *reinterpret_cast<uint32_t*>(&v2);
        }
        tmem_st32(tS + c * 32, pk);
      }
      l += rs;
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&bar->p_full[i]);
    }
    // epilogue
    const int h = h0 + i;
    const int64_t row = ((int64_t)b * p.H + h) * p.Tq + t;
    __nv_bfloat16* orow = p.o + row * DV;
    if (ok && ntiles > 0) ok = mbar_wait(&bar->pv_done[i], (tc + ntiles - 1) & 1, abort);
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      // O_i goes to registers in one go (the score registers are free by now) and is handed back at once: the first
      // PV of the next item may overwrite it while this warp converts and stores.
      uint32_t ov[DV / 32][32];
      if (ntiles > 0) {
#pragma unroll
        for (int c = 0; c < DV / 32; ++c) tmem_ld32(tO + c * 32, ov[c]);
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(&bar->o_free[i]);
      } else {
#pragma unroll
        for (int c = 0; c < DV / 32; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) ov[c][e] = 0;
      }
#pragma unroll
      for (int c = 0; c < DV / 32; ++c) {
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint4 pkt;
          __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(ov[c][e]) * inv, __uint_as_float(ov[c][e + 1]) * inv);
          __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(ov[c][e + 2]) * inv, __uint_as_float(ov[c][e + 3]) * inv);
          __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(ov[c][e + 4]) * inv, __uint_as_float(ov[c][e + 5]) * inv);
          __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(ov[c][e + 6]) * inv, __uint_as_float(ov[c][e + 7]) * inv);
          pkt.x = *reinterpret_cast<uint32_t*>(&a0);
          pkt.y = *reinterpret_cast<uint32_t*>(&a1);
          pkt.z = *reinterpret_cast<uint32_t*>(&a2);
          pkt.w = *reinterpret_cast<uint32_t*>(&a3);
          *reinterpret_cast<uint4*>(orow + c * 32 + e) = pkt;
        }
      }
      if (p.L) p.L[row] = l > 0.f ? logf(l) + (m_ref - m_true) * kLn2 : -CUDART_INF_F;
      if (p.M) p.M[row] = m_true * kLn2;  // back from log2 units to the natural-log scale of the logits
      if (p.lse2) p.lse2[row] = l > 0.f ? m_ref + log2f(l) : CUDART_INF_F;   // log-sum-exp in log2 units (+inf: the row saw nothing)
    }
    tc += ntiles;
    }  // items
  }

  // ------------------------------------------------------------ teardown (every thread gets here)
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && bar->abort) report_timeout(&g_timeout_record.count);
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

// bf16 row-major [rows, cols] matrix, box [box_rows, 64 cols] (128 B inner extent), 128-byte swizzle
int make_tmap_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(NSA_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(NSA_ERR_LAUNCH, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return NSA_OK;
}

// Head-major rows [heads_total][T][width] (bf16, contiguous) -> rank-5 map whose box is one token's rows of `heads`
// consecutive heads (a multiple of 8, starting at a multiple of 8), delivered as [heads/8][width/64][8 rows][64 columns]
// with 128-byte swizzle: every 8-row x 128-byte swizzle atom of the (token, head group) in one copy, the atoms of a row
// group next to each other.  Coordinates: (0, 0, 0, first_head / 8, token).
int make_tmap_head_rows(CUtensorMap* map, const void* base, uint64_t heads_total, uint64_t T, uint32_t heads, uint32_t width) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(NSA_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t head_bytes = (cuuint64_t)T * width * 2;
  cuuint64_t dims[5] = {64, 8, width / 64, heads_total / 8, T};
  cuuint64_t strides[4] = {head_bytes, 128, 8 * head_bytes, (cuuint64_t)width * 2};
  cuuint32_t box[5] = {64, 8, width / 64, heads / 8, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(NSA_ERR_LAUNCH, "cuTensorMapEncodeTiled (head rows) failed with %d", (int)r);
  return NSA_OK;
}

static int sm_count() {
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

template <int DK, int DV, int MODE, bool EXACT>
static int launch_fa_fwd_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tklo,
                           const FaFwdParams& p, cudaStream_t st) {
  using SM = FaSmem<DK, DV>;
  auto kern = fa_fwd_kernel<DK, DV, MODE, EXACT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kDynamic);
  if (e != cudaSuccess) return fail(NSA_ERR_LAUNCH, "fa_fwd: cannot reserve %d bytes of shared memory: %s", SM::kDynamic, cudaGetErrorString(e));
  const int nitems = (p.Tq / kBM) * p.B * (p.H / 2);
  dim3 grid((unsigned)std::min(nitems, sm_count()));   // persistent: one CTA per SM walks the item list
  KernelTimer kt(MODE == kWin ? "fa_fwd_win" : (EXACT ? "fa_fwd_cmp_exact" : "fa_fwd_cmp"), st);
  kern<<<grid, kFaThreads, SM::kDynamic, st>>>(tq, tk, tv, tklo, p);
  return check_launch("fa_fwd_sm100");
}

bool fa_fwd_sm100_supported(int H, int G, int Tq, int Tk, int dk, int dv) {
  const bool dims = (dk == 192 && dv == 128) || (dk == 128 && dv == 128) || (dk == 64 && dv == 64);
  return dims && G > 0 && H % G == 0 && (H / G) % 2 == 0 && Tq % kBM == 0 && Tk % kBN == 0 && Tq > 0 && Tk > 0;
}

int fa_fwd_sm100(const void* q, const void* k, const void* v, void* o, float* L, float* M, int B, int H, int G, int Tq,
                 int Tk, int dk, int dv, int mode, int window, int cmp_l, int cmp_d, int cmp_nb, float scale,
                 const void* k_lo, float* lse2, cudaStream_t st) {
  if (!fa_fwd_sm100_supported(H, G, Tq, Tk, dk, dv)) return fail(NSA_ERR_UNSUPPORTED, "fa_fwd_sm100: unsupported shape");
  if (!fa_timeout_counter()) return fail(NSA_ERR_LAUNCH, "fa_fwd_sm100: cannot set up the time-out record of this device");
  if ((int64_t)B * (H / 2) * (Tq / kBM) > 0x7fffffff) return fail(NSA_ERR_UNSUPPORTED, "fa_fwd_sm100: too many work items");
  if (k_lo && mode != kCmp) return fail(NSA_ERR_ARG, "fa_fwd_sm100: a low-order key part belongs to the compressed branch");
  CUtensorMap tq, tk, tv, tklo;
  if (int rc = make_tmap_bf16_2d(&tq, q, (uint64_t)B * H * Tq, dk, kBM)) return rc;
  if (int rc = make_tmap_bf16_2d(&tk, k, (uint64_t)B * G * dk, Tk, dk)) return rc;
  if (int rc = make_tmap_bf16_2d(&tklo, k_lo ? k_lo : k, (uint64_t)B * G * dk, Tk, dk)) return rc;
  if (int rc = make_tmap_bf16_2d(&tv, v, (uint64_t)B * G * Tk, dv, kBN)) return rc;
  FaFwdParams p;
  p.o = (__nv_bfloat16*)o; p.L = L; p.M = M;
  p.B = B; p.H = H; p.G = G; p.Tq = Tq; p.Tk = Tk;
  p.window = window; p.cmp_l = cmp_l; p.cmp_d = cmp_d; p.cmp_nb = cmp_nb;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse2 = lse2;
#define NSA_FA_CASE(DK_, DV_)                                                                                            \
  if (dk == DK_ && dv == DV_)                                                                                            \
    return mode == kWin ? launch_fa_fwd_t<DK_, DV_, kWin, false>(tq, tk, tv, tklo, p, st)                               \
                        : (k_lo ? launch_fa_fwd_t<DK_, DV_, kCmp, true>(tq, tk, tv, tklo, p, st)                          \
                                : launch_fa_fwd_t<DK_, DV_, kCmp, false>(tq, tk, tv, tklo, p, st));
  NSA_FA_CASE(192, 128)
  NSA_FA_CASE(128, 128)
  NSA_FA_CASE(64, 64)
#undef NSA_FA_CASE
  return fail(NSA_ERR_UNSUPPORTED, "fa_fwd_sm100: unsupported head dims");
}

// Host side of the time-out record.  One page of this library's own host memory is pinned and mapped into the device
// address space once per process (no allocation); a CTA that gives up on a wait sets its first word, so every entry
// point can notice a time-out without synchronising.  Each device's record learns the flag's device address on the first
// tensor-core launch on that device.
alignas(4096) static int g_host_timeout_flag[1024];

bool timeout_flagged() { return *(volatile int*)&g_host_timeout_flag[0] != 0; }

int* fa_timeout_counter() {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static int* cached[kMaxDevices] = {};
  static int host_state = 0;  // 0: not tried, 1: registered, -1: registration refused (count-only reporting)
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (cached[dev]) return cached[dev];
  TimeoutRecord* rec = nullptr;
  if (cudaGetSymbolAddress((void**)&rec, g_timeout_record) != cudaSuccess || !rec) return nullptr;
  if (host_state == 0) {
    const cudaError_t e = cudaHostRegister(g_host_timeout_flag, sizeof(g_host_timeout_flag), cudaHostRegisterPortable | cudaHostRegisterMapped);
    host_state = e == cudaSuccess ? 1 : -1;
    if (e != cudaSuccess) cudaGetLastError();
  }
  int* flag_dev = nullptr;
  if (host_state == 1 && cudaHostGetDevicePointer((void**)&flag_dev, g_host_timeout_flag, 0) != cudaSuccess) {
    flag_dev = nullptr;
    cudaGetLastError();
  }
  if (cudaMemcpy(&rec->host_flag, &flag_dev, sizeof(flag_dev), cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
  cached[dev] = &rec->count;
  return cached[dev];
}

int fa_fwd_sm100_timeouts(int* count, bool reset) {
  cudaError_t e = cudaMemcpyFromSymbol(count, g_timeout_record, sizeof(int));
  if (e != cudaSuccess) return fail(NSA_ERR_LAUNCH, "cannot read the timeout counter: %s", cudaGetErrorString(e));
  if (reset) {
    const int z = 0;
    cudaMemcpyToSymbol(g_timeout_record, &z, sizeof(int));
    *(volatile int*)&g_host_timeout_flag[0] = 0;
  }
  return NSA_OK;
}

// ------------------------------------------------------------------------------------------------
// Self-test of the bounded wait: one warp waits on a barrier that nothing ever arrives at, with a short limit, and
// leaves through the same report path as the product kernels.  No fault, no trap, no unbounded spin.
// ------------------------------------------------------------------------------------------------
__global__ void wait_timeout_selftest_kernel(int* timeouts, long long limit_clocks, int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  const bool ok = mbar_wait_warp(&bar, 0, &abort_flag, limit_clocks);
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok && abort_flag) report_timeout(timeouts);
    if (gave_up) *gave_up = ok ? 0 : 1;
  }
}

int wait_timeout_selftest(long long limit_clocks, int* gave_up_dev, cudaStream_t st) {
  int* t = fa_timeout_counter();
  if (!t) return fail(NSA_ERR_LAUNCH, "selftest: no time-out record on this device");
  wait_timeout_selftest_kernel<<<1, 32, 0, st>>>(t, limit_clocks, gave_up_dev);
  return check_launch("wait_timeout_selftest");
}

}  // namespace nsa
