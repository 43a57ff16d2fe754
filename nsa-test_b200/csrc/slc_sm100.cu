// Selected-block attention on tcgen05 tensor cores, key-block-major
// (replaces _nsa_sparse_selection_fwd_kernel / _bwd_kernel, nsa/kernels.py:594-833, 836-1148, for bf16
// tensors in canonical layouts with a 64-key selection block).
//
// The reference walks queries and, for each, gathers its selected blocks: every KV block is fetched once
// per (query, head).  Here the work is turned around with the inverse index "block -> (query, slot)"
// (select_csr.cu): a CTA keeps one KV block in shared memory and streams the queries that selected it
// past it, 128 MMA rows at a time (128/heads_per_group queries x all heads of the GQA group), so a block
// is read once per group of queries and shared by all their heads.  Each (query, slot) pair yields a
// partial result; partials of a query are merged afterwards in slot order, which keeps everything
// deterministic:
//   forward   partial O (normalised, bf16) + (max, sum) per (query, slot, head) -> slc_combine_fwd
//   backward  one fused kernel: dQ partials per (query, slot, head) -> slc_combine_dq; dK/dV accumulate
//             (transposed, in TMEM) inside the CTA that owns the block and are flushed once per CTA and block.
// CTAs own fixed-size ranges of the inverse index (not whole blocks), so a block selected by every
// query (block 0) is spread over many CTAs.
#include <cuda.h>

#include "attn_args.cuh"
#include "common.cuh"
#include "fa_sm100.cuh"
#include "slc_sm100.cuh"
#include "sm100_ptx.cuh"

namespace nsa {

using namespace ptx;

constexpr int kEntriesPerCta = 1024;  // inverse-index entries handled by one CTA
constexpr float kLn2f = 0.6931471805599453f;
constexpr float kLog2ef = 1.4426950408889634f;


struct SlcParams {
  const __nv_bfloat16* q;      // [B,H,Tq,dk]
  const __nv_bfloat16* dout;   // [B,H,Tq,dv] (backward)
  const int* csr_off;          // [BG, nblk+1]
  const int* csr_t;            // [BG, Tq*nslots]
  __nv_bfloat16* o_part;       // [BG,Tq,nslots,hpg,dv]  normalised partial outputs
  float2* st_part;             // [BG,Tq,nslots,hpg]     (row max in log2 units, sum of exp2)
  const float *D, *lse2;       // [B,H,Tq] backward statistics
  __nv_bfloat16* dq_part;      // [BG,Tq,nslots,hpg,dk]
  float *dk_part, *dv_part;    // [BG, nparts+nblk, 64, dk|dv] per-(CTA, block) partial sums (backward)
  __nv_bfloat16 *dk_out, *dv_out;  // [B,G,Tk,dk|dv] gradients the reduced partials are added into
  int B, H, G, Tq, Tk, nslots, nblk, hpg;
  int q0;  // position of query row 0 in the sequence (query-sharded runs; 0 otherwise)
  int g5;  // gathered rows arrive as one rank-5 tile per query ([heads/8][width/64][8 rows][64 columns]) instead of one tile per 64 columns
  float scale, scale_log2;
  int* timeouts;
};

// Walks the chunk schedule of a CTA: chunks of up to `qpc` consecutive entries that stay inside one block.
struct ChunkWalker {
  const int* off;
  int e, e1, blk, blk_end, nblk, qpc;
  __device__ ChunkWalker(const int* off_, int nblk_, int e0, int e1_, int qpc_) : off(off_), e(e0), e1(e1_), nblk(nblk_), qpc(qpc_) {
    const int total = off[nblk];
    e1 = min(e1, total);
    // block holding entry e0: largest blk with off[blk] <= e0
    int lo = 0, hi = nblk;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (off[mid] <= e) lo = mid; else hi = mid;
    }
    blk = lo;
    blk_end = off[blk + 1];
    skip_empty();
  }
  __device__ void skip_empty() {
    while (e < e1 && e >= blk_end && blk + 1 < nblk) {
      ++blk;
      blk_end = off[blk + 1];
    }
  }
  __device__ bool done() const { return e >= e1; }
  __device__ int count() const { return min(qpc, min(blk_end, e1) - e); }
  __device__ void next() {
    e += count();
    skip_empty();
  }
};

// ------------------------------------------------------------------------------------------------
// forward: partial attention of every (query, slot) against its block
// ------------------------------------------------------------------------------------------------
template <int DK, int DV>
struct SlcFwdSmem {
  static constexpr int kK = 64 * DK * 2, kV = 64 * DV * 2, kQ = 128 * DK * 2;
  static constexpr int kQStages = 2;
  static constexpr int kStage = 8 * 4096;  // per compute warp: 32 rows x 64 bf16 columns on their way to global memory
  static constexpr int oK = 0, oV = oK + 2 * kK, oQ = oV + 2 * kV, oStage = oQ + kQStages * kQ, oBar = oStage + kStage;
  static constexpr int kDynamic = oBar + 256 + 1024;
};
struct SlcFwdBarriers {
  uint64_t kv_full[2], kv_empty[2], q_full[2], q_empty[2], s_full[2], p_full[2], o_full[2], o_read[2];
  uint32_t tmem_base;
  int abort;
};

// Token-major copy [B,H,T,W] -> [B,G,T,H/G,W]: the rows of all heads of a group for one query become one contiguous
// [H/G x W] box, so a chunk of queries is gathered with a handful of TMA tile loads instead of thousands of 16-byte copies.
template <int W>
__global__ void to_token_major_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int B, int H, int G,
                                      int T) {
  const int64_t ro = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (ro >= (int64_t)B * H * T) return;
  const int hpg = H / G;
  const int hh = ro % hpg;
  const int64_t bgt = ro / hpg;
  const int t = bgt % T;
  const int bg = bgt / T, b = bg / G, g = bg % G;
  const uint4* src = reinterpret_cast<const uint4*>(in + (((int64_t)b * H + g * hpg + hh) * T + t) * W);
  uint4* dst = reinterpret_cast<uint4*>(out + ro * W);
  if (lane < W / 8) dst[lane] = src[lane];
}

// One chunk = up to qpc queries; query qi fills rows [qi*hpg, (qi+1)*hpg) of the 128-row K-major swizzled tiles.
// Two tile layouts: one 64-column block after the other ([width/64][128 rows][128 B], a 2-D tile load per query and
// column block), or, when the heads of a group fill whole 8-row swizzle atoms, [128/8 row groups][width/64][8 rows][128 B]
// with ONE rank-5 tile load per query.  The UMMA descriptors take the layout as (row-group stride, column-block stride).
// Unused query slots are loaded from beyond the tensor (TMA fills zeros), so every chunk delivers the same byte count.
// Lane qi of the producer warp fetches its query's inverse-index entry and issues that query's tile loads, so the entry
// loads of a chunk are one coalesced request instead of a chain of dependent ones.

template <int DK, int DV>
__global__ void __launch_bounds__(320, 1)
slc_fwd_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
               const __grid_constant__ CUtensorMap tmQt, const __grid_constant__ CUtensorMap tmOp, const SlcParams p) {
  using SM = SlcFwdSmem<DK, DV>;
  constexpr int NQ = SM::kQStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t *sK = smem + SM::oK, *sV = smem + SM::oV, *sQ = smem + SM::oQ;
  SlcFwdBarriers* bar = reinterpret_cast<SlcFwdBarriers*>(smem + SM::oBar);
  volatile int* abort = &bar->abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bg = blockIdx.y, b = bg / p.G, g = bg % p.G;
  const int* off = p.csr_off + (int64_t)bg * (p.nblk + 1);
  const int* ent = p.csr_t + (int64_t)bg * p.Tq * p.nslots;
  const int e0 = blockIdx.x * kEntriesPerCta;
  const int qpc = 128 / p.hpg;
  // once any block has given up on a wait the device results are void: later blocks skip their work and end at once
  const bool has_work = e0 < off[p.nblk] && !(p.timeouts && *(volatile const int*)p.timeouts != 0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->q_full[i], 1);
      mbar_init(&bar->q_empty[i], 1);
      mbar_init(&bar->kv_full[i], 1);
      mbar_init(&bar->kv_empty[i], 1);
      mbar_init(&bar->s_full[i], 1);
      mbar_init(&bar->p_full[i], 128);
      mbar_init(&bar->o_full[i], 1);
      mbar_init(&bar->o_read[i], 128);
    }
    bar->abort = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 8) tmem_alloc(&bar->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;

  if (!has_work) {
    // nothing to do for this CTA
  } else if (warp == 9) {
    // ------------------------------------------------------------ producer warp: K/V blocks and gathered Q rows, all by TMA
    ChunkWalker w(off, p.nblk, e0, e0 + kEntriesPerCta, qpc);
    const int oob_row = p.B * p.H * p.Tq;
    const int oct0 = (b * p.H + g * p.hpg) >> 3;  // first head of the group, in units of 8 heads (rank-5 loads)
    bool ok = true;
    int c = 0, kvidx = -1, last_blk = -1;
    for (; !w.done(); w.next(), ++c) {
      const int s = c % NQ;
      if (w.blk != last_blk) {
        last_blk = w.blk;
        ++kvidx;
        const int ks = kvidx & 1;
        ok = mbar_wait_warp(&bar->kv_empty[ks], ((kvidx >> 1) & 1) ^ 1, abort);
        if (!ok) break;
        if (lane == 0) {
          mbar_arrive_expect_tx(&bar->kv_full[ks], SM::kK + SM::kV);
          tma_load_2d(&tmK, &bar->kv_full[ks], sK + ks * SM::kK, w.blk * 64, (b * p.G + g) * DK);
          for (int cc = 0; cc < DV / 64; ++cc)
            tma_load_2d(&tmV, &bar->kv_full[ks], sV + ks * SM::kV + cc * 8192, cc * 64, (b * p.G + g) * p.Tk + w.blk * 64);
        }
      }
      // this chunk's entries are fetched while the stage is still busy
      const int cnt = w.count();
      int tok = p.Tq, row = oob_row;  // beyond the tensor: the tile is filled with zeros
      if (lane < cnt) {
        tok = ent[w.e + lane] & 0xFFFFFF;
        row = (int)(((int64_t)bg * p.Tq + tok) * p.hpg);
      }
      ok = mbar_wait_warp(&bar->q_empty[s], ((c / NQ) & 1) ^ 1, abort);
      if (!ok) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&bar->q_full[s], SM::kQ);
      }
      __syncwarp();
      for (int qi = lane; qi < qpc; qi += 32) {
        const int r2 = qi < 32 ? row : (qi < cnt ? (int)(((int64_t)bg * p.Tq + (ent[w.e + qi] & 0xFFFFFF)) * p.hpg) : oob_row);
        if (p.g5) {
          tma_load_5d_outer(&tmQt, &bar->q_full[s], sQ + s * SM::kQ + qi * p.hpg * (DK * 2), oct0, tok);
        } else {
#pragma unroll
          for (int cc = 0; cc < DK / 64; ++cc)
            tma_load_2d(&tmQt, &bar->q_full[s], sQ + s * SM::kQ + cc * 16384 + qi * p.hpg * 128, cc * 64, r2);
        }
      }
    }
    if (!ok && lane == 0) {  // let copies in flight land before the CTA gives its shared memory back
      if (kvidx >= 0) mbar_wait(&bar->kv_full[kvidx & 1], (kvidx >> 1) & 1, abort);
      for (int cc = max(0, c - NQ); cc < c; ++cc) mbar_wait(&bar->q_full[cc % NQ], (cc / NQ) & 1, abort);
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------ UMMA issuer: the warp runs the schedule uniformly, one
    // elected lane issues the tensor-core instructions
    constexpr uint32_t idS = idesc_bf16(128, 64, 0, 1);   // Q rows (K-major) x K block (MN-major: keys contiguous)
    constexpr uint32_t idO = idesc_bf16(128, DV, 0, 1);   // P (TMEM) x V block (MN-major: dv contiguous)
    const uint32_t sboQ = p.g5 ? (DK / 64) * 1024 : 1024, cbQ = p.g5 ? 1024 : 16384;  // Q tile: row-group / column-block strides
    ChunkWalker w(off, p.nblk, e0, e0 + kEntriesPerCta, qpc);
    bool ok = true;
    int c = 0, kvidx = 0, ks_cur = 0, cur_blk = w.blk;
    auto issue_s = [&](int cc, int ks) -> bool {
      const int s = cc % NQ, buf = cc & 1;
      if (!mbar_wait_warp(&bar->q_full[s], (cc / NQ) & 1, abort)) return false;
      if (!mbar_wait_warp(&bar->o_read[buf], ((cc >> 1) & 1) ^ 1, abort)) return false;
      tc_fence_after();
      const uint64_t dQ = smem_desc_sw128(smem_u32(sQ + s * SM::kQ), 16, sboQ);
      const uint64_t dK = smem_desc_sw128(smem_u32(sK + ks * SM::kK), 16, 1024);  // one 64-key MN block: LBO unused
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk)
          umma_ss(tmem + buf * 192, desc_advance(dQ, (kk >> 2) * cbQ + (kk & 3) * 32), desc_advance(dK, kk * 2048), idS, kk > 0);
        umma_commit(&bar->s_full[buf]);
        umma_commit(&bar->q_empty[s]);
      }
      __syncwarp();
      return true;
    };
    // prologue: S(0)
    ok = mbar_wait_warp(&bar->kv_full[0], 0, abort);
    if (ok) ok = issue_s(0, 0);
    while (ok && !w.done()) {
      w.next();
      // look ahead: S(c+1) is issued before PV(c)
      bool last_of_block = true;
      int ks_next = ks_cur;
      if (!w.done()) {
        if (w.blk != cur_blk) {
          cur_blk = w.blk;
          ++kvidx;
          ks_next = kvidx & 1;
          ok = mbar_wait_warp(&bar->kv_full[ks_next], (kvidx >> 1) & 1, abort);
          if (!ok) break;
        } else {
          last_of_block = false;
        }
        ok = issue_s(c + 1, ks_next);
        if (!ok) break;
      }
      const int buf = c & 1;
      ok = mbar_wait_warp(&bar->p_full[buf], (c >> 1) & 1, abort);
      if (!ok) break;
      tc_fence_after();
      const uint64_t dV = smem_desc_sw128(smem_u32(sV + ks_cur * SM::kV), 8192, 1024);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ts(tmem + buf * 192 + 64, tmem + buf * 192 + kk * 8, desc_advance(dV, kk * 2048), idO, kk > 0);
        umma_commit(&bar->o_full[buf]);
        if (last_of_block) umma_commit(&bar->kv_empty[ks_cur]);
      }
      __syncwarp();
      ks_cur = ks_next;
      ++c;
    }
  } else {
    // ------------------------------------------------------------ softmax + partial epilogue (two groups alternate chunks)
    const int grp = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const int qi = r / p.hpg, hh = r % p.hpg;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    // partial outputs leave through a per-warp staging area (128-byte swizzle) and TMA tile stores: one box per query
    // (or per 32 rows of it), so global memory sees whole lines instead of one 16-byte piece per row
    uint8_t* stage = smem + SM::oStage + warp * 4096;
    const int boxrows = min(p.hpg, 32), nbox = 32 / boxrows;
    const int box_lane = (lane * boxrows) & 31;  // lane owning the first row of the box this lane would store
    ChunkWalker w(off, p.nblk, e0, e0 + kEntriesPerCta, qpc);
    bool ok = true;
    if (grp == 1 && !w.done()) w.next();
    int entry_next = 0;
    if (!w.done() && qi < w.count()) entry_next = ent[w.e + qi];
    for (int c = grp; !w.done() && ok; c += 2) {
      const int buf = grp, it = c >> 1;
      const bool valid = qi < w.count();
      const int entry = entry_next;
      const int t = entry & 0xFFFFFF, slot = entry >> 24;
      const int key0 = w.blk * 64;
      // move on to this group's next chunk and fetch its entry early
      w.next();
      if (!w.done()) w.next();
      if (!w.done() && qi < w.count()) entry_next = ent[w.e + qi];
      ok = mbar_wait(&bar->s_full[buf], it & 1, abort);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[2][32];
      tmem_ld32(tmem + lane_base + buf * 192, sv[0]);
      tmem_ld32(tmem + lane_base + buf * 192 + 32, sv[1]);
      tc_wait_ld();
      const int chi = valid ? p.q0 + t - key0 : 63;  // causal: keys key0 + c <= position of the query
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc)
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float x = (cc * 32 + e <= chi) ? __uint_as_float(sv[cc][e]) * p.scale_log2 : -CUDART_INF_F;
          sv[cc][e] = __float_as_uint(x);
          mx = fmaxf(mx, x);
        }
      float l = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const int cc = e >> 4, ee = (e & 15) * 2;
        const float p0 = ex2(__uint_as_float(sv[cc][ee]) - mx), p1 = ex2(__uint_as_float(sv[cc][ee + 1]) - mx);
        l += p0 + p1;
        __nv_bfloat162 v2 = __floats2bfloat162_rn(p0, p1);
        pk[e] = *reinterpret_cast<uint32_t*>(&v2);
      }
      tmem_st32(tmem + lane_base + buf * 192, pk);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&bar->p_full[buf]);
      const float inv = 1.f / l;
      const int64_t prow = (((int64_t)bg * p.Tq + t) * p.nslots + slot) * p.hpg + hh;
      if (valid) p.st_part[prow] = make_float2(mx, l);
      // the lane that stores a box needs the global row of the box's first row
      const int box_row = __shfl_sync(0xffffffffu, valid ? (int)prow : -1, box_lane);
      ok = mbar_wait(&bar->o_full[buf], it & 1, abort);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int half = 0; half < DV / 64; ++half) {
        uint32_t ov[2][32];
        tmem_ld32(tmem + lane_base + buf * 192 + 64 + half * 64, ov[0]);
        tmem_ld32(tmem + lane_base + buf * 192 + 64 + half * 64 + 32, ov[1]);
        tc_wait_ld();
        if (half == DV / 64 - 1) {  // the accumulator is free again as soon as it sits in registers
          tc_fence_before();
          mbar_arrive(&bar->o_read[buf]);
        }
        bulk_wait_read<0>();  // the staging area is no longer being read by the previous store
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t* src = &ov[j >> 2][(j & 3) * 8];
          uint4 wv;
          __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(src[0]) * inv, __uint_as_float(src[1]) * inv);
          __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(src[2]) * inv, __uint_as_float(src[3]) * inv);
          __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(src[4]) * inv, __uint_as_float(src[5]) * inv);
          __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(src[6]) * inv, __uint_as_float(src[7]) * inv);
          wv.x = *reinterpret_cast<uint32_t*>(&a0); wv.y = *reinterpret_cast<uint32_t*>(&a1);
          wv.z = *reinterpret_cast<uint32_t*>(&a2); wv.w = *reinterpret_cast<uint32_t*>(&a3);
          *reinterpret_cast<uint4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) = wv;
        }
        fence_proxy_async();
        __syncwarp();
        if (lane < nbox && box_row >= 0) tma_store_2d(&tmOp, stage + lane * boxrows * 128, half * 64, box_row);
        bulk_commit();
      }
    }
    bulk_wait_read<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && bar->abort) ptx::report_timeout(p.timeouts);
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// Which slots of a query's index row contribute (see slot_block): lane s decides for slot s from one load per lane,
// repeats are found with shuffles.  Returns the ballot of contributing slots.
__device__ __forceinline__ unsigned valid_slot_mask(const int* irow, int64_t s3, int nslots, int t, int Tk, int lprime, int lane) {
  const int id = lane < nslots ? irow[lane * s3] : -1;
  bool ok = id >= 0 && (int64_t)id * lprime < Tk && (int64_t)id * lprime <= t;
  for (int s2 = 0; s2 < nslots; ++s2) {
    const int other = __shfl_sync(0xffffffffu, id, s2);
    if (s2 < lane && other == id) ok = false;
  }
  return __ballot_sync(0xffffffffu, ok);
}

// Gate + mix epilogue of the merge kernels: the warp holds the finished (rounded) O_slc row of (b,h,t), lane owning VPL
// consecutive columns; the mixed row is (o_cmp g0 + o_slc g1) + o_win g2, the operation order of the stand-alone pass.
template <int VPL>
__device__ __forceinline__ void slc_mix_row(const SlcMix& mix, const __nv_bfloat162 (&oslc)[VPL / 2], int64_t row, int b, int h, int t,
                                            int H, int Tq, int dv, int lane) {
  const __nv_bfloat16* oc = (const __nv_bfloat16*)mix.o_cmp + row * dv + lane * VPL;
  const __nv_bfloat16* ow = (const __nv_bfloat16*)mix.o_win + row * dv + lane * VPL;
  __nv_bfloat162 a[VPL / 2], w[VPL / 2];
#pragma unroll
  for (int c = 0; c < VPL / 2; ++c) {
    a[c] = *reinterpret_cast<const __nv_bfloat162*>(oc + 2 * c);
    w[c] = *reinterpret_cast<const __nv_bfloat162*>(ow + 2 * c);
  }
  float g[3];
  gates3(mix.logits + ((int64_t)b * Tq + t) * 3 * H + 3 * h, mix.mode, g);
  if (lane < 3) mix.gates[row * 3 + lane] = g[lane];
  __nv_bfloat16* dst = (__nv_bfloat16*)mix.out + mixed_row(row, b, h, t, H, Tq, mix.token_major) * dv + lane * VPL;
#pragma unroll
  for (int c = 0; c < VPL / 2; ++c) {
    const float2 fa = __bfloat1622float2(a[c]), fs = __bfloat1622float2(oslc[c]), fw = __bfloat1622float2(w[c]);
    *reinterpret_cast<__nv_bfloat162*>(dst + 2 * c) =
        __floats2bfloat162_rn((fa.x * g[0] + fs.x * g[1]) + fw.x * g[2], (fa.y * g[0] + fs.y * g[1]) + fw.y * g[2]);
  }
}

// merge the partials of a query in slot order: one warp per (b,h,t).  Every load of the row (index row, statistics,
// all slots' partial outputs) is issued before the first value is used; slots that turn out not to contribute were
// never written and their loads are discarded.
template <int DV>
__global__ void slc_combine_fwd_kernel(const __nv_bfloat16* __restrict__ o_part, const float2* __restrict__ st_part,
                                       const int* __restrict__ indices, int64_t s0, int64_t s1, int64_t s2, int64_t s3,
                                       __nv_bfloat16* __restrict__ out, float* __restrict__ L, float* __restrict__ M, int B,
                                       int H, int G, int Tq, int Tk, int nslots, int lprime, int q0, const SlcMix mix) {
  static_assert(DV % 64 == 0, "lanes own 2 or 4 consecutive output columns");
  constexpr int VPL = DV / 32;  // values per lane
  // consecutive warps take the heads of one (group, query): together they stream that query's contiguous block of partials
  const int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (int64_t)B * H * Tq) return;
  const int hpg = H / G;
  const int hh = wid % hpg, t = (wid / hpg) % Tq, bgi = wid / ((int64_t)hpg * Tq);
  const int b = bgi / G, g = bgi % G, h = g * hpg + hh;
  const int64_t row = ((int64_t)b * H + h) * Tq + t;
  const int* irow = indices + b * s0 + g * s1 + (int64_t)t * s2;
  const int64_t base = (((int64_t)(b * G + g) * Tq + t) * nslots) * hpg + hh;
  float2 st = make_float2(-CUDART_INF_F, 0.f);
  if (lane < nslots) st = st_part[base + (int64_t)lane * hpg];
  float lsum = 0.f, mx = 0.f, wmine = 0.f, acc[VPL];
  unsigned validmask = 0;
#pragma unroll
  for (int c = 0; c < VPL; ++c) acc[c] = 0.f;
  for (int s16 = 0; s16 < nslots; s16 += 16) {
    uint2 raw[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      raw[u] = make_uint2(0u, 0u);
      if (s16 + u < nslots) {
        const __nv_bfloat16* src = o_part + (base + (int64_t)(s16 + u) * hpg) * DV + lane * VPL;
        if (VPL == 4) raw[u] = *reinterpret_cast<const uint2*>(src);
        else raw[u].x = *reinterpret_cast<const uint32_t*>(src);
      }
    }
    if (s16 == 0) {
      validmask = valid_slot_mask(irow, s3, nslots, q0 + t, Tk, lprime, lane);
      const bool mine = (validmask >> lane) & 1;
      if (!mine) st = make_float2(-CUDART_INF_F, 0.f);
      mx = warp_max(st.x);
      wmine = mine ? st.y * ex2(st.x - mx) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const int s = s16 + u;
      const float wgt = __shfl_sync(0xffffffffu, wmine, s & 31);
      if (s >= nslots || !((validmask >> s) & 1)) continue;
      lsum += wgt;
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[u].x));
      acc[0] = fmaf(wgt, a.x, acc[0]); acc[1] = fmaf(wgt, a.y, acc[1]);
      if (VPL == 4) {
        const float2 c2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[u].y));
        acc[2 % VPL] = fmaf(wgt, c2.x, acc[2 % VPL]); acc[3 % VPL] = fmaf(wgt, c2.y, acc[3 % VPL]);
      }
    }
  }
  const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
  __nv_bfloat16* dst = out + row * DV + lane * VPL;
  __nv_bfloat162 rounded[VPL / 2];
#pragma unroll
  for (int c = 0; c < VPL; c += 2) {
    rounded[c / 2] = __floats2bfloat162_rn(acc[c] * inv, acc[c + 1] * inv);
    *reinterpret_cast<__nv_bfloat162*>(dst + c) = rounded[c / 2];
  }
  if (lane == 0) {
    L[row] = lsum > 0.f ? logf(lsum) : -CUDART_INF_F;
    M[row] = lsum > 0.f ? mx * kLn2f : -CUDART_INF_F;
  }
  if (mix.out) slc_mix_row<VPL>(mix, rounded, row, b, h, t, H, Tq, DV, lane);
}

// Same merge with the whole contiguous block of a query's partials ([slots][heads][dv]) brought into shared memory by
// one bulk copy: one thread block per (group, query), one warp per head.  No registers are spent on loads in flight,
// so several blocks per SM keep enough bytes on their way to saturate HBM.
template <int DV>
__global__ void slc_combine_fwd_bulk_kernel(const __nv_bfloat16* __restrict__ o_part, const float2* __restrict__ st_part,
                                            const int* __restrict__ indices, int64_t s0, int64_t s1, int64_t s2, int64_t s3,
                                            __nv_bfloat16* __restrict__ out, float* __restrict__ L, float* __restrict__ M, int B,
                                            int H, int G, int Tq, int Tk, int nslots, int lprime, int q0, int* timeouts,
                                            const SlcMix mix) {
  constexpr int VPL = DV / 32;
  extern __shared__ __align__(128) uint8_t sm_part[];
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  const int hpg = H / G, hh = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t q = blockIdx.x;  // (batch, group, query)
  const int t = q % Tq, bgi = q / Tq, b = bgi / G, g = bgi % G, h = g * hpg + hh;
  const uint32_t bytes = (uint32_t)nslots * hpg * DV * 2;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(&bar, bytes);
    bulk_load_1d(sm_part, o_part + q * (int64_t)nslots * hpg * DV, bytes, &bar);
  }
  const int64_t row = ((int64_t)b * H + h) * Tq + t;
  const int* irow = indices + b * s0 + g * s1 + (int64_t)t * s2;
  const int64_t base = (q * nslots) * hpg + hh;
  float2 st = make_float2(-CUDART_INF_F, 0.f);
  if (lane < nslots) st = st_part[base + (int64_t)lane * hpg];
  const unsigned validmask = valid_slot_mask(irow, s3, nslots, q0 + t, Tk, lprime, lane);
  const bool mine = (validmask >> lane) & 1;
  if (!mine) st = make_float2(-CUDART_INF_F, 0.f);
  const float mx = warp_max(st.x);
  const float wmine = mine ? st.y * ex2(st.x - mx) : 0.f;
  float lsum = 0.f, acc[VPL];
#pragma unroll
  for (int c = 0; c < VPL; ++c) acc[c] = 0.f;
  const bool ok = mbar_wait_warp(&bar, 0, &abort_flag);
  if (ok) {
    for (int s = 0; s < nslots; ++s) {
      const float wgt = __shfl_sync(0xffffffffu, wmine, s);
      if (!((validmask >> s) & 1)) continue;  // never written: skip
      lsum += wgt;
      const uint8_t* src = sm_part + ((size_t)(s * hpg + hh) * DV + lane * VPL) * 2;
      uint2 raw = make_uint2(0u, 0u);
      if (VPL == 4) raw = *reinterpret_cast<const uint2*>(src);
      else raw.x = *reinterpret_cast<const uint32_t*>(src);
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
      acc[0] = fmaf(wgt, a.x, acc[0]); acc[1] = fmaf(wgt, a.y, acc[1]);
      if (VPL == 4) {
        const float2 c2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        acc[2 % VPL] = fmaf(wgt, c2.x, acc[2 % VPL]); acc[3 % VPL] = fmaf(wgt, c2.y, acc[3 % VPL]);
      }
    }
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    __nv_bfloat16* dst = out + row * DV + lane * VPL;
    __nv_bfloat162 rounded[VPL / 2];
#pragma unroll
    for (int c = 0; c < VPL; c += 2) {
      rounded[c / 2] = __floats2bfloat162_rn(acc[c] * inv, acc[c + 1] * inv);
      *reinterpret_cast<__nv_bfloat162*>(dst + c) = rounded[c / 2];
    }
    if (lane == 0) {
      L[row] = lsum > 0.f ? logf(lsum) : -CUDART_INF_F;
      M[row] = lsum > 0.f ? mx * kLn2f : -CUDART_INF_F;
    }
    if (mix.out) slc_mix_row<VPL>(mix, rounded, row, b, h, t, H, Tq, DV, lane);
  }
  __syncthreads();  // the copy has landed (or was given up on) before shared memory is handed back
  if (threadIdx.x == 0 && abort_flag) ptx::report_timeout(timeouts);
}

// ------------------------------------------------------------------------------------------------
// backward: combine of the per-(query, slot) dQ partials written by the fused kernel below
// ------------------------------------------------------------------------------------------------
// dQ[b,h,t,:] = scale * sum of the contributing slots' partials, slot order: one warp per row; the loads of 8 slots
// are in flight together and do not wait for the index row
// dQ of the selection branch plus, when given, the dQ of the two other branches (same layout): one rounding of the sum
__device__ __forceinline__ __nv_bfloat162 slc_dq_total(float x, float y, const __nv_bfloat16* add0, const __nv_bfloat16* add1,
                                                       int64_t at) {
  if (add0) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(add0 + at));
    x += a.x;
    y += a.y;
  }
  if (add1) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(add1 + at));
    x += a.x;
    y += a.y;
  }
  return __floats2bfloat162_rn(x, y);
}

template <int DK>
__global__ void slc_combine_dq_kernel(const __nv_bfloat16* __restrict__ dq_part, const int* __restrict__ indices, int64_t s0,
                                      int64_t s1, int64_t s2, int64_t s3, __nv_bfloat16* __restrict__ dq, int B, int H, int G,
                                      int Tq, int Tk, int nslots, int lprime, float scale, int q0,
                                      const __nv_bfloat16* __restrict__ add0, const __nv_bfloat16* __restrict__ add1) {
  // consecutive warps take the heads of one (group, query): together they stream that query's contiguous block of partials
  const int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (int64_t)B * H * Tq) return;
  const int hpg = H / G;
  const int hh = wid % hpg, t = (wid / hpg) % Tq, bgi = wid / ((int64_t)hpg * Tq);
  const int b = bgi / G, g = bgi % G, h = g * hpg + hh;
  const int64_t row = ((int64_t)b * H + h) * Tq + t;
  const int* irow = indices + b * s0 + g * s1 + (int64_t)t * s2;
  const int64_t base = (((int64_t)(b * G + g) * Tq + t) * nslots) * hpg + hh;
  unsigned validmask = 0;
  float acc[DK / 32];
#pragma unroll
  for (int c = 0; c < DK / 32; ++c) acc[c] = 0.f;
  for (int s8 = 0; s8 < nslots; s8 += 8) {
    uint32_t raw[8][DK / 64];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const __nv_bfloat16* src = dq_part + (base + (int64_t)(s8 + u) * hpg) * DK;
#pragma unroll
      for (int c = 0; c < DK / 64; ++c) raw[u][c] = s8 + u < nslots ? *reinterpret_cast<const uint32_t*>(src + c * 64 + lane * 2) : 0u;
    }
    if (s8 == 0) validmask = valid_slot_mask(irow, s3, nslots, q0 + t, Tk, lprime, lane);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (s8 + u >= nslots || !((validmask >> (s8 + u)) & 1)) continue;  // never written: discard
#pragma unroll
      for (int c = 0; c < DK / 64; ++c) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[u][c]));
        acc[2 * c] += a.x;
        acc[2 * c + 1] += a.y;
      }
    }
  }
#pragma unroll
  for (int c = 0; c < DK / 64; ++c) {
    const int64_t at = row * DK + c * 64 + lane * 2;
    *reinterpret_cast<__nv_bfloat162*>(dq + at) = slc_dq_total(acc[2 * c] * scale, acc[2 * c + 1] * scale, add0, add1, at);
  }
}

// Same sum with the query's contiguous block of partials ([slots][heads][dk]) brought in by one bulk copy:
// one thread block per (group, query), one warp per head.
template <int DK>
__global__ void slc_combine_dq_bulk_kernel(const __nv_bfloat16* __restrict__ dq_part, const int* __restrict__ indices, int64_t s0,
                                           int64_t s1, int64_t s2, int64_t s3, __nv_bfloat16* __restrict__ dq, int B, int H, int G,
                                           int Tq, int Tk, int nslots, int lprime, float scale, int q0, int* timeouts,
                                           const __nv_bfloat16* __restrict__ add0, const __nv_bfloat16* __restrict__ add1) {
  extern __shared__ __align__(128) uint8_t sm_part[];
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  const int hpg = H / G, hh = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t q = blockIdx.x;
  const int t = q % Tq, bgi = q / Tq, b = bgi / G, g = bgi % G, h = g * hpg + hh;
  const uint32_t bytes = (uint32_t)nslots * hpg * DK * 2;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(&bar, bytes);
    bulk_load_1d(sm_part, dq_part + q * (int64_t)nslots * hpg * DK, bytes, &bar);
  }
  const int64_t row = ((int64_t)b * H + h) * Tq + t;
  const int* irow = indices + b * s0 + g * s1 + (int64_t)t * s2;
  const unsigned validmask = valid_slot_mask(irow, s3, nslots, q0 + t, Tk, lprime, lane);
  float acc[DK / 32];
#pragma unroll
  for (int c = 0; c < DK / 32; ++c) acc[c] = 0.f;
  const bool ok = mbar_wait_warp(&bar, 0, &abort_flag);
  if (ok) {
    for (int s = 0; s < nslots; ++s) {
      if (!((validmask >> s) & 1)) continue;
      const uint8_t* src = sm_part + (size_t)(s * hpg + hh) * DK * 2;
#pragma unroll
      for (int c = 0; c < DK / 64; ++c) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + (c * 64 + lane * 2) * 2));
        acc[2 * c] += a.x;
        acc[2 * c + 1] += a.y;
      }
    }
#pragma unroll
    for (int c = 0; c < DK / 64; ++c) {
      const int64_t at = row * DK + c * 64 + lane * 2;
      *reinterpret_cast<__nv_bfloat162*>(dq + at) = slc_dq_total(acc[2 * c] * scale, acc[2 * c + 1] * scale, add0, add1, at);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag) ptx::report_timeout(timeouts);
}

// accumulator rows [M x 64 keys] in TMEM -> part[(key_base + key) * W + off + row]; M = 128: row = TMEM lane,
// M = 64: 16 rows per warp in its first 16 lanes
template <int M>
__device__ __forceinline__ void slc_flush_rows(uint32_t taddr, float* __restrict__ part, int64_t key_base, int W, int off, int warp4,
                                               int lane) {
  const int row = M == 128 ? warp4 * 32 + lane : warp4 * 16 + (lane & 15);
  const bool active = M == 128 || lane < 16;
  const uint32_t lane_base = (uint32_t)(warp4 * 32) << 16;
#pragma unroll
  for (int cc = 0; cc < 2; ++cc) {
    uint32_t ov[32];
    tmem_ld32(taddr + lane_base + cc * 32, ov);
    tc_wait_ld();
    if (active) {
      float* dst = part + (key_base + cc * 32) * W + off + row;
#pragma unroll
      for (int e = 0; e < 32; ++e) dst[(int64_t)e * W] = __uint_as_float(ov[e]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// backward, fused: dQ partials AND dK/dV of each block from one pass over the gathered rows.
// Per chunk: S = Q K^T, dP = dO V^T (one TMEM buffer), rows -> P, dS; dS goes back to TMEM (bf16, over
// the dP columns) for dQ_part = dS K, and P / dS go through shared memory (64-row halves) for the
// transposed accumulations dV^T += dO^T P, dK^T += Q^T dS.  TMEM: S 64 | dP 64 | dQ dk | dV^T 64 | dK^T 64 (+64)
// = 512 columns at dk = 192.  The rows are gathered once and S / dP computed once, instead of once per kernel.
// The issuer polls four kinds of work: S of the next chunk, dQ of the current one, dP of the next one (program
// order after dQ, which reads dS from the same columns), and the accumulation steps.
// ------------------------------------------------------------------------------------------------
template <int DK, int DV>
struct SlcBwdSmem {
  static constexpr int kK = 64 * DK * 2, kV = 64 * DV * 2, kQ = 128 * DK * 2, kdO = 128 * DV * 2;
  static constexpr int kStage = kQ + kdO;
  static constexpr int kHalf = 64 * 128;   // 64 rows x 64 keys of bf16 P (or dS), 128-byte swizzle
  static constexpr int oK = 0, oV = oK + kK, oSt = oV + kV, oP = oSt + 2 * kStage, odS = oP + kHalf, oBar = odS + kHalf;
  static constexpr int kDynamic = oBar + 256 + 1024;
};
struct SlcBwdBarriers {
  // sdp_full / dq_full: one barrier per compute group (chunk parity).  A group only sees every other chunk, and a parity
  // wait on a barrier shared by both groups could not tell its chunk's completion from the one two chunks earlier.
  uint64_t kv_full, kv_empty, q_full[2], q_empty[2], sdp_full[2], sdp_free, dst_full, dq_full[2], dq_read, p_full, p_free[4], ds_full,
      ds_free[4], acc_full, acc_read;
  uint32_t tmem_base;
  int abort;
};

template <int DK, int DV>
__global__ void __launch_bounds__(384, 1)
slc_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ CUtensorMap tmQt, const __grid_constant__ CUtensorMap tmdOt, const SlcParams p) {
  using SM = SlcBwdSmem<DK, DV>;
  constexpr int MK1 = DK >= 128 ? 128 : 64, MK2 = DK - MK1;  // dK^T as one or two accumulators
  static_assert(MK2 == 0 || MK2 == 64, "dk is 64, 128 or 192");
  static_assert(DV == 64 || DV == 128, "dv is 64 or 128");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t *sK = smem + SM::oK, *sV = smem + SM::oV, *sSt = smem + SM::oSt, *sP = smem + SM::oP, *sdS = smem + SM::odS;
  SlcBwdBarriers* bar = reinterpret_cast<SlcBwdBarriers*>(smem + SM::oBar);
  volatile int* abort = &bar->abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bg = blockIdx.y, b = bg / p.G, g = bg % p.G;
  const int* off = p.csr_off + (int64_t)bg * (p.nblk + 1);
  const int* ent = p.csr_t + (int64_t)bg * p.Tq * p.nslots;
  const int e0 = blockIdx.x * kEntriesPerCta;
  const int qpc = 128 / p.hpg;
  // once any block has given up on a wait the device results are void: later blocks skip their work and end at once
  const bool has_work = e0 < off[p.nblk] && !(p.timeouts && *(volatile const int*)p.timeouts != 0);
  const int nseg = gridDim.x + p.nblk;

  if (threadIdx.x == 0) {
    mbar_init(&bar->kv_full, 1);
    mbar_init(&bar->kv_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->q_full[i], 1);
      mbar_init(&bar->q_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->sdp_full[i], 1);
      mbar_init(&bar->dq_full[i], 1);
    }
    mbar_init(&bar->sdp_free, 128);
    mbar_init(&bar->dst_full, 128);
    mbar_init(&bar->dq_read, 128);
    mbar_init(&bar->p_full, 64);
    mbar_init(&bar->ds_full, 64);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bar->p_free[i], 1);
      mbar_init(&bar->ds_free[i], 1);
    }
    mbar_init(&bar->acc_full, 1);
    mbar_init(&bar->acc_read, 256);
    bar->abort = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 8) tmem_alloc(&bar->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  constexpr uint32_t cS = 0, cdP = 64, cdQ = 128, cdV = 128 + DK, cdK1 = cdV + 64, cdK2 = cdK1 + 64;
  static_assert(cdK2 + (MK2 ? 64 : 0) <= 512, "TMEM columns");
  if (warp >= 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 136;");

  if (warp == 11) {
  } else if (!has_work) {
  } else if (warp == 9) {
    // producer warp: K/V block and gathered Q / dO rows by TMA (lane qi issues query qi)
    ChunkWalker w(off, p.nblk, e0, e0 + kEntriesPerCta, qpc);
    const int oob_row = p.B * p.H * p.Tq;
    const int oct0 = (b * p.H + g * p.hpg) >> 3;  // first head of the group, in units of 8 heads (rank-5 loads)
    bool ok = true;
    int c = 0, kvidx = -1, last_blk = -1;
    for (; !w.done(); w.next(), ++c) {
      const int cnt = w.count();
      int tok = p.Tq, row = oob_row;  // beyond the tensor: the tile is filled with zeros
      if (lane < cnt) {
        tok = ent[w.e + lane] & 0xFFFFFF;
        row = (int)(((int64_t)bg * p.Tq + tok) * p.hpg);
      }
      if (w.blk != last_blk) {
        last_blk = w.blk;
        ++kvidx;
        ok = mbar_wait_warp(&bar->kv_empty, (kvidx & 1) ^ 1, abort);
        if (!ok) break;
        if (lane == 0) {
          mbar_arrive_expect_tx(&bar->kv_full, SM::kK + SM::kV);
          tma_load_2d(&tmK, &bar->kv_full, sK, w.blk * 64, (b * p.G + g) * DK);
          for (int cc = 0; cc < DV / 64; ++cc)
            tma_load_2d(&tmV, &bar->kv_full, sV + cc * 8192, cc * 64, (b * p.G + g) * p.Tk + w.blk * 64);
        }
      }
      const int s = c & 1;
      // the stage is usually still busy: start the rows on their way to L2 so that the tile loads find them there
      if (lane < cnt && lane < qpc) {
        if (p.g5) {
          tma_prefetch_5d_outer(&tmQt, oct0, tok);
          tma_prefetch_5d_outer(&tmdOt, oct0, tok);
        } else {
#pragma unroll
          for (int cc = 0; cc < DK / 64; ++cc) tma_prefetch_2d(&tmQt, cc * 64, row);
#pragma unroll
          for (int cc = 0; cc < DV / 64; ++cc) tma_prefetch_2d(&tmdOt, cc * 64, row);
        }
      }
      ok = mbar_wait_warp(&bar->q_empty[s], ((c >> 1) & 1) ^ 1, abort);
      if (!ok) break;
      uint8_t* st = sSt + s * SM::kStage;
      if (lane == 0) mbar_arrive_expect_tx(&bar->q_full[s], SM::kQ + SM::kdO);
      __syncwarp();
      for (int qi = lane; qi < qpc; qi += 32) {
        const int r2 = qi < 32 ? row : (qi < cnt ? (int)(((int64_t)bg * p.Tq + (ent[w.e + qi] & 0xFFFFFF)) * p.hpg) : oob_row);
        if (p.g5) {
          tma_load_5d_outer(&tmQt, &bar->q_full[s], st + qi * p.hpg * (DK * 2), oct0, tok);
          tma_load_5d_outer(&tmdOt, &bar->q_full[s], st + SM::kQ + qi * p.hpg * (DV * 2), oct0, tok);
        } else {
          uint8_t* dst = st + qi * p.hpg * 128;
#pragma unroll
          for (int cc = 0; cc < DK / 64; ++cc) tma_load_2d(&tmQt, &bar->q_full[s], dst + cc * 16384, cc * 64, r2);
#pragma unroll
          for (int cc = 0; cc < DV / 64; ++cc) tma_load_2d(&tmdOt, &bar->q_full[s], dst + SM::kQ + cc * 16384, cc * 64, r2);
        }
      }
    }
    if (!ok && lane == 0) {
      if (kvidx >= 0) mbar_wait(&bar->kv_full, kvidx & 1, abort);
      for (int cc = max(0, c - 2); cc < c; ++cc) mbar_wait(&bar->q_full[cc & 1], (cc >> 1) & 1, abort);
    }
  } else if (warp == 8) {
    // UMMA issuer of the per-chunk chain (S, dQ, dP), warp-uniform, one elected lane issues.  Fixed order with blocking
    // waits: S(c+1) as soon as the compute warps hold S / dP of chunk c in registers, dQ(c) once dS(c) sits in TMEM, then
    // dP(c+1), which overwrites the dS columns and therefore follows dQ(c) in program order.  Where chunk c+1 starts
    // another block, S(c+1) waits until dQ(c) has been issued: the single K/V slot is refilled in between.
    constexpr uint32_t idS = idesc_bf16(128, 64, 0, 1);     // Q rows (K-major) x K block (keys contiguous)
    constexpr uint32_t iddP = idesc_bf16(128, 64, 0, 0);    // dO rows (K-major) x V block read K-major (dv contiguous)
    constexpr uint32_t iddQh = idesc_bf16(128, DK / 2, 0, 0);  // dS (TMEM) x half of the K block's dk rows, read K-major
    const uint64_t dKmn = smem_desc_sw128(smem_u32(sK), 16, 1024);
    const uint64_t dVk = smem_desc_sw128(smem_u32(sV), 16, 1024);
    const uint32_t sboQ = p.g5 ? (DK / 64) * 1024 : 1024, cbQ = p.g5 ? 1024 : 16384;  // Q tile: row-group / column-block strides
    const uint32_t sboO = p.g5 ? (DV / 64) * 1024 : 1024, cbO = p.g5 ? 1024 : 16384;  // dO tile
    ChunkWalker w(off, p.nblk, e0, e0 + kEntriesPerCta, qpc);
    bool ok = true;
    int kvidx = 0;
    auto issue_s = [&](int cc) -> bool {  // S of chunk cc: its rows have landed, S / dP of the chunk before are in registers
      const int s = cc & 1;
      if (!mbar_wait_warp(&bar->q_full[s], (cc >> 1) & 1, abort)) return false;
      if (cc > 0 && !mbar_wait_warp(&bar->sdp_free, (cc - 1) & 1, abort)) return false;
      tc_fence_after();
      const uint64_t dQ = smem_desc_sw128(smem_u32(sSt + s * SM::kStage), 16, sboQ);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk)
          umma_ss(tmem + cS, desc_advance(dQ, (kk >> 2) * cbQ + (kk & 3) * 32), desc_advance(dKmn, kk * 2048), idS, kk > 0);
      }
      __syncwarp();
      return true;
    };
    auto issue_dp = [&](int cc) {  // after S(cc) and, in program order, after dQ(cc - 1)
      const uint64_t ddO = smem_desc_sw128(smem_u32(sSt + (cc & 1) * SM::kStage) + SM::kQ, 16, sboO);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < DV / 16; ++kk)
          umma_ss(tmem + cdP, desc_advance(ddO, (kk >> 2) * cbO + (kk & 3) * 32), desc_advance(dVk, (kk >> 2) * 8192 + (kk & 3) * 32), iddP,
                  kk > 0);
        umma_commit(&bar->sdp_full[cc & 1]);
      }
      __syncwarp();
    };
    ok = mbar_wait_warp(&bar->kv_full, 0, abort);
    if (ok) ok = issue_s(0);
    if (ok) issue_dp(0);
    for (int c = 0; ok && !w.done(); ++c) {
      const int blk_c = w.blk;
      w.next();
      const bool have_next = !w.done(), switch_kv = have_next && w.blk != blk_c;
      if (have_next && !switch_kv) {
        ok = issue_s(c + 1);
        if (!ok) break;
      }
      // dQ partial of chunk c: dS is in TMEM, the accumulator has been drained by the previous chunk's epilogue
      ok = mbar_wait_warp(&bar->dst_full, c & 1, abort);
      if (ok && c > 0) ok = mbar_wait_warp(&bar->dq_read, (c - 1) & 1, abort);
      if (!ok) break;
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int hh2 = 0; hh2 < 2; ++hh2)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ts(tmem + cdQ + hh2 * (DK / 2), tmem + cdP + kk * 8, desc_advance(dKmn, hh2 * (DK / 2) * 128 + kk * 32), iddQh, kk > 0);
        umma_commit(&bar->dq_full[c & 1]);
        if (switch_kv) umma_commit(&bar->kv_empty);  // every MMA that reads the old block's K / V has been issued
      }
      __syncwarp();
      if (switch_kv) {
        ++kvidx;
        ok = mbar_wait_warp(&bar->kv_full, kvidx & 1, abort);
        if (ok) ok = issue_s(c + 1);
        if (!ok) break;
      }
      if (have_next) issue_dp(c + 1);
    }
  } else if (warp == 10) {
    // UMMA issuer of the transposed accumulations dV^T += dO^T P, dK^T += Q^T dS: per 64-row half of a chunk, in the order
    // the compute warps hand P and dS over.  Its MMAs touch only the accumulator columns, so they need no ordering
    // against the other issuer's.
    constexpr uint32_t iddV = idesc_bf16(DV, 64, 1, 1);     // dO^T (dv contiguous) x P (keys contiguous), K = gathered rows
    constexpr uint32_t iddK1 = idesc_bf16(MK1, 64, 1, 1);   // Q^T (dk contiguous) x dS (keys contiguous)
    constexpr uint32_t iddK2 = idesc_bf16(64, 64, 1, 1);
    const uint64_t dPb = smem_desc_sw128(smem_u32(sP), 16, 1024);    // one 64-key MN block: LBO unused
    const uint64_t dSb = smem_desc_sw128(smem_u32(sdS), 16, 1024);
    const uint32_t sboQ = p.g5 ? (DK / 64) * 1024 : 1024, cbQ = p.g5 ? 1024 : 16384;
    const uint32_t sboO = p.g5 ? (DV / 64) * 1024 : 1024, cbO = p.g5 ? 1024 : 16384;
    ChunkWalker w(off, p.nblk, e0, e0 + kEntriesPerCta, qpc);
    bool ok = true, fresh = true;      // fresh: the next accumulation starts a new segment
    int seg = 0, u = 0;
    for (int ch = 0; ok && !w.done(); ++ch) {
      const uint32_t st = smem_u32(sSt + (ch & 1) * SM::kStage);
      // transposed operands: 64-element runs along dk / dv, gathered rows 128 bytes apart inside an 8-row group
      const uint64_t dQt = smem_desc_sw128(st, cbQ, sboQ), dOt = smem_desc_sw128(st + SM::kQ, cbO, sboO);
      const int blk_c = w.blk;
      w.next();
      const bool last = w.done() || w.blk != blk_c;
#pragma unroll
      for (int h = 0; h < 2; ++h, ++u) {
        ok = mbar_wait_warp(&bar->p_full, u & 1, abort);
        // a new segment overwrites the accumulators: the previous segment's sums must have been read out
        if (ok && fresh && h == 0 && seg > 0) ok = mbar_wait_warp(&bar->acc_read, (seg - 1) & 1, abort);
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tmem + cdV, desc_advance(dOt, (h * 8 + kk * 2) * sboO), desc_advance(dPb, kk * 2048), iddV, !(fresh && h == 0 && kk == 0));
          umma_commit(&bar->p_free[u & 3]);
        }
        __syncwarp();
        ok = mbar_wait_warp(&bar->ds_full, u & 1, abort);
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            umma_ss(tmem + cdK1, desc_advance(dQt, (h * 8 + kk * 2) * sboQ), desc_advance(dSb, kk * 2048), iddK1,
                    !(fresh && h == 0 && kk == 0));
            if (MK2)
              umma_ss(tmem + cdK2, desc_advance(dQt, 2 * cbQ + (h * 8 + kk * 2) * sboQ), desc_advance(dSb, kk * 2048), iddK2,
                      !(fresh && h == 0 && kk == 0));
          }
          umma_commit(&bar->ds_free[u & 3]);
          if (h == 1) {
            umma_commit(&bar->q_empty[ch & 1]);  // the chunk's Q / dO stage is free again
            if (last) umma_commit(&bar->acc_full);  // last chunk of the block (or of the CTA): hand the accumulators over
          }
        }
        __syncwarp();
      }
      fresh = false;
      if (last) {
        ++seg;
        fresh = true;
      }
    }
  } else {
    // compute: one gathered row per thread; groups alternate chunks; both groups take part in every flush
    asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
    const int grp = warp >> 2, warp4 = warp & 3;
    const int r = warp4 * 32 + lane;
    const int half = warp4 >> 1, rr = r & 63;  // which 64-row half of the chunk this row is handed over in
    const uint32_t lane_base = (uint32_t)(warp4 * 32) << 16;
    ChunkWalker w(off, p.nblk, e0, e0 + kEntriesPerCta, qpc);
    bool ok = true;
    int c = 0, last_blk = -1, seg = 0;
    auto flush = [&](int blk) -> bool {
      if (!mbar_wait(&bar->acc_full, seg & 1, abort)) return false;
      tc_fence_after();
      const int64_t key_base = ((int64_t)bg * nseg + blockIdx.x + blk) * 64;
      if (grp == 0) {
        slc_flush_rows<MK1>(tmem + cdK1, p.dk_part, key_base, DK, 0, warp4, lane);
        if (MK2) slc_flush_rows<64>(tmem + cdK2, p.dk_part, key_base, DK, MK1, warp4, lane);
      } else {
        slc_flush_rows<DV>(tmem + cdV, p.dv_part, key_base, DV, 0, warp4, lane);
      }
      tc_fence_before();
      mbar_arrive(&bar->acc_read);
      ++seg;
      return true;
    };
    // this thread's row in a given chunk: entry (-1: row not in use), lse2 (+inf then, so P = 0), D
    const int qi = r / p.hpg, hh = r % p.hpg;
    int ent_next = -1;
    float lse_next = CUDART_INF_F, D_next = 0.f;
    auto fetch = [&](const ChunkWalker& wk) {
      ent_next = -1; lse_next = CUDART_INF_F; D_next = 0.f;
      if (!wk.done() && qi < wk.count()) {
        ent_next = ent[wk.e + qi];
        const int64_t srow = ((int64_t)b * p.H + g * p.hpg + hh) * p.Tq + (ent_next & 0xFFFFFF);
        lse_next = p.lse2[srow];
        D_next = p.D[srow];
      }
    };
    {
      ChunkWalker w0 = w;
      if (grp == 1 && !w0.done()) w0.next();
      fetch(w0);
    }
    for (; !w.done() && ok; w.next(), ++c) {
      if (w.blk != last_blk) {
        if (last_blk >= 0) ok = flush(last_blk);
        if (!ok) break;
        last_blk = w.blk;
      }
      if ((c & 1) != grp) continue;
      const int entry = ent_next;
      const float lse2 = lse_next, Dr = D_next;
      const int t = entry < 0 ? -1 : (entry & 0xFFFFFF), slot = entry < 0 ? 0 : (entry >> 24);
      const int chi = t < 0 ? -1 : p.q0 + t - w.blk * 64;
      {  // this group's next chunk: fetch its statistics one chunk ahead
        ChunkWalker w2 = w;
        w2.next();
        if (!w2.done()) w2.next();
        fetch(w2);
      }
      ok = mbar_wait(&bar->sdp_full[grp], (c >> 1) & 1, abort);
      if (!ok) break;
      tc_fence_after();
      uint32_t pP[32], pS[32];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t sv[32], dp[32];
        tmem_ld32(tmem + lane_base + cS + cc * 32, sv);
        tmem_ld32(tmem + lane_base + cdP + cc * 32, dp);
        tc_wait_ld();
        if (cc == 1) {  // both tiles are in registers: S of the next chunk may be issued
          tc_fence_before();
          mbar_arrive(&bar->sdp_free);
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int c0 = cc * 32 + 2 * e;
          const float p0 = c0 <= chi ? ex2(fmaf(__uint_as_float(sv[2 * e]), p.scale_log2, -lse2)) : 0.f;
          const float p1 = c0 + 1 <= chi ? ex2(fmaf(__uint_as_float(sv[2 * e + 1]), p.scale_log2, -lse2)) : 0.f;
          __nv_bfloat162 x = __floats2bfloat162_rn(p0, p1);
          __nv_bfloat162 y = __floats2bfloat162_rn(p0 * (__uint_as_float(dp[2 * e]) - Dr), p1 * (__uint_as_float(dp[2 * e + 1]) - Dr));
          pP[cc * 16 + e] = *reinterpret_cast<uint32_t*>(&x);
          pS[cc * 16 + e] = *reinterpret_cast<uint32_t*>(&y);
        }
      }
      // dS for the dQ MMA: bf16 over the first half of the dP columns (dP of the next chunk is issued after that MMA)
      tmem_st32(tmem + lane_base + cdP, pS);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&bar->dst_full);
      // hand-over of P / dS for the transposed accumulations: the staging tiles are used by (chunk, half) in order
      const int u = 2 * c + half;
      if (u > 0) {
        ok = mbar_wait(&bar->p_free[(u - 1) & 3], ((u - 1) >> 2) & 1, abort);
        if (!ok) break;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(sP + rr * 128 + ((j ^ (rr & 7)) << 4)) = make_uint4(pP[4 * j], pP[4 * j + 1], pP[4 * j + 2], pP[4 * j + 3]);
      fence_proxy_async();
      mbar_arrive(&bar->p_full);
      if (u > 0) {
        ok = mbar_wait(&bar->ds_free[(u - 1) & 3], ((u - 1) >> 2) & 1, abort);
        if (!ok) break;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(sdS + rr * 128 + ((j ^ (rr & 7)) << 4)) = make_uint4(pS[4 * j], pS[4 * j + 1], pS[4 * j + 2], pS[4 * j + 3]);
      fence_proxy_async();
      mbar_arrive(&bar->ds_full);
      // dQ partial of this chunk: TMEM -> registers -> this row of the partial array, one 32-byte sector per store
      __nv_bfloat16* drow = entry >= 0 ? p.dq_part + ((((int64_t)bg * p.Tq + t) * p.nslots + slot) * p.hpg + hh) * DK : nullptr;
      ok = mbar_wait(&bar->dq_full[grp], (c >> 1) & 1, abort);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < DK / 32; ++cc) {
        uint32_t ov[32];
        tmem_ld32(tmem + lane_base + cdQ + cc * 32, ov);
        tc_wait_ld();
        if (cc == DK / 32 - 1) {  // the accumulator sits in registers: the next chunk's dQ may be issued
          tc_fence_before();
          mbar_arrive(&bar->dq_read);
        }
        if (drow) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            uint32_t wv[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(ov[j * 16 + 2 * e]), __uint_as_float(ov[j * 16 + 2 * e + 1]));
              wv[e] = *reinterpret_cast<uint32_t*>(&a2);
            }
            st_global_v8(drow + cc * 32 + j * 16, wv);
          }
        }
      }
    }
    if (ok && last_blk >= 0) flush(last_blk);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && bar->abort) ptx::report_timeout(p.timeouts);
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// dK/dV of block `blk` += sum of its segment partials in segment order; a thread owns four consecutive columns of a row
__global__ void slc_reduce_dkv_kernel(const float* __restrict__ dk_part, const float* __restrict__ dv_part,
                                      const int* __restrict__ csr_off, __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                                      int G, int Tk, int nblk, int nparts, int DK, int DV, float scale) {
  const int blk = blockIdx.x, bg = blockIdx.y;
  const int* off = csr_off + (int64_t)bg * (nblk + 1);
  const int lo = off[blk], hi = off[blk + 1];
  if (hi <= lo) return;
  const int p_lo = lo / kEntriesPerCta, p_hi = (hi - 1) / kEntriesPerCta;
  const int nseg = nparts + nblk;
  const int W4 = (DK + DV) / 4, DK4 = DK / 4;
  for (int i = threadIdx.x; i < 64 * W4; i += blockDim.x) {
    const int r = i / W4, c4 = i - r * W4;
    const bool is_k = c4 < DK4;
    const int col = is_k ? c4 * 4 : (c4 - DK4) * 4, width = is_k ? DK : DV;
    const float* part = is_k ? dk_part : dv_part;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int pp = p_lo; pp <= p_hi; ++pp) {
      const int64_t sidx = ((int64_t)bg * nseg + pp + blk) * 64 + r;
      const float4 v = *reinterpret_cast<const float4*>(part + sidx * width + col);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const float mul = is_k ? scale : 1.f;
    const int64_t krow = (int64_t)bg * Tk + blk * 64 + r;
    __nv_bfloat16* dst = (is_k ? dk : dv) + krow * width + col;
    uint2 raw = *reinterpret_cast<const uint2*>(dst);
    float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    __nv_bfloat162 o0 = __floats2bfloat162_rn(a0.x + acc.x * mul, a0.y + acc.y * mul);
    __nv_bfloat162 o1 = __floats2bfloat162_rn(a1.x + acc.z * mul, a1.y + acc.w * mul);
    raw.x = *reinterpret_cast<uint32_t*>(&o0);
    raw.y = *reinterpret_cast<uint32_t*>(&o1);
    *reinterpret_cast<uint2*>(dst) = raw;
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static size_t al256(size_t x) { return (x + 255) & ~size_t(255); }

bool slc_sm100_supported(int H, int G, int Tq, int Tk, int dk, int dv, int nslots, int lprime) {
  const bool dims = (dk == 192 && dv == 128) || (dk == 128 && dv == 128) || (dk == 64 && dv == 64);
  if (!dims || G <= 0 || H % G != 0) return false;
  const int hpg = H / G;
  return hpg <= 128 && 128 % hpg == 0 && lprime == 64 && Tk % 64 == 0 && Tk > 0 && Tq > 0 && Tq < (1 << 24) &&
         nslots > 0 && nslots <= 32;  // (the caller also keeps B*H*Tq below 2^31: rows are 32-bit TMA coordinates)
}

size_t slc_fwd_sm100_workspace_bytes(int B, int H, int G, int Tq, int Tk, int dk, int dv, int nslots, int lprime) {
  const size_t rows = (size_t)B * H * Tq * nslots;
  return al256(slc_csr_workspace_bytes(B, G, Tq, Tk, nslots, lprime)) + al256(rows * dv * 2) + al256(rows * sizeof(float2)) +
         al256((size_t)B * H * Tq * dk * 2);
}

template <int W>
static int token_major_copy(const void* in, void* out, int B, int H, int G, int T, const char* what, cudaStream_t st) {
  const int64_t rows = (int64_t)B * H * T;
  KernelTimer kt(what, st);
  to_token_major_kernel<W><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, B, H, G, T);
  return check_launch(what);
}
static int token_major_copy_w(int W, const void* in, void* out, int B, int H, int G, int T, const char* what, cudaStream_t st) {
  if (W == 192) return token_major_copy<192>(in, out, B, H, G, T, what, st);
  if (W == 128) return token_major_copy<128>(in, out, B, H, G, T, what, st);
  return token_major_copy<64>(in, out, B, H, G, T, what, st);
}

template <int DK, int DV>
static int launch_slc_fwd_t(const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tqt, const CUtensorMap& top,
                            const SlcParams& p, const int* indices,
                            const int64_t* sidx, __nv_bfloat16* out, float* L, float* M, const SlcMix& mix, cudaStream_t st) {
  using SM = SlcFwdSmem<DK, DV>;
  auto kern = slc_fwd_kernel<DK, DV>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kDynamic) != cudaSuccess)
    return fail(NSA_ERR_LAUNCH, "slc_fwd: cannot reserve shared memory");
  const int nparts = (int)(((int64_t)p.Tq * p.nslots + kEntriesPerCta - 1) / kEntriesPerCta);
  {
    KernelTimer kt("slc_fwd", st);
    kern<<<dim3(nparts, p.B * p.G), 320, SM::kDynamic, st>>>(tk, tv, tqt, top, p);
  }
  if (int rc = check_launch("slc_fwd_sm100")) return rc;
  const int64_t rows = (int64_t)p.B * p.H * p.Tq;
  const size_t qbytes = (size_t)p.nslots * p.hpg * DV * 2;  // one query's partials
  KernelTimer kt(mix.out ? "slc_combine_fwd_mix" : "slc_combine_fwd", st);
  if (p.hpg <= 32 && qbytes <= 100 * 1024 && (int64_t)p.B * p.G * p.Tq < (1ll << 31)) {
    auto kc = slc_combine_fwd_bulk_kernel<DV>;
    if (cudaFuncSetAttribute(kc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)qbytes) != cudaSuccess)
      return fail(NSA_ERR_LAUNCH, "slc_combine_fwd: cannot reserve shared memory");
    kc<<<(unsigned)((int64_t)p.B * p.G * p.Tq), p.hpg * 32, qbytes, st>>>(p.o_part, p.st_part, indices, sidx[0], sidx[1], sidx[2], sidx[3],
                                                                      out, L, M, p.B, p.H, p.G, p.Tq, p.Tk, p.nslots, 64, p.q0, p.timeouts, mix);
  } else {
    slc_combine_fwd_kernel<DV><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(p.o_part, p.st_part, indices, sidx[0], sidx[1], sidx[2],
                                                                           sidx[3], out, L, M, p.B, p.H, p.G, p.Tq, p.Tk, p.nslots, 64, p.q0, mix);
  }
  return check_launch("slc_combine_fwd");
}

int slc_fwd_sm100(const void* q, const void* k, const void* v, const int* indices, const int64_t* sidx, void* out, float* L,
                  float* M, int B, int H, int G, int Tq, int Tk, int dk, int dv, int nslots, int lprime, float scale, int q0,
                  const SlcMix& mix, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (!slc_sm100_supported(H, G, Tq, Tk, dk, dv, nslots, lprime)) return fail(NSA_ERR_UNSUPPORTED, "slc_fwd_sm100: unsupported shape");
  const size_t need = slc_fwd_sm100_workspace_bytes(B, H, G, Tq, Tk, dk, dv, nslots, lprime);
  if (!workspace || workspace_bytes < need)
    return fail(NSA_ERR_WORKSPACE, "selection forward needs %zu workspace bytes, got %zu", need, workspace_bytes);
  SlcParams p = {};
  char* w = (char*)workspace;
  const size_t csr_bytes = al256(slc_csr_workspace_bytes(B, G, Tq, Tk, nslots, lprime));
  if (int rc = build_slc_csr(indices, sidx, B, G, Tq, Tk, nslots, lprime, 1, q0, w, csr_bytes, &p.csr_off, &p.csr_t, st)) return rc;
  p.q0 = q0;
  const size_t rows = (size_t)B * H * Tq * nslots;
  p.o_part = (__nv_bfloat16*)(w + csr_bytes);
  p.st_part = (float2*)(w + csr_bytes + al256(rows * dv * 2));
  void* qt = w + csr_bytes + al256(rows * dv * 2) + al256(rows * sizeof(float2));
  p.q = (const __nv_bfloat16*)q;
  p.B = B; p.H = H; p.G = G; p.Tq = Tq; p.Tk = Tk; p.nslots = nslots; p.nblk = (Tk + 63) / 64; p.hpg = H / G;
  p.scale = scale; p.scale_log2 = scale * kLog2ef;
  p.timeouts = fa_timeout_counter();
  CUtensorMap tk, tv;
  if (int rc = make_tmap_bf16_2d(&tk, k, (uint64_t)B * G * dk, Tk, dk)) return rc;
  if (int rc = make_tmap_bf16_2d(&tv, v, (uint64_t)B * G * Tk, dv, 64)) return rc;
  CUtensorMap tqt;
  // heads of a group filling whole 8-row swizzle atoms: one rank-5 tile load per query straight from q; otherwise the
  // rows of a query are first made contiguous (token-major copy) and fetched with one 2-D tile per 64 columns
  p.g5 = (H / G) % 8 == 0 ? 1 : 0;
  if (p.g5) {
    if (int rc = make_tmap_head_rows(&tqt, q, (uint64_t)B * H, Tq, H / G, dk)) return rc;
  } else {
    if (int rc = token_major_copy_w(dk, q, qt, B, H, G, Tq, "slc_q_token_major", st)) return rc;
    if (int rc = make_tmap_bf16_2d(&tqt, qt, (uint64_t)B * H * Tq, dk, H / G)) return rc;
  }
  CUtensorMap top;  // partial outputs as rows of dv values; one box = the heads of a group for one (query, slot)
  if (int rc = make_tmap_bf16_2d(&top, p.o_part, (uint64_t)rows, dv, (uint32_t)(H / G < 32 ? H / G : 32))) return rc;
  if (dk == 192 && dv == 128) return launch_slc_fwd_t<192, 128>(tk, tv, tqt, top, p, indices, sidx, (__nv_bfloat16*)out, L, M, mix, st);
  if (dk == 128 && dv == 128) return launch_slc_fwd_t<128, 128>(tk, tv, tqt, top, p, indices, sidx, (__nv_bfloat16*)out, L, M, mix, st);
  if (dk == 64 && dv == 64) return launch_slc_fwd_t<64, 64>(tk, tv, tqt, top, p, indices, sidx, (__nv_bfloat16*)out, L, M, mix, st);
  return fail(NSA_ERR_UNSUPPORTED, "slc_fwd_sm100: unsupported head dims");
}

// prep kernel shared with the dense backward (defined in fa_bwd_sm100.cu)
void launch_bwd_prep(const void* o, const void* dout, const float* L, const float* M, const float* delta, float* D, float* lse2,
                     int64_t rows, int dv, cudaStream_t st);

static void slc_bwd_layout(int B, int H, int G, int Tq, int Tk, int dk, int dv, int nslots, int lprime, size_t* o_stat,
                           size_t* o_dq, size_t* o_dk, size_t* o_dv, size_t* o_qt, size_t* o_dot, size_t* total) {
  const size_t rows = (size_t)B * H * Tq;
  const size_t nparts = ((size_t)Tq * nslots + kEntriesPerCta - 1) / kEntriesPerCta;
  const size_t nseg = nparts + (size_t)(Tk + 63) / 64;
  size_t o = al256(slc_csr_workspace_bytes(B, G, Tq, Tk, nslots, lprime));
  *o_stat = o; o += 2 * al256(rows * sizeof(float));
  *o_dq = o;   o += al256(rows * nslots * dk * 2);
  *o_dk = o;   o += al256((size_t)B * G * nseg * 64 * dk * sizeof(float));
  *o_dv = o;   o += al256((size_t)B * G * nseg * 64 * dv * sizeof(float));
  *o_qt = o;   o += al256(rows * dk * 2);
  *o_dot = o;  o += al256(rows * dv * 2);
  *total = o;
}

size_t slc_bwd_sm100_workspace_bytes(int B, int H, int G, int Tq, int Tk, int dk, int dv, int nslots, int lprime) {
  size_t a, b, c, d, e, f, total;
  slc_bwd_layout(B, H, G, Tq, Tk, dk, dv, nslots, lprime, &a, &b, &c, &d, &e, &f, &total);
  return total;
}

template <int DK, int DV>
static int launch_slc_bwd_t(const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tqt, const CUtensorMap& tdot,
                            const SlcParams& p, const int* indices,
                            const int64_t* sidx, __nv_bfloat16* dq, const void* add0, const void* add1, cudaStream_t st) {
  const int nparts = (int)(((int64_t)p.Tq * p.nslots + kEntriesPerCta - 1) / kEntriesPerCta);
  {
    auto kf = slc_bwd_fused_kernel<DK, DV>;
    if (cudaFuncSetAttribute(kf, cudaFuncAttributeMaxDynamicSharedMemorySize, SlcBwdSmem<DK, DV>::kDynamic) != cudaSuccess)
      return fail(NSA_ERR_LAUNCH, "slc_bwd: cannot reserve shared memory");
    KernelTimer kt("slc_bwd_fused", st);
    kf<<<dim3(nparts, p.B * p.G), 384, SlcBwdSmem<DK, DV>::kDynamic, st>>>(tk, tv, tqt, tdot, p);
  }
  if (int rc = check_launch("slc_bwd_fused_sm100")) return rc;
  const int64_t rows = (int64_t)p.B * p.H * p.Tq;
  {
    KernelTimer kt("slc_combine_dq", st);
    const size_t qbytes = (size_t)p.nslots * p.hpg * DK * 2;  // one query's partials
    if (p.hpg <= 32 && qbytes <= 100 * 1024 && (int64_t)p.B * p.G * p.Tq < (1ll << 31)) {
      auto kc = slc_combine_dq_bulk_kernel<DK>;
      if (cudaFuncSetAttribute(kc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)qbytes) != cudaSuccess)
        return fail(NSA_ERR_LAUNCH, "slc_combine_dq: cannot reserve shared memory");
      kc<<<(unsigned)((int64_t)p.B * p.G * p.Tq), p.hpg * 32, qbytes, st>>>(p.dq_part, indices, sidx[0], sidx[1], sidx[2], sidx[3], dq, p.B,
                                                                        p.H, p.G, p.Tq, p.Tk, p.nslots, 64, p.scale, p.q0, p.timeouts,
                                                                        (const __nv_bfloat16*)add0, (const __nv_bfloat16*)add1);
    } else {
      slc_combine_dq_kernel<DK><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(p.dq_part, indices, sidx[0], sidx[1], sidx[2], sidx[3], dq,
                                                                            p.B, p.H, p.G, p.Tq, p.Tk, p.nslots, 64, p.scale, p.q0,
                                                                            (const __nv_bfloat16*)add0, (const __nv_bfloat16*)add1);
    }
  }
  if (int rc = check_launch("slc_combine_dq")) return rc;
  KernelTimer kt("slc_reduce_dkv", st);
  slc_reduce_dkv_kernel<<<dim3(p.nblk, p.B * p.G), 256, 0, st>>>(p.dk_part, p.dv_part, p.csr_off, p.dk_out, p.dv_out, p.G, p.Tk,
                                                                 p.nblk, nparts, DK, DV, p.scale);
  return check_launch("slc_reduce_dkv");
}

int slc_bwd_sm100(const void* q, const void* k, const void* v, const int* indices, const int64_t* sidx, const void* out,
                  const void* dout, const float* L, const float* M, void* dq, void* dk_out, void* dv_out, int B, int H, int G,
                  int Tq, int Tk, int dk, int dv, int nslots, int lprime, float scale, int q0, const float* row_delta,
                  const void* dq_add0, const void* dq_add1, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (!slc_sm100_supported(H, G, Tq, Tk, dk, dv, nslots, lprime)) return fail(NSA_ERR_UNSUPPORTED, "slc_bwd_sm100: unsupported shape");
  size_t o_stat, o_dq, o_dk, o_dv, o_qt, o_dot, need;
  slc_bwd_layout(B, H, G, Tq, Tk, dk, dv, nslots, lprime, &o_stat, &o_dq, &o_dk, &o_dv, &o_qt, &o_dot, &need);
  if (!workspace || workspace_bytes < need)
    return fail(NSA_ERR_WORKSPACE, "selection backward needs %zu workspace bytes, got %zu", need, workspace_bytes);
  SlcParams p = {};
  char* w = (char*)workspace;
  if (int rc = build_slc_csr(indices, sidx, B, G, Tq, Tk, nslots, lprime, 1, q0, w, o_stat, &p.csr_off, &p.csr_t, st)) return rc;
  p.q0 = q0;
  const size_t rows = (size_t)B * H * Tq;
  float* D = (float*)(w + o_stat);
  float* lse2 = (float*)(w + o_stat + al256(rows * sizeof(float)));
  launch_bwd_prep(out, dout, L, M, row_delta, D, lse2, (int64_t)rows, dv, st);
  if (int rc = check_launch("fa_bwd_prep")) return rc;
  p.q = (const __nv_bfloat16*)q; p.dout = (const __nv_bfloat16*)dout;
  p.D = D; p.lse2 = lse2;
  p.dq_part = (__nv_bfloat16*)(w + o_dq);
  p.dk_part = (float*)(w + o_dk); p.dv_part = (float*)(w + o_dv);
  p.dk_out = (__nv_bfloat16*)dk_out; p.dv_out = (__nv_bfloat16*)dv_out;
  p.B = B; p.H = H; p.G = G; p.Tq = Tq; p.Tk = Tk; p.nslots = nslots; p.nblk = (Tk + 63) / 64; p.hpg = H / G;
  p.scale = scale; p.scale_log2 = scale * kLog2ef;
  p.timeouts = fa_timeout_counter();
  CUtensorMap tk, tv;
  if (int rc = make_tmap_bf16_2d(&tk, k, (uint64_t)B * G * dk, Tk, dk)) return rc;
  if (int rc = make_tmap_bf16_2d(&tv, v, (uint64_t)B * G * Tk, dv, 64)) return rc;
  CUtensorMap tqt, tdot;
  p.g5 = (H / G) % 8 == 0 ? 1 : 0;  // whole 8-row swizzle atoms per query: one rank-5 tile load per query and tensor
  if (p.g5) {
    if (int rc = make_tmap_head_rows(&tqt, q, (uint64_t)B * H, Tq, H / G, dk)) return rc;
    if (int rc = make_tmap_head_rows(&tdot, dout, (uint64_t)B * H, Tq, H / G, dv)) return rc;
  } else {
    if (int rc = token_major_copy_w(dk, q, w + o_qt, B, H, G, Tq, "slc_q_token_major", st)) return rc;
    if (int rc = token_major_copy_w(dv, dout, w + o_dot, B, H, G, Tq, "slc_do_token_major", st)) return rc;
    if (int rc = make_tmap_bf16_2d(&tqt, w + o_qt, (uint64_t)B * H * Tq, dk, H / G)) return rc;
    if (int rc = make_tmap_bf16_2d(&tdot, w + o_dot, (uint64_t)B * H * Tq, dv, H / G)) return rc;
  }
  if (dk == 192 && dv == 128) return launch_slc_bwd_t<192, 128>(tk, tv, tqt, tdot, p, indices, sidx, (__nv_bfloat16*)dq, dq_add0, dq_add1, st);
  if (dk == 128 && dv == 128) return launch_slc_bwd_t<128, 128>(tk, tv, tqt, tdot, p, indices, sidx, (__nv_bfloat16*)dq, dq_add0, dq_add1, st);
  if (dk == 64 && dv == 64) return launch_slc_bwd_t<64, 64>(tk, tv, tqt, tdot, p, indices, sidx, (__nv_bfloat16*)dq, dq_add0, dq_add1, st);
  return fail(NSA_ERR_UNSUPPORTED, "slc_bwd_sm100: unsupported head dims");
}

}  // namespace nsa

