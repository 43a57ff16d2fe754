// Inverse index for the selected-block attention backward: for every (batch, group, key block) the
// list of (query position | slot << 24) entries of the queries that selected the block, in ascending
// query order.
//
// The reference accumulates dK/dV of selected blocks with atomics from every query tile
// (nsa/kernels.py:1111-1115, 1140-1144); here each key block instead walks its own query list in a
// fixed order, which needs this "block -> queries" map.  It is a counting sort of the (query, slot)
// pairs by block id: per-chunk histograms, a scan, and an ordered fill.  Integer atomics are used
// only for counts, whose totals do not depend on the order of arrival.
#include "attn_args.cuh"
#include "common.cuh"

namespace nsa {

constexpr int kChunk = 128;  // queries per histogram chunk (one warp orders the entries of a chunk)

struct CsrArgs {
  const int* indices;
  int64_t sidx[4];
  int B, G, Tq, Tkv, nslots, lprime, nblk, nchunks, causal, q0;
  int *hist, *off, *csr_t;
};

__global__ void csr_count(const CsrArgs a) {
  extern __shared__ int sh[];
  const int c = blockIdx.x, bg = blockIdx.y, b = bg / a.G, g = bg % a.G;
  for (int i = threadIdx.x; i < a.nblk; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const int t0 = c * kChunk, t1 = min(a.Tq, t0 + kChunk);
  for (int e = threadIdx.x; e < (t1 - t0) * a.nslots; e += blockDim.x) {
    const int t = t0 + e / a.nslots, s = e % a.nslots;
    const int* row = a.indices + b * a.sidx[0] + g * a.sidx[1] + (int64_t)t * a.sidx[2];
    const int id = slot_block(row, a.sidx[3], s, a.q0 + t, a.Tkv, a.lprime, a.causal);
    if (id >= 0) atomicAdd(&sh[id], 1);
  }
  __syncthreads();
  int* h = a.hist + ((int64_t)bg * a.nchunks + c) * a.nblk;
  for (int i = threadIdx.x; i < a.nblk; i += blockDim.x) h[i] = sh[i];
}

// hist[bg][c][blk] becomes the count of entries of blk in chunks < c; off[bg][blk] the block's start.
__global__ void csr_scan(const CsrArgs a) {
  __shared__ int part[1024];
  const int bg = blockIdx.x, tid = threadIdx.x;
  int* h = a.hist + (int64_t)bg * a.nchunks * a.nblk;
  int* off = a.off + (int64_t)bg * (a.nblk + 1);
  const int per = (a.nblk + 1023) / 1024;
  const int lo = min(a.nblk, tid * per), hi = min(a.nblk, lo + per);
  int mine = 0;
  for (int blk = lo; blk < hi; ++blk) {
    int run = 0;
    for (int c = 0; c < a.nchunks; ++c) {
      const int v = h[(int64_t)c * a.nblk + blk];
      h[(int64_t)c * a.nblk + blk] = run;
      run += v;
    }
    off[blk + 1] = run;  // totals for now
    mine += run;
  }
  part[tid] = mine;
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int i = 0; i < 1024; ++i) {
      const int v = part[i];
      part[i] = run;
      run += v;
    }
    off[0] = 0;
  }
  __syncthreads();
  int run = part[tid];
  for (int blk = lo; blk < hi; ++blk) {
    const int v = off[blk + 1];
    run += v;
    off[blk + 1] = run;  // inclusive end = next block's start
  }
}

// One warp per chunk walks its queries in order; lanes cover (query, slot) pairs so that a lower lane
// is always an earlier query, and equal block ids inside a step are ranked by lane.
__global__ void csr_fill(const CsrArgs a, int slots_pad) {
  extern __shared__ int cur[];
  const int c = blockIdx.x, bg = blockIdx.y, b = bg / a.G, g = bg % a.G, lane = threadIdx.x;
  const int* h = a.hist + ((int64_t)bg * a.nchunks + c) * a.nblk;
  const int* off = a.off + (int64_t)bg * (a.nblk + 1);
  for (int i = lane; i < a.nblk; i += 32) cur[i] = off[i] + h[i];
  __syncwarp();
  int* out = a.csr_t + (int64_t)bg * a.Tq * a.nslots;
  const int qpw = 32 / slots_pad;  // queries per warp step
  const int t0 = c * kChunk, t1 = min(a.Tq, t0 + kChunk);
  for (int tb = t0; tb < t1; tb += qpw) {
    const int t = tb + lane / slots_pad, s = lane % slots_pad;
    int id = -1;
    if (t < t1 && s < a.nslots) {
      const int* row = a.indices + b * a.sidx[0] + g * a.sidx[1] + (int64_t)t * a.sidx[2];
      id = slot_block(row, a.sidx[3], s, a.q0 + t, a.Tkv, a.lprime, a.causal);
    }
    const unsigned peers = __match_any_sync(0xffffffffu, id >= 0 ? id : -1 - lane);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (id >= 0) out[cur[id] + rank] = t | (s << 24);  // query position and its slot
    __syncwarp();
    if (id >= 0 && rank == 0) cur[id] += __popc(peers);
    __syncwarp();
  }
}

static size_t align_up(size_t x) { return (x + 255) & ~size_t(255); }

static void csr_layout(int B, int G, int Tq, int Tkv, int nslots, int lprime, int* nblk, int* nchunks,
                       size_t* o_hist, size_t* o_off, size_t* o_t, size_t* total) {
  *nblk = (Tkv + lprime - 1) / lprime;
  *nchunks = (Tq + kChunk - 1) / kChunk;
  const size_t BG = (size_t)B * G;
  *o_hist = 0;
  *o_off = align_up(*o_hist + BG * *nchunks * *nblk * sizeof(int));
  *o_t = align_up(*o_off + BG * (*nblk + 1) * sizeof(int));
  *total = align_up(*o_t + BG * (size_t)Tq * nslots * sizeof(int));
}

size_t slc_csr_workspace_bytes(int B, int G, int Tq, int Tkv, int nslots, int lprime) {
  int nblk, nchunks;
  size_t a, b, c, total;
  csr_layout(B, G, Tq, Tkv, nslots, lprime, &nblk, &nchunks, &a, &b, &c, &total);
  return total;
}

int build_slc_csr(const int* indices, const int64_t* sidx, int B, int G, int Tq, int Tkv, int nslots,
                  int lprime, int causal, int q0, void* workspace, size_t workspace_bytes, const int** csr_off,
                  const int** csr_t, cudaStream_t st) {
  CsrArgs a;
  size_t o_hist, o_off, o_t, total;
  csr_layout(B, G, Tq, Tkv, nslots, lprime, &a.nblk, &a.nchunks, &o_hist, &o_off, &o_t, &total);
  if (!workspace || workspace_bytes < total)
    return fail(NSA_ERR_WORKSPACE, "selection backward needs %zu workspace bytes, got %zu", total, workspace_bytes);
  if (nslots > 32) return fail(NSA_ERR_UNSUPPORTED, "selection supports at most 32 slots per query here");
  if (Tq >= (1 << 24)) return fail(NSA_ERR_UNSUPPORTED, "selection inverse index supports fewer than 2^24 queries");
  if ((size_t)a.nblk * sizeof(int) > 160 * 1024) return fail(NSA_ERR_UNSUPPORTED, "too many key blocks (%d)", a.nblk);
  a.indices = indices;
  for (int i = 0; i < 4; ++i) a.sidx[i] = sidx[i];
  a.B = B; a.G = G; a.Tq = Tq; a.Tkv = Tkv; a.nslots = nslots; a.lprime = lprime; a.causal = causal; a.q0 = q0;
  char* w = (char*)workspace;
  a.hist = (int*)(w + o_hist);
  a.off = (int*)(w + o_off);
  a.csr_t = (int*)(w + o_t);
  const size_t sm = (size_t)a.nblk * sizeof(int);
  if (sm > 48 * 1024) {
    cudaFuncSetAttribute(csr_count, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    cudaFuncSetAttribute(csr_fill, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  }
  KernelTimer kt("slc_inverse_index", st);
  dim3 grid(a.nchunks, B * G);
  csr_count<<<grid, 256, sm, st>>>(a);
  if (int rc = check_launch("csr_count")) return rc;
  csr_scan<<<B * G, 1024, 0, st>>>(a);
  if (int rc = check_launch("csr_scan")) return rc;
  int slots_pad = 1;
  while (slots_pad < nslots) slots_pad *= 2;
  csr_fill<<<grid, 32, sm, st>>>(a, slots_pad);
  if (int rc = check_launch("csr_fill")) return rc;
  *csr_off = a.off;
  *csr_t = a.csr_t;
  return NSA_OK;
}

}  // namespace nsa
