// Argument block shared by the attention kernels of the three NSA branches.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace nsa {

enum AttnMode { kWin = 0, kCmp = 1, kSlc = 2 };

struct AttnArgs {
  // forward
  const void *q, *k, *v;
  void* o;
  float *L, *M;
  // backward
  const void *o_in, *dout;
  const float *Lc, *Mc;
  void *dq, *dk_out, *dv_out;
  // masks
  const int* block_ends;  // kCmp: [Tk]
  const int* indices;     // kSlc: [B,G,Tq,nslots] with strides sidx
  const int* csr_off;     // kSlc backward: [B*G, nblk+1] offsets into csr_t
  const int* csr_t;       // kSlc backward: [B*G, Tq*nslots] entries (query position | slot << 24) grouped by key block
  // element strides; sk/sdk are ordered (z, g, n = key position, k = head dim)
  int64_t sq[4], sk[4], sv[4], so[4], sL[3], sM[3], sdq[4], sdk[4], sdv[4], sidx[4];
  int B, H, G, Tq, Tk, dk, dv;
  int window, nslots, lprime, nblk, causal;
  float scale;
};

// Block id held by slot s of a query's index row, or -1 when the slot contributes nothing: empty (-1),
// block starting beyond the keys or (causal) after the query, or an id already seen in an earlier slot.
__device__ __forceinline__ int slot_block(const int* row, int64_t sn, int s, int t, int Tkv, int lprime, int causal) {
  const int id = row[s * sn];
  if (id < 0) return -1;
  const int64_t beg = (int64_t)id * lprime;
  if (beg >= Tkv || (causal && beg > t)) return -1;
  for (int s2 = 0; s2 < s; ++s2)
    if (row[s2 * sn] == id) return -1;
  return id;
}

int launch_attn_generic(const AttnArgs& a, int mode, int dtype, bool backward, cudaStream_t st);

// Inverse index "key block -> queries that selected it" for the selection backward.
size_t slc_csr_workspace_bytes(int B, int G, int Tq, int Tkv, int nslots, int lprime);
int build_slc_csr(const int* indices, const int64_t* sidx, int B, int G, int Tq, int Tkv, int nslots,
                  int lprime, int causal, int q0, void* workspace, size_t workspace_bytes, const int** csr_off,
                  const int** csr_t, cudaStream_t st);

}  // namespace nsa
