// Selected-block attention, tensor-core (tcgen05) key-block-major kernels: host entry points.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace nsa {

// bf16, canonical contiguous layouts, 64-key selection blocks, heads-per-group dividing 128
bool slc_sm100_supported(int H, int G, int Tq, int Tk, int dk, int dv, int nslots, int lprime);

// Gate + mix epilogue of the selection forward (out == null: none).  The kernel that merges a query's per-slot partials
// holds the finished O_slc row in registers; with the other two branch outputs given it also writes
// out = g0 o_cmp + g1 o_slc + g2 o_win (gates from logits [B,Tq,3H]: sigmoid or softmax over the three) and the gates,
// which saves the separate gate/mix pass its read of O_slc.  out is head-major [B,H,Tq,dv] or token-major [B,Tq,H,dv].
struct SlcMix {
  const float* logits;
  const void *o_cmp, *o_win;
  void* out;
  float* gates;  // [B,H,Tq,3]
  int mode, token_major;
};

size_t slc_fwd_sm100_workspace_bytes(int B, int H, int G, int Tq, int Tk, int dk, int dv, int nslots, int lprime);
int slc_fwd_sm100(const void* q, const void* k, const void* v, const int* indices, const int64_t* sidx, void* out, float* L,
                  float* M, int B, int H, int G, int Tq, int Tk, int dk, int dv, int nslots, int lprime, float scale, int q0,
                  const SlcMix& mix, void* workspace, size_t workspace_bytes, cudaStream_t st);


// row_delta: row sums dO.O [B,H,Tq] fp32 or null (computed here); dq_add0/1: dQ of the other branches (bf16, laid out like
// dq) added to the selection dQ in fp32 before the one rounding, or null.
size_t slc_bwd_sm100_workspace_bytes(int B, int H, int G, int Tq, int Tk, int dk, int dv, int nslots, int lprime);
int slc_bwd_sm100(const void* q, const void* k, const void* v, const int* indices, const int64_t* sidx, const void* out,
                  const void* dout, const float* L, const float* M, void* dq, void* dk_out, void* dv_out, int B, int H, int G,
                  int Tq, int Tk, int dk, int dv, int nslots, int lprime, float scale, int q0, const float* row_delta,
                  const void* dq_add0, const void* dq_add1, void* workspace, size_t workspace_bytes, cudaStream_t st);

}  // namespace nsa
