// C ABI of the attention entry points declared in include/nsa_b200.h, plus error reporting.
// Argument checking happens here; kernels never see a null pointer or an inconsistent size.
#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "attn_args.cuh"
#include "common.cuh"
#include "fa_sm100.cuh"
#include "slc_sm100.cuh"

namespace nsa {

char* error_buffer() {
  static thread_local char buf[512] = "";
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

namespace {
struct ProfRecord { const char* name; cudaEvent_t a, b; };
std::mutex g_prof_mu;
std::vector<ProfRecord> g_prof;
std::atomic<int> g_prof_on{0};
}  // namespace

KernelTimer::KernelTimer(const char* name, cudaStream_t st) : st_(st), slot_(-1) {
  if (!g_prof_on.load(std::memory_order_relaxed)) return;
  ProfRecord r;
  r.name = name;
  if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return;
  cudaEventRecord(r.a, st);
  std::lock_guard<std::mutex> lk(g_prof_mu);
  slot_ = (int)g_prof.size();
  g_prof.push_back(r);
}
KernelTimer::~KernelTimer() {
  if (slot_ < 0) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  cudaEventRecord(g_prof[slot_].b, st_);
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(NSA_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return NSA_OK;
}

static void fill_fwd_strides(AttnArgs& a, const int64_t* s) {
  for (int i = 0; i < 4; ++i) { a.sq[i] = s[i]; a.sk[i] = s[4 + i]; a.sv[i] = s[8 + i]; a.so[i] = s[12 + i]; }
  for (int i = 0; i < 3; ++i) { a.sL[i] = s[16 + i]; a.sM[i] = s[19 + i]; }
}
static void fill_bwd_strides(AttnArgs& a, const int64_t* s) {
  fill_fwd_strides(a, s);
  for (int i = 0; i < 4; ++i) { a.sdq[i] = s[22 + i]; a.sdk[i] = s[26 + i]; a.sdv[i] = s[30 + i]; }
}

static int check_common(const char* who, int B, int H, int G, int Tq, int Tk, int dk, int dv, int dtype) {
  NSA_REQUIRE(B >= 0 && H > 0 && G > 0 && H % G == 0, "%s: bad B/H/G = %d/%d/%d", who, B, H, G);
  NSA_REQUIRE(Tq >= 0 && Tk >= 0, "%s: negative sequence length", who);
  NSA_REQUIRE(dk > 0 && dk <= kMaxHeadDim && dv > 0 && dv <= kMaxHeadDim, "%s: head dims %d/%d outside 1..%d", who, dk,
              dv, kMaxHeadDim);
  NSA_REQUIRE(dtype == NSA_F32 || dtype == NSA_BF16, "%s: unsupported dtype %d", who, dtype);
  NSA_REQUIRE((int64_t)B * H <= 65535, "%s: B*H = %lld exceeds 65535", who, (long long)B * H);
  return NSA_OK;
}

template <typename T>
__global__ void add_dq_addends_kernel(T* __restrict__ dq, const T* __restrict__ a, const T* __restrict__ b, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float x = Elem<T>::ld(dq + i);
  if (a) x += Elem<T>::ld(a + i);
  if (b) x += Elem<T>::ld(b + i);
  Elem<T>::st(dq + i, x);
}

// canonical contiguous layouts: q [B,H,T,dk], k [B,G,dk,Tk] (strides given as z,g,n,k), v [B,G,Tk,dv], o [B,H,T,dv]
static bool canonical_fwd(const int64_t* s, int H, int G, int Tq, int Tk, int dk, int dv) {
  const int64_t q[4] = {(int64_t)H * Tq * dk, (int64_t)Tq * dk, dk, 1};
  const int64_t k[4] = {(int64_t)G * dk * Tk, (int64_t)dk * Tk, 1, Tk};
  const int64_t v[4] = {(int64_t)G * Tk * dv, (int64_t)Tk * dv, dv, 1};
  const int64_t o[4] = {(int64_t)H * Tq * dv, (int64_t)Tq * dv, dv, 1};
  const int64_t lm[3] = {(int64_t)H * Tq, Tq, 1};
  for (int i = 0; i < 4; ++i)
    if (s[i] != q[i] || s[4 + i] != k[i] || s[8 + i] != v[i] || s[12 + i] != o[i]) return false;
  for (int i = 0; i < 3; ++i)
    if (s[16 + i] != lm[i] || s[19 + i] != lm[i]) return false;
  return true;
}
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// canonical contiguous gradients: dq like q, dk [B,G,Tk,dk], dv [B,G,Tk,dv]
static bool tensor_core_bwd_ok(const int64_t* s, int dtype, int B, int H, int G, int Tq, int Tk, int dk, int dv,
                               const void* q, const void* k, const void* v, const void* o, const void* dout, const void* dq,
                               const void* dkey, const void* dval) {
  if (dtype != NSA_BF16 || !fa_fwd_sm100_supported(H, G, Tq, Tk, dk, dv)) return false;
  if (!canonical_fwd(s, H, G, Tq, Tk, dk, dv) || (int64_t)B * H > 65535) return false;
  const int64_t gq[4] = {(int64_t)H * Tq * dk, (int64_t)Tq * dk, dk, 1};
  const int64_t gk[4] = {(int64_t)G * Tk * dk, (int64_t)Tk * dk, dk, 1};
  const int64_t gv[4] = {(int64_t)G * Tk * dv, (int64_t)Tk * dv, dv, 1};
  for (int i = 0; i < 4; ++i)
    if (s[22 + i] != gq[i] || s[26 + i] != gk[i] || s[30 + i] != gv[i]) return false;
  return aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o) && aligned16(dout) && aligned16(dq) &&
         aligned16(dkey) && aligned16(dval);
}

static bool tensor_core_bwd_ok_slc(const int64_t* s, int dtype, int H, int G, int Tq, int Tk, int dk, int dv, const void* q,
                                   const void* k, const void* v, const void* o, const void* dout, const void* dq,
                                   const void* dkey, const void* dval) {
  if (dtype != NSA_BF16 || !canonical_fwd(s, H, G, Tq, Tk, dk, dv)) return false;
  const int64_t gq[4] = {(int64_t)H * Tq * dk, (int64_t)Tq * dk, dk, 1};
  const int64_t gk[4] = {(int64_t)G * Tk * dk, (int64_t)Tk * dk, dk, 1};
  const int64_t gv[4] = {(int64_t)G * Tk * dv, (int64_t)Tk * dv, dv, 1};
  for (int i = 0; i < 4; ++i)
    if (s[22 + i] != gq[i] || s[26 + i] != gk[i] || s[30 + i] != gv[i]) return false;
  return aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o) && aligned16(dout) && aligned16(dq) &&
         aligned16(dkey) && aligned16(dval);
}

}  // namespace nsa

using namespace nsa;

extern "C" NSA_API int nsa_profile_enable(int on) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (auto& r : g_prof) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
  g_prof.clear();
  g_prof_on.store(on ? 1 : 0);
  return NSA_OK;
}

extern "C" NSA_API int nsa_profile_report(char* buf, size_t buf_bytes) {
  NSA_REQUIRE(buf && buf_bytes > 0, "profile_report: no buffer");
  if (cudaDeviceSynchronize() != cudaSuccess) return fail(NSA_ERR_LAUNCH, "profile_report: device error");
  std::lock_guard<std::mutex> lk(g_prof_mu);
  std::map<std::string, std::pair<int, double>> agg;
  std::vector<std::string> order;
  for (auto& r : g_prof) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, r.a, r.b) != cudaSuccess) continue;
    auto it = agg.find(r.name);
    if (it == agg.end()) { agg[r.name] = {1, ms}; order.push_back(r.name); }
    else { it->second.first += 1; it->second.second += ms; }
  }
  size_t off = 0;
  buf[0] = 0;
  for (auto& n : order) {
    const int w = snprintf(buf + off, buf_bytes - off, "%s %d %.6f\n", n.c_str(), agg[n].first, agg[n].second);
    if (w < 0 || (size_t)w >= buf_bytes - off) break;
    off += (size_t)w;
  }
  return NSA_OK;
}

// An earlier tensor-core launch gave up on a bounded wait: everything launched since then skipped its work, so no entry
// point may report success until the caller has acknowledged it (nsa_device_timeouts(1)).
#define NSA_REFUSE_AFTER_TIMEOUT(what)                                                                                      \
  do {                                                                                                                      \
    if (timeout_flagged())                                                                                                  \
      return fail(NSA_ERR_LAUNCH, what ": a tensor-core kernel gave up on a barrier wait earlier (device time-out); results " \
                  "since then are invalid.  nsa_device_timeouts(1) reports and clears the condition");                      \
  } while (0)

#define NSA_NO_QUERY_OFFSET(what) \
  NSA_REQUIRE(q_pos0 == 0, what ": a query offset needs the bf16 tensor-core path of this call")

static bool want_tc(int flags) { return (flags & NSA_FLAG_GENERIC) == 0; }

extern "C" NSA_API int nsa_selftest_wait_timeout(long long limit_clocks, void* stream) {
  NSA_REQUIRE(limit_clocks > 0 && limit_clocks <= (1ll << 24), "selftest: limit must be within 1..2^24 clocks");
  if (int rc = wait_timeout_selftest(limit_clocks, nullptr, (cudaStream_t)stream)) return rc;
  if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) return fail(NSA_ERR_LAUNCH, "selftest: device error");
  return NSA_OK;
}

extern "C" NSA_API size_t nsa_attn_bwd_workspace_bytes(int B, int H, int G, int Tq, int Tk, int dk, int dv, int is_compression,
                                                       int window, int flags) {
  if (B <= 0 || H <= 0 || G <= 0 || Tq <= 0 || Tk <= 0 || H % G != 0) return 256;
  if (!is_compression && window <= 0) return 256;
  return fa_bwd_sm100_workspace_bytes(B, H, G, Tq, Tk, dk, dv, is_compression ? kCmp : kWin, is_compression ? 0 : window,
                                      (flags & NSA_FLAG_RECOMPUTE) != 0);
}

extern "C" NSA_API int nsa_device_timeouts(int reset) {
  int n = 0;
  if (int rc = fa_fwd_sm100_timeouts(&n, reset != 0)) return rc;
  return n;
}

extern "C" NSA_API const char* nsa_last_error(void) { return error_buffer(); }
extern "C" NSA_API const char* nsa_version(void) { return "nsa_b200 0.1.0 sm_100a"; }

extern "C" NSA_API int nsa_sliding_fwd(const void* q, const void* k, const void* v, void* out, float* L, float* M,
                               const int64_t* strides, int B, int H, int G, int T, int dk, int dv, int window,
                               float scale, int dtype, int flags, void* stream) {
  if (int rc = check_common("sliding_fwd", B, H, G, T, T, dk, dv, dtype)) return rc;
  NSA_REQUIRE(q && k && v && out && strides, "sliding_fwd: null pointer");
  NSA_REQUIRE(window > 0, "sliding_fwd: window must be positive");
  NSA_REFUSE_AFTER_TIMEOUT("sliding_fwd");
  if (want_tc(flags) && dtype == NSA_BF16 && L && M && fa_fwd_sm100_supported(H, G, T, T, dk, dv) &&
      canonical_fwd(strides, H, G, T, T, dk, dv) && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) &&
      (int64_t)B * (H / 2) <= 65535)
    return fa_fwd_sm100(q, k, v, out, L, M, B, H, G, T, T, dk, dv, kWin, window, 0, 0, 0, scale, nullptr, nullptr, (cudaStream_t)stream);
  AttnArgs a = {};
  a.q = q; a.k = k; a.v = v; a.o = out; a.L = L; a.M = M;
  fill_fwd_strides(a, strides);
  a.B = B; a.H = H; a.G = G; a.Tq = T; a.Tk = T; a.dk = dk; a.dv = dv; a.window = window; a.scale = scale; a.causal = 1;
  return launch_attn_generic(a, kWin, dtype, false, (cudaStream_t)stream);
}

extern "C" NSA_API int nsa_sliding_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                               const float* L, const float* M, void* dq, void* dkey, void* dval,
                               const int64_t* strides, int B, int H, int G, int T, int dk, int dv, int window,
                               float scale, int dtype, const float* row_delta, int flags, void* workspace,
                               size_t workspace_bytes, void* stream) {
  if (int rc = check_common("sliding_bwd", B, H, G, T, T, dk, dv, dtype)) return rc;
  NSA_REQUIRE(q && k && v && out && dout && L && M && dq && dkey && dval && strides, "sliding_bwd: null pointer");
  NSA_REQUIRE(window > 0, "sliding_bwd: window must be positive");
  NSA_REFUSE_AFTER_TIMEOUT("sliding_bwd");
  if (want_tc(flags) && tensor_core_bwd_ok(strides, dtype, B, H, G, T, T, dk, dv, q, k, v, out, dout, dq, dkey, dval))
    return fa_bwd_sm100(q, k, v, out, dout, L, M, dq, dkey, dval, B, H, G, T, T, dk, dv, kWin, window, 0, 0, 0, scale,
                        row_delta, workspace, workspace_bytes, (cudaStream_t)stream);
  AttnArgs a = {};
  a.q = q; a.k = k; a.v = v; a.o_in = out; a.dout = dout; a.Lc = L; a.Mc = M; a.dq = dq; a.dk_out = dkey; a.dv_out = dval;
  fill_bwd_strides(a, strides);
  a.B = B; a.H = H; a.G = G; a.Tq = T; a.Tk = T; a.dk = dk; a.dv = dv; a.window = window; a.scale = scale; a.causal = 1;
  return launch_attn_generic(a, kWin, dtype, true, (cudaStream_t)stream);
}

extern "C" NSA_API int nsa_cmp_attn_fwd(const void* q, const void* k_cmp, const void* v_cmp, const int32_t* block_ends,
                                void* out, float* L, float* M, const int64_t* strides, int B, int H, int G, int T,
                                int NB, int dk, int dv, float scale, int dtype, int blocks_l, int blocks_d,
                                int blocks_n, int q_pos0, int flags, const void* k_cmp_lo, float* lse2_out, void* stream) {
  if (int rc = check_common("cmp_attn_fwd", B, H, G, T, NB, dk, dv, dtype)) return rc;
  NSA_REQUIRE((k_cmp_lo == nullptr) == (lse2_out == nullptr), "cmp_attn_fwd: the low-order key part and the log-sum-exp output go together");
  NSA_REQUIRE(q && k_cmp && v_cmp && block_ends && out && strides, "cmp_attn_fwd: null pointer");
  NSA_REQUIRE(blocks_d >= 0 && (blocks_d == 0 || (blocks_l > 0 && blocks_n >= 0 && blocks_n <= NB)),
              "cmp_attn_fwd: bad block layout hint (l=%d, d=%d, n=%d)", blocks_l, blocks_d, blocks_n);
  NSA_REQUIRE(q_pos0 >= 0, "cmp_attn_fwd: negative query offset");
  NSA_REFUSE_AFTER_TIMEOUT("cmp_attn_fwd");
  if (want_tc(flags) && blocks_d > 0 && dtype == NSA_BF16 && L && M && fa_fwd_sm100_supported(H, G, T, NB, dk, dv) &&
      canonical_fwd(strides, H, G, T, NB, dk, dv) && aligned16(q) && aligned16(k_cmp) && aligned16(v_cmp) &&
      aligned16(out) && (int64_t)B * (H / 2) <= 65535)
    // block i is visible to the query at position q0 + t iff i*d + l - 1 <= q0 + t: the same rule with l - q0 for row t
    return fa_fwd_sm100(q, k_cmp, v_cmp, out, L, M, B, H, G, T, NB, dk, dv, kCmp, 0, blocks_l - q_pos0, blocks_d, blocks_n,
                        scale, k_cmp_lo, lse2_out, (cudaStream_t)stream);
  if (k_cmp_lo)
    return fail(NSA_ERR_UNSUPPORTED, "cmp_attn_fwd: the hi + lo key form needs the bf16 tensor-core path (see nsa_cmp_attn_exact_supported)");
  NSA_NO_QUERY_OFFSET("cmp_attn_fwd");
  AttnArgs a = {};
  a.q = q; a.k = k_cmp; a.v = v_cmp; a.o = out; a.L = L; a.M = M; a.block_ends = block_ends;
  fill_fwd_strides(a, strides);
  a.B = B; a.H = H; a.G = G; a.Tq = T; a.Tk = NB; a.dk = dk; a.dv = dv; a.scale = scale; a.causal = 1;
  return launch_attn_generic(a, kCmp, dtype, false, (cudaStream_t)stream);
}

extern "C" NSA_API int nsa_cmp_attn_exact_supported(int B, int H, int G, int T, int NB, int dk, int dv, int dtype) {
  return dtype == NSA_BF16 && B > 0 && fa_fwd_sm100_supported(H, G, T, NB, dk, dv) && (int64_t)B * (H / 2) <= 65535 ? 1 : 0;
}

extern "C" NSA_API int nsa_cmp_attn_bwd(const void* q, const void* k_cmp, const void* v_cmp, const int32_t* block_ends,
                                const void* out, const void* dout, const float* L, const float* M, void* dq,
                                void* dk_cmp, void* dv_cmp, const int64_t* strides, int B, int H, int G, int T, int NB,
                                int dk, int dv, float scale, int dtype, int blocks_l, int blocks_d, int blocks_n,
                                int q_pos0, const float* row_delta, int flags, void* workspace, size_t workspace_bytes,
                                void* stream) {
  if (int rc = check_common("cmp_attn_bwd", B, H, G, T, NB, dk, dv, dtype)) return rc;
  NSA_REQUIRE(q && k_cmp && v_cmp && block_ends && out && dout && L && M && dq && dk_cmp && dv_cmp && strides,
              "cmp_attn_bwd: null pointer");
  NSA_REQUIRE(blocks_d >= 0 && (blocks_d == 0 || (blocks_l > 0 && blocks_n >= 0 && blocks_n <= NB)),
              "cmp_attn_bwd: bad block layout hint (l=%d, d=%d, n=%d)", blocks_l, blocks_d, blocks_n);
  NSA_REQUIRE(q_pos0 >= 0, "cmp_attn_bwd: negative query offset");
  NSA_REFUSE_AFTER_TIMEOUT("cmp_attn_bwd");
  if (want_tc(flags) && blocks_d > 0 &&
      tensor_core_bwd_ok(strides, dtype, B, H, G, T, NB, dk, dv, q, k_cmp, v_cmp, out, dout, dq, dk_cmp, dv_cmp))
    return fa_bwd_sm100(q, k_cmp, v_cmp, out, dout, L, M, dq, dk_cmp, dv_cmp, B, H, G, T, NB, dk, dv, kCmp, 0,
                        blocks_l - q_pos0, blocks_d, blocks_n, scale, row_delta, workspace, workspace_bytes,
                        (cudaStream_t)stream);
  NSA_NO_QUERY_OFFSET("cmp_attn_bwd");
  AttnArgs a = {};
  a.q = q; a.k = k_cmp; a.v = v_cmp; a.o_in = out; a.dout = dout; a.Lc = L; a.Mc = M; a.block_ends = block_ends;
  a.dq = dq; a.dk_out = dk_cmp; a.dv_out = dv_cmp;
  fill_bwd_strides(a, strides);
  a.B = B; a.H = H; a.G = G; a.Tq = T; a.Tk = NB; a.dk = dk; a.dv = dv; a.scale = scale; a.causal = 1;
  return launch_attn_generic(a, kCmp, dtype, true, (cudaStream_t)stream);
}

static int slc_fwd_impl(const char* who, const void* q, const void* k, const void* v, const int32_t* indices, void* out, float* L,
                        float* M, const int64_t* strides, int B, int H, int G, int Tq, int Tkv, int n_slots, int l_prime, int dk,
                        int dv, float scale, int dtype, int q_pos0, int flags, const SlcMix& mix, void* workspace,
                        size_t workspace_bytes, void* stream) {
  if (int rc = check_common(who, B, H, G, Tq, Tkv, dk, dv, dtype)) return rc;
  NSA_REQUIRE(q && k && v && indices && out && strides, "%s: null pointer", who);
  NSA_REQUIRE(l_prime > 0 && n_slots >= 0, "%s: bad block size / slot count", who);
  NSA_REQUIRE(q_pos0 >= 0, "%s: negative query offset", who);
  if (timeout_flagged())
    return fail(NSA_ERR_LAUNCH, "%s: a tensor-core kernel gave up on a barrier wait earlier (device time-out); results since "
                "then are invalid.  nsa_device_timeouts(1) reports and clears the condition", who);
  if (want_tc(flags) && dtype == NSA_BF16 && L && M && B > 0 && slc_sm100_supported(H, G, Tq, Tkv, dk, dv, n_slots, l_prime) &&
      canonical_fwd(strides, H, G, Tq, Tkv, dk, dv) && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) &&
      (!mix.out || (aligned16(mix.out) && aligned16(mix.o_cmp) && aligned16(mix.o_win))))
    return slc_fwd_sm100(q, k, v, indices, strides + 22, out, L, M, B, H, G, Tq, Tkv, dk, dv, n_slots, l_prime, scale,
                         q_pos0, mix, workspace, workspace_bytes, (cudaStream_t)stream);
  NSA_REQUIRE(q_pos0 == 0, "%s: a query offset needs the bf16 tensor-core path of this call", who);
  AttnArgs a = {};
  a.q = q; a.k = k; a.v = v; a.o = out; a.L = L; a.M = M; a.indices = indices;
  fill_fwd_strides(a, strides);
  for (int i = 0; i < 4; ++i) a.sidx[i] = strides[22 + i];
  a.B = B; a.H = H; a.G = G; a.Tq = Tq; a.Tk = Tkv; a.dk = dk; a.dv = dv; a.scale = scale; a.causal = 1;
  a.nslots = n_slots; a.lprime = l_prime; a.nblk = (Tkv + l_prime - 1) / l_prime;
  if (int rc = launch_attn_generic(a, kSlc, dtype, false, (cudaStream_t)stream)) return rc;
  if (!mix.out) return NSA_OK;
  // stride-generic kernels: the mix runs as its own pass over the three branch outputs (contiguous [B,H,Tq,dv])
  NSA_REQUIRE(strides[15] == 1 && strides[14] == dv && strides[13] == (int64_t)Tq * dv && strides[12] == (int64_t)H * Tq * dv,
              "%s: the gate/mix epilogue needs a contiguous [B,H,T,dv] selection output", who);
  return nsa_gate_mix_fwd(mix.logits, mix.o_cmp, out, mix.o_win, mix.out, mix.gates, B, H, Tq, dv, mix.mode, dtype,
                          mix.token_major, stream);
}

extern "C" NSA_API int nsa_slc_fwd(const void* q, const void* k, const void* v, const int32_t* indices, void* out, float* L,
                           float* M, const int64_t* strides, int B, int H, int G, int Tq, int Tkv, int n_slots,
                           int l_prime, int dk, int dv, float scale, int dtype, int q_pos0, int flags, void* workspace,
                           size_t workspace_bytes, void* stream) {
  const SlcMix none = {};
  return slc_fwd_impl("slc_fwd", q, k, v, indices, out, L, M, strides, B, H, G, Tq, Tkv, n_slots, l_prime, dk, dv, scale, dtype,
                      q_pos0, flags, none, workspace, workspace_bytes, stream);
}

extern "C" NSA_API int nsa_slc_fwd_mix(const void* q, const void* k, const void* v, const int32_t* indices, void* out, float* L,
                               float* M, const int64_t* strides, int B, int H, int G, int Tq, int Tkv, int n_slots,
                               int l_prime, int dk, int dv, float scale, int dtype, int q_pos0, int flags,
                               const float* gate_logits, const void* o_cmp, const void* o_win, void* out_mixed,
                               float* gates_out, int gate_mode, int out_token_major, void* workspace,
                               size_t workspace_bytes, void* stream) {
  NSA_REQUIRE(gate_logits && o_cmp && o_win && out_mixed && gates_out, "slc_fwd_mix: null pointer");
  NSA_REQUIRE(gate_mode == NSA_GATE_SIGMOID || gate_mode == NSA_GATE_SOFTMAX, "slc_fwd_mix: bad gate mode %d", gate_mode);
  SlcMix mix = {};
  mix.logits = gate_logits; mix.o_cmp = o_cmp; mix.o_win = o_win; mix.out = out_mixed; mix.gates = gates_out;
  mix.mode = gate_mode; mix.token_major = out_token_major ? 1 : 0;
  return slc_fwd_impl("slc_fwd_mix", q, k, v, indices, out, L, M, strides, B, H, G, Tq, Tkv, n_slots, l_prime, dk, dv, scale,
                      dtype, q_pos0, flags, mix, workspace, workspace_bytes, stream);
}

extern "C" NSA_API size_t nsa_slc_fwd_workspace_bytes(int B, int H, int G, int Tq, int Tkv, int dk, int dv, int n_slots,
                                                      int l_prime, int dtype, int flags) {
  if (!want_tc(flags) || dtype != NSA_BF16 || B <= 0 || !slc_sm100_supported(H, G, Tq, Tkv, dk, dv, n_slots, l_prime)) return 256;
  return slc_fwd_sm100_workspace_bytes(B, H, G, Tq, Tkv, dk, dv, n_slots, l_prime);
}

extern "C" NSA_API size_t nsa_slc_bwd_workspace_bytes(int B, int H, int G, int Tq, int Tkv, int dk, int dv, int n_slots,
                                                      int l_prime, int dtype, int flags) {
  if (B <= 0 || G <= 0 || Tq <= 0 || Tkv <= 0 || n_slots <= 0 || l_prime <= 0) return 256;
  if (want_tc(flags) && dtype == NSA_BF16 && slc_sm100_supported(H, G, Tq, Tkv, dk, dv, n_slots, l_prime))
    return slc_bwd_sm100_workspace_bytes(B, H, G, Tq, Tkv, dk, dv, n_slots, l_prime);
  return slc_csr_workspace_bytes(B, G, Tq, Tkv, n_slots, l_prime);
}

extern "C" NSA_API int nsa_slc_bwd(const void* q, const void* k, const void* v, const int32_t* indices, const void* out,
                           const void* dout, const float* L, const float* M, void* dq, void* dkey, void* dval,
                           const int64_t* strides, int B, int H, int G, int Tq, int Tkv, int n_slots, int l_prime,
                           int dk, int dv, float scale, int dtype, int q_pos0, const float* row_delta,
                           const void* dq_add0, const void* dq_add1, int flags, void* workspace, size_t workspace_bytes,
                           void* stream) {
  if (int rc = check_common("slc_bwd", B, H, G, Tq, Tkv, dk, dv, dtype)) return rc;
  NSA_REQUIRE(q && k && v && indices && out && dout && L && M && dq && dkey && dval && strides, "slc_bwd: null pointer");
  NSA_REQUIRE(l_prime > 0 && n_slots > 0, "slc_bwd: bad block size / slot count");
  NSA_REQUIRE(q_pos0 >= 0, "slc_bwd: negative query offset");
  NSA_REFUSE_AFTER_TIMEOUT("slc_bwd");
  if (B == 0 || Tq == 0 || Tkv == 0) return NSA_OK;
  if (want_tc(flags) && slc_sm100_supported(H, G, Tq, Tkv, dk, dv, n_slots, l_prime) &&
      tensor_core_bwd_ok_slc(strides, dtype, H, G, Tq, Tkv, dk, dv, q, k, v, out, dout, dq, dkey, dval))
    return slc_bwd_sm100(q, k, v, indices, strides + 34, out, dout, L, M, dq, dkey, dval, B, H, G, Tq, Tkv, dk, dv, n_slots,
                         l_prime, scale, q_pos0, row_delta, dq_add0, dq_add1, workspace, workspace_bytes,
                         (cudaStream_t)stream);
  NSA_NO_QUERY_OFFSET("slc_bwd");
  const void *add0 = dq_add0, *add1 = dq_add1;
  if (add0 || add1)
    NSA_REQUIRE(strides[25] == 1 && strides[24] == dk && strides[23] == (int64_t)Tq * dk && strides[22] == (int64_t)H * Tq * dk,
                "slc_bwd: dQ addends need a contiguous [B,H,T,dk] dq");
  AttnArgs a = {};
  a.q = q; a.k = k; a.v = v; a.o_in = out; a.dout = dout; a.Lc = L; a.Mc = M; a.indices = indices;
  a.dq = dq; a.dk_out = dkey; a.dv_out = dval;
  fill_bwd_strides(a, strides);
  for (int i = 0; i < 4; ++i) a.sidx[i] = strides[34 + i];
  a.B = B; a.H = H; a.G = G; a.Tq = Tq; a.Tk = Tkv; a.dk = dk; a.dv = dv; a.scale = scale; a.causal = 1;
  a.nslots = n_slots; a.lprime = l_prime; a.nblk = (Tkv + l_prime - 1) / l_prime;
  cudaStream_t st = (cudaStream_t)stream;
  if (int rc = build_slc_csr(indices, a.sidx, B, G, Tq, Tkv, n_slots, l_prime, 1, 0, workspace, workspace_bytes,
                             &a.csr_off, &a.csr_t, st))
    return rc;
  if (int rc = launch_attn_generic(a, kSlc, dtype, true, st)) return rc;
  if (add0 || add1) {
    const int64_t n = (int64_t)B * H * Tq * dk;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == NSA_F32)
      add_dq_addends_kernel<float><<<blocks, 256, 0, st>>>((float*)dq, (const float*)add0, (const float*)add1, n);
    else
      add_dq_addends_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((__nv_bfloat16*)dq, (const __nv_bfloat16*)add0,
                                                                  (const __nv_bfloat16*)add1, n);
    return check_launch("slc_bwd dq addends");
  }
  return NSA_OK;
}
