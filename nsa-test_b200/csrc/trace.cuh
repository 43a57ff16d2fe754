// Optional timeline probe for development builds (-DNSA_TRACE): one thread block records clock64() at role
// hand-offs into a per-file device array that a reader function copies to the host.  Compiles to nothing otherwise.
#pragma once
#ifdef NSA_TRACE
#define NSA_TRACE_STORAGE static __device__ long long g_trace[4][128][16];
#define NSA_TR(role, c, ev)                                                                \
  do {                                                                                     \
    if (blockIdx.x == 3 && blockIdx.y == 0 && (c) < 128) g_trace[role][c][ev] = clock64(); \
  } while (0)
#define NSA_TRACE_READER(fn)                                                        \
  extern "C" __attribute__((visibility("default"))) int fn(long long* host) {       \
    return (int)cudaMemcpyFromSymbol(host, nsa::g_trace, sizeof(nsa::g_trace));     \
  }
#else
#define NSA_TRACE_STORAGE
#define NSA_TR(role, c, ev)
#define NSA_TRACE_READER(fn)
#endif
