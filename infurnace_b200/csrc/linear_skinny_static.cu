// The few-rows matrix product with its scratch memory inside the library: see linear_skinny_static.h
// for who needs this and for the rules of use.  The kernel is the one of linear_skinny.cu, included
// here unchanged; only the place the scratch comes from differs.
#include "linear_skinny.cu"
#include "linear_skinny_static.h"

// The scratch of every call on this device.  In host code these names are handles for the runtime,
// not device addresses: the addresses are looked up once per device below.
static __device__ __align__(256) float g_static_partials[IFB_STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) int g_static_counters[IFB_STATIC_SCRATCH_COUNTERS];

#include <mutex>

#define IFB_STATIC_MAX_DEVICES 64
static std::mutex g_setup_lock;                 // first calls from several threads: one looks up, the others wait
static float* g_partials_addr[IFB_STATIC_MAX_DEVICES];
static int* g_counters_addr[IFB_STATIC_MAX_DEVICES];

IFB_EXPORT void ifb_linear_skinny_static_need(int n_rows, int out_features, int epilogue, int splits, long long* floats,
                                              long long* counters) {
  ifb_linear_skinny_scratch(n_rows, out_features, epilogue, splits, floats, counters);
}

IFB_EXPORT int ifb_linear_skinny_static(const void* x, const void* w, void* out, int out_dtype, int n_rows,
                                        int out_features, int k_dim, int epilogue, int splits, cudaStream_t stream) {
  if (n_rows <= 0 || out_features <= 0) return IFB_OK;
  if (splits < 1) return IFB_ERR_ARG;
  if (k_dim < 8 || k_dim % 8) return IFB_ERR_SIZE;
  // the number of splits that will really run (no empty split), as the ordinary entry point computes it
  const int kps = ((k_dim + splits - 1) / splits + 127) / 128 * 128;
  const int real_splits = (k_dim + kps - 1) / kps;
  long long need_f = 0, need_c = 0;
  ifb_linear_skinny_scratch(n_rows, out_features, epilogue, real_splits, &need_f, &need_c);
  if (need_f > IFB_STATIC_SCRATCH_FLOATS || need_c > IFB_STATIC_SCRATCH_COUNTERS) return IFB_ERR_SIZE;

  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return -(int)e;
  if (dev < 0 || dev >= IFB_STATIC_MAX_DEVICES) return IFB_ERR_ARG;
  float* partials = nullptr;
  int* counters = nullptr;
  {
    std::lock_guard<std::mutex> hold(g_setup_lock);
    if (!g_partials_addr[dev] || !g_counters_addr[dev]) {      // set-up, once per device, with that device current
      float* p = nullptr;
      int* c = nullptr;
      e = cudaGetSymbolAddress((void**)&p, g_static_partials);
      if (e != cudaSuccess) return -(int)e;
      e = cudaGetSymbolAddress((void**)&c, g_static_counters);
      if (e != cudaSuccess) return -(int)e;
      if (!p || !c) return IFB_ERR_ARG;
      g_counters_addr[dev] = c;
      g_partials_addr[dev] = p;
    }
    partials = g_partials_addr[dev];
    counters = g_counters_addr[dev];
  }
  if (need_c > 0) {
    // the counters must start at zero; an earlier call that failed half-way may have left some raised
    e = cudaMemsetAsync(counters, 0, (size_t)need_c * sizeof(int), stream);
    if (e != cudaSuccess) return -(int)e;
  }
  return ifb_linear_skinny(x, w, out, out_dtype, real_splits > 1 ? partials : nullptr, real_splits > 1 ? counters : nullptr,
                           n_rows, out_features, k_dim, epilogue, real_splits, stream);
}
