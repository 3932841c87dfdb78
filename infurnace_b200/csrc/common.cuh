// Shared helpers of the kernel libraries: dtype codes, conversions, reductions.
// Every exported function returns 0 on success, a positive IFB_ERR_* code when it refuses
// its arguments, or the negated cudaError_t of a failed launch.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

#define IFB_F32 0
#define IFB_BF16 1

#define IFB_OK 0
#define IFB_ERR_DTYPE 1      // a dtype code or a combination of dtypes has no kernel
#define IFB_ERR_SIZE 2       // a size is outside what the kernel was written for
#define IFB_ERR_ALIGN 3      // a pointer or a row length breaks the kernel's alignment rule
#define IFB_ERR_ARG 4        // an argument contradicts another

// Codes that kernels record in the device error word (an int the caller passes and reads back later).  Codes below
// 900 are given by the kernels that wait on barriers: which wait gave up.
#define IFB_DEV_ERR_TOKEN_ID 900   // a token id outside the vocabulary reached the embedding

#define IFB_EXPORT extern "C" __attribute__((visibility("default")))

static inline int ifb_launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? IFB_OK : -(int)e;
}

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of these libraries is launched so that it may be
// scheduled while the kernel before it in the stream is still finishing: launch latency and the
// kernel's own set-up then overlap the predecessor's tail.  The price is a rule that every kernel
// keeps: nothing that a predecessor may have written is read, and nothing at all is written, before
// ifb_pdl_wait(), which returns once every kernel before this one has completed and its writes
// are visible.  What may come before the wait is work on constants (weights), such as asking the
// L2 cache to fetch them.  ifb_pdl_trigger() lets the next kernel in the stream start being
// scheduled; it is called right after the wait, so that one kernel, not the rest of the graph, runs
// ahead and sits on the SMs.  IFB_PDL=0 in the environment turns the launch attribute off.
__device__ __forceinline__ void ifb_pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void ifb_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void ifb_prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p)); }

// A bound in time for polled waits, beside their bound in polls (a poll of an mbarrier may itself block for a while, so
// a count of polls bounds nothing in seconds): true once more than IFB_WAIT_LIMIT_NS have passed since the wait's first
// look at the clock.  The clock is read every 256 polls; t0 starts as 0.
constexpr unsigned long long IFB_WAIT_LIMIT_NS = 2000000000ull;      // two seconds: a thousand times the longest honest wait
__device__ __forceinline__ bool ifb_wait_expired(uint32_t poll, unsigned long long& t0) {
  if ((poll & 255u) != 255u) return false;
  unsigned long long now;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
  if (t0 == 0) { t0 = now; return false; }
  return now - t0 > IFB_WAIT_LIMIT_NS;
}

static inline bool ifb_pdl_enabled() {
  static int on = -1;
  if (on < 0) { const char* e = getenv("IFB_PDL"); on = (e && e[0] == '0') ? 0 : 1; }
  return on != 0;
}

// The largest dynamic shared memory a kernel may be launched with is an attribute of (kernel, device), so what has been
// set is remembered per device, at the call site.  On failure the enclosing function returns the negated CUDA error.
#define IFB_MAX_DEVICES 64
#define IFB_ALLOW_SMEM(kernel, bytes)                                                                                   \
  do {                                                                                                                  \
    static size_t ifb_allowed_[IFB_MAX_DEVICES] = {};                                                                   \
    int ifb_dev_ = 0;                                                                                                   \
    if (cudaGetDevice(&ifb_dev_) != cudaSuccess || ifb_dev_ < 0 || ifb_dev_ >= IFB_MAX_DEVICES) return IFB_ERR_ARG;     \
    if ((size_t)(bytes) > 48 * 1024 && (size_t)(bytes) > ifb_allowed_[ifb_dev_]) {                                      \
      cudaError_t ifb_e_ = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes));     \
      if (ifb_e_ != cudaSuccess) return -(int)ifb_e_;                                                                   \
      ifb_allowed_[ifb_dev_] = (size_t)(bytes);                                                                         \
    }                                                                                                                   \
  } while (0)

// early: whether this launch may be scheduled before its predecessor has finished.  A kernel that lives on its bytes in
// flight is better off without: launched early, its CTAs sit on registers and shared memory of SMs where the
// predecessor still has CTAs to place, and at these sizes the launch latency that the overlap hides is small change.
template <typename... KArgs, typename... Args>
static inline int ifb_launch_opt(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (early && ifb_pdl_enabled()) ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
  if (e != cudaSuccess) { cudaGetLastError(); return -(int)e; }
  return IFB_OK;
}

template <typename... KArgs, typename... Args>
static inline int ifb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  return ifb_launch_opt(true, kernel, grid, block, smem, stream, args...);
}

// ---------------------------------------------------------------------------------------------
// A small host-side store of encoded tensor maps, for files that include <cuda.h> before this header.
// Encoding a map is a driver call of several microseconds; a step encodes the same few hundred maps
// (weights, activation buffers and page pools keep their addresses), so they are kept by their key.
#ifdef CUDA_VERSION
struct IfbMapKey {
  const void* ptr;
  unsigned long long dims[3], strides[2];
  unsigned box[3];
  int rank;
  bool operator==(const IfbMapKey& o) const {
    return ptr == o.ptr && rank == o.rank && dims[0] == o.dims[0] && dims[1] == o.dims[1] && dims[2] == o.dims[2] &&
           strides[0] == o.strides[0] && strides[1] == o.strides[1] && box[0] == o.box[0] && box[1] == o.box[1] && box[2] == o.box[2];
  }
};
typedef CUresult (*IfbEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                     const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// A bfloat16 tensor of rank 2 or 3 (dims and box innermost first, strides in bytes for dims 1..rank-1), 128-byte
// swizzle, zeros outside.  Returns IFB_OK or IFB_ERR_ARG.
static inline int ifb_tensor_map_bf16(CUtensorMap* out, const void* ptr, int rank, const unsigned long long* dims,
                                      const unsigned long long* strides, const unsigned* box) {
  constexpr int SLOTS = 4096;
  static IfbMapKey keys[SLOTS];
  static CUtensorMap maps[SLOTS];
  static bool used[SLOTS];
  static IfbEncodeTiledFn enc = nullptr;
  IfbMapKey k = {};
  k.ptr = ptr; k.rank = rank;
  for (int i = 0; i < rank; ++i) { k.dims[i] = dims[i]; k.box[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) k.strides[i] = strides[i];
  unsigned long long h = (unsigned long long)(uintptr_t)ptr * 0x9E3779B97F4A7C15ull;
  for (int i = 0; i < rank; ++i) h = (h ^ (k.dims[i] + 0x632BE59BD9B4E019ull * k.box[i])) * 0xD6E8FEB86659FD93ull;
  int slot = (int)((h >> 40) % SLOTS);
  for (int probe = 0; probe < 16; ++probe, slot = (slot + 1) % SLOTS) {
    if (used[slot] && keys[slot] == k) { *out = maps[slot]; return IFB_OK; }
    if (!used[slot]) break;
  }
  if (!enc) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return IFB_ERR_ARG;
    enc = (IfbEncodeTiledFn)fn;
  }
  cuuint64_t d[3] = {1, 1, 1}, st[2] = {0, 0};
  cuuint32_t b[3] = {1, 1, 1}, es[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) st[i] = strides[i];
  CUtensorMap m;
  if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return IFB_ERR_ARG;
  if (!used[slot]) { keys[slot] = k; maps[slot] = m; used[slot] = true; }      // a full neighbourhood: encode every time
  *out = m;
  return IFB_OK;
}
#endif

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Element i of an array whose dtype is known only at run time.
__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
  return dtype == IFB_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void store_from_f32(void* p, int dtype, size_t i, float v) {
  if (dtype == IFB_F32) ((float*)p)[i] = v; else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
