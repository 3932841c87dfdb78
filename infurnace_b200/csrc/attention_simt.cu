// Attention over the paged cache, plain float32 arithmetic: one warp per (query token, query head).
// It serves every way a step can be cut (whole prompts, portions, single decoded tokens, mixed),
// any head size up to 256, any number of heads and groups, any page size, with or without a
// window, in float32 and in bfloat16 storage.  Scores, softmax and the weighted sum are float32.
//
// A query at position p reads the keys at positions first .. p from the pages its request's block
// table names, first = max(0, p - window + 1) with a window, else 0.  Block-table entries below
// `first` may be stale (-1): they are never read.
#include "common.cuh"
#include <math.h>

#define ATT_MAX_D 256

template <typename T>
__global__ void __launch_bounds__(128)
paged_attention_simt_kernel(const T* __restrict__ qkv, int row_stride, const T* __restrict__ pages,
                            const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ cu_q,
                            const int* __restrict__ seq_lens, T* __restrict__ out, int n_tokens, int n_req, int nq,
                            int nkv, int d, int page_size, float scale, int window) {
  extern __shared__ float sm[];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * warps + warp;
  if (item >= (long long)n_tokens * nq) return;
  const int tok = (int)(item / nq), h = (int)(item % nq);
  const int kvh = h / (nq / nkv);
  int lo = 0, hi = n_req;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (cu_q[mid] <= tok) lo = mid; else hi = mid; }
  const int r = lo;
  T* o = out + (size_t)tok * nq * d + (size_t)h * d;
  if (tok >= cu_q[n_req]) { for (int i = lane; i < d; i += 32) o[i] = from_f32<T>(0.f); return; }
  const int q_len = cu_q[r + 1] - cu_q[r];
  const int p = seq_lens[r] - q_len + (tok - cu_q[r]);
  if (p < 0) { for (int i = lane; i < d; i += 32) o[i] = from_f32<T>(0.f); return; }
  const int first = window > 0 ? max(0, p - window + 1) : 0;
  float* qs = sm + (size_t)warp * d;
  const T* qp = qkv + (size_t)tok * row_stride + (size_t)h * d;
  for (int i = lane; i < d; i += 32) qs[i] = to_f32<T>(qp[i]);
  __syncwarp();
  const int* bt = block_tables + (size_t)r * bt_stride;
  const size_t head_stride = (size_t)page_size * d, page_stride = 2 * (size_t)nkv * head_stride;
  float m = -INFINITY, l = 0.f;
  float acc[ATT_MAX_D / 32];
#pragma unroll
  for (int c = 0; c < ATT_MAX_D / 32; ++c) acc[c] = 0.f;
  for (int kb = first; kb <= p; kb += 32) {
    const int key = kb + lane;
    const bool valid = key <= p;
    float s = -INFINITY;
    if (valid) {
      const int page = bt[key / page_size];
      const T* kp = pages + (size_t)page * page_stride + (size_t)kvh * head_stride + (size_t)(key % page_size) * d;
      float dot = 0.f;
      for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32<T>(kp[i]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float pj = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int c = 0; c < ATT_MAX_D / 32; ++c) acc[c] *= corr;
    const int count = min(32, p - kb + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float pv = __shfl_sync(0xffffffffu, pj, jj);
      const int kj = kb + jj;
      const int page = bt[kj / page_size];
      const T* vp = pages + (size_t)page * page_stride + ((size_t)nkv + kvh) * head_stride + (size_t)(kj % page_size) * d;
#pragma unroll
      for (int c = 0; c < ATT_MAX_D / 32; ++c) {
        const int dim = lane + 32 * c;
        if (dim < d) acc[c] = fmaf(pv, to_f32<T>(vp[dim]), acc[c]);
      }
    }
    m = m_new;
  }
  const float inv = 1.f / l;
#pragma unroll
  for (int c = 0; c < ATT_MAX_D / 32; ++c) {
    const int dim = lane + 32 * c;
    if (dim < d) o[dim] = from_f32<T>(acc[c] * inv);
  }
}

IFB_EXPORT int ifb_paged_attention_simt(const void* qkv, int dtype, int row_stride, const void* pages,
                                        const int* block_tables, int bt_stride, const int* cu_q, const int* seq_lens,
                                        void* out, int n_tokens, int n_req, int nq, int nkv, int d, int page_size,
                                        float scale, int window, cudaStream_t stream) {
  if (n_tokens <= 0 || n_req <= 0) return IFB_OK;
  if (d < 1 || d > ATT_MAX_D) return IFB_ERR_SIZE;
  if (nkv < 1 || nq % nkv || page_size < 1 || window < 0) return IFB_ERR_ARG;
  const int warps = 4;
  const long long items = (long long)n_tokens * nq;
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  const size_t smem = (size_t)warps * d * sizeof(float);
  if (dtype == IFB_F32)
    return ifb_launch(paged_attention_simt_kernel<float>, dim3(blocks), dim3(warps * 32), smem, stream, (const float*)qkv,
                      row_stride, (const float*)pages, block_tables, bt_stride, cu_q, seq_lens, (float*)out, n_tokens, n_req,
                      nq, nkv, d, page_size, scale, window);
  if (dtype == IFB_BF16)
    return ifb_launch(paged_attention_simt_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, stream,
                      (const __nv_bfloat16*)qkv, row_stride, (const __nv_bfloat16*)pages, block_tables, bt_stride, cu_q,
                      seq_lens, (__nv_bfloat16*)out, n_tokens, n_req, nq, nkv, d, page_size, scale, window);
  return IFB_ERR_DTYPE;
}
