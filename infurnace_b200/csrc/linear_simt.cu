// Matrix product out[n, o] = sum_k x[n, k] * w[o, k] with plain float32 multiply-adds: no tensor
// cores and no reduced-precision mode.  It is the product of the true 32-bit path and the
// fallback for operand dtypes or sizes that the tensor-core kernels refuse.  Any n, o, k.
//
// Each output element is summed by one thread over k in ascending order, so its value does not
// depend on how many rows the batch has or where the row stands in it.
#include "common.cuh"

#define TILE_N 64
#define TILE_O 64
#define TILE_K 16

// EPI 0: out = y.  EPI 1 (silu_gate): w has 2*o_out rows, gate rows first;
// out[n, o] = silu(y[n, o]) * y[n, o_out + o].
template <typename TX, typename TW, typename TO, int EPI>
__global__ void __launch_bounds__(256)
linear_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out, int n_rows, int o_out,
                   int k_dim) {
  __shared__ float xs[TILE_K][TILE_N + 1];
  __shared__ float ws[EPI ? 2 : 1][TILE_K][TILE_O + 1];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int tid = threadIdx.x;
  const int tn = tid / 16, to = tid % 16;          // thread's 4x4 patch: rows tn*4.., columns to*4..
  const int n0 = blockIdx.y * TILE_N, o0 = blockIdx.x * TILE_O;
  float acc[EPI ? 2 : 1][4][4];
#pragma unroll
  for (int e = 0; e < (EPI ? 2 : 1); ++e)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[e][i][j] = 0.f;

  for (int k0 = 0; k0 < k_dim; k0 += TILE_K) {
    // 64 rows x 16 k = 1024 elements per operand tile, 4 per thread
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int idx = tid + it * 256;
      const int r = idx / TILE_K, kk = idx % TILE_K;
      const int k = k0 + kk;
      float xv = 0.f;
      if (n0 + r < n_rows && k < k_dim) xv = to_f32<TX>(x[(size_t)(n0 + r) * k_dim + k]);
      xs[kk][r] = xv;
#pragma unroll
      for (int e = 0; e < (EPI ? 2 : 1); ++e) {
        float wv = 0.f;
        if (o0 + r < o_out && k < k_dim) wv = to_f32<TW>(w[((size_t)e * o_out + o0 + r) * k_dim + k]);
        ws[e][kk][r] = wv;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TILE_K; ++kk) {
      float xv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = xs[kk][tn * 4 + i];
#pragma unroll
      for (int e = 0; e < (EPI ? 2 : 1); ++e) {
        float wv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) wv[j] = ws[e][kk][to * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[e][i][j] = fmaf(xv[i], wv[j], acc[e][i][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int n = n0 + tn * 4 + i;
    if (n >= n_rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int o = o0 + to * 4 + j;
      if (o >= o_out) continue;
      float y = acc[0][i][j];
      if (EPI) { const float g = y; y = g / (1.f + expf(-g)) * acc[EPI ? 1 : 0][i][j]; }
      out[(size_t)n * o_out + o] = from_f32<TO>(y);
    }
  }
}

template <typename TX, typename TW, typename TO>
static int launch(const void* x, const void* w, void* out, int n, int o, int k, int epi, cudaStream_t s) {
  dim3 grid((o + TILE_O - 1) / TILE_O, (n + TILE_N - 1) / TILE_N);
  if (epi == 0)
    return ifb_launch(linear_simt_kernel<TX, TW, TO, 0>, grid, dim3(256), 0, s, (const TX*)x, (const TW*)w, (TO*)out, n, o, k);
  return ifb_launch(linear_simt_kernel<TX, TW, TO, 1>, grid, dim3(256), 0, s, (const TX*)x, (const TW*)w, (TO*)out, n, o, k);
}

// out_features is the width of `out` (for the silu_gate epilogue, half of w's rows).
IFB_EXPORT int ifb_linear_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype,
                               int n_rows, int out_features, int k_dim, int epilogue, cudaStream_t stream) {
  if (n_rows <= 0 || out_features <= 0) return IFB_OK;
  if (k_dim < 1) return IFB_ERR_SIZE;
  if (epilogue != 0 && epilogue != 1) return IFB_ERR_ARG;
  if ((n_rows + TILE_N - 1) / TILE_N > 65535) return IFB_ERR_SIZE;
  typedef __nv_bfloat16 bf;
  const int key = x_dtype * 4 + w_dtype * 2 + out_dtype;
  switch (key) {
    case 0: return launch<float, float, float>(x, w, out, n_rows, out_features, k_dim, epilogue, stream);
    case 1: return launch<float, float, bf>(x, w, out, n_rows, out_features, k_dim, epilogue, stream);
    case 2: return launch<float, bf, float>(x, w, out, n_rows, out_features, k_dim, epilogue, stream);
    case 3: return launch<float, bf, bf>(x, w, out, n_rows, out_features, k_dim, epilogue, stream);
    case 4: return launch<bf, float, float>(x, w, out, n_rows, out_features, k_dim, epilogue, stream);
    case 5: return launch<bf, float, bf>(x, w, out, n_rows, out_features, k_dim, epilogue, stream);
    case 6: return launch<bf, bf, float>(x, w, out, n_rows, out_features, k_dim, epilogue, stream);
    case 7: return launch<bf, bf, bf>(x, w, out, n_rows, out_features, k_dim, epilogue, stream);
  }
  return IFB_ERR_DTYPE;
}
