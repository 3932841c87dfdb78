// Embedding gather, RMSNorm with the residual addition, fused q/k norm + rotation + paged
// store, and sampling.  These kernels take every size: widths, head sizes and vocabularies
// need not be powers of two or multiples of anything (head_dim even when rotated).
#include "common.cuh"
#include <math.h>

// ------------------------------------------------------------------------------------------
// embed: out[n, :] = float(table[ids[n], :])
// An id outside [0, vocab) (ids may come straight from the sampling kernel of the step before, unseen by the
// host) reads no memory: the row is written as zeros and IFB_DEV_ERR_TOKEN_ID is recorded in *err (if given).
// ------------------------------------------------------------------------------------------
__global__ void embed_kernel(const void* __restrict__ table, int table_dtype, const int* __restrict__ ids,
                             float* __restrict__ out, int hidden, int vocab, int* __restrict__ err) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int n = blockIdx.x;
  const int id = ids[n];
  if (id < 0 || id >= vocab) {
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) out[(size_t)n * hidden + h] = 0.f;
    if (err && threadIdx.x == 0) atomicCAS(err, 0, IFB_DEV_ERR_TOKEN_ID);
    return;
  }
  const size_t row = (size_t)id * hidden;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x)
    out[(size_t)n * hidden + h] = load_as_f32(table, table_dtype, row + h);
}

IFB_EXPORT int ifb_embed(const void* table, int table_dtype, const int* ids, float* out, int n, int hidden, int vocab,
                         int* err, cudaStream_t stream) {
  if (n <= 0) return IFB_OK;
  if (table_dtype != IFB_F32 && table_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  if (vocab < 1) return IFB_ERR_SIZE;
  return ifb_launch(embed_kernel, dim3(n), dim3(256), 0, stream, table, table_dtype, ids, out, hidden, vocab, err);
}

// ------------------------------------------------------------------------------------------
// random_normal: out[i] = mean + std * z_i, z_i approximately N(0, 1), a pure function of (seed, i).
// z_i is the sum of twelve 16-bit integers, taken from three 64-bit words of a counter-based mixer at counters
// 3i, 3i+1, 3i+2, minus its mean, over 65536: integer arithmetic and then one exact scaling, one rounded multiply and
// one rounded addition (never contracted into a fused multiply-add), so that a host program doing the same steps in
// float32 gets the same bits.  The sum of twelve uniform terms has variance 1 and reaches +-6.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long rnd_mix(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, long long n, unsigned long long seed, float mean, float std) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int sum = 0;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const unsigned long long z = rnd_mix(seed + (3ull * (unsigned long long)i + j) * 0x9E3779B97F4A7C15ull);
      sum += (int)(z & 0xFFFF) + (int)((z >> 16) & 0xFFFF) + (int)((z >> 32) & 0xFFFF) + (int)(z >> 48);
    }
    const float zf = (float)(sum - 393210) * (1.0f / 65536.0f);
    out[i] = from_f32<T>(__fadd_rn(mean, __fmul_rn(std, zf)));
  }
}

IFB_EXPORT int ifb_random_normal(void* out, int dtype, long long n, unsigned long long seed, float mean, float std,
                                 cudaStream_t stream) {
  if (n <= 0) return IFB_OK;
  const unsigned blocks = (unsigned)((n + 1023) / 1024 < 148 * 16 ? (n + 1023) / 1024 : 148 * 16);
  if (dtype == IFB_F32) random_normal_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, n, seed, mean, std);
  else if (dtype == IFB_BF16) random_normal_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, n, seed, mean, std);
  else return IFB_ERR_DTYPE;
  return ifb_launch_status();
}

// ------------------------------------------------------------------------------------------
// rmsnorm: v = x[row] + sum_s delta[s][row];  out = v * rsqrt(mean(v^2) + eps) * w
// Without `rows`, row = blockIdx.x and v is written back to x.  With `rows`, row = rows[blockIdx.x]
// and x stays as it is.  One block per output row; v is kept in shared memory between the passes.
// ------------------------------------------------------------------------------------------
__global__ void rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, int num_splits,
                               size_t split_stride, const void* __restrict__ w, int w_dtype, float eps,
                               void* __restrict__ out, int out_dtype, const int* __restrict__ rows, int hidden) {
  extern __shared__ float vbuf[];
  __shared__ float scratch[33];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int orow = blockIdx.x;
  const int row = rows ? rows[orow] : orow;
  float* xr = x + (size_t)row * hidden;
  float ss = 0.f;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
    float v = xr[h];
    for (int s = 0; s < num_splits; ++s) v += delta[(size_t)s * split_stride + (size_t)row * hidden + h];
    vbuf[h] = v;
    if (!rows && num_splits) xr[h] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float r = rsqrtf(ss / (float)hidden + eps);
  for (int h = threadIdx.x; h < hidden; h += blockDim.x)
    store_from_f32(out, out_dtype, (size_t)orow * hidden + h, vbuf[h] * r * load_as_f32(w, w_dtype, h));
}

// The same with a block of 256 threads per row and the row in registers (16 bytes per thread and pass, all passes
// requested at once), for widths up to 1024 * IT that are a multiple of 4: one pass over global memory and one block
// barrier.
template <int IT>
__global__ void __launch_bounds__(256)
rmsnorm_block_kernel(float* __restrict__ x, const float* __restrict__ delta, int num_splits, size_t split_stride,
                     const void* __restrict__ w, int w_dtype, float eps, void* __restrict__ out, int out_dtype,
                     const int* __restrict__ rows, int hidden) {
  __shared__ float scratch[33];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int orow = blockIdx.x;
  const int row = rows ? rows[orow] : orow;
  float* xr = x + (size_t)row * hidden;
  float4 v[IT];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int idx = (it * 256 + threadIdx.x) * 4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (idx < hidden) {
      a = *reinterpret_cast<const float4*>(xr + idx);
      for (int sp = 0; sp < num_splits; ++sp) {
        const float4 d = *reinterpret_cast<const float4*>(delta + (size_t)sp * split_stride + (size_t)row * hidden + idx);
        a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
      }
      if (!rows && num_splits) *reinterpret_cast<float4*>(xr + idx) = a;
    }
    v[it] = a;
    ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  ss = block_sum(ss, scratch);
  const float r = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int idx = (it * 256 + threadIdx.x) * 4;
    if (idx >= hidden) break;
    float g0, g1, g2, g3;
    if (w_dtype == IFB_F32) {
      const float4 g = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + idx);
      g0 = g.x; g1 = g.y; g2 = g.z; g3 = g.w;
    } else {
      const uint2 g = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(w) + idx);
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&g.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&g.y);
      g0 = __low2float(lo); g1 = __high2float(lo); g2 = __low2float(hi); g3 = __high2float(hi);
    }
    const float y0 = v[it].x * r * g0, y1 = v[it].y * r * g1, y2 = v[it].z * r * g2, y3 = v[it].w * r * g3;
    if (out_dtype == IFB_F32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (size_t)orow * hidden + idx) = make_float4(y0, y1, y2, y3);
    } else {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
      uint2 pk;
      pk.x = *reinterpret_cast<const uint32_t*>(&lo); pk.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + (size_t)orow * hidden + idx) = pk;
    }
  }
}

template <int IT>
static int rmsnorm_block_launch(float* x, const float* delta, int num_splits, size_t split_stride, const void* w, int w_dtype,
                                float eps, void* out, int out_dtype, const int* rows, int num_out_rows, int hidden, cudaStream_t stream) {
  return ifb_launch(rmsnorm_block_kernel<IT>, dim3(num_out_rows), dim3(256), 0, stream, x, delta, num_splits, split_stride, w, w_dtype,
                    eps, out, out_dtype, rows, hidden);
}

IFB_EXPORT int ifb_rmsnorm(float* x, const float* delta, int num_splits, long long split_stride, const void* w,
                           int w_dtype, float eps, void* out, int out_dtype, const int* rows, int num_out_rows,
                           int hidden, cudaStream_t stream) {
  if (num_out_rows <= 0) return IFB_OK;
  if ((w_dtype != IFB_F32 && w_dtype != IFB_BF16) || (out_dtype != IFB_F32 && out_dtype != IFB_BF16)) return IFB_ERR_DTYPE;
  // the row in registers where the width allows 16-byte accesses (measured against a warp per row with the row in its
  // registers, in a chain of its own kind: 1.7 against 4.3 us at 64 rows of 1,024, 7.0 against 10.8 at 2,048 rows; a
  // warp's eight requests per tensor are too few in flight)
  if (hidden % 4 == 0 && hidden <= 8192 && !(((uintptr_t)x | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)out) & 15) &&
      (split_stride % 4) == 0) {
    const int ns = delta ? num_splits : 0;
#define IFB_RMS_CASE(IT) case IT: return rmsnorm_block_launch<IT>(x, delta, ns, (size_t)split_stride, w, w_dtype, eps, out, out_dtype, rows, num_out_rows, hidden, stream);
    switch ((hidden + 1023) / 1024) {
      IFB_RMS_CASE(1) IFB_RMS_CASE(2) IFB_RMS_CASE(3) IFB_RMS_CASE(4) IFB_RMS_CASE(5) IFB_RMS_CASE(6) IFB_RMS_CASE(7) IFB_RMS_CASE(8)
    }
#undef IFB_RMS_CASE
  }
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return IFB_ERR_SIZE;
  IFB_ALLOW_SMEM(rmsnorm_kernel, smem);
  const int threads = hidden >= 2048 ? 512 : 256;
  return ifb_launch(rmsnorm_kernel, dim3(num_out_rows), dim3(threads), smem, stream, x, delta, delta ? num_splits : 0,
                    (size_t)split_stride, w, w_dtype, eps, out, out_dtype, rows, hidden);
}

// ------------------------------------------------------------------------------------------
// rope_table: table[tok][i] = (cos, sin)(positions[tok] * inv_freq[i]), i < half.  A step computes it once and
// every layer's rotation reads it (the angles do not depend on the layer).
// ------------------------------------------------------------------------------------------
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int half,
                                  float2* __restrict__ table, int n_tokens) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_tokens * half) return;
  float s, c;
  sincosf((float)positions[idx / half] * inv_freq[idx % half], &s, &c);
  table[idx] = make_float2(c, s);
}

IFB_EXPORT int ifb_rope_table(const int* positions, const float* inv_freq, int half, float* table, int n_tokens,
                              cudaStream_t stream) {
  if (n_tokens <= 0 || half <= 0) return IFB_OK;
  const long long total = (long long)n_tokens * half;
  return ifb_launch(rope_table_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, positions, inv_freq, half,
                    reinterpret_cast<float2*>(table), n_tokens);
}

// ------------------------------------------------------------------------------------------
// qk_norm_rope_store: one warp per (token, head) of the fused qkv row [q heads | k heads | v heads].
//   q, k heads: optional RMSNorm over the head (weight shared by all heads), optional rotation of
//   the first rotary_dim elements by angle position * inv_freq[i]; written back in place.
//   k, v heads: stored to the page slot of the token, [page][k|v][kv_head][offset][d], when slot >= 0.
// Statistics, angles and the rotation are float32; sincosf is the accurate routine.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void qk_norm_rope_store_kernel(T* __restrict__ qkv, int n_tokens, int nq, int nkv, int d,
                                          const void* __restrict__ qw, const void* __restrict__ kw, int w_dtype,
                                          float eps, const float* __restrict__ inv_freq,
                                          const float* __restrict__ rope_table, int rotary_dim,
                                          int interleaved, const int* __restrict__ positions,
                                          const int* __restrict__ slots, T* __restrict__ pages, int page_size) {
  extern __shared__ float sm[];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const long long item = (long long)blockIdx.x * warps + warp;
  if (item >= (long long)n_tokens * heads) return;
  const int tok = (int)(item / heads), head = (int)(item % heads);
  float* buf = sm + (size_t)warp * d;
  T* src = qkv + (size_t)tok * heads * d + (size_t)head * d;
  const bool is_v = head >= nq + nkv, is_k = head >= nq && !is_v;
  const void* w = is_v ? nullptr : (is_k ? kw : qw);
  const bool rotate = !is_v && inv_freq != nullptr;
  const int slot = (slots && head >= nq) ? slots[tok] : -1;
  if (is_v) {
    if (slot >= 0) {
      const int kvh = head - nq - nkv;
      T* dst = pages + ((((size_t)(slot / page_size) * 2 + 1) * nkv + kvh) * page_size + (slot % page_size)) * d;
      for (int i = lane; i < d; i += 32) dst[i] = src[i];
    }
    return;
  }
  if (!w && !rotate && slot < 0) return;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) { float v = to_f32<T>(src[i]); buf[i] = v; ss += v * v; }
  if (w) {
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)d + eps);
    __syncwarp();
    for (int i = lane; i < d; i += 32) buf[i] = buf[i] * r * load_as_f32(w, w_dtype, i);
  }
  __syncwarp();
  T* dst = nullptr;
  if (slot >= 0) {
    const int kvh = head - nq;
    dst = pages + ((((size_t)(slot / page_size) * 2 + 0) * nkv + kvh) * page_size + (slot % page_size)) * d;
  }
  const float pos = rotate ? (float)positions[tok] : 0.f;
  const int half = rotary_dim >> 1;
  for (int i = lane; i < d; i += 32) {
    float v = buf[i];
    if (rotate && i < rotary_dim) {
      int pair, fi; bool first;
      if (interleaved) { first = (i & 1) == 0; pair = first ? i + 1 : i - 1; fi = i >> 1; }
      else { first = i < half; pair = first ? i + half : i - half; fi = first ? i : i - half; }
      float s, c;
      if (rope_table) { const float2 t = reinterpret_cast<const float2*>(rope_table)[(size_t)tok * half + fi]; c = t.x; s = t.y; }
      else sincosf(pos * inv_freq[fi], &s, &c);
      const float o = buf[pair];
      v = first ? v * c - o * s : v * c + o * s;
    }
    const T t = from_f32<T>(v);
    if (w || rotate) src[i] = t;
    if (dst) dst[i] = t;
  }
}

// The same for the common shape: the whole head is rotated in the half-split pairing (or nothing is) and the head
// size is 32 * EPL with EPL in {2, 4, 8}.  A lane keeps EPL consecutive elements in registers (one vector load and
// store), the element's partner in the rotation sits in lane ^ 16, and no shared memory is used.
template <typename T, int EPL> struct alignas(sizeof(T) * EPL) QkVec { T v[EPL]; };

constexpr int QK_HPW = 4;      // heads of one token that a warp of the vector kernel handles: the angles are computed once for them

template <typename T, int EPL>
__global__ void __launch_bounds__(128)
qk_norm_rope_store_vec_kernel(T* __restrict__ qkv, int n_tokens, int nq, int nkv, const void* __restrict__ qw,
                              const void* __restrict__ kw, int w_dtype, float eps, const float* __restrict__ inv_freq,
                              const float* __restrict__ rope_table, const int* __restrict__ positions,
                              const int* __restrict__ slots, T* __restrict__ pages, int page_size) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  constexpr int d = 32 * EPL;
  typedef QkVec<T, EPL> Vec;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const int blocks_per_token = (heads + QK_HPW - 1) / QK_HPW;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long long)n_tokens * blocks_per_token) return;
  const int tok = (int)(item / blocks_per_token), head0 = (int)(item % blocks_per_token) * QK_HPW;
  const int slot = slots ? slots[tok] : -1;
  // cos and sin of this lane's EPL angles, once for all heads of the block (lanes l and l ^ 16 share them)
  float cs[EPL], sn[EPL];
  if (inv_freq != nullptr && head0 < nq + nkv) {
    if (rope_table) {
      const float2* t = reinterpret_cast<const float2*>(rope_table) + (size_t)tok * (d / 2) + (lane & 15) * EPL;
#pragma unroll
      for (int e = 0; e < EPL; ++e) { cs[e] = t[e].x; sn[e] = t[e].y; }
    } else {
      const float pos = (float)positions[tok];
#pragma unroll
      for (int e = 0; e < EPL; ++e) sincosf(pos * inv_freq[(lane & 15) * EPL + e], &sn[e], &cs[e]);
    }
  }
  // all of the block's heads are requested before the first is worked on: four loads in flight per lane
  Vec in[QK_HPW];
#pragma unroll
  for (int hh = 0; hh < QK_HPW; ++hh)
    if (head0 + hh < heads) in[hh] = *reinterpret_cast<const Vec*>(qkv + (size_t)tok * heads * d + (size_t)(head0 + hh) * d + lane * EPL);
  // what does not depend on the head is computed once: the norm weights of this lane's elements and the token's
  // place in the pages
  float wq[EPL], wk[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    wq[e] = qw && head0 < nq ? load_as_f32(qw, w_dtype, lane * EPL + e) : 1.f;
    wk[e] = kw && head0 + QK_HPW > nq && head0 < nq + nkv ? load_as_f32(kw, w_dtype, lane * EPL + e) : 1.f;
  }
  size_t page_base = 0;
  if (slot >= 0) page_base = (size_t)(slot / page_size) * 2 * nkv * page_size + (slot % page_size);
  const bool rotate = inv_freq != nullptr;
#pragma unroll
  for (int hh = 0; hh < QK_HPW; ++hh) {
    const int head = head0 + hh;
    if (head >= heads) continue;
    T* src = qkv + (size_t)tok * heads * d + (size_t)head * d + lane * EPL;
    const bool is_v = head >= nq + nkv, is_k = head >= nq && !is_v;
    T* dst = nullptr;
    if (slot >= 0 && head >= nq)       // pages[page][k or v][kv head][place][d]
      dst = pages + (page_base + (size_t)(is_v ? nkv + head - nq - nkv : head - nq) * page_size) * d + lane * EPL;
    if (is_v) {
      if (dst) *reinterpret_cast<Vec*>(dst) = in[hh];
      continue;
    }
    const bool has_w = is_k ? kw != nullptr : qw != nullptr;
    if (!has_w && !rotate && !dst) continue;
    float v[EPL];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) { v[e] = to_f32<T>(in[hh].v[e]); ss += v[e] * v[e]; }
    if (has_w) {
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / (float)d + eps);
#pragma unroll
      for (int e = 0; e < EPL; ++e) v[e] = v[e] * r * (is_k ? wk[e] : wq[e]);
    }
    if (rotate) {
      const bool first = lane < 16;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float o = __shfl_xor_sync(0xffffffffu, v[e], 16);
        v[e] = first ? v[e] * cs[e] - o * sn[e] : v[e] * cs[e] + o * sn[e];
      }
    }
    Vec res;
#pragma unroll
    for (int e = 0; e < EPL; ++e) res.v[e] = from_f32<T>(v[e]);
    if (has_w || rotate) *reinterpret_cast<Vec*>(src) = res;
    if (dst) *reinterpret_cast<Vec*>(dst) = res;
  }
}

// The same for bfloat16 heads of 128 and steps of many tokens, where the bytes count: a warp takes 16 heads of one token,
// half a warp one head at a time with 16 bytes (8 elements) per lane: eight passes, all requested at once; the rotation
// partner of an element sits 8 lanes on.
__global__ void __launch_bounds__(128)
qk_norm_rope_store_d128_kernel(__nv_bfloat16* __restrict__ qkv, int n_tokens, int nq, int nkv, const void* __restrict__ qw,
                               const void* __restrict__ kw, int w_dtype, float eps, const float* __restrict__ rope_table,
                               const int* __restrict__ slots, __nv_bfloat16* __restrict__ pages, int page_size) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
#ifndef IFB_QK_B
#define IFB_QK_B 4
#endif
  constexpr int d = 128, B = IFB_QK_B;                         // B passes (two heads each) in flight
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane >> 4, l16 = lane & 15;
  const int heads = nq + 2 * nkv, groups = (heads + 2 * B - 1) / (2 * B);      // a warp takes 16 heads of a token
  const int item = blockIdx.x * (blockDim.x >> 5) + warp;
  const int tok = item / groups;
  if (tok >= n_tokens) return;
  const int slot = slots ? slots[tok] : -1;
  float cs[8], sn[8];                                          // the angles of elements l16 * 8 .. + 7 of the first half
  if (rope_table) {
    const float2* t = reinterpret_cast<const float2*>(rope_table) + (size_t)tok * (d / 2) + (l16 & 7) * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) { cs[e] = t[e].x; sn[e] = t[e].y; }
  }
  float wq[8], wk[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    wq[e] = qw ? load_as_f32(qw, w_dtype, l16 * 8 + e) : 1.f;
    wk[e] = kw ? load_as_f32(kw, w_dtype, l16 * 8 + e) : 1.f;
  }
  size_t page_base = 0;
  if (slot >= 0) page_base = (size_t)(slot / page_size) * 2 * nkv * page_size + (slot % page_size);
  __nv_bfloat16* row = qkv + (size_t)tok * heads * d;
  {
    const int h0 = (item % groups) * 2 * B;
    uint4 in[B];
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const int head = h0 + 2 * b + sub;
      in[b] = head < heads ? *reinterpret_cast<const uint4*>(row + (size_t)head * d + l16 * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const int head = h0 + 2 * b + sub;
      const bool live = head < heads;
      const bool is_v = head >= nq + nkv, is_k = head >= nq && !is_v;
      __nv_bfloat16* dst = nullptr;
      if (live && slot >= 0 && head >= nq)                    // pages[page][k or v][kv head][place][d]
        dst = pages + (page_base + (size_t)(is_v ? nkv + head - nq - nkv : head - nq) * page_size) * d + l16 * 8;
      const bool has_w = live && !is_v && (is_k ? kw != nullptr : qw != nullptr);
      const bool rotate = live && !is_v && rope_table != nullptr;
      float v[8];
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&in[b]);
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[2 * e] = __low2float(p2[e]); v[2 * e + 1] = __high2float(p2[e]);
        ss += v[2 * e] * v[2 * e] + v[2 * e + 1] * v[2 * e + 1];
      }
      // the sum over the head's 16 lanes (both halves of the warp do this together, each for its own head)
      ss += __shfl_xor_sync(0xffffffffu, ss, 8);
      ss += __shfl_xor_sync(0xffffffffu, ss, 4);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      if (has_w) {
        const float r = rsqrtf(ss / (float)d + eps);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = v[e] * r * (is_k ? wk[e] : wq[e]);
      }
      const bool first = l16 < 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float o = __shfl_xor_sync(0xffffffffu, v[e], 8);
        if (rotate) v[e] = first ? v[e] * cs[e] - o * sn[e] : v[e] * cs[e] + o * sn[e];
      }
      uint4 res = in[b];
      if (has_w || rotate) {
        __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int e = 0; e < 4; ++e) r2[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
        *reinterpret_cast<uint4*>(row + (size_t)head * d + l16 * 8) = res;
      }
      if (dst) *reinterpret_cast<uint4*>(dst) = res;
    }
  }
}

template <typename T>
static int qk_vec_launch(int epl, unsigned blocks, cudaStream_t stream, T* qkv, int n_tokens, int nq, int nkv, const void* qw,
                         const void* kw, int w_dtype, float eps, const float* inv_freq, const float* rope_table,
                         const int* positions, const int* slots, T* pages, int page_size) {
  if (epl == 2)
    return ifb_launch(qk_norm_rope_store_vec_kernel<T, 2>, dim3(blocks), dim3(128), 0, stream, qkv, n_tokens, nq, nkv, qw, kw,
                      w_dtype, eps, inv_freq, rope_table, positions, slots, pages, page_size);
  if (epl == 4)
    return ifb_launch(qk_norm_rope_store_vec_kernel<T, 4>, dim3(blocks), dim3(128), 0, stream, qkv, n_tokens, nq, nkv, qw, kw,
                      w_dtype, eps, inv_freq, rope_table, positions, slots, pages, page_size);
  return ifb_launch(qk_norm_rope_store_vec_kernel<T, 8>, dim3(blocks), dim3(128), 0, stream, qkv, n_tokens, nq, nkv, qw, kw,
                    w_dtype, eps, inv_freq, rope_table, positions, slots, pages, page_size);
}

IFB_EXPORT int ifb_qk_norm_rope_store(void* qkv, int dtype, int n_tokens, int nq, int nkv, int d, const void* qw,
                                      const void* kw, int w_dtype, float eps, const float* inv_freq,
                                      const float* rope_table, int rotary_dim, int interleaved, const int* positions,
                                      const int* slots, void* pages, int page_size, cudaStream_t stream) {
  if (n_tokens <= 0) return IFB_OK;
  if (d < 1 || d > 1024) return IFB_ERR_SIZE;
  if (inv_freq && (rotary_dim < 2 || rotary_dim > d || (rotary_dim & 1) || !positions)) return IFB_ERR_ARG;
  if (slots && (!pages || page_size < 1)) return IFB_ERR_ARG;
  if ((qw || kw) && w_dtype != IFB_F32 && w_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  const int warps = 4;
  const long long items = (long long)n_tokens * (nq + 2 * nkv);
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  if (d == 128 && dtype == IFB_BF16 && n_tokens >= 64 && (!inv_freq || (rotary_dim == d && !interleaved && rope_table)) &&
      ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)pages & 15) == 0)
    return ifb_launch(qk_norm_rope_store_d128_kernel,
                      dim3((unsigned)(((long long)n_tokens * ((nq + 2 * nkv + 2 * IFB_QK_B - 1) / (2 * IFB_QK_B)) + warps - 1) / warps)), dim3(warps * 32), 0, stream,
                      (__nv_bfloat16*)qkv, n_tokens, nq, nkv, qw, kw, w_dtype, eps, inv_freq ? rope_table : nullptr, slots,
                      (__nv_bfloat16*)pages, page_size);
  if ((d == 64 || d == 128 || d == 256) && (!inv_freq || (rotary_dim == d && !interleaved)) &&
      (dtype == IFB_F32 || dtype == IFB_BF16) && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)pages & 15) == 0) {
    const long long vitems = (long long)n_tokens * ((nq + 2 * nkv + QK_HPW - 1) / QK_HPW);
    const unsigned vblocks = (unsigned)((vitems + warps - 1) / warps);
    if (dtype == IFB_F32)
      return qk_vec_launch<float>(d / 32, vblocks, stream, (float*)qkv, n_tokens, nq, nkv, qw, kw, w_dtype, eps, inv_freq,
                                  rope_table, positions, slots, (float*)pages, page_size);
    return qk_vec_launch<__nv_bfloat16>(d / 32, vblocks, stream, (__nv_bfloat16*)qkv, n_tokens, nq, nkv, qw, kw, w_dtype, eps,
                                        inv_freq, rope_table, positions, slots, (__nv_bfloat16*)pages, page_size);
  }
  const size_t smem = (size_t)warps * d * sizeof(float);
  if (dtype == IFB_F32)
    return ifb_launch(qk_norm_rope_store_kernel<float>, dim3(blocks), dim3(warps * 32), smem, stream, (float*)qkv, n_tokens,
                      nq, nkv, d, qw, kw, w_dtype, eps, inv_freq, rope_table, rotary_dim, interleaved, positions, slots, (float*)pages,
                      page_size);
  if (dtype == IFB_BF16)
    return ifb_launch(qk_norm_rope_store_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, stream,
                      (__nv_bfloat16*)qkv, n_tokens, nq, nkv, d, qw, kw, w_dtype, eps, inv_freq, rope_table, rotary_dim, interleaved,
                      positions, slots, (__nv_bfloat16*)pages, page_size);
  return IFB_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------
// sample: one block per row of float32 logits.
//   temperature == 0: index of the largest logit, the lowest index among equals.
//   else: smallest i with sum_{j<=i} exp((l_j - max)/T) > u * sum_j exp((l_j - max)/T).
// Each thread owns a contiguous chunk of the row, so the running sum follows index order.
// ------------------------------------------------------------------------------------------
__global__ void sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                              const float* __restrict__ uniform, int* __restrict__ out) {
  __shared__ float scratch[33];
  __shared__ float sums[1024];
  __shared__ int best_idx[32];
  __shared__ float best_val[32];
  __shared__ int chosen;
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int row = blockIdx.x, tid = threadIdx.x, nthreads = blockDim.x;
  const float* l = logits + (size_t)row * vocab;
  const float temp = temperature ? temperature[row] : 0.f;
  const int chunk = (vocab + nthreads - 1) / nthreads;
  const int begin = min(vocab, tid * chunk), end = min(vocab, begin + chunk);
  // the largest value and its lowest index; the row is walked with consecutive threads on consecutive
  // elements (any partition gives the same answer, since ties go to the lower index)
  float bv = -INFINITY; int bi = 0;      // a row without any comparable value (all NaN) gives index 0, never an id outside the vocabulary
  if ((((uintptr_t)l) & 15) == 0) {      // 16-byte loads, four in flight per thread
    const int v4 = vocab >> 2;
    const float4* l4 = reinterpret_cast<const float4*>(l);
#pragma unroll 4
    for (int i = tid; i < v4; i += nthreads) {
      const float4 v = l4[i];
      const int b = i << 2;
      if (v.x > bv || (v.x == bv && b < bi)) { bv = v.x; bi = b; }
      if (v.y > bv || (v.y == bv && b + 1 < bi)) { bv = v.y; bi = b + 1; }
      if (v.z > bv || (v.z == bv && b + 2 < bi)) { bv = v.z; bi = b + 2; }
      if (v.w > bv || (v.w == bv && b + 3 < bi)) { bv = v.w; bi = b + 3; }
    }
    for (int i = (v4 << 2) + tid; i < vocab; i += nthreads) { const float v = l[i]; if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; } }
  } else {
    for (int i = tid; i < vocab; i += nthreads) { const float v = l[i]; if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; } }
  }
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, bv, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if ((tid & 31) == 0) { best_val[tid >> 5] = bv; best_idx[tid >> 5] = bi; }
  __syncthreads();
  if (tid < 32) {
    const int nw = (nthreads + 31) >> 5;
    bv = tid < nw ? best_val[tid] : -INFINITY; bi = tid < nw ? best_idx[tid] : 0;
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (tid == 0) { best_val[0] = bv; best_idx[0] = bi; }
  }
  __syncthreads();
  const float mx = best_val[0];
  if (temp == 0.f) { if (tid == 0) out[row] = best_idx[0]; return; }
  const float inv_t = 1.f / temp;
  float part = 0.f;
  for (int i = begin; i < end; ++i) part += expf((l[i] - mx) * inv_t);
  sums[tid] = part;
  const float total = block_sum(part, scratch);
  const float target = uniform[row] * total;
  if (tid == 0) {
    // walk the chunk sums in index order, then the elements of the chunk that crosses the target
    float run = 0.f; int t = 0;
    for (; t < nthreads; ++t) { if (run + sums[t] > target) break; run += sums[t]; }
    int pick = -1;
    if (t < nthreads) {
      const int b = min(vocab, t * chunk), e = min(vocab, b + chunk);
      for (int i = b; i < e; ++i) { run += expf((l[i] - mx) * inv_t); if (run > target) { pick = i; break; } }
      if (pick < 0) pick = e - 1;
    }
    if (pick < 0) {   // rounding left the target unreached: the last index with non-zero weight
      pick = best_idx[0];
      for (int i = vocab - 1; i >= 0; --i) if (expf((l[i] - mx) * inv_t) > 0.f) { pick = i; break; }
    }
    chosen = min(max(pick, 0), vocab - 1);
  }
  __syncthreads();
  if (tid == 0) out[row] = chosen;
}

// ------------------------------------------------------------------------------------------
// argmax of every row with several blocks per row (greedy sampling of a large vocabulary: one block per row leaves
// most of the device idle).  Block (b, row) scans slice b of the row and writes its (largest value, lowest index of
// it); the block of a row that finishes last (a counter per row, which it sets back to zero) takes the best of the
// slices, the lowest index among equals, so the result is the one of sample_kernel.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
argmax_rows_kernel(const float* __restrict__ logits, int vocab, float* __restrict__ part_val, int* __restrict__ part_idx,
                   int* __restrict__ counters, int* __restrict__ out) {
  __shared__ float best_val[8];
  __shared__ int best_idx[8];
  __shared__ int is_last;
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int row = blockIdx.y, b = blockIdx.x, bpr = gridDim.x, tid = threadIdx.x;
  const float* l = logits + (size_t)row * vocab;
  const int chunk = ((vocab + bpr - 1) / bpr + 3) & ~3;
  const int begin = min(vocab, b * chunk), end = min(vocab, begin + chunk);
  float bv = -INFINITY; int bi = 0;      // a slice without any comparable value (all NaN) gives index 0
  auto take = [&](float v, int i) { if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; } };
  if ((((uintptr_t)l) & 15) == 0) {
    const int v4 = (end - begin) >> 2;
    const float4* l4 = reinterpret_cast<const float4*>(l + begin);
#pragma unroll 4
    for (int i = tid; i < v4; i += 256) {
      const float4 v = l4[i];
      const int at = begin + (i << 2);
      take(v.x, at); take(v.y, at + 1); take(v.z, at + 2); take(v.w, at + 3);
    }
    for (int i = begin + (v4 << 2) + tid; i < end; i += 256) take(l[i], i);
  } else {
    for (int i = begin + tid; i < end; i += 256) take(l[i], i);
  }
  if (bv == -INFINITY && bi == 0) bi = begin < vocab ? begin : 0;     // nothing taken: stay inside the slice
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if ((tid & 31) == 0) { best_val[tid >> 5] = bv; best_idx[tid >> 5] = bi; }
  __syncthreads();
  if (tid == 0) {
    for (int wv = 1; wv < 8; ++wv)
      if (best_val[wv] > bv || (best_val[wv] == bv && best_idx[wv] < bi)) { bv = best_val[wv]; bi = best_idx[wv]; }
    part_val[(size_t)row * bpr + b] = bv;
    part_idx[(size_t)row * bpr + b] = bi;
    __threadfence();
    is_last = atomicAdd(&counters[row], 1) == bpr - 1;
  }
  __syncthreads();
  if (!is_last || tid >= 32) return;
  __threadfence();
  bv = -INFINITY; bi = 0x7fffffff;
  for (int p = tid; p < bpr; p += 32) {
    const float v = part_val[(size_t)row * bpr + p]; const int i = part_idx[(size_t)row * bpr + p];
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (tid == 0) { out[row] = min(max(bi, 0), vocab - 1); counters[row] = 0; }
}

// scratch: blocks_per_row * rows floats and as many ints; counters: rows ints, zero before the first call (the kernel
// leaves them zero).  blocks_per_row <= 1024.
IFB_EXPORT int ifb_argmax_rows(const float* logits, int rows, int vocab, int blocks_per_row, float* part_val, int* part_idx,
                               int* counters, int* out, cudaStream_t stream) {
  if (rows <= 0) return IFB_OK;
  if (vocab < 1 || blocks_per_row < 1 || blocks_per_row > 1024 || rows > 65535) return IFB_ERR_SIZE;
  if (!part_val || !part_idx || !counters) return IFB_ERR_ARG;
  return ifb_launch(argmax_rows_kernel, dim3(blocks_per_row, rows), dim3(256), 0, stream, logits, vocab, part_val, part_idx,
                    counters, out);
}

IFB_EXPORT int ifb_sample(const float* logits, int rows, int vocab, const float* temperature, const float* uniform,
                          int* out, cudaStream_t stream) {
  if (rows <= 0) return IFB_OK;
  if (vocab < 1) return IFB_ERR_SIZE;
  return ifb_launch(sample_kernel, dim3(rows), dim3(1024), 0, stream, logits, vocab, temperature, uniform, out);
}
