// Attention over the paged cache on tensor cores (bfloat16 operands, float32 accumulation and
// softmax), compiled for one head size: -DHEAD_DIM=<multiple of 16, at most 256>.
//
// Two kernels share the tile code and split a step's requests between them by the number of
// score rows a request brings, rows = query tokens x (query heads per key/value head):
//
//   small-q kernel (rows <= 16: decoded tokens and portions of a few tokens).  The work is the
//     reading of keys and values, so the context of a request is split over `num_splits` CTAs per
//     key/value head, the four warps of a CTA take different keys of each 64-key tile, and all
//     query heads of a group share every key and value that is read.  With more than one split a
//     CTA writes unnormalised partial sums with their running maximum and denominator to scratch
//     memory, and a second kernel merges them.
//   tile kernel (rows > 16: prompts and long portions).  A CTA takes 4 x floor(16/group) query
//     tokens of one key/value head; its four warps share each 64-key tile and keep 16 rows each.
//
// Both read every key, this step's own included, from the pages named by the request's block
// table: the query at position p sees positions max(0, p-window+1) .. p.  Keys outside what a
// CTA needs are not fetched (block-table entries of pages that a window has passed are stale).
#include "common.cuh"
#include <math.h>

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size>"
#endif
#if HEAD_DIM % 16 != 0 || HEAD_DIM < 16 || HEAD_DIM > 256
#error "HEAD_DIM must be a multiple of 16 between 16 and 256"
#endif

typedef __nv_bfloat16 bf16;
constexpr int D = HEAD_DIM;
constexpr int DP = D + 8;          // shared-memory row length: the 16-byte pad keeps ldmatrix conflict-free
constexpr int BN = 64;             // keys per tile
constexpr int THREADS = 128;
constexpr int KCH = D / 8;         // 16-byte pieces of a row
constexpr int KB = D / 16;         // k-blocks of a q.k product, n-block pairs of a p.v product
constexpr int SQ_STAGES = 3;       // tile buffers of the small-q kernel: two tiles are in flight while one is used

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;   // 0: the 16 bytes are filled with zeros and src is not read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the hardware approximation (relative error about 2^-22, far below bfloat16's and the softmax's needs);
// -inf gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Keys key0 .. key0+BN-1 of one key/value head into Ks and Vs ([BN][DP]); keys outside [lo, hi] are zeros.
// Consecutive threads copy consecutive 16-byte pieces of a row, so a warp's copy instruction covers whole
// 128-byte lines (a piece per thread at scattered rows would cost a memory request each).
__device__ __forceinline__ void load_kv_tile(bf16* Ks, bf16* Vs, const bf16* __restrict__ pages,
                                             const int* __restrict__ bt, int key0, int lo, int hi, int kvh, int nkv,
                                             int page_size, int tid) {
  const size_t head_stride = (size_t)page_size * D, page_stride = 2 * (size_t)nkv * head_stride;
  const int ps_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;   // power of two: shift, else divide
  constexpr int PASSES = (BN * KCH + THREADS - 1) / THREADS;
#pragma unroll
  for (int ps = 0; ps < PASSES; ++ps) {
    const int c = tid + ps * THREADS;
    if ((BN * KCH) % THREADS != 0 && c >= BN * KCH) break;
    const int row = c / KCH, ch = c % KCH;
    const int key = key0 + row;
    const bool valid = key >= lo && key <= hi;
    const bf16* src = pages;
    if (valid) {
      int pi, off;
      if (ps_shift >= 0) { pi = key >> ps_shift; off = key & (page_size - 1); }
      else { pi = key / page_size; off = key - pi * page_size; }
      src = pages + (size_t)bt[pi] * page_stride + (size_t)kvh * head_stride + (size_t)off * D + ch * 8;
    }
    cp_async16(Ks + row * DP + ch * 8, src, valid);
    cp_async16(Vs + row * DP + ch * 8, valid ? src + (size_t)nkv * head_stride : pages, valid);
  }
}

// One warp: scores of its 16 query rows (fragments qf) against keys [kbeg, kbeg + 8*NB) of the tile in
// Ks/Vs, masking, online softmax update of (m, l, o).  Row A of a thread is lane/4, row B is that + 8.
// pA/pB: position of the row's query (-1000000000: the row does not exist); wlo: window (0: none).
template <int NB, bool MASK>
__device__ __forceinline__ void warp_tile(const uint32_t (&qf)[KB][4], const bf16* Ks, const bf16* Vs, int kbeg,
                                          int key0, int klo, int khi, int pA, int pB, int window, float scale_log2,
                                          float (&m)[2], float (&l)[2], float (&o)[D / 8][4], int lane) {
  float s[NB][4];
#pragma unroll
  for (int j = 0; j < NB; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
  for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
    for (int j = 0; j < NB; j += 2) {
      uint32_t b[4];
      const int key = kbeg + j * 8 + (lane & 7) + ((lane >> 4) << 3);
      const int col = kb * 16 + (((lane >> 3) & 1) << 3);
      ldmatrix_x4(b, Ks + key * DP + col);
      mma_bf16(s[j], qf[kb], b[0], b[1]);
      mma_bf16(s[j + 1], qf[kb], b[2], b[3]);
    }
  }
  // mask and scale
  const int loA = window > 0 ? pA - window + 1 : 0, loB = window > 0 ? pB - window + 1 : 0;
  float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
  for (int j = 0; j < NB; ++j) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      bool va = true, vb = true;
      if (MASK) {
        const int key = key0 + kbeg + j * 8 + ((lane & 3) << 1) + e;
        const bool in = key >= klo && key <= khi;
        va = in && key <= pA && key >= loA;
        vb = in && key <= pB && key >= loB;
      }
      s[j][e] = va ? s[j][e] * scale_log2 : -INFINITY;
      s[j][2 + e] = vb ? s[j][2 + e] * scale_log2 : -INFINITY;
      mxA = fmaxf(mxA, s[j][e]);
      mxB = fmaxf(mxB, s[j][2 + e]);
    }
  }
  mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
  mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
  mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
  mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
  const float mA = fmaxf(m[0], mxA), mB = fmaxf(m[1], mxB);
  const float uA = mA == -INFINITY ? 0.f : mA, uB = mB == -INFINITY ? 0.f : mB;   // all keys masked so far
  const float cA = fast_exp2(m[0] - uA), cB = fast_exp2(m[1] - uB);
  const bool moved = (mA != m[0]) || (mB != m[1]);          // did a running maximum rise in this tile?
  m[0] = mA; m[1] = mB;
  float sumA = 0.f, sumB = 0.f;
#pragma unroll
  for (int j = 0; j < NB; ++j) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      s[j][e] = fast_exp2(s[j][e] - uA);
      s[j][2 + e] = fast_exp2(s[j][2 + e] - uB);
      sumA += s[j][e];
      sumB += s[j][2 + e];
    }
  }
  l[0] = l[0] * cA + sumA;   // per-thread partial of the row's denominator; summed over the quad at the end
  l[1] = l[1] * cB + sumB;
  if (__any_sync(0xffffffffu, moved)) {                     // else both factors are exactly 1 for every lane
#pragma unroll
    for (int n = 0; n < D / 8; ++n) { o[n][0] *= cA; o[n][1] *= cA; o[n][2] *= cB; o[n][3] *= cB; }
  }
  // o += p v
#pragma unroll
  for (int kk = 0; kk < NB / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int n2 = 0; n2 < KB; ++n2) {
      uint32_t b[4];
      const int key = kbeg + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int col = n2 * 16 + ((lane >> 4) << 3);
      ldmatrix_x4_trans(b, Vs + key * DP + col);
      mma_bf16(o[2 * n2], a, b[0], b[1]);
      mma_bf16(o[2 * n2 + 1], a, b[2], b[3]);
    }
  }
}

__device__ __forceinline__ void load_q_frags(uint32_t (&qf)[KB][4], const bf16* Qs, int lane) {
#pragma unroll
  for (int kb = 0; kb < KB; ++kb) {
    const int row = (lane & 7) + (((lane >> 3) & 1) << 3);
    const int col = kb * 16 + ((lane >> 4) << 3);
    ldmatrix_x4(qf[kb], Qs + row * DP + col);
  }
}

constexpr int NO_ROW = -1000000000;

// --------------------------------------------------------------------------------------------
// small-q kernel: grid (num_splits, kv heads, requests)
// --------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS)
attn_small_q_kernel(const bf16* __restrict__ qkv, int row_stride, const bf16* __restrict__ pages,
                    const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ cu_q,
                    const int* __restrict__ seq_lens, bf16* __restrict__ out, float* __restrict__ part_o,
                    float* __restrict__ part_ml, int* __restrict__ counters, int nq, int nkv, int page_size,
                    float scale_log2, int window, int num_splits) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int is_last;
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);              // [16][DP]
  bf16* KV = Qs + 16 * DP;                                   // SQ_STAGES x (K [BN][DP], V [BN][DP])
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = nq / nkv;
  const int q0 = cu_q[r], q_len = cu_q[r + 1] - q0, L = seq_lens[r];
  const int rows = q_len * G;
  if (q_len <= 0 || rows > 16) return;
  const int p_first = L - q_len;
  const int lo = window > 0 ? max(0, p_first - window + 1) : 0, hi = L - 1;
  const int total = hi + 1 - lo;
  int per = total > 0 ? (total + num_splits - 1) / num_splits : 0;
  per = (per + BN - 1) / BN * BN;
  const int k_begin = lo + split * per, k_end = min(hi + 1, k_begin + per);
  const int n_tiles = k_end > k_begin ? (k_end - k_begin + BN - 1) / BN : 0;
  const int* bt = block_tables + (size_t)r * bt_stride;

  // the query rows: row = token * G + head-in-group
  for (int c = tid; c < 16 * KCH; c += THREADS) {
    const int row = c / KCH, ch = c % KCH;
    const bool valid = row < rows && n_tiles > 0;
    const bf16* src = valid ? qkv + (size_t)(q0 + row / G) * row_stride + (size_t)(kvh * G + row % G) * D + ch * 8 : qkv;
    cp_async16(Qs + row * DP + ch * 8, src, valid);
  }
  // prologue: tiles 0 .. SQ_STAGES-2 in flight (one commit group per tile, empty groups past the end)
#pragma unroll
  for (int st = 0; st < SQ_STAGES - 1; ++st) {
    if (st < n_tiles) {
      bf16* Kn = KV + st * 2 * BN * DP;
      load_kv_tile(Kn, Kn + BN * DP, pages, bt, k_begin + st * BN, k_begin, k_end - 1, kvh, nkv, page_size, tid);
    }
    cp_async_commit();
  }

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  const int rowA = lane >> 2, rowB = rowA + 8;
  const int pA = rowA < rows ? p_first + rowA / G : NO_ROW, pB = rowB < rows ? p_first + rowB / G : NO_ROW;
  uint32_t qf[KB][4];
  for (int t = 0; t < n_tiles; ++t) {
    const int stage = t % SQ_STAGES;
    bf16* Ks = KV + stage * 2 * BN * DP;
    bf16* Vs = Ks + BN * DP;
    cp_async_wait<SQ_STAGES - 2>();          // tile t has landed (for this thread's copies)
    __syncthreads();                         // ... for everyone's; and everyone is done with tile t-1
    const int nt = t + SQ_STAGES - 1;        // refill the stage that tile t-1 used
    if (nt < n_tiles) {
      bf16* Kn = KV + (nt % SQ_STAGES) * 2 * BN * DP;
      load_kv_tile(Kn, Kn + BN * DP, pages, bt, k_begin + nt * BN, k_begin, k_end - 1, kvh, nkv, page_size, tid);
    }
    cp_async_commit();
    if (t == 0) load_q_frags(qf, Qs, lane);
    // a tile every key of which every existing row sees needs no masking (rows that do not exist have
    // zero queries and are never written)
    const int tile0 = k_begin + t * BN;
    const bool interior = tile0 + BN - 1 <= min(p_first, k_end - 1) && (window == 0 || tile0 >= L - window);
    if (interior)
      warp_tile<2, false>(qf, Ks, Vs, warp * 16, tile0, k_begin, k_end - 1, pA, pB, window, scale_log2, m, l, o, lane);
    else
      warp_tile<2, true>(qf, Ks, Vs, warp * 16, tile0, k_begin, k_end - 1, pA, pB, window, scale_log2, m, l, o, lane);
  }
  cp_async_wait<0>();
  __syncthreads();
  // merge the four warps' (m, l, o) through shared memory (the tile buffers are free now)
  float* sm_o = reinterpret_cast<float*>(KV);                // [4][16][D]
  float* sm_m = sm_o + 4 * 16 * D;                           // [4][16]
  float* sm_l = sm_m + 64;                                   // [4][16]
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    l[e] += __shfl_xor_sync(0xffffffffu, l[e], 1);
    l[e] += __shfl_xor_sync(0xffffffffu, l[e], 2);
  }
  if ((lane & 3) == 0) {
    sm_m[warp * 16 + rowA] = m[0]; sm_m[warp * 16 + rowB] = m[1];
    sm_l[warp * 16 + rowA] = l[0]; sm_l[warp * 16 + rowB] = l[1];
  }
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    const int col = n * 8 + ((lane & 3) << 1);
    float* pa = sm_o + ((size_t)warp * 16 + rowA) * D + col;
    float* pb = sm_o + ((size_t)warp * 16 + rowB) * D + col;
    pa[0] = o[n][0]; pa[1] = o[n][1]; pb[0] = o[n][2]; pb[1] = o[n][3];
  }
  __syncthreads();
  for (int idx = tid; idx < rows * D; idx += THREADS) {
    const int row = idx / D, dim = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * 16 + row]);
    const float U = M == -INFINITY ? 0.f : M;
    float den = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(sm_m[w * 16 + row] - U);
      den += sm_l[w * 16 + row] * f;
      acc += sm_o[((size_t)w * 16 + row) * D + dim] * f;
    }
    const int tok = q0 + row / G, head = kvh * G + row % G;
    if (num_splits == 1) {
      out[((size_t)tok * nq + head) * D + dim] = __float2bfloat16_rn(den > 0.f ? acc / den : 0.f);
    } else {
      const size_t base = ((size_t)tok * nq + head) * num_splits + split;
      part_o[base * D + dim] = acc;
      if (dim == 0) { part_ml[base * 2] = M; part_ml[base * 2 + 1] = den; }
    }
  }
  if (num_splits == 1) return;
  // the CTA that finishes last for this (request, key/value head) merges the splits, in split order
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&counters[r * nkv + kvh], 1);
    is_last = (old == num_splits - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int idx = tid; idx < rows * D; idx += THREADS) {
    const int row = idx / D, dim = idx % D;
    const int tok = q0 + row / G, head = kvh * G + row % G;
    const size_t base = ((size_t)tok * nq + head) * num_splits;
    float M = -INFINITY;
    for (int sp = 0; sp < num_splits; ++sp) M = fmaxf(M, part_ml[(base + sp) * 2]);
    const float U = M == -INFINITY ? 0.f : M;
    float den = 0.f, acc = 0.f;
    for (int sp = 0; sp < num_splits; ++sp) {
      const float f = exp2f(part_ml[(base + sp) * 2] - U);
      den += part_ml[(base + sp) * 2 + 1] * f;
      acc += part_o[(base + sp) * D + dim] * f;
    }
    out[((size_t)tok * nq + head) * D + dim] = __float2bfloat16_rn(den > 0.f ? acc / den : 0.f);
  }
  if (tid == 0) counters[r * nkv + kvh] = 0;       // ready for the next launch
}

// --------------------------------------------------------------------------------------------
// tile kernel: grid (query tiles, kv heads, requests); a warp keeps floor(16/G) tokens x G heads
// --------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS)
attn_tile_kernel(const bf16* __restrict__ qkv, int row_stride, const bf16* __restrict__ pages,
                 const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ cu_q,
                 const int* __restrict__ seq_lens, bf16* __restrict__ out, int nq, int nkv, int page_size,
                 float scale_log2, int window) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);              // [64][DP]
  bf16* KV = Qs + 64 * DP;
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int kvh = blockIdx.y, r = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = nq / nkv;
  const int q0 = cu_q[r], q_len = cu_q[r + 1] - q0, L = seq_lens[r];
  if (q_len * G <= 16) return;                               // the small-q kernel's request
  const int tpw = 16 / G, tpc = 4 * tpw;                     // tokens per warp, per CTA
  const int t0 = blockIdx.x * tpc;
  if (t0 >= q_len) return;
  const int t1 = min(q_len, t0 + tpc);
  const int p_first = L - q_len;
  const int lo = window > 0 ? max(0, p_first + t0 - window + 1) : 0, hi = p_first + t1 - 1;
  const int n_tiles = hi >= lo ? (hi + 1 - lo + BN - 1) / BN : 0;
  const int* bt = block_tables + (size_t)r * bt_stride;
  for (int c = tid; c < 64 * KCH; c += THREADS) {
    const int row = c / KCH, ch = c % KCH;
    const int w = row >> 4, rr = row & 15;
    const int tok = t0 + w * tpw + rr / G;
    const bool valid = rr < tpw * G && tok < t1;
    const bf16* src = valid ? qkv + (size_t)(q0 + tok) * row_stride + (size_t)(kvh * G + rr % G) * D + ch * 8 : qkv;
    cp_async16(Qs + row * DP + ch * 8, src, valid);
  }
  if (n_tiles > 0) load_kv_tile(KV, KV + BN * DP, pages, bt, lo, lo, hi, kvh, nkv, page_size, tid);
  cp_async_commit();
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  const int rowA = lane >> 2, rowB = rowA + 8;
  const int tokA = t0 + warp * tpw + rowA / G, tokB = t0 + warp * tpw + rowB / G;
  const int pA = (rowA < tpw * G && tokA < t1) ? p_first + tokA : NO_ROW;
  const int pB = (rowB < tpw * G && tokB < t1) ? p_first + tokB : NO_ROW;
  const int warp_hi = p_first + min(t1, t0 + (warp + 1) * tpw) - 1;        // last position this warp's rows see
  uint32_t qf[KB][4];
  for (int t = 0; t < n_tiles; ++t) {
    bf16* Ks = KV + (t & 1) * 2 * BN * DP;
    bf16* Vs = Ks + BN * DP;
    if (t + 1 < n_tiles) {
      bf16* Kn = KV + ((t + 1) & 1) * 2 * BN * DP;
      load_kv_tile(Kn, Kn + BN * DP, pages, bt, lo + (t + 1) * BN, lo, hi, kvh, nkv, page_size, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (t == 0) load_q_frags(qf, Qs + warp * 16 * DP, lane);
    const int tile0 = lo + t * BN;
    if (tile0 <= warp_hi) {
      // every key of the tile is seen by every row of this warp: no masking
      const bool interior = t0 + warp * tpw < t1 && tile0 >= lo && tile0 + BN - 1 <= min(hi, p_first + t0 + warp * tpw) &&
                            (window == 0 || tile0 >= warp_hi - window + 1);
      if (interior)
        warp_tile<8, false>(qf, Ks, Vs, 0, tile0, lo, hi, pA, pB, window, scale_log2, m, l, o, lane);
      else
        warp_tile<8, true>(qf, Ks, Vs, 0, tile0, lo, hi, pA, pB, window, scale_log2, m, l, o, lane);
    }
    __syncthreads();
  }
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    l[e] += __shfl_xor_sync(0xffffffffu, l[e], 1);
    l[e] += __shfl_xor_sync(0xffffffffu, l[e], 2);
  }
  const float iA = l[0] > 0.f ? 1.f / l[0] : 0.f, iB = l[1] > 0.f ? 1.f / l[1] : 0.f;
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    const int col = n * 8 + ((lane & 3) << 1);
    if (pA != NO_ROW) {
      bf16* dst = out + ((size_t)(q0 + tokA) * nq + kvh * G + rowA % G) * D + col;
      *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(o[n][0] * iA, o[n][1] * iA);
    }
    if (pB != NO_ROW) {
      bf16* dst = out + ((size_t)(q0 + tokB) * nq + kvh * G + rowB % G) * D + col;
      *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(o[n][2] * iB, o[n][3] * iB);
    }
  }
}

static size_t small_q_smem() { return (size_t)(16 * DP + SQ_STAGES * 2 * BN * DP) * sizeof(bf16); }
static size_t tile_smem() { return (size_t)(64 * DP + 4 * BN * DP) * sizeof(bf16); }

IFB_EXPORT int ifb_attention_mma_head_dim() { return D; }

// Floats of scratch the small-q kernel needs for `n_tokens` tokens of `nq` heads in `num_splits` splits.
IFB_EXPORT long long ifb_attention_mma_scratch_floats(int n_tokens, int nq, int num_splits) {
  return num_splits > 1 ? (long long)n_tokens * nq * num_splits * (D + 2) : 0;
}

// max_q_len: the most query tokens any request brings.  small: launch the small-q kernel (and the merge);
// tiles: launch the tile kernel.  Requests are routed by rows = q_len * (nq / nkv) <= 16.
IFB_EXPORT int ifb_attention_mma(const void* qkv, int row_stride, const void* pages, const int* block_tables,
                                 int bt_stride, const int* cu_q, const int* seq_lens, void* out, float* scratch,
                                 int* counters, int n_tokens, int n_req, int nq, int nkv, int d, int page_size, float scale,
                                 int window, int max_q_len, int num_splits, int run_small, int run_tiles,
                                 cudaStream_t stream) {
  if (n_tokens <= 0 || n_req <= 0) return IFB_OK;
  if (d != D) return IFB_ERR_SIZE;
  if (nkv < 1 || nq % nkv || page_size < 1 || window < 0 || num_splits < 1) return IFB_ERR_ARG;
  const int G = nq / nkv;
  if (G > 16 && run_tiles) return IFB_ERR_SIZE;
  if (row_stride % 8 || ((uintptr_t)qkv & 15) || ((uintptr_t)pages & 15) || ((uintptr_t)out & 3)) return IFB_ERR_ALIGN;
  if (n_req > 65535 || nkv > 65535) return IFB_ERR_SIZE;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_small_q_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)small_q_smem());
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile_smem());
    if (e != cudaSuccess) return -(int)e;
    configured = true;
  }
  const float scale_log2 = scale * 1.4426950408889634f;
  if (run_small) {
    if (num_splits > 1 && (!scratch || !counters)) return IFB_ERR_ARG;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)n_tokens * nq * num_splits * D : nullptr;
    dim3 grid(num_splits, nkv, n_req);
    int st = ifb_launch(attn_small_q_kernel, grid, dim3(THREADS), small_q_smem(), stream, (const bf16*)qkv, row_stride,
                        (const bf16*)pages, block_tables, bt_stride, cu_q, seq_lens, (bf16*)out, part_o, part_ml, counters,
                        nq, nkv, page_size, scale_log2, window, num_splits);
    if (st) return st;
  }
  if (run_tiles) {
    const int tpc = 4 * (16 / G);
    dim3 grid((max_q_len + tpc - 1) / tpc, nkv, n_req);
    return ifb_launch(attn_tile_kernel, grid, dim3(THREADS), tile_smem(), stream, (const bf16*)qkv, row_stride,
                      (const bf16*)pages, block_tables, bt_stride, cu_q, seq_lens, (bf16*)out, nq, nkv, page_size,
                      scale_log2, window);
  }
  return IFB_OK;
}
