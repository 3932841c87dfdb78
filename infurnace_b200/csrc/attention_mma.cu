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
//
// How a tile of keys and values reaches shared memory.  With head sizes that are multiples of 64 and
// pages of 16, 32 or 64 tokens, TMA brings it: the page pool is described by one tensor map as a
// matrix [pages * 2 * kv_heads * page_size, head_dim], a page's keys (or values) of one head are one
// box per 64 columns, written in the 128-byte swizzle, which ldmatrix then reads without bank
// conflicts.  Sixteen lanes of warp 0 issue a tile's boxes; a stage's mbarrier counts the bytes.  A
// page that lies outside the keys a CTA needs is fetched from a row beyond the tensor (zeros).  Waits
// on the barriers are bounded: after ATT_SPIN_LIMIT polls a thread records a code in `*err`, raises
// the CTA's abort flag and the CTA leaves.  Other sizes take the cp.async path: 16-byte copies by all
// threads into padded rows.
#include <cuda.h>
#include "common.cuh"
#include <math.h>
#include <string.h>

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
constexpr bool TMA_D = (D % 64 == 0);            // head sizes the TMA path takes
constexpr int HALVES = TMA_D ? D / 64 : 1;       // 64-column (128-byte) boxes per row
constexpr uint32_t ATT_SPIN_LIMIT = 1u << 22;

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

__device__ __forceinline__ void att_mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void att_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool att_mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  False: gave up (the abort flag is up and *err holds `code`).
__device__ __forceinline__ bool att_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
  unsigned long long t0 = 0;
  for (uint32_t i = 0; i < ATT_SPIN_LIMIT; ++i) {
    if (att_mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (ifb_wait_expired(i, t0)) break;
  }
  *abort_flag = 1;
  atomicExch(err, code);
  return false;
}
__device__ __forceinline__ void att_tma_load_2d(void* smem, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// Address of 8 elements (key, col .. col+7) of a K or V tile.  Padded layout: [BN][DP].  Swizzled layout (what
// TMA wrote): [HALVES][BN][64], the 16-byte piece c of a row stored at c ^ (row & 7); the tile is 1024-byte aligned.
template <bool SWZ>
__device__ __forceinline__ const bf16* kv_at(const bf16* tile, int key, int col) {
  if (SWZ) return tile + (col >> 6) * (BN * 64) + key * 64 + ((((col & 63) >> 3) ^ (key & 7)) << 3);
  return tile + key * DP + col;
}

// One tile by TMA, issued by warp 0 (all 32 lanes call): K to `stage`, V to `stage + BN*D`.  Pages that do not
// overlap the keys [k_lo, k_hi] are read from beyond the tensor's last row, which gives zeros.
__device__ __forceinline__ void tma_issue_tile(const CUtensorMap* map, bf16* stage, uint64_t* bar, const int* __restrict__ bt,
                                               int tile_key0, int k_lo, int k_hi, int kvh, int nkv, int page_size,
                                               int ps_shift, int total_rows, int lane) {
  const int ppt = BN >> ps_shift;                    // pages per tile
  const int n_ops = ppt * HALVES * 2;                // at most 4 * 4 * 2 = 32
  if (lane == 0) att_mbar_expect_tx(bar, 2u * BN * D * sizeof(bf16));
  __syncwarp();
  if (lane < n_ops) {
    const int kv = lane / (ppt * HALVES), rem = lane % (ppt * HALVES), pg = rem / HALVES, half = rem % HALVES;
    const int key0 = tile_key0 + pg * page_size;
    int y = total_rows;
    if (key0 <= k_hi && key0 + page_size - 1 >= k_lo) y = ((bt[key0 >> ps_shift] * 2 + kv) * nkv + kvh) * page_size;
    att_tma_load_2d(stage + kv * (BN * D) + half * (BN * 64) + pg * page_size * 64, map, bar, half * 64, y);
  }
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
template <int NB, bool MASK, bool SWZ>
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
      ldmatrix_x4(b, kv_at<SWZ>(Ks, key, col));
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
      ldmatrix_x4_trans(b, kv_at<SWZ>(Vs, key, col));
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

// The end of a small-q CTA: its four consumer warps' (m, l, o) are merged through shared memory (`scratch`, at least
// 4*16*D + 128 floats, free by now); then the output row is written, or with several splits the partial sums go to
// global memory and the CTA that arrives last for its (request, key/value head) merges the splits in split order.
// Every thread of the CTA calls this (threads of warps above 3 only keep the barriers company).
__device__ __forceinline__ void small_q_finish(float* scratch, float (&m)[2], float (&l)[2], float (&o)[D / 8][4], int rows,
                                               int G, int q0, int kvh, int r, int split, int num_splits, int nq, int nkv,
                                               bf16* __restrict__ out, float* __restrict__ part_o,
                                               float* __restrict__ part_ml, int* __restrict__ counters, int* is_last_p) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nthreads = blockDim.x;
  const int rowA = lane >> 2, rowB = rowA + 8;
  float* sm_o = scratch;                                     // [4][16][D]
  float* sm_m = sm_o + 4 * 16 * D;                           // [4][16]
  float* sm_l = sm_m + 64;                                   // [4][16]
  if (warp < 4) {
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
  }
  __syncthreads();
  for (int idx = tid; idx < rows * D; idx += nthreads) {
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
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&counters[r * nkv + kvh], 1);
    *is_last_p = (old == num_splits - 1);
  }
  __syncthreads();
  if (!*is_last_p) return;
  __threadfence();
  for (int idx = tid; idx < rows * D; idx += nthreads) {
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
// small-q kernel: grid (num_splits, kv heads, requests)
// --------------------------------------------------------------------------------------------
template <bool TMA>
__global__ void __launch_bounds__(THREADS)
attn_small_q_kernel(const __grid_constant__ CUtensorMap kv_map, int total_rows, int* __restrict__ err,
                    const bf16* __restrict__ qkv, int row_stride, const bf16* __restrict__ pages,
                    const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ cu_q,
                    const int* __restrict__ seq_lens, bf16* __restrict__ out, float* __restrict__ part_o,
                    float* __restrict__ part_ml, int* __restrict__ counters, int nq, int nkv, int page_size,
                    float scale_log2, int window, int num_splits) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int is_last;
  __shared__ uint64_t full_bar[SQ_STAGES];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  constexpr int STAGE = TMA ? 2 * BN * D : 2 * BN * DP;       // elements of one stage: K tile then V tile
  // the stages first (TMA wants them 1024-byte aligned), then the 16 query rows
  const uint32_t raw = smem_u32(smem_raw);
  bf16* KV = reinterpret_cast<bf16*>(smem_raw + (TMA ? ((raw + 1023u) & ~1023u) - raw : 0u));
  bf16* Qs = KV + SQ_STAGES * STAGE;                          // [16][DP]
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
  // tiles start at multiples of BN keys with TMA (a box is a whole page), else at the first key
  const int T0 = TMA ? (k_begin / BN) * BN : k_begin;
  const int n_tiles = k_end > k_begin ? (k_end - T0 + BN - 1) / BN : 0;
  const int* bt = block_tables + (size_t)r * bt_stride;
  const int ps_shift = __ffs(page_size) - 1;                  // TMA path: page_size is a power of two

  if (TMA) {
    if (tid == 0) {
      for (int st = 0; st < SQ_STAGES; ++st) att_mbar_init(&full_bar[st], 1);
      abort_word = 0;
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();
  }
  // the query rows: row = token * G + head-in-group
  for (int c = tid; c < 16 * KCH; c += THREADS) {
    const int row = c / KCH, ch = c % KCH;
    const bool valid = row < rows && n_tiles > 0;
    const bf16* src = valid ? qkv + (size_t)(q0 + row / G) * row_stride + (size_t)(kvh * G + row % G) * D + ch * 8 : qkv;
    cp_async16(Qs + row * DP + ch * 8, src, valid);
  }
  cp_async_commit();
  // prologue: tiles 0 .. SQ_STAGES-2 in flight
#pragma unroll
  for (int st = 0; st < SQ_STAGES - 1; ++st) {
    if (st < n_tiles) {
      bf16* Kn = KV + st * STAGE;
      if (TMA) {
        if (warp == 0)
          tma_issue_tile(&kv_map, Kn, &full_bar[st], bt, T0 + st * BN, k_begin, k_end - 1, kvh, nkv, page_size, ps_shift,
                         total_rows, lane);
      } else {
        load_kv_tile(Kn, Kn + BN * DP, pages, bt, T0 + st * BN, k_begin, k_end - 1, kvh, nkv, page_size, tid);
      }
    }
    if (!TMA) cp_async_commit();
  }

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  const int rowA = lane >> 2, rowB = rowA + 8;
  const int pA = rowA < rows ? p_first + rowA / G : NO_ROW, pB = rowB < rows ? p_first + rowB / G : NO_ROW;
  uint32_t qf[KB][4];
  bool ok = true;
  for (int t = 0; t < n_tiles; ++t) {
    const int stage = t % SQ_STAGES;
    bf16* Ks = KV + stage * STAGE;
    bf16* Vs = Ks + (TMA ? BN * D : BN * DP);
    if (TMA) {
      if (t == 0) cp_async_wait<0>();        // the query rows
      ok = att_mbar_wait(&full_bar[stage], (t / SQ_STAGES) & 1, abort_flag, err, 1);
    } else {
      cp_async_wait<SQ_STAGES - 2>();        // tile t has landed (for this thread's copies)
    }
    __syncthreads();                         // ... for everyone's; and everyone is done with tile t-1
    if (TMA && *abort_flag) { ok = false; break; }
    const int nt = t + SQ_STAGES - 1;        // refill the stage that tile t-1 used
    if (nt < n_tiles) {
      bf16* Kn = KV + (nt % SQ_STAGES) * STAGE;
      if (TMA) {
        if (warp == 0)
          tma_issue_tile(&kv_map, Kn, &full_bar[nt % SQ_STAGES], bt, T0 + nt * BN, k_begin, k_end - 1, kvh, nkv, page_size,
                         ps_shift, total_rows, lane);
      } else {
        load_kv_tile(Kn, Kn + BN * DP, pages, bt, T0 + nt * BN, k_begin, k_end - 1, kvh, nkv, page_size, tid);
      }
    }
    if (!TMA) cp_async_commit();
    if (t == 0) load_q_frags(qf, Qs, lane);
    // a tile every key of which every existing row sees needs no masking (rows that do not exist have
    // zero queries and are never written)
    const int tile0 = T0 + t * BN;
    const bool interior = tile0 >= k_begin && tile0 + BN - 1 <= min(p_first, k_end - 1) && (window == 0 || tile0 >= L - window);
    if (interior)
      warp_tile<2, false, TMA>(qf, Ks, Vs, warp * 16, tile0, k_begin, k_end - 1, pA, pB, window, scale_log2, m, l, o, lane);
    else
      warp_tile<2, true, TMA>(qf, Ks, Vs, warp * 16, tile0, k_begin, k_end - 1, pA, pB, window, scale_log2, m, l, o, lane);
  }
  cp_async_wait<0>();
  if (TMA && !ok) {                          // a wait gave up: let copies in flight land, then leave
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    return;
  }
  __syncthreads();
  small_q_finish(reinterpret_cast<float*>(KV), m, l, o, rows, G, q0, kvh, r, split, num_splits, nq, nkv, out, part_o, part_ml,
                 counters, &is_last);
}

// --------------------------------------------------------------------------------------------
// small-q kernel, TMA form with a producer warp: grid (num_splits, kv heads, requests), 160 threads.
// Warps 0-3 are the consumers (16 keys of every tile each, as above); warp 4 only issues TMA loads.  A stage has a
// "full" barrier (armed with the tile's bytes by the producer) and an "empty" barrier (one arrival per consumer warp
// when it has read the tile), so no warp waits for another at a tile's end: a slow warp holds back only the refill
// of its own stage.
// --------------------------------------------------------------------------------------------
constexpr int WS_THREADS = 160;
__device__ __forceinline__ void att_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(WS_THREADS)
attn_small_q_ws_kernel(const __grid_constant__ CUtensorMap kv_map, int total_rows, int* __restrict__ err,
                       const bf16* __restrict__ qkv, int row_stride, const int* __restrict__ block_tables, int bt_stride,
                       const int* __restrict__ cu_q, const int* __restrict__ seq_lens, bf16* __restrict__ out,
                       float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters, int nq,
                       int nkv, int page_size, float scale_log2, int window, int num_splits) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int is_last;
  __shared__ uint64_t full_bar[SQ_STAGES], empty_bar[SQ_STAGES];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  constexpr int STAGE = 2 * BN * D;
  const uint32_t raw = smem_u32(smem_raw);
  bf16* KV = reinterpret_cast<bf16*>(smem_raw + (((raw + 1023u) & ~1023u) - raw));
  bf16* Qs = KV + SQ_STAGES * STAGE;                          // [16][DP]
  // (cu_q, seq_lens and the block tables were written at the start of the step, not by the kernel before this one:
  // they may be read before waiting for it)
  const int split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = nq / nkv;
  const int q0 = cu_q[r], q_len = cu_q[r + 1] - q0, L = seq_lens[r];
  const int rows = q_len * G;
  if (q_len <= 0 || rows > 16) {
    // not this kernel's request.  Even so it waits for the kernel before it: a grid none of whose threads waited could
    // end before its predecessor, and the kernel after this one, which waits for this one only, would start too early.
    ifb_pdl_wait();
    return;
  }
  const int p_first = L - q_len;
  const int lo = window > 0 ? max(0, p_first - window + 1) : 0, hi = L - 1;
  const int total = hi + 1 - lo;
  int per = total > 0 ? (total + num_splits - 1) / num_splits : 0;
  per = (per + BN - 1) / BN * BN;
  const int k_begin = lo + split * per, k_end = min(hi + 1, k_begin + per);
  const int T0 = (k_begin / BN) * BN;
  const int n_tiles = k_end > k_begin ? (k_end - T0 + BN - 1) / BN : 0;
  const int* bt = block_tables + (size_t)r * bt_stride;
  const int ps_shift = __ffs(page_size) - 1;
  if (tid == 0) {
    for (int st = 0; st < SQ_STAGES; ++st) { att_mbar_init(&full_bar[st], 1); att_mbar_init(&empty_bar[st], 4); }
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  __syncthreads();

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  bool ok = true;
  if (warp == 4) {
    // ---- producer: tile t goes to stage t % S once the consumers have released that stage's previous tile.
    // The kernel before this one wrote the keys and values of this step's tokens (positions >= p_first) and nothing
    // else that is read here, so tiles of older keys are requested without waiting for it: the first stages fill
    // while it still runs.
    bool waited = false;
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int stage = t % SQ_STAGES;
      if (!waited && T0 + (t + 1) * BN > p_first) {
        ifb_pdl_wait();
        waited = true;
      }
      if (t >= SQ_STAGES) ok = att_mbar_wait(&empty_bar[stage], ((t / SQ_STAGES) - 1) & 1, abort_flag, err, 3);
      if (!ok) break;
      tma_issue_tile(&kv_map, KV + stage * STAGE, &full_bar[stage], bt, T0 + t * BN, k_begin, k_end - 1, kvh, nkv, page_size,
                     ps_shift, total_rows, lane);
    }
  } else {
    // ---- consumers: the query rows (row = token * G + head-in-group), then the tiles
    ifb_pdl_wait();
    ifb_pdl_trigger();
    for (int c = tid; c < 16 * KCH; c += 128) {
      const int row = c / KCH, ch = c % KCH;
      const bool valid = row < rows && n_tiles > 0;
      const bf16* src = valid ? qkv + (size_t)(q0 + row / G) * row_stride + (size_t)(kvh * G + row % G) * D + ch * 8 : qkv;
      cp_async16(Qs + row * DP + ch * 8, src, valid);
    }
    cp_async_commit();
    cp_async_wait<0>();
    asm volatile("bar.sync 1, 128;\n" ::: "memory");           // the four consumer warps only
    const int rowA = lane >> 2, rowB = rowA + 8;
    const int pA = rowA < rows ? p_first + rowA / G : NO_ROW, pB = rowB < rows ? p_first + rowB / G : NO_ROW;
    uint32_t qf[KB][4];
    if (n_tiles > 0) load_q_frags(qf, Qs, lane);
    for (int t = 0; t < n_tiles; ++t) {
      const int stage = t % SQ_STAGES;
      const bf16* Ks = KV + stage * STAGE;
      const bf16* Vs = Ks + BN * D;
      ok = att_mbar_wait(&full_bar[stage], (t / SQ_STAGES) & 1, abort_flag, err, 1);
      if (!ok) break;
      const int tile0 = T0 + t * BN;
      const bool interior = tile0 >= k_begin && tile0 + BN - 1 <= min(p_first, k_end - 1) && (window == 0 || tile0 >= L - window);
      if (interior)
        warp_tile<2, false, true>(qf, Ks, Vs, warp * 16, tile0, k_begin, k_end - 1, pA, pB, window, scale_log2, m, l, o, lane);
      else
        warp_tile<2, true, true>(qf, Ks, Vs, warp * 16, tile0, k_begin, k_end - 1, pA, pB, window, scale_log2, m, l, o, lane);
      __syncwarp();
      if (lane == 0) att_mbar_arrive(&empty_bar[stage]);        // this warp is done with the stage
    }
  }
  __syncthreads();                                              // every tile has been read; the stages are free
  if (*abort_flag) {                                            // a wait gave up: let copies in flight land, then leave
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    return;
  }
  small_q_finish(reinterpret_cast<float*>(KV), m, l, o, rows, G, q0, kvh, r, split, num_splits, nq, nkv, out, part_o, part_ml,
                 counters, &is_last);
}

// --------------------------------------------------------------------------------------------
// tile kernel: grid (query tiles, kv heads, requests); a warp keeps floor(16/G) tokens x G heads
// --------------------------------------------------------------------------------------------
template <bool TMA>
__global__ void __launch_bounds__(THREADS, D <= 128 ? 3 : 1)      // three CTAs per SM where the accumulators allow
attn_tile_kernel(const __grid_constant__ CUtensorMap kv_map, int total_rows, int* __restrict__ err,
                 const bf16* __restrict__ qkv, int row_stride, const bf16* __restrict__ pages,
                 const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ cu_q,
                 const int* __restrict__ seq_lens, bf16* __restrict__ out, int nq, int nkv, int page_size,
                 float scale_log2, int window) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ uint64_t full_bar[2];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  constexpr int STAGE = TMA ? 2 * BN * D : 2 * BN * DP;
  const uint32_t raw = smem_u32(smem_raw);
  bf16* KV = reinterpret_cast<bf16*>(smem_raw + (TMA ? ((raw + 1023u) & ~1023u) - raw : 0u));
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int kvh = blockIdx.y, r = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = nq / nkv;
  const int q0 = cu_q[r], q_len = cu_q[r + 1] - q0, L = seq_lens[r];
  if (q_len * G <= 16) return;                               // the small-q kernel's request
  const int tpw = 16 / G, tpc = 4 * tpw;                     // tokens per warp, per CTA
  // the last query tiles have the longest key ranges: they go first, so that the grid's tail is short work
  const int t0 = (int)(gridDim.x - 1 - blockIdx.x) * tpc;
  if (t0 >= q_len) return;
  const int t1 = min(q_len, t0 + tpc);
  const int p_first = L - q_len;
  const int lo = window > 0 ? max(0, p_first + t0 - window + 1) : 0, hi = p_first + t1 - 1;
  const int T0 = TMA ? (lo / BN) * BN : lo;
  const int n_tiles = hi >= lo ? (hi + 1 - T0 + BN - 1) / BN : 0;
  const int* bt = block_tables + (size_t)r * bt_stride;
  const int ps_shift = __ffs(page_size) - 1;
  if (TMA) {
    if (tid == 0) {
      att_mbar_init(&full_bar[0], 1);
      att_mbar_init(&full_bar[1], 1);
      abort_word = 0;
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();
  }
  if (n_tiles > 0) {
    if (TMA) {
      if (warp == 0) tma_issue_tile(&kv_map, KV, &full_bar[0], bt, T0, lo, hi, kvh, nkv, page_size, ps_shift, total_rows, lane);
    } else {
      load_kv_tile(KV, KV + BN * DP, pages, bt, T0, lo, hi, kvh, nkv, page_size, tid);
    }
  }
  if (!TMA) cp_async_commit();
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  const int rowA = lane >> 2, rowB = rowA + 8;
  const int tokA = t0 + warp * tpw + rowA / G, tokB = t0 + warp * tpw + rowB / G;
  const int pA = (rowA < tpw * G && tokA < t1) ? p_first + tokA : NO_ROW;
  const int pB = (rowB < tpw * G && tokB < t1) ? p_first + tokB : NO_ROW;
  const int warp_hi = p_first + min(t1, t0 + (warp + 1) * tpw) - 1;        // last position this warp's rows see
  // the warp's query rows as MMA fragments, straight from global memory (rows that do not exist are zeros)
  uint32_t qf[KB][4];
  {
    const bf16* qa = pA != NO_ROW ? qkv + (size_t)(q0 + tokA) * row_stride + (size_t)(kvh * G + rowA % G) * D : nullptr;
    const bf16* qb = pB != NO_ROW ? qkv + (size_t)(q0 + tokB) * row_stride + (size_t)(kvh * G + rowB % G) * D : nullptr;
    const int c0 = (lane & 3) << 1;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
      qf[kb][0] = qa ? *reinterpret_cast<const uint32_t*>(qa + kb * 16 + c0) : 0u;
      qf[kb][1] = qb ? *reinterpret_cast<const uint32_t*>(qb + kb * 16 + c0) : 0u;
      qf[kb][2] = qa ? *reinterpret_cast<const uint32_t*>(qa + kb * 16 + 8 + c0) : 0u;
      qf[kb][3] = qb ? *reinterpret_cast<const uint32_t*>(qb + kb * 16 + 8 + c0) : 0u;
    }
  }
  bool ok = true;
  for (int t = 0; t < n_tiles; ++t) {
    bf16* Ks = KV + (t & 1) * STAGE;
    bf16* Vs = Ks + (TMA ? BN * D : BN * DP);
    // tile t+1 goes to the other stage, which every warp left at the barrier that ended iteration t-1
    if (t + 1 < n_tiles) {
      bf16* Kn = KV + ((t + 1) & 1) * STAGE;
      if (TMA) {
        if (warp == 0)
          tma_issue_tile(&kv_map, Kn, &full_bar[(t + 1) & 1], bt, T0 + (t + 1) * BN, lo, hi, kvh, nkv, page_size, ps_shift,
                         total_rows, lane);
      } else {
        load_kv_tile(Kn, Kn + BN * DP, pages, bt, T0 + (t + 1) * BN, lo, hi, kvh, nkv, page_size, tid);
        cp_async_commit();
      }
    }
    if (TMA) {
      ok = att_mbar_wait(&full_bar[t & 1], (t >> 1) & 1, abort_flag, err, 2);
    } else {
      if (t + 1 < n_tiles) cp_async_wait<1>(); else cp_async_wait<0>();
    }
    __syncthreads();
    if (TMA && *abort_flag) { ok = false; break; }
    const int tile0 = T0 + t * BN;
    if (tile0 <= warp_hi) {
      // every key of the tile is seen by every row of this warp: no masking
      const bool interior = t0 + warp * tpw < t1 && tile0 >= lo && tile0 + BN - 1 <= min(hi, p_first + t0 + warp * tpw) &&
                            (window == 0 || tile0 >= warp_hi - window + 1);
      if (interior)
        warp_tile<8, false, TMA>(qf, Ks, Vs, 0, tile0, lo, hi, pA, pB, window, scale_log2, m, l, o, lane);
      else
        warp_tile<8, true, TMA>(qf, Ks, Vs, 0, tile0, lo, hi, pA, pB, window, scale_log2, m, l, o, lane);
    }
    __syncthreads();
  }
  if (TMA && !ok) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    return;
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

// ---------------------------------------------------------------------------------------------------
static size_t small_q_smem(bool tma) {
  return tma ? (size_t)(SQ_STAGES * 2 * BN * D + 16 * DP) * sizeof(bf16) + 1024 : (size_t)(SQ_STAGES * 2 * BN * DP + 16 * DP) * sizeof(bf16);
}
static size_t tile_smem(bool tma) {
  return tma ? (size_t)(2 * 2 * BN * D) * sizeof(bf16) + 1024 : (size_t)(2 * 2 * BN * DP) * sizeof(bf16);
}

// The pool [pages, 2, kv_heads, page_size, D] as a matrix [rows, D] with boxes of page_size rows x 64 columns in
// the 128-byte swizzle.
static int kv_tensor_map(CUtensorMap* out, const void* pages, long long rows, int page_size) {
  const unsigned long long dims[2] = {(unsigned long long)D, (unsigned long long)rows};
  const unsigned long long strides[1] = {(unsigned long long)D * sizeof(bf16)};
  const unsigned box[2] = {64, (unsigned)page_size};
  return ifb_tensor_map_bf16(out, pages, 2, dims, strides, box);
}

IFB_EXPORT int ifb_attention_mma_head_dim() { return D; }

// Floats of scratch the small-q kernel needs for `n_tokens` tokens of `nq` heads in `num_splits` splits.
IFB_EXPORT long long ifb_attention_mma_scratch_floats(int n_tokens, int nq, int num_splits) {
  return num_splits > 1 ? (long long)n_tokens * nq * num_splits * (D + 2) : 0;
}

template <bool TMA>
static int att_launch(const CUtensorMap& map, int total_rows, int* err, const void* qkv, int row_stride, const void* pages,
                      const int* block_tables, int bt_stride, const int* cu_q, const int* seq_lens, void* out, float* scratch,
                      int* counters, int n_tokens, int n_req, int nq, int nkv, int page_size, float scale_log2, int window,
                      int max_q_len, int num_splits, int run_small, int run_tiles, cudaStream_t stream) {
  if (TMA) IFB_ALLOW_SMEM(attn_small_q_ws_kernel, small_q_smem(true));
  else IFB_ALLOW_SMEM(attn_small_q_kernel<false>, small_q_smem(false));
  IFB_ALLOW_SMEM(attn_tile_kernel<TMA>, tile_smem(TMA));
  const int G = nq / nkv;
  if (run_small) {
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)n_tokens * nq * num_splits * D : nullptr;
    dim3 grid(num_splits, nkv, n_req);
    int st;
    if (TMA)
      st = ifb_launch(attn_small_q_ws_kernel, grid, dim3(WS_THREADS), small_q_smem(true), stream, map, total_rows, err,
                      (const bf16*)qkv, row_stride, block_tables, bt_stride, cu_q, seq_lens, (bf16*)out, part_o, part_ml,
                      counters, nq, nkv, page_size, scale_log2, window, num_splits);
    else
      st = ifb_launch(attn_small_q_kernel<false>, grid, dim3(THREADS), small_q_smem(false), stream, map, total_rows, err,
                      (const bf16*)qkv, row_stride, (const bf16*)pages, block_tables, bt_stride, cu_q, seq_lens, (bf16*)out,
                      part_o, part_ml, counters, nq, nkv, page_size, scale_log2, window, num_splits);
    if (st) return st;
  }
  if (run_tiles) {
    const int tpc = 4 * (16 / G);
    dim3 grid((max_q_len + tpc - 1) / tpc, nkv, n_req);
    return ifb_launch(attn_tile_kernel<TMA>, grid, dim3(THREADS), tile_smem(TMA), stream, map, total_rows, err, (const bf16*)qkv,
                      row_stride, (const bf16*)pages, block_tables, bt_stride, cu_q, seq_lens, (bf16*)out, nq, nkv, page_size,
                      scale_log2, window);
  }
  return IFB_OK;
}

// max_q_len: the most query tokens any request brings.  run_small / run_tiles: which of the two kernels to
// launch; requests are routed by rows = q_len * (nq / nkv) <= 16.  num_pages: pages of the pool `pages`.
// err: a device int that stays 0 unless a bounded wait gave up (TMA path).  use_tma 0 forces the cp.async path.
IFB_EXPORT int ifb_attention_mma(const void* qkv, int row_stride, const void* pages, long long num_pages,
                                 const int* block_tables, int bt_stride, const int* cu_q, const int* seq_lens, void* out,
                                 float* scratch, int* counters, int* err, int n_tokens, int n_req, int nq, int nkv, int d,
                                 int page_size, float scale, int window, int max_q_len, int num_splits, int run_small,
                                 int run_tiles, int use_tma, cudaStream_t stream) {
  if (n_tokens <= 0 || n_req <= 0) return IFB_OK;
  if (d != D) return IFB_ERR_SIZE;
  if (nkv < 1 || nq % nkv || page_size < 1 || window < 0 || num_splits < 1) return IFB_ERR_ARG;
  const int G = nq / nkv;
  if (G > 16 && run_tiles) return IFB_ERR_SIZE;
  if (row_stride % 8 || ((uintptr_t)qkv & 15) || ((uintptr_t)pages & 15) || ((uintptr_t)out & 3)) return IFB_ERR_ALIGN;
  if (n_req > 65535 || nkv > 65535) return IFB_ERR_SIZE;
  if (run_small && num_splits > 1 && (!scratch || !counters)) return IFB_ERR_ARG;
  const float scale_log2 = scale * 1.4426950408889634f;
  const long long rows = num_pages * 2 * nkv * page_size;
  const bool tma = use_tma && TMA_D && err && (page_size == 16 || page_size == 32 || page_size == 64) && rows < 0x7fffffffLL &&
                   ((uintptr_t)pages & 127) == 0;
  CUtensorMap map;
  if (tma) {
    int st = kv_tensor_map(&map, pages, rows, page_size);
    if (st) return st;
    return att_launch<true>(map, (int)rows, err, qkv, row_stride, pages, block_tables, bt_stride, cu_q, seq_lens, out, scratch,
                            counters, n_tokens, n_req, nq, nkv, page_size, scale_log2, window, max_q_len, num_splits, run_small,
                            run_tiles, stream);
  }
  memset(&map, 0, sizeof(map));
  return att_launch<false>(map, 0, err, qkv, row_stride, pages, block_tables, bt_stride, cu_q, seq_lens, out, scratch, counters,
                           n_tokens, n_req, nq, nkv, page_size, scale_log2, window, max_q_len, num_splits, run_small, run_tiles,
                           stream);
}
