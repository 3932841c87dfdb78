// Attention for prompts and long portions on the fifth-generation tensor cores, head size 128.
//
// A CTA takes one query tile of 128 score rows of one key/value head: 128/G query tokens times the G query heads
// of the group (row = token * G + head-in-group).  The keys are loaded in tiles of 128 (two stages each for K and V)
// and worked on in halves of 64 by two streams: stream x takes half x of every tile, with its own score buffers,
// running maxima and sums, and its own output accumulator; the two are merged at the end.  So the chain of one row's
// softmax (scores out of tensor memory, maximum, 64 exponentials, P back into tensor memory: 1,340 cycles a half,
// which no mix of ex2.approx and polynomials shortened, a lone warp per scheduler being bound by the latency of its
// own instructions) runs twice side by side, on the two warps that every scheduler of the SM then holds, and a tile
// of 128 keys costs one such chain where one stream needed two.  Per stream and its i-th half:
//   S[i & 1] = Q K^T  tcgen05.mma, Q and K in shared memory (TMA, 128-byte swizzle), the scores in one of the
//                     stream's two score buffers in tensor memory, so that S(i+1) is formed while the softmax of
//                     S(i) runs;
//   softmax           four warps per stream, one thread per row: the row's 64 scores are read from tensor
//                     memory into registers, masked, exponentiated against the running maximum (float32), summed,
//                     and written back over the scores as bfloat16 P; the running output is rescaled in tensor
//                     memory only when a maximum grew by more than 2^8 (the kept maximum may lag by that much,
//                     which float32 sums and bfloat16 P hold without loss);
//   O += P V          tcgen05.mma with P as the A operand in tensor memory and V from shared memory as an
//                     MN-major B operand (V is stored [key][dim], the dim running fastest).
// Warp 0 issues the TMA loads (the query tile through a three-dimensional tensor map over the fused qkv rows,
// key/value tiles page by page as in attention_mma.cu) after waiting for the kernel before this one; warps 1 and
// 2 issue the MMAs of stream 0 and 1 (all lanes wait on the barriers, one lane elected by elect.sync issues:
// descriptors then live in uniform registers, which is worth 40 cycles per MMA); warp 3 idles; warps 4-7 and 8-11
// do the softmax of stream 0 and 1 and, after exchanging their maxima and sums through shared memory, each the
// final division and store of half of the head's columns.  Tensor memory: per stream two score buffers of 64 columns
// and 128 columns of output, 512 columns in all, so one CTA per SM.  The grid is the tiles of the longest request
// times the key/value heads, the tiles with the most keys first, so that the short ones fill the SMs' last rounds.
//
// Requests are routed as in attention_mma.cu: this kernel takes those with more than 16 score rows,
// the small-q kernel there takes the others.  Waits on barriers are bounded (TC_SPIN_LIMIT polls, then
// a code in *err and the CTA's abort flag).
#include <cuda.h>
#include <type_traits>
#include "common.cuh"
#include <math.h>
#include <string.h>

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
#if HEAD_DIM != 128
#error "attention_tc.cu is written for head size 128"
#endif

typedef __nv_bfloat16 bf16;
constexpr int D = 128;
constexpr int ROWS = 128;                 // score rows per CTA (MMA M)
constexpr int BK = 128;                   // keys per tile loaded
constexpr int SUB = 64;                   // keys per score buffer (MMA N of S, K of P V per half)
constexpr int TC_THREADS = 384;                // producer warp, two MMA warps, an idle warp, two softmax groups of four
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;
constexpr int HALF_BYTES = 128 * 128;     // a [128 rows][64 columns] bf16 half tile in the 128-byte swizzle: 16 KB
constexpr int TILE_BYTES = 2 * HALF_BYTES;
constexpr int SMEM_BYTES = 5 * TILE_BYTES /* Q, 2 K, 2 V */ + 1024 /* alignment */;   // 161 KB
// tensor memory columns (32-bit), per stream: two score buffers [0,64) and [64,128), P (bfloat16 pairs) written
// over the first 32 columns of a buffer once its row has been read, O [128,256).  Two streams: all 512 columns.
constexpr int COL_S = 0, COL_O = 128, COLS_PER_TILE = 256, TMEM_COLS = 512;
constexpr int NO_ROW = -1000000000;


__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(tc_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(tc_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool tc_mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(tc_smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool tc_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
  unsigned long long t0 = 0;
  for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
    if (tc_mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (ifb_wait_expired(i, t0)) break;
  }
  *abort_flag = 1;
  atomicExch(err, code);
  return false;
}
__device__ __forceinline__ void tc_tma_2d(void* smem, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(tc_smem_u32(smem)), "l"(map), "r"(tc_smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_tma_3d(void* smem, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
               ::"r"(tc_smem_u32(smem)), "l"(map), "r"(tc_smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
// True in exactly one lane of a converged warp.  Code under it is known to the compiler as single-threaded, which lets
// it keep the descriptors of the copies and products it issues in uniform registers.
__device__ __forceinline__ bool tc_elect_one() {
  uint32_t pred;
  asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tc_smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] B[smem]
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// D[tmem] (+)= A[tmem] B[smem]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ float tc_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// 2^x for x <= 8 without the special-function unit: x = n + f with n = round(x) (the magic-number addition leaves n
// in the low mantissa bits), 2^f by a cubic on [-0.5, 0.5] (largest relative error 7.5e-5, a fiftieth of the rounding
// of P to bfloat16), n added into the exponent bits.  Five operations on the FMA pipe and two on the integer pipe,
// against eight cycles of the special-function unit per warp for ex2.approx.
__device__ __forceinline__ float tc_exp2_poly(float x) {
  x = fmaxf(x, -125.f);
  const float magic = 12582912.f;                    // 1.5 * 2^23
  const float xf = x + magic;
  const float f = x - (xf - magic);
  float pl = fmaf(0.0551716648f, f, 0.2426111251f);
  pl = fmaf(pl, f, 0.6932609677f);
  pl = fmaf(pl, f, 0.9999280572f);
  return __int_as_float(__float_as_int(pl) + (__float_as_int(xf) << 23));
}
#ifndef IFB_TC_POLY_MASK
#define IFB_TC_POLY_MASK 0x0000
#endif
template <int N, int I = 0, typename F> __device__ __forceinline__ void tc_static_for(F&& f) {
  if constexpr (I < N) { f(std::integral_constant<int, I>{}); tc_static_for<N, I + 1>(f); }
}
// which of a row's 16 consecutive scores take the cubic (bit i of the mask for score i mod 16), the rest ex2.approx
template <int I> __device__ __forceinline__ float tc_exp2_mixed(float x) {
  if constexpr ((IFB_TC_POLY_MASK >> (I & 15)) & 1) return tc_exp2_poly(x);
  else return tc_exp2(x);
}
__device__ __forceinline__ float tc_max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
#ifndef IFB_TC_PACK_INT
#define IFB_TC_PACK_INT 1
#endif
__device__ __forceinline__ uint32_t tc_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// The same for the probabilities (non-negative, finite), rounded to nearest with halves away from zero, by two integer
// additions and a byte permutation.
__device__ __forceinline__ uint32_t tc_pack_p(float lo, float hi) {
#if IFB_TC_PACK_INT
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, 0x7632;\n" : "=r"(r) : "r"(__float_as_uint(lo) + 0x8000u), "r"(__float_as_uint(hi) + 0x8000u));
  return r;
#else
  return tc_pack(lo, hi);
#endif
}

// K-major operand (rows of 128 bytes = 64 k, groups of 8 rows 1024 bytes apart), 128-byte swizzle: Q and K tiles.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand, 128-byte swizzle: the V tile [key][dim] as B = [dim (N)][key (K)].  64 dims (128 bytes) are one
// swizzle row; the next 64 dims lie HALF_BYTES further (leading byte offset); 8 keys are 1024 bytes (stride byte offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)(HALF_BYTES >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
// float32 accumulator, bfloat16 A and B, M = 128; S = Q K^T: N = 64 keys, B K-major; O += P V: N = 128 (the head
// size), B MN-major.
constexpr uint32_t IDESC_BASE = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 4) << 24);
constexpr uint32_t IDESC_S = IDESC_BASE | ((uint32_t)(SUB >> 3) << 17);
constexpr uint32_t IDESC_PV = IDESC_BASE | ((uint32_t)(128 >> 3) << 17) | (1u << 16);

struct TcBars {
  // [stream][stage or buffer]; q_empty: both issuers have read the query tile; o_free: the softmax warps have read the
  // outputs of the item before
  uint64_t q_full, q_empty, o_free, k_full[2], v_full[2], k_empty[2][2], v_empty[2][2], s_full[2][2], p_ready[2][2], o_done[2];
};

// One work item: a query tile of one key/value head.
struct TcItem {
  int kvh, t0, t1, lo, hi, T0, n_half, n_tiles;
};
// Round k of a CTA's walk over the request's items (item = tile rank * nkv + head, the tiles with the most keys first):
// forwards in even rounds, backwards in odd ones, so that the CTAs with the longest items of one round get the
// shortest of the next.  False: the round has no item for this CTA.
__device__ __forceinline__ bool tc_item(int k, int cta, int ctas, int nt, int nkv, int tpt, int q_len, int p_first, int window,
                                        TcItem& it) {
  const int idx = (k & 1) ? (k + 1) * ctas - 1 - cta : k * ctas + cta;
  if (idx >= nt * nkv) return false;
  const int rank = idx / nkv;
  it.kvh = idx % nkv;
  it.t0 = (nt - 1 - rank) * tpt;
  it.t1 = min(q_len, it.t0 + tpt);
  it.lo = window > 0 ? max(0, p_first + it.t0 - window + 1) : 0;
  it.hi = p_first + it.t1 - 1;
  it.T0 = (it.lo / BK) * BK;
  it.n_half = (it.hi + 1 - it.T0 + SUB - 1) / SUB;       // halves of 64 keys; stream x works on half x of every tile of 128
  it.n_tiles = (it.n_half + 1) / 2;
  return true;
}

__global__ void __launch_bounds__(TC_THREADS, 1)
attn_tile_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map, int total_rows,
                    int* __restrict__ err, const int* __restrict__ block_tables, int bt_stride,
                    const int* __restrict__ cu_q, const int* __restrict__ seq_lens, bf16* __restrict__ out, int nq, int nkv,
                    int page_size, float scale_log2, int window) {
  extern __shared__ unsigned char tc_smem_raw[];
  __shared__ TcBars bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;
  __shared__ float merge_m[2][2][ROWS], merge_l[2][2][ROWS];       // [item parity][stream][row]: maxima and sums, exchanged
  volatile int* abort_flag = &abort_word;
  const uint32_t raw = tc_smem_u32(tc_smem_raw);
  unsigned char* smem = tc_smem_raw + (((raw + 1023u) & ~1023u) - raw);
  unsigned char* Qs = smem;                                  // the query tile, [2 halves][128 rows][128 bytes]
  unsigned char* Ks = smem + TILE_BYTES;                     // two stages of K tiles, same layout
  unsigned char* Vs = smem + 3 * TILE_BYTES;                 // two stages of V tiles
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;     // warp-uniform
  const int r = blockIdx.z, cta = blockIdx.x, ctas = gridDim.x;
  const int G = nq / nkv;
  const int q0 = cu_q[r], q_len = cu_q[r + 1] - q0, L = seq_lens[r];
  // every exit path waits for the predecessor: a grid none of whose threads waited could end before the kernel that
  // stores this step's keys, and its own successor, which waits for this grid alone, would then start too early
  if (q_len * G <= 16) { ifb_pdl_wait(); return; }           // the small-q kernel's request
  const int tpt = ROWS / G;                                  // tokens per query tile
  const int nt = (q_len + tpt - 1) / tpt;
  const int n_items = nt * nkv;
  if (cta >= n_items) { ifb_pdl_wait(); return; }
  const int n_rounds = (n_items + ctas - 1) / ctas;
  const int p_first = L - q_len;
  const int* bt = block_tables + (size_t)r * bt_stride;
  const int ps_shift = __ffs(page_size) - 1;

  if (threadIdx.x == 0) {
    tc_mbar_init(&bars.q_full, 1);
    tc_mbar_init(&bars.q_empty, 2);
    tc_mbar_init(&bars.o_free, 256);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      tc_mbar_init(&bars.k_full[i], 1); tc_mbar_init(&bars.v_full[i], 1);
      tc_mbar_init(&bars.o_done[i], 1);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        tc_mbar_init(&bars.k_empty[i][h], 1); tc_mbar_init(&bars.v_empty[i][h], 1);
        tc_mbar_init(&bars.s_full[i][h], 1); tc_mbar_init(&bars.p_ready[i][h], 128);
      }
    }
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 0 || warp == 3) {
    // ---------------- producers.  Warp 0 brings the query tiles and the K tiles, warp 3 the V tiles, each as soon as
    // both streams have left the stage: were one warp to bring both in turn, the next K tile would wait behind the
    // release of a V tile it has nothing to do with.  Their wait for the kernel before this one (which wrote the queries
    // and this step's keys and values) orders the whole CTA behind it: the other warps act only on what these loads bring.
    const int kv = warp == 3;
    ifb_pdl_wait();
    if (!kv) ifb_pdl_trigger();
    const int ppt = BK >> ps_shift;                          // pages per tile: 8, 4 or 2
    const int n_ops = ppt * 2;                               // x 2 halves: at most 16 per tile
    bool ok = true;
    int jt = 0, ic = 0;                                      // tiles and items so far
    for (int k = 0; k < n_rounds && ok; ++k) {
      TcItem it;
      if (!tc_item(k, cta, ctas, nt, nkv, tpt, q_len, p_first, window, it)) continue;
      if (!kv) {
        if (ic > 0) ok = tc_mbar_wait(&bars.q_empty, (ic - 1) & 1, abort_flag, err, 10);
        if (!ok) break;
        if (lane == 0) {
          tc_mbar_expect_tx(&bars.q_full, TILE_BYTES);
          tc_tma_3d(Qs, &q_map, &bars.q_full, 0, it.kvh * G, q0 + it.t0);
          tc_tma_3d(Qs + HALF_BYTES, &q_map, &bars.q_full, 64, it.kvh * G, q0 + it.t0);
        }
        __syncwarp();
      }
      for (int j = 0; j < it.n_tiles && ok; ++j, ++jt) {
        const int st = jt & 1;
        uint64_t* full = kv ? &bars.v_full[st] : &bars.k_full[st];
        if (jt >= 2) {                                       // the tile two back has left this stage, for both streams
#pragma unroll
          for (int x = 0; x < 2; ++x)
            if (ok) ok = tc_mbar_wait(kv ? &bars.v_empty[x][st] : &bars.k_empty[x][st], ((jt >> 1) - 1) & 1, abort_flag, err, 11);
        }
        if (!ok) break;
        if (lane == 0) tc_mbar_expect_tx(full, TILE_BYTES);
        __syncwarp();
        if (lane < n_ops) {
          const int pg = lane >> 1, half = lane & 1;
          const int key0 = it.T0 + j * BK + pg * page_size;
          int y = total_rows;                                // beyond the tensor: zeros
          if (key0 <= it.hi && key0 + page_size - 1 >= it.lo) y = ((bt[key0 >> ps_shift] * 2 + kv) * nkv + it.kvh) * page_size;
          tc_tma_2d((kv ? Vs : Ks) + st * TILE_BYTES + half * HALF_BYTES + pg * page_size * 128, &kv_map, full, half * 64, y);
        }
      }
      ++ic;
    }
  } else if (warp == 1 || warp == 2) {
    // ---------------- MMA issuers, one warp per stream x.  The stream has two score buffers of 64 keys; its halves go
    // to them in turn (counted over all items), and P is written over a buffer's first columns.  The tensor core
    // takes a warp's operations in the order they are issued:
    //   S(0) S(1) | O(i) S(i+2) | ...
    // so the scores of the next half are there before the softmax of this half ends, and S(i+2) lands where P(i)
    // lay only after O(i) has read it.  While one warp checks its barriers the other's products keep the pipe full.
    const int x = warp - 1;
    const uint32_t q_addr = tc_smem_u32(Qs), k_addr = tc_smem_u32(Ks) + x * (SUB * 128), v_addr = tc_smem_u32(Vs) + x * (SUB * 128);
    const uint32_t tb = tmem + x * COLS_PER_TILE;
    bool ok = true;
    int kc = 0, hc = 0, ic = 0;                              // key tiles, this stream's halves, and items so far
    for (int k = 0; k < n_rounds && ok; ++k) {
      TcItem it;
      if (!tc_item(k, cta, ctas, nt, nkv, tpt, q_len, p_first, window, it)) continue;
      const int n_mine = (it.n_half + 1 - x) / 2;
      ok = tc_mbar_wait(&bars.q_full, ic & 1, abort_flag, err, 12);
      auto issue_qk = [&](int i) {
        // S = Q K^T for the stream's 64 keys of the item's tile i: 8 steps of 16 along the head size, 4 per 64-column
        // half of Q and K; then the stream is done with the tile of keys (and, after its last half, with the queries)
        const int st = (kc + i) & 1, buf = (hc + i) & 1;
        ok = ok && tc_mbar_wait(&bars.k_full[st], ((kc + i) >> 1) & 1, abort_flag, err, 13);
        if (!ok) return;
        tc_fence_after();
        if (tc_elect_one()) {
          const uint64_t qd = desc_k_major(q_addr), kd = desc_k_major(k_addr + st * TILE_BYTES);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t off = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;       // descriptor addresses count 16 bytes
            tc_mma_ss(tb + COL_S + buf * SUB, qd + off, kd + off, IDESC_S, ks != 0);
          }
          tc_commit(&bars.s_full[x][buf]);
          tc_commit(&bars.k_empty[x][st]);
          if (i == n_mine - 1) tc_commit(&bars.q_empty);
        }
        __syncwarp();
      };
      if (ok && n_mine > 0) issue_qk(0);
      if (ok && n_mine > 1) issue_qk(1);
      for (int i = 0; i < n_mine && ok; ++i) {
        const int st = (kc + i) & 1, buf = (hc + i) & 1;
        ok = tc_mbar_wait(&bars.v_full[st], ((kc + i) >> 1) & 1, abort_flag, err, 18);
        ok = ok && tc_mbar_wait(&bars.p_ready[x][buf], ((hc + i) >> 1) & 1, abort_flag, err, 14);
        // the first product of an item overwrites the outputs of the item before, which the softmax warps must have read
        if (ok && i == 0 && ic > 0) ok = tc_mbar_wait(&bars.o_free, (ic - 1) & 1, abort_flag, err, 9);
        if (!ok) break;
        tc_fence_after();
        // O += P V: 4 steps of 16 keys; P at 8 columns (16 bfloat16) per step, V 2048 bytes (16 key rows) per step
        if (tc_elect_one()) {
          const uint64_t vd = desc_mn_major(v_addr + st * TILE_BYTES);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            tc_mma_ts(tb + COL_O, tb + COL_S + buf * SUB + ks * 8, vd + ks * (2048 >> 4), IDESC_PV, (i | ks) != 0);
          tc_commit(&bars.o_done[x]);
          tc_commit(&bars.v_empty[x][st]);
        }
        __syncwarp();
        if (i + 2 < n_mine) issue_qk(i + 2);
      }
      if (!ok) break;
      if (n_mine < it.n_tiles) {
        // an odd number of halves: the last tile has none for stream 1, which leaves it (and, if it had no half at
        // all, the queries) untouched; the producers count on a release from both streams
        const int last = kc + it.n_tiles - 1;
        ok = tc_mbar_wait(&bars.k_full[last & 1], (last >> 1) & 1, abort_flag, err, 20) &&
             tc_mbar_wait(&bars.v_full[last & 1], (last >> 1) & 1, abort_flag, err, 21);
        if (!ok) break;
        if (tc_elect_one()) {
          const int st = last & 1;
          tc_commit(&bars.k_empty[x][st]);
          tc_commit(&bars.v_empty[x][st]);
          if (n_mine == 0) tc_commit(&bars.q_empty);
        }
        __syncwarp();
      }
      kc += it.n_tiles; hc += n_mine; ++ic;
    }
  } else if (warp >= 4) {
    // ---------------- softmax: warps 4-7 take stream 0, warps 8-11 stream 1; one thread per row
    const int x = (warp - 4) >> 2;
    const int qd = warp & 3;                                 // this warp's quarter of the 128 lanes
    const int row = qd * 32 + lane;
    const uint32_t lane_addr = tmem + ((uint32_t)(qd * 32) << 16) + x * COLS_PER_TILE;
    uint64_t* o_done = &bars.o_done[x];
    bool ok = true;
    int hc = 0, ic = 0;                                      // this stream's halves and the items so far
    for (int k = 0; k < n_rounds; ++k) {
      TcItem it;
      if (!tc_item(k, cta, ctas, nt, nkv, tpt, q_len, p_first, window, it)) continue;
      const int n_mine = (it.n_half + 1 - x) / 2;
      const int t0x = it.t0, t1x = it.t1, T0 = it.T0, kvh = it.kvh;
      const int tok = t0x + row / G;
      const int p = tok < t1x ? p_first + tok : NO_ROW;
      const int row_lo = window > 0 ? p - window + 1 : 0;
      const int lox = it.lo, hix = it.hi;
      float m_used = -INFINITY, l = 0.f;
      for (int u = 0; u < n_mine && ok; ++u) {
        const int c = hc + u, h = c & 1;
        ok = __all_sync(0xffffffffu, tc_mbar_wait(&bars.s_full[x][h], (c >> 1) & 1, abort_flag, err, 15)) != 0;    // warp-uniform
        if (!ok) break;
        tc_fence_after();
        const int key0 = T0 + (2 * u + x) * SUB;             // the stream's half of the item's key tile u
        const uint32_t s_addr = lane_addr + COL_S + h * SUB;
        // a half every key of which every row of the query tile sees needs no masking (rows past the request's tokens
        // are computed like the others and never stored)
        const bool interior = key0 >= lox && key0 + SUB - 1 <= min(hix, p_first + t0x) && (window == 0 || key0 >= hix - window + 1);
        // the row's visible keys of this half are those with index in [vis_lo, vis_hi): the causal rule, the window and
        // the ends of what the item's tile may see, in two numbers (a row past the request's tokens sees none)
        const int vis_hi = min(p, hix) - key0 + 1, vis_lo = max(row_lo, lox) - key0;
        // the row's 64 scores into registers with one wait
        uint32_t v[2][32];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) tc_ld32(s_addr + cc * 32, v[cc]);
        tc_wait_ld();
        // the row's maximum over the visible keys, four chains
        float mxc[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (interior) {
#pragma unroll
          for (int cc = 0; cc < 2; ++cc)
#pragma unroll
            for (int i = 0; i < 32; i += 2)                      // the three-input maximum: half the instructions
              mxc[(cc << 1) | ((i >> 1) & 1)] = tc_max3(mxc[(cc << 1) | ((i >> 1) & 1)], __uint_as_float(v[cc][i]), __uint_as_float(v[cc][i + 1]));
        } else {
#pragma unroll
          for (int cc = 0; cc < 2; ++cc)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const bool vis = cc * 32 + i < vis_hi && cc * 32 + i >= vis_lo;
              if (vis) mxc[(cc << 1) | (i & 1)] = fmaxf(mxc[(cc << 1) | (i & 1)], __uint_as_float(v[cc][i]));
            }
        }
        const float mx = fmaxf(fmaxf(mxc[0], mxc[1]), fmaxf(mxc[2], mxc[3])) * scale_log2;   // the scale is positive
        // keep the old reference maximum unless the new one is more than 2^8 above it (warp-uniform decision,
        // since the tensor-memory loads and stores of the rescaling are warp-wide)
        const float m_new = fmaxf(m_used, mx);
        const bool grow = m_new > m_used + 8.f;
        const bool any_grow = __any_sync(0xffffffffu, grow) != 0;
        float factor = 1.f;
        if (any_grow && grow) {
          factor = m_used == -INFINITY ? 0.f : tc_exp2(m_used - m_new);
          m_used = m_new;
        }
        const float ref = m_used == -INFINITY ? 0.f : m_used;
        bool o_waited = false;                 // whether this step has waited for the previous half's P V
        if (u > 0 && any_grow) {
          // O is rescaled between the previous half's P V, which must have landed, and this half's, which waits for P
          ok = __all_sync(0xffffffffu, tc_mbar_wait(o_done, (c - 1) & 1, abort_flag, err, 16)) != 0;
          if (!ok) break;
          o_waited = true;
          tc_fence_after();
          l *= factor;
#pragma unroll 1
          for (int cc = 0; cc < 8; ++cc) {
            uint32_t o[16];
            tc_ld16(lane_addr + COL_O + cc * 16, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
            tc_st16(lane_addr + COL_O + cc * 16, o);
          }
        }
        // p = 2^(s - ref), the row sum, and P as bfloat16 pairs over the first 32 columns of this score buffer (its
        // scores are all in registers by now)
        float lc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t pk[16];
          if (interior) {
#pragma unroll
            tc_static_for<16>([&](auto idx) {
              constexpr int i = decltype(idx)::value * 2;
              const float e0 = tc_exp2_mixed<i>(fmaf(__uint_as_float(v[cc][i]), scale_log2, -ref));
              const float e1 = tc_exp2_mixed<i + 1>(fmaf(__uint_as_float(v[cc][i + 1]), scale_log2, -ref));
              lc[i & 2] += e0; lc[(i & 2) + 1] += e1;
              pk[i >> 1] = tc_pack_p(e0, e1);
            });
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const bool v0 = cc * 32 + i < vis_hi && cc * 32 + i >= vis_lo;
              const bool v1 = cc * 32 + i + 1 < vis_hi && cc * 32 + i + 1 >= vis_lo;
              const float e0 = v0 ? tc_exp2(fmaf(__uint_as_float(v[cc][i]), scale_log2, -ref)) : 0.f;
              const float e1 = v1 ? tc_exp2(fmaf(__uint_as_float(v[cc][i + 1]), scale_log2, -ref)) : 0.f;
              lc[i & 2] += e0; lc[(i & 2) + 1] += e1;
              pk[i >> 1] = tc_pack_p(e0, e1);
            }
          }
          tc_st16(s_addr + cc * 16, pk);
        }
        l += (lc[0] + lc[1]) + (lc[2] + lc[3]);
        tc_wait_st();
        tc_fence_before();
        // A wait by parity tells phase k of o_done from phase k - 2 only for a waiter that has seen phase k - 1.  This
        // half's scores imply that P V of the half two back has landed (the tensor core runs one warp's operations in
        // order) but say nothing of the half before, so every step waits for it (by now it has almost always landed)
        // before it hands over P: the step that skipped it when no row's maximum grew would leave the wait after the
        // last half one phase short, and that wait would pass on the phase two back while P V was still in flight.
        // (The first half of an item has nothing to wait for: the item before ended with such a wait.)
        if (u > 0 && !o_waited) {
          ok = __all_sync(0xffffffffu, tc_mbar_wait(o_done, (c - 1) & 1, abort_flag, err, 19)) != 0;
          if (!ok) break;
        }
        tc_mbar_arrive(&bars.p_ready[x][h]);
      }
      if (ok && n_mine > 0) ok = __all_sync(0xffffffffu, tc_mbar_wait(o_done, (hc + n_mine - 1) & 1, abort_flag, err, 17)) != 0;
      // The streams hand each other their maxima and sums; each then divides and stores half of the head's columns,
      // out = (2^(m0 - m) O0 + 2^(m1 - m) O1) / (2^(m0 - m) l0 + 2^(m1 - m) l1) with m the larger of the two maxima.
      const int par = ic & 1;
      merge_m[par][x][row] = m_used;
      merge_l[par][x][row] = l;
      tc_fence_before();
      asm volatile("bar.sync 2, 256;\n" ::: "memory");          // the eight softmax warps, on every path
      tc_fence_after();
      const bool go = __all_sync(0xffffffffu, !*abort_flag) != 0;      // warp-uniform: the loads below are the whole warp's
      if (go) {
        const float m0 = merge_m[par][0][row], m1 = merge_m[par][1][row], l0 = merge_l[par][0][row], l1 = merge_l[par][1][row];
        const float m = fmaxf(m0, m1);
        const float a0 = m0 == -INFINITY ? 0.f : tc_exp2(m0 - m), a1 = m1 == -INFINITY ? 0.f : tc_exp2(m1 - m);
        const float denom = a0 * l0 + a1 * l1;
        const float inv = denom > 0.f ? 1.f / denom : 0.f;
        const float w0 = a0 * inv, w1 = a1 * inv;
        const bool two = it.n_half > 1;                          // stream 1's accumulator holds something of this item
        const uint32_t o_addr = tmem + ((uint32_t)(qd * 32) << 16) + COL_O;
        bf16* dst = p != NO_ROW ? out + ((size_t)(q0 + tok) * nq + kvh * G + row % G) * D + x * 64 : nullptr;
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t oa[32], ob[32];
          tc_ld32(o_addr + x * 64 + cc * 32, oa);
          if (two) tc_ld32(o_addr + COLS_PER_TILE + x * 64 + cc * 32, ob);
          tc_wait_ld();
          float y[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) y[i] = __uint_as_float(oa[i]) * w0;
          if (two) {
#pragma unroll
            for (int i = 0; i < 32; ++i) y[i] = fmaf(__uint_as_float(ob[i]), w1, y[i]);
          }
          if (dst) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 pk;
              pk.x = tc_pack(y[i], y[i + 1]);
              pk.y = tc_pack(y[i + 2], y[i + 3]);
              pk.z = tc_pack(y[i + 4], y[i + 5]);
              pk.w = tc_pack(y[i + 6], y[i + 7]);
              *reinterpret_cast<uint4*>(dst + cc * 32 + i) = pk;
            }
          }
        }
      }
      tc_fence_before();
      tc_mbar_arrive(&bars.o_free);            // this item's outputs have been read
      if (!go) break;
      ok = true;
      hc += n_mine; ++ic;
    }
  }
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}


// ---------------------------------------------------------------------------------------------------
// qkv [n_tokens, row_stride] bfloat16 (the q heads are the first nq * 128 columns), pages [num_pages, 2, nkv, page_size, 128],
// out [n_tokens, nq * 128].  Takes the requests with q_len * (nq / nkv) > 16.  The group size nq / nkv must divide 128 and
// page_size must be 16, 32 or 64.  err: a device int that stays 0 unless a bounded wait gave up.
IFB_EXPORT int ifb_attention_tc(const void* qkv, int row_stride, const void* pages, long long num_pages, const int* block_tables,
                                int bt_stride, const int* cu_q, const int* seq_lens, void* out, int* err, int n_tokens, int n_req,
                                int nq, int nkv, int d, int page_size, float scale, int window, int max_q_len,
                                cudaStream_t stream) {
  if (n_tokens <= 0 || n_req <= 0) return IFB_OK;
  if (d != D) return IFB_ERR_SIZE;
  if (nkv < 1 || nq % nkv || window < 0 || !err) return IFB_ERR_ARG;
  const int G = nq / nkv;
  if (G > ROWS || ROWS % G) return IFB_ERR_SIZE;
  if (page_size != 16 && page_size != 32 && page_size != 64) return IFB_ERR_SIZE;
  if (row_stride % 8 || ((uintptr_t)qkv & 15) || ((uintptr_t)pages & 127) || ((uintptr_t)out & 15)) return IFB_ERR_ALIGN;
  const long long rows = num_pages * 2 * nkv * page_size;
  if (rows >= 0x7fffffffLL || n_req > 65535) return IFB_ERR_SIZE;
  CUtensorMap q_map, kv_map;
  {
    const unsigned long long dims[3] = {(unsigned long long)D, (unsigned long long)nq, (unsigned long long)n_tokens};
    const unsigned long long strides[2] = {(unsigned long long)D * 2, (unsigned long long)row_stride * 2};
    const unsigned box[3] = {64, (unsigned)G, (unsigned)(ROWS / G)};
    if (ifb_tensor_map_bf16(&q_map, qkv, 3, dims, strides, box)) return IFB_ERR_ARG;
  }
  {
    const unsigned long long dims[2] = {(unsigned long long)D, (unsigned long long)rows};
    const unsigned long long strides[1] = {(unsigned long long)D * 2};
    const unsigned box[2] = {64, (unsigned)page_size};
    if (ifb_tensor_map_bf16(&kv_map, pages, 2, dims, strides, box)) return IFB_ERR_ARG;
  }
  IFB_ALLOW_SMEM(attn_tile_tc_kernel, SMEM_BYTES);
  const int tpt = ROWS / G;                                  // tokens per query tile
  const long long items = (long long)((max_q_len + tpt - 1) / tpt) * nkv;      // of the longest request
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      sm_count = 1;
  }
  dim3 grid((unsigned)(items < sm_count ? items : sm_count), 1, n_req);       // a CTA per SM walks the request's items
  return ifb_launch(attn_tile_tc_kernel, grid, dim3(TC_THREADS), (size_t)SMEM_BYTES, stream, q_map, kv_map, (int)rows, err, block_tables,
                    bt_stride, cu_q, seq_lens, (bf16*)out, nq, nkv, page_size, scale * 1.4426950408889634f, window);
}
