// Attention for prompts and long portions on the fifth-generation tensor cores, head size 128.
//
// A CTA takes two query tiles of 128 score rows of one key/value head: a tile is 128/G query tokens times the G
// query heads of the group (row = token * G + head-in-group).  Both tiles walk the same keys, loaded once, in
// tiles of 128 (two stages each for K and V) and worked on in halves of 64.  Per query tile and half u:
//   S[u & 1] = Q K^T  tcgen05.mma, Q and K in shared memory (TMA, 128-byte swizzle), the scores in one of the
//                     tile's two score buffers in tensor memory, so that S(u+1) is formed while the softmax of
//                     S(u) runs;
//   softmax           four warps per query tile, one thread per row: the row's 64 scores are read from tensor
//                     memory into registers, masked, exponentiated against the running maximum (float32), summed,
//                     and written back over the scores as bfloat16 P; the running output is rescaled in tensor
//                     memory only when a maximum grew by more than 2^8 (the kept maximum may lag by that much,
//                     which float32 sums and bfloat16 P hold without loss);
//   O += P V          tcgen05.mma with P as the A operand in tensor memory and V from shared memory as an
//                     MN-major B operand (V is stored [key][dim], the dim running fastest).
// Warp 0 issues the TMA loads (the query tiles through a three-dimensional tensor map over the fused qkv rows,
// key/value tiles page by page as in attention_mma.cu) after waiting for the kernel before this one; warps 1 and
// 2 issue the MMAs of query tile 0 and 1 (all lanes wait on the barriers, one lane elected by elect.sync issues:
// descriptors then live in uniform registers, which is worth 40 cycles per MMA); warp 3 idles; warps 4-7 and 8-11
// do the softmax and the final division and store of query tile 0 and 1.  Tensor memory: per query tile two score
// buffers of 64 columns and 128 columns of output, 512 columns in all, so one CTA per SM.
//
// Requests are routed as in attention_mma.cu: this kernel takes those with more than 16 score rows,
// the small-q kernel there takes the others.  Waits on barriers are bounded (TC_SPIN_LIMIT polls, then
// a code in *err and the CTA's abort flag).
#include <cuda.h>
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
constexpr int SMEM_BYTES = 6 * TILE_BYTES /* 2 Q, 2 K, 2 V */ + 1024 /* alignment */;   // 193 KB: one CTA per SM
// tensor memory columns (32-bit), per query tile: two score buffers [0,64) and [64,128), P (bfloat16 pairs) written
// over the first 32 columns of a buffer once its row has been read, O [128,256).  Two query tiles: all 512 columns.
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
  for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
    if (tc_mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
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
__device__ __forceinline__ float tc_max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
__device__ __forceinline__ uint32_t tc_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
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

// One softmax group: four warps, one thread per score row of query tile `x`.
struct TcBars {
  uint64_t q_full, k_full[2], v_full[2], k_empty[2][2], v_empty[2][2], s_full[2][2], p_ready[2][2], o_done[2];   // [query tile][stage or buffer]
};

__global__ void __launch_bounds__(TC_THREADS, 1)
attn_tile_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map, int total_rows,
                    int* __restrict__ err, const int* __restrict__ block_tables, int bt_stride,
                    const int* __restrict__ cu_q, const int* __restrict__ seq_lens, bf16* __restrict__ out, int nq, int nkv,
                    int page_size, float scale_log2, int window) {
  extern __shared__ unsigned char tc_smem_raw[];
  __shared__ TcBars bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const uint32_t raw = tc_smem_u32(tc_smem_raw);
  unsigned char* smem = tc_smem_raw + (((raw + 1023u) & ~1023u) - raw);
  unsigned char* Qs = smem;                                  // two query tiles, each [2 halves][128 rows][128 bytes]
  unsigned char* Ks = smem + 2 * TILE_BYTES;                 // two stages of K tiles, same layout
  unsigned char* Vs = smem + 4 * TILE_BYTES;                 // two stages of V tiles
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;     // warp-uniform
  const int kvh = blockIdx.y, r = blockIdx.z;
  const int G = nq / nkv;
  const int q0 = cu_q[r], q_len = cu_q[r + 1] - q0, L = seq_lens[r];
  // every exit path waits for the predecessor: a grid none of whose threads waited could end before the kernel that
  // stores this step's keys, and its own successor, which waits for this grid alone, would then start too early
  if (q_len * G <= 16) { ifb_pdl_wait(); return; }           // the small-q kernel's request
  const int tpt = ROWS / G;                                  // tokens per query tile; a CTA takes two tiles
  // Which two.  A tile's work grows with the keys it sees, so under the causal rule alone the CTA takes the j-th tile
  // from the front and the j-th from the back of the request's tokens: every CTA then has the same work (the keys of
  // the early tile are a prefix of the late tile's, so they still share them), where neighbouring tiles would give the
  // last CTA twice the average.  With a window every tile sees about as many keys, and neighbours share the most.
  const int nt = (q_len + tpt - 1) / tpt;
  int tok0[2];                                               // first token of each tile; tile 1 absent: q_len
  if (window > 0) {
    tok0[0] = (int)(gridDim.x - 1 - blockIdx.x) * 2 * tpt;   // longest key ranges first
    tok0[1] = min(q_len, tok0[0] + tpt);
  } else {
    const int j = blockIdx.x, other = nt - 1 - j;
    tok0[0] = j <= other ? j * tpt : q_len;
    tok0[1] = other > j ? other * tpt : q_len;
  }
  if (tok0[0] >= q_len) { ifb_pdl_wait(); return; }
  const int p_first = L - q_len;
  const int t_end = tok0[1] < q_len ? min(q_len, tok0[1] + tpt) : min(q_len, tok0[0] + tpt);    // one past the CTA's last token
  const int lo = window > 0 ? max(0, p_first + tok0[0] - window + 1) : 0, hi = p_first + t_end - 1;
  const int T0 = (lo / BK) * BK;
  // Keys are loaded in tiles of 128 and worked on in halves of 64: n_x[x] halves for query tile x (the second tile's
  // tokens come later, it sees at least as far).
  int n_x[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int t0x = tok0[x];
    const int hix = p_first + min(q_len, t0x + tpt) - 1;
    n_x[x] = (t0x < q_len && hix >= T0) ? (hix + 1 - T0 + SUB - 1) / SUB : 0;
  }
  const int n_sub = max(n_x[0], n_x[1]);
  const int n_tiles = (n_sub + 1) / 2;
  const int* bt = block_tables + (size_t)r * bt_stride;
  const int ps_shift = __ffs(page_size) - 1;

  if (threadIdx.x == 0) {
    tc_mbar_init(&bars.q_full, 1);
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

  if (warp == 0) {
    // ---------------- producer.  Its wait orders the whole CTA behind the kernel before this one (which wrote the
    // queries and this step's keys and values): the other warps act only on what its loads bring.
    ifb_pdl_wait();
    ifb_pdl_trigger();
    if (lane == 0) {
      tc_mbar_expect_tx(&bars.q_full, (n_x[1] > 0 ? 2 : 1) * TILE_BYTES);
#pragma unroll
      for (int x = 0; x < 2; ++x)
        if (n_x[x] > 0 || x == 0) {
          tc_tma_3d(Qs + x * TILE_BYTES, &q_map, &bars.q_full, 0, kvh * G, q0 + tok0[x]);
          tc_tma_3d(Qs + x * TILE_BYTES + HALF_BYTES, &q_map, &bars.q_full, 64, kvh * G, q0 + tok0[x]);
        }
    }
    const int ppt = BK >> ps_shift;                          // pages per tile: 8, 4 or 2
    const int n_ops = ppt * 2;                               // x 2 halves: at most 16 per tile
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j & 1;
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {                       // the K tile, then the V tile
        uint64_t* full = kv ? &bars.v_full[st] : &bars.k_full[st];
        if (j >= 2) {                                        // the tile two back has left this stage, for both query tiles
#pragma unroll
          for (int x = 0; x < 2; ++x)
            if (ok && 2 * (j - 2) < n_x[x])
              ok = tc_mbar_wait(kv ? &bars.v_empty[x][st] : &bars.k_empty[x][st], ((j >> 1) - 1) & 1, abort_flag, err, 11);
        }
        if (!ok) break;
        if (lane == 0) tc_mbar_expect_tx(full, TILE_BYTES);
        __syncwarp();
        if (lane < n_ops) {
          const int pg = lane >> 1, half = lane & 1;
          const int key0 = T0 + j * BK + pg * page_size;
          int y = total_rows;                                // beyond the tensor: zeros
          if (key0 <= hi && key0 + page_size - 1 >= lo) y = ((bt[key0 >> ps_shift] * 2 + kv) * nkv + kvh) * page_size;
          tc_tma_2d((kv ? Vs : Ks) + st * TILE_BYTES + half * HALF_BYTES + pg * page_size * 128, &kv_map, full, half * 64, y);
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ---------------- MMA issuers, one warp per query tile x.  The tile has two score buffers S[0], S[1] of 64 keys;
    // half u of the keys goes to S[u & 1], and P(u) is written over its first columns.  The tensor core takes a warp's
    // operations in the order they are issued:
    //   S(0) S(1) | O(u) S(u+2) | ...
    // so the scores of the next half are there before the softmax of this half ends, and S(u+2) lands where P(u)
    // lay only after O(u) has read it.  While one warp checks its barriers the other's products keep the pipe full.
    const int x = warp - 1;
    const int n_mine = x ? n_x[1] : n_x[0];
    bool ok = n_mine > 0 && tc_mbar_wait(&bars.q_full, 0, abort_flag, err, 12);
    const uint32_t q_addr = tc_smem_u32(Qs) + x * TILE_BYTES, k_addr = tc_smem_u32(Ks), v_addr = tc_smem_u32(Vs);
    const uint32_t tb = tmem + x * COLS_PER_TILE;
    auto issue_qk = [&](int u) {
      // S[u & 1] = Q K^T for 64 keys: 8 steps of 16 along the head size, 4 per 64-column half of Q and K; then the
      // tile of keys is released if this was its last half
      const int st = (u >> 1) & 1;
      if (tc_elect_one()) {
        const uint64_t qd = desc_k_major(q_addr), kd = desc_k_major(k_addr + st * TILE_BYTES + (u & 1) * (SUB * 128));
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;       // descriptor addresses count 16 bytes
          tc_mma_ss(tb + COL_S + (u & 1) * SUB, qd + off, kd + off, IDESC_S, ks != 0);
        }
        tc_commit(&bars.s_full[x][u & 1]);
        if ((u & 1) || u == n_mine - 1) tc_commit(&bars.k_empty[x][st]);
      }
      __syncwarp();
    };
    auto wait_k = [&](int u) {                               // half u opens a new tile of keys
      if (!(u & 1)) {
        ok = ok && tc_mbar_wait(&bars.k_full[(u >> 1) & 1], (u >> 2) & 1, abort_flag, err, 13);
        tc_fence_after();
      }
    };
    if (ok) { wait_k(0); if (ok) issue_qk(0); }
    if (ok && n_mine > 1) issue_qk(1);
    for (int u = 0; u < n_mine && ok; ++u) {
      const int st = (u >> 1) & 1;
      if (!(u & 1)) ok = tc_mbar_wait(&bars.v_full[st], (u >> 2) & 1, abort_flag, err, 18);
      ok = ok && tc_mbar_wait(&bars.p_ready[x][u & 1], (u >> 1) & 1, abort_flag, err, 14);
      if (!ok) break;
      tc_fence_after();
      // O += P(u) V: 4 steps of 16 keys; P at 8 columns (16 bfloat16) per step, V 2048 bytes (16 key rows) per step
      if (tc_elect_one()) {
        const uint64_t vd = desc_mn_major(v_addr + st * TILE_BYTES + (u & 1) * (SUB * 128));
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          tc_mma_ts(tb + COL_O, tb + COL_S + (u & 1) * SUB + ks * 8, vd + ks * (2048 >> 4), IDESC_PV, (u | ks) != 0);
        tc_commit(&bars.o_done[x]);
        if ((u & 1) || u == n_mine - 1) tc_commit(&bars.v_empty[x][st]);
      }
      __syncwarp();
      if (u + 2 < n_mine) {
        wait_k(u + 2);
        if (!ok) break;
        issue_qk(u + 2);
      }
    }
  } else if (warp >= 4) {
    // ---------------- softmax: warps 4-7 take query tile 0, warps 8-11 query tile 1; one thread per row
    const int x = (warp - 4) >> 2;
    const int qd = warp & 3;                                 // this warp's quarter of the 128 lanes
    const int row = qd * 32 + lane;
    const int t0x = tok0[x], t1x = min(q_len, t0x + tpt);
    const int tok = t0x + row / G;
    const int p = tok < t1x ? p_first + tok : NO_ROW;
    const int row_lo = window > 0 ? p - window + 1 : 0;
    const int lox = window > 0 ? max(0, p_first + t0x - window + 1) : 0, hix = p_first + t1x - 1;
    const uint32_t lane_addr = tmem + ((uint32_t)(qd * 32) << 16) + x * COLS_PER_TILE;
    uint64_t* o_done = &bars.o_done[x];
    const int n_mine = x ? n_x[1] : n_x[0];
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int u = 0; u < n_mine && ok; ++u) {
      const int h = u & 1;
      ok = __all_sync(0xffffffffu, tc_mbar_wait(&bars.s_full[x][h], (u >> 1) & 1, abort_flag, err, 15)) != 0;    // warp-uniform
      if (!ok) break;
      tc_fence_after();
      const int key0 = T0 + u * SUB;
      const uint32_t s_addr = lane_addr + COL_S + h * SUB;
      // a half every key of which every row of the query tile sees needs no masking (rows past the request's tokens
      // are computed like the others and never stored)
      const bool interior = key0 >= lox && key0 + SUB - 1 <= min(hix, p_first + t0x) && (window == 0 || key0 >= hix - window + 1);
      // the row's 64 scores into registers with one wait
      uint32_t v[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) tc_ld32(s_addr + c * 32, v[c]);
      tc_wait_ld();
      // the row's maximum over the visible keys, four chains
      float mxc[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (interior) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; i += 2)                        // the three-input maximum: half the instructions
            mxc[(c << 1) | ((i >> 1) & 1)] = tc_max3(mxc[(c << 1) | ((i >> 1) & 1)], __uint_as_float(v[c][i]), __uint_as_float(v[c][i + 1]));
      } else {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + c * 32 + i;
            const bool vis = key <= p && key >= row_lo && key >= lox && key <= hix;
            if (vis) mxc[(c << 1) | (i & 1)] = fmaxf(mxc[(c << 1) | (i & 1)], __uint_as_float(v[c][i]));
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
        ok = __all_sync(0xffffffffu, tc_mbar_wait(o_done, (u - 1) & 1, abort_flag, err, 16)) != 0;
        if (!ok) break;
        o_waited = true;
        tc_fence_after();
        l *= factor;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t o[16];
          tc_ld16(lane_addr + COL_O + c * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
          tc_st16(lane_addr + COL_O + c * 16, o);
        }
      }
      // p = 2^(s - ref), the row sum, and P as bfloat16 pairs over the first 32 columns of this score buffer (its
      // scores are all in registers by now)
      float lc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[16];
        if (interior) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float e0 = tc_exp2(fmaf(__uint_as_float(v[c][i]), scale_log2, -ref));
            const float e1 = tc_exp2(fmaf(__uint_as_float(v[c][i + 1]), scale_log2, -ref));
            lc[i & 2] += e0; lc[(i & 2) + 1] += e1;
            pk[i >> 1] = tc_pack(e0, e1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int key = key0 + c * 32 + i;
            const bool v0 = key <= p && key >= row_lo && key >= lox && key <= hix;
            const bool v1 = key + 1 <= p && key + 1 >= row_lo && key + 1 >= lox && key + 1 <= hix;
            const float e0 = v0 ? tc_exp2(fmaf(__uint_as_float(v[c][i]), scale_log2, -ref)) : 0.f;
            const float e1 = v1 ? tc_exp2(fmaf(__uint_as_float(v[c][i + 1]), scale_log2, -ref)) : 0.f;
            lc[i & 2] += e0; lc[(i & 2) + 1] += e1;
            pk[i >> 1] = tc_pack(e0, e1);
          }
        }
        tc_st16(s_addr + c * 16, pk);
      }
      l += (lc[0] + lc[1]) + (lc[2] + lc[3]);
      tc_wait_st();
      tc_fence_before();
      // A wait by parity tells phase k of o_done from phase k - 2 only for a waiter that has seen phase k - 1.  Half u's
      // scores imply that P V of half u - 2 has landed (the tensor core runs one warp's operations in order) but say
      // nothing of half u - 1, so every step waits for it (by now it has almost always landed) before it hands over P:
      // the step that skipped it when no row's maximum grew would leave the wait after the last half one phase short,
      // and that wait would pass on the phase two back while P V was still in flight.
      if (u > 0 && !o_waited) {
        ok = __all_sync(0xffffffffu, tc_mbar_wait(o_done, (u - 1) & 1, abort_flag, err, 19)) != 0;
        if (!ok) break;
      }
      tc_mbar_arrive(&bars.p_ready[x][h]);
    }
    if (ok && n_mine > 0) {
      ok = __all_sync(0xffffffffu, tc_mbar_wait(o_done, (n_mine - 1) & 1, abort_flag, err, 17)) != 0;
      if (ok) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        bf16* dst = p != NO_ROW ? out + ((size_t)(q0 + tok) * nq + kvh * G + row % G) * D : nullptr;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tc_ld32(lane_addr + COL_O + c * 32, o);
          tc_wait_ld();
          if (dst) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 pk;
              pk.x = tc_pack(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
              pk.y = tc_pack(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
              pk.z = tc_pack(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
              pk.w = tc_pack(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + i) = pk;
            }
          }
        }
      }
    } else if (n_mine == 0 && p != NO_ROW) {
      bf16* dst = out + ((size_t)(q0 + tok) * nq + kvh * G + row % G) * D;
      for (int i = 0; i < D; ++i) dst[i] = __float2bfloat16_rn(0.f);
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
  if (rows >= 0x7fffffffLL || n_req > 65535 || nkv > 65535) return IFB_ERR_SIZE;
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
  const int tpc = 2 * (ROWS / G);                            // tokens per CTA: two query tiles
  dim3 grid((max_q_len + tpc - 1) / tpc, nkv, n_req);
  return ifb_launch(attn_tile_tc_kernel, grid, dim3(TC_THREADS), (size_t)SMEM_BYTES, stream, q_map, kv_map, (int)rows, err, block_tables,
                    bt_stride, cu_q, seq_lens, (bf16*)out, nq, nkv, page_size, scale * 1.4426950408889634f, window);
}
