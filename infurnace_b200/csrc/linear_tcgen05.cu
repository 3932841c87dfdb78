// Matrix product for many rows (prompts): out[n, o] = sum_k x[n, k] w[o, k], bfloat16 operands,
// float32 accumulation, on the fifth-generation tensor cores: tcgen05.mma issued by one thread, operands
// brought to shared memory by TMA (128-byte swizzle), the accumulator in tensor memory, read back with
// tcgen05.ld for the epilogue.
//
// A CTA of 320 threads takes one output tile:
//   warp 0: TMA producer.  Per 64-wide k block it waits for a free stage, arms the stage's "full" barrier with
//           the byte count and issues the loads of the x tile and the w tile(s).
//   warp 1: MMA issuer.  It waits for "full", issues the k=16 MMAs of the stage and commits them to the stage's
//           "empty" barrier, so the stage is reused as soon as the tensor core has read it.  After the last
//           k block it commits to the "accumulator ready" barrier.  Warp 1 also owns the tensor memory.
//   warps 2-9: epilogue.  A warp reads its quarter (warp index mod 4) of the accumulator's 128 lanes, one token per
//           thread and half; warps 2-5 take the first half of the tile's features and warps 6-9 the second.
// In warps 0 and 1 all lanes wait and one elected lane issues.
// Rows, features or k beyond the matrices are zero-filled by TMA and dropped at the store.
//
// Tile shapes (GemmCfg): MH halves of 128 tokens share the w tile of a stage; each half accumulates NACC
// columns in tensor memory with one MMA of N = NACC per k step.
//   narrow  MH 1, NACC 128: 128 tokens x 128 features, 3 stages of 32 KB, two CTAs per SM;
//   deep    the same with 6 stages, for grids of at most one CTA per SM (o and down projections of prompts of
//           a few thousand tokens): the stages in flight are what hides the latency of the loads;
//   wide    MH 2, NACC 256: 256 tokens x 256 features, 3 stages of 64 KB, all 512 columns of tensor memory:
//           half the bytes from L2 per product of the narrow shape.
// Epilogue 1 (silu_gate): w holds gate rows [0, O) and up rows [O, 2O).  A stage carries a gate tile and an up
// tile back to back as one B operand, the accumulator's first NACC/2 columns are gate and the rest up, and
// out = silu(gate) * up has NACC/2 features per CTA (narrow: NACC 256).
//
// Every wait on a barrier is bounded: after G_SPIN_LIMIT polls the thread writes a code to `*err`, raises
// the CTA's abort flag, and everything falls through to the common exit, which frees the tensor memory.
#include <cuda.h>
#include "common.cuh"

typedef __nv_bfloat16 bf16;
constexpr int G_BM = 128;          // tokens per half tile (MMA M)
constexpr int G_BK = 64;           // k per stage: 128 bytes, one swizzle row
constexpr int G_UK = 16;           // k per MMA
constexpr int G_THREADS = 320;      // producer warp, MMA warp, eight epilogue warps
constexpr uint32_t G_SPIN_LIMIT = 1u << 22;
constexpr int G_TILE_BYTES = G_BM * G_BK * 2;   // 16 KB: 128 rows of one k block

template <int EPI_, int MH_, int NACC_, int STAGES_> struct GemmCfg {
  static constexpr int EPI = EPI_, MH = MH_, NACC = NACC_, STAGES = STAGES_;
  static constexpr int FO = EPI ? NACC / 2 : NACC;            // output features per CTA
  static constexpr int A_BYTES = MH * G_TILE_BYTES;           // x rows of a stage
  static constexpr int B_BYTES = NACC * G_BK * 2;             // w rows of a stage
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = MH * NACC;                 // 128, 256 or 512 columns of 32 bits
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */;
  // float32 accumulator, bfloat16 a and b, both K-major, M = 128, N = NACC
  static constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NACC >> 3) << 17) | ((uint32_t)(G_BM >> 4) << 24);
};

__device__ __forceinline__ uint32_t g_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(g_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(g_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(g_smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  False: gave up (the abort flag is up and *err says where).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
  unsigned long long t0 = 0;
  for (uint32_t i = 0; i < G_SPIN_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (ifb_wait_expired(i, t0)) break;
  }
  *abort_flag = 1;
  atomicExch(err, code);
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(g_smem_u32(smem)), "l"(map), "r"(g_smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, int cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(g_smem_u32(slot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, int cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols) : "memory");
}
// True in exactly one lane of a converged warp.  Code under it is known to the compiler as single-threaded, which lets
// it keep the descriptors of the copies and products it issues in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(g_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// All threads of all CTAs of the cluster: arrive (release) and wait (acquire).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Four floats at this CTA's shared address `addr`, read from the CTA of rank `rank` in the cluster.
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr, int rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(addr), "r"(rank));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}

// Shared-memory matrix descriptor of a K-major tile in the 128-byte swizzle: rows of 128 bytes, groups of 8
// rows 1024 bytes apart (stride byte offset), leading byte offset unused (1), descriptor version 1.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// A normalisation folded into the products around it (RMSNorm(v) = v * g * r with one r per row): the product that
// makes v (plain epilogue) adds the residual stream, writes v back to it, writes v * g as its output and leaves sums of
// v^2 over slices of the features; the product that reads v * g multiplies its rows by r, from those sums added in a
// fixed order, before its own epilogue.  No kernel runs for the norm itself.
struct TcFold {
  const float* rs_partials;   // reading side: [rs_parts][n_rows] sums of squares (null: rows are not scaled)
  int rs_parts;
  float rs_eps, rs_inv_width; // r = rsqrt(sum * inv_width + eps)
  float* res_x;               // making side: [n_rows][o_out] float32 residual stream, v = x + y in place (null: plain)
  const void* res_g;          // [o_out] norm weight
  int res_g_dtype;
  float* res_partials;        // [parts][n_rows], written; what a part covers depends on the launch (tc_fold_parts)
  // The product is the fused q | k | v projection of an attention layer with heads of 128, in the shared-k form, whose
  // tile of 128 features is one head: the sum over the cluster finishes what follows the projection (RMSNorm over the q
  // and k heads, rotation in the half-split pairing, q to its row, k and v to the token's place in the pages).
  int qk_nq, qk_nkv;          // qk_nq > 0: on
  const void* qk_qw;          // [128] norm weights (null: no norm)
  const void* qk_kw;
  int qk_w_dtype;
  float qk_eps;
  const float2* qk_rope;      // [n_rows][64] (cos, sin) of each token's angles (null: no rotation)
  const int* qk_slots;        // [n_rows] page * page_size + offset, negative: store nothing (null: no store)
  bf16* qk_pages;             // [page][k | v][kv head][offset][128]
  int qk_page_size;
};
__device__ __forceinline__ float tc_row_factor(const TcFold& f, int row, int n_rows) {
  if (!f.rs_partials || row >= n_rows) return 1.f;
  float sum = 0.f;
#pragma unroll 4
  for (int p = 0; p < f.rs_parts; ++p) sum += __ldg(f.rs_partials + (size_t)p * n_rows + row);
  return rsqrtf(sum * f.rs_inv_width + f.rs_eps);
}
// v = x + y for 32 consecutive features of one row (x updated in place), y <- v * g; returns the sum of v^2.
__device__ __forceinline__ float tc_residual_chunk(const TcFold& f, float (&y)[32], int row, int n_rows, int col0, int o_out) {
  float ss = 0.f;
  if (row >= n_rows) return 0.f;
  float* xr = f.res_x + (size_t)row * o_out + col0;
  if (col0 + 32 <= o_out && (o_out & 3) == 0) {
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      float4 xv = *reinterpret_cast<float4*>(xr + j);
      xv.x += y[j]; xv.y += y[j + 1]; xv.z += y[j + 2]; xv.w += y[j + 3];
      *reinterpret_cast<float4*>(xr + j) = xv;
      ss += xv.x * xv.x + xv.y * xv.y + xv.z * xv.z + xv.w * xv.w;
      y[j] = xv.x * load_as_f32(f.res_g, f.res_g_dtype, col0 + j);
      y[j + 1] = xv.y * load_as_f32(f.res_g, f.res_g_dtype, col0 + j + 1);
      y[j + 2] = xv.z * load_as_f32(f.res_g, f.res_g_dtype, col0 + j + 2);
      y[j + 3] = xv.w * load_as_f32(f.res_g, f.res_g_dtype, col0 + j + 3);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < o_out) {
        const float v = xr[j] + y[j];
        xr[j] = v;
        ss += v * v;
        y[j] = v * load_as_f32(f.res_g, f.res_g_dtype, col0 + j);
      }
  }
  return ss;
}

template <typename Cfg, typename TO>
__global__ void __launch_bounds__(G_THREADS)
linear_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                      TO* __restrict__ out, int n_rows, int o_out, int k_dim, int* __restrict__ err,
                      int splits, TcFold fold) {
  constexpr int EPI = Cfg::EPI, MH = Cfg::MH, NACC = Cfg::NACC, FO = Cfg::FO;
  extern __shared__ unsigned char g_smem_raw[];
  const uint32_t raw = g_smem_u32(g_smem_raw);
  unsigned char* smem = g_smem_raw + (((raw + 1023u) & ~1023u) - raw);      // tiles need 1024-byte alignment
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty = full + Cfg::STAGES;
  uint64_t* accum = empty + Cfg::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;     // warp-uniform
  const int m0 = blockIdx.y * (MH * G_BM), n0 = blockIdx.x * FO;
  // With splits > 1 (plain epilogue, one 128-row tile per CTA) the CTAs of a tile are a cluster along z: CTA z
  // multiplies the z-th part of the k range, leaves its float32 tile in its shared memory, and after a cluster barrier
  // adds, in the order of z, a slice of the tile's rows over all CTAs' copies and stores it.
  const int kb_all = (k_dim + G_BK - 1) / G_BK;
  const int kb_per = (kb_all + splits - 1) / splits;
  const int kb0 = blockIdx.z * kb_per;
  const int kblocks = max(0, min(kb_all, kb0 + kb_per) - kb0);    // this CTA's k blocks are kb0 .. kb0 + kblocks - 1
  constexpr int RED_PITCH = NACC + 4;                             // floats per row of the tile left in shared memory

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(accum, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // The first fill of the stages: the w tiles, which no kernel of the step writes, are requested before this kernel
    // waits for its predecessor in the stream; the x tiles after.  (The other warps act only on what these loads
    // bring, so the wait of this warp orders the whole CTA behind the predecessor.)
    const int first = min(kblocks, Cfg::STAGES);
    if (elect_one()) {
      for (int kb = 0; kb < first; ++kb) {
        unsigned char* stage = smem + kb * Cfg::STAGE_BYTES;
        mbar_expect_tx(&full[kb], Cfg::STAGE_BYTES);
        tma_load_2d(stage + Cfg::A_BYTES, &tmap_w, &full[kb], (kb0 + kb) * G_BK, n0);       // FO rows of w
        if (EPI) tma_load_2d(stage + Cfg::A_BYTES + Cfg::B_BYTES / 2, &tmap_w, &full[kb], (kb0 + kb) * G_BK, o_out + n0);
      }
    }
    __syncwarp();
    ifb_pdl_wait();
    ifb_pdl_trigger();
    if (elect_one()) {
      for (int kb = 0; kb < first; ++kb)
        tma_load_2d(smem + kb * Cfg::STAGE_BYTES, &tmap_x, &full[kb], (kb0 + kb) * G_BK, m0);   // MH * 128 rows of x
    }
    __syncwarp();
    for (int kb = first; kb < kblocks; ++kb) {
      const int s = kb % Cfg::STAGES;
      const uint32_t ph = (kb / Cfg::STAGES) & 1;
      if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, err, 1)) break;
      if (elect_one()) {
        unsigned char* stage = smem + s * Cfg::STAGE_BYTES;
        mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
        tma_load_2d(stage, &tmap_x, &full[s], (kb0 + kb) * G_BK, m0);
        tma_load_2d(stage + Cfg::A_BYTES, &tmap_w, &full[s], (kb0 + kb) * G_BK, n0);
        if (EPI) tma_load_2d(stage + Cfg::A_BYTES + Cfg::B_BYTES / 2, &tmap_w, &full[s], (kb0 + kb) * G_BK, o_out + n0);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    bool ok = true;
    for (int kb = 0; kb < kblocks && ok; ++kb) {
      const int s = kb % Cfg::STAGES;
      const uint32_t ph = (kb / Cfg::STAGES) & 1;
      ok = mbar_wait(&full[s], ph, abort_flag, err, 2);
      if (!ok) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t a_addr = g_smem_u32(smem + s * Cfg::STAGE_BYTES);
        const uint64_t a_desc = make_smem_desc(a_addr);
        const uint64_t b_desc = make_smem_desc(a_addr + Cfg::A_BYTES);
#pragma unroll
        for (int k = 0; k < G_BK / G_UK; ++k) {
          const uint64_t step = (uint64_t)((k * G_UK * 2) >> 4);          // 32 bytes per k step, in 16-byte units
          const uint32_t acc = (kb | k) != 0;
#pragma unroll
          for (int hf = 0; hf < MH; ++hf)
            umma_bf16(tmem_base + hf * NACC, a_desc + (uint64_t)((hf * G_TILE_BYTES) >> 4) + step, b_desc + step, Cfg::IDESC, acc);
        }
        umma_commit(&empty[s]);
        if (kb == kblocks - 1) umma_commit(accum);
      }
      __syncwarp();
    }
  } else {
    // A warp's piece of the tile is 32 tokens (its lanes) by CW features.  A lane holds a token's row, so storing
    // from registers would send the 32 lanes of a store to 32 different rows of `out`; the piece goes through shared
    // memory instead (the stages, all consumed by now) and leaves in whole row segments, 512 bytes per store.
    constexpr int CW = FO / 2;
    // staged PW features at a time: all of the piece if eight warps' rows fit in the stages, else half of it
    constexpr int PW = 8 * 32 * (CW * (int)sizeof(TO) + 16) <= Cfg::STAGES * Cfg::STAGE_BYTES ? CW : CW / 2;
    constexpr int ROWB = PW * (int)sizeof(TO);                   // bytes of a row segment
    constexpr int PITCH = ROWB + 16;                             // an odd number of 16-byte units: no bank conflicts
    static_assert(8 * 32 * PITCH <= Cfg::STAGES * Cfg::STAGE_BYTES, "the staging rows must fit in the stages");
    const int q = warp & 3;                                      // this warp's quarter of the 128 lanes
    const int c_lo = ((warp - 2) >> 2) * CW;                     // and its half of the tile's features
    if (kblocks > 0 && mbar_wait(accum, 0, abort_flag, err, 3)) {
      tc_fence_after();
      if (fold.rs_partials || fold.res_x) ifb_pdl_wait();         // what the predecessor wrote is read here directly
      const bool vec = ((size_t)o_out * sizeof(TO)) % 16 == 0 && (((uintptr_t)out) & 15) == 0 && n0 + c_lo + CW <= o_out;
      unsigned char* buf = smem + (warp - 2) * (32 * PITCH);
#pragma unroll 1
      for (int hf = 0; hf < MH; ++hf) {
        const int row0 = m0 + hf * G_BM + q * 32;
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16) + hf * NACC;
        const float rfac = tc_row_factor(fold, row0 + lane, n_rows);
        float ss = 0.f;                                          // this row's v^2 over this warp's features
#pragma unroll 1
       for (int p0 = c_lo; p0 < c_lo + CW; p0 += PW) {
#pragma unroll 1
        for (int c0 = p0; c0 < p0 + PW; c0 += 32) {
          if (n0 + c0 >= o_out) break;                           // warp-uniform
          uint32_t v[32];
          float y[32];
          tmem_ld32(lane_base + c0, v);
          if (splits > 1) {
            // the part stays here for the cluster's sum (with the silu_gate epilogue: the gate columns, then the up
            // columns FO further on; the epilogue itself comes after the sum)
            float* dst = reinterpret_cast<float*>(smem) + (size_t)(hf * G_BM + q * 32 + lane) * RED_PITCH + c0;
            uint32_t u[32];
            if (EPI) tmem_ld32(lane_base + FO + c0, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(v[j]) * rfac, __uint_as_float(v[j + 1]) * rfac,
                                                                __uint_as_float(v[j + 2]) * rfac, __uint_as_float(v[j + 3]) * rfac);
            if (EPI) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(dst + FO + j) = make_float4(__uint_as_float(u[j]) * rfac, __uint_as_float(u[j + 1]) * rfac,
                                                                       __uint_as_float(u[j + 2]) * rfac, __uint_as_float(u[j + 3]) * rfac);
            }
            continue;
          }
          if (EPI) {
            uint32_t u[32];
            tmem_ld32(lane_base + FO + c0, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              // silu(g) * u with the hardware's exp2 and reciprocal (relative error about 1e-6; the result is
              // rounded to the output type)
              const float g = __uint_as_float(v[j]) * rfac;
              y[j] = g * fast_rcp(1.f + fast_exp2(-1.4426950408889634f * g)) * (__uint_as_float(u[j]) * rfac);
            }
          } else {
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) y[j] = __uint_as_float(v[j]) * rfac;
          }
          if (!EPI && fold.res_x) ss += tc_residual_chunk(fold, y, row0 + lane, n_rows, n0 + c0, o_out);
          if (vec) {
            unsigned char* dst = buf + lane * PITCH + (c0 - p0) * (int)sizeof(TO);
            if (sizeof(TO) == 2) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 pk;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(y[j], y[j + 1]), p1 = __floats2bfloat162_rn(y[j + 2], y[j + 3]);
                __nv_bfloat162 p2 = __floats2bfloat162_rn(y[j + 4], y[j + 5]), p3 = __floats2bfloat162_rn(y[j + 6], y[j + 7]);
                pk.x = *reinterpret_cast<uint32_t*>(&p0); pk.y = *reinterpret_cast<uint32_t*>(&p1);
                pk.z = *reinterpret_cast<uint32_t*>(&p2); pk.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(dst + j * 2) = pk;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(dst + j * 4) = make_float4(y[j], y[j + 1], y[j + 2], y[j + 3]);
            }
          } else if (row0 + lane < n_rows) {
            TO* dst = out + (size_t)(row0 + lane) * o_out + n0 + c0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + c0 + j < o_out) dst[j] = from_f32<TO>(y[j]);
          }
        }
        if (vec && splits == 1) {
          __syncwarp();
          unsigned char* obase = reinterpret_cast<unsigned char*>(out + (size_t)row0 * o_out + n0 + p0);
#pragma unroll 4
          for (int off = lane * 16; off < 32 * ROWB; off += 512) {
            const int r = off / ROWB, cb = off % ROWB;
            if (row0 + r < n_rows)
              *reinterpret_cast<uint4*>(obase + (size_t)r * o_out * sizeof(TO) + cb) = *reinterpret_cast<const uint4*>(buf + r * PITCH + cb);
          }
          __syncwarp();                                          // before the next rows overwrite the buffer
        }
       }
       if (!EPI && splits == 1 && fold.res_x && row0 + lane < n_rows)
         fold.res_partials[(size_t)(blockIdx.x * 2 + (c_lo ? 1 : 0)) * n_rows + row0 + lane] = ss;
      }
    }
  }
  if (splits > 1) {
    cluster_sync_all();                        // every CTA's part is in its shared memory
    if (fold.res_x || fold.qk_nq) ifb_pdl_wait();
    const int rows = min(G_BM, n_rows - m0), cols = min(FO, o_out - n0);
    const int used = (kb_all + kb_per - 1) / kb_per;                       // CTAs that had k blocks
    const int per = (rows + splits - 1) / splits;
    const int r_lo = blockIdx.z * per, r_hi = min(rows, r_lo + per);
    const bool vec = ((size_t)o_out * sizeof(TO)) % 16 == 0 && (((uintptr_t)out) & 15) == 0 && cols == FO;
    const uint32_t tile_addr = g_smem_u32(smem);
    for (int i = threadIdx.x; i < (r_hi - r_lo) * (FO / 4); i += G_THREADS) {
      const int r = r_lo + i / (FO / 4), c = (i % (FO / 4)) * 4;
      const uint32_t at = tile_addr + (uint32_t)((r * RED_PITCH + c) * 4);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int z = 0; z < used; ++z) {
        const float4 v = ld_cluster_f4(at, z);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      if (EPI) {
        float4 up = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int z = 0; z < used; ++z) {
          const float4 v = ld_cluster_f4(at + FO * 4, z);
          up.x += v.x; up.y += v.y; up.z += v.z; up.w += v.w;
        }
        acc.x = acc.x * fast_rcp(1.f + fast_exp2(-1.4426950408889634f * acc.x)) * up.x;
        acc.y = acc.y * fast_rcp(1.f + fast_exp2(-1.4426950408889634f * acc.y)) * up.y;
        acc.z = acc.z * fast_rcp(1.f + fast_exp2(-1.4426950408889634f * acc.z)) * up.z;
        acc.w = acc.w * fast_rcp(1.f + fast_exp2(-1.4426950408889634f * acc.w)) * up.w;
      }
      TO* dst = out + (size_t)(m0 + r) * o_out + n0 + c;
      if (!EPI && fold.res_x) {
        // a warp holds one row of the tile: v = x + y, x <- v, the output becomes v * g, the warp's sum of v^2 one part
        float* xr = fold.res_x + (size_t)(m0 + r) * o_out + n0 + c;
        float yv[4] = {acc.x, acc.y, acc.z, acc.w}, ss = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (c + j < cols) {
            const float v = xr[j] + yv[j];
            xr[j] = v;
            ss += v * v;
            yv[j] = v * load_as_f32(fold.res_g, fold.res_g_dtype, n0 + c + j);
          }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
        if ((threadIdx.x & 31) == 0) fold.res_partials[(size_t)blockIdx.x * n_rows + m0 + r] = ss;
        acc = make_float4(yv[0], yv[1], yv[2], yv[3]);
      }
      if (!EPI && sizeof(TO) == 2 && fold.qk_nq) {
        // a warp holds one head of one token (lane l its elements 4l .. 4l + 3; the rotation partner 16 lanes on)
        const int head = blockIdx.x, ln = threadIdx.x & 31;
        const bool is_v = head >= fold.qk_nq + fold.qk_nkv, is_k = head >= fold.qk_nq && !is_v;
        float yv[4] = {acc.x, acc.y, acc.z, acc.w};
        const void* wn = is_k ? fold.qk_kw : fold.qk_qw;
        if (!is_v && wn) {
          float ss = yv[0] * yv[0] + yv[1] * yv[1] + yv[2] * yv[2] + yv[3] * yv[3];
#pragma unroll
          for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
          const float rn = rsqrtf(ss * (1.f / 128.f) + fold.qk_eps);
#pragma unroll
          for (int j = 0; j < 4; ++j) yv[j] = yv[j] * rn * load_as_f32(wn, fold.qk_w_dtype, c + j);
        }
        if (!is_v && fold.qk_rope) {
          const float2* t = fold.qk_rope + (size_t)(m0 + r) * 64 + (c & 63);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float o = __shfl_xor_sync(0xffffffffu, yv[j], 16);
            const float2 cs = t[j];
            yv[j] = ln < 16 ? yv[j] * cs.x - o * cs.y : yv[j] * cs.x + o * cs.y;
          }
        }
        __nv_bfloat162 lo = __floats2bfloat162_rn(yv[0], yv[1]), hi = __floats2bfloat162_rn(yv[2], yv[3]);
        const uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        *reinterpret_cast<uint2*>(dst) = pk;
        if (head >= fold.qk_nq && fold.qk_slots) {
          const int slot = fold.qk_slots[m0 + r];
          if (slot >= 0) {
            const int kvh = is_v ? head - fold.qk_nq - fold.qk_nkv : head - fold.qk_nq;
            const size_t row = ((size_t)(slot / fold.qk_page_size) * 2 + (is_v ? 1 : 0)) * fold.qk_nkv + kvh;
            *reinterpret_cast<uint2*>(fold.qk_pages + (row * fold.qk_page_size + slot % fold.qk_page_size) * 128 + c) = pk;
          }
        }
        continue;
      }
      if (vec) {
        if (sizeof(TO) == 4) {
          *reinterpret_cast<float4*>(dst) = acc;
        } else {
          __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
          *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
      } else {
        const float y[4] = {acc.x, acc.y, acc.z, acc.w};
        for (int j = 0; j < 4; ++j)
          if (c + j < cols) dst[j] = from_f32<TO>(y[j]);
      }
    }
    cluster_sync_all();                        // nobody leaves while its shared memory is being read
  }
  if (*abort_flag) {                         // a wait gave up: let copies in flight land before the CTA goes away
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, Cfg::TMEM_COLS); }
}


// ---------------------------------------------------------------------------------------------------
// A [rows, k] bfloat16 row-major matrix as a tensor map with boxes of 64 k x box_rows rows, 128-byte swizzle.
static int make_map(CUtensorMap* m, const void* ptr, int rows, int k, int box_rows) {
  const unsigned long long dims[2] = {(unsigned long long)k, (unsigned long long)rows};
  const unsigned long long strides[1] = {(unsigned long long)k * 2};
  const unsigned box[2] = {(unsigned)G_BK, (unsigned)box_rows};
  return ifb_tensor_map_bf16(m, ptr, 2, dims, strides, box);
}

// ---------------------------------------------------------------------------------------------------
// The persistent form.  A CTA per SM walks a list of output tiles (tile t of the list goes to CTA t mod grid), with two
// accumulators in tensor memory: while the epilogue warps read and store tile i from one, the issuer already
// multiplies tile i + 1 into the other, and the producer's ring of stages never drains between tiles.  Tiles are
// 128 tokens x NACC accumulator columns (128 or 256; with the silu_gate epilogue 128 gate + 128 up columns give 128
// features); consecutive tiles of the list share their w tile, so it is read from L2 by the CTAs of one round.
// The epilogue has its own staging rows in shared memory (the stages are busy with the next tile).
// ---------------------------------------------------------------------------------------------------
template <int EPI_, int NACC_, int STAGES_> struct PersistCfg {
  static constexpr int EPI = EPI_, NACC = NACC_, STAGES = STAGES_;
  static constexpr int FO = EPI ? NACC / 2 : NACC;            // output features per tile
  static constexpr int A_BYTES = G_TILE_BYTES;                // 128 x rows of a stage
  static constexpr int B_BYTES = NACC * G_BK * 2;             // w rows of a stage
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 2 * NACC;                  // two accumulators: 256 or 512 columns
  static constexpr int STAGING_PITCH = 128 + 16;              // a row segment of 128 bytes, padded against bank conflicts
  static constexpr int STAGING_BYTES = 8 * 32 * STAGING_PITCH;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 /* alignment */ + 256 /* barriers */;
  static constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NACC >> 3) << 17) | ((uint32_t)(G_BM >> 4) << 24);
};

template <typename Cfg, typename TO>
__global__ void __launch_bounds__(G_THREADS, 1)
linear_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                                 TO* __restrict__ out, int n_rows, int o_out, int k_dim, int tiles_m, int tiles_total,
                                 int* __restrict__ err, TcFold fold) {
  constexpr int EPI = Cfg::EPI, NACC = Cfg::NACC, FO = Cfg::FO, STAGES = Cfg::STAGES;
  extern __shared__ unsigned char g_smem_raw[];
  const uint32_t raw = g_smem_u32(g_smem_raw);
  unsigned char* smem = g_smem_raw + (((raw + 1023u) & ~1023u) - raw);      // tiles need 1024-byte alignment
  unsigned char* staging = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + Cfg::STAGING_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;                         // [2]: the issuer has finished a tile in accumulator b
  uint64_t* acc_empty = acc_full + 2;                          // [2]: the eight epilogue warps have read accumulator b
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;     // warp-uniform
  const int kblocks = (k_dim + G_BK - 1) / G_BK;
  // this CTA's tiles: first, first + gridDim.x, ...; tile t covers tokens (t % tiles_m) * 128 and features (t / tiles_m) * FO
  const int first = blockIdx.x, step = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- producer.  The w tiles of the first stages, which no kernel of the step writes, are requested before this
    // kernel waits for its predecessor in the stream; every x tile after.  (The other warps act only on what these
    // loads bring, so the wait of this warp orders the whole CTA behind the predecessor.)
    int g = 0;                                                  // k blocks issued so far, over all tiles
    bool waited = false, ok = true;
    for (int t = first; t < tiles_total && ok; t += step) {
      const int m0 = (t % tiles_m) * G_BM, n0 = (t / tiles_m) * FO;
      for (int kb = 0; kb < kblocks; ++kb, ++g) {
        const int s = g % STAGES;
        if (g >= STAGES && !mbar_wait(&empty[s], ((g / STAGES) - 1) & 1, abort_flag, err, 1)) { ok = false; break; }
        unsigned char* stage = smem + s * Cfg::STAGE_BYTES;
        if (elect_one()) {
          mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
          tma_load_2d(stage + Cfg::A_BYTES, &tmap_w, &full[s], kb * G_BK, n0);
          if (EPI) tma_load_2d(stage + Cfg::A_BYTES + Cfg::B_BYTES / 2, &tmap_w, &full[s], kb * G_BK, o_out + n0);
        }
        __syncwarp();
        if (!waited && (g == STAGES - 1 || (kb == kblocks - 1 && t + step >= tiles_total))) {
          // the ring is full of w tiles (or there are no more): now the predecessor, then the x tiles held back
          ifb_pdl_wait();
          ifb_pdl_trigger();
          waited = true;
          if (elect_one()) {
            int gg = 0;
            for (int tt = first; tt < tiles_total && gg <= g; tt += step)
              for (int kk = 0; kk < kblocks && gg <= g; ++kk, ++gg)
                tma_load_2d(smem + (gg % STAGES) * Cfg::STAGE_BYTES, &tmap_x, &full[gg % STAGES], kk * G_BK, (tt % tiles_m) * G_BM);
          }
          __syncwarp();
        } else if (waited) {
          if (elect_one()) tma_load_2d(stage, &tmap_x, &full[s], kb * G_BK, m0);
          __syncwarp();
        }
      }
    }
    if (!waited) { ifb_pdl_wait(); ifb_pdl_trigger(); }         // a CTA without tiles still orders itself behind the predecessor
  } else if (warp == 1) {
    // ---- issuer: tile i of this CTA accumulates in accumulator i & 1
    int g = 0, it = 0;
    bool ok = true;
    for (int t = first; t < tiles_total && ok; t += step, ++it) {
      const int b = it & 1;
      if (it >= 2) ok = mbar_wait(&acc_empty[b], ((it >> 1) - 1) & 1, abort_flag, err, 4);
      if (!ok) break;
      tc_fence_after();
      for (int kb = 0; kb < kblocks && ok; ++kb, ++g) {
        const int s = g % STAGES;
        ok = mbar_wait(&full[s], (g / STAGES) & 1, abort_flag, err, 2);
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          const uint32_t a_addr = g_smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint64_t a_desc = make_smem_desc(a_addr);
          const uint64_t b_desc = make_smem_desc(a_addr + Cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < G_BK / G_UK; ++k) {
            const uint64_t kstep = (uint64_t)((k * G_UK * 2) >> 4);          // 32 bytes per k step, in 16-byte units
            umma_bf16(tmem_base + b * NACC, a_desc + kstep, b_desc + kstep, Cfg::IDESC, (kb | k) != 0);
          }
          umma_commit(&empty[s]);
          if (kb == kblocks - 1) umma_commit(&acc_full[b]);
        }
        __syncwarp();
      }
    }
  } else {
    // ---- epilogue.  A warp's piece of a tile is 32 tokens (its lanes) by CW features, taken 128 bytes of a row at a
    // time: from tensor memory to registers, to the warp's staging rows, and from there in whole row segments to `out`.
    constexpr int CW = FO / 2;
    constexpr int PW = 128 / (int)sizeof(TO);                    // features per staged row segment
    constexpr int PITCH = Cfg::STAGING_PITCH;
    static_assert(CW % PW == 0, "a warp's features are whole row segments");
    const int q = warp & 3;                                      // this warp's quarter of the 128 lanes
    const int c_lo = ((warp - 2) >> 2) * CW;                     // and its half of the tile's features
    unsigned char* buf = staging + (warp - 2) * (32 * PITCH);
    int it = 0;
    bool ok = true;
    for (int t = first; t < tiles_total && ok; t += step, ++it) {
      const int b = it & 1;
      const int m0 = (t % tiles_m) * G_BM, n0 = (t / tiles_m) * FO;
      ok = mbar_wait(&acc_full[b], (it >> 1) & 1, abort_flag, err, 3);
      if (!ok) break;
      tc_fence_after();
      const bool vec = ((size_t)o_out * sizeof(TO)) % 16 == 0 && (((uintptr_t)out) & 15) == 0 && n0 + c_lo + CW <= o_out;
      const int row0 = m0 + q * 32;
      const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16) + b * NACC;
      if (fold.rs_partials && it == 0) ifb_pdl_wait();             // the sums are the predecessor's: read them after it
      const float rfac = tc_row_factor(fold, row0 + lane, n_rows);
#pragma unroll 1
      for (int p0 = c_lo; p0 < c_lo + CW; p0 += PW) {
        if (n0 + p0 >= o_out) break;                             // warp-uniform
#pragma unroll
        for (int c0 = p0; c0 < p0 + PW; c0 += 32) {
          uint32_t v[32];
          float y[32];
          tmem_ld32(lane_base + c0, v);
          if (EPI) {
            uint32_t u[32];
            tmem_ld32(lane_base + FO + c0, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float gte = __uint_as_float(v[j]) * rfac;
              y[j] = gte * fast_rcp(1.f + fast_exp2(-1.4426950408889634f * gte)) * (__uint_as_float(u[j]) * rfac);
            }
          } else {
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) y[j] = __uint_as_float(v[j]) * rfac;
          }
          if (vec) {
            unsigned char* dst = buf + lane * PITCH + (c0 - p0) * (int)sizeof(TO);
            if (sizeof(TO) == 2) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 pk;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(y[j], y[j + 1]), h1 = __floats2bfloat162_rn(y[j + 2], y[j + 3]);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(y[j + 4], y[j + 5]), h3 = __floats2bfloat162_rn(y[j + 6], y[j + 7]);
                pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
                pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(dst + j * 2) = pk;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(dst + j * 4) = make_float4(y[j], y[j + 1], y[j + 2], y[j + 3]);
            }
          } else if (row0 + lane < n_rows) {
            TO* dst = out + (size_t)(row0 + lane) * o_out + n0 + c0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + c0 + j < o_out) dst[j] = from_f32<TO>(y[j]);
          }
        }
        if (vec) {
          __syncwarp();
          unsigned char* obase = reinterpret_cast<unsigned char*>(out + (size_t)row0 * o_out + n0 + p0);
#pragma unroll
          for (int off = lane * 16; off < 32 * 128; off += 512) {
            const int r = off >> 7, cb = off & 127;
            if (row0 + r < n_rows)
              *reinterpret_cast<uint4*>(obase + (size_t)r * o_out * sizeof(TO) + cb) = *reinterpret_cast<const uint4*>(buf + r * PITCH + cb);
          }
          __syncwarp();                                          // before the next segment overwrites the rows
        }
      }
      // this warp has read its part of accumulator b: the issuer may overwrite it (with the tile after next)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(g_smem_u32(&acc_empty[b])) : "memory");
    }
  }
  if (*abort_flag) {                         // a wait gave up: let copies in flight land before the CTA goes away
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, Cfg::TMEM_COLS); }
}

template <typename Cfg, typename TO>
static int tc_launch_persistent(const void* x, const void* w, void* out, int n, int o, int k, int* err, int sm_count, cudaStream_t s,
                                const TcFold& fold) {
  CUtensorMap mx, mw;
  int st = make_map(&mx, x, n, k, G_BM);
  if (st) return st;
  st = make_map(&mw, w, Cfg::EPI ? 2 * o : o, k, Cfg::EPI ? Cfg::NACC / 2 : Cfg::NACC);
  if (st) return st;
  IFB_ALLOW_SMEM((linear_tcgen05_persistent_kernel<Cfg, TO>), Cfg::SMEM_BYTES);
  const long long tiles_m = (n + G_BM - 1) / G_BM, tiles_n = (o + Cfg::FO - 1) / Cfg::FO;
  if (tiles_m * tiles_n > 0x7fffffffLL) return IFB_ERR_SIZE;
  const int total = (int)(tiles_m * tiles_n);
  const int grid = total < sm_count ? total : sm_count;
  return ifb_launch(linear_tcgen05_persistent_kernel<Cfg, TO>, dim3(grid), dim3(G_THREADS), (size_t)Cfg::SMEM_BYTES, s, mx, mw, (TO*)out, n,
                    o, k, (int)tiles_m, total, err, fold);
}

template <typename Cfg, typename TO>
static int tc_launch_cfg(const void* x, const void* w, void* out, int n, int o, int k, int* err, cudaStream_t s, const TcFold& fold,
                         int splits = 1) {
  CUtensorMap mx, mw;
  int st = make_map(&mx, x, n, k, Cfg::MH * G_BM);
  if (st) return st;
  st = make_map(&mw, w, Cfg::EPI ? 2 * o : o, k, Cfg::EPI ? Cfg::NACC / 2 : Cfg::NACC);
  if (st) return st;
  IFB_ALLOW_SMEM((linear_tcgen05_kernel<Cfg, TO>), Cfg::SMEM_BYTES);
  dim3 grid((o + Cfg::FO - 1) / Cfg::FO, (n + Cfg::MH * G_BM - 1) / (Cfg::MH * G_BM), splits);
  if (grid.y > 65535) return IFB_ERR_SIZE;
  if (splits == 1)
    return ifb_launch(linear_tcgen05_kernel<Cfg, TO>, grid, dim3(G_THREADS), (size_t)Cfg::SMEM_BYTES, s, mx, mw, (TO*)out, n, o, k, err, 1, fold);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(G_THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = splits;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ifb_pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, linear_tcgen05_kernel<Cfg, TO>, mx, mw, (TO*)out, n, o, k, err, splits, fold);
  if (e != cudaSuccess) { cudaGetLastError(); return -(int)e; }
  return IFB_OK;
}

// The shape of the tiles: a wave of wide tiles does four 128 x 128 products per SM in little more time than a wave of
// narrow tiles (two CTAs per SM) does two, but only if there are enough wide tiles to fill the SMs.  shape: 0 chooses
// (see below), 1 narrow, 2 deep, 3 wide, 4 and 5 persistent (for tests and measurements).
static int tc_sm_count() {
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      sm_count = 1;
  }
  return sm_count;
}
// By measurement.  With the silu_gate epilogue: the persistent kernel (its tile already accumulates 256 columns per
// product, and the heavy epilogue of one tile runs beside the products of the next).  Otherwise one tile per CTA:
// the wide shape when there are enough wide tiles to fill the SMs (a 256 x 256 tile reads half the operand bytes
// per product from shared memory, which is what bounds these kernels), else the deep or the narrow one.
static int tc_pick_shape(int epi, int n, int o) {
  if (epi) return 4;
  const int sm_count = tc_sm_count();
  const long long tn = (long long)((o + 127) / 128) * ((n + G_BM - 1) / G_BM);
  const long long tw = (long long)((o + 255) / 256) * ((n + 2 * G_BM - 1) / (2 * G_BM));
  const double cost_narrow = (double)((tn + 2 * sm_count - 1) / (2 * sm_count));
  const double cost_wide = (double)((tw + sm_count - 1) / sm_count) * 1.15;
  return (n > G_BM && cost_wide < cost_narrow) ? 3 : (tn <= sm_count ? 2 : 1);
}

template <int EPI, typename TO>
static int tc_launch(const void* x, const void* w, void* out, int n, int o, int k, int* err, int shape, int splits, const TcFold& fold,
                     cudaStream_t s) {
  using Narrow = GemmCfg<EPI, 1, EPI ? 256 : 128, EPI ? 2 : 3>;
  using Deep = GemmCfg<EPI, 1, EPI ? 256 : 128, EPI ? 4 : 6>;
  using Wide = GemmCfg<EPI, 2, 256, 3>;
  using P128 = PersistCfg<EPI, EPI ? 256 : 128, EPI ? 3 : 5>;      // 128 features per tile
  using P256 = PersistCfg<EPI, 256, 3>;                            // 256 features per tile (plain epilogue only)
  if (splits > 1) {
    static_assert(G_BM * (Deep::NACC + 4) * 4 <= Deep::STAGES * Deep::STAGE_BYTES, "the float32 tile must fit in the stages");
    if (splits > 8) return IFB_ERR_ARG;
    // one tile of rows: a CTA per SM with a deep ring; more: two CTAs per SM, one's sum beside the other's products
    if ((n <= G_BM && shape != 1) || G_BM * (Narrow::NACC + 4) * 4 > Narrow::STAGES * Narrow::STAGE_BYTES)
      return tc_launch_cfg<Deep, TO>(x, w, out, n, o, k, err, s, fold, splits);
    return tc_launch_cfg<Narrow, TO>(x, w, out, n, o, k, err, s, fold, splits);
  }
  if (shape == 0) shape = tc_pick_shape(EPI, n, o);
  if (fold.res_x && (EPI || shape > 3)) return IFB_ERR_ARG;        // the making side is the one-tile kernel's
  if (shape == 5 && !EPI) return tc_launch_persistent<P256, TO>(x, w, out, n, o, k, err, tc_sm_count(), s, fold);
  if (shape == 4 || shape == 5) return tc_launch_persistent<P128, TO>(x, w, out, n, o, k, err, tc_sm_count(), s, fold);
  if (shape == 3) return tc_launch_cfg<Wide, TO>(x, w, out, n, o, k, err, s, fold);
  if (shape == 2) return tc_launch_cfg<Deep, TO>(x, w, out, n, o, k, err, s, fold);
  return tc_launch_cfg<Narrow, TO>(x, w, out, n, o, k, err, s, fold);
}

// x [n_rows, k] and w [out_features (x2 for the silu_gate epilogue), k] bfloat16, 16-byte aligned, k a multiple of 8;
// out bfloat16 or float32.  `err` points to a device int that stays 0 unless a bounded wait gave up.  shape: 0 lets the
// library choose, 1-3 force the one-tile-per-CTA kernel narrow, deep or wide, 4 and 5 the persistent kernel with tiles
// of 128 or 256 features.  splits 2 to 8: the k range of a tile of 128 x 128 is shared by a cluster of
// that many CTAs, whose parts are added in a fixed order; for few tiles of a long k (a step of some tens of tokens).
// scale_partials (may be null): [scale_parts][n_rows] sums of squares; output row n is multiplied by
// rsqrt(sum_p partials[p][n] / scale_width + scale_eps) before the epilogue.
// res_x (may be null; plain epilogue, shape 0-3): the residual stream [n_rows][out_features] float32: v = x + y is
// written back to it, out = v * res_g, and res_partials [ifb_linear_tcgen05_fold_parts(...)][n_rows] gets sums of v^2.
IFB_EXPORT int ifb_linear_tcgen05_ex(const void* x, const void* w, void* out, int out_dtype, int n_rows, int out_features,
                                     int k_dim, int epilogue, int shape, int splits, const float* scale_partials, int scale_parts,
                                     float scale_eps, int scale_width, float* res_x, const void* res_g, int res_g_dtype,
                                     float* res_partials, int* err, cudaStream_t stream) {
  if (n_rows <= 0 || out_features <= 0) return IFB_OK;
  if (k_dim < 8 || k_dim % 8) return IFB_ERR_SIZE;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return IFB_ERR_ALIGN;
  if (epilogue != 0 && epilogue != 1) return IFB_ERR_ARG;
  if (shape < 0 || shape > 5 || splits < 0 || splits > 8) return IFB_ERR_ARG;
  if (scale_partials && (scale_parts < 1 || scale_width < 1)) return IFB_ERR_ARG;
  if (res_x && (!res_g || !res_partials || ((uintptr_t)res_x & 15))) return IFB_ERR_ARG;
  TcFold fold = {};
  fold.rs_partials = scale_partials; fold.rs_parts = scale_parts; fold.rs_eps = scale_eps;
  fold.rs_inv_width = scale_partials ? 1.f / (float)scale_width : 0.f;
  fold.res_x = res_x; fold.res_g = res_g; fold.res_g_dtype = res_g_dtype; fold.res_partials = res_partials;
  if (out_dtype == IFB_BF16)
    return epilogue ? tc_launch<1, bf16>(x, w, out, n_rows, out_features, k_dim, err, shape, splits, fold, stream)
                    : tc_launch<0, bf16>(x, w, out, n_rows, out_features, k_dim, err, shape, splits, fold, stream);
  if (out_dtype == IFB_F32)
    return epilogue ? tc_launch<1, float>(x, w, out, n_rows, out_features, k_dim, err, shape, splits, fold, stream)
                    : tc_launch<0, float>(x, w, out, n_rows, out_features, k_dim, err, shape, splits, fold, stream);
  return IFB_ERR_DTYPE;
}

IFB_EXPORT int ifb_linear_tcgen05(const void* x, const void* w, void* out, int out_dtype, int n_rows, int out_features,
                                  int k_dim, int epilogue, int* err, int shape, cudaStream_t stream) {
  return ifb_linear_tcgen05_ex(x, w, out, out_dtype, n_rows, out_features, k_dim, epilogue, shape, 1, nullptr, 0, 0.f, 0, nullptr,
                               nullptr, 0, nullptr, err, stream);
}

// The fused q | k | v projection of an attention layer in the shared-k form with what follows it in the sum over the
// cluster (see TcFold): qkv [n_rows, (nq + 2 nkv) * 128] bfloat16 gets the normalised and rotated q heads (and the k and
// v heads as they are stored), the pages get k and v at slots[n].  Heads of 128, rotated whole in the half-split pairing
// (rope: [n_rows][64] pairs of cos and sin, or null); splits 2 to 8.  scale_*: as in ifb_linear_tcgen05_ex.
IFB_EXPORT int ifb_linear_tcgen05_qkv(const void* x, const void* w, void* qkv, int n_rows, int nq, int nkv, int head_dim, int k_dim,
                                      int splits, const float* scale_partials, int scale_parts, float scale_eps, int scale_width,
                                      const void* q_weight, const void* k_weight, int w_dtype, float eps, const float* rope,
                                      const int* slots, void* pages, int page_size, int* err, cudaStream_t stream) {
  if (n_rows <= 0) return IFB_OK;
  if (head_dim != 128 || nq < 1 || nkv < 1 || splits < 2 || splits > 8) return IFB_ERR_SIZE;
  if (k_dim < 8 || k_dim % 8) return IFB_ERR_SIZE;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)qkv & 15) || ((uintptr_t)pages & 15) || ((uintptr_t)rope & 7))
    return IFB_ERR_ALIGN;
  if ((q_weight || k_weight) && w_dtype != IFB_F32 && w_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  if (scale_partials && (scale_parts < 1 || scale_width < 1)) return IFB_ERR_ARG;
  if (slots && (!pages || page_size < 1)) return IFB_ERR_ARG;
  TcFold fold = {};
  fold.rs_partials = scale_partials; fold.rs_parts = scale_parts; fold.rs_eps = scale_eps;
  fold.rs_inv_width = scale_partials ? 1.f / (float)scale_width : 0.f;
  fold.qk_nq = nq; fold.qk_nkv = nkv; fold.qk_qw = q_weight; fold.qk_kw = k_weight; fold.qk_w_dtype = w_dtype; fold.qk_eps = eps;
  fold.qk_rope = reinterpret_cast<const float2*>(rope); fold.qk_slots = slots; fold.qk_pages = (bf16*)pages;
  fold.qk_page_size = page_size;
  return tc_launch<0, bf16>(x, w, qkv, n_rows, (nq + 2 * nkv) * 128, k_dim, err, 0, splits, fold, stream);
}

// Parts of sums of squares that a product with res_x writes per row (the launch with shape 0 and these splits).
IFB_EXPORT int ifb_linear_tcgen05_fold_parts(int n_rows, int out_features, int splits) {
  if (splits > 1) return (out_features + 127) / 128;
  return tc_pick_shape(0, n_rows, out_features) == 3 ? 2 * ((out_features + 255) / 256) : 2 * ((out_features + 127) / 128);
}

using SplitCfg = GemmCfg<0, 1, 128, 6>;

// How many clusters of `splits` CTAs of that kernel the device holds at a time (0 if it cannot say): a product whose
// tiles are no more than this runs in one wave.
IFB_EXPORT int ifb_linear_tcgen05_split_clusters(int splits) {
  static int cached_all[IFB_MAX_DEVICES][9] = {};
  static bool known_all[IFB_MAX_DEVICES][9] = {};
  int dev = 0;
  if (splits < 2 || splits > 8 || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= IFB_MAX_DEVICES) return 0;
  int* cached = cached_all[dev];
  bool* known = known_all[dev];
  if (!known[splits]) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, splits);
    cfg.blockDim = dim3(G_THREADS);
    cfg.dynamicSmemBytes = SplitCfg::SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = splits;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaFuncSetAttribute(linear_tcgen05_kernel<SplitCfg, float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)SplitCfg::SMEM_BYTES) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&clusters, linear_tcgen05_kernel<SplitCfg, float>, &cfg) != cudaSuccess) {
      cudaGetLastError();
      clusters = 0;
    }
    cached[splits] = clusters;
    known[splits] = true;
  }
  return cached[splits];
}
