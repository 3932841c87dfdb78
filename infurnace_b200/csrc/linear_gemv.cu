// Matrix product for few rows (decoded tokens): out[n, o] = sum_k x[n, k] w[o, k], bfloat16 operands,
// float32 accumulation on tensor cores (mma.sync m16n8k16 with the weight rows on the M side).
//
// A decode step runs a few hundred of these, each over a few megabytes of weights, so what counts is
// the length of the chain of dependent memory round trips inside one launch, not only the bytes.
// Hence: a CTA owns 16 output features over the whole k range; its warps split k among themselves and
// add their partial tiles through shared memory (no partials in global memory, no second pass); weight
// and activation fragments are loaded straight from global memory into registers, all at once; and the
// first weight fragments are requested before the kernel waits for its predecessor in the stream,
// since weights do not depend on it.
//
// k is walked in a permuted order inside each MMA: a thread's 16-byte load brings 8 consecutive k of a
// weight row, which feed two MMAs; the activation fragment is read at the same 8 positions.
#include "common.cuh"

typedef __nv_bfloat16 bf16;
constexpr int GV_ROWS = 16;
// CTAs per SM asked of the compiler for the plain one-stage kernel of 8 warps and one block of tokens (the LM head of a
// small model, 9,496 CTAs): with 80 registers three fit and the 311 MB stream at 5.8 to 6.3 TB/s; with the 103 the
// compiler took unasked two fit (4.8 to 5.0 TB/s), with four (64 registers, spills) it is slower again.
#ifndef IFB_GV_LM_BLOCKS
#define IFB_GV_LM_BLOCKS 3
#endif
constexpr size_t GV_EARLY_BYTES = 24u << 20;     // weight bytes up to which a launch may start before its predecessor ends

__device__ __forceinline__ uint4 gv_ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void gv_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// A normalisation folded into the products around it.  RMSNorm is y = v * r * g with r = rsqrt(mean(v^2) + eps) one
// number per row, so a product of y equals r times the product of v * g: the producer of v (epilogue 2) writes v * g and
// the sums of v^2 over its own features, and the consumer adds those partial sums in a fixed order and multiplies its
// accumulators by r before its own epilogue.  No kernel runs for the norm itself.
struct GvRowScale {        // consumer side: null `partials` = none
  const float* partials;   // [parts][n_rows] partial sums of squares
  int parts;
  float eps, inv_width;    // r = rsqrt(sum * inv_width + eps)
};
struct GvResidual {        // producer side, epilogue 2
  float* x;                // [n_rows][o_out] float32 residual stream, updated in place: v = x + y
  const void* g;           // [o_out] norm weight
  int g_dtype;
  float* partials;         // [gridDim.x][n_rows], written
  int feat;                // features per CTA for the plain epilogue and epilogue 2: 16, or 8 (the tile's rows 8-15 stay
};                         // empty) where 16 would leave more than half of the SMs without a CTA

// EPI 3: the product is the fused q | k | v projection of an attention layer and the kernel finishes what follows it for
// every head: RMSNorm over the head (q and k heads), rotation in the half-split pairing, q written to the qkv row, k and v
// to the token's place in the pages.  A CTA owns the 16 features [c*16, c*16+16) of a head's first half and their
// partners in the second half, so the rotation is local; the head_dim/32 CTAs of a head form a thread-block cluster and
// hand one another their sums of squares through distributed shared memory (one write to every peer, one cluster barrier).
struct GvQkv {
  int nq, nkv, head_dim;
  const void* qw;           // [head_dim] norm weights (null: no norm)
  const void* kw;
  int w_dtype;
  float eps;
  const float2* rope;       // [n_rows][head_dim / 2] (cos, sin) of each token's angles (null: no rotation)
  const int* slots;         // [n_rows] page * page_size + offset, negative: store nothing (null: no store)
  bf16* pages;              // [page][k | v][kv head][offset][head_dim]
  int page_size;
};

__device__ __forceinline__ uint32_t gv_cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t gv_cluster_size() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(r)); return r; }
__device__ __forceinline__ void gv_store_to_peer(float* local, uint32_t peer, float v) {
  const uint32_t laddr = (uint32_t)__cvta_generic_to_shared(local);
  uint32_t raddr;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(raddr) : "r"(laddr), "r"(peer));
  asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(raddr), "f"(v) : "memory");
}
__device__ __forceinline__ void gv_cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// NB: blocks of 8 tokens per CTA.  EPI 0: out = y.  EPI 1: w holds gate rows [0, O) and up rows [O, 2O);
// out = silu(gate) * up.  EPI 2: v = x + y is written back to x, out = v * g.  EPI 4: as EPI 1 with 8 features per
// CTA, whose 8 gate rows and 8 up rows are the two halves of one 16-row tile (half the registers of EPI 1, so two CTAs
// per SM where EPI 1 with two stages has one).  WARPS: warps of a CTA (they split k).
// STAGES: steps of 128 of k whose weights (and, for one block of tokens, activations) a warp has requested at any
// time.  1: every warp's k range is one step (the sizes of small models, where the chain of round trips counts);
// 2: a warp walks a long k range and keeps the memory pipe full while it multiplies (large models, where the
// bytes count).
template <int NB, int EPI, int WARPS, typename TO, int STAGES>
__global__ void __launch_bounds__(WARPS * 32, (EPI == 4 && WARPS == 8) ? 2 : (EPI == 0 && WARPS == 8 && STAGES == 1 && NB == 1) ? IFB_GV_LM_BLOCKS : 0)
linear_gemv_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, TO* __restrict__ out, int n_rows, int o_out,
                   int k_dim, GvRowScale rs, GvResidual res, GvQkv qk) {
  extern __shared__ float gv_red[];                 // [WARPS][NE][NB*8][GV_ROWS], then [NB*8] row factors
  constexpr int NE = (EPI == 1 || EPI == 3) ? 2 : 1;
  static_assert(EPI != 3 || (NB <= 2 && WARPS * 32 >= NB * 8 * GV_ROWS), "the fused qkv epilogue keeps one (token, feature pair) per thread");
  constexpr bool STAGE_X = STAGES > 1 && NB == 1;    // activations requested ahead with the weights
  float* row_factor = gv_red + (size_t)WARPS * NE * NB * 8 * GV_ROWS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = lane & 3, rr = lane >> 2;
  // EPI 3: blockIdx.x = head * (head_dim / 32) + c; the first 16 features are the head's [c*16, c*16+16), the second 16
  // their rotation partners head_dim/2 further on
  const int qk_per_head = EPI == 3 ? qk.head_dim / 32 : 1;
  const int qk_head = EPI == 3 ? blockIdx.x / qk_per_head : 0, qk_c = EPI == 3 ? blockIdx.x % qk_per_head : 0;
  const bool half_tile = (EPI == 0 || EPI == 2) && res.feat == 8;     // 8 features per CTA: no weight rows for the tile's second half
  const int feat = (EPI == 4 || half_tile) ? 8 : GV_ROWS;
  const int o0 = EPI == 3 ? qk_head * qk.head_dim + qk_c * GV_ROWS : blockIdx.x * feat, n0 = blockIdx.y * (NB * 8);
  const int second = EPI == 3 ? qk.head_dim / 2 : o_out;      // distance of the second set of 16 weight rows from the first
  const int kw = ((k_dim + WARPS - 1) / WARPS + 127) / 128 * 128;      // k per warp, whole 128-wide steps
  const int kbeg = warp * kw, kend = min(k_dim, kbeg + kw);
  const int w_rows = (EPI == 1 || EPI == 4) ? 2 * o_out : o_out;
  const bf16* wrow[NE][2];
#pragma unroll
  for (int e = 0; e < NE; ++e) {
    wrow[e][0] = w + (size_t)min(e * second + o0 + rr, w_rows - 1) * k_dim;
    wrow[e][1] = w + (size_t)min(e * second + o0 + rr + 8, w_rows - 1) * k_dim;
  }
  if (EPI == 4) {                                               // rows 0-7 of the tile: gate; rows 8-15: up of the same features
    wrow[0][0] = w + (size_t)min(o0 + rr, o_out - 1) * k_dim;
    wrow[0][1] = w + (size_t)min(o_out + o0 + rr, w_rows - 1) * k_dim;
  }
  const bf16* xrow[NB];
  bool xok[NB];
#pragma unroll
  for (int j = 0; j < NB; ++j) {
    const int n = n0 + j * 8 + rr;
    xok[j] = n < n_rows;
    xrow[j] = x + (size_t)min(n, n_rows - 1) * k_dim;
  }
  float acc[NE][NB][4];
#pragma unroll
  for (int e = 0; e < NE; ++e)
#pragma unroll
    for (int j = 0; j < NB; ++j) acc[e][j][0] = acc[e][j][1] = acc[e][j][2] = acc[e][j][3] = 0.f;

  if constexpr (STAGES == 1) {
    // every warp's k range is (mostly) one step: weights requested, then the wait for whoever writes x, then the products
    bool waited = false;
    for (int k0 = kbeg; k0 < kend || !waited; k0 += 128) {
      uint4 wa[NE][4], wb[NE][4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int k = k0 + c * 32 + q * 8;
        const bool in = k < kend;
#pragma unroll
        for (int e = 0; e < NE; ++e) {
          wa[e][c] = in ? gv_ld_stream16(wrow[e][0] + k) : make_uint4(0, 0, 0, 0);
          wb[e][c] = (in && !half_tile) ? gv_ld_stream16(wrow[e][1] + k) : make_uint4(0, 0, 0, 0);
        }
      }
      if (!waited) {           // the weights are on their way; now wait for whoever writes x
        ifb_pdl_wait();
        ifb_pdl_trigger();
        waited = true;
        if (rs.partials) {     // the rows' factors, requested now and used after the products
          for (int n = warp; n < NB * 8; n += WARPS) {
            float ssum = 0.f;
            if (n0 + n < n_rows)
              for (int p = lane; p < rs.parts; p += 32) ssum += rs.partials[(size_t)p * n_rows + n0 + n];
            ssum = warp_sum(ssum);
            if (lane == 0) row_factor[n] = rsqrtf(ssum * rs.inv_width + rs.eps);
          }
        }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int k = k0 + c * 32 + q * 8;
        if (k0 + c * 32 >= kend) break;
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          uint4 xv = make_uint4(0, 0, 0, 0);
          if (xok[j] && k < kend) xv = *reinterpret_cast<const uint4*>(xrow[j] + k);
#pragma unroll
          for (int e = 0; e < NE; ++e) {
            gv_mma(acc[e][j], wa[e][c].x, wb[e][c].x, wa[e][c].y, wb[e][c].y, xv.x, xv.y);
            gv_mma(acc[e][j], wa[e][c].z, wb[e][c].z, wa[e][c].w, wb[e][c].w, xv.z, xv.w);
          }
        }
      }
    }
  } else {
    uint4 wa[STAGES][NE][4], wb[STAGES][NE][4], xs[STAGE_X ? STAGES : 1][4];
    auto load_w = [&](int st, int k0) {
  #pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int k = k0 + c * 32 + q * 8;
        const bool in = k < kend;
  #pragma unroll
        for (int e = 0; e < NE; ++e) {
          wa[st][e][c] = in ? gv_ld_stream16(wrow[e][0] + k) : make_uint4(0, 0, 0, 0);
          wb[st][e][c] = (in && !half_tile) ? gv_ld_stream16(wrow[e][1] + k) : make_uint4(0, 0, 0, 0);
        }
      }
    };
    auto load_x = [&](int st, int k0) {
      if (STAGE_X) {
  #pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int k = k0 + c * 32 + q * 8;
          xs[st][c] = (xok[0] && k < kend) ? *reinterpret_cast<const uint4*>(xrow[0] + k) : make_uint4(0, 0, 0, 0);
        }
      }
    };
    auto multiply = [&](int st, int k0) {
      // the activations of the whole step are requested before the first product, so that they make one round trip to L2,
      // not one per 32 of k (for many blocks of tokens that would be too many registers: a round trip per 32 of k then)
      constexpr bool X_AHEAD = !STAGE_X && NB <= 2;
      uint4 xl[X_AHEAD ? 4 : 1][NB];
      if (X_AHEAD) {
  #pragma unroll
        for (int c = 0; c < 4; ++c)
  #pragma unroll
          for (int j = 0; j < NB; ++j) {
            const int k = k0 + c * 32 + q * 8;
            xl[c][j] = (xok[j] && k < kend) ? *reinterpret_cast<const uint4*>(xrow[j] + k) : make_uint4(0, 0, 0, 0);
          }
      }
  #pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int k = k0 + c * 32 + q * 8;
        if (k0 + c * 32 >= kend) break;
  #pragma unroll
        for (int j = 0; j < NB; ++j) {
          uint4 xv = make_uint4(0, 0, 0, 0);
          if (STAGE_X) xv = xs[st][c];
          else if (X_AHEAD) xv = xl[c][j];
          else if (xok[j] && k < kend) xv = *reinterpret_cast<const uint4*>(xrow[j] + k);
  #pragma unroll
          for (int e = 0; e < NE; ++e) {
            gv_mma(acc[e][j], wa[st][e][c].x, wb[st][e][c].x, wa[st][e][c].y, wb[st][e][c].y, xv.x, xv.y);
            gv_mma(acc[e][j], wa[st][e][c].z, wb[st][e][c].z, wa[st][e][c].w, wb[st][e][c].w, xv.z, xv.w);
          }
        }
      }
    };

    // the first weights are on their way before this kernel waits for whoever writes x
  #pragma unroll
    for (int st = 0; st < STAGES; ++st) load_w(st, kbeg + st * 128);
    ifb_pdl_wait();
  #pragma unroll
    for (int st = 0; st < STAGES; ++st) load_x(st, kbeg + st * 128);
    if (rs.partials) {     // the rows' factors, requested now and used after the products
      for (int n = warp; n < NB * 8; n += WARPS) {
        float ssum = 0.f;
        if (n0 + n < n_rows)
          for (int p = lane; p < rs.parts; p += 32) ssum += rs.partials[(size_t)p * n_rows + n0 + n];
        ssum = warp_sum(ssum);
        if (lane == 0) row_factor[n] = rsqrtf(ssum * rs.inv_width + rs.eps);
      }
    }
    for (int k0 = kbeg; k0 < kend; k0 += 128 * STAGES) {
  #pragma unroll
      for (int st = 0; st < STAGES; ++st) {
        const int ks = k0 + st * 128;
        if (ks < kend) {
          if (STAGES == 1 && ks > kbeg) {                   // a single stage: each further step is requested when its turn comes
            load_w(0, ks);
            load_x(0, ks);
          }
          multiply(st, ks);
          if (STAGES > 1 && ks + 128 * STAGES < kend) {     // this stage's registers are free: request the step after next
            load_w(st, ks + 128 * STAGES);
            load_x(st, ks + 128 * STAGES);
          }
        }
      }
    }
    // A kernel that walks long k ranges lives on its bytes in flight: the next kernel of the stream, which would sit on
    // the SMs' registers and wait, is let in only now that this CTA has no more weights to ask for.
    ifb_pdl_trigger();
  }
  // acc[e][j]: c0,c1 -> (feature rr, tokens j*8 + 2q, +1); c2,c3 -> feature rr + 8
  float* mine = gv_red + (size_t)warp * NE * NB * 8 * GV_ROWS;
#pragma unroll
  for (int e = 0; e < NE; ++e)
#pragma unroll
    for (int j = 0; j < NB; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = rr + (i >> 1) * 8, n = j * 8 + 2 * q + (i & 1);
        mine[((size_t)e * NB * 8 + n) * GV_ROWS + m] = acc[e][j][i];
      }
  __syncthreads();
  // NB * 8 * GV_ROWS is a multiple of 32 and so is the stride: whole warps walk this loop together, and the 16
  // features of a token sit in 16 neighbouring lanes
  float qk_y0 = 0.f, qk_y1 = 0.f;
  for (int idx = tid; idx < NB * 8 * GV_ROWS; idx += WARPS * 32) {
    const int n = idx / GV_ROWS, m = idx % GV_ROWS;
    const int o = o0 + m, tok = n0 + n;
    const bool valid = o < o_out && tok < n_rows && (!half_tile || m < 8);
    float y[NE];
#pragma unroll
    for (int e = 0; e < NE; ++e) {
      float s = 0.f;
#pragma unroll
      for (int wv = 0; wv < WARPS; ++wv) s += gv_red[(((size_t)wv * NE + e) * NB * 8 + n) * GV_ROWS + m];
      y[e] = rs.partials ? s * row_factor[n] : s;
    }
    float r = y[0];
    if (EPI == 1) r = r / (1.f + expf(-r)) * y[NE - 1];
    if (EPI == 4) {                                    // this item is the gate of feature o0 + m; its up sits 8 rows on
      if (m >= 8) continue;
      float up = 0.f;
#pragma unroll
      for (int wv = 0; wv < WARPS; ++wv) up += gv_red[((size_t)wv * NB * 8 + n) * GV_ROWS + m + 8];
      if (rs.partials) up *= row_factor[n];
      if (valid) out[(size_t)tok * o_out + o] = from_f32<TO>(r / (1.f + expf(-r)) * up);
      continue;
    }
    if (EPI == 3) { qk_y0 = y[0]; qk_y1 = y[NE - 1]; continue; }      // finished below, after the loop (one item per thread)
    if (EPI == 2) {
      float v = 0.f;
      if (valid) {
        v = res.x[(size_t)tok * o_out + o] + r;
        res.x[(size_t)tok * o_out + o] = v;
        out[(size_t)tok * o_out + o] = from_f32<TO>(v * load_as_f32(res.g, res.g_dtype, o));
      }
      float sq = v * v;                              // the sum over this CTA's 16 features, in a fixed order
      sq += __shfl_xor_sync(0xffffffffu, sq, 8);
      sq += __shfl_xor_sync(0xffffffffu, sq, 4);
      sq += __shfl_xor_sync(0xffffffffu, sq, 2);
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      if (m == 0 && tok < n_rows) res.partials[(size_t)blockIdx.x * n_rows + tok] = sq;
    } else if (valid) {
      out[(size_t)tok * o_out + o] = from_f32<TO>(r);
    }
  }
  if (EPI == 3) {
    __shared__ float qk_ssq[8][NB * 8];                 // [CTA of the head][token]: sums of squares over 32 features
    const bool mine = tid < NB * 8 * GV_ROWS;           // this thread holds the pair (m, m + head_dim/2) of token n
    const int n = tid / GV_ROWS, m = tid % GV_ROWS, tok = n0 + n;
    const bool is_v = qk_head >= qk.nq + qk.nkv, is_k = qk_head >= qk.nq && !is_v;
    const void* nw = is_v ? nullptr : (is_k ? qk.kw : qk.qw);
    const uint32_t rank = gv_cluster_rank(), peers = gv_cluster_size();
    float sq = mine ? qk_y0 * qk_y0 + qk_y1 * qk_y1 : 0.f;
    sq += __shfl_xor_sync(0xffffffffu, sq, 8);
    sq += __shfl_xor_sync(0xffffffffu, sq, 4);
    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
    if (mine && m == 0)
      for (uint32_t p = 0; p < peers; ++p) gv_store_to_peer(&qk_ssq[rank][n], p, sq);
    gv_cluster_barrier();                               // every thread of every CTA of the head, on every path
    if (!mine || tok >= n_rows) return;
    const int D = qk.head_dim, half = D / 2, i = qk_c * GV_ROWS + m;
    float a = qk_y0, b = qk_y1;
    if (nw) {
      float total = 0.f;
      for (uint32_t p = 0; p < peers; ++p) total += qk_ssq[p][n];      // in a fixed order
      const float rn = rsqrtf(total / (float)D + qk.eps);
      a *= rn * load_as_f32(nw, qk.w_dtype, i);
      b *= rn * load_as_f32(nw, qk.w_dtype, i + half);
    }
    if (!is_v && qk.rope) {
      const float2 cs = qk.rope[(size_t)tok * half + i];
      const float ra = a * cs.x - b * cs.y, rb = b * cs.x + a * cs.y;
      a = ra; b = rb;
    }
    const bf16 oa = __float2bfloat16_rn(a), ob = __float2bfloat16_rn(b);
    bf16* row = reinterpret_cast<bf16*>(out) + (size_t)tok * o_out + (size_t)qk_head * D;
    row[i] = oa;
    row[i + half] = ob;
    if (qk_head >= qk.nq && qk.slots) {
      const int slot = qk.slots[tok];
      if (slot >= 0) {
        const int kvh = is_v ? qk_head - qk.nq - qk.nkv : qk_head - qk.nq;
        bf16* dst = qk.pages + ((((size_t)(slot / qk.page_size) * 2 + (is_v ? 1 : 0)) * qk.nkv + kvh) * qk.page_size +
                                (slot % qk.page_size)) * D;
        dst[i] = oa;
        dst[i + half] = ob;
      }
    }
  }
}

// Features per CTA of the plain epilogue and epilogue 2: 8 for a single row where tiles of 16 would leave more than
// half of the SMs without a CTA (the o and down products of a small model: 1,024 features are 64 CTAs of 16, each
// pulling twice the bytes a CTA of 8 pulls, on a device of 148 SMs).  Measured in a decode step of the 0.6B sizes:
// 0.802 to 0.787 ms at one row; with 2, 4 and 8 rows the 128 CTAs' reads of the rows outweigh it (0.894 to 0.948,
// 1.020 to 1.117, 1.314 to 1.374 ms), so those keep 16.
static int gv_features_per_cta(int o, int n_rows) {
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      sm_count = 1;
  }
  static int forced = -1;                    // IFB_GV_FEAT=16 keeps tiles of 16 (for measurements)
  if (forced < 0) { const char* v = getenv("IFB_GV_FEAT"); forced = v ? atoi(v) : 0; }
  if (forced == 16 || n_rows > 1) return GV_ROWS;
  return 2 * ((o + GV_ROWS - 1) / GV_ROWS) <= sm_count ? 8 : GV_ROWS;
}

template <int NB, int EPI, int WARPS, typename TO, int STAGES = 1>
static int gv_launch(const void* x, const void* w, void* out, int n, int o, int k, const GvRowScale& rs, const GvResidual& res,
                     cudaStream_t s) {
  static_assert(EPI != 3, "the fused qkv epilogue is launched by gv_launch_qkv");
  const size_t smem = ((size_t)WARPS * (EPI == 1 ? 2 : 1) * NB * 8 * GV_ROWS + NB * 8) * sizeof(float);
  IFB_ALLOW_SMEM((linear_gemv_kernel<NB, EPI, WARPS, TO, STAGES>), smem);
  GvResidual res_f = res;
  res_f.feat = (EPI == 0 || EPI == 2) ? gv_features_per_cta(o, n) : GV_ROWS;
  const int per_cta = EPI == 4 ? 8 : res_f.feat;
  dim3 grid((o + per_cta - 1) / per_cta, (n + NB * 8 - 1) / (NB * 8));
  // matrices beyond GV_EARLY_BYTES are streamed; a launch ahead of the predecessor's end costs them more than it hides
  const bool early = (size_t)o * k * ((EPI == 1 || EPI == 4) ? 4 : 2) <= GV_EARLY_BYTES;
  return ifb_launch_opt(early, linear_gemv_kernel<NB, EPI, WARPS, TO, STAGES>, grid, dim3(WARPS * 32), smem, s, (const bf16*)x,
                        (const bf16*)w, (TO*)out, n, o, k, rs, res_f, GvQkv{});
}

// The fused q | k | v product: one CTA per (head, 16 feature pairs), the CTAs of a head as a thread-block cluster.
template <int NB, int WARPS, int STAGES>
static int gv_launch_qkv(const void* x, const void* w, void* out, int n, int k, const GvRowScale& rs, const GvQkv& qk,
                         cudaStream_t s) {
  const size_t smem = ((size_t)WARPS * 2 * NB * 8 * GV_ROWS + NB * 8) * sizeof(float);
  IFB_ALLOW_SMEM((linear_gemv_kernel<NB, 3, WARPS, bf16, STAGES>), smem);
  const int per_head = qk.head_dim / 32, heads = qk.nq + 2 * qk.nkv;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(heads * per_head, 1, 1);
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = per_head;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (ifb_pdl_enabled() && (size_t)heads * qk.head_dim * k * 2 <= GV_EARLY_BYTES) ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, linear_gemv_kernel<NB, 3, WARPS, bf16, STAGES>, (const bf16*)x, (const bf16*)w, (bf16*)out, n,
                                     heads * qk.head_dim, k, rs, GvResidual{nullptr, nullptr, 0, nullptr}, qk);
  if (e != cudaSuccess) { cudaGetLastError(); return -(int)e; }
  return IFB_OK;
}

static int g_gv_gate_plan = 0;      // a plan (see below) for products with the silu_gate epilogue alone; negative: the
IFB_EXPORT void ifb_linear_gemv_set_gate_plan(int plan) { g_gv_gate_plan = plan; }      // 16-features-per-CTA form throughout

template <int EPI, int WARPS, typename TO, int STAGES = 1>
static int gv_by_n(int nb, const void* x, const void* w, void* out, int n, int o, int k, const GvRowScale& rs,
                   const GvResidual& res, cudaStream_t s) {
  switch (nb) {
    // one block of tokens of a long k (two stages): the silu_gate epilogue in its 8-features-per-CTA form, two CTAs per SM
    // (40 against 35 to 37 us for the 201 MB of the 8B sizes, 90 against 83 to 85 for the 524 MB of the 32B sizes; with more
    // blocks of tokens it is the slower one, and for a short k it gains in a chain of its own kind but not in the step)
    case 1:
      if (g_gv_gate_plan < 0) return gv_launch<1, EPI, WARPS, TO, STAGES>(x, w, out, n, o, k, rs, res, s);
      return gv_launch<1, ((EPI == 1 && STAGES == 2) ? 4 : EPI), WARPS, TO, STAGES>(x, w, out, n, o, k, rs, res, s);
    case 2: return gv_launch<2, EPI, WARPS, TO, STAGES>(x, w, out, n, o, k, rs, res, s);
    case 4: return gv_launch<4, EPI, WARPS, TO, STAGES>(x, w, out, n, o, k, rs, res, s);
    default: return gv_launch<8, EPI, WARPS, TO, STAGES>(x, w, out, n, o, k, rs, res, s);
  }
}

// plan 0: chosen from the sizes.  Otherwise warps * 10 + stages, one of 81, 161, 241, 82 (for measurements); 83: as 82
// with the silu_gate epilogue in its 8-features-per-CTA form.
static int g_gv_plan = 0;
IFB_EXPORT void ifb_linear_gemv_set_plan(int plan) { g_gv_plan = plan; }


template <int EPI, typename TO>
static int gv_by_k(int nb, const void* x, const void* w, void* out, int n, int o, int k, const GvRowScale& rs,
                   const GvResidual& res, cudaStream_t s) {
  int plan = g_gv_plan;
  if (plan == 0 && EPI == 1 && g_gv_gate_plan > 0) plan = g_gv_gate_plan;
  if (plan == 0) {
    // 128 of k per warp and step.  Up to k = 3072 every warp's range is one step: 8 warps cover 1024, 16 warps 2048, 24
    // warps 3072 (one or two blocks of tokens; more do not fit the registers of 768 threads).  Beyond that a warp walks
    // its range with the weights of further steps requested while it multiplies.
    if (k <= 1024) plan = 81;
    else if (k <= 2048) plan = 161;
    else if (k <= 3072 && nb <= 2) plan = 241;
    else plan = 82;       // two stages: a third measured slower at every size (its registers leave one CTA per SM)
  }
  switch (plan) {
    case 81: return gv_by_n<EPI, 8, TO, 1>(nb, x, w, out, n, o, k, rs, res, s);
    case 161: return gv_by_n<EPI, 16, TO, 1>(nb, x, w, out, n, o, k, rs, res, s);
    case 241:
      if (nb == 1) return gv_launch<1, EPI, 24, TO, 1>(x, w, out, n, o, k, rs, res, s);
      if (nb == 2) return gv_launch<2, EPI, 24, TO, 1>(x, w, out, n, o, k, rs, res, s);
      return gv_by_n<EPI, 16, TO, 1>(nb, x, w, out, n, o, k, rs, res, s);
    case 82: return gv_by_n<EPI, 8, TO, 2>(nb, x, w, out, n, o, k, rs, res, s);
    case 83: return gv_by_n<EPI == 1 ? 4 : EPI, 8, TO, 2>(nb, x, w, out, n, o, k, rs, res, s);
    default: return IFB_ERR_ARG;
  }
}

static int gv_blocks_of_8(int n_rows) { return n_rows <= 8 ? 1 : n_rows <= 16 ? 2 : n_rows <= 32 ? 4 : 8; }

// x [n_rows, k] and w [out_features (x2 for the silu_gate epilogue), k] bfloat16, 16-byte aligned, k a multiple of 8;
// out bfloat16 or float32.  Needs no scratch memory.
// scale_partials (may be null): [scale_parts][n_rows] float32 partial sums of squares of the rows of the vector that x
// was taken from; every output row n is multiplied by rsqrt(sum_p partials[p][n] / scale_width + scale_eps) before the
// epilogue.
IFB_EXPORT int ifb_linear_gemv(const void* x, const void* w, void* out, int out_dtype, int n_rows, int out_features,
                               int k_dim, int epilogue, const float* scale_partials, int scale_parts, float scale_eps,
                               int scale_width, cudaStream_t stream) {
  if (n_rows <= 0 || out_features <= 0) return IFB_OK;
  if (k_dim < 8 || k_dim % 8) return IFB_ERR_SIZE;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return IFB_ERR_ALIGN;
  if (epilogue != 0 && epilogue != 1) return IFB_ERR_ARG;
  if (scale_partials && (scale_parts < 1 || scale_width < 1)) return IFB_ERR_ARG;
  const int nb = gv_blocks_of_8(n_rows);
  if ((n_rows + nb * 8 - 1) / (nb * 8) > 65535) return IFB_ERR_SIZE;
  GvRowScale rs{scale_partials, scale_parts, scale_eps, scale_partials ? 1.f / (float)scale_width : 0.f};
  GvResidual res{nullptr, nullptr, 0, nullptr};
  if (out_dtype == IFB_BF16)
    return epilogue ? gv_by_k<1, bf16>(nb, x, w, out, n_rows, out_features, k_dim, rs, res, stream)
                    : gv_by_k<0, bf16>(nb, x, w, out, n_rows, out_features, k_dim, rs, res, stream);
  if (out_dtype == IFB_F32)
    return epilogue ? gv_by_k<1, float>(nb, x, w, out, n_rows, out_features, k_dim, rs, res, stream)
                    : gv_by_k<0, float>(nb, x, w, out, n_rows, out_features, k_dim, rs, res, stream);
  return IFB_ERR_DTYPE;
}

// The fused q | k | v projection of an attention layer with what follows it (see GvQkv): qkv [n_rows, (nq + 2 nkv) *
// head_dim] bfloat16 gets the normalised and rotated q heads (and the k and v heads as they are stored), the pages get k
// and v at slots[n].  head_dim 64, 128 or 256, rotated whole in the half-split pairing (rope: [n_rows][head_dim/2] pairs
// of cos and sin, or null), at most 16 rows.  scale_*: as in ifb_linear_gemv.
IFB_EXPORT int ifb_linear_gemv_qkv(const void* x, const void* w, void* qkv, int n_rows, int nq, int nkv, int head_dim, int k_dim,
                                   const float* scale_partials, int scale_parts, float scale_eps, int scale_width,
                                   const void* q_weight, const void* k_weight, int w_dtype, float eps, const float* rope,
                                   const int* slots, void* pages, int page_size, cudaStream_t stream) {
  if (n_rows <= 0) return IFB_OK;
  if (n_rows > 16 || (head_dim != 64 && head_dim != 128 && head_dim != 256) || nq < 1 || nkv < 1) return IFB_ERR_SIZE;
  if (k_dim < 8 || k_dim % 8) return IFB_ERR_SIZE;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return IFB_ERR_ALIGN;
  if (slots && (!pages || page_size < 1)) return IFB_ERR_ARG;
  if ((q_weight || k_weight) && w_dtype != IFB_F32 && w_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  if (scale_partials && (scale_parts < 1 || scale_width < 1)) return IFB_ERR_ARG;
  GvRowScale rs{scale_partials, scale_parts, scale_eps, scale_partials ? 1.f / (float)scale_width : 0.f};
  GvQkv qk{nq, nkv, head_dim, q_weight, k_weight, w_dtype, eps, reinterpret_cast<const float2*>(rope), slots,
           reinterpret_cast<bf16*>(pages), page_size};
  const int nb = n_rows <= 8 ? 1 : 2;
  if (k_dim <= 1024) return nb == 1 ? gv_launch_qkv<1, 8, 1>(x, w, qkv, n_rows, k_dim, rs, qk, stream)
                                    : gv_launch_qkv<2, 8, 1>(x, w, qkv, n_rows, k_dim, rs, qk, stream);
  if (k_dim <= 2048) return nb == 1 ? gv_launch_qkv<1, 16, 1>(x, w, qkv, n_rows, k_dim, rs, qk, stream)
                                    : gv_launch_qkv<2, 16, 1>(x, w, qkv, n_rows, k_dim, rs, qk, stream);
  return nb == 1 ? gv_launch_qkv<1, 8, 2>(x, w, qkv, n_rows, k_dim, rs, qk, stream)
                 : gv_launch_qkv<2, 8, 2>(x, w, qkv, n_rows, k_dim, rs, qk, stream);
}

// How many partial sums per row ifb_linear_gemv_residual_norm writes for this many output features and rows.
IFB_EXPORT int ifb_linear_gemv_parts(int out_features, int n_rows) {
  const int feat = gv_features_per_cta(out_features, n_rows);
  return (out_features + feat - 1) / feat;
}

// The product with the residual addition and the weight of the norm that follows folded in: v = resid + a w^T is
// written back to resid (float32 [n_rows, out_features]), out = v * g in bfloat16, and partials[p][n] = the sum of
// v[n][f]^2 over the 16 (or 8) features f of part p (ifb_linear_gemv_parts(out_features, n_rows) parts).  A later ifb_linear_gemv with
// these partials as its scale completes the RMSNorm.
IFB_EXPORT int ifb_linear_gemv_residual_norm(const void* a, const void* w, float* resid, const void* g, int g_dtype,
                                             void* out, float* partials, int n_rows, int out_features, int k_dim,
                                             cudaStream_t stream) {
  if (n_rows <= 0 || out_features <= 0) return IFB_OK;
  if (k_dim < 8 || k_dim % 8) return IFB_ERR_SIZE;
  if (((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return IFB_ERR_ALIGN;
  if (!resid || !g || !out || !partials) return IFB_ERR_ARG;
  if (g_dtype != IFB_F32 && g_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  const int nb = gv_blocks_of_8(n_rows);
  if (nb * 8 < n_rows) return IFB_ERR_SIZE;          // one block of tokens per feature group: the partials have one writer
  GvRowScale rs{nullptr, 0, 0.f, 0.f};
  GvResidual res{resid, g, g_dtype, partials};
  return gv_by_k<2, bf16>(nb, a, w, out, n_rows, out_features, k_dim, rs, res, stream);
}
