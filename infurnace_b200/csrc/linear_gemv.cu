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
};

// NB: blocks of 8 tokens per CTA.  EPI 0: out = y.  EPI 1: w holds gate rows [0, O) and up rows [O, 2O);
// out = silu(gate) * up.  EPI 2: v = x + y is written back to x, out = v * g.  WARPS: warps of a CTA (they split k).
template <int NB, int EPI, int WARPS, typename TO>
__global__ void __launch_bounds__(WARPS * 32)
linear_gemv_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, TO* __restrict__ out, int n_rows, int o_out,
                   int k_dim, GvRowScale rs, GvResidual res) {
  extern __shared__ float gv_red[];                 // [WARPS][NE][NB*8][GV_ROWS], then [NB*8] row factors
  constexpr int NE = EPI == 1 ? 2 : 1;
  float* row_factor = gv_red + (size_t)WARPS * NE * NB * 8 * GV_ROWS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = lane & 3, rr = lane >> 2;
  const int o0 = blockIdx.x * GV_ROWS, n0 = blockIdx.y * (NB * 8);
  const int kw = ((k_dim + WARPS - 1) / WARPS + 127) / 128 * 128;      // k per warp, whole 128-wide steps
  const int kbeg = warp * kw, kend = min(k_dim, kbeg + kw);
  const bf16* wrow[NE][2];
#pragma unroll
  for (int e = 0; e < NE; ++e) {
    wrow[e][0] = w + (size_t)(e * o_out + min(o0 + rr, o_out - 1)) * k_dim;
    wrow[e][1] = w + (size_t)(e * o_out + min(o0 + rr + 8, o_out - 1)) * k_dim;
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
        wb[e][c] = in ? gv_ld_stream16(wrow[e][1] + k) : make_uint4(0, 0, 0, 0);
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
  for (int idx = tid; idx < NB * 8 * GV_ROWS; idx += WARPS * 32) {
    const int n = idx / GV_ROWS, m = idx % GV_ROWS;
    const int o = o0 + m, tok = n0 + n;
    const bool valid = o < o_out && tok < n_rows;
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
}

template <int NB, int EPI, int WARPS, typename TO>
static int gv_launch(const void* x, const void* w, void* out, int n, int o, int k, const GvRowScale& rs, const GvResidual& res,
                     cudaStream_t s) {
  const size_t smem = ((size_t)WARPS * (EPI == 1 ? 2 : 1) * NB * 8 * GV_ROWS + NB * 8) * sizeof(float);
  IFB_ALLOW_SMEM((linear_gemv_kernel<NB, EPI, WARPS, TO>), smem);
  dim3 grid((o + GV_ROWS - 1) / GV_ROWS, (n + NB * 8 - 1) / (NB * 8));
  return ifb_launch(linear_gemv_kernel<NB, EPI, WARPS, TO>, grid, dim3(WARPS * 32), smem, s, (const bf16*)x, (const bf16*)w,
                    (TO*)out, n, o, k, rs, res);
}

template <int EPI, int WARPS, typename TO>
static int gv_by_n(int nb, const void* x, const void* w, void* out, int n, int o, int k, const GvRowScale& rs,
                   const GvResidual& res, cudaStream_t s) {
  switch (nb) {
    case 1: return gv_launch<1, EPI, WARPS, TO>(x, w, out, n, o, k, rs, res, s);
    case 2: return gv_launch<2, EPI, WARPS, TO>(x, w, out, n, o, k, rs, res, s);
    case 4: return gv_launch<4, EPI, WARPS, TO>(x, w, out, n, o, k, rs, res, s);
    default: return gv_launch<8, EPI, WARPS, TO>(x, w, out, n, o, k, rs, res, s);
  }
}

template <int EPI, typename TO>
static int gv_by_k(int nb, const void* x, const void* w, void* out, int n, int o, int k, const GvRowScale& rs,
                   const GvResidual& res, cudaStream_t s) {
  // 128 of k per warp and step: 8 warps cover k up to 1024 in one step, 16 warps up to 2048, 24 warps up to 3072 (a second
  // step would request its weights only after the first step's products)
  if (k > 2048 && nb == 1) return gv_launch<1, EPI, 24, TO>(x, w, out, n, o, k, rs, res, s);
  if (k > 2048 && nb == 2) return gv_launch<2, EPI, 24, TO>(x, w, out, n, o, k, rs, res, s);
  return k > 1024 ? gv_by_n<EPI, 16, TO>(nb, x, w, out, n, o, k, rs, res, s) : gv_by_n<EPI, 8, TO>(nb, x, w, out, n, o, k, rs, res, s);
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

// How many partial sums per row ifb_linear_gemv_residual_norm writes for this many output features.
IFB_EXPORT int ifb_linear_gemv_parts(int out_features) { return (out_features + GV_ROWS - 1) / GV_ROWS; }

// The product with the residual addition and the weight of the norm that follows folded in: v = resid + a w^T is
// written back to resid (float32 [n_rows, out_features]), out = v * g in bfloat16, and partials[p][n] = the sum of
// v[n][f]^2 over the 16 features f of part p (ifb_linear_gemv_parts(out_features) parts).  A later ifb_linear_gemv with
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
