// Matrix product for few rows (decoded tokens and short portions): out[n, o] = sum_k x[n, k] w[o, k],
// bfloat16 operands, float32 accumulation, on tensor cores.  The work is the reading of w once, so the
// weight rows are the M side of the MMA (16 output features per warp), the tokens the N side (blocks
// of 8), and k is split over `splits` CTAs per 64-feature tile until the grid covers the SMs.
//
// With splits > 1 every CTA writes its float32 partial tile to scratch and bumps the tile's counter;
// the CTA that arrives last adds the partials in split order (so the result does not depend on which
// CTA that is), applies the epilogue and resets the counter.  Nothing waits on anything.
//
// k is walked in an order that differs from the textbook fragment layout: a thread's 16-byte load
// brings 8 consecutive k of one weight row, which feed two MMAs; the activation fragment of the same
// thread column is read at the same 8 positions, so every product pairs equal k.
#include "common.cuh"

typedef __nv_bfloat16 bf16;
constexpr int SK_THREADS = 128;
constexpr int SK_ROWS = 64;        // output features per CTA (4 warps x 16)
constexpr int SK_KC = 512;         // k per shared-memory chunk of x
constexpr int SK_XPAD = 32;        // elements of padding per x row: rows land 64 bytes apart modulo 128

__device__ __forceinline__ uint32_t sk_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void sk_cp_async16(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(sk_smem_u32(dst)), "l"(src), "r"(sz));
}
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void sk_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NB: blocks of 8 tokens.  EPI 0: out = y.  EPI 1: w holds gate rows [0, O) and up rows [O, 2O); out = silu(g) * u.
template <int NB, int EPI, typename TO>
__global__ void __launch_bounds__(SK_THREADS)
linear_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, TO* __restrict__ out,
                     float* __restrict__ partials, int* __restrict__ counters, int n_rows, int o_out, int k_dim,
                     int splits, int k_per_split) {
  extern __shared__ __align__(16) unsigned char sk_smem[];
  bf16* xs = reinterpret_cast<bf16*>(sk_smem);                   // [NB*8][SK_KC + SK_XPAD]
  __shared__ int is_last;
  constexpr int XS = SK_KC + SK_XPAD;
  constexpr int NE = EPI ? 2 : 1;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = lane & 3, rr = lane >> 2;
  const int tile = blockIdx.x, split = blockIdx.y, n0 = blockIdx.z * (NB * 8);
  const int o0 = tile * SK_ROWS + warp * 16;
  const int kb = split * k_per_split, ke = min(k_dim, kb + k_per_split);
  // the weights are constants: ask L2 for this CTA's slice of them while the kernel before this one
  // is still finishing, then wait for it (x is its output)
  {
    const int row_bytes = (ke - kb) * 2;                                     // bytes of one weight row in this split
    const int lines = (row_bytes + 127) >> 7;
    for (int i = tid; i < (EPI ? 2 : 1) * SK_ROWS * lines; i += SK_THREADS) {
      const int e = i / (SK_ROWS * lines), r = (i / lines) % SK_ROWS, l = i % lines;
      const int o = min(tile * SK_ROWS + r, o_out - 1);
      ifb_prefetch_l2(reinterpret_cast<const char*>(w + (size_t)(e * o_out + o) * k_dim + kb) + l * 128);
    }
  }
  ifb_pdl_wait();
  ifb_pdl_trigger();
  // weight rows of this thread (clamped: rows past the end are computed and dropped)
  const bf16* wrow[NE][2];
#pragma unroll
  for (int e = 0; e < NE; ++e) {
    wrow[e][0] = w + (size_t)(e * o_out + min(o0 + rr, o_out - 1)) * k_dim;
    wrow[e][1] = w + (size_t)(e * o_out + min(o0 + rr + 8, o_out - 1)) * k_dim;
  }
  float acc[NE][NB][4];
#pragma unroll
  for (int e = 0; e < NE; ++e)
#pragma unroll
    for (int j = 0; j < NB; ++j) acc[e][j][0] = acc[e][j][1] = acc[e][j][2] = acc[e][j][3] = 0.f;

  for (int kc = kb; kc < ke; kc += SK_KC) {
    const int klen = min(SK_KC, ke - kc);
    __syncthreads();
    // x[n0 .. n0+NB*8) x [kc, kc+klen) into shared memory, zeros beyond n_rows and beyond klen
    const int chunks = (klen + 7) >> 3;
    for (int c = tid; c < NB * 8 * chunks; c += SK_THREADS) {
      const int n = c / chunks, ch = c % chunks;
      const bool valid = n0 + n < n_rows;
      sk_cp_async16(xs + n * XS + ch * 8, valid ? x + (size_t)(n0 + n) * k_dim + kc + ch * 8 : x, valid);
    }
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();
    for (int k0 = 0; k0 < klen; k0 += 128) {
      uint4 wa[NE][4], wb[NE][4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int k = k0 + c * 32 + q * 8;
        const bool in = k < klen;
#pragma unroll
        for (int e = 0; e < NE; ++e) {
          wa[e][c] = in ? ld_stream16(wrow[e][0] + kc + k) : make_uint4(0, 0, 0, 0);
          wb[e][c] = in ? ld_stream16(wrow[e][1] + kc + k) : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int k = k0 + c * 32 + q * 8;
        if (k0 + c * 32 >= klen) break;
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          uint4 xv = make_uint4(0, 0, 0, 0);
          if (k < klen) xv = *reinterpret_cast<const uint4*>(xs + (j * 8 + rr) * XS + k);
#pragma unroll
          for (int e = 0; e < NE; ++e) {
            sk_mma(acc[e][j], wa[e][c].x, wb[e][c].x, wa[e][c].y, wb[e][c].y, xv.x, xv.y);
            sk_mma(acc[e][j], wa[e][c].z, wb[e][c].z, wa[e][c].w, wb[e][c].w, xv.z, xv.w);
          }
        }
      }
    }
  }

  // acc[e][j]: c0,c1 -> (feature o0+rr, tokens n0 + j*8 + 2q, +1); c2,c3 -> feature o0+rr+8
  if (splits == 1) {
#pragma unroll
    for (int j = 0; j < NB; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int o = o0 + rr + (i >> 1) * 8, n = n0 + j * 8 + 2 * q + (i & 1);
        if (o < o_out && n < n_rows) {
          float y = acc[0][j][i];
          if (EPI) y = y / (1.f + expf(-y)) * acc[NE - 1][j][i];
          out[(size_t)n * o_out + o] = from_f32<TO>(y);
        }
      }
    return;
  }
  // partial tile to scratch: [(z, tile)][split][e][token (NB*8)][feature (64)]
  const size_t tile_id = (size_t)blockIdx.z * gridDim.x + tile;
  float* mine = partials + ((tile_id * splits + split) * NE) * (NB * 8) * SK_ROWS;
#pragma unroll
  for (int e = 0; e < NE; ++e)
#pragma unroll
    for (int j = 0; j < NB; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = warp * 16 + rr + (i >> 1) * 8, n = j * 8 + 2 * q + (i & 1);
        mine[((size_t)e * (NB * 8) + n) * SK_ROWS + m] = acc[e][j][i];
      }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&counters[tile_id], 1);
    is_last = (old == splits - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const float* base = partials + (tile_id * splits * NE) * (NB * 8) * SK_ROWS;
  for (int idx = tid; idx < NB * 8 * SK_ROWS; idx += SK_THREADS) {
    const int n = idx / SK_ROWS, m = idx % SK_ROWS;
    const int o = tile * SK_ROWS + m, tok = n0 + n;
    if (o >= o_out || tok >= n_rows) continue;
    float y[NE];
#pragma unroll
    for (int e = 0; e < NE; ++e) {
      float s = 0.f;
      for (int sp = 0; sp < splits; ++sp) s += base[(((size_t)sp * NE + e) * (NB * 8) + n) * SK_ROWS + m];
      y[e] = s;
    }
    float r = y[0];
    if (EPI) r = r / (1.f + expf(-r)) * y[NE - 1];
    out[(size_t)tok * o_out + o] = from_f32<TO>(r);
  }
  if (tid == 0) counters[tile_id] = 0;       // ready for the next launch
}

template <int NB, int EPI, typename TO>
static int sk_launch(const void* x, const void* w, void* out, float* partials, int* counters, int n, int o, int k,
                     int splits, int kps, cudaStream_t s) {
  const size_t smem = (size_t)NB * 8 * (SK_KC + SK_XPAD) * sizeof(bf16);
  IFB_ALLOW_SMEM((linear_skinny_kernel<NB, EPI, TO>), smem);
  dim3 grid((o + SK_ROWS - 1) / SK_ROWS, splits, (n + NB * 8 - 1) / (NB * 8));
  return ifb_launch(linear_skinny_kernel<NB, EPI, TO>, grid, dim3(SK_THREADS), smem, s, (const bf16*)x, (const bf16*)w,
                    (TO*)out, partials, counters, n, o, k, splits, kps);
}

template <int EPI, typename TO>
static int sk_by_n(int nb, const void* x, const void* w, void* out, float* partials, int* counters, int n, int o, int k,
                   int splits, int kps, cudaStream_t s) {
  switch (nb) {
    case 1: return sk_launch<1, EPI, TO>(x, w, out, partials, counters, n, o, k, splits, kps, s);
    case 2: return sk_launch<2, EPI, TO>(x, w, out, partials, counters, n, o, k, splits, kps, s);
    case 4: return sk_launch<4, EPI, TO>(x, w, out, partials, counters, n, o, k, splits, kps, s);
    default: return sk_launch<8, EPI, TO>(x, w, out, partials, counters, n, o, k, splits, kps, s);
  }
}

static inline int sk_blocks(int n_rows) { return n_rows <= 8 ? 1 : n_rows <= 16 ? 2 : n_rows <= 32 ? 4 : 8; }

// Scratch the call needs: floats of partial tiles and ints of counters (both 0 when splits == 1).
IFB_EXPORT void ifb_linear_skinny_scratch(int n_rows, int out_features, int epilogue, int splits, long long* floats,
                                          long long* counters) {
  const int nb = sk_blocks(n_rows);
  const long long tiles = (long long)((out_features + SK_ROWS - 1) / SK_ROWS) * ((n_rows + nb * 8 - 1) / (nb * 8));
  *floats = splits > 1 ? tiles * splits * (epilogue ? 2 : 1) * nb * 8 * SK_ROWS : 0;
  *counters = splits > 1 ? tiles : 0;
}

// x, w bfloat16; out bfloat16 or float32.  k_dim must be a multiple of 8 and the pointers 16-byte aligned.
// `counters` must be zero before the first call; every call leaves it zero.
IFB_EXPORT int ifb_linear_skinny(const void* x, const void* w, void* out, int out_dtype, float* partials, int* counters,
                                 int n_rows, int out_features, int k_dim, int epilogue, int splits,
                                 cudaStream_t stream) {
  if (n_rows <= 0 || out_features <= 0) return IFB_OK;
  if (k_dim < 8 || k_dim % 8) return IFB_ERR_SIZE;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return IFB_ERR_ALIGN;
  if (epilogue != 0 && epilogue != 1) return IFB_ERR_ARG;
  if (splits < 1 || (splits > 1 && (!partials || !counters))) return IFB_ERR_ARG;
  int kps = ((k_dim + splits - 1) / splits + 127) / 128 * 128;
  splits = (k_dim + kps - 1) / kps;             // no empty split
  const int nb = sk_blocks(n_rows);
  if ((n_rows + nb * 8 - 1) / (nb * 8) > 65535) return IFB_ERR_SIZE;
  if (out_dtype == IFB_BF16)
    return epilogue ? sk_by_n<1, bf16>(nb, x, w, out, partials, counters, n_rows, out_features, k_dim, splits, kps, stream)
                    : sk_by_n<0, bf16>(nb, x, w, out, partials, counters, n_rows, out_features, k_dim, splits, kps, stream);
  if (out_dtype == IFB_F32)
    return epilogue ? sk_by_n<1, float>(nb, x, w, out, partials, counters, n_rows, out_features, k_dim, splits, kps, stream)
                    : sk_by_n<0, float>(nb, x, w, out, partials, counters, n_rows, out_features, k_dim, splits, kps, stream);
  return IFB_ERR_DTYPE;
}
