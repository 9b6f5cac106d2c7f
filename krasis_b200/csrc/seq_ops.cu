// Ragged-batch sequence operators: the kernels a decoder needs when one step carries portions of several prompts next to single
// decoded tokens.  Every kernel works on a flat token axis [T] with per-token (sequence, position) and per-sequence
// (first row, state slot, page list) metadata, so prefill, chunked prefill, decode and any mixture run the same code.
//
//   embed_scale            x = table[token] * scale                                   (fp32 residual stream)
//   gemm_nt / gemv_nt      C = A B^T for any M, N, K; fp32 or bf16 operands, fp32 accumulation in a fixed K order per output
//   residual_norm          x += norm(y) (+ x0);  h = layer_norm(x)                    (residual update fused with the next norm)
//   residual_scale_rms     x += m y;  h = x / rms(x) * (shift + w)                    (the same for RMS norms and a residual multiplier)
//   act_mul                gelu_tanh(a) * b                                           (gated feed-forward)
//   side_gate              gelu_tanh(g) * per-layer slice of a token table            (per-layer token input)
//   latent_prep            RMS-normed latent + rotated shared key -> paged cache, rotary on the query's rotated part (any frequency
//                          table); the latent columns follow the queries or come from a buffer of their own
//   latent_window_attn     absorbed-form latent attention over the page list: sliding window, softmax with an optional per-head sink
//   conv_silu (+ state)    short causal convolution per channel over time with a carried tail, optional bias ahead of the taps or on
//                          their result, then SiLU or nothing; conv_run reads every input once on long steps
//   delta_rule             gated delta rule S <- g S; u = beta (v - S^T k); S += k u^T; o = S^T q, state in fp32 slots,
//                          unit-norm q / k, per-head RMS norm of o with a SiLU or sigmoid gate; g is one decay per head, or one
//                          per head and key channel (it then multiplies the rows of S)
//
// Precision: the residual stream, every norm, softmax, the rotary angles, decays, gates and the recurrent state are fp32 (angles
// are reduced in fp64).  `dt` codes: 0 = float32, 1 = bfloat16.
#include "seq_common.cuh"

namespace kb2seq {

thread_local char g_err[512] = "";
long long g_launches = 0;

// ------------------------------------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_scale_kernel(const T* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ x, int W,
                                   float scale) {
  const long long t = blockIdx.x;
  const long long row = tokens[t];
  for (int d = threadIdx.x; d < W; d += blockDim.x) x[t * W + d] = ldf(table, row * W + d) * scale;
}

// ------------------------------------------------------------------------------------------------ GEMM
// C[M,N] = A[M,K] * B[N,K]^T.  64x64 tile, 16-wide K steps, 4x4 outputs per thread, fp32 FMA.  Each output sums its K products
// in the same order whatever M and N are, so a row's result does not depend on which other rows share the launch.
template <typename TA, typename TB, typename TC>
__global__ void __launch_bounds__(256) gemm_nt_kernel(const TA* __restrict__ A, long long lda, const TB* __restrict__ B, long long ldb,
                                                      TC* __restrict__ C, long long ldc, int M, int N, int K, long long sA,
                                                      long long sB, long long sC) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4], Bs[BK][BN + 4];
  A += (long long)blockIdx.z * sA;
  B += (long long)blockIdx.z * sB;
  C += (long long)blockIdx.z * sC;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int i = tid + it * 256, r = i >> 4, c = i & 15;
      const int m = m0 + r, n = n0 + r, k = k0 + c;
      As[c][r] = (m < M && k < K) ? ldf(A, (long long)m * lda + k) : 0.f;
      Bs[c][r] = (n < N && k < K) ? ldf(B, (long long)n * ldb + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) stf(C, (long long)m * ldc + n, acc[i][j]);
    }
  }
}

// Few rows (decode): one warp per output column, all M <= MR rows at once, so the weight matrix is read once at full width.
template <typename TA, typename TB, typename TC, int MR>
__global__ void __launch_bounds__(256) gemv_nt_kernel(const TA* __restrict__ A, long long lda, const TB* __restrict__ B, long long ldb,
                                                      TC* __restrict__ C, long long ldc, int M, int N, int K, long long sA,
                                                      long long sB, long long sC) {
  A += (long long)blockIdx.z * sA;
  B += (long long)blockIdx.z * sB;
  C += (long long)blockIdx.z * sC;
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  float acc[MR];
#pragma unroll
  for (int m = 0; m < MR; ++m) acc[m] = 0.f;
  const TB* b = B + (long long)n * ldb;
  for (int k = lane; k < K; k += 32) {
    const float w = ldf(b, k);
#pragma unroll
    for (int m = 0; m < MR; ++m)
      if (m < M) acc[m] = fmaf(ldf(A, (long long)m * lda + k), w, acc[m]);
  }
#pragma unroll
  for (int m = 0; m < MR; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && m < M) stf(C, (long long)m * ldc + n, v);
  }
}

// streamed once: keep the weights out of L1 so that the few activation rows every warp re-reads stay there
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
template <typename TA> __device__ __forceinline__ void load8(const TA* p, float* f);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* f) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float* f) { unpack8(*reinterpret_cast<const uint4*>(p), f); }

// A warp owns CPW neighbouring output columns: the rows of A it loads (L1 hits after the first warp) serve CPW weight rows, and CPW
// 16-byte weight loads per lane are in flight at once.
template <typename TA, typename TC, int MR, int CPW, int KS>
__global__ void __launch_bounds__(256) gemv_nt_vec_kernel(const TA* __restrict__ A, long long lda, const bf16* __restrict__ B, long long ldb,
                                                          TC* __restrict__ C, long long ldc, int M, int N, int K, long long sA,
                                                          long long sB, long long sC) {
  A += (long long)blockIdx.z * sA;
  B += (long long)blockIdx.z * sB;
  C += (long long)blockIdx.z * sC;
  const int lane = threadIdx.x & 31;
  const int group = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) / KS, kpart = (threadIdx.x >> 5) % KS;
  const int n0 = group * CPW;
  if (KS == 1 && n0 >= N) return;            // with K split over warps every warp stays for the block barrier
  float acc[MR][CPW];
#pragma unroll
  for (int m = 0; m < MR; ++m)
#pragma unroll
    for (int c = 0; c < CPW; ++c) acc[m][c] = 0.f;
  // KS warps share a column group and take interleaved 256-element pieces of K; the weights of the next piece are requested before
  // the current ones are used
  const int kstep = 256 * KS;
  uint4 wv[CPW], wn[CPW];
  int k = (kpart * 32 + lane) * 8;
#pragma unroll
  for (int c = 0; c < CPW; ++c) wv[c] = (k < K && n0 + c < N) ? ld_stream16(B + (long long)(n0 + c) * ldb + k) : make_uint4(0, 0, 0, 0);
  for (; k < K; k += kstep) {
    const int kn = k + kstep;
#pragma unroll
    for (int c = 0; c < CPW; ++c) wn[c] = (kn < K && n0 + c < N) ? ld_stream16(B + (long long)(n0 + c) * ldb + kn) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int m = 0; m < MR; ++m)
      if (m < M) {
        float a[8];
        load8<TA>(A + (long long)m * lda + k, a);
#pragma unroll
        for (int c = 0; c < CPW; ++c) {
          float w[8];
          unpack8(wv[c], w);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[m][c] = fmaf(a[i], w[i], acc[m][c]);
        }
      }
#pragma unroll
    for (int c = 0; c < CPW; ++c) wv[c] = wn[c];
  }
  if constexpr (KS > 1) {
    __shared__ float red[8][MR * CPW];
    const int warp = threadIdx.x >> 5;
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
      for (int c = 0; c < CPW; ++c) {
        const float v = warp_sum(acc[m][c]);
        if (lane == 0) red[warp][m * CPW + c] = v;
      }
    __syncthreads();
    if (kpart == 0 && lane < MR * CPW) {
      const int m = lane / CPW, c = lane % CPW;
      float v = 0.f;
      for (int p = 0; p < KS; ++p) v += red[warp + p][lane];
      if (m < M && n0 + c < N) stf(C, (long long)m * ldc + n0 + c, v);
    }
    return;
  }
#pragma unroll
  for (int m = 0; m < MR; ++m)
#pragma unroll
    for (int c = 0; c < CPW; ++c) {
      const float v = warp_sum(acc[m][c]);
      if (lane == 0 && m < M && n0 + c < N) stf(C, (long long)m * ldc + n0 + c, v);
    }
}

template <typename TA, typename TC>
static bool launch_gemv_vec(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc, int M, int N, int K,
                            int batch, long long sA, long long sB, long long sC, cudaStream_t s) {
  const bool a16 = sizeof(TA) == 2;
  if (K % 8 || ldb % 8 || sB % 8 || ((uintptr_t)B & 15) || ((uintptr_t)A & 15) || lda % (a16 ? 8 : 4) || sA % (a16 ? 8 : 4)) return false;
  // columns per warp: 4 where that still leaves two blocks per SM; few columns: one per warp group, K split over 4 warps.
  // Up to 4 rows run the 4-row instantiation (half the accumulators: more blocks per SM, more weight bytes in flight).
  const long long warps = (long long)N * batch;
#define KB2_GEMV(MRV, CPWV, KSV, GX)                                                                                        \
  gemv_nt_vec_kernel<TA, TC, MRV, CPWV, KSV><<<dim3(GX, 1, batch), 256, 0, s>>>((const TA*)A, lda, (const bf16*)B, ldb, (TC*)C, ldc, M, N, K, \
                                                                                sA, sB, sC)
  if (warps >= 4 * 8 * 296) {
    if (M <= 4) KB2_GEMV(4, 4, 1, (N + 31) / 32); else KB2_GEMV(8, 4, 1, (N + 31) / 32);
  } else if (warps >= 2 * 8 * 296) {
    if (M <= 4) KB2_GEMV(4, 2, 1, (N + 15) / 16); else KB2_GEMV(8, 2, 1, (N + 15) / 16);
  } else if (K >= 2048) {
    if (M <= 4) KB2_GEMV(4, 1, 4, (N + 1) / 2); else KB2_GEMV(8, 1, 4, (N + 1) / 2);
  } else {
    if (M <= 4) KB2_GEMV(4, 1, 1, (N + 7) / 8); else KB2_GEMV(8, 1, 1, (N + 7) / 8);
  }
#undef KB2_GEMV
  return true;
}

template <typename TA, typename TB, typename TC>
static void launch_gemm(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc, int M, int N, int K,
                        int batch, long long sA, long long sB, long long sC, cudaStream_t s) {
  if (M <= 8) {
    if constexpr (sizeof(TB) == 2) {
      if (launch_gemv_vec<TA, TC>(A, lda, B, ldb, C, ldc, M, N, K, batch, sA, sB, sC, s)) return;
    }
    dim3 grid((N + 7) / 8, 1, batch);
    gemv_nt_kernel<TA, TB, TC, 8><<<grid, 256, 0, s>>>((const TA*)A, lda, (const TB*)B, ldb, (TC*)C, ldc, M, N, K, sA, sB, sC);
  } else {
    dim3 grid((N + 63) / 64, (M + 63) / 64, batch);
    gemm_nt_kernel<TA, TB, TC><<<grid, 256, 0, s>>>((const TA*)A, lda, (const TB*)B, ldb, (TC*)C, ldc, M, N, K, sA, sB, sC);
  }
}

// ------------------------------------------------------------------------------------------------ residual update + norm
// One block per token row.  x (fp32) += norm_a(y) where norm_a is a layer norm (y_mode 1: weight wa, bias ba), an RMS norm
// (y_mode 2: weight wa), the plain sum y + y2 (y_mode 3: two sublayers that read the same normed input; y2 may be null) or absent
// (y == nullptr); x += x0 if given; then h = layer_norm(x; wb, bb) if h is given (bb == nullptr: no bias).
// Variances are means of squared deviations (two passes over the row held in shared memory).
__global__ void __launch_bounds__(256) residual_norm_kernel(float* __restrict__ x, const float* __restrict__ y, int y_mode,
                                                            const float* __restrict__ wa, const float* __restrict__ ba,
                                                            const float* __restrict__ x0, const float* __restrict__ wb,
                                                            const float* __restrict__ bb, void* __restrict__ h, int dt_h, int W,
                                                            float eps, const float* __restrict__ y2) {
  extern __shared__ float rowbuf[];
  __shared__ float red[32];
  const long long row = blockIdx.x;
  float* xr = x + row * W;
  const float inv_w = 1.f / (float)W;
  if (y != nullptr) {
    const float* yr = y + row * W;
    float s = 0.f;
    for (int d = threadIdx.x; d < W; d += blockDim.x) {
      const float v = yr[d];
      rowbuf[d] = v;
      s += y_mode == 1 ? v : v * v;
    }
    s = block_sum(s, red);
    float mean = 0.f, rstd;
    if (y_mode == 3) {
      for (int d = threadIdx.x; d < W; d += blockDim.x) {
        float v = rowbuf[d];
        if (y2 != nullptr) v += y2[row * W + d];
        v += xr[d];
        if (x0 != nullptr) v += x0[row * W + d];
        xr[d] = v;
        rowbuf[d] = v;
      }
      rstd = 0.f;
    } else if (y_mode == 1) {
      mean = s * inv_w;
      float q = 0.f;
      for (int d = threadIdx.x; d < W; d += blockDim.x) {
        const float c = rowbuf[d] - mean;
        q += c * c;
      }
      q = block_sum(q, red);
      rstd = 1.f / sqrtf(q * inv_w + eps);
    } else {
      rstd = 1.f / sqrtf(s * inv_w + eps);
    }
    for (int d = threadIdx.x; y_mode != 3 && d < W; d += blockDim.x) {
      float v = (rowbuf[d] - mean) * rstd * wa[d];
      if (y_mode == 1) v += ba[d];
      v += xr[d];
      if (x0 != nullptr) v += x0[row * W + d];
      xr[d] = v;
      rowbuf[d] = v;
    }
  } else {
    for (int d = threadIdx.x; d < W; d += blockDim.x) {
      float v = xr[d];
      if (x0 != nullptr) {
        v += x0[row * W + d];
        xr[d] = v;
      }
      rowbuf[d] = v;
    }
  }
  if (h == nullptr) return;
  float s = 0.f;
  for (int d = threadIdx.x; d < W; d += blockDim.x) s += rowbuf[d];
  const float mean = block_sum(s, red) * inv_w;
  float q = 0.f;
  for (int d = threadIdx.x; d < W; d += blockDim.x) {
    const float c = rowbuf[d] - mean;
    q += c * c;
  }
  q = block_sum(q, red);
  const float rstd = 1.f / sqrtf(q * inv_w + eps);
  for (int d = threadIdx.x; d < W; d += blockDim.x) st_dt(h, dt_h, row * W + d, (rowbuf[d] - mean) * rstd * wb[d] + (bb != nullptr ? bb[d] : 0.f));
}

// One block per token row.  x (fp32) += y_mult * y (y may be null); then h = x / sqrt(mean(x^2) + eps) * (w_shift + w) if h is given
// (w_shift 1: w holds the offset from one).  h may be x itself when y is null and dt_h is fp32 (a norm in place).
__global__ void __launch_bounds__(256) residual_scale_rms_kernel(float* x, const float* __restrict__ y, float y_mult,
                                                                 const float* __restrict__ w, float w_shift, void* h, int dt_h, int W,
                                                                 float eps) {
  extern __shared__ float rowbuf[];
  __shared__ float red[32];
  const long long row = blockIdx.x;
  float* xr = x + row * W;
  float s = 0.f;
  for (int d = threadIdx.x; d < W; d += blockDim.x) {
    float v = xr[d];
    if (y != nullptr) {
      v = fmaf(y_mult, y[row * W + d], v);
      xr[d] = v;
    }
    rowbuf[d] = v;
    s = fmaf(v, v, s);
  }
  if (h == nullptr) return;
  s = block_sum(s, red);
  const float rstd = 1.f / sqrtf(s / (float)W + eps);
  for (int d = threadIdx.x; d < W; d += blockDim.x) st_dt(h, dt_h, row * W + d, rowbuf[d] * rstd * (w_shift + w[d]));
}

// ------------------------------------------------------------------------------------------------ elementwise
__global__ void act_mul_kernel(const void* __restrict__ in, int dt_in, void* __restrict__ out, int dt_out, long long T, int F) {
  const long long t = blockIdx.y;
  const int f = blockIdx.x * blockDim.x + threadIdx.x;
  if (f >= F) return;
  const float a = ld_dt(in, dt_in, t * 2 * F + f), b = ld_dt(in, dt_in, t * 2 * F + F + f);
  st_dt(out, dt_out, t * F + f, gelu_tanh(a) * b);
}
// bf16 in and out, F a multiple of 8: 16-byte accesses
__global__ void act_mul_bf16x8_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int F) {
  const long long t = blockIdx.y;
  const int f = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (f >= F) return;
  float a[8], b[8];
  unpack8(*reinterpret_cast<const uint4*>(in + t * 2 * F + f), a);
  unpack8(*reinterpret_cast<const uint4*>(in + t * 2 * F + F + f), b);
  uint4 o;
  __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(gelu_tanh(a[2 * i]) * b[2 * i], gelu_tanh(a[2 * i + 1]) * b[2 * i + 1]);
  *reinterpret_cast<uint4*>(out + t * F + f) = o;
}

__global__ void side_gate_kernel(const float* __restrict__ g, const void* __restrict__ table, int dt_table, long long table_ld,
                                 const int* __restrict__ tokens, int col0, int dim, long long T, void* __restrict__ out, int dt_out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * dim) return;
  const long long t = i / dim;
  const int d = (int)(i - t * dim);
  const float e = ld_dt(table, dt_table, (long long)tokens[t] * table_ld + col0 + d);
  st_dt(out, dt_out, i, gelu_tanh(g[i]) * e);
}

// ------------------------------------------------------------------------------------------------ latent attention
// proj [T, ldp] fp32 = [q (H x (dn + dr)) | latent (r) | shared rotated key (dr)].  Per token: RMS-normed latent and rotated key part
// go to the page the token's position maps to; the query's rotated parts are rotated in place.
__global__ void __launch_bounds__(128) latent_prep_kernel(float* __restrict__ proj, long long ldp, int H, int dn, int dr, int r,
                                                          const float* __restrict__ cw, float eps, const double* __restrict__ freq,
                                                          int rot_dims, float amp, const int* __restrict__ positions,
                                                          const int* __restrict__ seq_of, const int* __restrict__ pages, int max_pages,
                                                          int page_size, void* __restrict__ ckv, void* __restrict__ kr, int dt_cache,
                                                          const float* __restrict__ lat_rows, long long ldl) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const int pos = positions[t];
  float* p = proj + t * ldp;
  const long long slot = (long long)pages[(long long)seq_of[t] * max_pages + pos / page_size] * page_size + pos % page_size;
  const float* lat = lat_rows != nullptr ? lat_rows + t * ldl : p + (long long)H * (dn + dr);
  float ss = 0.f;
  for (int d = threadIdx.x; d < r; d += blockDim.x) ss += lat[d] * lat[d];
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)r + eps);
  for (int d = threadIdx.x; d < r; d += blockDim.x) st_dt(ckv, dt_cache, slot * r + d, lat[d] * rstd * cw[d]);
  const int half = rot_dims / 2;
  // (H + 1) vectors of dr: the heads' query parts (in place) and the shared key part (to the cache)
  for (int i = threadIdx.x; i < (H + 1) * half; i += blockDim.x) {
    const int hh = i / half, j = i - hh * half;
    float c, s;
    rot_cs(pos, freq[j], amp, &c, &s);
    if (hh < H) {
      float* q = p + (long long)hh * (dn + dr) + dn;
      const float u = q[2 * j], v = q[2 * j + 1];
      q[2 * j] = u * c - v * s;
      q[2 * j + 1] = v * c + u * s;
    } else {
      const float* k = lat + r;
      const float u = k[2 * j], v = k[2 * j + 1];
      st_dt(kr, dt_cache, slot * dr + 2 * j, u * c - v * s);
      st_dt(kr, dt_cache, slot * dr + 2 * j + 1, v * c + u * s);
    }
  }
  for (int d = rot_dims + threadIdx.x; d < dr; d += blockDim.x) st_dt(kr, dt_cache, slot * dr + d, lat[r + d]);
}

// Absorbed form: score(t, h, j) = (q_abs[t,h] . c_j + q_rot[t,h] . kr_j) * scale over the keys j of the token's sequence with
// 0 <= pos - j < window; the softmax denominator also holds exp(sink_h) (a key with no value: running max starts at the sink,
// running sum at 1).  Output: sum_j p_j c_j (the value up-projection follows as a per-head GEMM).
// One block per (token, group of HG heads); keys in tiles of KT, shared by the heads of the group.
constexpr int kAttnThreads = 256, kAttnAcc = 16;
__global__ void __launch_bounds__(kAttnThreads) latent_window_attn_kernel(
    const float* __restrict__ q_abs, const float* __restrict__ proj, long long ldp, int H, int HG, int dn, int dr, int r,
    const void* __restrict__ ckv, const void* __restrict__ kr, int dt_cache, const int* __restrict__ positions,
    const int* __restrict__ seq_of, const int* __restrict__ pages, int max_pages, int page_size, const float* __restrict__ sinks,
    float scale, int window, int KT, float* __restrict__ out, const int* __restrict__ cu, int skip_from, int nsplit,
    float* __restrict__ part_acc, float* __restrict__ part_ml) {
  extern __shared__ __align__(16) float sm[];
  if (cu != nullptr) {                    // sequences whose portion has skip_from tokens or more are served by another kernel
    const int sq = seq_of[blockIdx.x];
    if (cu[sq + 1] - cu[sq] >= skip_from) return;
  }
  const int D = r + dr, DP = D + 1;
  long long* krow = (long long*)sm;       // [KT] cache rows of the tile's keys
  float* qs = sm + 2 * KT;                // [HG][D]
  float* kt = qs + HG * D;                // [KT][DP]
  float* pr = kt + KT * DP;               // [HG][KT]
  float* sp = pr + HG * KT;               // [warps][KT] partial scores: a head's dot product is cut into warps / HG pieces
  float* m_run = sp + (kAttnThreads / 32) * KT;   // [HG]
  float* l_run = m_run + HG;              // [HG]
  float* alpha = l_run + HG;              // [HG]
  const long long t = blockIdx.x;
  const int h0 = blockIdx.y * HG;
  const int nh = min(HG, H - h0);
  const int pos = positions[t], seq = seq_of[t];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < nh * D; i += kAttnThreads) {
    const int hh = i / D, d = i - hh * D;
    qs[i] = d < r ? q_abs[(t * H + h0 + hh) * r + d] : proj[t * ldp + (long long)(h0 + hh) * (dn + dr) + dn + (d - r)];
  }
  // nsplit > 1: block z takes the z-th piece of the token's key range and leaves an unnormalised partial result (running max, sum,
  // weighted latents) for latent_attn_combine_kernel; the sink belongs to piece 0
  const int z = blockIdx.z;
  if (tid < nh) {
    const bool sk = z == 0 && sinks != nullptr;       // no sinks: an ordinary softmax over the keys
    m_run[tid] = sk ? sinks[h0 + tid] : -INFINITY;
    l_run[tid] = sk ? 1.f : 0.f;
  }
  float acc[kAttnAcc];
#pragma unroll
  for (int a = 0; a < kAttnAcc; ++a) acc[a] = 0.f;
  const int j_lo = max(0, pos - window + 1);
  int j_begin = j_lo, j_end = pos;
  if (nsplit > 1) {
    const int piece = (((pos - j_lo + 1) + nsplit - 1) / nsplit + KT - 1) / KT * KT;
    j_begin = j_lo + z * piece;
    j_end = min(pos, j_begin + piece - 1);
  }
  for (int j0 = j_begin; j0 <= j_end; j0 += KT) {
    const int nk = min(KT, j_end - j0 + 1);
    __syncthreads();
    if (tid < nk) {
      const int j = j0 + tid;
      krow[tid] = (long long)pages[(long long)seq * max_pages + j / page_size] * page_size + j % page_size;
    }
    __syncthreads();
    if (dt_cache == 1 && (r & 7) == 0 && (dr & 7) == 0) {
      const int D8 = D >> 3;
      for (int i = tid; i < nk * D8; i += kAttnThreads) {
        const int k = i / D8, d = (i - k * D8) << 3;
        const bf16* src = d < r ? (const bf16*)ckv + krow[k] * r + d : (const bf16*)kr + krow[k] * dr + (d - r);
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(src), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) kt[k * DP + d + e] = f[e];
      }
    } else {
      for (int i = tid; i < nk * D; i += kAttnThreads) {
        const int k = i / D, d = i - k * D;
        kt[k * DP + d] = d < r ? ld_dt(ckv, dt_cache, krow[k] * r + d) : ld_dt(kr, dt_cache, krow[k] * dr + (d - r));
      }
    }
    __syncthreads();
    // scores: warp w takes piece w / HG of head w % HG, a lane per key (HG is a power of two <= 8, KT == 32)
    {
      const int P = (kAttnThreads / 32) / HG, part = warp / HG, hw = warp % HG;
      const int dseg = (D + P - 1) / P, d_lo = part * dseg, d_hi = min(D, d_lo + dseg);
      float dot = 0.f;
      if (hw < nh && lane < nk) {
        const float* qh = qs + hw * D;
        const float* kk = kt + lane * DP;
        for (int d = d_lo; d < d_hi; ++d) dot = fmaf(qh[d], kk[d], dot);
      }
      sp[warp * KT + lane] = dot;
    }
    __syncthreads();
    // running softmax: warp hh < nh
    for (int hh = warp; hh < nh; hh += kAttnThreads / 32) {
      const float m_old = m_run[hh];
      float m_new = m_old;
      {
        const int P = (kAttnThreads / 32) / HG;
        float sc = -INFINITY;
        if (lane < nk) {
          float dot = 0.f;
          for (int pp = 0; pp < P; ++pp) dot += sp[(pp * HG + hh) * KT + lane];
          sc = dot * scale;
        }
        pr[hh * KT + lane] = sc;
        m_new = fmaxf(m_new, warp_max(sc));
      }
      float lsum = 0.f;
      for (int kb = 0; kb < nk; kb += 32) {
        const int k = kb + lane;
        float p = 0.f;
        if (k < nk) {
          p = expf(pr[hh * KT + k] - m_new);
          pr[hh * KT + k] = p;
        }
        lsum += warp_sum(p);
      }
      if (lane == 0) {
        const float al = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
        alpha[hh] = al;
        l_run[hh] = l_run[hh] * al + lsum;
        m_run[hh] = m_new;
      }
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < kAttnAcc; ++a) {
      const int i = tid + a * kAttnThreads;
      if (i < nh * r) {
        const int hh = i / r, d = i - hh * r;
        float v = acc[a] * alpha[hh];
        const float* ph = pr + hh * KT;
        for (int k = 0; k < nk; ++k) v = fmaf(ph[k], kt[k * DP + d], v);
        acc[a] = v;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int a = 0; a < kAttnAcc; ++a) {
    const int i = tid + a * kAttnThreads;
    if (i < nh * r) {
      const int hh = i / r, d = i - hh * r;
      if (nsplit > 1) part_acc[((t * nsplit + z) * H + h0 + hh) * r + d] = acc[a];
      else out[(t * H + h0 + hh) * r + d] = acc[a] / l_run[hh];
    }
  }
  if (nsplit > 1 && tid < nh) {
    part_ml[((t * nsplit + z) * H + h0 + tid) * 2] = m_run[tid];
    part_ml[((t * nsplit + z) * H + h0 + tid) * 2 + 1] = l_run[tid];
  }
}

// out[t, h, :] = sum_z w_z acc_z / sum_z w_z l_z with w_z = exp(m_z - max_z m_z); pieces without keys have l_z = 0
__global__ void __launch_bounds__(128) latent_attn_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                                                  int H, int r, int nsplit, float* __restrict__ out,
                                                                  const int* __restrict__ seq_of, const int* __restrict__ cu, int skip_from) {
  const long long t = blockIdx.x;
  const int h = blockIdx.y;
  if (cu != nullptr) {
    const int sq = seq_of[t];
    if (cu[sq + 1] - cu[sq] >= skip_from) return;
  }
  float M = -INFINITY;
  for (int zz = 0; zz < nsplit; ++zz) {
    const float* ml = part_ml + ((t * nsplit + zz) * H + h) * 2;
    if (ml[1] > 0.f) M = fmaxf(M, ml[0]);
  }
  float L = 0.f;
  for (int zz = 0; zz < nsplit; ++zz) {
    const float* ml = part_ml + ((t * nsplit + zz) * H + h) * 2;
    if (ml[1] > 0.f) L += ml[1] * expf(ml[0] - M);
  }
  for (int d = threadIdx.x; d < r; d += blockDim.x) {
    float v = 0.f;
    for (int zz = 0; zz < nsplit; ++zz) {
      const float* ml = part_ml + ((t * nsplit + zz) * H + h) * 2;
      if (ml[1] > 0.f) v = fmaf(part_acc[((t * nsplit + zz) * H + h) * r + d], expf(ml[0] - M), v);
    }
    out[(t * H + h) * r + d] = v / L;
  }
}

// ------------------------------------------------------------------------------------------------ short convolution + delta rule
// y[t, c] = act(sum_j taps[c, j] * x[i - (K - 1) + j, c]) with i the token's index in its portion and x = proj + bias (bias may be null);
// act 1: silu, 0: none.  Inputs before the portion come from the sequence's carried tail (the last K - 1 inputs of earlier portions,
// bias included; zeros at the start of a sequence).
__global__ void conv_silu_kernel(const float* __restrict__ proj, long long ldp, int C, int K, const float* __restrict__ taps,
                                 const float* __restrict__ tail, const int* __restrict__ seq_of, const int* __restrict__ cu,
                                 const int* __restrict__ slots, long long T, float* __restrict__ out, const float* __restrict__ bias,
                                 int act, int bias_after) {
  const long long t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const long long idx = t * C + c;
  const int s = seq_of[t];
  const int i = (int)(t - cu[s]);
  const float* tl = tail + ((long long)slots[s] * C + c) * (K - 1);
  const float bv = bias != nullptr ? bias[c] : 0.f;
  const float b = bias_after ? 0.f : bv;       // bias_after: the bias joins the convolution's result, not its inputs
  float acc = bias_after ? bv : 0.f;
  for (int j = 0; j < K; ++j) {
    const int src = i - (K - 1) + j;
    const float xv = src >= 0 ? proj[(t - i + src) * ldp + c] + b : tl[(K - 1) + src];
    acc = fmaf(taps[(long long)c * K + j], xv, acc);
  }
  out[idx] = act ? silu(acc) : acc;
}

// The same for long steps and K <= kConvMaxTaps: a thread owns a channel over kConvRun consecutive rows and keeps the last K inputs in
// registers, so that every input is read once (plus K - 1 rows of overlap per run) instead of K times.
constexpr int kConvMaxTaps = 8, kConvRun = 16;
__global__ void __launch_bounds__(256) conv_run_kernel(const float* __restrict__ proj, long long ldp, int C, int K,
                                                       const float* __restrict__ taps, const float* __restrict__ tail,
                                                       const int* __restrict__ seq_of, const int* __restrict__ cu,
                                                       const int* __restrict__ slots, long long T, float* __restrict__ out,
                                                       const float* __restrict__ bias, int act, int bias_after) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const long long r0 = (long long)blockIdx.y * kConvRun, r1 = min(T, r0 + kConvRun);
  float w[kConvMaxTaps], x[kConvMaxTaps] = {};     // x[j]: the input K - 1 - j rows back, x[K - 1] the current one
#pragma unroll
  for (int j = 0; j < kConvMaxTaps; ++j) w[j] = j < K ? taps[(long long)c * K + j] : 0.f;
  const float bv = bias != nullptr ? bias[c] : 0.f;
  const float b = bias_after ? 0.f : bv, b_out = bias_after ? bv : 0.f;
  int s = -1;
  for (long long t = r0; t < r1; ++t) {
    const int st = seq_of[t];
    if (st != s || t == r0) {                        // first row of this run, or of another sequence: fetch the K - 1 earlier inputs
      s = st;
      const int i = (int)(t - cu[s]);
      const float* tl = tail + ((long long)slots[s] * C + c) * (K - 1);
#pragma unroll
      for (int j = 0; j < kConvMaxTaps - 1; ++j)
        if (j < K - 1) {
          const int src = i - (K - 1) + j;
          x[j + 1] = src >= 0 ? proj[(t - i + src) * ldp + c] + b : tl[(K - 1) + src];
        }
    }
#pragma unroll
    for (int j = 0; j < kConvMaxTaps - 1; ++j) x[j] = x[j + 1];
    // after the shift x[0 .. K - 2] hold the K - 1 earlier inputs; the current one goes to x[K - 1]
    const float cur = proj[t * ldp + c] + b;
    float acc = b_out;
#pragma unroll
    for (int j = 0; j < kConvMaxTaps; ++j) {
      if (j == K - 1) x[j] = cur;
      if (j < K) acc = fmaf(w[j], x[j], acc);
    }
    out[t * C + c] = act ? silu(acc) : acc;
  }
}

// after the convolution: the tail becomes the last K - 1 inputs seen so far (one thread per (sequence, channel), ascending order)
__global__ void conv_tail_kernel(const float* __restrict__ proj, long long ldp, int C, int K, float* __restrict__ tail,
                                 const int* __restrict__ cu, const int* __restrict__ slots, int S, const float* __restrict__ bias) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)S * C) return;
  const int s = (int)(idx / C), c = (int)(idx - (long long)s * C);
  const int t0 = cu[s], n = cu[s + 1] - cu[s];
  float* tl = tail + ((long long)slots[s] * C + c) * (K - 1);
  const float b = bias != nullptr ? bias[c] : 0.f;
  for (int j = 0; j < K - 1; ++j) {
    const int src = n - (K - 1) + j;         // index in the portion of the input that lands in tail[j]
    tl[j] = src >= 0 ? proj[(long long)(t0 + src) * ldp + c] + b : tl[j + n];
  }
}

// One block per (sequence, head); thread j owns column j of the head's state S [dk][dv] (kept in shared memory for the portion).
// conv [T, C] = silu(conv(q | k | v)); proj holds the gate (g_off), the decay input (a_off) and the write-strength input (b_off).
// ch 0: one decay per (token, head), from a[t, h] and dt_bias[h].  ch 1: one per (token, head, key channel), from a[t, h dk + i] and
// dt_bias[h dk + i]; it multiplies the rows of the state.  gate_act 0: silu(gate), 1: sigmoid(gate).
constexpr int kDeltaTile = 16;
__global__ void __launch_bounds__(1024) delta_rule_kernel(const float* __restrict__ conv, int C, const float* __restrict__ bproj,
                                                          long long ldb, const float* __restrict__ aproj, long long lda, int ch,
                                                          const float* __restrict__ gproj, long long ldg, int gate_act, int H, int Hk,
                                                          int dk, int dv, const float* __restrict__ A_log,
                                                          const float* __restrict__ dt_bias, const float* __restrict__ norm_w, float eps,
                                                          float* __restrict__ state, const int* __restrict__ cu,
                                                          const int* __restrict__ slots, void* __restrict__ out, int dt_out, int dvb,
                                                          float* __restrict__ o_raw) {
  // dvb = value columns of this block (the columns of the state do not meet in the recurrence).  dvb < dv: blockIdx.z picks the slice,
  // the raw read-out goes to o_raw [T, H, dv] and the norm and gate are left to delta_out_kernel.
  extern __shared__ float sm[];
  float* S = sm;                                  // [dk][dvb]
  float* qn = S + (long long)dk * dvb;            // [tile][dk]
  float* kn = qn + kDeltaTile * dk;               // [tile][dk]
  float* ob = kn + kDeltaTile * dk;               // [tile][dvb]
  float* beta = ob + kDeltaTile * dvb;            // [tile]
  float* dec = beta + kDeltaTile;                 // [tile] or [tile][dk]
  const int dstr = ch ? dk : 1;
  const int s = blockIdx.x, h = blockIdx.y, hk = h / (H / Hk);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  const int t0 = cu[s], n = cu[s + 1] - cu[s];
  const int col0 = blockIdx.z * dvb, nc = min(dvb, dv - col0);
  float* Sg = state + ((long long)slots[s] * H + h) * dk * dv + col0;
  for (int i = tid; i < dk * nc; i += blockDim.x) S[(i / nc) * dvb + i % nc] = Sg[(long long)(i / nc) * dv + i % nc];
  const double rate_h = exp((double)A_log[h]);
  const float qscale = 1.f / sqrtf((float)dk);
  const int q_col = hk * dk, k_col = Hk * dk + hk * dk, v_col = 2 * Hk * dk + h * dv;
  for (int b0 = 0; b0 < n; b0 += kDeltaTile) {
    const int nt = min(kDeltaTile, n - b0);
    __syncthreads();
    for (int tt = warp; tt < nt; tt += nw) {
      const float* row = conv + (long long)(t0 + b0 + tt) * C;
      float sq = 0.f, sk = 0.f;
      for (int i = lane; i < dk; i += 32) {
        const float qv = row[q_col + i], kv = row[k_col + i];
        sq += qv * qv;
        sk += kv * kv;
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      const float rq = qscale / sqrtf(sq + 1e-6f), rk = 1.f / sqrtf(sk + 1e-6f);
      for (int i = lane; i < dk; i += 32) {
        qn[tt * dk + i] = row[q_col + i] * rq;
        kn[tt * dk + i] = row[k_col + i] * rk;
      }
      const float* ar = aproj + (long long)(t0 + b0 + tt) * lda + (long long)h * dstr;
      for (int i = lane; i < dstr; i += 32) dec[tt * dstr + i] = decay_from_rate(rate_h, ar[i], dt_bias[h * dstr + i]);
      if (lane == 0) beta[tt] = 1.f / (1.f + expf(-bproj[(long long)(t0 + b0 + tt) * ldb + h]));
    }
    __syncthreads();
    if (tid < nc) {
      for (int tt = 0; tt < nt; ++tt) {
        const float* gg = dec + tt * dstr;
        const float* kk = kn + tt * dk;
        const float* qq = qn + tt * dk;
        float sk = 0.f;
        for (int i = 0; i < dk; ++i) {
          const float sv = S[i * dvb + tid] * gg[ch ? i : 0];
          S[i * dvb + tid] = sv;
          sk = fmaf(sv, kk[i], sk);
        }
        const float u = beta[tt] * (conv[(long long)(t0 + b0 + tt) * C + v_col + col0 + tid] - sk);
        float o = 0.f;
        for (int i = 0; i < dk; ++i) {
          const float sv = fmaf(kk[i], u, S[i * dvb + tid]);
          S[i * dvb + tid] = sv;
          o = fmaf(sv, qq[i], o);
        }
        if (o_raw != nullptr) o_raw[((long long)(t0 + b0 + tt) * H + h) * dv + col0 + tid] = o;
        else ob[tt * dvb + tid] = o;
      }
    }
    __syncthreads();
    for (int tt = warp; o_raw == nullptr && tt < nt; tt += nw) {
      float ss = 0.f;
      for (int j = lane; j < dv; j += 32) ss += ob[tt * dv + j] * ob[tt * dv + j];
      ss = warp_sum(ss);
      const float rstd = 1.f / sqrtf(ss / (float)dv + eps);
      const long long t = t0 + b0 + tt;
      for (int j = lane; j < dv; j += 32) {
        const float gz = gproj[t * ldg + h * dv + j];
        st_dt(out, dt_out, (t * H + h) * dv + j, ob[tt * dv + j] * rstd * norm_w[j] * (gate_act ? 1.f / (1.f + expf(-gz)) : silu(gz)));
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < dk * nc; i += blockDim.x) Sg[(long long)(i / nc) * dv + i % nc] = S[(i / nc) * dvb + i % nc];
}


// ---- the same recurrence for key sizes 32 / 64 / 128 and value sizes that are multiples of 32: state in registers.
// delta_prep: unit-norm q (times dk^-1/2) and k per (token, key head), write strength and decay per (token, head), all tokens in
// parallel.  delta_rule_reg: one block per (sequence, head, 32 value columns); lane = column, warp p holds rows [p DK/8, (p+1) DK/8) of
// the state in registers, so the k and q values a warp needs are the same for all its lanes (one shared-memory transaction per 16
// bytes); the pieces of S^T k meet through shared memory and one block barrier per token, those of S^T q once per 8 tokens; q / k / v /
// gates of the next 8 tokens stream into shared memory with cp.async while the current 8 are processed.  delta_out: per-head RMS norm and SiLU gate.
__global__ void __launch_bounds__(256) delta_prep_kernel(const float* __restrict__ conv, int C, const float* __restrict__ bproj,
                                                         long long ldb, const float* __restrict__ aproj, long long lda, int ch, int H,
                                                         int Hk, int dk, const float* __restrict__ A_log,
                                                         const float* __restrict__ dt_bias, long long T, float* __restrict__ qn,
                                                         float* __restrict__ kn, float* __restrict__ beta, float* __restrict__ dec) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= T * Hk) return;
  const long long t = w / Hk;
  const int hk = (int)(w - t * Hk);
  const float* row = conv + t * C;
  const int q_col = hk * dk, k_col = Hk * dk + hk * dk;
  float sq = 0.f, sk = 0.f;
  for (int i = lane; i < dk; i += 32) {
    const float qv = row[q_col + i], kv = row[k_col + i];
    sq += qv * qv;
    sk += kv * kv;
  }
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  const float rq = (1.f / sqrtf((float)dk)) / sqrtf(sq + 1e-6f), rk = 1.f / sqrtf(sk + 1e-6f);
  for (int i = lane; i < dk; i += 32) {
    qn[w * dk + i] = row[q_col + i] * rq;
    kn[w * dk + i] = row[k_col + i] * rk;
  }
  const int rep = H / Hk;
  for (int j = lane; j < rep; j += 32) {
    const int h = hk * rep + j;
    beta[t * H + h] = 1.f / (1.f + expf(-bproj[t * ldb + h]));
    if (!ch) dec[t * H + h] = decay_of(A_log[h], aproj[t * lda + h], dt_bias[h]);
  }
  if (ch)                                    // one decay per key channel of each of this key head's heads: dec [T][H][dk]
    for (int j = 0; j < rep; ++j) {
      const int h = hk * rep + j;
      const double rate = exp((double)A_log[h]);
      for (int i = lane; i < dk; i += 32) {
        const long long c = (long long)h * dk + i;
        dec[t * H * dk + c] = decay_from_rate(rate, aproj[t * lda + c], dt_bias[c]);
      }
    }
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

constexpr int kRegTile = 8;
constexpr int kRegPieces = 8;                // warps of a block (the sum of the pieces below is written for 8): warp p holds rows [p DK/8, (p+1) DK/8) of 32 state columns
template <int DK, bool CH>
__global__ void __launch_bounds__(32 * kRegPieces) delta_rule_reg_kernel(const float* __restrict__ qn, const float* __restrict__ kn,
                                                                         const float* __restrict__ conv, int C, int v_col0,
                                                                         const float* __restrict__ beta, const float* __restrict__ dec,
                                                                         int H, int Hk, int dv, float* __restrict__ state,
                                                                         const int* __restrict__ cu, const int* __restrict__ slots,
                                                                         float* __restrict__ o_out) {
  constexpr int P = kRegPieces, NT = 32 * P;
  constexpr int Q = DK / P;                 // state rows per thread
  __shared__ __align__(16) float ks[2][kRegTile][DK];
  __shared__ __align__(16) float qs[2][kRegTile][DK];
  __shared__ __align__(16) float vs[2][kRegTile][32];
  __shared__ float bs[2][kRegTile], gs[2][kRegTile];
  __shared__ __align__(16) float gc[CH ? 2 : 1][CH ? kRegTile : 1][CH ? DK : 4];   // per-channel decays of the tile's tokens
  __shared__ float part[2][P][32];          // per token: the pieces of S^T k, summed by every warp after one barrier
  __shared__ float os_part[kRegTile][P][32];   // pieces of S^T q, summed once per tile
  const int s = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * 32;
  const int hk = h / (H / Hk);
  const int tid = threadIdx.x, lane = tid & 31, piece = tid >> 5;
  const int t0 = cu[s], n = cu[s + 1] - cu[s];
  float* Sg = state + ((long long)slots[s] * H + h) * DK * dv;
  float S[Q];
#pragma unroll
  for (int ii = 0; ii < Q; ++ii) S[ii] = Sg[(long long)(piece * Q + ii) * dv + j0 + lane];

  auto load_tile = [&](int buf, int b0) {
    const int nt = min(kRegTile, n - b0);
    for (int c = tid; c < nt * (DK / 4); c += NT) {                  // 16-byte chunks of the q and k rows
      const int tt = c / (DK / 4), cc = c - tt * (DK / 4);
      const long long src = ((long long)(t0 + b0 + tt) * Hk + hk) * DK + cc * 4;
      cp_async16(&ks[buf][tt][cc * 4], kn + src);
      cp_async16(&qs[buf][tt][cc * 4], qn + src);
      if (CH) cp_async16(&gc[CH ? buf : 0][CH ? tt : 0][cc * 4], dec + ((long long)(t0 + b0 + tt) * H + h) * DK + cc * 4);
    }
    for (int c = tid; c < nt * 8; c += NT) {
      const int tt = c >> 3, cc = c & 7;
      cp_async16(&vs[buf][tt][cc * 4], conv + (long long)(t0 + b0 + tt) * C + v_col0 + h * dv + j0 + cc * 4);
    }
    if (tid < nt) {
      cp_async4(&bs[buf][tid], beta + (long long)(t0 + b0 + tid) * H + h);
      if (!CH) cp_async4(&gs[buf][tid], dec + (long long)(t0 + b0 + tid) * H + h);
    }
    cp_async_commit();
  };

  load_tile(0, 0);
  int buf = 0;
  for (int b0 = 0; b0 < n; b0 += kRegTile, buf ^= 1) {
    const int nt = min(kRegTile, n - b0);
    cp_async_wait_all();
    __syncthreads();                                  // tile `buf` is in place; everyone is done with the other buffer and with os_part
    if (b0 + kRegTile < n) load_tile(buf ^ 1, b0 + kRegTile);
    for (int tt = 0; tt < nt; ++tt) {
      const float g = CH ? 1.f : gs[buf][tt], b = bs[buf][tt];
      // the same address for every lane: one shared-memory transaction per 16 bytes.  All of the token's k and q values are fetched
      // up front (the loads are in flight together, none has to wait behind the barrier below)
      const float4* k4 = reinterpret_cast<const float4*>(&ks[buf][tt][piece * Q]);
      const float4* q4 = reinterpret_cast<const float4*>(&qs[buf][tt][piece * Q]);
      float4 kr[Q / 4], qr[Q / 4];
#pragma unroll
      for (int ii = 0; ii < Q / 4; ++ii) kr[ii] = k4[ii];
#pragma unroll
      for (int ii = 0; ii < Q / 4; ++ii) qr[ii] = q4[ii];
      const float vv = vs[buf][tt][lane];
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      if (CH) {                               // the rows of the state decay each by its own factor before anything reads them
        const float4* g4 = reinterpret_cast<const float4*>(&gc[CH ? buf : 0][CH ? tt : 0][piece * Q]);
#pragma unroll
        for (int ii = 0; ii < Q / 4; ++ii) {
          const float4 gr = g4[ii];
          S[4 * ii] *= gr.x;
          S[4 * ii + 1] *= gr.y;
          S[4 * ii + 2] *= gr.z;
          S[4 * ii + 3] *= gr.w;
        }
      }
#pragma unroll
      for (int ii = 0; ii < Q / 4; ++ii) {
        a0 = fmaf(S[4 * ii], kr[ii].x, a0);
        a1 = fmaf(S[4 * ii + 1], kr[ii].y, a1);
        a2 = fmaf(S[4 * ii + 2], kr[ii].z, a2);
        a3 = fmaf(S[4 * ii + 3], kr[ii].w, a3);
      }
      part[tt & 1][piece][lane] = (a0 + a1) + (a2 + a3);
      __syncthreads();
      float pp[P];
#pragma unroll
      for (int p = 0; p < P; ++p) pp[p] = part[tt & 1][p][lane];
      const float sk = ((pp[0] + pp[1]) + (pp[2] + pp[3])) + ((pp[4] + pp[5]) + (pp[6] + pp[7]));
      const float u = b * (vv - g * sk);
      a0 = a1 = a2 = a3 = 0.f;
#pragma unroll
      for (int ii = 0; ii < Q / 4; ++ii) {
        S[4 * ii] = fmaf(kr[ii].x, u, g * S[4 * ii]);
        S[4 * ii + 1] = fmaf(kr[ii].y, u, g * S[4 * ii + 1]);
        S[4 * ii + 2] = fmaf(kr[ii].z, u, g * S[4 * ii + 2]);
        S[4 * ii + 3] = fmaf(kr[ii].w, u, g * S[4 * ii + 3]);
        a0 = fmaf(S[4 * ii], qr[ii].x, a0);
        a1 = fmaf(S[4 * ii + 1], qr[ii].y, a1);
        a2 = fmaf(S[4 * ii + 2], qr[ii].z, a2);
        a3 = fmaf(S[4 * ii + 3], qr[ii].w, a3);
      }
      os_part[tt][piece][lane] = (a0 + a1) + (a2 + a3);
    }
    __syncthreads();
    for (int i = tid; i < nt * 32; i += NT) {
      const int tt = i >> 5, c = i & 31;
      float o = 0.f;
#pragma unroll
      for (int p = 0; p < P; ++p) o += os_part[tt][p][c];
      o_out[((long long)(t0 + b0 + tt) * H + h) * dv + j0 + c] = o;
    }
  }
#pragma unroll
  for (int ii = 0; ii < Q; ++ii) Sg[(long long)(piece * Q + ii) * dv + j0 + lane] = S[ii];
}

// out[t, h, :] = o / rms(o) * norm_w * silu(gate) (gate_act 1: sigmoid(gate)); a warp per (token, head)
__global__ void __launch_bounds__(256) delta_out_kernel(const float* __restrict__ o, const float* __restrict__ gproj, long long ldg,
                                                        int gate_act, int H, int dv, const float* __restrict__ norm_w, float eps,
                                                        long long T, void* __restrict__ out, int dt_out) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= T * H) return;
  const long long t = w / H;
  const int h = (int)(w - t * H);
  const float* row = o + w * dv;
  float ss = 0.f;
  for (int j = lane; j < dv; j += 32) ss += row[j] * row[j];
  ss = warp_sum(ss);
  const float rstd = 1.f / sqrtf(ss / (float)dv + eps);
  for (int j = lane; j < dv; j += 32) {
    const float gz = gproj[t * ldg + h * dv + j];
    st_dt(out, dt_out, w * dv + j, row[j] * rstd * norm_w[j] * (gate_act ? 1.f / (1.f + expf(-gz)) : silu(gz)));
  }
}

}  // namespace kb2seq

using namespace kb2seq;

extern "C" {

KB2SEQ_API const char* kb2_seq_last_error(void) { return g_err; }
KB2SEQ_API long long kb2_seq_total_launches(void) { return g_launches; }

KB2SEQ_API int kb2_seq_embed(const void* table, int dt, const int* tokens, float* x, int T, int W, float scale, void* stream) {
  if (!table || !tokens || !x || T <= 0 || W <= 0 || bad_dt(dt)) return failf(KB2SEQ_ERR_VALUE, "embed: bad argument");
  if (dt) embed_scale_kernel<bf16><<<T, 128, 0, (cudaStream_t)stream>>>((const bf16*)table, tokens, x, W, scale);
  else embed_scale_kernel<float><<<T, 128, 0, (cudaStream_t)stream>>>((const float*)table, tokens, x, W, scale);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_gemm(const void* A, int dtA, long long lda, const void* B, int dtB, long long ldb, void* C, int dtC,
                            long long ldc, int M, int N, int K, int batch, long long sA, long long sB, long long sC, void* stream) {
  if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0 || batch <= 0 || batch > 65535 || bad_dt(dtA) || bad_dt(dtB) || bad_dt(dtC))
    return failf(KB2SEQ_ERR_VALUE, "gemm: bad argument (M=%d N=%d K=%d batch=%d)", M, N, K, batch);
  cudaStream_t s = (cudaStream_t)stream;
  const int code = dtA * 4 + dtB * 2 + dtC;
#define G(TA, TB, TC) launch_gemm<TA, TB, TC>(A, lda, B, ldb, C, ldc, M, N, K, batch, sA, sB, sC, s)
  switch (code) {
    case 0: G(float, float, float); break;
    case 1: G(float, float, bf16); break;
    case 2: G(float, bf16, float); break;
    case 3: G(float, bf16, bf16); break;
    case 4: G(bf16, float, float); break;
    case 5: G(bf16, float, bf16); break;
    case 6: G(bf16, bf16, float); break;
    default: G(bf16, bf16, bf16); break;
  }
#undef G
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_residual_norm(float* x, const float* y, int y_mode, const float* wa, const float* ba, const float* x0,
                                     const float* wb, const float* bb, void* h, int dt_h, int T, int W, float eps, void* stream) {
  if (!x || T <= 0 || W <= 0 || bad_dt(dt_h)) return failf(KB2SEQ_ERR_VALUE, "residual_norm: bad argument");
  if (y && (y_mode < 1 || y_mode > 2 || !wa || (y_mode == 1 && !ba))) return failf(KB2SEQ_ERR_VALUE, "residual_norm: norm of y needs its weights");
  if (h && (!wb || !bb)) return failf(KB2SEQ_ERR_VALUE, "residual_norm: output norm needs weight and bias");
  const size_t smem = (size_t)W * 4;
  if (smem > 200 * 1024) return failf(KB2SEQ_ERR_VALUE, "residual_norm: width %d too large", W);
  if (smem > 48 * 1024) SEQ_CUDA(cudaFuncSetAttribute(residual_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  residual_norm_kernel<<<T, 256, smem, (cudaStream_t)stream>>>(x, y, y_mode, wa, ba, x0, wb, bb, h, dt_h, W, eps, nullptr);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_residual_add_norm(float* x, const float* y, const float* y2, const float* wb, const float* bb, void* h, int dt_h,
                                         int T, int W, float eps, void* stream) {
  if (!x || T <= 0 || W <= 0 || bad_dt(dt_h) || (y2 && !y)) return failf(KB2SEQ_ERR_VALUE, "residual_add_norm: bad argument");
  if (h && !wb) return failf(KB2SEQ_ERR_VALUE, "residual_add_norm: output norm needs its weight");
  const size_t smem = (size_t)W * 4;
  if (smem > 200 * 1024) return failf(KB2SEQ_ERR_VALUE, "residual_add_norm: width %d too large", W);
  if (smem > 48 * 1024) SEQ_CUDA(cudaFuncSetAttribute(residual_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  residual_norm_kernel<<<T, 256, smem, (cudaStream_t)stream>>>(x, y, 3, nullptr, nullptr, nullptr, wb, bb, h, dt_h, W, eps, y2);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_act_mul(const void* in, int dt_in, void* out, int dt_out, int T, int F, void* stream) {
  if (!in || !out || T <= 0 || F <= 0 || bad_dt(dt_in) || bad_dt(dt_out)) return failf(KB2SEQ_ERR_VALUE, "act_mul: bad argument");
  if (T > 65535) return failf(KB2SEQ_ERR_VALUE, "act_mul: more than 65535 rows in one step");
  if (dt_in == 1 && dt_out == 1 && F % 8 == 0 && !((uintptr_t)in & 15) && !((uintptr_t)out & 15))
    act_mul_bf16x8_kernel<<<dim3((F / 8 + 127) / 128, T), 128, 0, (cudaStream_t)stream>>>((const bf16*)in, (bf16*)out, F);
  else
    act_mul_kernel<<<dim3((F + 255) / 256, T), 256, 0, (cudaStream_t)stream>>>(in, dt_in, out, dt_out, T, F);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_side_gate(const float* g, const void* table, int dt_table, long long table_ld, const int* tokens, int col0,
                                 int dim, int T, void* out, int dt_out, void* stream) {
  if (!g || !table || !tokens || !out || T <= 0 || dim <= 0 || col0 < 0 || bad_dt(dt_table) || bad_dt(dt_out))
    return failf(KB2SEQ_ERR_VALUE, "side_gate: bad argument");
  const long long n = (long long)T * dim;
  side_gate_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(g, table, dt_table, table_ld, tokens, col0, dim, T, out,
                                                                                  dt_out);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_latent_prep(float* proj, long long ldp, int T, int H, int dn, int dr, int r, const float* cw, float eps,
                                   const double* freq, int rot_dims, float amp, const int* positions, const int* seq_of,
                                   const int* pages, int max_pages, int page_size, void* ckv, void* kr, int dt_cache, const float* lat,
                                   long long ldl, void* stream) {
  if (!proj || !cw || !freq || !positions || !seq_of || !pages || !ckv || !kr || T <= 0 || H <= 0 || dn < 0 || dr < 0 || r <= 0 ||
      rot_dims < 0 || rot_dims > dr || (rot_dims & 1) || page_size <= 0 || max_pages <= 0 || bad_dt(dt_cache))
    return failf(KB2SEQ_ERR_VALUE, "latent_prep: bad argument");
  latent_prep_kernel<<<T, 128, 0, (cudaStream_t)stream>>>(proj, ldp, H, dn, dr, r, cw, eps, freq, rot_dims, amp, positions, seq_of, pages,
                                                          max_pages, page_size, ckv, kr, dt_cache, lat, ldl);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_latent_window_attn(const float* q_abs, const float* proj, long long ldp, int T, int H, int dn, int dr, int r,
                                          const void* ckv, const void* kr, int dt_cache, const int* positions, const int* seq_of,
                                          const int* pages, int max_pages, int page_size, const float* sinks, float scale, int window,
                                          float* out, const int* cu, int skip_from, int nsplit, float* part_acc, float* part_ml,
                                          void* stream) {
  if (!q_abs || !proj || !ckv || !kr || !positions || !seq_of || !pages || !out || T <= 0 || H <= 0 || r <= 0 || dr < 0 ||
      window <= 0 || bad_dt(dt_cache))
    return failf(KB2SEQ_ERR_VALUE, "latent_window_attn: bad argument");
  if (r > kAttnThreads * kAttnAcc) return failf(KB2SEQ_ERR_VALUE, "latent_window_attn: latent size %d > %d", r, kAttnThreads * kAttnAcc);
  int HG = 8;                              // heads per block: a power of two, so that the 8 warps split evenly over the heads
  while (HG > 1 && (HG > H || HG * r > kAttnThreads * kAttnAcc)) HG >>= 1;
  const int D = r + dr;
  const int KT = 32;
  auto smem_of = [&](int hg, int kt) { return (size_t)(hg * D + kt * (D + 1) + hg * kt + 8 * kt + 3 * hg) * 4 + (size_t)kt * 8; };
  while (HG > 1 && smem_of(HG, KT) > 200 * 1024) HG >>= 1;
  if (nsplit < 1 || nsplit > 1024 || (nsplit > 1 && (!part_acc || !part_ml))) return failf(KB2SEQ_ERR_VALUE, "latent_window_attn: bad key split");
  const size_t smem = smem_of(HG, KT);
  if (smem > 200 * 1024) return failf(KB2SEQ_ERR_VALUE, "latent_window_attn: latent + rotated size %d too large", D);
  if (smem > 48 * 1024) SEQ_CUDA(cudaFuncSetAttribute(latent_window_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(T, (H + HG - 1) / HG, nsplit);
  latent_window_attn_kernel<<<grid, kAttnThreads, smem, (cudaStream_t)stream>>>(q_abs, proj, ldp, H, HG, dn, dr, r, ckv, kr, dt_cache, positions,
                                                                                 seq_of, pages, max_pages, page_size, sinks, scale, window, KT,
                                                                                 out, cu, skip_from, nsplit, part_acc, part_ml);
  SEQ_LAUNCHED();
  if (nsplit > 1) {
    latent_attn_combine_kernel<<<dim3(T, H), 128, 0, (cudaStream_t)stream>>>(part_acc, part_ml, H, r, nsplit, out, seq_of, cu, skip_from);
    SEQ_LAUNCHED();
  }
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_conv(const float* proj, long long ldp, int T, int S, int C, int K, const float* taps, const float* bias, int act,
                            float* tail, const int* seq_of, const int* cu, const int* slots, float* out, void* stream) {
  const int bias_after = act >> 1;
  act &= 1;
  if (!proj || !taps || !tail || !seq_of || !cu || !slots || !out || T <= 0 || S <= 0 || C <= 0 || K <= 0 || bias_after > 1)
    return failf(KB2SEQ_ERR_VALUE, "conv: bad argument");
  if (T > 65535) return failf(KB2SEQ_ERR_VALUE, "conv: more than 65535 rows in one step");
  if (T >= 4 * kConvRun && K <= kConvMaxTaps)
    conv_run_kernel<<<dim3((C + 255) / 256, (T + kConvRun - 1) / kConvRun), 256, 0, (cudaStream_t)stream>>>(proj, ldp, C, K, taps, tail, seq_of,
                                                                                                          cu, slots, T, out, bias, act, bias_after);
  else
    conv_silu_kernel<<<dim3((C + 255) / 256, T), 256, 0, (cudaStream_t)stream>>>(proj, ldp, C, K, taps, tail, seq_of, cu, slots, T, out, bias,
                                                                                 act, bias_after);
  SEQ_LAUNCHED();
  if (K > 1) {
    const long long m = (long long)S * C;
    conv_tail_kernel<<<(unsigned)((m + 255) / 256), 256, 0, (cudaStream_t)stream>>>(proj, ldp, C, K, tail, cu, slots, S, bias_after ? nullptr : bias);
    SEQ_LAUNCHED();
  }
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_conv_silu(const float* proj, long long ldp, int T, int S, int C, int K, const float* taps, float* tail,
                                 const int* seq_of, const int* cu, const int* slots, float* out, void* stream) {
  return kb2_seq_conv(proj, ldp, T, S, C, K, taps, nullptr, 1, tail, seq_of, cu, slots, out, stream);
}

KB2SEQ_API int kb2_seq_residual_scale_rms(float* x, const float* y, float y_mult, const float* w, float w_shift, void* h, int dt_h, int T,
                                          int W, float eps, void* stream) {
  if (!x || T <= 0 || W <= 0 || bad_dt(dt_h) || (h && !w)) return failf(KB2SEQ_ERR_VALUE, "residual_scale_rms: bad argument");
  if (h == (void*)x && (y || dt_h != 0)) return failf(KB2SEQ_ERR_VALUE, "residual_scale_rms: a norm in place takes no addend and is fp32");
  const size_t smem = (size_t)W * 4;
  if (smem > 200 * 1024) return failf(KB2SEQ_ERR_VALUE, "residual_scale_rms: width %d too large", W);
  if (smem > 48 * 1024) SEQ_CUDA(cudaFuncSetAttribute(residual_scale_rms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  residual_scale_rms_kernel<<<T, 256, smem, (cudaStream_t)stream>>>(x, y, y_mult, w, w_shift, h, dt_h, W, eps);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

static int delta_rule_launch(const float* conv, int C, const float* bproj, long long ldb, const float* aproj, long long lda, int ch,
                             const float* gproj, long long ldg, int gate_act, int T, int S, int H, int Hk, int dk, int dv,
                             const float* A_log, const float* dt_bias, const float* norm_w, float eps, float* state, const int* cu,
                             const int* slots, float* scratch, void* out, int dt_out, void* stream) {
  if (!conv || !bproj || !aproj || !gproj || !A_log || !dt_bias || !norm_w || !state || !cu || !slots || !out || S <= 0 || H <= 0 ||
      Hk <= 0 || H % Hk || dk <= 0 || dv <= 0 || bad_dt(dt_out))
    return failf(KB2SEQ_ERR_VALUE, "delta_rule: bad argument");
  if (scratch && (dk == 32 || dk == 64 || dk == 128) && dv % 32 == 0 && C % 4 == 0 && ((2 * Hk * dk) % 4) == 0) {
    // scratch: qn [T, Hk, dk] | kn [T, Hk, dk] | beta [T, H] | dec [T, H] or [T, H, dk] | o [T, H, dv]   (fp32)
    cudaStream_t st = (cudaStream_t)stream;
    float* qn = scratch;
    float* kn = qn + (long long)T * Hk * dk;
    float* be = kn + (long long)T * Hk * dk;
    float* de = be + (long long)T * H;
    if (ch) de = (float*)(((uintptr_t)de + 15) & ~(uintptr_t)15);
    float* ob = de + (long long)T * H * (ch ? dk : 1);
    ob = (float*)(((uintptr_t)ob + 15) & ~(uintptr_t)15);
    const long long nw = (long long)T * Hk;
    delta_prep_kernel<<<(unsigned)((nw + 7) / 8), 256, 0, st>>>(conv, C, bproj, ldb, aproj, lda, ch, H, Hk, dk, A_log, dt_bias, T, qn, kn, be, de);
    SEQ_LAUNCHED();
    dim3 grid(S, H, dv / 32);
    const int v_col0 = 2 * Hk * dk;
#define R(DK, CHV) delta_rule_reg_kernel<DK, CHV><<<grid, 32 * kRegPieces, 0, st>>>(qn, kn, conv, C, v_col0, be, de, H, Hk, dv, state, cu, slots, ob)
    if (ch) {
      if (dk == 32) R(32, true); else if (dk == 64) R(64, true); else R(128, true);
    } else {
      if (dk == 32) R(32, false); else if (dk == 64) R(64, false); else R(128, false);
    }
#undef R
    SEQ_LAUNCHED();
    const long long no = (long long)T * H;
    delta_out_kernel<<<(unsigned)((no + 7) / 8), 256, 0, st>>>(ob, gproj, ldg, gate_act, H, dv, norm_w, eps, T, out, dt_out);
    SEQ_LAUNCHED();
    return KB2SEQ_OK;
  }
  auto smem_of = [&](int cols) { return ((size_t)dk * cols + (size_t)kDeltaTile * (2 * dk + cols + 1 + (ch ? dk : 1))) * 4; };
  int dvb = dv;                                // a state too large for one block's shared memory is cut into slices of value columns
  if (dv > 1024 || smem_of(dv) > 220 * 1024) {
    dvb = dv < 1024 ? dv / 32 * 32 : 1024;
    while (dvb > 32 && smem_of(dvb) > 220 * 1024) dvb -= 32;
    if (dvb < 32 || smem_of(dvb) > 220 * 1024)
      return failf(KB2SEQ_ERR_VALUE, "delta_rule: %d key channels do not fit one block's shared memory", dk);
    if (!scratch) return failf(KB2SEQ_ERR_VALUE, "delta_rule: a %d x %d state needs the scratch buffer (T H dv floats)", dk, dv);
  }
  const size_t smem = smem_of(dvb);
  if (smem > 48 * 1024) SEQ_CUDA(cudaFuncSetAttribute(delta_rule_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int threads = (dvb + 31) / 32 * 32;
  if (threads < 128) threads = 128;
  const bool cut = dvb < dv;
  dim3 grid(S, H, (dv + dvb - 1) / dvb);
  delta_rule_kernel<<<grid, threads, smem, (cudaStream_t)stream>>>(conv, C, bproj, ldb, aproj, lda, ch, gproj, ldg, gate_act, H, Hk, dk, dv, A_log,
                                                                  dt_bias, norm_w, eps, state, cu, slots, out, dt_out, dvb,
                                                                  cut ? scratch : nullptr);
  SEQ_LAUNCHED();
  if (cut) {
    const long long no = (long long)T * H;
    delta_out_kernel<<<(unsigned)((no + 7) / 8), 256, 0, (cudaStream_t)stream>>>(scratch, gproj, ldg, gate_act, H, dv, norm_w, eps, T, out, dt_out);
    SEQ_LAUNCHED();
  }
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_delta_rule(const float* conv, int C, const float* proj, long long ldp, int g_off, int a_off, int b_off, int T,
                                  int S, int H, int Hk, int dk, int dv, const float* A_log, const float* dt_bias, const float* norm_w,
                                  float eps, float* state, const int* cu, const int* slots, float* scratch, void* out, int dt_out,
                                  void* stream) {
  if (!proj) return failf(KB2SEQ_ERR_VALUE, "delta_rule: bad argument");
  return delta_rule_launch(conv, C, proj + b_off, ldp, proj + a_off, ldp, 0, proj + g_off, ldp, 0, T, S, H, Hk, dk, dv, A_log, dt_bias, norm_w,
                           eps, state, cu, slots, scratch, out, dt_out, stream);
}

KB2SEQ_API int kb2_seq_delta_rule_ch(const float* conv, int C, const float* beta_in, long long ldb, const float* decay_in, long long lda,
                                     const float* gate_in, long long ldg, int gate_act, int T, int S, int H, int Hk, int dk, int dv,
                                     const float* A_log, const float* dt_bias, const float* norm_w, float eps, float* state, const int* cu,
                                     const int* slots, float* scratch, void* out, int dt_out, void* stream) {
  if (gate_act < 0 || gate_act > 1) return failf(KB2SEQ_ERR_VALUE, "delta_rule_ch: bad argument");
  return delta_rule_launch(conv, C, beta_in, ldb, decay_in, lda, 1, gate_in, ldg, gate_act, T, S, H, Hk, dk, dv, A_log, dt_bias, norm_w, eps,
                           state, cu, slots, scratch, out, dt_out, stream);
}

}  // extern "C"
