// Ragged-batch sequence operators, third part: linear recurrences with per-sequence state slots and the small row kernels of
// designs that run several mixers side by side or average their residual stream over depth.
//
//   gla_scan / gla_reg     gated linear attention, S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t per head, with one decay per key
//                          channel alpha = sigmoid(z)^(1 / tau); the state of a (sequence, head, slice of value columns) lives in
//                          registers: a generic form (P lanes share a column and each keeps dk / P of its rows) and, for key sizes
//                          32 / 64 / 128 / 256, a form with lane = column, warp = slice of rows and cp.async token tiles
//   selective_scan         S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n, y_c = sum_n S[c, n] C_n + D_c x_c, times silu(z);
//                          the lanes of a channel keep its states in registers; their pieces of y meet in shared memory once per tile
//   head_norm_gate         per head: o / rms(o) * w (optional) times silu or sigmoid of a gate column (optional)
//   rms_rows               RMS norm of a column range of strided fp32 rows
//   branch_merge           c (a / rms(a) * wa + b / rms(b) * wb): two mixers that read the same input, each normed, averaged
//   depth_mix              the residual stream as a learned weighted sum of the embedding output and every layer's result, fused with
//                          the residual add that completes the newest result and with the next norm
//
// Precision: decays, step sizes, softplus / exponentials, states, norms and every accumulation are fp32; `dt` selects storage only.
#include "seq_common.cuh"

namespace kb2seq {

constexpr int kRecThreads = 256, kRecTok = 16;

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ------------------------------------------------------------------------------------------------ gated linear attention
// q, k [T, ld] (H x dk columns from q_off / k_off), v (H x dv from v_off), decay_in [T, lda] (H x dk logits, + decay_bias).
// Block (sequence s, head h, slice of CB value columns).  Lane l of a warp: column l % CW, key slice p = l / CW of P = 32 / CW;
// thread rows are i = p + P ii, ii < KR.  Tokens are staged kRecTok at a time as (alpha, k, q) triples in shared memory.
template <int KR>
__global__ void __launch_bounds__(kRecThreads) gla_scan_kernel(const float* __restrict__ qkv, long long ld, int q_off, int k_off, int v_off,
                                                               const float* __restrict__ decay_in, long long lda,
                                                               const float* __restrict__ decay_bias, float inv_tau, float q_scale, int H,
                                                               int dk, int dv, int P, float* __restrict__ state, const int* __restrict__ cu,
                                                               const int* __restrict__ slots, float* __restrict__ out) {
  extern __shared__ __align__(16) float sm[];
  float4* akq = reinterpret_cast<float4*>(sm);              // [kRecTok][dk]
  const int CW = 32 / P, CB = (kRecThreads / 32) * CW;
  float* vs = sm + 4 * kRecTok * dk;                        // [kRecTok][CB]
  const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int p = lane / CW, cl = warp * CW + lane % CW, c = c0 + cl;
  const bool live = c < dv;
  const int row0 = cu[s], n = cu[s + 1] - row0;
  float* S = state + ((long long)slots[s] * H + h) * dk * dv;
  float st[KR];
#pragma unroll
  for (int ii = 0; ii < KR; ++ii) {
    const int i = p + P * ii;
    st[ii] = (live && i < dk) ? S[(long long)i * dv + c] : 0.f;
  }
  for (int t0 = 0; t0 < n; t0 += kRecTok) {
    const int nt = min(kRecTok, n - t0);
    __syncthreads();
    for (int e = tid; e < nt * dk; e += kRecThreads) {
      const int tt = e / dk, i = e - tt * dk;
      const long long t = row0 + t0 + tt;
      const float z = decay_in[t * lda + h * dk + i] + (decay_bias ? decay_bias[h * dk + i] : 0.f);
      float4 f;
      f.x = expf(-softplus_f(-z) * inv_tau);                // sigmoid(z)^(1 / tau)
      f.y = qkv[t * ld + k_off + h * dk + i];
      f.z = qkv[t * ld + q_off + h * dk + i] * q_scale;
      f.w = 0.f;
      akq[e] = f;
    }
    for (int e = tid; e < nt * CB; e += kRecThreads) {
      const int tt = e / CB, cc = e - tt * CB;
      vs[e] = c0 + cc < dv ? qkv[(long long)(row0 + t0 + tt) * ld + v_off + h * dv + c0 + cc] : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float v = vs[tt * CB + cl];
      const float4* row = akq + tt * dk;
      float o = 0.f;
#pragma unroll
      for (int ii = 0; ii < KR; ++ii) {
        const int i = p + P * ii;
        if (i < dk) {
          const float4 f = row[i];
          st[ii] = fmaf(st[ii], f.x, f.y * v);
          o = fmaf(st[ii], f.z, o);
        }
      }
      for (int off = CW; off < 32; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (p == 0 && live) out[(long long)(row0 + t0 + tt) * H * dv + h * dv + c] = o;
    }
  }
#pragma unroll
  for (int ii = 0; ii < KR; ++ii) {
    const int i = p + P * ii;
    if (live && i < dk) S[(long long)i * dv + c] = st[ii];
  }
}

// The same recurrence for key sizes 32, 64, 128 and 256 with value sizes that are multiples of 32 (the sizes of real models): a block
// owns 32 value columns of a (sequence, head); lane = column, so that the state moves in whole 128-byte rows; warp w keeps rows
// [w DK / 8, (w + 1) DK / 8) of its column in registers.  A token's alpha, k and q values are the same address for every lane (one
// shared-memory transaction per 16 bytes); tiles of kGlaTile tokens arrive by cp.async, double-buffered, from the projection itself and
// from the decays that gla_decay_kernel wrote; the warps' pieces of S^T q meet in shared memory once per tile.  No barrier inside a token.
__global__ void gla_decay_kernel(const float* __restrict__ decay_in, long long lda, const float* __restrict__ decay_bias, float inv_tau,
                                 long long T, int n, float* __restrict__ alpha) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * n) return;
  const long long t = i / n;
  const int c = (int)(i - t * n);
  const float z = decay_in[t * lda + c] + (decay_bias ? decay_bias[c] : 0.f);
  alpha[i] = expf(-softplus_f(-z) * inv_tau);
}

__device__ __forceinline__ void rec_cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void rec_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void rec_cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

constexpr int kGlaTile = 8, kGlaWarps = 8;
template <int DK>
__global__ void __launch_bounds__(32 * kGlaWarps) gla_reg_kernel(const float* __restrict__ qkv, long long ld, int q_off, int k_off, int v_off,
                                                                 const float* __restrict__ alpha, float q_scale, int H, int dv,
                                                                 float* __restrict__ state, const int* __restrict__ cu,
                                                                 const int* __restrict__ slots, float* __restrict__ out) {
  constexpr int P = kGlaWarps, NT = 32 * P, Q = DK / P;
  extern __shared__ __align__(16) float sm[];
  float* as = sm;                                   // [2][kGlaTile][DK]
  float* ks = as + 2 * kGlaTile * DK;
  float* qs = ks + 2 * kGlaTile * DK;
  float* vs = qs + 2 * kGlaTile * DK;               // [2][kGlaTile][32]
  float* os_part = vs + 2 * kGlaTile * 32;          // [kGlaTile][P][32]
  const int s = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * 32;
  const int tid = threadIdx.x, lane = tid & 31, piece = tid >> 5;
  const int t0 = cu[s], n = cu[s + 1] - cu[s];
  float* Sg = state + ((long long)slots[s] * H + h) * DK * dv;
  float S[Q];
#pragma unroll
  for (int ii = 0; ii < Q; ++ii) S[ii] = Sg[(long long)(piece * Q + ii) * dv + j0 + lane];

  auto load_tile = [&](int buf, int b0) {
    const int nt = min(kGlaTile, n - b0);
    for (int c = tid; c < nt * (DK / 4); c += NT) {                  // 16-byte chunks of the alpha, k and q rows
      const int tt = c / (DK / 4), cc = c - tt * (DK / 4);
      const long long row = t0 + b0 + tt;
      const int dst = (buf * kGlaTile + tt) * DK + cc * 4;
      rec_cp_async16(as + dst, alpha + (row * H + h) * DK + cc * 4);
      rec_cp_async16(ks + dst, qkv + row * ld + k_off + h * DK + cc * 4);
      rec_cp_async16(qs + dst, qkv + row * ld + q_off + h * DK + cc * 4);
    }
    for (int c = tid; c < nt * 8; c += NT) {
      const int tt = c >> 3, cc = c & 7;
      rec_cp_async16(vs + (buf * kGlaTile + tt) * 32 + cc * 4, qkv + (long long)(t0 + b0 + tt) * ld + v_off + h * dv + j0 + cc * 4);
    }
    rec_cp_async_commit();
  };

  load_tile(0, 0);
  int buf = 0;
  for (int b0 = 0; b0 < n; b0 += kGlaTile, buf ^= 1) {
    const int nt = min(kGlaTile, n - b0);
    rec_cp_async_wait_all();
    __syncthreads();                                  // tile `buf` is in place; everyone is done with the other buffer and with os_part
    if (b0 + kGlaTile < n) load_tile(buf ^ 1, b0 + kGlaTile);
    for (int tt = 0; tt < nt; ++tt) {
      const int base = (buf * kGlaTile + tt) * DK + piece * Q;
      const float4* a4 = reinterpret_cast<const float4*>(as + base);
      const float4* k4 = reinterpret_cast<const float4*>(ks + base);
      const float4* q4 = reinterpret_cast<const float4*>(qs + base);
      const float vv = vs[(buf * kGlaTile + tt) * 32 + lane];
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int ii = 0; ii < Q / 4; ++ii) {
        const float4 ar = a4[ii], kr = k4[ii], qr = q4[ii];
        S[4 * ii] = fmaf(S[4 * ii], ar.x, kr.x * vv);
        S[4 * ii + 1] = fmaf(S[4 * ii + 1], ar.y, kr.y * vv);
        S[4 * ii + 2] = fmaf(S[4 * ii + 2], ar.z, kr.z * vv);
        S[4 * ii + 3] = fmaf(S[4 * ii + 3], ar.w, kr.w * vv);
        a0 = fmaf(S[4 * ii], qr.x, a0);
        a1 = fmaf(S[4 * ii + 1], qr.y, a1);
        a2 = fmaf(S[4 * ii + 2], qr.z, a2);
        a3 = fmaf(S[4 * ii + 3], qr.w, a3);
      }
      os_part[(tt * P + piece) * 32 + lane] = (a0 + a1) + (a2 + a3);
    }
    __syncthreads();
    for (int i = tid; i < nt * 32; i += NT) {
      const int tt = i >> 5, c = i & 31;
      float o = 0.f;
#pragma unroll
      for (int p = 0; p < P; ++p) o += os_part[(tt * P + p) * 32 + c];
      out[((long long)(t0 + b0 + tt) * H + h) * dv + j0 + c] = o * q_scale;
    }
  }
#pragma unroll
  for (int ii = 0; ii < Q; ++ii) Sg[(long long)(piece * Q + ii) * dv + j0 + lane] = S[ii];
}

// ------------------------------------------------------------------------------------------------ selective scan
// x [T, ldx] (inner channels after convolution and activation), dt_in [T, ldd] (+ dt_bias, then softplus), bc [T, ldb] = [B: N | C: N]
// from b_off, z [T, ldz] from z_off, A_log [inner, N], D [inner].  Block (sequence, group of CB channels); lane l: state slice
// p = l % P, channel l / P of the warp; thread states are n = p + P ii, ii < NR.
__device__ __forceinline__ float ex2_approx_ftz(float x) {       // 2^x, MUFU.EX2 (2 ulp, as exp2f); results below 2^-126 become 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void rec_cp_async4(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}

// Tiles of kRecTok tokens arrive by cp.async, double-buffered (dt input, x, z of the block's channels; B and C of the token), so that
// the loads of the next tile run under the recurrence of this one.  Per tile: step sizes (softplus) once per (token, channel); the
// recurrence with nothing but shared memory and registers inside and no exchange between lanes; then the lanes' pieces of y are summed,
// D x added, the gate applied and the rows written.
template <int NR>
__global__ void __launch_bounds__(kRecThreads) selective_scan_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ dt_in,
                                                                     long long ldd, const float* __restrict__ dt_bias,
                                                                     const float* __restrict__ bc, long long ldb, int b_off,
                                                                     const float* __restrict__ z, long long ldz, int z_off,
                                                                     const float* __restrict__ A_log, const float* __restrict__ Dw, int inner,
                                                                     int N, int P, float* __restrict__ state, const int* __restrict__ cu,
                                                                     const int* __restrict__ slots, void* __restrict__ out, int dt_out) {
  extern __shared__ __align__(16) float sm[];
  const int CW = 32 / P, CB = (kRecThreads / 32) * CW;
  float* bcs = sm;                                   // [2][kRecTok][2 N]: B | C of the token
  float* dts = bcs + 2 * kRecTok * 2 * N;            // [2][kRecTok][CB]: dt input, then the step size
  float* xs = dts + 2 * kRecTok * CB;                // [2][kRecTok][CB]
  float* zs = xs + 2 * kRecTok * CB;                 // [2][kRecTok][CB]
  float* yp = zs + 2 * kRecTok * CB;                 // [kRecTok][CB][P + 1]: every lane's piece of y, summed once per tile (odd pitch: no bank conflicts)
  const int s = blockIdx.x, c0 = blockIdx.y * CB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int p = lane % P, cl = warp * CW + lane / P, c = c0 + cl;   // tid == cl * P + p
  const bool live = c < inner;
  const int row0 = cu[s], n = cu[s + 1] - row0;
  float* S = state + (long long)slots[s] * inner * N;
  float st[NR], a[NR];
#pragma unroll
  for (int ii = 0; ii < NR; ++ii) {
    const int j = p + P * ii;
    const bool ok = live && j < N;
    st[ii] = ok ? S[(long long)c * N + j] : 0.f;
    a[ii] = ok ? -expf(A_log[(long long)c * N + j]) * 1.4426950408889634f : 0.f;      // A log2(e): exp(dt A) = 2^(dt a)
  }
  const int cb_shift = __ffs(CB) - 1;                // CB = 256 / P is a power of two: rows and channels of a tile by shift and mask

  auto load_tile = [&](int buf, int b0) {
    const int nt = min(kRecTok, n - b0);
    for (int e = tid; e < nt * 2 * N; e += kRecThreads) {
      const int tt = e / (2 * N), j = e - tt * 2 * N;
      rec_cp_async4(bcs + (buf * kRecTok + tt) * 2 * N + j, bc + (long long)(row0 + b0 + tt) * ldb + b_off + j);
    }
    for (int e = tid; e < nt * CB; e += kRecThreads) {
      const int tt = e >> cb_shift, cc = e & (CB - 1);
      if (c0 + cc >= inner) continue;
      const long long t = row0 + b0 + tt;
      const int dst = (buf * kRecTok + tt) * CB + cc;
      rec_cp_async4(dts + dst, dt_in + t * ldd + c0 + cc);
      rec_cp_async4(xs + dst, x + t * ldx + c0 + cc);
      rec_cp_async4(zs + dst, z + t * ldz + z_off + c0 + cc);
    }
    rec_cp_async_commit();
  };

  load_tile(0, 0);
  int buf = 0;
  for (int t0 = 0; t0 < n; t0 += kRecTok, buf ^= 1) {
    const int nt = min(kRecTok, n - t0);
    rec_cp_async_wait_all();
    __syncthreads();                                 // tile `buf` is in place; everyone is done with the other buffer and with yp
    if (t0 + kRecTok < n) load_tile(buf ^ 1, t0 + kRecTok);
    for (int e = tid; e < nt * CB; e += kRecThreads) {
      const int cc = e & (CB - 1);
      if (c0 + cc >= inner) continue;
      float* d = dts + buf * kRecTok * CB + e;
      *d = softplus_f(*d + dt_bias[c0 + cc]);
    }
    __syncthreads();
    if (live) {
      const float* dp = dts + buf * kRecTok * CB + cl;
      const float* xq = xs + buf * kRecTok * CB + cl;
      const float* row = bcs + buf * kRecTok * 2 * N + p;
      float* yq = yp + cl * (P + 1) + p;
      const int ypitch = CB * (P + 1);
#pragma unroll 4
      for (int tt = 0; tt < nt; ++tt, dp += CB, xq += CB, row += 2 * N, yq += ypitch) {
        const float dtv = *dp;
        const float dtx = dtv * *xq;
        float y = 0.f;
#pragma unroll
        for (int ii = 0; ii < NR; ++ii) {
          if (p + P * ii < N) {                      // a[] is A log2(e): one MUFU per state update
            st[ii] = fmaf(ex2_approx_ftz(dtv * a[ii]), st[ii], dtx * row[P * ii]);
            y = fmaf(st[ii], row[N + P * ii], y);
          }
        }
        *yq = y;
      }
    }
    __syncthreads();
    for (int e = tid; e < nt * CB; e += kRecThreads) {
      const int tt = e >> cb_shift, cc = e & (CB - 1);
      if (c0 + cc >= inner) continue;
      const float* pieces = yp + (tt * CB + cc) * (P + 1);
      float y = 0.f;
      for (int q = 0; q < P; ++q) y += pieces[q];
      const int src = (buf * kRecTok + tt) * CB + cc;
      y = fmaf(Dw[c0 + cc], xs[src], y);
      st_dt(out, dt_out, (long long)(row0 + t0 + tt) * inner + c0 + cc, y * silu(zs[src]));
    }
  }
#pragma unroll
  for (int ii = 0; ii < NR; ++ii) {
    const int j = p + P * ii;
    if (live && j < N) S[(long long)c * N + j] = st[ii];
  }
}

// ------------------------------------------------------------------------------------------------ row kernels
// out[t, h, :] = o[t, h, :] (/ rms * w[:] if w) (* act(gate[t, h dv + :]) if gate); a warp per (token, head).  gate_act 0: silu, 1: sigmoid
__global__ void __launch_bounds__(256) head_norm_gate_kernel(const float* __restrict__ o, long long ldo, const float* __restrict__ w, float eps,
                                                             const float* __restrict__ gate, long long ldg, int gate_act, int H, int dv,
                                                             long long T, void* __restrict__ out, int dt_out) {
  const long long wi = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wi >= T * H) return;
  const long long t = wi / H;
  const int h = (int)(wi - t * H);
  const float* row = o + t * ldo + (long long)h * dv;
  float rstd = 1.f;
  if (w != nullptr) {
    float ss = 0.f;
    for (int j = lane; j < dv; j += 32) ss = fmaf(row[j], row[j], ss);
    ss = warp_sum(ss);
    rstd = 1.f / sqrtf(ss / (float)dv + eps);
  }
  for (int j = lane; j < dv; j += 32) {
    float v = row[j] * rstd;
    if (w != nullptr) v *= w[j];
    if (gate != nullptr) {
      const float gz = gate[t * ldg + h * dv + j];
      v *= gate_act ? 1.f / (1.f + expf(-gz)) : silu(gz);
    }
    st_dt(out, dt_out, wi * dv + j, v);
  }
}

// out[t, :n] = in[t, :n] / rms * w; a block per row
__global__ void __launch_bounds__(256) rms_rows_kernel(const float* __restrict__ in, long long ld_in, int n, const float* __restrict__ w,
                                                       float eps, void* __restrict__ out, int dt_out, long long ld_out) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const float* r = in + t * ld_in;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(r[i], r[i], ss);
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) st_dt(out, dt_out, t * ld_out + i, r[i] * rstd * w[i]);
}

// out[t] = coef (a[t] / rms(a[t]) * wa + b[t] / rms(b[t]) * wb)
__global__ void __launch_bounds__(256) branch_merge_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ wa,
                                                           const float* __restrict__ wb, float eps, float coef, float* __restrict__ out, int W) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const float* ra = a + t * W;
  const float* rb = b + t * W;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    sa = fmaf(ra[i], ra[i], sa);
    sb = fmaf(rb[i], rb[i], sb);
  }
  sa = block_sum(sa, red);
  sb = block_sum(sb, red);
  const float fa = 1.f / sqrtf(sa / (float)W + eps), fb = 1.f / sqrtf(sb / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) out[t * W + i] = coef * (ra[i] * fa * wa[i] + rb[i] * fb * wb[i]);
}

// stack [n][T][W]: results 0 .. n - 2 are there; result n - 1 = x + y (y may be null) is stored; then x <- sum_j coef[j] stack[j] and
// h = x / rms(x) * w (w may be null: no h)
__global__ void __launch_bounds__(256) depth_mix_kernel(float* __restrict__ stack, long long stride, int n, const float* __restrict__ coef,
                                                        float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w,
                                                        void* __restrict__ h, int dt_h, int W, float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  float* xr = x + t * W;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float newest = xr[i] + (y ? y[t * W + i] : 0.f);
    stack[(long long)(n - 1) * stride + t * W + i] = newest;
    float acc = 0.f;
    for (int j = 0; j < n - 1; ++j) acc = fmaf(coef[j], stack[(long long)j * stride + t * W + i], acc);
    acc = fmaf(coef[n - 1], newest, acc);
    xr[i] = acc;
    ss = fmaf(acc, acc, ss);
  }
  if (w == nullptr) return;
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) st_dt(h, dt_h, t * W + i, xr[i] * rstd * w[i]);
}

static int pow2_at_least(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

template <int DK>
static int launch_gla_reg(const float* qkv, long long ld, int q_off, int k_off, int v_off, const float* alpha, float q_scale, int S, int H,
                          int dv, float* state, const int* cu, const int* slots, float* out, cudaStream_t st) {
  const size_t smem = (size_t)(3 * 2 * kGlaTile * DK + 2 * kGlaTile * 32 + kGlaTile * kGlaWarps * 32) * 4;
  if (smem > 48 * 1024) SEQ_CUDA(cudaFuncSetAttribute(gla_reg_kernel<DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  gla_reg_kernel<DK><<<dim3(S, H, dv / 32), 32 * kGlaWarps, smem, st>>>(qkv, ld, q_off, k_off, v_off, alpha, q_scale, H, dv, state, cu, slots, out);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

}  // namespace kb2seq

using namespace kb2seq;

extern "C" {

KB2SEQ_API int kb2_seq_gla(const float* qkv, long long ld, int q_off, int k_off, int v_off, const float* decay_in, long long lda,
                           const float* decay_bias, float tau, float q_scale, int T, int S, int H, int dk, int dv, float* state,
                           const int* cu, const int* slots, float* scratch, float* out, void* stream) {
  if (!qkv || !decay_in || !state || !cu || !slots || !out || T <= 0 || S <= 0 || H <= 0 || dk <= 0 || dv <= 0 || !(tau > 0.f))
    return failf(KB2SEQ_ERR_VALUE, "gla: bad argument");
  if (dk > 1024) return failf(KB2SEQ_ERR_VALUE, "gla: key size %d > 1024", dk);
  if (H > 65535) return failf(KB2SEQ_ERR_VALUE, "gla: too many heads");
  const bool aligned = ((uintptr_t)qkv & 15) == 0 && (ld & 3) == 0 && (q_off & 3) == 0 && (k_off & 3) == 0 && (v_off & 3) == 0 &&
                       scratch != nullptr && ((uintptr_t)scratch & 15) == 0;
  if (aligned && (dk == 32 || dk == 64 || dk == 128 || dk == 256) && dv % 32 == 0 && dv / 32 <= 65535) {
    cudaStream_t st0 = (cudaStream_t)stream;
    const long long ne = (long long)T * H * dk;
    gla_decay_kernel<<<(unsigned)((ne + 255) / 256), 256, 0, st0>>>(decay_in, lda, decay_bias, 1.f / tau, T, H * dk, scratch);
    SEQ_LAUNCHED();
    if (dk == 32) return launch_gla_reg<32>(qkv, ld, q_off, k_off, v_off, scratch, q_scale, S, H, dv, state, cu, slots, out, st0);
    if (dk == 64) return launch_gla_reg<64>(qkv, ld, q_off, k_off, v_off, scratch, q_scale, S, H, dv, state, cu, slots, out, st0);
    if (dk == 128) return launch_gla_reg<128>(qkv, ld, q_off, k_off, v_off, scratch, q_scale, S, H, dv, state, cu, slots, out, st0);
    return launch_gla_reg<256>(qkv, ld, q_off, k_off, v_off, scratch, q_scale, S, H, dv, state, cu, slots, out, st0);
  }
  // P lanes share a value column; each keeps at most 32 (16 for small heads) of its rows
  int P = 1;
  while ((dk + P - 1) / P > 32) P <<= 1;
  const int KR = (dk + P - 1) / P;
  const int CB = (kRecThreads / 32) * (32 / P);
  const size_t smem = (size_t)(4 * kRecTok * dk + kRecTok * CB) * 4;
  dim3 grid(S, H, (dv + CB - 1) / CB);
  cudaStream_t st = (cudaStream_t)stream;
  if (smem > 48 * 1024) {
    SEQ_CUDA(cudaFuncSetAttribute(gla_scan_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SEQ_CUDA(cudaFuncSetAttribute(gla_scan_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  if (KR <= 16)
    gla_scan_kernel<16><<<grid, kRecThreads, smem, st>>>(qkv, ld, q_off, k_off, v_off, decay_in, lda, decay_bias, 1.f / tau, q_scale, H, dk, dv,
                                                         P, state, cu, slots, out);
  else
    gla_scan_kernel<32><<<grid, kRecThreads, smem, st>>>(qkv, ld, q_off, k_off, v_off, decay_in, lda, decay_bias, 1.f / tau, q_scale, H, dk, dv,
                                                         P, state, cu, slots, out);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_selective_scan(const float* x, long long ldx, const float* dt_in, long long ldd, const float* dt_bias, const float* bc,
                                      long long ldb, int b_off, const float* z, long long ldz, int z_off, const float* A_log,
                                      const float* D, int T, int S, int inner, int N, float* state, const int* cu, const int* slots,
                                      void* out, int dt_out, void* stream) {
  if (!x || !dt_in || !dt_bias || !bc || !z || !A_log || !D || !state || !cu || !slots || !out || T <= 0 || S <= 0 || inner <= 0 || N <= 0 ||
      bad_dt(dt_out))
    return failf(KB2SEQ_ERR_VALUE, "selective_scan: bad argument");
  if (N > 256) return failf(KB2SEQ_ERR_VALUE, "selective_scan: state size %d > 256", N);
  const int NR = N <= 32 ? 1 : (N <= 64 ? 2 : (N <= 128 ? 4 : 8));
  const int P = pow2_at_least((N + NR - 1) / NR);
  const int CB = (kRecThreads / 32) * (32 / P);
  const size_t smem = (size_t)(2 * kRecTok * 2 * N + 3 * 2 * kRecTok * CB + kRecTok * CB * (P + 1)) * 4;
  dim3 grid(S, (inner + CB - 1) / CB);
  cudaStream_t st = (cudaStream_t)stream;
#define KB2_SCAN(NRV)                                                                                                                  \
  if (smem > 48 * 1024) SEQ_CUDA(cudaFuncSetAttribute(selective_scan_kernel<NRV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
  selective_scan_kernel<NRV><<<grid, kRecThreads, smem, st>>>(x, ldx, dt_in, ldd, dt_bias, bc, ldb, b_off, z, ldz, z_off, A_log, D, inner, N, \
                                                              P, state, cu, slots, out, dt_out)
  if (NR == 1) { KB2_SCAN(1); } else if (NR == 2) { KB2_SCAN(2); } else if (NR == 4) { KB2_SCAN(4); } else { KB2_SCAN(8); }
#undef KB2_SCAN
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_head_norm_gate(const float* o, long long ldo, const float* w, float eps, const float* gate, long long ldg, int gate_act,
                                      int T, int H, int dv, void* out, int dt_out, void* stream) {
  if (!o || !out || T <= 0 || H <= 0 || dv <= 0 || bad_dt(dt_out) || gate_act < 0 || gate_act > 1)
    return failf(KB2SEQ_ERR_VALUE, "head_norm_gate: bad argument");
  const long long nw = (long long)T * H;
  head_norm_gate_kernel<<<(unsigned)((nw + 7) / 8), 256, 0, (cudaStream_t)stream>>>(o, ldo, w, eps, gate, ldg, gate_act, H, dv, T, out, dt_out);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_rms_rows(const float* in, long long ld_in, int n, const float* w, float eps, void* out, int dt_out, long long ld_out,
                                int T, void* stream) {
  if (!in || !w || !out || T <= 0 || n <= 0 || bad_dt(dt_out)) return failf(KB2SEQ_ERR_VALUE, "rms_rows: bad argument");
  rms_rows_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(in, ld_in, n, w, eps, out, dt_out, ld_out);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_branch_merge(const float* a, const float* b, const float* wa, const float* wb, float eps, float coef, float* out, int T,
                                    int W, void* stream) {
  if (!a || !b || !wa || !wb || !out || T <= 0 || W <= 0) return failf(KB2SEQ_ERR_VALUE, "branch_merge: bad argument");
  branch_merge_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(a, b, wa, wb, eps, coef, out, W);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_depth_mix(float* stack, long long stride, int n, const float* coef, float* x, const float* y, const float* w, void* h,
                                 int dt_h, int T, int W, float eps, void* stream) {
  if (!stack || !coef || !x || n <= 0 || T <= 0 || W <= 0 || (w && (!h || bad_dt(dt_h)))) return failf(KB2SEQ_ERR_VALUE, "depth_mix: bad argument");
  depth_mix_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(stack, stride, n, coef, x, y, w, h, dt_h, W, eps);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

}  // extern "C"
