// Ragged-batch sequence operators, third part: linear recurrences with per-sequence state slots and the small row kernels of
// designs that run several mixers side by side or average their residual stream over depth.
//
//   gla_scan               gated linear attention, S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t per head, with one decay per key
//                          channel alpha = sigmoid(z)^(1 / tau); the state of a (sequence, head, slice of value columns) lives in
//                          registers, P lanes share a column and each keeps dk / P of its rows
//   selective_scan         S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n, y_c = sum_n S[c, n] C_n + D_c x_c, times silu(z);
//                          the lanes of a channel keep its states in registers
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

// ------------------------------------------------------------------------------------------------ selective scan
// x [T, ldx] (inner channels after convolution and activation), dt_in [T, ldd] (+ dt_bias, then softplus), bc [T, ldb] = [B: N | C: N]
// from b_off, z [T, ldz] from z_off, A_log [inner, N], D [inner].  Block (sequence, group of CB channels); lane l: state slice
// p = l % P, channel l / P of the warp; thread states are n = p + P ii, ii < NR.
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
  float2* bcs = reinterpret_cast<float2*>(sm);              // [kRecTok][N]: (B_n, C_n)
  float2* dx = reinterpret_cast<float2*>(sm + 2 * kRecTok * N);   // [kRecTok][CB]: (dt_c, x_c)
  const int s = blockIdx.x, c0 = blockIdx.y * CB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int p = lane % P, cl = warp * CW + lane / P, c = c0 + cl;
  const bool live = c < inner;
  const int row0 = cu[s], n = cu[s + 1] - row0;
  float* S = state + (long long)slots[s] * inner * N;
  float st[NR], a[NR];
#pragma unroll
  for (int ii = 0; ii < NR; ++ii) {
    const int j = p + P * ii;
    const bool ok = live && j < N;
    st[ii] = ok ? S[(long long)c * N + j] : 0.f;
    a[ii] = ok ? -expf(A_log[(long long)c * N + j]) : 0.f;
  }
  const float dw = live ? Dw[c] : 0.f;
  for (int t0 = 0; t0 < n; t0 += kRecTok) {
    const int nt = min(kRecTok, n - t0);
    __syncthreads();
    for (int e = tid; e < nt * N; e += kRecThreads) {
      const int tt = e / N, j = e - tt * N;
      const float* r = bc + (long long)(row0 + t0 + tt) * ldb + b_off;
      bcs[e] = make_float2(r[j], r[N + j]);
    }
    for (int e = tid; e < nt * CB; e += kRecThreads) {
      const int tt = e / CB, cc = e - tt * CB;
      const long long t = row0 + t0 + tt;
      float2 f = make_float2(0.f, 0.f);
      if (c0 + cc < inner) {
        f.x = softplus_f(dt_in[t * ldd + c0 + cc] + dt_bias[c0 + cc]);
        f.y = x[t * ldx + c0 + cc];
      }
      dx[e] = f;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float2 f = dx[tt * CB + cl];
      const float dtx = f.x * f.y;
      const float2* row = bcs + tt * N;
      float y = 0.f;
#pragma unroll
      for (int ii = 0; ii < NR; ++ii) {
        const int j = p + P * ii;
        if (j < N) {
          const float2 g = row[j];
          st[ii] = fmaf(expf(f.x * a[ii]), st[ii], dtx * g.x);
          y = fmaf(st[ii], g.y, y);
        }
      }
      for (int off = 1; off < P; off <<= 1) y += __shfl_xor_sync(0xffffffffu, y, off);
      if (p == 0 && live) {
        const long long t = row0 + t0 + tt;
        y = fmaf(dw, f.y, y);
        st_dt(out, dt_out, t * inner + c, y * silu(z[t * ldz + z_off + c]));
      }
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

}  // namespace kb2seq

using namespace kb2seq;

extern "C" {

KB2SEQ_API int kb2_seq_gla(const float* qkv, long long ld, int q_off, int k_off, int v_off, const float* decay_in, long long lda,
                           const float* decay_bias, float tau, float q_scale, int T, int S, int H, int dk, int dv, float* state,
                           const int* cu, const int* slots, float* out, void* stream) {
  if (!qkv || !decay_in || !state || !cu || !slots || !out || T <= 0 || S <= 0 || H <= 0 || dk <= 0 || dv <= 0 || !(tau > 0.f))
    return failf(KB2SEQ_ERR_VALUE, "gla: bad argument");
  if (dk > 1024) return failf(KB2SEQ_ERR_VALUE, "gla: key size %d > 1024", dk);
  if (H > 65535) return failf(KB2SEQ_ERR_VALUE, "gla: too many heads");
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
  const size_t smem = (size_t)(2 * kRecTok * N + 2 * kRecTok * CB) * 4;
  dim3 grid(S, (inner + CB - 1) / CB);
  cudaStream_t st = (cudaStream_t)stream;
#define KB2_SCAN(NRV)                                                                                                                  \
  selective_scan_kernel<NRV><<<grid, kRecThreads, smem, st>>>(x, ldx, dt_in, ldd, dt_bias, bc, ldb, b_off, z, ldz, z_off, A_log, D, inner, N, \
                                                              P, state, cu, slots, out, dt_out)
  if (NR == 1) KB2_SCAN(1); else if (NR == 2) KB2_SCAN(2); else if (NR == 4) KB2_SCAN(4); else KB2_SCAN(8);
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
