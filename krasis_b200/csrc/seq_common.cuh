// Shared by the translation units of libkrasis_b200_seq.so: error text and launch counter, launch-check macros, dtype-generic loads
// and stores (`dt` codes: 0 = float32, 1 = bfloat16), warp / block reductions, activations.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/krasis_b200_seq.h"

namespace kb2seq {

typedef __nv_bfloat16 bf16;

extern thread_local char g_err[512];
extern long long g_launches;

inline int failf(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define SEQ_CUDA(expr)                                                                              \
  do {                                                                                              \
    cudaError_t _e = (expr);                                                                        \
    if (_e != cudaSuccess) return failf(KB2SEQ_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)
#define SEQ_LAUNCHED()                                                                                       \
  do {                                                                                                       \
    ++g_launches;                                                                                            \
    cudaError_t _e = cudaGetLastError();                                                                     \
    if (_e != cudaSuccess) return failf(KB2SEQ_ERR_CUDA, "launch at line %d: %s", __LINE__, cudaGetErrorString(_e)); \
  } while (0)

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float ld_dt(const void* p, int dt, long long i) {
  return dt ? __bfloat162float(((const bf16*)p)[i]) : ((const float*)p)[i];
}
__device__ __forceinline__ void st_dt(void* p, int dt, long long i, float v) {
  if (dt) ((bf16*)p)[i] = __float2bfloat16_rn(v); else ((float*)p)[i] = v;
}

// eight bf16 values of one 16-byte load
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }
// Per-token decay exp(-exp(A_log) * softplus(a + dt_bias)).  A recurrent state multiplies by it at every token, so a rounding bias of
// the fp32 exp / log1p chain (a fraction of an ulp, but of one sign) would grow linearly with the distance to a far token; evaluated in
// fp64 and rounded once, the fp32 decay carries only its own unbiased half ulp.
__device__ __forceinline__ float decay_from_rate(double rate, float a, float dt_bias) {      // rate = exp(A_log) in fp64
  const double z = (double)a + (double)dt_bias;
  const double sp = z > 40.0 ? z : log1p(exp(z));
  return (float)exp(-rate * sp);
}
__device__ __forceinline__ float decay_of(float a_log, float a, float dt_bias) { return decay_from_rate(exp((double)a_log), a, dt_bias); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// sum over the block; `red` holds 32 floats; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

// Rotation angle pos * freq reduced in fp64, sin / cos in fp32.
__device__ __forceinline__ void rot_cs(int pos, double freq, float amp, float* c, float* s) {
  double a = (double)pos * freq;
  a -= 6.283185307179586476925286766559 * rint(a * 0.15915494309189533576888376337251);
  float sf, cf;
  sincosf((float)a, &sf, &cf);
  *c = cf * amp;
  *s = sf * amp;
}

inline bool bad_dt(int dt) { return dt != 0 && dt != 1; }

}  // namespace kb2seq
