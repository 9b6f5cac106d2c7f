// Ragged-batch sequence operators, second part: per-head key/value caches, multi-map (differential) attention over a page list with
// a causal mask that may be cut into chunks and / or a sliding window, gated linear units, and routed experts.
//
//   head_kv_prep           bias, RMS norm (per vector, or one over the whole of q and one over the whole of k) and rotary positions
//                          (pairs 2i / 2i + 1, or i / i + dims / 2) on the query and key vectors of every head and map; keys and
//                          values go to the paged cache rows of the tokens' positions; optionally the values are rotated by their
//                          positions over all of their dimensions
//   kv_pool                the tokens that complete a block of `pool` positions write the mean of the block's cached keys and values
//                          into pooled pools that share the page numbering
//   paged_attn             softmax attention of every (head, map) query vector over the cached keys of its key/value head; the maps of
//                          a head have keys of their own and share the values; keys j <= i of the same chunk and inside the window;
//                          optional tanh cap on the scaled scores; optional sink per head in the denominator; optionally one pooled
//                          key / value per block that lies wholly before the window, in the same softmax;
//                          for steps of few tokens the key range is cut into pieces that run as separate blocks
//   pool_merge             joins the pooled blocks' piece to a tensor-core result over the window by the two log-sum-exps
//   attn_finish            merges the pieces, combines the maps with per-map coefficients (differential attention: 1, -lambda),
//                          unit RMS norm per head, turning rotated values back by the query's position, output gate sigmoid(g) per
//                          head or per element
//   glu                    act(gate) * up in three flavours (tanh-GELU, SiLU, clamped swish with up + 1), or relu^2 without an up half
//   route_topk             scores (softmax or sigmoid) -> + correction -> best groups (by their best or two best members) -> top-k
//                          -> weights
//   moe_bin / moe_gemm / moe_gemv / moe_combine
//                          tokens binned per expert in tiles of 64 rows, tile GEMMs that pick their expert's weights, a GEMV form for
//                          steps of few tokens, and the weighted sum over a token's experts (identity experts return the input)
//                          plus the shared expert's rows, optionally times a per-token sigmoid gate
//
// Precision: scores, softmax, norms, rotary angles, router and every accumulation are fp32; `dt` selects storage only.
#include "seq_common.cuh"

namespace kb2seq {

// ------------------------------------------------------------------------------------------------ query / key / value preparation
// proj [T, ldp] fp32 = [q: H x M x d | k: G x M x d | v: G x dv | ...] (G == 0: the layer reads another layer's cache and has no k, v).
// A warp per vector of d.  norm_whole 0: every vector is normed by itself with the weight qw / kw [d]; 1: one root mean square over all
// of q (and one over all of k) with weights of the projection's size.  rot_half 0: dimension 2j turns with 2j + 1; 1: j with
// j + rot_dims / 2.
__global__ void __launch_bounds__(256) head_kv_prep_kernel(float* __restrict__ proj, long long ldp, int H, int G, int M, int d, int dv,
                                                           const float* __restrict__ bias, const float* __restrict__ qw,
                                                           const float* __restrict__ kw, float eps, const double* __restrict__ freq,
                                                           int rot_dims, const int* __restrict__ positions,
                                                           const int* __restrict__ seq_of, const int* __restrict__ pages, int max_pages,
                                                           int page_size, void* __restrict__ kc, void* __restrict__ vc, int dt_cache,
                                                           int norm_whole, int rot_half, const double* __restrict__ vfreq) {
  extern __shared__ float rot_tab[];          // [rot_dims / 2][2]: cos, sin of the token's position, shared by all its vectors
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const int pos = positions[t];
  float* p = proj + t * ldp;
  const long long slot = (long long)pages[(long long)seq_of[t] * max_pages + pos / page_size] * page_size + pos % page_size;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int nq = H * M, nvec = (H + G) * M, half = rot_dims >> 1;
  for (int j = threadIdx.x; j < half; j += blockDim.x) rot_cs(pos, freq[j], 1.f, &rot_tab[2 * j], &rot_tab[2 * j + 1]);
  float rstd_q = 1.f, rstd_k = 1.f;
  if (norm_whole) {
    const int nqe = nq * d, nke = (nvec - nq) * d;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nqe + nke; i += blockDim.x) {
      const float v = p[i] + (bias ? bias[i] : 0.f);
      if (i < nqe) sq = fmaf(v, v, sq); else sk = fmaf(v, v, sk);
    }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    if (qw != nullptr) rstd_q = 1.f / sqrtf(sq / (float)nqe + eps);
    if (kw != nullptr && nke > 0) rstd_k = 1.f / sqrtf(sk / (float)nke + eps);
  }
  __syncthreads();
  for (int vi = warp; vi < nvec; vi += nw) {
    const bool is_q = vi < nq;
    float* x = p + (long long)vi * d;
    const float* b = bias ? bias + (long long)vi * d : nullptr;
    const float* w = is_q ? qw : kw;
    if (norm_whole && w != nullptr) w += (long long)(is_q ? vi : vi - nq) * d;
    float rstd = 1.f;
    if (norm_whole) {
      rstd = is_q ? rstd_q : rstd_k;
    } else if (w != nullptr) {
      float ss = 0.f;
      for (int i = lane; i < d; i += 32) {
        const float v = x[i] + (b ? b[i] : 0.f);
        ss += v * v;
      }
      ss = warp_sum(ss);
      rstd = 1.f / sqrtf(ss / (float)d + eps);
    }
    const long long krow = (slot * G * M + (vi - nq)) * d;      // used for keys only
    for (int j = lane; j < half; j += 32) {
      const int iu = rot_half ? j : 2 * j, iv = rot_half ? j + half : 2 * j + 1;
      float u = x[iu] + (b ? b[iu] : 0.f), v = x[iv] + (b ? b[iv] : 0.f);
      u *= rstd;
      v *= rstd;
      if (w != nullptr) {
        u *= w[iu];
        v *= w[iv];
      }
      const float c = rot_tab[2 * j], s = rot_tab[2 * j + 1];
      const float ru = u * c - v * s, rv = v * c + u * s;
      if (is_q) {
        x[iu] = ru;
        x[iv] = rv;
      } else {
        st_dt(kc, dt_cache, krow + iu, ru);
        st_dt(kc, dt_cache, krow + iv, rv);
      }
    }
    for (int i = rot_dims + lane; i < d; i += 32) {
      float v = (x[i] + (b ? b[i] : 0.f)) * rstd;
      if (w != nullptr) v *= w[i];
      if (is_q) x[i] = v; else st_dt(kc, dt_cache, krow + i, v);
    }
  }
  const long long v0 = (long long)nvec * d;
  if (vfreq == nullptr) {
    for (int i = threadIdx.x; i < G * dv; i += blockDim.x)
      st_dt(vc, dt_cache, slot * G * dv + i, p[v0 + i] + (bias ? bias[v0 + i] : 0.f));
    return;
  }
  // rotated values: every pair of the value vector turns by position * vfreq[pair], in the pair layout of the keys
  const int vh = dv >> 1;
  for (int i = threadIdx.x; i < G * vh; i += blockDim.x) {
    const int g = i / vh, j = i - g * vh;
    const int iu = rot_half ? j : 2 * j, iv = rot_half ? j + vh : 2 * j + 1;
    const long long b0 = v0 + (long long)g * dv;
    const float u = p[b0 + iu] + (bias ? bias[b0 + iu] : 0.f), v = p[b0 + iv] + (bias ? bias[b0 + iv] : 0.f);
    float c, sn;
    rot_cs(pos, vfreq[j], 1.f, &c, &sn);
    st_dt(vc, dt_cache, (slot * G + g) * dv + iu, u * c - v * sn);
    st_dt(vc, dt_cache, (slot * G + g) * dv + iv, v * c + u * sn);
  }
}

// ------------------------------------------------------------------------------------------------ pooled blocks
// A block of `pool` consecutive positions b pool .. b pool + pool - 1 is summarised by the mean of its cached keys and the mean of its
// cached values.  The summary of block b lives in the page of the block's last position: pooled pools have rows_per_page =
// ceil(page_size / pool) rows per page, and block b is row b - floor(page first position / pool) of that page.
__device__ __forceinline__ long long pooled_row(int b, int pool, int page_size, int rows_per_page, const int* __restrict__ seq_pages) {
  const int pg = (b * pool + pool - 1) / page_size;
  return (long long)seq_pages[pg] * rows_per_page + (b - pg * page_size / pool);
}

// One block per token of the step; only a token that completes a block works: it averages the block's cache rows (fp32, in position
// order) into the pooled pools.  Runs after head_kv_prep of the same step.
__global__ void __launch_bounds__(256) kv_pool_kernel(const void* __restrict__ kc, const void* __restrict__ vc, void* __restrict__ kp,
                                                      void* __restrict__ vp, int dt_cache, int kw, int vw, int pool, int rows_per_page,
                                                      const int* __restrict__ positions, const int* __restrict__ seq_of,
                                                      const int* __restrict__ pages, int max_pages, int page_size) {
  const long long t = blockIdx.x;
  const int pos = positions[t];
  if (pos % pool != pool - 1) return;
  const int* sp = pages + (long long)seq_of[t] * max_pages;
  const long long dst = pooled_row(pos / pool, pool, page_size, rows_per_page, sp);
  const float inv = 1.f / (float)pool;
  for (int i = threadIdx.x; i < kw + vw; i += blockDim.x) {
    const bool is_k = i < kw;
    const int c = is_k ? i : i - kw, wdt = is_k ? kw : vw;
    const void* src = is_k ? kc : vc;
    float acc = 0.f;
    for (int j = pos - pool + 1; j <= pos; ++j) {
      const long long row = (long long)sp[j / page_size] * page_size + j % page_size;
      acc += ld_dt(src, dt_cache, row * wdt + c);
    }
    st_dt(is_k ? kp : vp, dt_cache, dst * wdt + c, acc * inv);
  }
}

// ------------------------------------------------------------------------------------------------ attention over the page list
// One block per (token, key/value head g, piece of the rows that share g, piece of the key range).  The rows of g are its H / G query
// heads times M maps; row r is head g (H / G) + r / M, map r % M, and reads the keys of map r % M.  Keys in tiles of 32.
constexpr int kPAThreads = 256, kPAAcc = 16, kPAKT = 32;
__global__ void __launch_bounds__(kPAThreads) paged_attn_kernel(
    const float* __restrict__ proj, long long ldp, int H, int G, int M, int d, int dv, int RB, const void* __restrict__ kc,
    const void* __restrict__ vc, int dt_cache, const int* __restrict__ positions, const int* __restrict__ seq_of,
    const int* __restrict__ pages, int max_pages, int page_size, float scale, int chunk, int window, float* __restrict__ out, int nsplit,
    float* __restrict__ part_acc, float* __restrict__ part_ml, const int* __restrict__ cu, int skip_from, float softcap,
    const float* __restrict__ sinks, int pool, int rows_per_page, const void* __restrict__ kp, const void* __restrict__ vp, int pool_only) {
  extern __shared__ __align__(16) float sm[];
  constexpr int KT = kPAKT;
  const long long t = blockIdx.x;
  const int seq = seq_of[t];
  // long portions are served by the tensor-core kernel; pool_only is the second pass over exactly those: the pooled blocks alone, left
  // as an unnormalised piece (running maximum, sum, weighted values) that pool_merge joins to the tensor-core result
  if (cu != nullptr && (cu[seq + 1] - cu[seq] >= skip_from) != (pool_only != 0)) return;
  const int R = (H / G) * M, nrb = (R + RB - 1) / RB;
  const int g = blockIdx.y / nrb, r0 = (blockIdx.y - g * nrb) * RB, nr = min(RB, R - r0);
  const int KD = M * d, KP = KD | 1;         // odd row pitch: a lane per key reads without bank conflicts
  long long* krow = (long long*)sm;          // [KT]
  float* qs = sm + 2 * KT;                   // [RB][d]
  float* kt = qs + RB * d;                   // [KT][KP]
  float* vt = kt + KT * KP;                  // [KT][dv]
  float* pr = vt + KT * dv;                  // [RB][KT]
  float* m_run = pr + RB * KT;               // [RB]
  float* l_run = m_run + RB;
  float* alpha = l_run + RB;
  const int pos = positions[t];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < nr * d; i += kPAThreads) {
    const int r = i / d, dd = i - r * d;
    qs[i] = proj[t * ldp + ((long long)g * R + r0 + r) * d + dd];
  }
  const int z = blockIdx.z;
  if (tid < nr) {          // a sink is a key without a value: the running maximum starts at it, the running sum at 1 (first piece only)
    const bool sk = sinks != nullptr && z == 0 && !pool_only;
    m_run[tid] = sk ? sinks[g * (H / G) + (r0 + tid) / M] : -INFINITY;
    l_run[tid] = sk ? 1.f : 0.f;
  }
  float acc[kPAAcc];
#pragma unroll
  for (int a = 0; a < kPAAcc; ++a) acc[a] = 0.f;
  int j_lo = max(0, pos - window + 1);
  if (chunk > 0) j_lo = max(j_lo, pos / chunk * chunk);
  // the keys of a token, in order: the pooled blocks that lie wholly before the window (block b: b pool + pool - 1 <= pos - window),
  // then the positions j_lo .. pos.  Index u of that list: u < nb is block u, else position j_lo + u - nb.
  const int nb = pool > 0 ? max(0, pos - window + 1) / pool : 0;
  const int total = pool_only ? nb : nb + pos - j_lo + 1;
  int u_begin = 0, u_end = total - 1;
  if (nsplit > 1) {
    const int piece = ((total + nsplit - 1) / nsplit + KT - 1) / KT * KT;
    u_begin = z * piece;
    u_end = min(total - 1, u_begin + piece - 1);
  }
  const int* sp = pages + (long long)seq * max_pages;
  for (int j0 = u_begin; j0 <= u_end; j0 += KT) {
    const int nk = min(KT, u_end - j0 + 1);
    __syncthreads();
    if (tid < nk) {
      const int u = j0 + tid;
      if (u < nb) {
        krow[tid] = -1 - pooled_row(u, pool, page_size, rows_per_page, sp);      // negative: a row of the pooled pools
      } else {
        const int j = j_lo + u - nb;
        krow[tid] = (long long)sp[j / page_size] * page_size + j % page_size;
      }
    }
    __syncthreads();
    if (dt_cache == 1 && (KD & 7) == 0 && (dv & 7) == 0) {
      const int K8 = KD >> 3, V8 = dv >> 3;
      for (int i = tid; i < nk * (K8 + V8); i += kPAThreads) {
        const int k = i / (K8 + V8), c = i - k * (K8 + V8);
        float f[8];
        const bool pooled = krow[k] < 0;
        const long long row = pooled ? -1 - krow[k] : krow[k];
        if (c < K8) {
          unpack8(*reinterpret_cast<const uint4*>((const bf16*)(pooled ? kp : kc) + (row * G + g) * KD + c * 8), f);
#pragma unroll
          for (int e = 0; e < 8; ++e) kt[k * KP + c * 8 + e] = f[e];
        } else {
          unpack8(*reinterpret_cast<const uint4*>((const bf16*)(pooled ? vp : vc) + (row * G + g) * dv + (c - K8) * 8), f);
#pragma unroll
          for (int e = 0; e < 8; ++e) vt[k * dv + (c - K8) * 8 + e] = f[e];
        }
      }
    } else {
      for (int i = tid; i < nk * KD; i += kPAThreads) {
        const int k = i / KD, c = i - k * KD;
        const bool pooled = krow[k] < 0;
        kt[k * KP + c] = ld_dt(pooled ? kp : kc, dt_cache, ((pooled ? -1 - krow[k] : krow[k]) * G + g) * KD + c);
      }
      for (int i = tid; i < nk * dv; i += kPAThreads) {
        const int k = i / dv, c = i - k * dv;
        const bool pooled = krow[k] < 0;
        vt[i] = ld_dt(pooled ? vp : vc, dt_cache, ((pooled ? -1 - krow[k] : krow[k]) * G + g) * dv + c);
      }
    }
    __syncthreads();
    // scores: a lane per key, a warp per row
    for (int r = warp; r < nr; r += kPAThreads / 32) {
      float sc = -INFINITY;
      if (lane < nk) {
        const float* qh = qs + r * d;
        const float* kk = kt + lane * KP + ((r0 + r) % M) * d;
        float dot = 0.f;
        for (int dd = 0; dd < d; ++dd) dot = fmaf(qh[dd], kk[dd], dot);
        sc = dot * scale;
        if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
      }
      const float m_old = m_run[r];
      const float m_new = fmaxf(m_old, warp_max(sc));
      const float pv = lane < nk ? expf(sc - m_new) : 0.f;
      pr[r * KT + lane] = pv;
      const float lsum = warp_sum(pv);
      if (lane == 0) {
        const float al = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
        alpha[r] = al;
        l_run[r] = l_run[r] * al + lsum;
        m_run[r] = m_new;
      }
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < kPAAcc; ++a) {
      const int i = tid + a * kPAThreads;
      if (i < nr * dv) {
        const int r = i / dv, c = i - r * dv;
        float v = acc[a] * alpha[r];
        const float* ph = pr + r * KT;
        for (int k = 0; k < nk; ++k) v = fmaf(ph[k], vt[k * dv + c], v);
        acc[a] = v;
      }
    }
  }
  __syncthreads();
  const long long row0 = (t * G + g) * R + r0;       // (t, h, m) in row-major order
#pragma unroll
  for (int a = 0; a < kPAAcc; ++a) {
    const int i = tid + a * kPAThreads;
    if (i < nr * dv) {
      const int r = i / dv, c = i - r * dv;
      if (nsplit > 1 || pool_only) part_acc[((row0 + r) * nsplit + z) * dv + c] = acc[a];
      else out[(row0 + r) * dv + c] = acc[a] / l_run[r];
    }
  }
  if ((nsplit > 1 || pool_only) && tid < nr) {
    part_ml[((row0 + tid) * nsplit + z) * 2] = m_run[tid];
    part_ml[((row0 + tid) * nsplit + z) * 2 + 1] = l_run[tid];
  }
}

// A warp per (token, head): o = sum_m coef[m] a_m (a_m merged from its key pieces when nsplit > 1), o / rms(o) * post_scale if
// unit_norm, times sigmoid(gate[t, h]) if gates are given.  dv <= 32 * kFinAcc.
constexpr int kFinAcc = 16;
__global__ void __launch_bounds__(256) attn_finish_kernel(const float* __restrict__ a, const float* __restrict__ part_acc,
                                                          const float* __restrict__ part_ml, int nsplit, long long T, int H, int M, int dv,
                                                          const float* __restrict__ coef, int unit_norm, float eps, float post_scale,
                                                          const float* __restrict__ gate, long long ldg, void* __restrict__ out,
                                                          int dt_out, const int* __restrict__ seq_of, const int* __restrict__ cu,
                                                          int skip_from, int gate_wide, const int* __restrict__ positions,
                                                          const double* __restrict__ vfreq, int rot_half) {
  __shared__ float turn_buf[8][32 * kFinAcc];
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= T * H) return;
  const long long t = w / H;
  const int h = (int)(w - t * H);
  if (cu != nullptr) {
    const int sq = seq_of[t];
    if (cu[sq + 1] - cu[sq] >= skip_from) return;
  }
  float o[kFinAcc];
#pragma unroll
  for (int i = 0; i < kFinAcc; ++i) o[i] = 0.f;
  for (int m = 0; m < M; ++m) {
    const long long row = w * M + m;
    const float cm = coef ? coef[m] : 1.f;
    if (nsplit > 1) {                        // the pieces' maxima and sums are spread over the lanes; weights travel by shuffle
      float mx = -INFINITY;
      for (int z = lane; z < nsplit; z += 32) mx = fmaxf(mx, part_ml[(row * nsplit + z) * 2]);
      mx = warp_max(mx);
      float den = 0.f;
      for (int z = lane; z < nsplit; z += 32) {
        const float mz = part_ml[(row * nsplit + z) * 2];
        if (mz != -INFINITY) den += expf(mz - mx) * part_ml[(row * nsplit + z) * 2 + 1];
      }
      den = warp_sum(den);
      for (int z0 = 0; z0 < nsplit; z0 += 32) {
        float wl = 0.f;
        if (z0 + lane < nsplit) {
          const float mz = part_ml[(row * nsplit + z0 + lane) * 2];
          if (mz != -INFINITY) wl = expf(mz - mx) / den * cm;
        }
        const int nz = min(32, nsplit - z0);
        // an empty piece holds zeros and has weight 0, so nothing is skipped and the loads of several pieces are in flight together
#pragma unroll 8
        for (int k = 0; k < nz; ++k) {
          const float wz = __shfl_sync(0xffffffffu, wl, k);
#pragma unroll
          for (int i = 0; i < kFinAcc; ++i) {
            const int c = lane + 32 * i;
            if (c < dv) o[i] = fmaf(wz, part_acc[(row * nsplit + z0 + k) * dv + c], o[i]);
          }
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < kFinAcc; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) o[i] = fmaf(cm, a[row * dv + c], o[i]);
      }
    }
  }
  float f = 1.f;
  if (unit_norm) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kFinAcc; ++i) ss += o[i] * o[i];
    ss = warp_sum(ss);
    f = post_scale / sqrtf(ss / (float)dv + eps);
  }
  if (vfreq != nullptr) {       // values were cached rotated by their positions: turn the sum back by the query's position
    float* tb = turn_buf[threadIdx.x >> 5];
#pragma unroll
    for (int i = 0; i < kFinAcc; ++i) {
      const int c = lane + 32 * i;
      if (c < dv) tb[c] = o[i];
    }
    __syncwarp();
    const int vh = dv >> 1, pos = positions[t];
#pragma unroll
    for (int i = 0; i < kFinAcc; ++i) {
      const int c = lane + 32 * i;
      if (c < dv) {
        const int j = rot_half ? (c < vh ? c : c - vh) : c >> 1;
        const bool first = rot_half ? c < vh : !(c & 1);
        const float other = tb[rot_half ? (first ? c + vh : c - vh) : c ^ 1];
        float cs, sn;
        rot_cs(pos, vfreq[j], 1.f, &cs, &sn);
        o[i] = first ? o[i] * cs + other * sn : o[i] * cs - other * sn;      // the turn by -pos * f
      }
    }
  }
  if (gate != nullptr && !gate_wide) f *= 1.f / (1.f + expf(-gate[t * ldg + h]));
#pragma unroll
  for (int i = 0; i < kFinAcc; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) {
      float v = o[i] * f;
      if (gate != nullptr && gate_wide) v *= 1.f / (1.f + expf(-gate[t * ldg + (long long)h * dv + c]));
      st_dt(out, dt_out, w * dv + c, v);
    }
  }
}

// a[t, h, :] is a normalised attention output whose softmax denominator has the logarithm lse[t, h]; (part_acc, part_ml) is an
// unnormalised piece over further keys (running maximum m, sum l, weighted values).  Both are joined into one softmax, in place.
// A warp per (token, head); only sequences whose portion has at least min_portion tokens.
__global__ void __launch_bounds__(256) pool_merge_kernel(float* __restrict__ a, const float* __restrict__ lse, const float* __restrict__ part_acc,
                                                         const float* __restrict__ part_ml, long long rows, int H, int dv,
                                                         const int* __restrict__ seq_of, const int* __restrict__ cu, int min_portion) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= rows) return;
  const int sq = seq_of[w / H];
  if (cu[sq + 1] - cu[sq] < min_portion) return;
  const float mp = part_ml[w * 2], lp = part_ml[w * 2 + 1];
  if (!(lp > 0.f)) return;                              // no pooled block is visible yet
  const float lw = lse[w];
  const float top = fmaxf(lw, mp);
  const float ww = lw == -INFINITY ? 0.f : expf(lw - top), wp = expf(mp - top);
  const float inv = 1.f / (ww + lp * wp);
  for (int c = lane; c < dv; c += 32) a[w * dv + c] = (a[w * dv + c] * ww + part_acc[w * dv + c] * wp) * inv;
}

// ------------------------------------------------------------------------------------------------ gated linear units
// in [rows, 2 F] = [gate | up].  kind 0: gelu_tanh(g) u; 1: silu(g) u; 2: g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit),
// u' = clamp(u, -limit, limit); 3: relu(g)^2 of in [rows, F] alone (no up half).  With n_tiles given only the first
// n_tiles[0] * tile_rows rows are computed.
__device__ __forceinline__ float glu_value(float g, float u, int kind, float limit, float alpha) {
  if (kind == 3) return g > 0.f ? g * g : 0.f;
  if (kind == 0) return gelu_tanh(g) * u;
  if (kind == 1) return silu(g) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + 1.f);
}
__global__ void glu_kernel(const void* __restrict__ in, int dt_in, long long ld_in, void* __restrict__ out, int dt_out, long long rows, int F,
                           int kind, float limit, float alpha, const int* __restrict__ n_tiles, int tile_rows) {
  if (n_tiles != nullptr) rows = min(rows, (long long)n_tiles[0] * tile_rows);
  const long long n = rows * F;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / F;
    const int f = (int)(i - r * F);
    st_dt(out, dt_out, i, glu_value(ld_dt(in, dt_in, r * ld_in + f), kind == 3 ? 0.f : ld_dt(in, dt_in, r * ld_in + F + f), kind, limit, alpha));
  }
}

// bf16 in and out, F and ld_in multiples of 8: 16-byte accesses
__global__ void glu_bf16x8_kernel(const bf16* __restrict__ in, long long ld_in, bf16* __restrict__ out, long long rows, int F, int kind, float limit,
                                  float alpha, const int* __restrict__ n_tiles, int tile_rows) {
  if (n_tiles != nullptr) rows = min(rows, (long long)n_tiles[0] * tile_rows);
  const int F8 = F >> 3;
  const long long n = rows * F8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / F8;
    const int f = (int)(i - r * F8) << 3;
    float a[8], b[8];
    unpack8(*reinterpret_cast<const uint4*>(in + r * ld_in + f), a);
    if (kind != 3) unpack8(*reinterpret_cast<const uint4*>(in + r * ld_in + F + f), b);
    uint4 o;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e)
      po[e] = __floats2bfloat162_rn(glu_value(a[2 * e], b[2 * e], kind, limit, alpha), glu_value(a[2 * e + 1], b[2 * e + 1], kind, limit, alpha));
    *reinterpret_cast<uint4*>(out + r * F + f) = o;
  }
}

// ------------------------------------------------------------------------------------------------ router
// A warp per token.  s = softmax(z) (score_kind 0) or sigmoid(z) (1) over the E router outputs; choice c = s + correction; with
// groups > 1 only the experts of the `keep` groups with the largest group score (their largest choice, or the sum of their two largest)
// stay in play; the `top` largest choices are taken (ties: lower index); weights are the chosen s, divided by their sum (+ 1e-20) if
// renorm, times out_scale.
__global__ void __launch_bounds__(128) route_topk_kernel(const float* __restrict__ z, long long ldz, int T, int E,
                                                         const float* __restrict__ correction, int score_kind, int groups, int keep,
                                                         int top, int renorm, float out_scale, int* __restrict__ ids,
                                                         float* __restrict__ weights, int group_kind) {
  extern __shared__ float rsm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const long long t = (long long)blockIdx.x * nw + warp;
  if (t >= T) return;
  float* s = rsm + (size_t)warp * (2 * E + groups);
  float* c = s + E;
  float* gsc = c + E;
  const float* zr = z + t * ldz;
  if (score_kind == 0) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zr[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float v = expf(zr[e] - mx);
      s[e] = v;
      sum += v;
    }
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) s[e] = s[e] / sum;
  } else {
    for (int e = lane; e < E; e += 32) s[e] = 1.f / (1.f + expf(-zr[e]));
  }
  for (int e = lane; e < E; e += 32) c[e] = s[e] + (correction ? correction[e] : 0.f);
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int gs = E / groups;
    for (int gi = lane; gi < groups; gi += 32) {      // group_kind 0: largest choice of the group; 1: sum of its two largest
      float mx = -INFINITY, m2 = -INFINITY;
      for (int e = gi * gs; e < (gi + 1) * gs; ++e) {
        const float v = c[e];
        if (v > mx) { m2 = mx; mx = v; } else if (v > m2) m2 = v;
      }
      gsc[gi] = (group_kind == 1 && m2 != -INFINITY) ? mx + m2 : mx;
    }
    __syncwarp();
    // the keep best groups get +inf as a mark, one after the other
    for (int it = 0; it < keep; ++it) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int gi = lane; gi < groups; gi += 32) {
        const float v = gsc[gi];
        if (v != INFINITY && (v > bv || (v == bv && gi < bi))) { bv = v; bi = gi; }
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (lane == 0 && bi < groups) gsc[bi] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gsc[e / gs] != INFINITY) c[e] = -INFINITY;
    __syncwarp();
  }
  float wsum = 0.f;
  for (int it = 0; it < top; ++it) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = c[e];
      if (v > bv || (v == bv && e < bi && v != -INFINITY)) { bv = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const bool found = bi < E;
    if (lane == 0) {
      ids[t * top + it] = found ? bi : -1;
      weights[t * top + it] = found ? s[bi] : 0.f;
      if (found) c[bi] = -INFINITY;
    }
    if (found) wsum += s[bi];
    __syncwarp();
  }
  if (lane == 0) {
    const float f = (renorm ? 1.f / (wsum + 1e-20f) : 1.f) * out_scale;
    if (f != 1.f)
      for (int it = 0; it < top; ++it) weights[t * top + it] *= f;
  }
}

// ------------------------------------------------------------------------------------------------ routed experts
constexpr int kMoeBM = 64;
// counts[e] = number of (token, k) slots routed to expert e < E (identity / absent experts have id >= E or < 0)
__global__ void moe_count_kernel(const int* __restrict__ ids, long long slots, int E, int* __restrict__ counts) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < slots; i += (long long)gridDim.x * blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
}
// One block: offs[e] = first row of expert e's run, runs padded to whole tiles of tile_rows; tile_expert[tile]; n_tiles[0]; cursor[e] = 0.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int tile_rows, int* __restrict__ offs, int* __restrict__ cursor,
                                int* __restrict__ tile_expert, int* __restrict__ n_tiles) {
  if (threadIdx.x == 0) {
    int tiles = 0;
    for (int e = 0; e < E; ++e) {
      offs[e] = tiles * tile_rows;
      tiles += (counts[e] + tile_rows - 1) / tile_rows;
    }
    offs[E] = tiles * tile_rows;
    n_tiles[0] = tiles;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    cursor[e] = 0;
    for (int tl = offs[e] / tile_rows; tl < offs[e + 1] / tile_rows; ++tl) tile_expert[tl] = e;
  }
}
// slot_row[p] = slot (t * top + k) that sits at row p of the binned order (-1: padding); pos_of_slot[slot] = p (-1: not routed here)
__global__ void moe_scatter_kernel(const int* __restrict__ ids, long long slots, int E, const int* __restrict__ offs,
                                   int* __restrict__ cursor, int* __restrict__ slot_row, int* __restrict__ pos_of_slot) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < slots; i += (long long)gridDim.x * blockDim.x) {
    const int e = ids[i];
    int p = -1;
    if (e >= 0 && e < E) {
      p = offs[e] + atomicAdd(&cursor[e], 1);
      slot_row[p] = (int)i;
    }
    pos_of_slot[i] = p;
  }
}

// C[p, :] = A[src(p), :] * B[expert of p's tile]^T for the rows p of tile blockIdx.y.  src(p) = p, or row_map[p] / div through a map
// (negative: a padding row, computed as zeros).  64 x 64 tile, fp32 FMA, every output sums its K products in one fixed order.
template <typename TA, typename TB, typename TC>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const TA* __restrict__ A, long long lda, const int* __restrict__ row_map, int div,
                                                       const TB* __restrict__ B, long long ldb, long long sB, TC* __restrict__ C,
                                                       long long ldc, int N, int K, const int* __restrict__ tile_expert,
                                                       const int* __restrict__ n_tiles, int tile_rows) {
  constexpr int BM = kMoeBM, BN = 64, BK = 16;           // tile_rows is a multiple of BM: a block never straddles two experts
  if ((long long)blockIdx.y * BM >= (long long)n_tiles[0] * tile_rows) return;
  __shared__ float As[BK][BM + 4], Bs[BK][BN + 4];
  __shared__ long long src[BM];
  B += (long long)tile_expert[(long long)blockIdx.y * BM / tile_rows] * sB;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const long long m0 = (long long)blockIdx.y * BM;
  const int n0 = blockIdx.x * BN;
  if (tid < BM) {
    long long r = m0 + tid;
    if (row_map != nullptr) {
      const int sr = row_map[r];
      r = sr < 0 ? -1 : sr / div;
    }
    src[tid] = r;
  }
  __syncthreads();
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int i = tid + it * 256, r = i >> 4, c = i & 15;
      const int n = n0 + r, k = k0 + c;
      As[c][r] = (src[r] >= 0 && k < K) ? ldf(A, src[r] * lda + k) : 0.f;
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
    const long long m = m0 + ty * 4 + i;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) stf(C, m * ldc + n, acc[i][j]);
    }
  }
}

// Steps of few tokens: no binning; a warp per (slot, output column) streams that column's weight row of the slot's expert.
// C[slot, n] = A[slot / div, :] . B[ids[slot]][n, :]; slots of identity / absent experts are skipped.
template <typename TA, typename TB, typename TC>
__global__ void __launch_bounds__(256) moe_gemv_kernel(const TA* __restrict__ A, long long lda, int div, const int* __restrict__ ids, int E,
                                                       const TB* __restrict__ B, long long ldb, long long sB, TC* __restrict__ C,
                                                       long long ldc, int N, int K) {
  const int slot = blockIdx.y;
  const int e = ids[slot];
  if (e < 0 || e >= E) return;
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  const TA* a = A + (long long)(slot / div) * lda;
  const TB* b = B + (long long)e * sB + (long long)n * ldb;
  float acc = 0.f;
  if (sizeof(TB) == 2 && (K & 7) == 0 && (ldb & 7) == 0 && (sB & 7) == 0 && !((uintptr_t)B & 15)) {
    for (int k = lane * 8; k < K; k += 256) {
      float wv[8];
      unpack8(*reinterpret_cast<const uint4*>(b + k), wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = fmaf(ldf(a, k + i), wv[i], acc);
    }
  } else {
    for (int k = lane; k < K; k += 32) acc = fmaf(ldf(a, k), ldf(b, k), acc);
  }
  acc = warp_sum(acc);
  if (lane == 0) stf(C, (long long)slot * ldc + n, acc);
}

// out[t, :] = sum_k w[t, k] * (expert row of slot (t, k) | h[t, :] for an identity expert) + sigmoid(shared_gate[t]) shared[t, :] (gate
// null: 1), k in selection order
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pos_of_slot, const int* __restrict__ ids,
                                   const float* __restrict__ weights, int top, int E, int ident, const void* __restrict__ h, int dt_h,
                                   const float* __restrict__ shared, float* __restrict__ out, int W,
                                   const float* __restrict__ shared_gate, long long ldsg) {
  const long long t = blockIdx.x;
  const float sgate = shared_gate != nullptr ? 1.f / (1.f + expf(-shared_gate[t * ldsg])) : 1.f;   // the shared expert's weight for this token
  if ((W & 3) == 0 && dt_h == 1) {           // four columns per thread, 16-byte loads of the expert rows; same order of the sum over k
    for (int d = threadIdx.x * 4; d < W; d += blockDim.x * 4) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = 0; k < top; ++k) {
        const long long slot = t * top + k;
        const int e = ids[slot];
        const float w = weights[slot];
        if (e >= 0 && e < E) {
          const long long p = pos_of_slot ? pos_of_slot[slot] : slot;
          const float4 r = *reinterpret_cast<const float4*>(y + p * W + d);
          v.x = fmaf(w, r.x, v.x); v.y = fmaf(w, r.y, v.y); v.z = fmaf(w, r.z, v.z); v.w = fmaf(w, r.w, v.w);
        } else if (e >= E && e < E + ident) {
          const bf16* hp = (const bf16*)h + t * W + d;
          v.x = fmaf(w, __bfloat162float(hp[0]), v.x); v.y = fmaf(w, __bfloat162float(hp[1]), v.y);
          v.z = fmaf(w, __bfloat162float(hp[2]), v.z); v.w = fmaf(w, __bfloat162float(hp[3]), v.w);
        }
      }
      if (shared != nullptr) {
        const float4 r = *reinterpret_cast<const float4*>(shared + t * W + d);
        v.x = fmaf(sgate, r.x, v.x); v.y = fmaf(sgate, r.y, v.y); v.z = fmaf(sgate, r.z, v.z); v.w = fmaf(sgate, r.w, v.w);
      }
      *reinterpret_cast<float4*>(out + t * W + d) = v;
    }
    return;
  }
  for (int d = threadIdx.x; d < W; d += blockDim.x) {
    float v = 0.f;
    for (int k = 0; k < top; ++k) {
      const long long slot = t * top + k;
      const int e = ids[slot];
      const float w = weights[slot];
      if (e >= 0 && e < E) {
        const long long p = pos_of_slot ? pos_of_slot[slot] : slot;
        v = fmaf(w, y[p * W + d], v);
      } else if (e >= E && e < E + ident) {
        v = fmaf(w, ld_dt(h, dt_h, t * W + d), v);
      }
    }
    if (shared != nullptr) v = fmaf(sgate, shared[t * W + d], v);
    out[t * W + d] = v;
  }
}

}  // namespace kb2seq

using namespace kb2seq;

extern "C" {

KB2SEQ_API int kb2_seq_head_kv_prep(float* proj, long long ldp, int T, int H, int G, int M, int d, int dv, const float* bias,
                                    const float* qw, const float* kw, float eps, const double* freq, int rot_dims, const int* positions,
                                    const int* seq_of, const int* pages, int max_pages, int page_size, void* kc, void* vc, int dt_cache,
                                    int norm_whole, int rot_half, const double* vfreq, void* stream) {
  if (vfreq && (dv & 1)) return failf(KB2SEQ_ERR_VALUE, "head_kv_prep: rotated values need an even value size");
  if (!proj || !positions || !seq_of || !pages || T <= 0 || H <= 0 || G < 0 || M <= 0 || d <= 0 || dv < 0 || rot_dims < 0 ||
      rot_dims > d || (rot_dims & 1) || (rot_dims && !freq) || page_size <= 0 || max_pages <= 0 || bad_dt(dt_cache) ||
      (G > 0 && (!kc || !vc)))
    return failf(KB2SEQ_ERR_VALUE, "head_kv_prep: bad argument");
  head_kv_prep_kernel<<<T, 256, (size_t)rot_dims * 4, (cudaStream_t)stream>>>(proj, ldp, H, G, M, d, dv, bias, qw, kw, eps, freq, rot_dims, positions, seq_of,
                                                           pages, max_pages, page_size, kc, vc, dt_cache, norm_whole, rot_half, vfreq);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_kv_pool(const void* kc, const void* vc, void* kp, void* vp, int dt_cache, int kw, int vw, int pool, int T,
                               const int* positions, const int* seq_of, const int* pages, int max_pages, int page_size, void* stream) {
  if (!kc || !vc || !kp || !vp || bad_dt(dt_cache) || kw <= 0 || vw <= 0 || pool <= 0 || T <= 0 || !positions || !seq_of || !pages ||
      max_pages <= 0 || page_size <= 0)
    return failf(KB2SEQ_ERR_VALUE, "kv_pool: bad argument");
  kv_pool_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(kc, vc, kp, vp, dt_cache, kw, vw, pool, (page_size + pool - 1) / pool, positions, seq_of,
                                                      pages, max_pages, page_size);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_paged_attn(const float* proj, long long ldp, int T, int H, int G, int M, int d, int dv, const void* kc,
                                  const void* vc, int dt_cache, const int* positions, const int* seq_of, const int* pages, int max_pages,
                                  int page_size, float scale, int chunk, int window, float* out, int nsplit, float* part_acc,
                                  float* part_ml, const int* cu, int skip_from, float softcap, const float* sinks, int pool, const void* kp,
                                  const void* vp, int pool_only, void* stream) {
  if (pool < 0 || (pool > 0 && (!kp || !vp || chunk > 0))) return failf(KB2SEQ_ERR_VALUE, "paged_attn: pooled blocks need their pools and no chunks");
  if (pool_only && (pool <= 0 || nsplit != 1 || !part_acc || !part_ml || !cu))
    return failf(KB2SEQ_ERR_VALUE, "paged_attn: the pass over the pooled blocks alone needs pool > 0, one key piece, the piece buffers and cu");
  if (!proj || !kc || !vc || !positions || !seq_of || !pages || !out || T <= 0 || H <= 0 || G <= 0 || H % G || M <= 0 || d <= 0 ||
      dv <= 0 || window <= 0 || chunk < 0 || page_size <= 0 || bad_dt(dt_cache) || !(softcap >= 0.f))
    return failf(KB2SEQ_ERR_VALUE, "paged_attn: bad argument");
  if (nsplit < 1 || nsplit > 1024 || (nsplit > 1 && (!part_acc || !part_ml))) return failf(KB2SEQ_ERR_VALUE, "paged_attn: bad key split");
  if (dv > kPAThreads * kPAAcc) return failf(KB2SEQ_ERR_VALUE, "paged_attn: value size %d > %d", dv, kPAThreads * kPAAcc);
  const int R = (H / G) * M;
  int RB = R;
  auto smem_of = [&](int rb) {
    return (size_t)(2 * kPAKT + rb * d + kPAKT * ((M * d) | 1) + kPAKT * dv + rb * kPAKT + 3 * rb) * 4;
  };
  while (RB > 1 && (RB * dv > kPAThreads * kPAAcc || smem_of(RB) > 200 * 1024)) RB = (RB + 1) / 2;
  const size_t smem = smem_of(RB);
  if (smem > 200 * 1024) return failf(KB2SEQ_ERR_VALUE, "paged_attn: head sizes %d / %d too large", M * d, dv);
  if (smem > 48 * 1024) SEQ_CUDA(cudaFuncSetAttribute(paged_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int nrb = (R + RB - 1) / RB;
  if ((long long)G * nrb > 65535) return failf(KB2SEQ_ERR_VALUE, "paged_attn: too many heads");
  paged_attn_kernel<<<dim3(T, G * nrb, nsplit), kPAThreads, smem, (cudaStream_t)stream>>>(
      proj, ldp, H, G, M, d, dv, RB, kc, vc, dt_cache, positions, seq_of, pages, max_pages, page_size, scale, chunk, window, out, nsplit,
      part_acc, part_ml, cu, skip_from, softcap, sinks, pool, pool > 0 ? (page_size + pool - 1) / pool : 0, kp, vp, pool_only);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_pool_merge(float* a, const float* lse, const float* part_acc, const float* part_ml, int T, int H, int dv,
                                  const int* seq_of, const int* cu, int min_portion, void* stream) {
  if (!a || !lse || !part_acc || !part_ml || !seq_of || !cu || T <= 0 || H <= 0 || dv <= 0) return failf(KB2SEQ_ERR_VALUE, "pool_merge: bad argument");
  const long long rows = (long long)T * H;
  pool_merge_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, (cudaStream_t)stream>>>(a, lse, part_acc, part_ml, rows, H, dv, seq_of, cu, min_portion);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_attn_finish(const float* a, const float* part_acc, const float* part_ml, int nsplit, int T, int H, int M, int dv,
                                   const float* coef, int unit_norm, float eps, float post_scale, const float* gate, long long ldg,
                                   void* out, int dt_out, const int* seq_of, const int* cu, int skip_from, int gate_wide,
                                   const int* positions, const double* vfreq, int rot_half, void* stream) {
  if (vfreq && (!positions || (dv & 1))) return failf(KB2SEQ_ERR_VALUE, "attn_finish: turning back needs positions and an even value size");
  if (!out || T <= 0 || H <= 0 || M <= 0 || dv <= 0 || bad_dt(dt_out) || nsplit < 1 || (nsplit == 1 && !a) ||
      (nsplit > 1 && (!part_acc || !part_ml)) || (cu && !seq_of))
    return failf(KB2SEQ_ERR_VALUE, "attn_finish: bad argument");
  if (dv > 32 * kFinAcc) return failf(KB2SEQ_ERR_VALUE, "attn_finish: value size %d > %d", dv, 32 * kFinAcc);
  const long long nwarps = (long long)T * H;
  attn_finish_kernel<<<(unsigned)((nwarps + 7) / 8), 256, 0, (cudaStream_t)stream>>>(a, part_acc, part_ml, nsplit, T, H, M, dv, coef, unit_norm,
                                                                                      eps, post_scale, gate, ldg, out, dt_out, seq_of, cu,
                                                                                      skip_from, gate_wide, positions, vfreq, rot_half);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_glu(const void* in, int dt_in, long long ld_in, void* out, int dt_out, long long rows, int F, int kind, float limit,
                           float alpha, const int* n_tiles, int tile_rows, void* stream) {
  if (!in || !out || rows <= 0 || F <= 0 || ld_in < (kind == 3 ? F : 2 * F) || kind < 0 || kind > 3 || bad_dt(dt_in) || bad_dt(dt_out))
    return failf(KB2SEQ_ERR_VALUE, "glu: bad argument");
  if (dt_in == 1 && dt_out == 1 && F % 8 == 0 && ld_in % 8 == 0 && !((uintptr_t)in & 15) && !((uintptr_t)out & 15)) {
    const long long n8 = rows * (F / 8);
    const unsigned blocks8 = (unsigned)((n8 + 255) / 256 > 148 * 16 ? 148 * 16 : (n8 + 255) / 256);
    glu_bf16x8_kernel<<<blocks8, 256, 0, (cudaStream_t)stream>>>((const bf16*)in, ld_in, (bf16*)out, rows, F, kind, limit, alpha, n_tiles, tile_rows);
    SEQ_LAUNCHED();
    return KB2SEQ_OK;
  }
  const long long n = rows * F;
  const unsigned blocks = (unsigned)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
  glu_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(in, dt_in, ld_in, out, dt_out, rows, F, kind, limit, alpha, n_tiles, tile_rows);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_route(const float* z, long long ldz, int T, int E, const float* correction, int score_kind, int groups, int keep,
                             int top, int renorm, float out_scale, int* ids, float* weights, int group_kind, void* stream) {
  if (!z || !ids || !weights || T <= 0 || E <= 0 || top <= 0 || top > E || score_kind < 0 || score_kind > 1 || groups < 1 || group_kind < 0 || group_kind > 1 ||
      E % groups || keep < 1 || keep > groups)
    return failf(KB2SEQ_ERR_VALUE, "route: bad argument (E=%d top=%d groups=%d keep=%d)", E, top, groups, keep);
  if ((long long)keep * (E / groups) < top) return failf(KB2SEQ_ERR_VALUE, "route: the kept groups hold fewer than top experts");
  const size_t smem = (size_t)4 * (2 * E + groups) * 4;
  if (smem > 200 * 1024) return failf(KB2SEQ_ERR_VALUE, "route: %d router outputs too many", E);
  if (smem > 48 * 1024) SEQ_CUDA(cudaFuncSetAttribute(route_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  route_topk_kernel<<<(T + 3) / 4, 128, smem, (cudaStream_t)stream>>>(z, ldz, T, E, correction, score_kind, groups, keep, top, renorm,
                                                                      out_scale, ids, weights, group_kind);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_moe_tile_rows(void) { return kMoeBM; }

KB2SEQ_API int kb2_seq_moe_bin(const int* ids, long long slots, int E, int tile_rows, int* counts, int* offs, int* cursor, int* tile_expert,
                               int* n_tiles, int* slot_row, long long max_rows, int* pos_of_slot, void* stream) {
  if (!ids || !counts || !offs || !cursor || !tile_expert || !n_tiles || !slot_row || !pos_of_slot || slots <= 0 || E <= 0 ||
      tile_rows <= 0 || tile_rows % kMoeBM || max_rows < slots + (long long)E * (tile_rows - 1))
    return failf(KB2SEQ_ERR_VALUE, "moe_bin: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  SEQ_CUDA(cudaMemsetAsync(counts, 0, (size_t)E * 4, s));
  SEQ_CUDA(cudaMemsetAsync(slot_row, 0xFF, (size_t)max_rows * 4, s));
  const unsigned blocks = (unsigned)((slots + 255) / 256 > 1024 ? 1024 : (slots + 255) / 256);
  moe_count_kernel<<<blocks, 256, 0, s>>>(ids, slots, E, counts);
  SEQ_LAUNCHED();
  moe_plan_kernel<<<1, 256, 0, s>>>(counts, E, tile_rows, offs, cursor, tile_expert, n_tiles);
  SEQ_LAUNCHED();
  moe_scatter_kernel<<<blocks, 256, 0, s>>>(ids, slots, E, offs, cursor, slot_row, pos_of_slot);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

KB2SEQ_API int kb2_seq_moe_gemm(const void* A, int dtA, long long lda, const int* row_map, int div, const void* B, int dtB, long long ldb,
                                long long sB, void* C, int dtC, long long ldc, int N, int K, const int* tile_expert, const int* n_tiles,
                                int max_tiles, int tile_rows, void* stream) {
  if (!A || !B || !C || !tile_expert || !n_tiles || N <= 0 || K <= 0 || max_tiles <= 0 || tile_rows <= 0 || tile_rows % kMoeBM ||
      (long long)max_tiles * (tile_rows / kMoeBM) > 65535 || div <= 0 || bad_dt(dtA) || bad_dt(dtB) || bad_dt(dtC))
    return failf(KB2SEQ_ERR_VALUE, "moe_gemm: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid((N + 63) / 64, max_tiles * (tile_rows / kMoeBM));
#define G(TA, TB, TC)                                                                                                          \
  moe_gemm_kernel<TA, TB, TC><<<grid, 256, 0, s>>>((const TA*)A, lda, row_map, div, (const TB*)B, ldb, sB, (TC*)C, ldc, N, K, tile_expert, \
                                                   n_tiles, tile_rows)
  switch (dtA * 4 + dtB * 2 + dtC) {
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

KB2SEQ_API int kb2_seq_moe_gemv(const void* A, int dtA, long long lda, int div, const int* ids, int E, const void* B, int dtB, long long ldb,
                                long long sB, void* C, int dtC, long long ldc, int slots, int N, int K, void* stream) {
  if (!A || !B || !C || !ids || N <= 0 || K <= 0 || slots <= 0 || slots > 65535 || div <= 0 || E <= 0 || bad_dt(dtA) || bad_dt(dtB) ||
      bad_dt(dtC))
    return failf(KB2SEQ_ERR_VALUE, "moe_gemv: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid((N + 7) / 8, slots);
#define G(TA, TB, TC) moe_gemv_kernel<TA, TB, TC><<<grid, 256, 0, s>>>((const TA*)A, lda, div, ids, E, (const TB*)B, ldb, sB, (TC*)C, ldc, N, K)
  switch (dtA * 4 + dtB * 2 + dtC) {
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

KB2SEQ_API int kb2_seq_moe_combine(const float* y, const int* pos_of_slot, const int* ids, const float* weights, int T, int top, int E,
                                   int ident, const void* h, int dt_h, const float* shared, float* out, int W, const float* shared_gate,
                                   long long ldsg, void* stream) {
  if (!ids || !weights || !out || T <= 0 || top <= 0 || E < 0 || ident < 0 || W <= 0 || (E > 0 && !y) || (ident > 0 && (!h || bad_dt(dt_h))))
    return failf(KB2SEQ_ERR_VALUE, "moe_combine: bad argument");
  moe_combine_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(y, pos_of_slot, ids, weights, top, E, ident, h, dt_h, shared, out, W, shared_gate, ldsg);
  SEQ_LAUNCHED();
  return KB2SEQ_OK;
}

}  // extern "C"
