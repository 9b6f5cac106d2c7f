/*
 * krasis_b200 — C ABI of the ragged-batch sequence operators (libkrasis_b200_seq.so).
 *
 * One step of a serving engine carries portions of several prompts next to single decoded tokens.  These entry points take
 * that step as a flat token axis [T] plus small int32 tables on the device:
 *   tokens[T], positions[T] (position of each token in its own sequence), seq_of[T] (index of its sequence in the step),
 *   cu[S + 1] (first row of each sequence's portion), slots[S] (recurrent-state slot of each sequence),
 *   pages[S][max_pages] (page list of each sequence in a paged cache with `page_size` tokens per page).
 * Conventions follow krasis_b200.h: device pointers owned by the caller, stream-ordered on `stream` (a cudaStream_t), no hidden
 * synchronisation, 0 = ok, text of the last error via kb2_seq_last_error().  `dt` arguments: 0 = float32, 1 = bfloat16.
 * There is no CPU fallback.
 */
#ifndef KRASIS_B200_SEQ_H
#define KRASIS_B200_SEQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define KB2SEQ_API __attribute__((visibility("default")))
#else
#define KB2SEQ_API
#endif

#define KB2SEQ_OK 0
#define KB2SEQ_ERR_VALUE 2
#define KB2SEQ_ERR_CUDA 3

KB2SEQ_API const char* kb2_seq_last_error(void);
KB2SEQ_API long long kb2_seq_total_launches(void);

/* x[t, :] = table[tokens[t], :] * scale, fp32 out */
KB2SEQ_API int kb2_seq_embed(const void* table, int dt, const int* tokens, float* x, int T, int W, float scale, void* stream);

/* C[b] = A[b] (M x K, row stride lda) * B[b]^T (N x K, row stride ldb), fp32 accumulation; b < batch with element strides sA, sB, sC */
KB2SEQ_API int kb2_seq_gemm(const void* A, int dtA, long long lda, const void* B, int dtB, long long ldb, void* C, int dtC,
                            long long ldc, int M, int N, int K, int batch, long long sA, long long sB, long long sC, void* stream);

/* x += norm(y) [+ x0]; h = layer_norm(x; wb, bb).  y_mode 1: layer norm (wa, ba), 2: RMS norm (wa).  y, x0 and h may be null. */
KB2SEQ_API int kb2_seq_residual_norm(float* x, const float* y, int y_mode, const float* wa, const float* ba, const float* x0,
                                     const float* wb, const float* bb, void* h, int dt_h, int T, int W, float eps, void* stream);

/* out[t, f] = gelu_tanh(in[t, f]) * in[t, F + f] */
KB2SEQ_API int kb2_seq_act_mul(const void* in, int dt_in, void* out, int dt_out, int T, int F, void* stream);

/* out[t, d] = gelu_tanh(g[t, d]) * table[tokens[t], col0 + d] */
KB2SEQ_API int kb2_seq_side_gate(const float* g, const void* table, int dt_table, long long table_ld, const int* tokens, int col0,
                                 int dim, int T, void* out, int dt_out, void* stream);

/* proj [T, ldp] = [q: H x (dn + dr) | latent: r | shared rotated key: dr].  Writes the RMS-normed latent and the rotated key to the
 * cache rows of the tokens' positions and rotates the queries' rotated parts in place.  freq[rot_dims / 2], amplitude amp.
 * lat (may be null) [T, ldl]: the [latent | shared rotated key] columns when they do not follow the queries in proj (queries that
 * come from a projection of their own). */
KB2SEQ_API int kb2_seq_latent_prep(float* proj, long long ldp, int T, int H, int dn, int dr, int r, const float* cw, float eps,
                                   const double* freq, int rot_dims, float amp, const int* positions, const int* seq_of,
                                   const int* pages, int max_pages, int page_size, void* ckv, void* kr, int dt_cache, const float* lat,
                                   long long ldl, void* stream);

/* out[t, h, :r] = sum_j softmax_j(...) latent_j over the keys with 0 <= pos - j < window; the denominator also holds exp(sinks[h])
 * (sinks may be null: ordinary softmax).
 * With cu != NULL the tokens of sequences whose portion has skip_from tokens or more are left out (another kernel serves them).
 * nsplit > 1 cuts every token's key range into nsplit pieces that run as separate blocks (steps of few tokens: decoding) and are merged
 * by a second kernel; part_acc [T][nsplit][H][r] and part_ml [T][nsplit][H][2] (fp32) hold the pieces. */
KB2SEQ_API int kb2_seq_latent_window_attn(const float* q_abs, const float* proj, long long ldp, int T, int H, int dn, int dr, int r,
                                          const void* ckv, const void* kr, int dt_cache, const int* positions, const int* seq_of,
                                          const int* pages, int max_pages, int page_size, const float* sinks, float scale, int window,
                                          float* out, const int* cu, int skip_from, int nsplit, float* part_acc, float* part_ml,
                                          void* stream);

/* out[t, c] = silu(causal conv over time of proj[:, c], K taps) for c < C; tail [slots][C][K - 1] is read, then advanced */
KB2SEQ_API int kb2_seq_conv_silu(const float* proj, long long ldp, int T, int S, int C, int K, const float* taps, float* tail,
                                 const int* seq_of, const int* cu, const int* slots, float* out, void* stream);

/* The same with a bias added to proj before the convolution (null: none; the carried tail holds biased inputs) and act 1: silu, 0: none.
 * act + 2: the bias joins the convolution's result instead of its inputs (ahead of the activation; the tail holds plain inputs). */
KB2SEQ_API int kb2_seq_conv(const float* proj, long long ldp, int T, int S, int C, int K, const float* taps, const float* bias, int act,
                            float* tail, const int* seq_of, const int* cu, const int* slots, float* out, void* stream);

/* x += y_mult * y (y may be null); h = x / sqrt(mean(x^2) + eps) * (w_shift + w) (h may be null; h == x with y null: in place, fp32) */
KB2SEQ_API int kb2_seq_residual_scale_rms(float* x, const float* y, float y_mult, const float* w, float w_shift, void* h, int dt_h, int T,
                                          int W, float eps, void* stream);

/* gated delta rule over each sequence's portion; state [slots][H][dk][dv] fp32 is read and written back.
 * scratch (fp32, 2 T Hk dk + 2 T H + T H dv + 4 elements, 16-byte aligned) selects the register-state kernels when dk is 32, 64 or
 * 128 and dv a multiple of 32; with scratch == NULL, or other sizes, one block per (sequence, head) keeps the state in shared memory
 * (a state too large for that is cut into slices of value columns, one block each; this needs scratch). */
KB2SEQ_API int kb2_seq_delta_rule(const float* conv, int C, const float* proj, long long ldp, int g_off, int a_off, int b_off, int T,
                                  int S, int H, int Hk, int dk, int dv, const float* A_log, const float* dt_bias, const float* norm_w,
                                  float eps, float* state, const int* cu, const int* slots, float* scratch, void* out, int dt_out,
                                  void* stream);

/* The delta rule with one decay per (token, head, key channel): S <- diag(g) S with g = exp(-exp(A_log[h]) softplus(decay_in[t, h dk + i]
 * + dt_bias[h dk + i])), then u = beta (v - S^T k), S <- S + k u^T, o = S^T q.  beta_in [T, ldb] holds H write-strength logits per row,
 * decay_in [T, lda] H dk decay inputs, gate_in [T, ldg] H dv output-gate inputs (gate_act 0: silu, 1: sigmoid).  scratch as above with
 * T H dk more elements. */
KB2SEQ_API int kb2_seq_delta_rule_ch(const float* conv, int C, const float* beta_in, long long ldb, const float* decay_in, long long lda,
                                     const float* gate_in, long long ldg, int gate_act, int T, int S, int H, int Hk, int dk, int dv,
                                     const float* A_log, const float* dt_bias, const float* norm_w, float eps, float* state, const int* cu,
                                     const int* slots, float* scratch, void* out, int dt_out, void* stream);

/* ---- second part (csrc/seq_mix.cu): per-head key/value caches, multi-map attention, gated linear units, routed experts ---- */

/* x += (y + y2) in that order (y2 may be null: x += y); h = layer_norm(x; wb, bb), bb may be null (no bias), h may be null */
KB2SEQ_API int kb2_seq_residual_add_norm(float* x, const float* y, const float* y2, const float* wb, const float* bb, void* h, int dt_h,
                                         int T, int W, float eps, void* stream);

/* proj [T, ldp] fp32 = [q: H x M x d | k: G x M x d | v: G x dv | ...]: H query heads with M maps each, G key/value heads (0: the layer
 * reads another layer's cache).  bias (same column order, may be null) is added; every q / k vector of d is RMS-normed with the weight
 * qw / kw [d] (null: no norm) and its first rot_dims dimensions are rotated as interleaved pairs by position * freq[i].  q is written
 * back in place; k [G M d] and v [G dv] go to the cache rows of the tokens' positions.  norm_whole 1: one root mean square over the whole
 * of q (and of k) with weights qw [H M d] / kw [G M d].  rot_half 1: dimension i turns with i + rot_dims / 2 instead of 2i with 2i + 1.
 * vfreq [dv / 2] (may be null): the value vectors are cached rotated too, pair m of all dv dimensions (same pair layout) by
 * position * vfreq[m]; kb2_seq_attn_finish turns the attention output back by the query's position. */
KB2SEQ_API int kb2_seq_head_kv_prep(float* proj, long long ldp, int T, int H, int G, int M, int d, int dv, const float* bias,
                                    const float* qw, const float* kw, float eps, const double* freq, int rot_dims, const int* positions,
                                    const int* seq_of, const int* pages, int max_pages, int page_size, void* kc, void* vc, int dt_cache,
                                    int norm_whole, int rot_half, const double* vfreq, void* stream);

/* Pooled blocks: every `pool` consecutive positions of a sequence, b pool .. b pool + pool - 1, are summarised by the mean of their
 * cached key rows (width kw) and the mean of their cached value rows (width vw), taken in fp32 from the cache as it holds them.  The
 * pooled pools kp / vp have ceil(page_size / pool) rows per page and share the page numbering of kc / vc; block b lies in the page of
 * its last position.  Call after kb2_seq_head_kv_prep of the same step: the tokens of the step that complete a block write its summary. */
KB2SEQ_API int kb2_seq_kv_pool(const void* kc, const void* vc, void* kp, void* vp, int dt_cache, int kw, int vw, int pool, int T,
                               const int* positions, const int* seq_of, const int* pages, int max_pages, int page_size, void* stream);

/* out [T, H, M, dv] fp32: softmax attention of each (head, map) query over the keys j <= pos of its sequence that lie in the same
 * chunk (chunk > 0: floor(j / chunk) == floor(pos / chunk)) and within 0 <= pos - j < window.  Head h reads key/value head h / (H / G);
 * map m reads the keys of map m; all maps read the same values.  cu / skip_from and nsplit / part_acc [T H M][nsplit][dv] /
 * part_ml [T H M][nsplit][2] as in kb2_seq_latent_window_attn, except that the pieces are merged by kb2_seq_attn_finish.
 * softcap > 0: a score s (after the scale) becomes softcap tanh(s / softcap).
 * sinks [H] (may be null): the softmax denominator of head h also holds exp(sinks[h]) (unscaled, no value).
 * pool > 0 (needs chunk == 0): beside the window's keys a token sees one key and value per block of `pool` positions that lies wholly
 * before its window (b pool + pool - 1 <= pos - window), read from the pooled pools kp / vp (see kb2_seq_kv_pool), in the same softmax. */
KB2SEQ_API int kb2_seq_paged_attn(const float* proj, long long ldp, int T, int H, int G, int M, int d, int dv, const void* kc,
                                  const void* vc, int dt_cache, const int* positions, const int* seq_of, const int* pages, int max_pages,
                                  int page_size, float scale, int chunk, int window, float* out, int nsplit, float* part_acc,
                                  float* part_ml, const int* cu, int skip_from, float softcap, const float* sinks, int pool, const void* kp,
                                  const void* vp, int pool_only, void* stream);

/* pool_only 1 (above; needs cu, nsplit 1 and the piece buffers): the pass that follows a tensor-core attention over the window of long
 * portions — only the tokens of sequences whose portion has skip_from tokens or more, only their pooled blocks, no sink; the result stays
 * an unnormalised piece in part_acc [T H][dv] / part_ml [T H][2].  kb2_seq_pool_merge joins it to the window's result a [T, H, dv]
 * (normalised, with lse [T, H] the logarithm of its softmax denominator), in place, for the same sequences (M == 1). */
KB2SEQ_API int kb2_seq_pool_merge(float* a, const float* lse, const float* part_acc, const float* part_ml, int T, int H, int dv,
                                  const int* seq_of, const int* cu, int min_portion, void* stream);

/* out[t, h, :] = f * sum_m coef[m] a[t, h, m, :] (coef null: ones), f = post_scale / rms(sum) if unit_norm, times sigmoid(gate[t * ldg + h])
 * if gate is given (gate_wide 1: one gate per output element, sigmoid(gate[t * ldg + h dv + c])).  nsplit > 1: a is merged from
 * part_acc / part_ml first.  vfreq [dv / 2] (may be null; needs positions): the head's output is turned back, pair m by
 * -positions[t] * vfreq[m] in the pair layout rot_half selects, before norm factor and gate are applied. */
KB2SEQ_API int kb2_seq_attn_finish(const float* a, const float* part_acc, const float* part_ml, int nsplit, int T, int H, int M, int dv,
                                   const float* coef, int unit_norm, float eps, float post_scale, const float* gate, long long ldg,
                                   void* out, int dt_out, const int* seq_of, const int* cu, int skip_from, int gate_wide,
                                   const int* positions, const double* vfreq, int rot_half, void* stream);

/* in [rows, ld_in] = [gate: F | up: F]; out [rows, F].  kind 0: gelu_tanh(g) u, 1: silu(g) u, 2: g' sigmoid(alpha g') (u' + 1) with
 * g' = min(g, limit), u' = clamp(u, -limit, limit), 3: relu(g)^2 of in [rows, ld_in >= F] (no up half).  n_tiles (device, may be null): only n_tiles[0] * tile_rows rows are computed. */
KB2SEQ_API int kb2_seq_glu(const void* in, int dt_in, long long ld_in, void* out, int dt_out, long long rows, int F, int kind, float limit,
                           float alpha, const int* n_tiles, int tile_rows, void* stream);

/* Router: z [T, ldz] fp32 logits of E outputs -> ids [T, top], weights [T, top].  score_kind 0 softmax, 1 sigmoid; choice = score +
 * correction (may be null); groups > 1: E / groups neighbours form a group, only the `keep` groups with the largest group score
 * (group_kind 0: the group's largest choice, 1: the sum of its two largest) can be chosen; weights are the chosen scores (without
 * correction), divided by their sum (+ 1e-20) if renorm, times out_scale. */
KB2SEQ_API int kb2_seq_route(const float* z, long long ldz, int T, int E, const float* correction, int score_kind, int groups, int keep,
                             int top, int renorm, float out_scale, int* ids, float* weights, int group_kind, void* stream);

/* Routed experts.  moe_bin: slots = T * top entries of ids; ids outside [0, E) are left out (identity experts).  Each expert's slots
 * form a run of rows padded to whole tiles of tile_rows (a multiple of kb2_seq_moe_tile_rows()): offs [E + 1], tile_expert [max_rows / tile], n_tiles [1],
 * slot_row [max_rows] (row -> slot, -1 padding), pos_of_slot [slots] (slot -> row, -1 left out); counts, cursor [E] are scratch;
 * max_rows >= slots + E * (tile - 1). */
KB2SEQ_API int kb2_seq_moe_tile_rows(void);
KB2SEQ_API int kb2_seq_moe_bin(const int* ids, long long slots, int E, int tile_rows, int* counts, int* offs, int* cursor, int* tile_expert,
                               int* n_tiles, int* slot_row, long long max_rows, int* pos_of_slot, void* stream);
/* C[p, :] = A[src(p), :] * B[tile_expert[p / tile]]^T (B: [experts][N][ldb], expert stride sB) for the rows of the first n_tiles[0] tiles;
 * src(p) = p, or row_map[p] / div when row_map is given (negative: zeros). */
KB2SEQ_API int kb2_seq_moe_gemm(const void* A, int dtA, long long lda, const int* row_map, int div, const void* B, int dtB, long long ldb,
                                long long sB, void* C, int dtC, long long ldc, int N, int K, const int* tile_expert, const int* n_tiles,
                                int max_tiles, int tile_rows, void* stream);
/* Few slots, no binning: C[slot, :] = A[slot / div, :] * B[ids[slot]]^T; slots with ids outside [0, E) are skipped. */
KB2SEQ_API int kb2_seq_moe_gemv(const void* A, int dtA, long long lda, int div, const int* ids, int E, const void* B, int dtB, long long ldb,
                                long long sB, void* C, int dtC, long long ldc, int slots, int N, int K, void* stream);
/* out[t, :] = sum_k weights[t, k] * (y[row of slot (t, k)] | h[t] if E <= ids < E + ident) + f shared[t] (may be null); pos_of_slot null:
 * the row of a slot is the slot itself.  f = sigmoid(shared_gate[t * ldsg]), or 1 when shared_gate is null. */
KB2SEQ_API int kb2_seq_moe_combine(const float* y, const int* pos_of_slot, const int* ids, const float* weights, int T, int top, int E,
                                   int ident, const void* h, int dt_h, const float* shared, float* out, int W, const float* shared_gate,
                                   long long ldsg, void* stream);

/* ---- third part (csrc/seq_rec.cu): linear recurrences with state slots, side-by-side mixers, depth-averaged residual stream ---- */

/* Gated linear attention over each sequence's portion: per head S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t with
 * alpha_t[i] = sigmoid(decay_in[t, h dk + i] + decay_bias[h dk + i])^(1 / tau) (decay_bias may be null).  qkv [T, ld] fp32 holds q and k
 * (H x dk columns from q_off / k_off; q is multiplied by q_scale) and v (H x dv from v_off).  state [slots][H][dk][dv] fp32 is read and
 * written back; out [T, H dv] fp32 is the raw read-out (kb2_seq_head_norm_gate finishes it).
 * scratch (fp32, T H dk elements, 16-byte aligned; may be null) selects the register-state kernel when dk is 32, 64, 128 or 256, dv a
 * multiple of 32, and qkv, ld and the three offsets are multiples of 16 bytes; otherwise a generic kernel runs (any dk <= 1024, any dv). */
KB2SEQ_API int kb2_seq_gla(const float* qkv, long long ld, int q_off, int k_off, int v_off, const float* decay_in, long long lda,
                           const float* decay_bias, float tau, float q_scale, int T, int S, int H, int dk, int dv, float* state,
                           const int* cu, const int* slots, float* scratch, float* out, void* stream);

/* Selective scan over each sequence's portion: per channel c and state n, S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,
 * y_c = sum_n S[c, n] C_n + D[c] x_c, out = y_c silu(z_c), with dt = softplus(dt_in + dt_bias), A = -exp(A_log [inner, N]).
 * x [T, ldx], dt_in [T, ldd], bc [T, ldb] = [B: N | C: N] from column b_off, z [T, ldz] from column z_off, all fp32.
 * state [slots][inner][N] fp32 is read and written back; out [T, inner] in dt_out. */
KB2SEQ_API int kb2_seq_selective_scan(const float* x, long long ldx, const float* dt_in, long long ldd, const float* dt_bias, const float* bc,
                                      long long ldb, int b_off, const float* z, long long ldz, int z_off, const float* A_log,
                                      const float* D, int T, int S, int inner, int N, float* state, const int* cu, const int* slots,
                                      void* out, int dt_out, void* stream);

/* out[t, h, :] = o[t, h, :] (o [T, ldo] fp32, H x dv columns), divided by its root mean square and times w [dv] if w is given, times
 * silu (gate_act 0) or sigmoid (1) of gate[t * ldg + h dv + :] if gate is given; out [T, H dv] in dt_out. */
KB2SEQ_API int kb2_seq_head_norm_gate(const float* o, long long ldo, const float* w, float eps, const float* gate, long long ldg, int gate_act,
                                      int T, int H, int dv, void* out, int dt_out, void* stream);

/* out[t, :n] = in[t, :n] / sqrt(mean(in[t, :n]^2) + eps) * w; in fp32 with row stride ld_in, out in dt_out with row stride ld_out */
KB2SEQ_API int kb2_seq_rms_rows(const float* in, long long ld_in, int n, const float* w, float eps, void* out, int dt_out, long long ld_out,
                                int T, void* stream);

/* out = coef (a / rms(a) * wa + b / rms(b) * wb) per row of W; a, b, out [T, W] fp32 */
KB2SEQ_API int kb2_seq_branch_merge(const float* a, const float* b, const float* wa, const float* wb, float eps, float coef, float* out, int T,
                                    int W, void* stream);

/* Depth-averaged residual stream.  stack [n][T][W] fp32 (element stride `stride` between results) holds the embedding output and the
 * results of the layers so far in its first n - 1 entries.  The newest result x + y (y may be null) is stored as entry n - 1; then
 * x <- sum_j coef[j] stack[j] (j < n, ascending), and h = x / rms(x) * w in dt_h if w is given. */
KB2SEQ_API int kb2_seq_depth_mix(float* stack, long long stride, int n, const float* coef, float* x, const float* y, const float* w, void* h,
                                 int dt_h, int T, int W, float eps, void* stream);

#ifdef __cplusplus
}
#endif
#endif
