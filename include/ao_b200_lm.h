/*
 * ao_b200_lm.h — C ABI of libao_b200_lm.so: B200 (sm_100a) kernels of the sequence-model mechanisms that are not
 * weight-only linears: fp32 residual stream with scalar-weight RMS norms, token shift, depth-weighted averaging of
 * layer results, latent (compressed key/value) attention with a softmax sink and an output gate, clipped-GLU experts
 * with a softmax top-k router; residual kept as several streams, gated per-channel recurrences, attention over chunks
 * with a ring cache; post-norm residual, causal attention with a sink, matrix-state recurrences (decayed linear
 * attention, state-space duality), sigmoid routers with group-limited choice.  Every constant of a mechanism is a parameter.
 *
 * Same boundary rules as ao_b200.h: device pointers + sizes + cudaStream_t as void*; nothing is allocated, freed,
 * synchronised or retained; every entry point can be captured into a CUDA graph; 0 = ok, else an AO_B200_ERR_* code.
 *
 * `dt` selects the storage type of weights, activations and caches: AO_LM_BF16 or AO_LM_F32.  The residual stream,
 * norm statistics, rotary angles, attention scores / weights and router scores are fp32 in both modes.
 * Per-token metadata lives in device memory: slot[t] = which sequence state the token belongs to, pos[t] = its
 * position in that sequence.  Tokens of one sequence are contiguous and in order.
 */
#ifndef AO_B200_LM_H_
#define AO_B200_LM_H_

#include "ao_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

enum { AO_LM_BF16 = 0, AO_LM_F32 = 1 };

AO_B200_API int ao_lm_abi_version(void);
/* text of the CUDA error behind the last AO_B200_ERR_CUDA that a call of this library returned ("" if none) */
AO_B200_API const char* ao_lm_last_cuda_error(void);

/* x[t][:] = table[tok[t]][:]  (fp32 out) */
AO_B200_API int ao_lm_embed(const void* table, int dt, const int64_t* tok, int64_t n, int64_t width, float* x, void* stream);

/* h[t] = x[t] + (prev - x[t]) * mu, prev = x[t-1] if that row is the same sequence's previous position, the saved row
 * state[slot[t]] if the sequence continues from an earlier step, zeros at position 0.  h is written in `dt`. */
AO_B200_API int ao_lm_token_shift(const float* x, const void* mu, int dt, const float* state, const int32_t* slot,
                                  const int32_t* pos, int64_t n, int64_t width, void* h, void* stream);

/* x_out = x_in + mult * g * y / sqrt(mean(y^2) + eps)   (g: ONE number, stored in `dt`; y in `y_dt`).
 * Optional, each skipped when its pointer is null:
 *   state:   the last row of every sequence in the batch saves x_in into state[slot] (the token-shift memory);
 *   streams: avg = sum_{j < n_streams} coef[j] * streams[j * stream_stride + ...] + coef[n_streams] * x_out  -> avg_out;
 *   cast_out: the last value computed (avg if streams, else x_out) in `dt`. */
AO_B200_API int ao_lm_residual_norm(const float* x_in, const void* y, int y_dt, const void* g, int dt, float mult, float eps,
                                    int64_t n, int64_t width, float* x_out, float* state, const int32_t* slot,
                                    const float* streams, int n_streams, int64_t stream_stride, const void* coef,
                                    float* avg_out, void* cast_out, void* stream);

/* out[i] = g * x[rows[i]] / sqrt(mean(x[rows[i]]^2) + eps) in `dt`; rows == null: all m rows in order. */
AO_B200_API int ao_lm_scalar_norm_rows(const float* x, const int32_t* rows, int64_t m, int64_t width, const void* g, int dt,
                                       float eps, void* out, void* stream);

/* Splits one projection row [q (H heads x (dn | dr)) at q_off | latent (R | dr) at kv_off, -1 = none | H gate logits
 * at g_off] of proj[n][ld]:
 *   qn[h][t][dn]  unrotated query parts, head-major, in `dt`;      qr[t][h][dr] rotated parts, fp32;
 *   gate[t][h] = sigmoid(logit), fp32;
 *   c_cache[slot][pos][R] = RMS norm (weight c_norm, eps) of the latent;  kr_cache[slot][pos][dr] = rotated shared key part.
 * Rotation: pairs (2i, 2i+1), i < rot_dims / 2, angle pos * inv_freq[i]; coordinates >= rot_dims pass through. */
AO_B200_API int ao_lm_latent_prep(const void* proj, int dt, int64_t ld, int64_t n, int H, int dn, int dr, int R, int64_t q_off,
                                  int64_t kv_off, int64_t g_off, const void* c_norm, float eps, int rot_dims,
                                  const float* inv_freq, const int32_t* slot, const int32_t* pos, void* c_cache,
                                  void* kr_cache, int64_t S, void* qn, float* qr, float* gate, void* stream);

/* Attention of (token, head) rows over the cached latents of their sequence, keys 0 .. pos[t]:
 *   score_j = scale * (qa[h][t] . c_j + qr[t][h] . kr_j);  weights = softmax with exp(sink[h]) added to the denominator;
 *   out[t][h][:] = gate[t][h] * sum_j weight_j * c_j      (R numbers, in `dt`).
 * tile_first / tile_count [n_tiles]: runs of <= tile_tokens consecutive rows of ONE sequence (ao_lm_latent_attention_plan
 * gives tile_tokens for a storage type and shape).  1 < n_split <= 64 splits the keys over CTAs (max_pos + 1 keys are
 * covered; workspace from ao_lm_latent_attention_workspace_bytes).
 * bf16 storage with R a multiple of 64 (<= 512) and dr a multiple of 16 runs on the tensor cores: queries and weights stay
 * fp32, split into two TF32 parts each, against the cached rows (exact in TF32); every other case is fp32 FMA code. */
AO_B200_API int ao_lm_latent_attention_plan(int dt, int H, int R, int dr, int* tile_tokens);
AO_B200_API int64_t ao_lm_latent_attention_workspace_bytes(int64_t n, int H, int R, int n_split);
AO_B200_API int ao_lm_latent_attention(const float* qa, const float* qr, const void* c_cache, const void* kr_cache, int dt,
                                       int64_t S, const int32_t* slot, const int32_t* pos, const int32_t* tile_first,
                                       const int32_t* tile_count, int n_tiles, int64_t n, int H, int R, int dr, float scale,
                                       const void* sink, const float* gate, int max_pos, int n_split, void* workspace,
                                       int64_t workspace_bytes, void* out, void* stream);

/* The same attention for prompt portions, in the expanded form (bf16 storage; tensor cores): the caller has up-projected
 * the cached latents of every sequence in the step into keys kx[row][h][dn] and values vx[row][h][dv], the rows of one
 * sequence contiguous from key 0;
 *   score_j = scale * (qn[h][t] . kx_j[h] + qr[t][h] . kr_j);  the same sink, gate and causal mask;  out[t][h][dv] in bf16.
 * tile_first / tile_count [n_tiles]: runs of <= tile_tokens consecutive rows of ONE sequence at consecutive positions;
 * tile_kv_row[tile]: the row of kx / vx that holds key 0 of the tile's sequence.  The plan call gives tile_tokens, or 0
 * when the shape is not covered (dn, dr, dv multiples of 16, dv up to 128): use ao_lm_latent_attention then.
 * Scores accumulate in fp32 (the fp32 rotated query part as two bf16 parts); the fp32 weights enter the value product
 * as three bf16 parts, i.e. exactly. */
AO_B200_API int ao_lm_latent_attention_expanded_plan(int dt, int dn, int dr, int dv, int* tile_tokens);
AO_B200_API int ao_lm_latent_attention_expanded(const void* qn, const float* qr, const void* kx, const void* vx,
                                                const void* kr_cache, int dt, int64_t S, const int32_t* slot,
                                                const int32_t* pos, const int32_t* tile_first, const int32_t* tile_count,
                                                const int32_t* tile_kv_row, int n_tiles, int64_t n, int H, int dn, int dr,
                                                int dv, float scale, const void* sink, const float* gate, void* out,
                                                void* stream);

/* Router: scores = softmax over all E logits (fp32 accumulation of h . w_router[e]); the `top` largest (ties: lowest
 * index) -> idx[t][top], weight[t][top] = their scores, not renormalised. */
AO_B200_API int ao_lm_router_topk(const void* h, const void* w_router, int dt, int64_t n, int64_t width, int E, int top,
                                  int32_t* idx, float* weight, void* stream);
/* The same choice from fp32 logits[n][E] that a GEMM has made (prompt portions). */
AO_B200_API int ao_lm_router_topk_logits(const float* logits, int64_t n, int E, int top, int32_t* idx, float* weight,
                                         void* stream);

/* Clipped GLU: g = min(a, limit), u = clamp(b, -limit, limit), y = g * sigmoid(alpha * g) * (u + 1).
 *   ao_lm_glu_act: gu[n][2 ff] = (a | b) -> y[n][ff].
 *   ao_lm_expert_gate_up: per (token, choice) pair p (t = p / top, expert = idx ? idx[p] : 0): a = w_gate[e] h[t],
 *       b = w_up[e] h[t] -> y[p][ff]        (w_gate / w_up: expert e's [ff][width] block starts expert_stride elements
 *       after expert e-1's, so one [E][2 ff][width] tensor can hold both).
 *   ao_lm_expert_down: out[t] (fp32) = (accumulate ? out[t] : 0) + sum_k weight[t][k] * w_down[e_k] y[t][k]
 *       (w_down: [E][width][ff]; weight == null: 1). */
AO_B200_API int ao_lm_glu_act(const void* gu, int dt, int64_t n, int64_t ff, float limit, float alpha, void* y, void* stream);
AO_B200_API int ao_lm_expert_gate_up(const void* h, const void* w_gate, const void* w_up, int dt, const int32_t* idx, int64_t n,
                                     int top, int64_t width, int64_t ff, int64_t expert_stride, float limit, float alpha,
                                     void* y, void* stream);
AO_B200_API int ao_lm_expert_down(const void* y, const void* w_down, int dt, const int32_t* idx, const float* weight, int64_t n,
                                  int top, int64_t width, int64_t ff, int accumulate, float* out, void* stream);

/* Prompt-sized mixtures: rows sorted by expert.  gather: xs[i] = h[src[i] / top]; scatter: out[src[i] / top] +=
 * weight[src[i]] * y[i] (fp32 atomics; out must hold the shared expert's output or zeros before). */
AO_B200_API int ao_lm_gather_rows(const void* h, int dt, const int64_t* src, int top, int64_t m, int64_t width, void* xs,
                                  void* stream);
AO_B200_API int ao_lm_scatter_add_rows(const void* y, int dt, const int64_t* src, const float* weight, int top, int64_t m,
                                       int64_t width, float* out, void* stream);

/* out[t][:] (fp32) = a[t][:] (fp32) + b[t][:] (dt) */
AO_B200_API int ao_lm_add_cast(const void* b, int dt, int64_t count, float* a_inout, void* stream);

/* greedy choice: out[b] = index of the largest of logits[b][0..V) (first one on ties) */
AO_B200_API int ao_lm_argmax(const float* logits, int64_t ld, int64_t B, int64_t V, int64_t* out, void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * Residual kept as n_streams fp32 copies per token, x[t][s][width] (one stream: the ordinary residual), recurrent
 * mixers with per-slot state, attention over chunks with a ring cache.  Rows of a step are runs ("segments") of
 * consecutive positions of one sequence: back[t] = rows of the same segment in front of row t, ahead[t] = behind it.
 */

/* x[t][s][:] = table[tok[t]][:] * scale + sinusoid(pos[t]) for every stream s; coordinate 2i of the sinusoid is
 * sin(pos * freq[i]), 2i+1 the cosine (freq: width / 2 rounded up doubles; the angle is reduced in double). */
AO_B200_API int ao_lm_embed_sinusoid(const void* table, int dt, const int64_t* tok, const int32_t* pos, int64_t n,
                                     int64_t width, float scale, const double* freq, int n_streams, float* x, void* stream);

/* Read-out + norm: u = sum_s coef_in[s] x[r][s] (coef_in == null: plain sum), out[i] = u / sqrt(mean(u^2) + eps) *
 * (weight_offset + weight[:]) for r = rows ? rows[i] : i, i < m.  Written as fp32 (out_f32) and / or in `dt` (out). */
AO_B200_API int ao_lm_streams_norm(const float* x, const int32_t* rows, int64_t m, int n_streams, int64_t width,
                                   const void* coef_in, const void* weight, int dt, float weight_offset, float eps,
                                   float* out_f32, void* out, void* stream);

/* Write-back: x[t][d] <- sum_s mix[s][d] x[t][s] + coef_out[d] * y[t], all streams from the old ones (mix == null:
 * identity; coef_out == null: ones; y in y_dt).  With conv_state: rows with ahead == 0 also move the last taps - 1 rows
 * of conv_in (fp32 [n][width]) into conv_state[slot][taps - 1][width], the memory of ao_lm_causal_conv. */
AO_B200_API int ao_lm_streams_update(float* x, const void* y, int y_dt, int64_t n, int n_streams, int64_t width,
                                     const void* mix, const void* coef_out, int dt, const float* conv_in, float* conv_state,
                                     int taps, const int32_t* slot, const int32_t* back, const int32_t* ahead, void* stream);

/* y[t][c] = gelu_tanh(gu[t][c]) * gu[t][ff + c] */
AO_B200_API int ao_lm_gelu_glu(const void* gu, int dt, int64_t n, int64_t ff, void* y, void* stream);

/* Causal convolution over time per channel: v(t) = x[t][c] + in_bias[c];
 * y[t][c] = (residual ? v(t) : 0) + out_bias[c] + sum_j kernel[c][j] * v(t - (taps - 1 - j)).  Inputs in front of the
 * step come from state[slot][taps - 1][channels] (oldest first, bias included), inputs in front of position 0 are zero.
 * The kernel does not write the state: ao_lm_streams_update / ao_lm_rglru_scan do, after every reader has run.
 * taps == 1 reads no state (pass any valid pointer). */
AO_B200_API int ao_lm_causal_conv(const float* x, int64_t ldx, const void* in_bias, int64_t n, int64_t channels, int taps,
                                  const void* kernel, const void* out_bias, int dt, int residual, const float* state,
                                  const int32_t* slot, const int32_t* pos, const int32_t* back, float* out_f32, void* out,
                                  void* stream);

/* Gated linear recurrences S_t = a_t S_(t-1) + b_t per channel, state[slot][channels] fp32 (read unless the segment
 * starts at position 0, written with the segment's last S).  tile_first / tile_count: runs of rows of ONE segment.
 * seg_tile0 == null: every tile is a whole segment (one launch).  Otherwise segment k owns tiles seg_tile0[k] ..
 * + seg_tiles[k] - 1 and the scan takes three launches (tile summaries, carries, rows) with a workspace of
 * ao_lm_scan_workspace_bytes.
 *   mingru: z = sigmoid(proj[t][z_off + c] + z_bias[c]), u = proj[t][x_off + c] + x_bias[c], cand = u + 1/2 (u >= 0) |
 *           sigmoid(u); a = 1 - z, b = z * cand;  out[t][c] = out_scale * S_t * silu(proj[t][g_off + c]).
 *   rglru:  gates[block][t][2 bw] = (r | i) pre-activations of the block's bw channels; r = sigmoid(. + r_bias),
 *           i = sigmoid(. + i_bias); log a = -decay * r * softplus(lam[c]); b = sqrt(1 - a^2) * i * u[t][c];
 *           out[t][c] = S_t * gelu_tanh(y_pre[t][c] + y_bias[c]).  With conv_state, the segment's last rows of
 *           conv_x (+ conv_in_bias) become the memory of the convolution that produced u. */
AO_B200_API int64_t ao_lm_scan_workspace_bytes(int n_tiles, int64_t channels);
AO_B200_API int ao_lm_mingru_scan(const float* proj, int64_t ld, int64_t z_off, int64_t x_off, int64_t g_off, const void* z_bias,
                                  const void* x_bias, int dt, int64_t channels, float* state, const int32_t* slot,
                                  const int32_t* pos, const int32_t* back, const int32_t* tile_first, const int32_t* tile_count,
                                  int n_tiles, const int32_t* seg_tile0, const int32_t* seg_tiles, int n_segments,
                                  float* workspace, float out_scale, void* out, int64_t ld_out, void* stream);
AO_B200_API int ao_lm_rglru_scan(const float* gates, int64_t n, int block_width, const void* r_bias, const void* i_bias,
                                 const void* lam, float decay, const float* u, const float* y_pre, int64_t ld_y,
                                 const void* y_bias, int dt, int64_t channels, float* state, const float* conv_x,
                                 int64_t conv_ld, const void* conv_in_bias, float* conv_state, int taps, const int32_t* slot,
                                 const int32_t* pos, const int32_t* back, const int32_t* tile_first, const int32_t* tile_count,
                                 int n_tiles, const int32_t* seg_tile0, const int32_t* seg_tiles, int n_segments,
                                 float* workspace, void* out, void* stream);

/* Attention over chunks of `chunk` positions (a query sees the keys of its own chunk up to itself), H query heads over
 * G key/value heads.  ao_lm_qk_prep: unit-RMS queries (fp32 [n][H][d]) and keys (`dt` [n][G][d]) and the values in
 * `dt` [n][G][dv] from an fp32 projection row.  ao_lm_chunk_attention:
 *   score = softcap * tanh(scale * q.k / softcap) (softcap <= 0: none) + dist_bias[head][min(i - j, n_dist - 1)];
 *   out[t][head * dv + c] = out_scale * softmax-weighted values * sigmoid(gate[t][head * dv + c]).
 * Keys of earlier steps come from the ring (ring_k [slots][chunk][G][d], ring_v likewise; position p in row p % chunk),
 * the step's own from kn / vn.  tile_first / tile_count: runs of <= tile_rows rows of one segment INSIDE one chunk
 * (ao_lm_chunk_attention_plan gives tile_rows, 0 = shape not covered).  ao_lm_ring_append, after the attention, stores
 * the step's rows that no later row of the step overwrites (ahead < chunk). */
AO_B200_API int ao_lm_qk_prep(const float* proj, int64_t ld, int64_t q_off, int64_t k_off, int64_t v_off, int64_t n, int H, int G,
                              int d, int dv, float eps, int dt, float* qn, void* kn, void* vn, void* stream);
AO_B200_API int ao_lm_chunk_attention_plan(int dt, int H, int G, int d, int dv, int* tile_rows);
/* 1 < n_split <= 64 spreads a tile's key blocks over that many CTAs and adds a merge launch (few rows over many keys:
 * a decoded token late in its chunk); shares past a sequence's keys leave at once, so n_split may be fixed for a graph. */
AO_B200_API int64_t ao_lm_chunk_attention_workspace_bytes(int n_tiles, int G, int dv, int n_split);
AO_B200_API int ao_lm_chunk_attention(const float* qn, const void* kn, const void* vn, const void* ring_k, const void* ring_v,
                                      int dt, const float* gate, int64_t ld_gate, const float* dist_bias, int n_dist,
                                      const int32_t* slot, const int32_t* pos, const int32_t* back, const int32_t* tile_first,
                                      const int32_t* tile_count, int n_tiles, int H, int G, int d, int dv, int chunk,
                                      float scale, float softcap, float out_scale, int n_split, void* workspace,
                                      int64_t workspace_bytes, void* out, int64_t ld_out, void* stream);
/* The same attention on the tensor cores for prompt portions (bf16 storage; d and dv multiples of 16, dv <= 128): tiles
 * of <= tile_rows (64) rows of one segment inside one chunk x one query head.  Queries and keys enter as bf16 operands
 * with fp32 accumulation; the fp32 weights enter the value product as three bf16 parts, i.e. exactly.  The plan call
 * gives tile_rows, or 0 when the shape is not covered (use ao_lm_chunk_attention then). */
AO_B200_API int ao_lm_chunk_attention_prompt_plan(int dt, int H, int G, int d, int dv, int* tile_rows);
AO_B200_API int ao_lm_chunk_attention_prompt(const float* qn, const void* kn, const void* vn, const void* ring_k,
                                             const void* ring_v, int dt, const float* gate, int64_t ld_gate,
                                             const float* dist_bias, int n_dist, const int32_t* slot, const int32_t* pos,
                                             const int32_t* back, const int32_t* tile_first, const int32_t* tile_count,
                                             int n_tiles, int H, int G, int d, int dv, int chunk, float scale, float softcap,
                                             float out_scale, void* out, int64_t ld_out, void* stream);
AO_B200_API int ao_lm_ring_append(const void* kn, const void* vn, int64_t n, int64_t k_row, int64_t v_row, int ring, int dt,
                                  const int32_t* slot, const int32_t* pos, const int32_t* ahead, void* ring_k, void* ring_v,
                                  void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * Post-norm residual, full causal attention with a sink, matrix-state recurrences (decayed linear attention, state-space
 * duality), sigmoid routers with group-limited choice, SiLU-gated experts.
 */

/* y[t] += y_bias (fp32 [width]);  x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * post_w;  x[t] += add_rows[t];  x[t] += add_vec;
 * h[t] = x[t] / sqrt(mean(x[t]^2) + eps) * next_w  (in `dt`).   Every part but x is optional (null): y with post_w (null:
 * ones) is a sublayer's result entering through its own norm (y_bias: the bias of the projection that made y, when its GEMM
 * left it out), add_rows (fp32 [n][width]) and add_vec (`dt` [width]) are
 * what a pass over a looped span of layers adds in front of its first layer, next_w is the next sublayer's input norm. */
AO_B200_API int ao_lm_postnorm_residual(float* x, const void* y, int y_dt, const float* y_bias, const void* post_w, const float* add_rows,
                                        const void* add_vec, const void* next_w, int dt, float eps, int64_t n, int64_t width,
                                        void* h, void* stream);

/* ao_lm_qk_prep with what a design may put between the projection and the attention (each optional, null / 0 = none):
 * biases added to the projection (`dt`; q_bias [H d], k_bias [G d], v_bias [G dv]), a weight per coordinate on the
 * unit-RMS queries and keys (`dt` [d], shared by the heads), and a query temperature
 * q *= 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1).  With ring_k / ring_v (a ring of `ring` rows that never wraps: a
 * full cache) the keys and values also go to row pos[t] of slot[t], which saves the ao_lm_ring_append launch: the attention
 * reads a step's own rows from kn / vn and only earlier positions from the ring, so the order does not matter there. */
AO_B200_API int ao_lm_qk_norm_prep(const float* proj, int64_t ld, int64_t q_off, int64_t k_off, int64_t v_off, const void* q_bias,
                                   const void* k_bias, const void* v_bias, const void* q_weight, const void* k_weight,
                                   float temp_coef, int temp_every, const int32_t* pos, const int32_t* slot, void* ring_k,
                                   void* ring_v, int ring, int64_t n, int H, int G, int d, int dv, float eps, int dt, float* qn,
                                   void* kn, void* vn, void* stream);

/* ao_lm_chunk_attention / ao_lm_chunk_attention_prompt with gate and dist_bias optional (null) and a sink: exp(sink[head])
 * (fp32 [H]; null: none) joins every row's softmax denominator, without a key or a value and unscaled.  With `chunk` = the
 * rows of the ring (the longest sequence a slot holds) this is plain causal attention over a full key/value cache. */
AO_B200_API int ao_lm_sink_attention(const float* qn, const void* kn, const void* vn, const void* ring_k, const void* ring_v,
                                     int dt, const float* gate, int64_t ld_gate, const float* dist_bias, int n_dist,
                                     const float* sink, const int32_t* slot, const int32_t* pos, const int32_t* back,
                                     const int32_t* tile_first, const int32_t* tile_count, int n_tiles, int H, int G, int d,
                                     int dv, int chunk, float scale, float softcap, float out_scale, int n_split,
                                     void* workspace, int64_t workspace_bytes, void* out, int64_t ld_out, void* stream);
AO_B200_API int ao_lm_sink_attention_prompt(const float* qn, const void* kn, const void* vn, const void* ring_k,
                                            const void* ring_v, int dt, const float* gate, int64_t ld_gate,
                                            const float* dist_bias, int n_dist, const float* sink, const int32_t* slot,
                                            const int32_t* pos, const int32_t* back, const int32_t* tile_first,
                                            const int32_t* tile_count, int n_tiles, int H, int G, int d, int dv, int chunk,
                                            float scale, float softcap, float out_scale, void* out, int64_t ld_out,
                                            void* stream);

/* Matrix-state recurrence per head: S_t = a_t S_(t-1) + b_t k_t v_t^T (S: d x dv, fp32 state[slots][H][d][dv], zeros at
 * position 0), out[t][h] = S_t^T q_t + skip[h] v_t (fp32).  q and k rows hold G groups of d (head h reads group
 * h / (H / G)), v rows H heads of dv; act = 1 applies SiLU to q, k and v on load.  a, b: fp32 [n][ld_ab] per (row, head);
 * a == null: a_t = a_head[h] and b_t = 1 (a fixed decay per head).
 * seg_tile0 == null: seg_first / seg_count are the step's segments (runs of consecutive rows of one sequence), whole; one
 * launch, a CTA walks its segment row by row (decoded tokens, short portions).
 * Otherwise seg_first / seg_count are TILES of rows inside segments and segment s of n_whole_segments owns tiles
 * seg_tile0[s] .. + seg_tiles[s] - 1: three launches (every tile from a zero state; the tiles' start states carried
 * through each segment, element by element; the read-out of each tile's start state added to its rows), with a workspace
 * of ao_lm_outer_recurrence_workspace_bytes.  Both forms compute the same sums in fp32; they differ in rounding only. */
AO_B200_API int64_t ao_lm_outer_recurrence_workspace_bytes(int n_tiles, int64_t n, int H, int d, int dv);
AO_B200_API int ao_lm_outer_recurrence(const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v, int64_t ldv,
                                       int act, const float* a, const float* b, int64_t ld_ab, const float* a_head,
                                       const float* skip, int H, int G, int d, int dv, float* state, const int32_t* slot,
                                       const int32_t* pos, const int32_t* seg_first, const int32_t* seg_count, int n_segments,
                                       const int32_t* seg_tile0, const int32_t* seg_tiles, int n_whole_segments, int64_t n,
                                       float* workspace, float* out, int64_t ld_out, void* stream);

/* Input side of a state-space mixer, from an fp32 projection row: conv_out[t][c] = silu(conv_b[c] + sum_j conv_w[c][j] *
 * u(t - (taps - 1 - j))) over the `channels` values at conv_off (inputs in front of the step from conv_state[slot][taps - 1]
 * [channels], oldest first; zeros in front of position 0), and per head step = softplus(proj[t][dt_off + h] + dt_bias[h]),
 * a_out = exp(-exp(a_log[h]) * step), b_out = step.  ao_lm_conv_state_save, after every reader has run, makes the last
 * taps - 1 inputs of each segment (x = the projection at conv_off, row stride ldx) the slot's new memory. */
AO_B200_API int ao_lm_ssd_prep(const float* proj, int64_t ld, int64_t conv_off, int64_t dt_off, int64_t n, int64_t channels,
                               int taps, const void* conv_w, const void* conv_b, int dt, const float* conv_state,
                               const int32_t* slot, const int32_t* pos, const int32_t* back, int H, const void* dt_bias,
                               const void* a_log, float* conv_out, float* a_out, float* b_out, void* stream);
AO_B200_API int ao_lm_conv_state_save(const float* x, int64_t ldx, int64_t n, int64_t channels, int taps, const int32_t* slot,
                                      const int32_t* pos, const int32_t* back, const int32_t* ahead, float* state,
                                      void* stream);

/* RMS norm over each of `groups` equal parts of a row, with a gate:  mode 0: out = norm(y) * weight * sigmoid(gate);
 * mode 1: out = norm(y * silu(gate)) * weight;  mode 2: out = norm(y) * weight * silu(gate).  weight == null: ones.
 * y, gate fp32 with row strides; out [n][width] in `dt`. */
AO_B200_API int ao_lm_gated_group_norm(const float* y, int64_t ldy, const float* gate, int64_t ldg, int mode, int64_t n,
                                       int64_t width, int groups, const void* weight, int dt, float eps, void* out,
                                       void* stream);

/* Router over fp32 logits[n][E]: s = sigmoid(logit), choice on s + correction (fp32 [E]; null: none), restricted to the
 * `keep` best of n_groups equal groups of neighbouring experts (group score = sum of its two largest choice scores);
 * idx[t][top] = the `top` largest choice scores (ties: lowest index), weight = s / (sum of the chosen s + 1e-20) * scale. */
AO_B200_API int ao_lm_router_group_topk_logits(const float* logits, int64_t n, int E, int top, const float* correction,
                                               int n_groups, int keep, float scale, int32_t* idx, float* weight,
                                               void* stream);

/* ao_lm_glu_act / ao_lm_expert_gate_up with the constant added to the up branch as a parameter:
 * y = g * sigmoid(alpha * g) * (u + shift); limit = +inf, alpha = 1, shift = 0 is the plain SiLU-gated unit. */
AO_B200_API int ao_lm_glu_act_shift(const void* gu, int dt, int64_t n, int64_t ff, float limit, float alpha, float shift, void* y,
                                    void* stream);
AO_B200_API int ao_lm_expert_gate_up_shift(const void* h, const void* w_gate, const void* w_up, int dt, const int32_t* idx,
                                           int64_t n, int top, int64_t width, int64_t ff, int64_t expert_stride, float limit,
                                           float alpha, float shift, void* y, void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * Layer-norm residual, rotary positions on a projection, time mixing with a decay per key channel, attention under a
 * sliding window that keeps the first tokens (with several maps per head), routers that renormalise over the chosen
 * experts, experts without a gate.
 */

/* x[r] += mult * y[r] (y fp32 [n][width]; null: nothing is added);  out[i] = (x[r] - mean) / sqrt(var + eps) * weight + bias
 * with var the mean of the squared deviations (weight null: no norm, only the add; bias null: none), r = rows ? rows[i] : i
 * (rows only without y).  The result is written as fp32 (out_f32) and / or in `dt` (out), [m][width]. */
AO_B200_API int ao_lm_add_layer_norm(float* x, const float* y, float mult, const int32_t* rows, int64_t m, int64_t width,
                                     const void* weight, const void* bias, int dt, float eps, float* out_f32, void* out,
                                     void* stream);

/* Rotary positions, in place, on two blocks of an fp32 projection row (block a: heads_a heads of d at off_a, block b
 * likewise; a block of 0 heads is skipped): the first rot_dims coordinates of every head turn by pos * inv_freq[i]
 * (fp32 [rot_dims / 2]); pairing 0 couples (2i, 2i + 1), pairing 1 couples (i, i + rot_dims / 2); then the whole head is
 * multiplied by the block's scale. */
AO_B200_API int ao_lm_rotary_rows(float* proj, int64_t ld, int64_t n, const int32_t* pos, const float* inv_freq, int rot_dims,
                                  int pairing, int d, int64_t off_a, int heads_a, float scale_a, int64_t off_b, int heads_b,
                                  float scale_b, void* stream);

/* mixes[s][t][:] = h[t] + (prev - h[t]) * mu[s][:] for s < n_mix (mu: `dt` [n_mix][width], mixes: `dt` [n_mix][n][width]);
 * prev = h[t - 1] when back[t] > 0, the slot's saved row state[slot[t]] when the segment continues an earlier step, zeros
 * at position 0.  The state is written by the recurrence that ends the layer (ao_lm_channel_recurrence). */
AO_B200_API int ao_lm_token_shift_mix(const float* h, const void* mu, int n_mix, int dt, const float* state, const int32_t* slot,
                                      const int32_t* pos, const int32_t* back, int64_t n, int64_t width, void* mixes,
                                      void* stream);

/* out[t][c] = f(in[t][c]) * row_scale[t * ld_scale] (row_scale null: 1); kind 0: relu(z)^2, kind 1: tanh(z), kind 2:
 * param * tanh(z / param) (a soft cap).  (in_dt, out_dt): (F32, F32), (F32, BF16) or (BF16, BF16); out may be in. */
AO_B200_API int ao_lm_unary_rows(const void* in, int in_dt, int64_t n, int64_t cols, int kind, float param, const float* row_scale,
                                 int64_t ld_scale, void* out, int out_dt, void* stream);

/* Matrix-state recurrence with a decay per key channel and a bonus for the current token, per head (S: d x dv, fp32
 * state[slots][H][d][dv], zeros at position 0):
 *   out[t][h] = (S_(t-1) + diag(bonus_h) k_t v_t^T)^T r_t,     S_t = diag(w_t) S_(t-1) + k_t v_t^T.
 * r, k, w rows hold H heads of d, v rows H heads of dv (fp32).  w_bias (`dt` [H d]) non-null: the decay is made on load
 * from its pre-activation, w = exp(-exp(w + w_bias)).  bonus: `dt` [H d] or null.  d <= 128.
 * Segments and the tiled form as in ao_lm_outer_recurrence (workspace from ao_lm_channel_recurrence_workspace_bytes).
 * With shift_state, the last row of every segment of shift_src (fp32 [n][shift_width]) becomes shift_state[slot]: the
 * memory of the token shift that made this layer's inputs. */
AO_B200_API int64_t ao_lm_channel_recurrence_workspace_bytes(int n_tiles, int64_t n, int H, int d, int dv);
AO_B200_API int ao_lm_channel_recurrence(const float* r, int64_t ldr, const float* k, int64_t ldk, const float* v, int64_t ldv,
                                         const float* w, int64_t ldw, const void* w_bias, const void* bonus, int dt, int H, int d,
                                         int dv, float* state, const int32_t* slot, const int32_t* pos, const int32_t* seg_first,
                                         const int32_t* seg_count, int n_segments, const int32_t* seg_tile0,
                                         const int32_t* seg_tiles, int n_whole_segments, int64_t n, float* workspace,
                                         const float* shift_src, float* shift_state, int64_t shift_width, float* out,
                                         int64_t ld_out, void* stream);

/* Attention under a sliding window that keeps the first tokens: the query at position i sees key j when j <= i and
 * (i - j < window or j < keep).  n_maps (1 or 2) attention maps per head with queries and keys of their own over the same
 * values: qn fp32 [n][H][n_maps][d], keys `dt` [..][G][n_maps][d], values `dt` [..][G][dv]; two maps give
 * a_1 - lambda * a_2.  unit_rms != 0 divides the result by sqrt(mean over dv of its squares + eps); then times out_scale.
 * ao_lm_qkv_rotary_prep: projection row (fp32) -> biases (`dt`, null: none), rotation (as ao_lm_rotary_rows) of q_heads
 * query heads and k_heads key heads of d, values copied; k_heads == 0: queries only.
 * Keys of earlier steps: position p in row p % ring of ring_k / ring_v [slots][ring][...] (ring >= window), and the first
 * first_rows (>= keep) positions in first_k / first_v [slots][first_rows][...]; the step's own rows from kn / vn.
 * ao_lm_window_append stores the step's rows, after the last layer that reads the cache has run.
 * tile_first / tile_count: runs of <= tile_rows consecutive rows of one segment (ao_lm_window_attention_plan; 0 = shape not
 * covered).  n_split > 1 (<= 64): the keys of a tile are shared out over that many CTAs and a second launch merges their
 * results (few rows over a long window: a decoded token); workspace of ao_lm_window_attention_workspace_bytes. */
AO_B200_API int ao_lm_qkv_rotary_prep(const float* proj, int64_t ld, int64_t q_off, int64_t k_off, int64_t v_off,
                                      const void* q_bias, const void* k_bias, const void* v_bias, const int32_t* pos,
                                      const float* inv_freq, int rot_dims, int pairing, int64_t n, int q_heads, int k_heads, int d,
                                      int v_width, int dt, float* qn, void* kn, void* vn, void* stream);
AO_B200_API int ao_lm_window_append(const void* kn, const void* vn, int64_t n, int64_t k_row, int64_t v_row, int ring,
                                    int first_rows, int dt, const int32_t* slot, const int32_t* pos, const int32_t* ahead,
                                    void* ring_k, void* ring_v, void* first_k, void* first_v, void* stream);
AO_B200_API int ao_lm_window_attention_plan(int dt, int n_maps, int H, int G, int d, int dv, int* tile_rows);
AO_B200_API int ao_lm_window_attention(const float* qn, const void* kn, const void* vn, const void* ring_k, const void* ring_v,
                                       const void* first_k, const void* first_v, int ring, int first_rows, int dt,
                                       const int32_t* slot, const int32_t* pos, const int32_t* back, const int32_t* tile_first,
                                       const int32_t* tile_count, int n_tiles, int n_maps, int H, int G, int d, int dv,
                                       int window, int keep, float scale, float lambda, int unit_rms, float eps, float out_scale,
                                       int n_split, void* workspace, int64_t workspace_bytes, void* out, int64_t ld_out,
                                       void* stream);
AO_B200_API int64_t ao_lm_window_attention_workspace_bytes(int n_tiles, int n_maps, int H, int G, int dv, int n_split);
/* The same attention for prompt portions on the tensor cores (bf16 storage; d and dv multiples of 16, dv <= 128): tiles of
 * ao_lm_window_attention_prompt_plan rows (0 = shape not covered), one CTA per (tile, query head). */
AO_B200_API int ao_lm_window_attention_prompt_plan(int dt, int n_maps, int H, int G, int d, int dv, int* tile_rows);
AO_B200_API int ao_lm_window_attention_prompt(const float* qn, const void* kn, const void* vn, const void* ring_k, const void* ring_v,
                                              const void* first_k, const void* first_v, int ring, int first_rows, int dt,
                                              const int32_t* slot, const int32_t* pos, const int32_t* back,
                                              const int32_t* tile_first, const int32_t* tile_count, int n_tiles, int n_maps,
                                              int H, int G, int d, int dv, int window, int keep, float scale, float lambda,
                                              int unit_rms, float eps, float out_scale, void* out, int64_t ld_out, void* stream);

/* Router over fp32 logits[n][ld] (+ bias, fp32 [E], null: none): the `top` largest logits (ties: lowest index) ->
 * idx[t][top], weight = softmax over the chosen logits only.  extra >= 0: extra_out[t] = sigmoid(logits[t][extra]), a gate
 * whose logit the same GEMM made. */
AO_B200_API int ao_lm_router_topk_renorm_logits(const float* logits, int64_t ld, const float* bias, int64_t n, int E, int top,
                                                int extra, int32_t* idx, float* weight, float* extra_out, void* stream);

/* ao_lm_expert_gate_up for experts without a gate: y[p][ff] = act(w_up[e] h[t]); act 0: relu(.)^2. */
AO_B200_API int ao_lm_expert_up_act(const void* h, const void* w_up, int dt, const int32_t* idx, int64_t n, int top, int64_t width,
                                    int64_t ff, int64_t expert_stride, int act, void* y, void* stream);

#ifdef __cplusplus
}
#endif
#endif
