/* omchat_b200 sequence-step kernels: the second C-ABI library (libomchat_b200_seq.so).
 *
 * Kernels for decoders that keep their residual stream in fp32 and run packed "steps" (portions of prompts beside single
 * decoded tokens) against a paged cache: latent (compressed key/value) attention with an optional softmax sink, rotary
 * tables with pairwise-interleaved layout and optional frequency blending, output-side RMS norms, a score-corrected router
 * with identity experts, and a linear layer for any shape and for fp32 as well as bf16 storage. Same conventions as
 * omchat_b200.h: device pointers + sizes, leading dimensions in ELEMENTS, asynchronous on `stream`, nothing is allocated,
 * 0 or a negative OMC_ERR_* code is returned and omc_last_error() holds the message.
 *
 * dtype codes: OMC_DT_F32 = 0 (float), OMC_DT_BF16 = 1 (raw bf16). Accumulation is always fp32.
 */
#ifndef OMCHAT_B200_SEQ_H_
#define OMCHAT_B200_SEQ_H_

#include <stdint.h>

#include "omchat_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define OMC_DT_F32 0
#define OMC_DT_BF16 1

#define OMC_ACT_NONE 0
#define OMC_ACT_RELU2 1     /* max(z, 0)^2 */
#define OMC_ACT_GELU_TANH 2 /* 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))) */
#define OMC_ACT_GELU_ERF 3  /* 0.5 z (1 + erf(z / sqrt 2)) */
#define OMC_ACT_CLAMP_SWISH 4 /* omc_glu_mul only: a clamped gate times a clamped, shifted second half */
#define OMC_ACT_SILU 5      /* omc_glu_mul only: z sigmoid(z) */

/* Y[b][M,N] = act(alpha * X[b][M,K] W[b][N,K]^T) for b < batch, any M, N, K >= 1 (edges are bounds-checked).
 * x_dt / w_dt / y_dt: dtype codes; allowed (x, w): (f32, f32), (f32, bf16), (bf16, bf16). sx / sw / sy: element offsets
 * between consecutive batch items (heads that are column slices of one row-major buffer: sx = slice width).
 * tile_group != NULL (batch must be 1): rows come in tiles of 64; tile i multiplies by W + tile_group[i] * group_stride
 * (elements) and is skipped when tile_group[i] < 0 - the expert-sorted rows of a mixture-of-experts block. The number of
 * tiles is ceil(M / 64). Every output element accumulates along K in the same order whatever M is, so a row's result does not
 * depend on what else is in the batch. */
int omc_linear(const void* X, int x_dt, long long ldx, long long sx, const void* W, int w_dt, long long ldw, long long sw,
               void* Y, int y_dt, long long ldy, long long sy, int M, int N, int K, int batch, float alpha, int act,
               const int32_t* tile_group, long long group_stride, void* stream);

/* h32[t,:] = table[ids[t],:] * scale (fp32 residual stream), xb[t,:] = the same rounded to xb_dt (the first sublayer's
 * input; NULL to skip). ids int32; ids outside [0, vocab) give zero rows. */
int omc_embed_scale(const int32_t* ids, int T, const void* table, int t_dt, int C, int vocab, float scale, float* h32,
                    long long ldh, void* xb, int xb_dt, long long ldxb, void* stream);

/* y[t,:] = x[t,:n] / sqrt(mean(x[t,:n]^2) + eps) * (w or 1 + w). x fp32, w of dtype w_dt (NULL: no weight), y of y_dt. */
int omc_rms_rows(const float* x, long long ldx, const void* w, int w_dt, int one_plus, float eps, void* y, int y_dt,
                 long long ldy, int rows, int n, void* stream);

/* Output-side norm + residual: h32[t,:] += y[t,:] / sqrt(mean(y[t,:]^2) + eps) * (1 + w); xb[t,:] = round(h32[t,:]) (NULL to skip).
 * y fp32 (the sublayer's output), w of w_dt. */
int omc_norm_residual(const float* y, long long ldy, const void* w, int w_dt, float eps, float* h32, long long ldh, void* xb,
                      int xb_dt, long long ldxb, int rows, int C, void* stream);

/* Latent key/value rows of a step -> paged cache. dkv fp32 [T, r + dr]: the first r columns are RMS-normed with weight w
 * (plain weight) and stored as the latent; of the last dr columns the first `rot_dims` are rotated pairwise (2i, 2i+1) by
 * cs[pos[t]] ([n_pos][rot_dims/2][2] fp32: cos, sin of position x pair frequency, built by the host) and all dr are stored behind the latent. Row t goes to page
 * block_table[slot[t]][pos[t] / page_size], place pos[t] % page_size; the pool is [pages][page_size][r + dr] of pool_dt. */
int omc_latent_kv_store(const float* dkv, long long ld, int T, int r, int dr, const void* w, int w_dt, float eps, const float* cs,
                        int rot_dims, const int32_t* pos, const int32_t* slot, const int32_t* block_table, int max_pages,
                        int page_size, void* pool, int pool_dt, void* stream);

/* omc_latent_kv_store and omc_rotary_q in one launch; w, pool, q and qcat share the dtype dt. */
int omc_latent_rope_store(const float* dkv, long long ld, int T, int r, int dr, const void* w, float eps, const float* cs, int rot_dims,
                          const int32_t* pos, const int32_t* slot, const int32_t* block_table, int max_pages, int page_size, void* pool,
                          const void* q, long long ldq, int H, int dn, void* qcat, int dt, void* stream);

/* Rotated query parts: q [T, H * (dn + dr)] of in_dt (per head dn unrotated then dr rotated dims) -> qcat[t][h][r + j] for
 * j < dr (qcat is [T, H, r + dr] of q_dt; its first r columns per head are written by the absorbing omc_linear). */
int omc_rotary_q(const void* q, int in_dt, long long ldq, int T, int H, int dn, int dr, const float* cs, int rot_dims,
                 const int32_t* pos, void* qcat, int q_dt, int r, void* stream);

/* Paged latent attention, any sizes (the plain kernel: fp32 arithmetic, one CTA per (row, head)).
 * qcat [T, H, r + dr] (absorbed query | rotated query), pool as omc_latent_kv_store writes it. Row t of slot[t] at position
 * pos[t] sees the cached entries 0..pos[t] of its slot: score_j = qcat[t,h] . entry_j * scale, softmax over j with the optional
 * extra denominator term exp(sink[h]) (sink fp32 [H] or NULL), out[t,h,:] = sum_j p_j entry_j[:r] (fp32 [T, H, r]). r <= 1024. */
int omc_latent_attn(const void* qcat, int q_dt, int T, int H, int r, int dr, const void* pool, int pool_dt,
                    const int32_t* block_table, int max_pages, int page_size, const int32_t* pos, const int32_t* slot,
                    const float* sink, float scale, float* out, void* stream);

/* Tensor-core version of the same (bf16 only; r a multiple of 16 up to 512, dr a multiple of 16, H <= 64): mma.sync over 64-key
 * tiles that serve as keys AND values; the 64 rows of a tile are (token, head) pairs. The host lists the work:
 *   items[i]  = int32[8] (first_row, n_tok, slot, first_pos, key_begin, key_end, part_slot, 0): n_tok <= 64 / H consecutive rows
 *               of one request at positions first_pos.. against the cached keys [key_begin, key_end) (clipped causally per row).
 *               part_slot < 0: the item sees all its keys and writes `out`; else it writes its (max, sum, unnormalised output)
 *               partial to ws_o[part_slot][64][r] / ws_ml[part_slot][64][2] (long decode contexts cut into key ranges);
 *   merges[i] = int32[4] (first_row * H, n_rows, first part_slot, n_parts): partials that belong together.
 * The sink term is added where the denominator is completed. out [T, H, r] of out_dt (fp32 or bf16). Same results as
 * omc_latent_attn up to the bf16 rounding of the probabilities. */
int omc_latent_attn_mma(const void* qcat, int T, int H, int r, int dr, const void* pool, const int32_t* block_table, int max_pages,
                        int page_size, const int32_t* items, int n_items, const int32_t* merges, int n_merges, const float* sink,
                        float scale, void* out, int out_dt, float* ws_o, float* ws_ml, void* stream);

/* The work list of a decode-only step, written on the device from pos / slot (one row per request, `parts` <= 64 key ranges each):
 * items int32 [B * parts][8], merges int32 [B][4] (untouched when parts == 1). Lets a CUDA graph replay the step as contexts grow. */
int omc_latent_decode_items(const int32_t* pos, const int32_t* slot, int B, int H, int parts, int32_t* items, int32_t* merges,
                            void* stream);

/* Router with score correction and identity experts. z fp32 [T, ldz]: logits of E_tot = experts + identity outputs, and, when
 * has_gate, one more column: the shared expert's gate logit. s = softmax(z[:E_tot] + bias) (bias fp32 [E_tot] or NULL);
 * choice = s + correction (fp32 [E_tot] or NULL); the `top` largest choices (ties: lowest index) -> ids int32 [T, top];
 * weights = s of the chosen -> w fp32 [T, top], as they are (renorm 0) or divided by their sum (renorm 1: the softmax over the
 * chosen logits alone); gate[t] = sigmoid(z[t, E_tot]); counts[e] += 1 for every chosen e < experts (identity experts - the
 * last E_tot - experts outputs - take no rows). score OMC_ROUTER_SIGMOID: s = sigmoid(z + bias), every output on its own, instead
 * of the softmax. E_tot <= 4096, top <= 32. */
#define OMC_ROUTER_SOFTMAX 0
#define OMC_ROUTER_SIGMOID 1
int omc_router_topk(const float* z, long long ldz, int T, int E_tot, int experts, int top, const float* correction,
                    const float* bias, int renorm, int score, int has_gate, int32_t* ids, float* w, float* gate, int32_t* counts,
                    void* stream);

/* Expert-sorted layout. plan: seg_start[e] = first row of expert e's segment, segments padded to whole `tile`-row tiles;
 * tile_group[i] = expert of tile i or -1 (max_tiles entries are written); counts and cursor are left zeroed for the next call.
 * scatter: row t is copied to one row of the segment of each chosen expert; slot_of[t, j] = that row, or -1 for an identity
 * expert. xs rows [max_tiles * tile, C] of dtype dt. row_w (fp32 [T, top] or NULL): the copy of row t for its j-th choice is
 * multiplied by row_w[t, j] - mixing weights that act on the experts' INPUT. */
int omc_moe_plan_tiles(int32_t* counts, int experts, int tile, int max_tiles, int32_t* seg_start, int32_t* cursor,
                       int32_t* tile_group, void* stream);
int omc_moe_scatter_rows(const void* x, int dt, long long ldx, int T, int C, const int32_t* ids, int top, int experts,
                         const int32_t* seg_start, int32_t* cursor, int32_t* slot_of, void* xs, long long ldxs, const float* row_w,
                         void* stream);

/* omc_moe_plan_tiles + omc_moe_scatter_rows as ONE single-CTA launch, for steps of a few rows (decode). */
int omc_moe_plan_scatter_small(int32_t* counts, int experts, int tile, int max_tiles, int32_t* seg_start, int32_t* tile_group,
                               const void* x, int dt, long long ldx, int T, int C, const int32_t* ids, int top, int32_t* slot_of, void* xs,
                               long long ldxs, const float* row_w, void* stream);

/* Combine + residual + depth-weighted average of the layer results in one pass over the row:
 *   y = sum_j (w[t, j], or 1 with w NULL) * ys[slot_of[t, j]]   (slot_of < 0: skipped; ys NULL: a layer without feed-forward, y = 0)
 *   xn = x[t] + a1 * y1[t] + a2 * y2[t] + mult * y  -> streams[n_streams - 1][t]   (y1 / y2 fp32 rows or NULL: sublayer outputs
 *        that have not entered the stream yet; streams NULL: not kept)
 *   out[t] = sum_{j < n_streams} coef[j] * streams[j][t]        (coef NULL: out = xn)
 * streams[j] = streams + j * stream_stride, rows at lds: the embedding output and the result of every earlier layer, fp32.
 * coef [n_streams] of coef_dt. out may alias x. */
int omc_moe_combine_depth(const float* ys, long long ldys, const int32_t* slot_of, const float* w, int top, const float* x, long long ldx,
                          const float* y1, long long ld1, float a1, const float* y2, long long ld2, float a2, float mult, float* streams, long long stream_stride, long long lds, int n_streams, const void* coef, int coef_dt,
                          float* out, long long ldo, int T, int C, void* stream);

/* Combine + output-side norm + residual in one pass over the row:
 * y = sum_j w[t,j] * (slot_of[t,j] >= 0 ? ys[slot_of[t,j]] : h32[t]) + gate[t] * ysh[t]   (ysh / gate may be NULL)
 * h32[t] += y / sqrt(mean(y^2) + eps) * (1 + nw);  xb[t] = round(h32[t]), or with w_next != NULL the next sublayer's normed input
 * h32[t] / rms(h32[t]) * (1 + w_next) (xb NULL to skip). ys / ysh fp32; nw and w_next of nw_dt. */
int omc_moe_combine_norm(const float* ys, long long ldys, const int32_t* slot_of, const float* w, int top, const float* gate,
                         const float* ysh, long long ldysh, const void* nw, int nw_dt, float eps, float* h32, long long ldh,
                         const void* w_next, void* xb, int xb_dt, long long ldxb, int T, int C, void* stream);

/* omc_linear with a bias row: Y = act(alpha * X W^T + bias). bias [N] has the weights' dtype; batch item b reads bias + b * sbias.
 * NULL bias: omc_linear. Not with a tile table. */
int omc_linear_bias(const void* X, int x_dt, long long ldx, long long sx, const void* W, int w_dt, long long ldw, long long sw,
                    void* Y, int y_dt, long long ldy, long long sy, int M, int N, int K, int batch, float alpha, int act,
                    const int32_t* tile_group, long long group_stride, const void* bias, long long sbias, void* stream);

/* Sublayer output -> residual stream -> next sublayer's input in one pass over the row:
 *   y = y1, or with y2 != NULL the mean of two branches, each normed with a plain weight first:
 *       y = (y1 / rms(y1) * wa + y2 / rms(y2) * wb) / 2
 *   h32 += mult * y / rms(y) * (1 + w_post)
 *   xb = h32 / rms(h32) * (1 + w_next); w_next NULL: xb = round(h32); xb NULL: skipped.
 * rms(z) = sqrt(mean(z^2) + eps). y1 / y2 fp32; all weights of w_dt. */
int omc_post_norm_residual(const float* y1, long long ld1, const void* wa, const float* y2, long long ld2, const void* wb,
                           const void* w_post, int w_dt, float eps, float mult, float* h32, long long ldh, const void* w_next,
                           void* xb, int xb_dt, long long ldxb, int rows, int C, void* stream);

/* y[t, c] = act(z[t, c]) * z[t, n + c] for c < n: the two halves of a stacked gate | up projection. z of z_dt, fp32 arithmetic.
 * act OMC_ACT_CLAMP_SWISH: g = min(z[t, c], limit), u = clamp(z[t, n + c], -limit, limit), y = g * sigmoid(slope * g) * (u + shift);
 * limit, slope and shift are ignored by the other activations. */
int omc_glu_mul(const void* z, int z_dt, long long ldz, int rows, int n, int act, float limit, float slope, float shift, void* y,
                int y_dt, long long ldy, void* stream);

/* h32[t, :] = table[ids[t], :] * scale + s(pos[t]) with the sinusoidal position vector s(p)[2i] = sin(p * freq[i]),
 * s(p)[2i + 1] = cos(p * freq[i]); freq is a device table of ceil(C / 2) doubles (the angle is formed and reduced in double precision).
 * ids outside [0, vocab) contribute no embedding row. */
int omc_embed_sinusoid(const int32_t* ids, const int32_t* pos, int T, const void* table, int t_dt, int C, int vocab, float scale,
                       const double* freq, float* h32, long long ldh, void* stream);

/* Causal convolution over time per channel, then silu, then optional unit vectors. Row t is position pos[t] of the request in
 * state slot slot[t]; rows of one request are consecutive and ascending. w [ch, taps] of w_dt: the last tap multiplies the row
 * itself (taps <= 32), tap j the input taps - 1 - j positions back - an earlier row of the step, else state[slot][position % (taps - 1)][ch]
 * (fp32 ring of the last taps - 1 inputs, updated by this call), else zero before position 0. Of the outputs the first
 * unit_channels are divided, in groups of unit_group, by sqrt(sum of squares + unit_eps); the first scaled_channels of those are
 * then multiplied by unit_mult (scaled_channels a multiple of unit_group). x / y fp32 (y may not alias x). single_rows != 0: the
 * caller vouches that every row is a request of its own (a decode step); the ring is then updated by the same launch. */
int omc_causal_conv_silu(const float* x, long long ldx, int T, int ch, const void* w, int w_dt, int taps, const int32_t* pos,
                         const int32_t* slot, float* state, float* y, long long ldy, int unit_channels, int unit_group,
                         float unit_eps, int scaled_channels, float unit_mult, int single_rows, void* stream);

/* The same convolution with the activation as a parameter: act OMC_CONV_LINEAR (the weighted sum itself) or OMC_CONV_SILU; with a
 * bias per channel in front of the activation (bias [ch] of w_dt or NULL) and an output of dtype y_dt. */
#define OMC_CONV_LINEAR 0
#define OMC_CONV_SILU 1
int omc_causal_conv(const float* x, long long ldx, int T, int ch, const void* w, const void* bias, int w_dt, int taps, const int32_t* pos,
                    const int32_t* slot, float* state, void* y, int y_dt, long long ldy, int act, int unit_channels, int unit_group,
                    float unit_eps, int scaled_channels, float unit_mult, int single_rows, void* stream);

/* Tanh norm + input convolution of a sublayer. With xv = x[t] (+ a1 * y1[t] + a2 * y2[t] when given: the previous sublayer's
 * output(s) enter the stream here, and the updated row is written to x_out, which must not be x):
 *   h = tanh(alpha * xv) * nw + nb                      (alpha: one fp32 scalar in device memory)
 *   u[t] = h_t + sum_j cw[:, j] * h_(t - taps + 1 + j)   (causal over the request's positions; zeros before position 0)
 * The last taps - 1 rows h of every request live in state[slot][position % (taps - 1)][C] (fp32 ring, updated by this call).
 * nw, nb [C] and cw [C, taps] of w_dt; u of u_dt. single_rows as in omc_causal_conv_silu. */
int omc_dyt_conv(const float* x, long long ldx, const float* y1, long long ld1, float a1, const float* y2, long long ld2, float a2,
                 float* x_out, long long ldxo, const float* alpha, const void* nw, const void* nb, const void* cw, int w_dt, int taps,
                 const int32_t* pos, const int32_t* slot, float* state, void* u, int u_dt, long long ldu, int T, int C, int single_rows,
                 void* stream);

/* y[t, c] = tanh(alpha * x[t, c]) * w[c] + b[c] (the same norm alone). */
int omc_dyt_rows(const float* x, long long ldx, const float* alpha, const void* w, const void* b, int w_dt, void* y, int y_dt, long long ldy,
                 int rows, int C, void* stream);

/* x[t, c] <- cap * tanh(x[t, c] / cap) in place (fp32): a soft cap on logits. */
int omc_tanh_cap_rows(float* x, long long ldx, int rows, int cols, float cap, void* stream);

/* Selective scan. Per channel c a state S[c, :N] (fp32, state[slot][inner][N]):
 *   dt = softplus(dt_raw[t, c] + dt_bias[c]);  S <- exp(dt * A[c, :]) * S + dt * x[t, c] * B[t, :];  y = S . C[t, :] + D[c] * x[t, c]
 * (the decay is applied as S + expm1(dt * A) * S)
 * with A = -exp(A_log) (fp32 [inner, N]); the output row is y * silu(z[t, c]) (z NULL: y). x of x_dt, dt_raw / B / C / z fp32 rows
 * (column slices are fine), y of y_dt. Portions and the zero start at position 0 as in omc_linear_state_scan. N <= 256. */
int omc_selective_scan(const void* x, int x_dt, long long ldx, const float* dt, long long lddt, const float* dt_bias, const float* B,
                       long long ldb, const float* Cm, long long ldc, const float* A_log, const float* D, const float* z, long long ldz,
                       float* state, void* y, int y_dt, long long ldy, const int32_t* row_begin, int portions, const int32_t* pos,
                       const int32_t* slot, int inner, int N, void* stream);

/* omc_causal_conv (linear) + omc_qk_norm_kv_store (per group) in one launch: x fp32 [T, ch] holds the projected q | k | v rows
 * (nq + nk + the rest), w [ch, taps] the three convolutions stacked, state the ring [slots][taps - 1][ch]. The convolved queries
 * and keys get an RMS norm per `group` channels with the weights wq / wk [group] (of w_dt); q_out [T, nq] and the cache row
 * [k | v] of (slot[t], pos[t]) in pool [pages][page_size][ch - nq] are of dtype dt. single_rows as in omc_causal_conv_silu. */
int omc_conv_qk_norm_kv_store(const float* x, long long ldx, int T, int ch, const void* w, int w_dt, int taps, const int32_t* pos,
                              const int32_t* slot, float* state, int nq, int nk, int group, const void* wq, const void* wk, float eps,
                              const int32_t* block_table, int max_pages, int page_size, void* pool, void* q_out, long long ldqo, int dt,
                              int single_rows, void* stream);

/* Linear-state recurrence per head with an fp32 state S [dim, vdim] in state[slot][head]:
 *   S <- diag(g_t) S;  u_t = beta_t (v_t - S^T k_t) (beta != NULL) or v_t;  S <- S + k_t u_t^T;  o_t = S^T q_t.
 * decay_mode 0: g = decay_const[head]; 1: g = exp(-exp(A_log[head]) softplus(a[t, head] + dt_bias[head])); 2: one decay per key
 * channel, a [T, H * dim], dt_bias [H * dim]; 3: a [T, H * dim] holds the decays themselves; 4: g = sigmoid(a + dt_bias)^decay_pow per
 * key channel (dt_bias [H * dim] or NULL); 5: a holds g - 1. Modes 4 and 5 apply the decay as S + (g - 1) S, which keeps the digits
 * of a decay close to 1. The read-out is multiplied by out_scale (a query scale). beta raw [T, H], squashed by a sigmoid here. silu_in: q, k, v pass silu first.
 * q / k [T, G * dim] (head h reads group h / (H / G)), v [T, H * vdim], out fp32 [T, H * vdim]. Portion i is rows
 * row_begin[i] .. row_begin[i + 1] - 1 (device int32 [portions + 1]), all of slot[row_begin[i]]; a portion whose first row has
 * position 0 starts from S = 0. Tokens are processed one after the other in every case. dim <= 256. */
int omc_linear_state_scan(const float* q, long long ldq, const float* k, long long ldk, const float* v, long long ldv, int silu_in,
                          int decay_mode, const float* decay_const, const float* a, long long lda, const float* A_log,
                          const float* dt_bias, const float* beta, long long ldb, float* state, float* out, long long ldo,
                          const int32_t* row_begin, int portions, const int32_t* pos, const int32_t* slot, int H, int G, int dim,
                          int vdim, float decay_pow, float out_scale, void* stream);

/* y[t, g * n + c] = x[t, g * n + c] / sqrt(mean_c(x[t, g * n + :]^2) + eps) * w[c] * act(gate[t, g * n + c]) for g < groups.
 * gate fp32 or NULL; gate_act 0: as is, 1: silu, 2: sigmoid. w [n] of w_dt, y of y_dt. */
int omc_gated_rms_rows(const float* x, long long ldx, int rows, int groups, int n, const void* w, int w_dt, float eps,
                       const float* gate, long long ldg, int gate_act, void* y, int y_dt, long long ldy, void* stream);

/* Rows of a step for windowed attention: q_out[t] = q[t, :nq] / rms * wq (plain weight); the cache row of (slot[t], pos[t]) <-
 * [k[t, :nk] / rms * wk | v[t, :nv]]. q_group / k_group 0: one norm over all nq (nk) columns at once, weight [nq] ([nk]); > 0: one norm
 * per that many consecutive columns (a head, or one score map of a head) with a weight of that size shared by the groups.
 * Pool [pages][page_size][nk + nv] and q_out of dtype dt. */
int omc_qk_norm_kv_store(const float* q, long long ldq, int nq, int q_group, const void* wq, const float* k, long long ldk, int nk,
                         int k_group, const void* wk, int w_dt, const float* v, long long ldv, int nv, float eps, int T,
                         const int32_t* pos, const int32_t* slot, const int32_t* block_table, int max_pages, int page_size, void* pool,
                         void* q_out, long long ldqo, int dt, void* stream);

/* Sliding-window attention over such a pool: row t (position p of its slot) sees the keys j <= p with p - j < window or
 * j < keep_first (the first keys of the sequence stay visible; 0: none). score = (q . k) * scale; softcap > 0: score = softcap *
 * tanh(score / softcap); dist_bias != NULL (fp32 [window, H]): score += dist_bias[p - j][h] for p - j < window; softmax;
 * out = sum_j p_j v_j. Query head h reads key/value head h / (H / G). maps >= 1 score maps per head: q is [T, H, maps, d], a cache
 * row [G, maps, d keys | G, dv values], out [T, H, maps, dv] - every map is a softmax of its own over the same values.
 * sink (fp32 [H] or NULL): the softmax denominator of head h holds one more term exp(sink[h]) - no key, no value, neither scaled
 * nor capped. gate (fp32 [T, ldg] laid out like out, or NULL): out *= act(gate), gate_act 0: as is, 1: silu, 2: sigmoid.
 * q and pool of dtype dt, out of out_dt. dv <= 256. */
int omc_window_attn(const void* q, long long ldq, int T, int H, int G, int d, int dv, int maps, const void* pool, int dt,
                    const int32_t* block_table, int max_pages, int page_size, const int32_t* pos, const int32_t* slot, int window,
                    int keep_first, float scale, float softcap, const float* dist_bias, const float* sink, const float* gate,
                    long long ldg, int gate_act, void* out, int out_dt, long long ldo, void* stream);

/* Rows of a step for an attention whose positions enter the queries and keys: per head the first rot_dims dimensions of q and k
 * are rotated pairwise, (u, v) at (2i, 2i + 1) -> (u cos a - v sin a, v cos a + u sin a) with a = position * freq[i] formed in fp32
 * (freq fp32 [rot_dims / 2], NULL: no rotation); q is multiplied by 1 + temp_coef * ln(floor((position + 1) / temp_every) + 1)
 * (temp_coef 0: off); v_unit != 0: each head's values are divided by sqrt(mean(v^2) + eps). q [T, H * d] -> q_out; k [T, G * d] and
 * v [T, G * dv] -> the cache row [k | v] of (slot[t], pos[t]). q / k / v fp32, pool and q_out of dtype dt. */
int omc_pos_qkv_store(const float* q, long long ldq, int H, const float* k, long long ldk, int G, int d, const float* v, long long ldv,
                      int dv, const float* freq, int rot_dims, float temp_coef, int temp_every, int v_unit, float eps, int T,
                      const int32_t* pos, const int32_t* slot, const int32_t* block_table, int max_pages, int page_size, void* pool,
                      void* q_out, long long ldqo, int dt, void* stream);

/* Tensor-core version of omc_window_attn (bf16 q and pool; d and dv multiples of 16, d <= 256, dv <= 128, H / G a divisor of 64 -
 * omc_window_attn_mma_ok says 1). items: int32 [n_items][4] (first_row, n_tok, slot, first_pos), n_tok <= 64 / (H / G) consecutive
 * rows of one request; items NULL: every one of the T rows is an item of its own, taken from pos / slot on the device. Same
 * results as omc_window_attn up to the bf16 rounding of the probabilities and the hardware exponentials. */
int omc_window_attn_mma_ok(int H, int G, int d, int dv);
int omc_window_attn_mma(const void* q, long long ldq, int T, int H, int G, int d, int dv, int maps, const void* pool,
                        const int32_t* block_table, int max_pages, int page_size, const int32_t* items, int n_items, const int32_t* pos,
                        const int32_t* slot, int window, int keep_first, float scale, float softcap, const float* dist_bias,
                        const float* sink, const float* gate, long long ldg, int gate_act, void* out, int out_dt, long long ldo, void* stream);

/* Differential heads: a fp32 [T, H, 2, dv] (two score maps per head) -> o = a1 - lambda * a2; o / sqrt(mean(o^2) + eps) over the
 * head's dv values; times mult; times act(gate[t, h * dv + c]) (gate fp32 or NULL; gate_act 0: as is, 1: silu, 2: sigmoid)
 * -> y [T, H * dv] of y_dt. */
int omc_diff_heads_gate(const float* a, long long lda, int T, int H, int dv, float lambda, float mult, float eps, const float* gate,
                        long long ldg, int gate_act, void* y, int y_dt, long long ldy, void* stream);

/* Differential attention of prompt portions in one kernel (bf16 q and pool; shapes as omc_window_attn_mma, and both maps' tiles must
 * fit shared memory - omc_diff_attn_pair_ok says 1): omc_window_attn_mma with two maps, no soft cap and no bias, followed by
 * omc_diff_heads_gate, with the values of a key tile staged once for both maps and the maps themselves kept in registers.
 * q [T, H, 2, d], pool rows [G, 2, d | G, dv], items as omc_window_attn_mma (not NULL), gate fp32 [T, ldg] or NULL, out [T, H * dv]. */
int omc_diff_attn_pair_ok(int H, int G, int d, int dv);
int omc_diff_attn_pair(const void* q, long long ldq, int T, int H, int G, int d, int dv, const void* pool, const int32_t* block_table,
                       int max_pages, int page_size, const int32_t* items, int n_items, int window, int keep_first, float scale,
                       float lambda, float mult, float eps, const float* gate, long long ldg, int gate_act, void* out, int out_dt,
                       long long ldo, void* stream);

/* In place over x[t, :cols] (fp32): op 1: silu; op 2: x <- exp(-exp(A_log[c / group]) * softplus(x + bias[c])); op 3: x <-
 * sigmoid(x + bias[c])^p_exp - 1 (bias may be NULL; decay mode 5 of omc_linear_state_scan) - the same functions the recurrence applies while staging, as one pass for steps
 * with long portions. */
int omc_map_rows(float* x, long long ldx, int rows, int cols, int op, const float* A_log, const float* bias, int group, float p_exp,
                 void* stream);

#ifdef __cplusplus
}
#endif
#endif /* OMCHAT_B200_SEQ_H_ */
