/*
 * qspec_b200_seq.h -- C ABI of the sequence-mixer kernels (library qspec_b200/_C/libqspec_b200_seq.so).
 *
 * These kernels serve decoder designs whose weights are plain bfloat16 / float32 matrices (no int4 path): layer
 * norms with a zero-centred weight, short causal convolutions over time with a per-sequence tail, per-head
 * query/key norms, chunk-local sigmoid attention over a per-slot key/value cache, squared-ReLU and clamped-gated
 * feed-forward activations, a softmax router with top-k choice, and mixture-of-experts feed-forward layers
 * (token-per-CTA form for decoding, tensor-core grouped form for prompts). Dense matrix products between them are
 * left to the vendor library.
 *
 * Conventions (as in qspec_b200.h): device pointers, contiguous row-major, `stream` is a cudaStream_t, `int`
 * status with qspec_last_error(). `dtype` is the element type of activations and of the large weight matrices:
 * QSPEC_DTYPE_BF16 or QSPEC_DTYPE_F32. The residual stream, norm / convolution / bias vectors, router weights,
 * convolution tails and everything the kernels reduce or exponentiate are float32 in both modes.
 *
 * Token batch: a step is a flat list of `ntok` tokens; the tokens of one sequence ("segment") are contiguous and in
 * ascending position. `meta` is int32 [5][ntok]:
 *   row 0 slot       cache / state slot of the token's sequence
 *   row 1 pos        position of the token in its sequence (from 0)
 *   row 2 seg_begin  batch index of the first token of its segment
 *   row 3 seg_end    batch index one past the last token of its segment
 *   row 4 phase      which of the two convolution-tail buffers holds the state BEFORE this step (0 / 1)
 */
#ifndef QSPEC_B200_SEQ_H_
#define QSPEC_B200_SEQ_H_

#include "qspec_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define QSPEC_DTYPE_F32   2
#define QSPEC_SEQ_META_ROWS 5

/* x[i, :] = float(table[ids[i], :]).  table [V, W] dtype; ids int32 [ntok]; x float32 [ntok, W]. */
int qspec_seq_embed(const void* table, const int* ids, float* x, int ntok, int W, int V, int dtype, void* stream);

/* Sublayer entry: close the previous sublayer and open the next one in one launch.
 *   r_t   = x_in[t] + unit_rms(y_t) * (1 + post_w)        (y_t = sum of `y_parts` rows; skipped when y == NULL)
 *   h_t   = unit_rms(r_t) * (1 + pre_w)
 *   out_t = h_t + sum_j conv_w[:, j] * h_(t - taps + 1 + j)  (rows before the segment come from the tail; before
 *                                                             position 0 they are zero; conv_w == NULL: out = h)
 * unit_rms(v) = v / sqrt(mean(v^2) + eps), all in float32. x_out receives r (must not alias x_in when y != NULL);
 * out == NULL stops after r. tail: float32 [2][slots][taps-1][W]; the step reads buffer `phase` and writes buffer
 * `1 - phase` with the last taps-1 rows of h of every segment (older rows are carried over).
 * y row p of token t is y + t * y_tok_stride + p * y_part_stride (elements); part weights y_w (float32
 * [ntok, y_parts], NULL = ones) multiply each part before the sum. W <= 16384, taps <= 8.
 * scratch (float32 [ntok, W], may be NULL): with it, batches of 256 tokens or more that have a convolution run as two
 * launches over independent rows (both norms of a row; then the convolution over the normalised rows), same results. */
int qspec_seq_norm_conv(const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride,
                        long long y_tok_stride, const float* y_w, const float* post_w, const float* pre_w,
                        const float* conv_w, int taps, float* tail, int slots, void* out, const int* meta, int ntok,
                        int W, float eps, float* scratch, int dtype, void* stream);

/* In-place per-head norm of the query and key sections of a fused projection buffer:
 * row t = [q (H x D) | k (G x D) | v ...] with leading dimension ld; head <- unit_rms(head) * w. */
int qspec_seq_qk_norm(void* qkv, int ld, const float* q_w, const float* k_w, int ntok, int H, int G, int D, float eps,
                      int dtype, void* stream);

/* Chunk-local sigmoid attention. Query at position i sees keys j <= i with floor(j / size) == floor(i / size);
 * weight = sigmoid(cap(score) + bias[h]), cap(s) = softcap * tanh(s / softcap) (softcap <= 0: none),
 * score = scale * q.k; weights are not normalised. Keys at positions inside the token's segment are read from the
 * projection buffer (already normalised), earlier ones from the cache: cache_k [slots, size, G, D],
 * cache_v [slots, size, G, DV], row = position % size. out [ntok, H*DV].
 * max_keys: an upper bound of the keys that any token of the batch sees (its position + 1), 0 if unknown. With few
 * tokens and many keys each, the key blocks of a token are spread over a thread-block cluster whose CTAs add their
 * partial sums through distributed shared memory in a fixed order. */
int qspec_seq_chunk_attention(const void* qkv, int ld, const void* cache_k, const void* cache_v, const float* bias,
                              void* out, const int* meta, int ntok, int H, int G, int D, int DV, int size, float scale,
                              float softcap, int max_keys, int dtype, void* stream);

/* Appends the step's keys / values to the cache: only the tokens in the chunk of their segment's LAST token are
 * written (earlier chunks can never be seen again). Runs after qspec_seq_chunk_attention of the same step. */
int qspec_seq_cache_append(const void* qkv, int ld, void* cache_k, void* cache_v, const int* meta, int ntok, int H,
                           int G, int D, int DV, int size, int dtype, void* stream);

/* Prompt form of the same attention on the tensor cores (bfloat16 only): one CTA per (64-query tile, kv head). */
int qspec_seq_chunk_attention_mma(const void* qkv, int ld, const void* cache_k, const void* cache_v, const float* bias,
                                  void* out, const int* meta, int ntok, int H, int G, int D, int DV, int size,
                                  float scale, float softcap, void* stream);
int qspec_seq_chunk_attention_mma_supported(int H, int G, int D, int DV);

/* a <- relu(a)^2, n elements. */
int qspec_seq_relu2(void* a, long long n, int dtype, void* stream);

/* Router: z = router_w h (float32), s = softmax(z) over all R outputs, choice = s + correction, the `top` largest
 * choices (lowest index among equals) -> idx int32 [ntok, top], weight float32 [ntok, top] = s of the chosen.
 * router_w float32 [R, W], correction float32 [R]. R <= 1024, top <= 32. */
int qspec_moe_route(const void* h, const float* router_w, const float* correction, int* idx, float* weight, int ntok,
                    int W, int R, int top, int dtype, void* stream);

/* Expert feed-forward, one CTA per (token, choice): y = min(g, limit) * sigmoid(1.702 min(g, limit)) *
 * (clamp(u, +-limit) + 1) with [g ; u] = gate_up[e] h, out = down[e] y. Choices e >= E are identity experts (out = h).
 * gate_up [E, 2*F, W] (gate rows first), down [E, W, F]; out [ntok, top, W] (unweighted). */
int qspec_moe_expert_tokens(const void* h, const void* gate_up, const void* down, const int* idx, void* out, int ntok,
                            int W, int F, int E, int top, float limit, int dtype, void* stream);

/* Grouped form for many tokens (bfloat16): the (token, choice) pairs are sorted by expert and every expert's rows go
 * through 128 x 128 tcgen05 tiles with the accumulator in tensor memory. Workspace: bytes from the query, zero-filled
 * once by the caller; its layout is internal except for the first int32, a status word that a CTA sets to 1 when a
 * bounded wait of its pipeline runs out (that CTA stores nothing); no call clears it. */
size_t qspec_moe_grouped_workspace_bytes(int ntok, int top, int E, int F);
int qspec_moe_expert_grouped(const void* h, const void* gate_up, const void* down, const int* idx, void* out, int ntok,
                             int W, int F, int E, int top, float limit, void* workspace, size_t workspace_bytes,
                             void* stream);
int qspec_moe_expert_grouped_supported(int W, int F);

/* Router that softmaxes over the chosen outputs only: z = router_w h (float32), the `top` largest z (lowest index among
 * equals) -> idx, weight = softmax over those `top` logits. */
int qspec_moe_route_chosen(const void* h, const float* router_w, int* idx, float* weight, int ntok, int W, int R, int top,
                           int dtype, void* stream);

/* Expert activations of the two expert kernels below. GATED: [gate ; up] rows, the clamped gated form described at
 * qspec_moe_expert_tokens. RELU2: up rows only (weights [E, F, W]), y = max(up h, 0)^2; `limit` is ignored. */
#define QSPEC_EXPERT_ACT_GATED 0
#define QSPEC_EXPERT_ACT_RELU2 1
#define QSPEC_EXPERT_ACT_SILU  2   /* [gate ; up] rows like GATED, y = silu(gate h) * (up h); `limit` is ignored */
int qspec_moe_expert_tokens_act(const void* h, const void* up, const void* down, const int* idx, void* out, int ntok, int W,
                                int F, int E, int top, float limit, int act, int dtype, void* stream);
int qspec_moe_expert_grouped_act(const void* h, const void* up, const void* down, const int* idx, void* out, int ntok, int W,
                                 int F, int E, int top, float limit, int act, void* workspace, size_t workspace_bytes,
                                 void* stream);

/* ---- mixers whose state outlives a chunk: token shift, windowed softmax attention with a sink (latent or grouped-query
 * keys), gated linear recurrence. Ring caches: row = position % cap; the step's own rows are written before they are read,
 * so cap >= window - 1 + (tokens of one sequence in a step). ---- */

/* out_t = x_t + (x_(t-1) - x_t) * shift. The row before a segment's first token is prev[phase][slot] (zero at position
 * 0); the segment's last row goes to prev[1 - phase][slot]. prev: float32 [2][slots][W]. */
int qspec_seq_token_shift(const float* x, const float* shift, float* prev, int slots, void* out, const int* meta, int ntok,
                          int W, int dtype, void* stream);

/* r = x_in + norm(v), v = sum_p y_w[t, p] * y[t, p, :] (y_w NULL: ones). kind 0: layer norm (v - mean) / sqrt(var + eps)
 * * w + b with var the mean of the squared deviations; kind 1: v / sqrt(mean(v^2) + eps) * w (+ b if given).
 * x_in NULL: r = norm(v). r goes to x_out (float32, may alias x_in, may be NULL) and, cast, to out (may be NULL).
 * y has element type y_dtype: the activation type or float32. */
int qspec_seq_add_norm(const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride,
                       long long y_tok_stride, const float* y_w, const float* w, const float* b, int kind, void* out, int ntok,
                       int W, float eps, int y_dtype, int dtype, void* stream);

/* Latent attention, after the down projections. Row t of d (leading dimension ld): [query latent (q_rank) | key/value
 * latent (kv_rank) | shared rotary key part (rot_dim)]. cq[t] = unit_rms(query latent) * qn_w. With a cache (the layer
 * owns one; otherwise cache == NULL and the row holds the query latent only): cache[slot, pos % cap] =
 * [unit_rms(key/value latent) * kvn_w | rotate(rotary key part)], row length kv_rank + rot_dim. The rotation turns the
 * pair (i, i + rot_dims/2) of the first rot_dims entries by the angle pos * inv_freq[i] (float32). */
int qspec_seq_latent_prep(const void* d, int ld, int q_rank, int kv_rank, int rot_dim, const float* qn_w, const float* kvn_w,
                          const float* inv_freq, int rot_dims, void* cq, void* cache, int cap, const int* meta, int ntok,
                          float eps, int dtype, void* stream);

/* dst[t, h, 0:n] (float32) = rotate(src[t, h, off : off + n]): strides in elements; the first rot_dims entries rotated as
 * above, the rest copied. */
int qspec_seq_rotary(const void* src, long long src_tok_stride, int src_head_stride, int off, float* dst,
                     long long dst_tok_stride, int dst_head_stride, int H, int n, int rot_dims, const float* inv_freq,
                     const int* meta, int ntok, int dtype, void* stream);

/* Grouped-query attention, after the fused projection (biases added): row t of p = [q (HD) | k (GD) | v (GDV) | ...].
 * qout[t] (float32) = unit_rms(q over all HD entries) * qn_w; cache_k[slot, pos % cap] = unit_rms(k over all GD entries)
 * * kn_w; cache_v[slot, pos % cap] = v. */
int qspec_seq_qkv_prep(const void* p, int ld, int HD, int GD, int GDV, const float* qn_w, const float* kn_w, float* qout,
                       void* cache_k, void* cache_v, int cap, const int* meta, int ntok, float eps, int dtype, void* stream);

/* Sliding-window softmax attention with a sink. Token at position i sees keys j with 0 <= i - j < window; the weights are
 * exp(score_j) / (sum_j exp(score_j) + exp(sink[h])), score = scale * (qa . key[0:DA] + qb . key[DA:DA+DB]). Queries are
 * float32 with free token / head strides (elements). Key of (slot, position j, key/value head g) lies at
 * k + slot * k_slot_stride + (j % cap) * k_row_stride + g * k_head_stride, values likewise (a latent cache passes the
 * same buffer twice with G = 1). Query head h uses key/value head h / (H / G). gate (may be NULL): the output is
 * multiplied by sigmoid(gate[t, h * DV + d]). out [ntok, H, DV]. sink may be NULL (no sink). DV <= 1024. */
typedef struct qspec_window_attn_args {
  const float* qa; long long qa_tok_stride, qa_head_stride; int DA;
  const float* qb; long long qb_tok_stride, qb_head_stride; int DB;
  const void* k; long long k_slot_stride; int k_row_stride, k_head_stride;
  const void* v; long long v_slot_stride; int v_row_stride, v_head_stride; int DV;
  const float* sink; const void* gate; int gate_ld;
  void* out; const int* meta; int ntok, H, G, window, cap; float scale;
  int gate_per_head;   /* 0: gate[t, h * DV + d] as above; 1: one gate per head, gate[t, h] (gate_ld >= H) */
} qspec_window_attn_args;
int qspec_seq_window_attention(const qspec_window_attn_args* args, int dtype, void* stream);

/* The same attention on the tensor cores (bfloat16; key parts 64 or 128 (+ a shared part of 64 with a per-head part of
 * 128), value size 64 or 128; rows and strides on 16-byte boundaries). args->qa is the whole query [DA] (args->DB = 0); the
 * last DB entries of a key come from k_shared (one row per slot and ring row, shared by all heads: the rotary part of a
 * latent cache), the first DA - DB from args->k. token_rows = 0: one CTA per (token, key/value head), the rows of the
 * products are the query heads of the group (H / G <= 16) -- decode-shaped batches; 1: one CTA per (16 consecutive batch
 * tokens, head) -- prompts. */
int qspec_seq_window_attention_mma(const qspec_window_attn_args* args, const void* k_shared, long long k_shared_slot_stride,
                                   int k_shared_row_stride, int DB, int token_rows, void* stream);
int qspec_seq_window_attention_mma_supported(int DA, int DB, int DV, int H, int G, int token_rows);

/* HGRN2 recurrence. Row t of p = [zq (H x D) | zf (H x D) | v (H x DV)]. q = silu(zq), f = lower + (1 - lower) *
 * sigmoid(zf + f_b); per head S <- diag(f) S + (1 - f) v^T, o = S^T q; out[t, h] = unit_rms(o over DV) * norm_w.
 * state: float32 [slots, H, D, DV], read at a segment's start (zero at position 0), written at its end.
 * scratch: float32 with room for ntok * H * (DV + 3 D) values (un-normalised outputs and the gates). D <= 256. seg_starts (may be NULL): int32 [nseg], the batch row of every segment's
 * first token; with it the grid has one CTA per segment instead of one per token. */
int qspec_seq_hgrn2(const void* p, int ld, const float* f_b, const float* lower, const float* norm_w, float* state,
                    float* scratch, void* out, const int* meta, const int* seg_starts, int nseg, int ntok, int H, int D, int DV,
                    float eps, int dtype, void* stream);

/* g[t, :] <- gelu_tanh(g[t, :]) * table[ids[t], col0 : col0 + sd]  (g [ntok, sd], table [V, table_ld]). */
int qspec_seq_side_gate(void* g, const void* table, const int* ids, int col0, int sd, int table_ld, int V, int ntok, int dtype,
                        void* stream);

/* ---- pre-norm designs with a scaled residual, full-length latent caches, scalar-decay linear attention, sigmoid routers with
 * expert groups. ---- */

/* Residual sum and the next sublayer's input norm in one launch:
 *   r = x_in + mult * (sum_p y_w[t, p] * y[t, p, :] + y2_w[t * y2_w_stride] * y2[t, :])      (y NULL: r = x_in; y2 NULL: no such term)
 *   out = r / sqrt(mean(r^2) + eps) * (w_offset + w)
 * y_w NULL: ones; y2_w NULL: one. r goes to x_out (float32, may alias x_in, may be NULL), the norm to out (activation type,
 * may be NULL). y and y2 have element type y_dtype: the activation type or float32. W <= 49152. */
int qspec_seq_residual_norm(const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride,
                            long long y_tok_stride, const float* y_w, const void* y2, const float* y2_w, int y2_w_stride,
                            float mult, const float* w, float w_offset, void* out, int ntok, int W, float eps, int y_dtype, int dtype,
                            void* stream);

/* Rotary pairings: HALVES turns entry i with entry i + rot_dims / 2; INTERLEAVED turns entry 2i with entry 2i + 1. In both the
 * angle of pair i is pos * inv_freq[i]. */
#define QSPEC_ROTARY_HALVES 0
#define QSPEC_ROTARY_INTERLEAVED 1
/* qspec_seq_latent_prep with the pairing as an argument; q_rank may be 0 (no query latent: qn_w and cq are not read). */
int qspec_seq_latent_prep_pairing(const void* d, int ld, int q_rank, int kv_rank, int rot_dim, const float* qn_w, const float* kvn_w,
                                  const float* inv_freq, int rot_dims, int pairing, void* cq, void* cache, int cap, const int* meta,
                                  int ntok, float eps, int dtype, void* stream);
/* qspec_seq_rotary with the pairing as an argument. */
int qspec_seq_rotary_pairing(const void* src, long long src_tok_stride, int src_head_stride, int off, float* dst,
                             long long dst_tok_stride, int dst_head_stride, int H, int n, int rot_dims, int pairing,
                             const float* inv_freq, const int* meta, int ntok, int dtype, void* stream);

/* a <- act(a), n elements. */
#define QSPEC_ACT_RELU2 0
#define QSPEC_ACT_GELU_ERF 1
int qspec_seq_act(void* a, long long n, int act, int dtype, void* stream);
/* out[t, f] = silu(gu[t, f]) * gu[t, F + f]: rows of gu are [gate (F) | up (F)] with leading dimension ld; out [ntok, F]. */
int qspec_seq_silu_mul(const void* gu, int ld, void* out, int ntok, int F, int dtype, void* stream);

/* Linear attention with one decay per head ("lightning"). Row t of p = [zq (H x D) | zk (H x D) | zv (H x DV) | zg (H x DV)].
 * q = silu(zq), k = silu(zk), v = silu(zv); per head S <- decay[h] * S + k v^T, o = S^T q; the concatenated heads are
 * normed together: out[t, :] = o / sqrt(mean over all H * DV of o^2 + eps) * norm_w * sigmoid(zg). state: float32
 * [slots, H, D, DV], read at a segment's start (zero at position 0), written at its end. scratch: float32 with room for
 * ntok * H * (DV + 2 D) values. seg_starts as for qspec_seq_hgrn2. D <= 256. */
int qspec_seq_lightning(const void* p, int ld, const float* decay, const float* norm_w, float* state, float* scratch, void* out,
                        const int* meta, const int* seg_starts, int nseg, int ntok, int H, int D, int DV, float eps, int dtype,
                        void* stream);

/* Router with a score function, expert groups and gate rows. z = router_w h (float32; router_w [R + n_extra, W]).
 * Scores s = softmax(z[0:R]) (score_fn 0) or sigmoid(z[0:R]) (score_fn 1); choice = s + correction (NULL: zeros). The R
 * experts form n_groups equal groups of neighbours; a group's score is the sum of its group_top largest choice scores; only
 * experts of the keep_groups best groups can be chosen (n_groups <= 1: no limit). The `top` largest remaining choices (lowest
 * index among equals) -> idx, weight = scale * s of the chosen. extra[t, x] = sigmoid(z[R + x]) for the n_extra gate rows
 * (extra float32 [ntok, extra_ld]). R + n_extra <= 1024, top <= 32. */
int qspec_moe_route_grouped(const void* h, const float* router_w, const float* correction, int* idx, float* weight, float* extra,
                            int extra_ld, int ntok, int W, int R, int top, int score_fn, int n_groups, int keep_groups,
                            int group_top, float scale, int n_extra, int dtype, void* stream);

/* Softmax attention of ONE prompt portion on the tensor cores, tile form (bfloat16): the ntok tokens are consecutive positions
 * pos0 .. pos0 + ntok - 1 of the sequence in slot `slot` (args->meta is not read). A CTA takes 64 tokens and one head and reads
 * every visible key / value row once, through shared memory. Arguments as for qspec_seq_window_attention_mma (window, sink,
 * gate, two-part keys); shapes: per-head key part 128 with a shared part of 64 or none and values of 128, or 64 / 64. */
int qspec_seq_prompt_attention_mma(const qspec_window_attn_args* args, const void* k_shared, long long k_shared_slot_stride,
                                   int k_shared_row_stride, int DB, int slot, int pos0, void* stream);
int qspec_seq_prompt_attention_mma_supported(int DA, int DB, int DV);

/* ---- mixers whose state is a matrix that every token rewrites, attention with mixed heads, layer scale ---- */

/* qspec_seq_residual_norm with one factor per column on the sublayer's result (a layer scale; NULL: ones):
 *   r = x_in + mult * y_scale * (sum of the weighted parts of y + y2_w * y2). */
int qspec_seq_residual_norm_scaled(const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride,
                                   long long y_tok_stride, const float* y_w, const void* y2, const float* y2_w, int y2_w_stride,
                                   float mult, const float* y_scale, const float* w, float w_offset, void* out, int ntok, int W,
                                   float eps, int y_dtype, int dtype, void* stream);

/* Short causal convolution over time with an activation: out[t, c] = act(bias[c] + sum_j w[c, j] * in[t - taps + 1 + j, c]),
 * in [ntok, ld] (the first C columns), w float32 [C, taps] (the last column meets the current token), bias float32 [C] or NULL.
 * Rows before a segment's first token come from tail: float32 [2][slots][taps - 1][C]; the step reads buffer `phase` and writes
 * buffer `1 - phase` with the sequence's last taps - 1 inputs. Rows before position 0 are zero. out [ntok, out_ld] is float32
 * if out_f32, else of the activation type. taps <= 64. */
#define QSPEC_CONV_ACT_NONE 0
#define QSPEC_CONV_ACT_SILU 1
int qspec_seq_conv_act(const void* in, int ld, const float* w, const float* bias, int C, int taps, int act, float* tail, int slots,
                       void* out, int out_ld, int out_f32, const int* meta, int ntok, int dtype, void* stream);

/* Gated delta rule. Row t of cs (float32, leading dimension ld, changed in place): [q (G x D) | k (G x D) | v (H x DV)], after
 * convolution and activation. q <- q / sqrt(sum q^2 + unit_eps) * q_mult, k <- k / sqrt(sum k^2 + unit_eps). ba float32
 * [ntok, 2 H] = [b | a]: beta = sigmoid(b), g = exp(-exp(A_log[h]) * softplus(a + dt_bias[h])). Per head h with the query / key
 * head h / (H / G) and S float32 [D, DV]:   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
 * out[t, h] = o / sqrt(mean(o^2) + eps) * norm_w * silu(gate[t, h * DV + c]) (gate of the activation type, leading dimension
 * gate_ld; NULL: no gate). state: float32 [slots, H, D, DV], read at a segment's start (zero at position 0), written at its
 * end. Scratch: gates float32 [ntok, 2 H + G], o float32 [ntok, H, DV]. seg_starts int32 [nseg]: the batch row of every
 * segment's first token. D <= 256. */
int qspec_seq_delta_rule(float* cs, int ld, const float* ba, const float* A_log, const float* dt_bias, const float* norm_w,
                         const void* gate, int gate_ld, float* state, float* gates, float* o, void* out, const int* meta,
                         const int* seg_starts, int nseg, int ntok, int H, int G, int D, int DV, float unit_eps, float q_mult, float eps,
                         int dtype, void* stream);

/* Selective scan. Per channel c and state n, with dt = softplus(dt_pre[t, c] + dt_bias[c]) and A = -exp(A_log[c, n]):
 *   S[c, n] <- exp(dt A) S[c, n] + dt x[t, c] B[t, n];   y = sum_n S[c, n] C[t, n] + D_skip[c] x[t, c];   out = y * silu(z[t, c]).
 * x, z, out and bc (row [B (N) | C (N)]) are of the activation type with their leading dimensions; dt_pre float32. state: float32
 * [slots, inner, N], read at a segment's start (zero at position 0), written at its end. N <= 512. */
int qspec_seq_selective_scan(const void* x, int x_ld, const float* dt_pre, int dt_ld, const float* dt_bias, const void* bc, int bc_ld,
                             const void* z, int z_ld, const float* A_log, const float* D_skip, float* state, void* out, int out_ld,
                             const int* meta, const int* seg_starts, int nseg, int ntok, int inner, int N, int dtype, void* stream);

/* Grouped-query attention, after the fused projection (biases added): row t of p = [q (H x D) | k (G x D) | v (G x DV)]. Per
 * head: q, k <- unit_rms over D * weight (qn_w / kn_w, D entries, the same for every head), then the first rot_dims entries are
 * rotated, entry i with entry i + rot_dims / 2 by the angle pos * inv_freq[i] (float32). v <- unit_rms over DV if v_norm. With
 * v_first_in (float32 [ntok, G, DV]): v <- (1 - mix[0]) v + mix[0] v_first_in; otherwise v_first_out, if given, receives v.
 * qout float32 [ntok, H, D]; cache_k [slots, cap, G, D] and cache_v [slots, cap, G, DV] take row pos % cap. */
int qspec_seq_gqa_prep(const void* p, int ld, const float* qn_w, const float* kn_w, const float* inv_freq, int rot_dims,
                       const float* v_first_in, float* v_first_out, const float* mix, float* qout, void* cache_k, void* cache_v, int cap,
                       const int* meta, int ntok, int H, int G, int D, int DV, float eps, int v_norm, int dtype, void* stream);

/* Softmax attention whose heads' weights are mixed after the softmax. Token at position i sees keys j with 0 <= i - j < window.
 * weight_g(j) = exp(s_g(j)) / (exp(sink[g]) + sum_j exp(s_g(j))), s = scale * q_g . key of g's key/value head (sink NULL: no such
 * term); head h applies sum_g talk[h, g] weight_g(j) to the values of its own key/value head h / (H / G). q float32 [ntok, H, D];
 * keys and values as rows of per-slot rings with element strides, as for qspec_seq_window_attention; talk float32 [H, H];
 * out [ntok, H, DV]. rows_per_cta: 4 lets a CTA take four consecutive batch rows, which share every key and value row they
 * read when they belong to one sequence (prompt portions); 1 gives every row a cluster of CTAs of its own (decode-shaped
 * batches). With four rows per CTA, bfloat16 caches, head sizes that are multiples of 16 and at most eight heads per key/value
 * head, the score and value products run on the tensor cores (queries rounded to bfloat16, weights as a two-term split). */
typedef struct qspec_talking_attn_args {
  const float* q;
  const void* k; long long k_slot_stride; int k_row_stride, k_head_stride;
  const void* v; long long v_slot_stride; int v_row_stride, v_head_stride;
  const float* talk; const float* sink;
  void* out; const int* meta; int ntok, H, G, D, DV, window, cap; float scale;
} qspec_talking_attn_args;
int qspec_seq_talking_attention(const qspec_talking_attn_args* args, int rows_per_cta, int dtype, void* stream);

/* out[t, f] = g * sigmoid(alpha g) * (u + 1), g = min(gu[t, f], limit), u = clamp(gu[t, F + f], -limit, limit): rows of gu are
 * [gate (F) | up (F)] with leading dimension ld; out [ntok, F]. */
int qspec_seq_glu_clamp(const void* gu, int ld, void* out, int ntok, int F, float limit, float alpha, int dtype, void* stream);

/* a <- s * a, n float32 values. */
int qspec_seq_scale_f32(float* a, long long n, float s, void* stream);

/* Arg max per row of float32 / bfloat16 logits [rows, V] (lowest index among equal maxima): int64 out. */
int qspec_seq_argmax_rows(const void* logits, int rows, int V, long long row_stride, long long* out_idx, int dtype,
                          void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* QSPEC_B200_SEQ_H_ */
