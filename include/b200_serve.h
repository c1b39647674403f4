/*
 * b200_serve.h — C ABI of the model-family layer of the library: a registry that picks the model class from a
 * checkpoint folder's config.json, a step function over a batch of (sequence slot, next tokens) entries with a paged
 * cache behind it, a continuous-batching scheduler with greedy sampling on top, and the kernels that the families
 * beyond LLaMA bring (layer norm pairs, grouped GEMM, latent attention with a softmax sink, mixture-of-experts
 * routing). b200_engine.h stays the LLaMA hot path; b200_model_open wraps it for checkpoints of that family.
 *
 * Families: "Nekodra" (config.json + model.safetensors: parallel layers of latent attention without positions and a
 * routed feed-forward with identity experts), "Musilorn" (sandwich-normed layers of convolved, capped attention with a
 * sink or of retention with a carried state, a span of layers run several times), "Tomalix" (pre-norm layers of
 * differential attention, of chunk-masked gated attention beside a selective scan, or of plain attention with ramped
 * frequency interpolation; dense or routed squared-relu feed-forwards; a repeated span of layers), "Sakevik" (norms on the
 * sublayers' outputs; a hashed pair embedding; layers of an element-wise gated recurrence, of windowed attention with sigmoid
 * weights, rotated values and head gates, or of windowed latent attention with a shared rotary key part; clamped gated
 * feed-forwards), "llama" (the reference's weight directory, llama_weights.cc:41-53, with
 * a config.json naming the b200_model_config fields).
 */
#ifndef B200_SERVE_H
#define B200_SERVE_H

#include <stddef.h>
#include <stdint.h>

#include "b200_llama.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------------------------------------
 * kernels
 * --------------------------------------------------------------------------------------------- */

/* out[t,:] = table[ids[t],:] + pos_table[pos[t],:] as fp32 (the residual stream is fp32); tables of `dtype`.
 * pos_table (and pos) may be NULL: a model without learned positions. */
int b200_embed_positions(const int* ids, const int* pos, const void* table, const void* pos_table, float* out,
                         int n_tokens, int width, int dtype, void* stream);

/* Layer norm with weight and bias, up to two (w, b) pairs applied to the SAME rows of x (mean and variance are
 * computed once, two-pass, in fp32): out_k[i,:] = (x[r_i,:] - mean) / sqrt(var + eps) * w_k + b_k, r_i = rows ? rows[i]
 * : i. x fp32 [*, width]; w, b fp32; out1 / out2 of out_dtype (out2, w2, b2 may be NULL). */
int b200_layernorm_pair(const float* x, const int* rows, int n_rows, int width, float eps, const float* w1,
                        const float* b1, void* out1, const float* w2, const float* b2, void* out2, int out_dtype,
                        void* stream);

/* epilogues of b200_gemm_grouped */
#define B200_GG_NONE 0
#define B200_GG_SIGMOID_MUL 1 /* C = acc * sigmoid(aux[row, col])                                   */
#define B200_GG_GLU 2         /* C = silu(A W[0:N]^T) * (A W[N:2N]^T); W has 2N rows; trans_b only  */
#define B200_GG_GLU_GELU 3    /* the same with gelu in its tanh form as the activation              */
#define B200_GG_RELU2 4       /* C = max(acc, 0)^2                                                   */
#define B200_GG_BIAS_SOFTPLUS 5 /* C = log(1 + exp(acc + aux[row, col])); ld_aux 0: a bias per column */
#define B200_GG_GLU_CLAMP 6   /* GLU layout; g = min(gate, L), u = clamp(up, -L, L), C = g * sigmoid(1.702 g) * (u + 1), L = epi_param */

typedef struct b200_gemm_grouped_args {
    const void* A; const void* W; void* C;
    const float* aux;          /* SIGMOID_MUL, BIAS_SOFTPLUS: fp32 [rows, ld_aux] (+ batch * stride_aux)        */
    const int* a_rows;         /* device: source row of A for each logical row (NULL = identity)               */
    const int* group_off;      /* device [batch + 1]: group g owns logical rows [off[g], off[g+1]) (NULL = none) */
    long long lda, ldw, ldc, ld_aux;                       /* leading dimensions in elements                   */
    long long stride_a, stride_w, stride_c, stride_aux;    /* per batch (stride_w also per group), in elements */
    int M;                     /* rows (groups: an upper bound of the rows of one group)                        */
    int N, K;
    int batch;                 /* batches or groups (grid z)                                                     */
    int trans_b;               /* 1: W is [N, K] (ldw >= K); 0: W is [K, N] (ldw >= N)                           */
    int epi;
    int a_dtype, w_dtype, c_dtype;   /* B200_F32 / B200_BF16                                                   */
    float epi_param;           /* B200_GG_GLU_CLAMP: the limit                                                   */
} b200_gemm_grouped_args;
int b200_gemm_grouped(const b200_gemm_grouped_args* args, void* stream);

/* y[n_tokens, N] = x[n_tokens, K] W[N, K]^T for contiguous operands (epi B200_GG_NONE, or B200_GG_RELU2 on every
 * output), or the GLU form with W [2N, K] (B200_GG_GLU, B200_GG_GLU_GELU). bfloat16 operands run on the tcgen05 / TMEM GEMM of the LLaMA path (weights streamed once through the
 * M axis up to 256 token rows, tokens on the M axis above; fp32 accumulation; out_dtype B200_BF16 or B200_F32) when the
 * shape allows (K % 8 == 0, 16-byte aligned pointers, GLU: N % 128 == 0); everything else, and B200_F32 operands, goes
 * to b200_gemm_grouped. workspace: split-K partials of the weight-streaming mode (may be NULL: single split). */
size_t b200_linear_ex_workspace_bytes(int n_tokens, int N, int K);
int b200_linear_ex(const void* x, const void* W, void* y, int n_tokens, int N, int K, int in_dtype, int out_dtype, int epi,
                   void* workspace, size_t workspace_bytes, void* stream);
/* the same with the parameter of the epilogue (B200_GG_GLU_CLAMP: its limit) */
int b200_linear_ex2(const void* x, const void* W, void* y, int n_tokens, int N, int K, int in_dtype, int out_dtype, int epi,
                    float epi_param, void* workspace, size_t workspace_bytes, void* stream);

/* Latent cache rows: for token t, row = raw[t, 0:rank] (fp32, leading dimension ld_raw) divided by its root mean
 * square (eps inside the root) times w, stored as `dtype` at position pos[t] of sequence slot[t]:
 * pool[(pages[slot[t] * max_pages + pos[t] / page_rows] * page_rows + pos[t] % page_rows) * rank + :]. */
int b200_latent_store(const float* raw, long long ld_raw, const float* w, float eps, void* pool, const int* pages,
                      int max_pages, int page_rows, const int* slot, const int* pos, int n_tokens, int rank, int dtype,
                      void* stream);

/* Attention over cached latent rows in absorbed form, with a softmax sink. For token t (sequence slot[t], position
 * pos[t]) and head h: s_j = scale * <qa[t,h,:], c_j> over the sequence's rows j <= pos[t]; p_j = exp(s_j - m) /
 * (sum_j exp(s_j - m) + exp(sink[h] - m)); out[t,h,:] = sum_j p_j c_j. qa, out fp32 [n_tokens, heads, rank] (qa is the
 * query already multiplied by the key up-projection; the caller applies the value up-projection to out). The sink
 * has no row and no value. Rows come from the page pool as in b200_latent_store.
 * Hints (0 / NULL = unknown): longest_entry = most consecutive tokens of one sequence in the batch (1: a decode batch,
 * one token per CTA); longest_context = most rows any token sees; with a workspace the bfloat16 kernel then splits long
 * contexts of small batches over several CTAs and merges the shares (and the sink) in a second launch. */
size_t b200_latent_attention_workspace_bytes(int n_tokens, int heads, int rank);
int b200_latent_attention(const float* qa, float* out, const void* pool, const int* pages, int max_pages, int page_rows,
                          const int* slot, const int* pos, const float* sink, float scale, int n_tokens, int heads,
                          int rank, int dtype, int longest_entry, int longest_context, void* workspace,
                          size_t workspace_bytes, void* stream);

/* The same attention with the options of designs that rotate one key part shared by all heads and look through a sliding
 * window: pool rows are [rank + extra] wide (b200_latent_store_rot: the normed latent, then `extra` rotated key
 * dimensions); qa and out are [n_tokens, heads, rank + extra] (qa: the absorbed query, then the head's rotated query part;
 * of out the caller uses the first `rank` columns of every head). window > 0: position p sees the rows j with
 * 0 <= p - j < window. sink may be NULL: plain softmax. */
typedef struct b200_latent_attention_args {
    const float* qa; float* out; const void* pool;
    const int* pages; int max_pages, page_rows;
    const int* slot; const int* pos;
    const float* sink; float scale;
    int n_tokens, heads, rank;       /* rank: the whole row width (latent + extra)                               */
    int window;
    int dtype, longest_entry, longest_context;
    void* workspace; size_t workspace_bytes;
    int out_cols;                    /* > 0: only out[t, h, 0:out_cols] is formed (the latent part of the rows); 0: all   */
} b200_latent_attention_args;
int b200_latent_attention_ex(const b200_latent_attention_args* a, void* stream);
/* Latent cache rows with a rotated part: row = [norm(raw[t, 0:rank]) * w | rot(raw[t, rank:rank+extra])], the rotation by
 * the token's cos / sin row ([n_tokens, extra/2], b200_rope_angles_amp) in `rot_layout`; stored as `dtype` at the token's
 * place of the pool, rows of rank + extra. */
int b200_latent_store_rot(const float* raw, long long ld_raw, const float* w, float eps, void* pool, const int* pages,
                          int max_pages, int page_rows, const int* slot, const int* pos, int n_tokens, int rank, int extra,
                          const float* cos, const float* sin, int rot_layout, int dtype, void* stream);
/* dst[t, h, dst_off + i] = rot(src[t, src_off + h * src_stride + 0:dims])[i] for i < dims: the rotated part of every head's
 * query placed behind its absorbed part (fp32 to fp32; dst rows of ld_dst floats, heads dst_stride apart) */
int b200_rotate_part(const float* src, long long ld_src, long long src_off, long long src_stride, float* dst, long long ld_dst,
                     long long dst_off, long long dst_stride, const float* cos, const float* sin, int rot_layout, int n_tokens,
                     int heads, int dims, void* stream);

/* Router of a mixture of experts with identity experts: z = h W_r^T (fp32 accumulate; h of h_dtype, W_r fp32
 * [n_out, width]); s = softmax(z) over all n_out outputs; the `top` largest of s + correction are chosen; their weights
 * are s * scale (no correction, not renormalised). chosen / weight: [n_tokens, top]. */
int b200_moe_route(const void* h, int h_dtype, const float* w_router, const float* correction, int n_tokens, int width,
                   int n_out, int top, float scale, int* chosen, float* weight, void* stream);
/* Router that chooses on its logits: z = h W_r^T + bias (fp32 accumulate; bias may be NULL); the `top` largest z are
 * chosen (ties: the lower index) and their weights are the softmax over the chosen logits only. */
int b200_moe_route_logits(const void* h, int h_dtype, const float* w_router, const float* bias, int n_tokens, int width,
                          int n_out, int top, int* chosen, float* weight, void* stream);
/* Counting sort of the (token, choice) pairs by expert: group_off [n_experts + 1], src_row [n_tokens * top] (token of
 * each sorted row), dest [n_tokens, top] (sorted row of each pair, -1 for chosen >= n_experts: identity experts own no
 * rows). One launch, no host sync. */
int b200_moe_dispatch(const int* chosen, int n_tokens, int top, int n_experts, int* group_off, int* src_row, int* dest,
                      void* stream);
/* dst[i, :] = src[rows[i], :] (both of `dtype`, contiguous rows of `width`): the sorted rows of b200_moe_dispatch side by side,
 * so that a dense GEMM can read one expert's group */
int b200_gather_rows(const void* src, const int* rows, void* dst, int n_rows, int width, int dtype, void* stream);
/* x[t,:] += mix[t,:] + shared[t,:] + sum_k weight[t,k] * (dest[t,k] >= 0 ? expert_out[dest[t,k],:] : h[t,:])
 * (fp32 sums in a fixed order; mix, shared, the routed part may each be NULL) */
int b200_residual_combine(float* x, const float* mix, const float* shared, const float* expert_out, const int* dest,
                          const float* weight, const void* h, int h_dtype, int n_tokens, int width, int top, void* stream);

/* Sandwich layers (a norm before AND after each sublayer): x[t,:] += mult * LN(y[t,:]; w, b) on the fp32 residual, then,
 * when out2 is given, out2[t,:] = LN(x[t,:]; w2, b2) as out_dtype (the input of the next sublayer) from the same row
 * while it is still on chip. Two-pass mean / variance in fp32 for both norms. */
int b200_layernorm_residual(float* x, const float* y, int n_rows, int width, float eps, float mult, const float* w,
                            const float* b, const float* w2, const float* b2, void* out2, int out_dtype, void* stream);
/* out[t, 0:width] = a[t,:], out[t, width:2 width] = b[t,:], as out_dtype (the operand of a projection of two streams) */
int b200_concat_cast(const float* a, const float* b, void* out, int n_rows, int width, int out_dtype, void* stream);
/* out[t, j] = act(gu[t, j]) * gu[t, n + j], act by epi (B200_GG_GLU: silu, B200_GG_GLU_GELU: tanh-gelu); gu fp32 [n_rows, 2 n]:
 * the GLU of a [gate | up] product computed without the fused epilogue (small batches, where the stacked weight streams
 * once through the split-K GEMM) */
int b200_glu_act(const float* gu, void* out, int n_rows, int n, int epi, int out_dtype, void* stream);
/* v[i] <- cap * tanh(v[i] / cap) */
int b200_softcap(float* v, size_t n, float cap, void* stream);

/* Residual update fused with the RMS norm of whatever reads the residual next, one launch per sublayer:
 *   x[t,:] += s1 * y1[t,:] + s2 * y2[t,:] + sum_k weight[t,k] * expert_out[dest[t,k],:] + bcast[:]
 *   out[t,:] = x[t,:] / sqrt(mean(x[t,:]^2) + eps) * (w_offset + w[:])        (as out_dtype; skipped when w is NULL)
 * Every addend may be NULL (fp32 sums in this fixed order). With `rows` the call only norms: out[i,:] from x[rows[i],:],
 * nothing is added. w_offset 1 is a weight stored around zero, 0 a weight stored around one. */
typedef struct b200_rmsnorm_residual_args {
    float* x;
    const float* y1; float s1;
    const float* y2; float s2;
    const float* expert_out; const int* dest; const float* weight; int top;
    const float* bcast;
    const int* rows;
    const float* w; float w_offset, eps;
    void* out; int out_dtype;
    int n_rows, width;
    /* norm_addend != 0 (layers whose norm sits on the sublayer's OUTPUT): x[t,:] += (y1[t,:] + y_bias[:]) / rms(y1[t,:] +
       y_bias[:]) * (w_offset + w[:]), then out[t,:] = x[t,:] as out_dtype (what the next sublayer reads; out may be NULL).
       Only y1 (and y_bias, fp32 [width] or NULL) is added. */
    int norm_addend; const float* y_bias;
} b200_rmsnorm_residual_args;
int b200_rmsnorm_residual(const b200_rmsnorm_residual_args* a, void* stream);

/* Rotary positions: cos_out / sin_out [n_tokens, n_freq] = cos / sin(pos[t] * freq[i]); the angle is formed and reduced in
 * double precision (freq is a device array of doubles, whatever scaling of the frequencies already applied by the
 * caller), so position 10^5 is as exact as position 1. One launch per step and frequency set, shared by all layers. */
int b200_rope_angles(const int* pos, int n_tokens, const double* freq, int n_freq, float* cos_out, float* sin_out, void* stream);
/* the same with both tables multiplied by `amplitude` (designs that stretch q and k together with their frequencies) */
int b200_rope_angles_amp(const int* pos, int n_tokens, const double* freq, int n_freq, double amplitude, float* cos_out,
                         float* sin_out, void* stream);
#define B200_ROPE_HALF 0        /* dimension i pairs with i + dims/2  */
#define B200_ROPE_INTERLEAVED 1 /* dimension 2i pairs with 2i + 1      */

/* What lies between the q / k projection of an attention layer and its cache, in one launch per token and head:
 * an optional short causal convolution over time on every channel (y_t = sum_j w[c, j] u_(t - taps + 1 + j), zeros before
 * position 0; inputs older than this step come from conv_state), an optional per-head RMS norm with a weight shared by
 * the heads, rotary positions on the first rot_dims dimensions, then q to q_out and k into the page pool. Values:
 * v_from_conv != 0 stores the convolved, un-normed, un-rotated keys as the values (a design without a value
 * projection). Everything in fp32 up to the store in `dtype`.
 * Channels: query heads first, then key heads (proj row = [heads*dim | kv_heads*dim], leading dimension ld_proj).
 * start[t] = position of the first token that the token's sequence brings in THIS step (older inputs are state).
 * conv_state: fp32 [n_slots, taps-1, channels], position p at ring place p % (taps-1); written by
 * b200_conv_state_update AFTER this launch (the same stream), never by this kernel. */
typedef struct b200_qk_prepare_args {
    const float* proj; long long ld_proj;
    const float* conv_w; int taps; const float* conv_state;   /* conv_w NULL: no convolution */
    const float* q_norm; const float* k_norm; float eps;       /* NULL: no norm               */
    const float* cos; const float* sin; int rot_dims, rot_layout;
    void* q_out;                    /* dtype [n_tokens, heads*dim]                                  */
    void* k_pool; void* v_pool;     /* dtype [n_pages*page_rows, kv_heads, dim]                     */
    int v_from_conv;
    const int* pages; int max_pages, page_rows;
    const int* slot; const int* pos; const int* start;
    int n_tokens, heads, kv_heads, dim, dtype;
    int update_state_inline;   /* 1 (only when EVERY sequence brings exactly one token): the launch also files the token's
                                  inputs in conv_state, and b200_conv_state_update is not needed */
    /* projected values: v_heads > 0 stores proj[t, v_off + g * vdim + :] unchanged (no convolution, norm or rotation) at the
       token's row of v_pool [n_pages*page_rows, v_heads, vdim]; not together with v_from_conv */
    int v_heads, vdim; long long v_off;
    /* bias: fp32 [ld_proj], added to every column of proj that the launch reads (q, k and the projected values) before
       anything else. v_cos / v_sin [n_tokens, vdim/2]: the projected values are rotated by their own position over all
       vdim dimensions (pairs in v_rot_layout) before the store. Both may be NULL. */
    const float* bias;
    const float* v_cos; const float* v_sin; int v_rot_layout;
} b200_qk_prepare_args;
int b200_qk_prepare(const b200_qk_prepare_args* a, void* stream);
/* The last taps-1 inputs of every sequence of the step go to their ring places (end[t] = the sequence's length after
 * the step). */
int b200_conv_state_update(const float* proj, long long ld_proj, float* conv_state, const int* slot, const int* pos,
                           const int* end, int n_tokens, int channels, int taps, void* stream);

/* Causal attention over paged per-head keys and values with grouped query heads (query head h reads key head
 * h / (heads / kv_heads)): s_j = scale * <q, k_j>, then s_j <- softcap * tanh(s_j / softcap) when softcap > 0, over the
 * sequence's rows j <= pos[t]; p_j = exp(s_j) / (denom_bias + sum_j exp(s_j)) (denom_bias 1: a sink of score 0 without
 * a value; 0: plain softmax); out[t, h, :] = sum_j p_j v_j. q [n_tokens, heads*dim], out [n_tokens, heads*vdim], pools
 * [n_pages*page_rows, kv_heads, dim | vdim], all of `dtype`; scores, softmax and sums in fp32.
 * longest_entry (0 = unknown): most tokens one sequence brings in this batch; bfloat16 batches with prompt portions run
 * on tensor-core tiles, single tokens and fp32 on the row kernel; with a workspace and longest_context given, a batch of few
 * rows with long contexts (decoding) splits every context over up to 16 CTAs and merges the shares in a second launch. */
typedef struct b200_paged_attention_args {
    const void* q; void* out; const void* k_pool; const void* v_pool;
    const int* pages; int max_pages, page_rows;
    const int* slot; const int* pos;
    int n_tokens, heads, kv_heads, dim, vdim;
    float scale, softcap, denom_bias;
    int dtype, longest_entry;
    int longest_context;                       /* most rows any token sees (0 = unknown)                          */
    void* workspace; size_t workspace_bytes;   /* shares of split contexts (may be NULL: no splitting)            */
    /* chunk > 0: position p only sees the keys of its own block of positions, j >= floor(p / chunk) * chunk (blocks are
       counted from position 0 of the sequence).
       maps > 1: every query head holds `maps` score maps over the same values: q [n_tokens, heads, maps, dim], k_pool
       [rows, kv_heads, maps, dim], v_pool [rows, kv_heads, vdim], out [n_tokens, heads, maps, vdim] (map m of head h scores
       against map m of its key head and weights that head's values). 0 or 1: one map.
       out_f32 != 0: out is fp32 whatever `dtype` (a caller that combines maps or gates in fp32). */
    int chunk, maps, out_f32;
    /* window > 0: position p only sees the keys j with 0 <= p - j < window (together with chunk: both masks).
       sigmoid_weights != 0: no softmax; the weight of a visible key is sigmoid(s_j + head_bias[h]) (head_bias fp32 [heads]
       or NULL), not normalised over the keys: out = sum_j w_j v_j. Not with softcap, denom_bias or maps > 1. */
    int window, sigmoid_weights; const float* head_bias;
} b200_paged_attention_args;
size_t b200_paged_attention_workspace_bytes(int n_tokens, int heads, int vdim);
int b200_paged_attention(const b200_paged_attention_args* a, void* stream);

/* Retention: linear attention with a fixed decay per head and a carried state, no softmax. For every entry (a run of
 * consecutive tokens of one sequence: first batch row ent_row[e], ent_len[e] tokens) and head h, with q, k rotated on
 * their first rot_dims dimensions and k multiplied by k_scale after the rotation:
 *   S <- decay[h] * S + k_t v_t^T,   out[t, h, :] = S^T q_t
 * S fp32 [n_slots, heads, dim, vdim], starting from zero when the entry starts at position 0 (a slot that is used
 * again needs no clearing) and left in place for the next step. proj fp32 [n_tokens, ld_proj] holds q at column q_off
 * (heads*dim), k at k_off, v at v_off (heads*vdim). All arithmetic fp32. out fp32 [n_tokens, heads*vdim]. */
typedef struct b200_retention_args {
    const float* proj; long long ld_proj; int q_off, k_off, v_off;
    const float* cos; const float* sin; int rot_dims, rot_layout;
    const float* decay; float k_scale;
    float* state; float* out;
    const int* ent_row; const int* ent_len; const int* slot; const int* pos;
    int n_entries, n_tokens, heads, dim, vdim, longest_entry;
    void* workspace; size_t workspace_bytes;   /* chunk states of long entries (b200_retention_workspace_bytes) */
} b200_retention_args;
size_t b200_retention_workspace_bytes(int n_tokens, int n_entries, int heads, int dim, int vdim);
int b200_retention(const b200_retention_args* a, void* stream);
/* out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * silu(gate[t, h, :]) as out_dtype (gate fp32, leading
 * dimension ld_gate) */
int b200_unit_rms_gate(const float* o, const float* gate, long long ld_gate, void* out, int n_tokens, int heads, int vdim,
                       float eps, int out_dtype, void* stream);
/* Differential combination of two attention maps: o = a[t,h,0,:] - lambda * a[t,h,1,:]; out[t,h,:] = o / sqrt(mean(o^2) + eps)
 * * out_scale, as out_dtype. a fp32 [n_tokens, heads, 2, vdim]. */
int b200_diff_combine(const float* a, float lambda, float eps, float out_scale, void* out, int n_tokens, int heads, int vdim,
                      int out_dtype, void* stream);
/* out[t, c] = o[t, c] * sigmoid(gate[t, c]) as out_dtype; o fp32 [n_tokens, n], gate fp32 with leading dimension ld_gate */
int b200_sigmoid_gate(const float* o, const float* gate, long long ld_gate, void* out, int n_tokens, int n, int out_dtype,
                      void* stream);

/* Heads whose values were rotated by their own position: out[t, h, :] = rot(-pos[t])(o[t, h, :]) * sigmoid(gate[t * ld_gate +
 * h]) as out_dtype. o fp32 [n_tokens, heads, vdim]; cos / sin [n_tokens, vdim/2] of the token's position (the same tables
 * that rotated the values; the turn back is their conjugate); gate (fp32, one number per head) may be NULL. */
int b200_unrotate_gate(const float* o, const float* cos, const float* sin, int rot_layout, const float* gate, long long ld_gate,
                       void* out, int n_tokens, int heads, int vdim, int out_dtype, void* stream);

/* Element-wise gated recurrence whose gate and candidate read only the current token. Per entry (a run of consecutive
 * tokens of one sequence) and channel c, with z = sigmoid(pre[t, z_off + c] + z_bias[c]), u = pre[t, u_off + c] + u_bias[c]
 * and the candidate cand = u + 1/2 where u >= 0, sigmoid(u) where u < 0:
 *   S[c] <- (1 - z) S[c] + z cand;   out[t, c] = S[c] * silu(pre[t, g_off + c])      (as out_dtype)
 * S fp32 [n_slots, channels], starting from zero when the entry starts at position 0 and left in place for the next
 * step. pre fp32 [n_tokens, ld_pre]; biases fp32 [channels] or NULL. All arithmetic fp32. Entries longer than a chunk of
 * tokens run in three launches (chunk summaries, their sequential combination, the chunks again from their true start
 * states) and need the workspace. */
typedef struct b200_gated_recurrence_args {
    const float* pre; long long ld_pre; int z_off, u_off, g_off;
    const float* z_bias; const float* u_bias;
    float* state; void* out; int out_dtype;
    const int* ent_row; const int* ent_len; const int* slot; const int* pos;
    int n_entries, n_tokens, channels, longest_entry;
    void* workspace; size_t workspace_bytes;
} b200_gated_recurrence_args;
size_t b200_gated_recurrence_workspace_bytes(int n_tokens, int n_entries, int channels);
int b200_gated_recurrence(const b200_gated_recurrence_args* a, void* stream);

/* out[t,:] = table[ids[t],:] * scale + pair_table[row(t),:] as fp32, row(t) = (prev[t] * mul_prev + ids[t] * mul_cur) mod
 * buckets (64-bit arithmetic), or row `buckets` (the table's last) where prev[t] < 0: a sequence's first token. pair_table
 * [buckets + 1, width] may be NULL. Tables of `dtype`; out_cast (may be NULL) receives the same rows as `dtype`: the operand of
 * a first sublayer that reads the residual stream itself. */
int b200_embed_pair_hash(const int* ids, const int* prev, const void* table, float scale, const void* pair_table, int buckets,
                         int mul_prev, int mul_cur, float* out, void* out_cast, int n_tokens, int width, int dtype, void* stream);
/* v[i] *= f */
int b200_scale(float* v, size_t n, float f, void* stream);
/* the clamped GLU of a [gate | up] product computed without the fused epilogue (B200_GG_GLU_CLAMP; gu fp32 [n_rows, 2 n]) */
int b200_glu_act_clamped(const float* gu, void* out, int n_rows, int n, float limit, int out_dtype, void* stream);

/* Selective scan (a recurrence with input-dependent step sizes and a diagonal transition per channel), in three pieces.
 *
 * b200_conv_act: y[t, c] = silu(bias[c] + sum_j w[c, j] u[(t) - taps + 1 + j, c]) over the channels' own history (zeros
 * before position 0; inputs older than this step come from conv_state, a ring as in b200_qk_prepare, written afterwards by
 * b200_conv_state_update). u fp32 [n_tokens, ld_u]; out32 fp32 [n_tokens, channels] and out (out_dtype, the operand of the
 * next projection) may each be NULL.
 *
 * b200_selective_scan: per entry (a run of consecutive tokens of one sequence), channel c and state n, with
 * dt = softplus(dt_raw[t, c] + dt_bias[c]) (or dt = dt_raw[t, c] as it is when dt_ready != 0: the caller's projection
 * has applied bias and softplus already):
 *   S[c, n] <- exp(dt * A[c, n]) * S[c, n] + dt * x[t, c] * B[t, n];   y = sum_n S[c, n] * C[t, n] + D[c] * x[t, c]
 *   out[t, c] = y * silu(z[t, c])        (as out_dtype)
 * A fp32 [channels, n_state] (already negative), S fp32 [n_slots, channels, n_state], starting from zero when the entry
 * starts at position 0 and left in place for the next step. x, dt_raw fp32 [n_tokens, channels]; B, C fp32 rows of
 * leading dimension ld_bc; z fp32 with leading dimension ld_z. All arithmetic fp32. */
typedef struct b200_conv_act_args {
    const float* u; long long ld_u; const float* w; const float* bias; int taps; const float* conv_state;
    float* out32; void* out; int out_dtype;
    const int* slot; const int* pos; const int* start;
    int n_tokens, channels;
    int update_state_inline;   /* as in b200_qk_prepare_args */
} b200_conv_act_args;
int b200_conv_act(const b200_conv_act_args* a, void* stream);
typedef struct b200_selective_scan_args {
    const float* x; const float* dt_raw; const float* dt_bias;
    const float* B; const float* C; long long ld_bc;
    const float* z; long long ld_z;
    const float* A; const float* D;
    float* state; void* out; int out_dtype;
    const int* ent_row; const int* ent_len; const int* slot; const int* pos;
    int n_entries, n_tokens, channels, n_state, longest_entry;
    void* workspace; size_t workspace_bytes;   /* chunk summaries of long entries (b200_selective_scan_workspace_bytes) */
    int dt_ready;
} b200_selective_scan_args;
size_t b200_selective_scan_workspace_bytes(int n_tokens, int n_entries, int channels, int n_state);
int b200_selective_scan(const b200_selective_scan_args* a, void* stream);

/* ---------------------------------------------------------------------------------------------
 * models
 * --------------------------------------------------------------------------------------------- */
typedef struct b200_model b200_model;

typedef struct b200_model_options {
    int dtype;        /* B200_BF16: bfloat16 weights / operands, fp32 accumulation, residual and norms; B200_F32: all fp32 */
    int max_tokens;   /* cache pool: live tokens, each sequence rounded up to whole pages                            */
    int max_slots;    /* sequences alive at once                                                                    */
    int max_step_tokens; /* most tokens one step may bring (0 = default); scratch is sized for it                   */
} b200_model_options;

const char* b200_serve_last_error(void);
/* comma-separated names of the registered families */
const char* b200_model_families(void);
/* Reads dir/config.json, picks the family by its "architecture", loads the weights. NULL on failure. */
b200_model* b200_model_open(const char* dir, const b200_model_options* opt);
void b200_model_close(b200_model* m);
const char* b200_model_family(const b200_model* m);
int b200_model_vocab(const b200_model* m);
int b200_model_width(const b200_model* m);
int b200_model_layer_count(const b200_model* m);
int b200_model_max_positions(const b200_model* m);
int b200_model_page_rows(const b200_model* m);
int b200_model_pages_total(const b200_model* m);
int b200_model_pages_free(const b200_model* m);
int b200_model_slot_length(const b200_model* m, int slot);   /* tokens cached for the slot */
/* host copy of the slot's page list; returns the number of pages written (<= max_n) */
int b200_model_slot_pages(const b200_model* m, int slot, int* out, int max_n);

/* One step of the engine: entry i appends n_tokens[i] tokens (tokens packed back to back) to sequence slot slots[i]
 * after what the slot has cached, all entries as ONE batch (prompt portions beside single decoded tokens). n_want[i]
 * places (indices into the entry's tokens, packed in `want`) are asked for: logits_out (host, fp32 [sum n_want, vocab],
 * may be NULL) and ids_out (host, greedy pick per wanted place, may be NULL). Pages are taken as slots grow;
 * B200_ENOMEM when the pool is empty (nothing is run). */
int b200_model_step(b200_model* m, int n_entries, const int* slots, const int* n_tokens, const int* tokens,
                    const int* n_want, const int* want, float* logits_out, int* ids_out);
/* the slot's pages go back to the pool, its length to 0 */
int b200_model_release(b200_model* m, int slot);
/* debugging / tests: keep the residual stream after every layer of the next steps (fp32 [layers, tokens, width]) */
int b200_model_capture_layers(b200_model* m, int on);
int b200_model_captured_layers(b200_model* m, float* out, size_t max_floats);
/* kernels launched by the last step */
int b200_model_step_launches(const b200_model* m);

/* Continuous-batching generation with greedy sampling: n_requests prompts (ids packed, lens[]), at most max_slots
 * alive at once; waiting requests are admitted when a slot and pages for their prompt + max_new tokens are free;
 * prompts are fed in portions of at most chunk tokens per step (0 = whole) beside the other sequences' single
 * tokens; a sequence ends at eos_id (>= 0) or after max_new tokens. out_ids [n_requests, max_new] padded with
 * eos_id, n_generated [n_requests] (may be NULL). Returns the number of engine steps (>= 0) or an error (< 0). */
int b200_model_generate(b200_model* m, int n_requests, const int* prompt_ids, const int* lens, int max_new, int eos_id,
                        int chunk, int* out_ids, int* n_generated);

/* ---------------------------------------------------------------------------------------------
 * trace sessions: requests named by strings, replayed step by step (bin/trace_run)
 * --------------------------------------------------------------------------------------------- */
typedef struct b200_session b200_session;
b200_session* b200_session_create(b200_model* m);
void b200_session_destroy(b200_session* s);
/* slot of a request id, admitting it (first free slot) when new; < 0 when no slot is free */
int b200_session_slot(b200_session* s, const char* request_id);
/* the request is over: its slot and pages are free again */
int b200_session_end(b200_session* s, const char* request_id);

#ifdef __cplusplus
}
#endif
#endif /* B200_SERVE_H */
