/*
 * umbrella_b200_seq -- C ABI of the batched step of sequence-state decoders (libumbrella_b200_seq.so).
 *
 * A "sequence-state" model carries, per live sequence, a fixed amount of state instead of a cache that grows
 * with the context: a matrix per head of a decayed linear-attention ("retention") mixer, the last `window`
 * latents of a sliding-window latent-attention mixer (a ring), and the previous token's normed activations of
 * every layer (token shift).  The state lives in slots; one step runs any number of new tokens of any number
 * of slots (a ragged batch, no padding) and leaves every slot's state ready for the next step.
 *
 * Conventions as in umbrella_b200.h: plain device pointers, sizes, a cudaStream_t (as void*); no allocation,
 * no host synchronisation, no default-stream use.  0 = ok, negative = UMB_ERR_*, positive = cudaError_t.
 *
 * Models of the pre-norm form (UMBS_FORM_PRENORM) also keep what their mixers need in the slot: the key | value rows of
 * cached attention (a ring for a window, every token without one), one mean key | value row per block of older tokens,
 * the last projected rows in front of a short convolution, and the matrix memory of mLSTM layers.  The latent-attention
 * mixer also runs in this form, with direct queries, a rotated key part all heads share (kept behind the latent in the
 * ring), a sink and an output gate; its ring holds the whole sequence when the layer has no window.
 *
 * The building blocks are exported on their own (umbs_group_norm_shift, umbs_retention, umbs_latent_attention,
 * umbs_moe_route, umbs_gemm, umbs_depth_mix ...), each with its constants as arguments, and umbs_forward chains
 * them for a model described by umbs_model_t.  Numerics: norms, rotary angles, attention scores and weights,
 * routers, the residual stream and every recurrent quantity are fp32 in both modes; with UMBS_BF16 the matrix
 * products read bf16 operands and accumulate in fp32, with UMBS_F32 they are plain fp32 FMA chains (no TF32).
 */
#ifndef UMBRELLA_B200_SEQ_H
#define UMBRELLA_B200_SEQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* umbs_stream_t; /* cudaStream_t */

#define UMBS_BF16 0
#define UMBS_F32 1

#define UMBS_MIX_RETENTION 0
#define UMBS_MIX_LATENT_ATTENTION 1
#define UMBS_MIX_CACHED_ATTENTION 2  /* grouped-query attention over a per-slot key/value cache; options: window, pooled
                                      * blocks of older keys, sink or sigmoid weights, short convolution on q and k,
                                      * values = unrotated keys, output gate per head or per element */
#define UMBS_MIX_MLSTM 3             /* matrix memory with exponential gates and a running maximum */
#define UMBS_MIX_TIME_MIX 4          /* matrix memory with a decay per key channel and token, computed from the token itself;
                                      * five token-shifted mixes of the input feed its projections */

/* How a layer is put together.  PARALLEL: one group norm feeds the mixer (token-shifted) and the feed-forward side by
 * side, the sum goes through the depth average.  PRENORM: x += mixer(norm1(x)), then x += ff(norm2(x)). */
#define UMBS_FORM_PARALLEL 0
#define UMBS_FORM_PRENORM 1

/* Gated activation of a gate|up pair of products (the `dual` argument of umbs_gemm; 0 = plain product). */
#define UMBS_ACT_CLAMPED_GLU 1       /* g' sigmoid(1.702 g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit) */
#define UMBS_ACT_GELU_TANH 2         /* gelu_tanh(g) u */
#define UMBS_ACT_SILU 3              /* g sigmoid(g) u */

/* Activation of a plain product (the `unary` argument of umbs_gemm_unary; 0 = none). */
#define UMBS_UNARY_TANH 1            /* tanh(z) */
#define UMBS_UNARY_XIELU 2           /* z > 0: p0 z^2 + z / 2; z <= 0: p1 (exp(z) - 1 - z) + z / 2 */

/* Norm of the pre-norm layer form. */
#define UMBS_NORM_RMS 0              /* x / sqrt(mean(x^2) + eps) * (offset + w) */
#define UMBS_NORM_LAYER 1            /* (x - mean) / sqrt(mean((x - mean)^2) + eps) * (offset + w) + b */
#define UMBS_NORM_DYT 2              /* tanh(alpha x) * (offset + w) + b: no mean, no variance */

/* How a router turns its logits into experts and weights. */
#define UMBS_ROUTE_SOFTMAX_TOP 0     /* the `top` largest logits, softmax over them */
#define UMBS_ROUTE_SIGMOID_GROUPS 1  /* scores sigmoid(z); the experts form `groups` equal groups of neighbours, a group
                                      * scores the sum of its two largest scores, only experts of the `keep` best groups are
                                      * eligible; the `top` largest eligible scores, divided by their sum (+ 1e-20) */
#define UMBS_ROUTE_SOFTMAX_ALL 2     /* softmax over all experts; the `top` largest scores, as they are (not renormalised) */

/* How attention turns scores into weights. */
#define UMBS_ATTN_SOFTMAX 0          /* p = exp(s) / sum exp(s) */
#define UMBS_ATTN_SOFTMAX_SINK 1     /* p = exp(s) / (1 + sum exp(s)): a sink of score 0 without a value */
#define UMBS_ATTN_SIGMOID 2          /* p = sigmoid(s + bias[head]), not normalised over keys */

/* One step's ragged batch.  Token t of the step belongs to sequence tok_seq[t] (an index into the seq_* arrays)
 * and sits at absolute position tok_pos[t]; a sequence's tokens are contiguous: [seq_start, seq_start + seq_len).
 * seq_parity flips on every step of a sequence: the token-shift state is double-buffered so that one kernel can
 * read the old and write the new value. */
typedef struct {
    int n_tokens, n_seqs, n_want, max_seq_len;
    const int32_t* tok_ids;   /* [n_tokens] */
    const int32_t* tok_seq;   /* [n_tokens] */
    const int32_t* tok_pos;   /* [n_tokens] */
    const int32_t* seq_slot;  /* [n_seqs] state slot */
    const int32_t* seq_start; /* [n_seqs] first token of the sequence in this step */
    const int32_t* seq_len;   /* [n_seqs] tokens of the sequence in this step */
    const int32_t* seq_pos0;  /* [n_seqs] position of its first token (0 = a fresh sequence: state read as zero) */
    const int32_t* seq_parity;/* [n_seqs] */
    const int32_t* want_rows; /* [n_want] tokens whose logits are wanted */
    int max_pos0;             /* host copy of the largest seq_pos0: 0 = every sequence of the step is fresh */
} umbs_batch_t;

/* Gated feed-forward block: y = W_down( act(W_gate h, W_up h) ), act = UMBS_ACT_* (0 reads as UMBS_ACT_CLAMPED_GLU).
 * w_gu holds the gate rows followed by the up rows, per expert.  A dense feed-forward is a shared expert alone. */
typedef struct {
    int experts, top, ff;      /* experts == 0: no routed part */
    float limit;
    const float* w_router;     /* fp32 [experts, width] */
    const void* w_gu;          /* [experts, 2 ff, width] */
    const void* w_down;        /* [experts, width, ff] */
    int shared_ff;             /* 0: no shared expert */
    float shared_limit;
    const void* ws_gu;         /* [2 shared_ff, width] */
    const void* ws_down;       /* [width, shared_ff] */
    int act;                   /* UMBS_ACT_* of both parts */
    int route_mode;            /* UMBS_ROUTE_* */
    int groups, keep;          /* UMBS_ROUTE_SIGMOID_GROUPS: number of expert groups and how many stay eligible */
    const float* bias_gu;      /* fp32 [2 shared_ff] or NULL: biases of the shared (dense) gate rows, then of its up rows */
    const float* bias_down;    /* fp32 [width] or NULL: bias of the shared (dense) down projection */
    const float* w_shared_gate;/* fp32 [width] or NULL: the shared expert's output is multiplied by sigmoid(w . h), a number per token */
    float route_scale;         /* factor on the chosen experts' weights (0 reads as 1) */
    int plain;                 /* the shared (dense) part has no gate rows: W_down unary(W_up h), ws_gu = [shared_ff, width] */
    int unary;                 /* UMBS_UNARY_* of a plain part, with its two numbers */
    float unary_p0, unary_p1;
} umbs_mlp_t;

typedef struct umbs_layer_s {
    int mixer;                 /* UMBS_MIX_* */
    int heads, dim, vdim;
    /* retention */
    int rot_dims;
    const float* inv_freq;     /* fp32 [rot_dims / 2] */
    const float* decay;        /* fp32 [heads] */
    float* ret_state;          /* fp32 [slots, heads, dim, vdim] */
    /* latent attention */
    int q_rank, kv_rank, window, ring_len;
    float scale;
    const float* q_norm;       /* fp32 [q_rank] */
    const float* kv_norm;      /* fp32 [kv_rank] */
    const void* w_uq;          /* [heads dim, q_rank] */
    const void* w_ukT;         /* [heads, kv_rank, dim]: the key up-projection, transposed per head */
    const void* w_uv;          /* [heads vdim, kv_rank] */
    const void* w_ukv;         /* [heads dim + heads vdim, kv_rank]: key rows then value rows, or NULL; with it a step of
                                * fresh sequences up-projects its latents once and attends over per-head keys */
    void* ring;                /* act dtype [slots, ring_len, kv_rank] */
    /* both */
    const void* w_in;          /* retention: [q | k | v | g] rows; latent attention: [dq | dkv] rows; [., width] */
    const void* w_o;           /* [width, heads vdim] */
    const float* norm_w;       /* fp32 [width] */
    const float* shift_w;      /* fp32 [width] or NULL (no token shift) */
    float* shift_state;        /* fp32 [2, slots, width] */
    const float* depth_w;      /* fp32 [layer index + 2] or NULL (no depth average) */
    int has_mlp;
    umbs_mlp_t mlp;
    /* pre-norm form and the mixers that come with it */
    int form;                  /* UMBS_FORM_* */
    float norm_offset;         /* added to every norm weight of the layer (1: weights stored around zero) */
    const float* norm2_w;      /* fp32 [width]: the norm in front of the feed-forward (PRENORM with a feed-forward) */
    /* cached attention (uses heads, dim, vdim, rot_dims, inv_freq, window (0: every earlier token), scale from above);
     * w_in rows: q (heads dim) | k (kv_heads dim) | v (kv_heads vdim; absent with values_are_keys) | gate (heads, heads
     * vdim or none, by gate_kind) */
    int kv_heads;              /* query head h reads key/value head h / (heads / kv_heads) */
    int attn_mode;             /* UMBS_ATTN_* */
    int gate_kind;             /* 0: no output gate, 1: sigmoid of one number per head, 2: of one per output element */
    int values_are_keys;       /* the values are the keys as they are before the rotation (vdim = dim, no value rows) */
    int pool;                  /* tokens per pooled block of keys that have left the window (0: none) */
    int taps;                  /* taps of the short causal convolution on q and k (1: none) */
    float rot_mag;             /* factor on cos and sin (inv_freq holds the scaled frequencies) */
    float gate_cap;            /* mlstm: soft cap of the gate pre-activations */
    const float* bias_in;      /* fp32 [rows of w_in] or NULL */
    const float* conv_w;       /* fp32 [heads dim + kv_heads dim, taps] */
    const float* head_bias;    /* fp32 [heads] or NULL: added to the scores (UMBS_ATTN_SIGMOID) */
    const float* out_norm_w;   /* fp32 [heads vdim]: mlstm's weight after the per-head unit norm */
    void* kv_cache;            /* act dtype [slots, kv_len, kv_heads (dim + vdim)]: keys then values of a token; position p at
                                * row p mod kv_len (with a window: a ring of at least max(window, pool) rows; without:
                                * every token of the sequence) */
    int kv_len;
    void* pool_cache;          /* act dtype [slots, pool_len, kv_heads (dim + vdim)]: mean key | mean value per block */
    int pool_len;
    float* conv_state;         /* fp32 [2, slots, taps - 1, heads dim + kv_heads dim]: the last projected q | k rows
                                * (double-buffered by the sequence's parity, as the shift state) */
    float* mlstm_state;        /* fp32 [slots, heads, dim (vdim + 1) + 1]: S with n as column vdim, then m */
    /* pre-norm form, further options */
    int norm_kind;             /* UMBS_NORM_* of norm_w / norm2_w */
    const float* norm_b;       /* fp32 [width]: bias of a layer norm */
    const float* norm2_b;
    const float* out_scale;    /* fp32 [width] or NULL: the mixer's output is multiplied by it element by element (layer scale) */
    const float* out_scale2;   /* the same for the feed-forward's output */
    float residual_mult;       /* x += residual_mult * block output (0 reads as 1) */
    /* latent attention in the pre-norm form (uses heads, dim, vdim, kv_rank, window (0: every earlier token), ring,
     * ring_len, scale, kv_norm, w_ukT, w_uv, w_ukv, rot_dims, inv_freq, rot_mag, attn_mode, gate_kind (0 or 2) from above).
     * q_rank == 0: queries come straight from the layer input.  w_in rows: q (heads (dim + rope_dim)) | latent (kv_rank) |
     * shared rotated key part (rope_dim) | gate (heads vdim with gate_kind 2).  Every head's query is [dim | rope_dim]; its
     * key is [W_uk latent | the shared part]; positions turn the first rot_dims dimensions of the rope_dim part.  A ring
     * row holds [latent | rotated shared part], kv_rank + rope_dim numbers. */
    int rope_dim;
    const float* sink;         /* fp32 [heads] or NULL: with UMBS_ATTN_SOFTMAX_SINK the denominator also holds exp(sink[h]) (NULL: 1) */
    /* UMBS_NORM_DYT: the scalars of norm_w and norm2_w */
    float norm_alpha, norm2_alpha;
    /* cached attention, further options (see umbs_attn_opts_t and umbs_attention_finish) */
    float softcap;             /* > 0: score <- cap tanh(score / cap), after the scale */
    const float* dist_r1;      /* fp32 [heads] or NULL: score -= r1[h] ln(1 + r2[h] (i - j)) */
    const float* dist_r2;
    const float* talk;         /* fp32 [heads, heads] or NULL: after the softmax head h's weights become sum_g talk[h, g] weights_g;
                                * the mixed weights meet the values of h's own key/value head */
    int chunk;                 /* > 0: row i sees key j only if i / chunk == j / chunk (positions from the sequence's start) */
    int maps;                  /* 0 / 1: one softmax per head; 2: two, [map 1 | map 2] of dim numbers per query and key head over
                                * the same values, combined as a1 - diff_lambda a2 */
    float diff_lambda;
    int head_unit_norm;        /* every head's output is divided by its root mean square (eps inside the root) ... */
    float out_mult;            /* ... and multiplied by this (0 reads as 1) */
    const float* q_norm_w;     /* fp32 [dim] or NULL: RMS norm of every query head (and map) with this weight */
    const float* k_norm_w;     /* fp32 [dim] or NULL: the same for the keys, before they are cached */
    int kv_from;               /* 0: own keys and values; j + 1: this layer has no key / value rows in w_in and reads layer j's
                                * step rows and cache (kv_cache, kv_len must be layer j's) */
    /* time mix (uses heads, dim (= vdim), w_in = [r | k | v | g] rows (4 heads dim), w_o, shift_state, out_norm_w) */
    const float* mix_mu;       /* fp32 [5, width]: mix s = h + (h_prev - h) mu_s for s = r, k, v, g, w */
    int decay_rank;
    const void* w_decay1;      /* [decay_rank, width] */
    const void* w_decay2;      /* [heads dim, decay_rank] */
    const float* decay_bias;   /* fp32 [heads dim]: w = exp(-exp(W_2 tanh(W_1 mix_w) + decay_bias)) */
    const float* bonus;        /* fp32 [heads dim]: weight of the current token's own k v^T in its read-out */
    float* tm_state;           /* fp32 [slots, heads, dim, dim] */
    /* a second mixer beside the first: both read the same normed input, the layer adds
     * mix_scale * first + second_scale * second.  Only its mixer fields are read (no norms, no feed-forward). */
    const struct umbs_layer_s* second;
    float mix_scale, second_scale;      /* read only with a second mixer */
} umbs_layer_t;

typedef struct {
    int dtype;                 /* UMBS_BF16 / UMBS_F32: type of weights, activations between matrix products, ring */
    int width, vocab, n_layers, norm_groups, slots;
    float norm_eps;
    const void* embed;         /* [vocab, width] */
    const float* final_norm;   /* fp32 [width] */
    const void* head;          /* [vocab, width] */
    const umbs_layer_t* layers;/* host array */
    float norm_offset;         /* added to the final norm's weight */
    float logit_softcap;       /* > 0: logits <- cap tanh(logits / cap) */
    float embed_scale;         /* the embedding row is multiplied by it (0 reads as 1) */
    int norm_kind;             /* UMBS_NORM_* of the final norm (pre-norm form) */
    const float* final_norm_b; /* fp32 [width]: bias of a final layer norm */
    float final_norm_alpha;    /* UMBS_NORM_DYT */
    const float* pos_freq;     /* fp32 [width / 2] or NULL: sinusoidal positions are added to the embedding,
                                * entry 2i += sin(position pos_freq[i]), entry 2i + 1 += cos(position pos_freq[i]) */
} umbs_model_t;

const char* umbs_version(void);
unsigned long long umbs_launch_count(void);

/* Bytes of scratch umbs_forward needs for a step of up to max_tokens tokens of which up to max_want want logits. */
size_t umbs_workspace_bytes(const umbs_model_t* model, int max_tokens, int max_want);

/* One step.  logits: fp32 [n_want, vocab].  layer_out: optional fp32 [n_layers, n_tokens, width], the residual
 * stream each layer hands to the next (debugging aid). */
int umbs_forward(const umbs_model_t* model, const umbs_batch_t* batch, float* logits, float* layer_out,
                 void* workspace, size_t workspace_bytes, umbs_stream_t stream);

/* ---- building blocks (dtype: UMBS_BF16 / UMBS_F32 for the `void*` activations and weights) ---- */

/* C[m, g*c_goff + n] = sum_k A[row(m), g*a_goff + k] * W[g*w_gstride + n*ldw + k], fp32 accumulation in k order
 * (a row's result does not depend on the other rows of the call).  groups > 1: batched over g.  grp_off != NULL:
 * group g owns rows [grp_off[g], grp_off[g+1]) (device array; M bounds a group's size), row_src != NULL gathers A rows.
 * dual != 0: W holds N gate rows then N up rows per group and C gets the gated activation (see umbs_mlp_t).
 * c_f32 != 0: C is fp32, otherwise of `dtype`. */
int umbs_gemm(int dtype, const void* A, int64_t lda, int a_goff, const void* W, int64_t ldw, int64_t w_gstride, void* C,
              int64_t ldc, int c_goff, int c_f32, int M, int N, int K, int groups, const int32_t* grp_off,
              const int32_t* row_src, int dual, float limit, umbs_stream_t stream);

/* umbs_gemm with an epilogue: bias (fp32 [N], with dual [2 N]: gate rows' then up rows'; the same for every group, or
 * NULL) is added to the sums before the activation; out_gate (fp32, or NULL) multiplies the result by
 * sigmoid(out_gate[row ld_gate + g gate_goff + n]).  dual: UMBS_ACT_*. */
int umbs_gemm_ex(int dtype, const void* A, int64_t lda, int a_goff, const void* W, int64_t ldw, int64_t w_gstride, void* C,
                 int64_t ldc, int c_goff, int c_f32, int M, int N, int K, int groups, const int32_t* grp_off,
                 const int32_t* row_src, int dual, float limit, const float* bias, const float* out_gate, int64_t ld_gate,
                 int gate_goff, umbs_stream_t stream);

/* h = group_rms_norm(x) * w (groups equal consecutive parts, eps inside the root); hs = h + (h_prev - h) * shift_w
 * with h_prev the previous token's h (the slot's state for the first token of a step, zero at position 0).  Writes
 * h and hs as `dtype` and the last token's h (fp32) into the other half of the double-buffered state. */
int umbs_group_norm_shift(int dtype, const float* x, const float* w, const float* shift_w, float* shift_state, int slots,
                          const umbs_batch_t* batch, int width, int groups, float eps, void* h, void* hs,
                          umbs_stream_t stream);

/* Rows `rows[i]` of x (fp32 [., width]) -> group norm * w -> y (`dtype` [n_rows, width]). */
int umbs_group_norm_rows(int dtype, const float* x, const int32_t* rows, int n_rows, const float* w, int width,
                         int groups, float eps, void* y, umbs_stream_t stream);

/* Decayed linear attention over qkvg = [q | k | v | g] (fp32 [n_tokens, ld]): rotary (rotate-half pairs, the first
 * rot_dims dimensions, angle = position * inv_freq[i]) on q and k, k *= dim^-1/2, S <- decay_h S + k v^T, o = S^T q,
 * o / rms(o) per head, * silu(g) -> out (`dtype` [n_tokens, heads vdim]).  state: fp32 [slots, heads, dim, vdim];
 * o_scratch: fp32 [n_tokens, heads vdim]; rot_scratch: fp32 [n_tokens, rot_dims] (the step's cos | sin table).
 * seg_scratch (optional, fp32, seg_bytes): room for segment states, heads dim vdim floats each.  With it a step of few
 * long sequences is cut into segments that run side by side in two passes; as many segments as fit are used. */
int umbs_retention(int dtype, const float* qkvg, int64_t ld, const umbs_batch_t* batch, int heads, int dim, int vdim,
                   int rot_dims, const float* inv_freq, const float* decay, float eps, float* state, float* o_scratch,
                   float* rot_scratch, float* seg_scratch, size_t seg_bytes, void* out, umbs_stream_t stream);

/* Plain RMS norms of the two latents: x (fp32 [n, q_rank + kv_rank]) -> cq (`dtype` [n, q_rank]), c (`dtype` [n, kv_rank]). */
int umbs_latent_norm(int dtype, const float* x, int n, int q_rank, int kv_rank, const float* q_norm, const float* kv_norm,
                     float eps, void* cq, void* c, umbs_stream_t stream);

/* Sliding-window softmax attention in the latent space: token at position i sees positions j, 0 <= i - j < window.
 * q_abs: fp32 [n_tokens, heads, kv_rank] (queries already multiplied by the key up-projection); keys and values are the
 * latents themselves: c (this step's, `dtype` [n_tokens, kv_rank]) for j >= seq_pos0, the slot's ring for older ones.
 * out: `dtype` [n_tokens, heads, kv_rank].  split_scratch (optional, fp32): a decode step (one token per sequence) splits
 * each row's keys over n blocks (as many as fill the GPU, at most one per 32 keys) and merges the partial softmax states;
 * it needs n_tokens heads n (kv_rank + 2) floats there and runs unsplit when it gets less. */
int umbs_latent_attention(int dtype, const float* q_abs, const void* c, const void* ring, int ring_len,
                          const umbs_batch_t* batch, int heads, int kv_rank, int window, float scale,
                          float* split_scratch, size_t split_bytes, void* out, umbs_stream_t stream);

/* Sliding-window softmax attention of a step whose keys all sit in the step (fresh sequences): q, k [n_tokens, heads,
 * dim] and v [n_tokens, heads, vdim] in `dtype` with row strides ldq / ldk / ldv (elements); row i of a sequence sees
 * rows j of the same sequence with 0 <= i - j < window.  fp32 scores and softmax.  out: `dtype`, row stride ldo, heads
 * side by side.  dim and vdim up to 128 (umbs_window_attention_fits), else UMB_ERR_UNSUPPORTED. */
int umbs_window_attention_fits(int dim, int vdim);
int umbs_window_attention(int dtype, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                          const umbs_batch_t* batch, int heads, int dim, int vdim, int window, float scale, void* out,
                          int64_t ldo, umbs_stream_t stream);

/* The same over keys that carry a part all heads share: a key row (of c and of the ring) is [latent (kv_rank) | shared
 * part (rope_dim)], a query row of q_abs [n_tokens, heads, kv_rank + rope_dim] likewise; the score is the dot product over
 * all kv_rank + rope_dim numbers, the value is the latent.  window <= 0: every earlier token (the ring then holds the whole
 * sequence).  mode: UMBS_ATTN_SOFTMAX or UMBS_ATTN_SOFTMAX_SINK, where the denominator also holds exp(sink[head]) (sink
 * NULL: exp(0)).  out: `dtype` [n_tokens, heads, kv_rank].  kv_rank <= 512, kv_rank + rope_dim <= 640. */
int umbs_latent_attention_ex(int dtype, const float* q_abs, const void* c, const void* ring, int ring_len,
                             const umbs_batch_t* batch, int heads, int kv_rank, int rope_dim, int window, float scale, int mode,
                             const float* sink, float* split_scratch, size_t split_bytes, void* out, umbs_stream_t stream);

/* What stands between the in-projection of a latent-attention layer with direct queries and its attention kernel.
 * proj: fp32 [n_tokens, ld] = [q (heads (dim + rope_dim)) | latent (kv_rank) | shared key part (rope_dim) | ...].
 * c (`dtype` [n_tokens, kv_rank + rope_dim]) = [latent / rms(latent) * kv_norm | shared part turned by its position];
 * q (`dtype` [n_tokens, heads, dim + rope_dim]) = every head's query with its last rope_dim numbers turned; q_rot (fp32, row
 * stride ld_qrot per head, or NULL) gets each head's turned part again, in fp32.  The turn: pairs (i, i + rot_dims / 2) of
 * the first rot_dims of the rope_dim numbers, angle = position inv_freq[i], cos and sin times rot_mag. */
int umbs_latent_prep(int dtype, const float* proj, int64_t ld, const umbs_batch_t* batch, int heads, int dim, int rope_dim,
                     int kv_rank, const float* kv_norm, float eps, int rot_dims, const float* inv_freq, float rot_mag, void* q,
                     void* c, float* q_rot, int64_t ld_qrot, umbs_stream_t stream);

/* umbs_window_attention with options: k_shared (`dtype` [n_tokens, shared_dim], row stride ldks, or NULL) is a key part all
 * heads share -- a head's key is its own dim numbers of k followed by it, and q holds dim + shared_dim numbers per head;
 * window <= 0: every earlier token of the step; mode UMBS_ATTN_SOFTMAX_SINK: the denominator also holds exp(sink[head])
 * (sink NULL: exp(0)); gate (fp32 [n_tokens, ldg] or NULL): the output is multiplied element by element by
 * sigmoid(gate[t ldg + h vdim + c]).  dim + shared_dim <= 192, vdim <= 128 (umbs_window_attention_ex_fits). */
int umbs_window_attention_ex_fits(int dim, int shared_dim, int vdim);
int umbs_window_attention_ex(int dtype, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* k_shared,
                             int64_t ldks, int shared_dim, const void* v, int64_t ldv, const umbs_batch_t* batch, int heads,
                             int dim, int vdim, int window, float scale, int mode, const float* sink, const float* gate,
                             int64_t ldg, void* out, int64_t ldo, umbs_stream_t stream);

/* Stores this step's latents into the slots' rings (position p at row p mod ring_len). */
int umbs_ring_append(int dtype, const void* c, void* ring, int ring_len, const umbs_batch_t* batch, int kv_rank,
                     umbs_stream_t stream);

/* Router: z = W_router h (fp32), the `top` largest logits, softmax over them; then the (token, choice) pairs sorted by
 * expert: grp_off [experts + 1], pair_tok [n top] (token of sorted pair), pair_pos [n top] (sorted place of pair t*top+k).
 * scratch: int32 [2 experts + n top]. */
int umbs_moe_route(int dtype, const void* h, int n, int width, const float* w_router, int experts, int top,
                   float* sel_w, int32_t* grp_off, int32_t* pair_tok, int32_t* pair_pos, int32_t* scratch,
                   umbs_stream_t stream);

/* umbs_moe_route with the rule as an argument (mode: UMBS_ROUTE_*; groups, keep: see UMBS_ROUTE_SIGMOID_GROUPS; at most 64
 * groups).  Ties go to the lower index.  gate_w (fp32 [width], or NULL): one more row beside the router's, whose sigmoid
 * goes to gate_out[t] (fp32 [n]) -- what umbs_token_gate computes, in the same pass over h. */
int umbs_moe_route_ex(int dtype, const void* h, int n, int width, const float* w_router, int experts, int top, int mode,
                      int groups, int keep, float* sel_w, int32_t* grp_off, int32_t* pair_tok, int32_t* pair_pos,
                      int32_t* scratch, const float* gate_w, float* gate_out, umbs_stream_t stream);

/* g[t] = sigmoid(w . h[t]) in fp32; h: `dtype` [n, width], w: fp32 [width]. */
int umbs_token_gate(int dtype, const void* h, int n, int width, const float* w, float* g, umbs_stream_t stream);

/* X_next = x + (mix + (sum_k sel_w[t,k] pair_out[pair_pos[t,k]] + shared)); stores it at stack[layer + 1] and writes
 * x_out = sum_j depth_w[j] stack[j] (j <= layer + 1), or X_next itself when depth_w is NULL.  All fp32 [n, width];
 * stack: [n_layers + 1, n, width].  pair_out / shared may be NULL. */
int umbs_depth_mix(const float* x, const float* mix, const float* pair_out, const float* sel_w, const int32_t* pair_pos,
                   int top, const float* shared, float* stack, int layer, const float* depth_w, float* x_out,
                   float* copy_out, int n, int width, umbs_stream_t stream);

/* ---- pre-norm layers: residual + norm, the attention kinds over a per-slot key/value cache, mLSTM ---- */

/* Residual add and RMS norm in one pass.  rows == NULL: for every row t < n: x[t] += delta[t] (delta may be NULL),
 * copy[t] = x[t] (copy may be NULL), y[t] = x[t] / sqrt(mean(x[t]^2) + eps) * (w_offset + w) as `dtype` (y may be NULL).
 * rows != NULL: y[r] is the norm of x[rows[r]] + delta[rows[r]], r < n; x is not written. */
int umbs_add_rms_norm(int dtype, float* x, const float* delta, const int32_t* rows, int n, const float* w, float w_offset,
                      int width, float eps, void* y, float* copy, umbs_stream_t stream);

/* A block's output waiting to be added to the residual stream: (delta_mult delta + delta2_mult delta2 +
 * sum_k sel_w[t, k] pair_out[pair_pos[t, k]] + shared[t] shared_gate[t]) * scale * mult.  Every pointer may be NULL (shared_gate NULL: 1; scale NULL: 1). */
typedef struct {
    const float* delta;        /* fp32 [n, width] */
    const float* pair_out;     /* fp32 [n top, width]: the routed experts' outputs in sorted-pair order */
    const float* sel_w;        /* fp32 [n, top] */
    const int32_t* pair_pos;   /* [n, top] */
    int top;
    const float* shared;       /* fp32 [n, width] */
    const float* shared_gate;  /* fp32 [n] */
    const float* scale;        /* fp32 [width] */
    float mult;
    float delta_mult;          /* factor on delta alone (with delta2 == NULL, 0 reads as 1) */
    const float* delta2;       /* fp32 [n, width] or NULL: a second dense part, added as delta2_mult * delta2 */
    float delta2_mult;
} umbs_delta_t;

/* umbs_add_rms_norm for any pending output and either norm: x[t] += pending(t) (d may be NULL), copy, and
 * y[t] = norm(x[t]) with kind = UMBS_NORM_* (b: the layer norm's bias).  rows != NULL: y[r] is the norm of
 * x[rows[r]] + pending(rows[r]); x is not written.  width <= 8192. */
int umbs_add_norm(int dtype, float* x, const umbs_delta_t* d, const int32_t* rows, int n, int kind, const float* w,
                  const float* b, float w_offset, int width, float eps, void* y, float* copy, umbs_stream_t stream);

/* umbs_add_norm with the scalar of UMBS_NORM_DYT: y = tanh(alpha x) (w_offset + w) + b. */
int umbs_add_norm_ex(int dtype, float* x, const umbs_delta_t* d, const int32_t* rows, int n, int kind, const float* w,
                     const float* b, float w_offset, float alpha, int width, float eps, void* y, float* copy,
                     umbs_stream_t stream);

/* z <- cap tanh(z / cap), fp32, n values. */
int umbs_softcap(float* z, int64_t n, float cap, umbs_stream_t stream);

/* Queries, keys and values of an attention layer from its in-projection.  proj: fp32 [n_tokens, ld] = [q (heads dim) |
 * k (kv_heads dim) | v (kv_heads vdim, absent when values are the keys) | gate ...].  Adds bias (or NULL), runs the
 * causal convolution of `taps` taps over q and k (conv_w fp32 [heads dim + kv_heads dim, taps]; the rows before a
 * sequence's step come from conv_state, zeros at position 0; the step's last taps - 1 projected rows are left there:
 * fp32 [2, slots, taps - 1, channels], double-buffered by the sequence's parity), turns the first rot_dims dimensions
 * of every head of q and k by position * inv_freq[i] (pairs i, i + rot_dims / 2; cos and sin times rot_mag), and writes
 * q (`dtype` [n_tokens, heads dim]) and kv (`dtype` [n_tokens, kv_heads (dim + vdim)]: rotated keys, then values; with
 * values_are_keys the values are the keys before the rotation and vdim = dim). */
int umbs_attention_prep(int dtype, const float* proj, int64_t ld, const float* bias, const umbs_batch_t* batch, int heads,
                        int kv_heads, int dim, int vdim, int values_are_keys, int taps, const float* conv_w,
                        float* conv_state, int slots, int rot_dims, const float* inv_freq, float rot_mag, void* q, void* kv,
                        umbs_stream_t stream);

/* Mean key | mean value of every block of `pool` tokens that this step completes -> pool_cache row b of the slot.
 * Tokens of the step come from kv, older ones of the block from the slot's rows in kv_cache (which umbs_ring_append
 * fills: the step's kv rows, position p at row p mod kv_len). */
int umbs_kv_pool(int dtype, const void* kv, const void* kv_cache, int kv_len, void* pool_cache, int pool_len,
                 const umbs_batch_t* batch, int row, int pool, umbs_stream_t stream);

/* Attention of a step over the step's own keys and the slot's cache.  The row at position i sees the tokens j with
 * 0 <= i - j < window (window <= 0: every j <= i) and, with pool > 0, block b's mean key and value for every block with
 * b pool + pool - 1 <= i - window.  Tokens j >= seq_pos0 are read from kv, older ones from kv_cache, blocks from pool_cache.
 * mode: UMBS_ATTN_*; scores (q . k) scale (+ head_bias[h] for the sigmoid), fp32 throughout.  The output of head h is
 * multiplied by sigmoid(gate[t ldg + h]) (gate_per_head) or element by element by sigmoid(gate[t ldg + h vdim + c]);
 * gate may be NULL.  out: `dtype` [n_tokens, heads vdim].  dim, vdim <= 256, else UMB_ERR_UNSUPPORTED.
 * split_scratch (optional, fp32): a decode step (one token per sequence) spreads every row's keys over several blocks
 * and merges their partial sums; it needs n_tokens heads n (vdim + 2) floats there and runs unsplit with less. */
int umbs_cached_attention(int dtype, int mode, const void* q, const void* kv, const void* kv_cache, int kv_len,
                          const void* pool_cache, int pool_len, const umbs_batch_t* batch, int heads, int kv_heads, int dim,
                          int vdim, int window, int pool, float scale, const float* head_bias, const float* gate, int64_t ldg,
                          int gate_per_head, float* split_scratch, size_t split_bytes, void* out, umbs_stream_t stream);

/* mLSTM over proj = [q | k | v | gate (heads vdim) | i (heads) | f (heads)] (fp32 [n_tokens, ld]); gate_bias: fp32
 * [2 heads] for i | f.  Per head, with the log gates i = cap tanh(i' / cap), f = logsigmoid(cap tanh(f' / cap)):
 * m_t = max(f + m_(t-1), i), S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T, n_t likewise with k alone,
 * o = S_t^T (q dim^-1/2) / (max(|n_t . q dim^-1/2|, e^(-m_t)) + 1e-6); then o / rms(o) per head (eps inside the root)
 * times out_norm_w times sigmoid(gate) -> out (`dtype` [n_tokens, heads vdim]).  state: fp32 [slots, heads,
 * dim (vdim + 1) + 1] (S with n as its last column, then m; read as zero at position 0).  gates_scratch: fp32
 * [n_tokens, heads, 3]; o_scratch: fp32 [n_tokens, heads, vdim + 1].  seg_scratch (optional, fp32, seg_bytes): room for
 * segment states; with it a step of few long sequences is cut into segments that run side by side in two passes (as many
 * segments as fit: heads (dim (vdim + 1) + 1) floats per sequence and segment). */
int umbs_mlstm(int dtype, const float* proj, int64_t ld, const float* gate_bias, const umbs_batch_t* batch, int heads,
               int dim, int vdim, float gate_cap, float eps, const float* out_norm_w, float* state, float* gates_scratch,
               float* o_scratch, float* seg_scratch, size_t seg_bytes, void* out, umbs_stream_t stream);

/* ---- score options of cached attention, the time-mix memory, and what comes with them ---- */

/* umbs_attention_prep for query and key heads that hold `maps` maps of dim numbers each ([map 1 | map 2 | ...] per head; the
 * values stay kv_heads vdim) and an RMS norm of every (head, map) over its dim numbers with the weights q_norm_w / k_norm_w
 * (fp32 [dim], NULL: none; after the convolution, before the rotation; eps inside the root).  kv_heads == 0: the layer
 * borrows its keys and values, proj holds the query rows only and kv is not written. */
int umbs_attention_prep_ex(int dtype, const float* proj, int64_t ld, const float* bias, const umbs_batch_t* batch, int heads,
                           int kv_heads, int dim, int vdim, int values_are_keys, int taps, const float* conv_w,
                           float* conv_state, int slots, int rot_dims, const float* inv_freq, float rot_mag, int maps,
                           const float* q_norm_w, const float* k_norm_w, float eps, void* q, void* kv, umbs_stream_t stream);

/* Options of umbs_cached_attention_ex.  With maps = M and value_heads = C the kernel runs heads M C independent softmax rows
 * per token, numbered (h M + m) C + c: queries (h M + m) dim of q [n_tokens, heads M dim], keys ((h / rep) M + m) dim of a
 * key/value row [kv_heads M dim | kv_heads vdim], values of head c (C = kv_heads: every query head against every value
 * head, what talking heads need) or of the query's own key/value head (C = 1). */
typedef struct {
    float softcap;             /* > 0: score <- cap tanh(score / cap) after the scale */
    const float* dist_r1;      /* fp32 [heads] or NULL: score -= r1[h] ln(1 + r2[h] (i - j)) */
    const float* dist_r2;
    int chunk;                 /* > 0: key j is visible to row i only if i / chunk == j / chunk */
    int maps;                  /* 0 reads as 1 */
    int value_heads;           /* 0 reads as 1 */
    float* raw_out;            /* fp32 [n_tokens, heads M C, vdim] or NULL: the normalised outputs go here (no gate) instead of out */
} umbs_attn_opts_t;

/* umbs_cached_attention with the options above (opts NULL: none).  Pooled blocks go with none of the options. */
int umbs_cached_attention_ex(int dtype, int mode, const void* q, const void* kv, const void* kv_cache, int kv_len,
                             const void* pool_cache, int pool_len, const umbs_batch_t* batch, int heads, int kv_heads, int dim,
                             int vdim, int window, int pool, float scale, const float* head_bias, const float* gate,
                             int64_t ldg, int gate_per_head, const umbs_attn_opts_t* opts, float* split_scratch,
                             size_t split_bytes, void* out, umbs_stream_t stream);

/* From raw attention outputs (fp32 [n_tokens, heads M C, vdim], see umbs_attn_opts_t) to the mixer's output (`dtype`
 * [n_tokens, heads vdim]).  talk (fp32 [heads, heads], needs M = 1, C = kv_heads): o_h = sum_g talk[h, g] raw[g, h / rep];
 * M = 2 (needs C = 1): o_h = raw[h, 0] - diff_lambda raw[h, 1]; unit_norm: o_h / sqrt(mean(o_h^2) + eps); times out_mult;
 * gate (fp32, or NULL): times sigmoid(gate[t ldg + h vdim + c]).  vdim <= 256. */
int umbs_attention_finish(int dtype, const float* raw, int n_tokens, int heads, int kv_heads, int vdim, int maps,
                          int value_heads, const float* talk, float diff_lambda, int unit_norm, float eps, float out_mult,
                          const float* gate, int64_t ldg, void* out, umbs_stream_t stream);

/* Token-shifted mixes: out[t, s, :] = h[t] + (h[t - 1] - h[t]) mu[s, :], s < n_mix (`dtype` [n_tokens, n_mix, width]); the
 * row before a sequence's first token of the step comes from shift_state (fp32 [2, slots, width], the half seq_parity names;
 * zeros at position 0), the step's last row goes to the other half. */
int umbs_shift_mix(int dtype, const void* h, const float* mu, int n_mix, float* shift_state, int slots,
                   const umbs_batch_t* batch, int width, void* out, umbs_stream_t stream);

/* The time-mix memory.  proj: fp32 [n_tokens, ld] = [r | k | v | g], heads dim each; decay_raw: fp32 [n_tokens, heads dim].
 * Per head, with w_t = exp(-exp(decay_raw_t + decay_bias)): o_t = (S + diag(bonus) k_t v_t^T)^T r_t, then
 * S <- diag(w_t) S + k_t v_t^T (S: dim x dim, key index first; fp32 [slots, heads, dim, dim], read as zero at position 0).
 * Then o / sqrt(mean(o^2) + eps) per head, times out_norm_w, times silu(g) -> out (`dtype` [n_tokens, heads dim]).
 * o_scratch: fp32 [n_tokens, heads dim].  dim <= 128. */
int umbs_time_mix(int dtype, const float* proj, int64_t ld, const float* decay_raw, const float* decay_bias,
                  const float* bonus, const umbs_batch_t* batch, int heads, int dim, float eps, const float* out_norm_w,
                  float* state, float* o_scratch, void* out, umbs_stream_t stream);

/* umbs_gemm_ex for a plain product followed by a unary activation (UMBS_UNARY_*, with its two numbers). */
int umbs_gemm_unary(int dtype, const void* A, int64_t lda, int a_goff, const void* W, int64_t ldw, int64_t w_gstride, void* C,
                    int64_t ldc, int c_goff, int c_f32, int M, int N, int K, int groups, const float* bias, int unary,
                    float p0, float p1, umbs_stream_t stream);

/* umbs_moe_route_ex with a factor on the chosen weights; mode may also be UMBS_ROUTE_SOFTMAX_ALL. */
int umbs_moe_route_scaled(int dtype, const void* h, int n, int width, const float* w_router, int experts, int top, int mode,
                          int groups, int keep, float weight_scale, float* sel_w, int32_t* grp_off, int32_t* pair_tok,
                          int32_t* pair_pos, int32_t* scratch, const float* gate_w, float* gate_out, umbs_stream_t stream);

/* y[t] = table[ids[t]] * scale + sinusoidal positions (pos_freq fp32 [width / 2] or NULL: none): entry 2i gets
 * sin(tok_pos[t] pos_freq[i]), entry 2i + 1 the cosine; angles and sums in fp32. */
int umbs_embedding_pos(int dtype, const int32_t* ids, const int32_t* tok_pos, const void* table, float scale,
                       const float* pos_freq, float* y, int n, int width, umbs_stream_t stream);

int umbs_embedding(int dtype, const int32_t* ids, const void* table, float* y, int n, int width, umbs_stream_t stream);
/* y[t] = table[ids[t]] * scale (fp32). */
int umbs_embedding_scaled(int dtype, const int32_t* ids, const void* table, float scale, float* y, int n, int width,
                          umbs_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
