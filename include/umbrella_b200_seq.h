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

/* Gated feed-forward block: y = W_down( act(W_gate h, W_up h) ), act(g, u) = g' sigmoid(1.702 g') (u' + 1) with
 * g' = min(g, limit), u' = clamp(u, -limit, limit).  w_gu holds the gate rows followed by the up rows, per expert. */
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
} umbs_mlp_t;

typedef struct {
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
} umbs_layer_t;

typedef struct {
    int dtype;                 /* UMBS_BF16 / UMBS_F32: type of weights, activations between matrix products, ring */
    int width, vocab, n_layers, norm_groups, slots;
    float norm_eps;
    const void* embed;         /* [vocab, width] */
    const float* final_norm;   /* fp32 [width] */
    const void* head;          /* [vocab, width] */
    const umbs_layer_t* layers;/* host array */
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

/* Stores this step's latents into the slots' rings (position p at row p mod ring_len). */
int umbs_ring_append(int dtype, const void* c, void* ring, int ring_len, const umbs_batch_t* batch, int kv_rank,
                     umbs_stream_t stream);

/* Router: z = W_router h (fp32), the `top` largest logits, softmax over them; then the (token, choice) pairs sorted by
 * expert: grp_off [experts + 1], pair_tok [n top] (token of sorted pair), pair_pos [n top] (sorted place of pair t*top+k).
 * scratch: int32 [2 experts + n top]. */
int umbs_moe_route(int dtype, const void* h, int n, int width, const float* w_router, int experts, int top,
                   float* sel_w, int32_t* grp_off, int32_t* pair_tok, int32_t* pair_pos, int32_t* scratch,
                   umbs_stream_t stream);

/* X_next = x + (mix + (sum_k sel_w[t,k] pair_out[pair_pos[t,k]] + shared)); stores it at stack[layer + 1] and writes
 * x_out = sum_j depth_w[j] stack[j] (j <= layer + 1), or X_next itself when depth_w is NULL.  All fp32 [n, width];
 * stack: [n_layers + 1, n, width].  pair_out / shared may be NULL. */
int umbs_depth_mix(const float* x, const float* mix, const float* pair_out, const float* sel_w, const int32_t* pair_pos,
                   int top, const float* shared, float* stack, int layer, const float* depth_w, float* x_out,
                   float* copy_out, int n, int width, umbs_stream_t stream);

int umbs_embedding(int dtype, const int32_t* ids, const void* table, float* y, int n, int width, umbs_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
