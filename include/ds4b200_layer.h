/* ds4b200_layer.h — the row stages of one transformer layer for a chunk of T tokens, in the
 * order ds4_forward_layer runs them for one token (cuda/forward_layer.cu:808-1461), each as
 * ONE launch over the whole chunk.  This is the batched counterpart of the inner loop of
 * ds4_forward_chunk (cuda/forward_batch.cu:264-284), restricted to what this library
 * implements: the matvec and attention stages between the row stages stay with the caller
 * and run through a hook, which is called at the six points where the reference calls them.
 * No reference counterpart exists for this entry point (the reference has no batched layer).
 *
 * Sequence (hook stages in capitals; buffers named as in ds4b200_layer_buffers):
 *   hc attn pre        resid_in -> x, post, comb                       (:808)
 *   attn norm + Q8_0   x -> x_norm, xq, xscale                        (:822, dense_q8.cu:122)
 *   QKV_A              caller: x_norm / xq -> q_lora, kv_raw           (:833, :856)
 *   q_a norm           q_lora -> q_lora_norm (+ ql_q, ql_scale: Q8_0)  (:845)
 *   kv chain           kv_raw -> raw_rows (norm, RoPE, FP8, f16)       (:868, :910, :921, :950)
 *   Q_B                caller: q_lora_norm -> q                        (:879)
 *   q norm + RoPE      q in place                                      (:890, :901)
 *   ATTENTION          caller: q, raw_rows, caches -> kqv              (:997-1166)
 *   inverse RoPE       kqv in place, or -> kqv_q, kqv_scale (Q8_0)     (:1179)
 *   ATTN_OUT           caller: kqv -> attn_out                         (:1190, :1205)
 *   hc attn post       attn_out, resid_in, post, comb -> resid_mid     (:1217)
 *   hc ffn pre         resid_mid -> x, post, comb                      (:1235)
 *   ffn norm + Q8_0    x -> x_norm, xq, xscale (+ ffn_kq...: Q8_K)    (:1249, moe_iq2_pair.cu:404)
 *   FFN_UP             caller: x_norm / xq -> sh_gate, sh_up, gate, up, router_w   (:1260-1350)
 *   shared silu*up     sh_gate, sh_up -> sh_mid, or -> sh_q, sh_scale (Q8_0)       (:1285)
 *   routed epilogue    gate, up, router_w -> mid_q, mid_scale, mid_bsums (Q8_K)    (moe_iq2_pair.cu:352, :159)
 *   FFN_DOWN           caller: sh_mid, mid_q... -> shexp_out, moe_out  (:1296, :1416)
 *   add + hc ffn post  moe_out + shexp_out, resid_mid, post, comb -> resid_out     (:1447, :1456)
 */
#ifndef DS4B200_LAYER_H
#define DS4B200_LAYER_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    DS4B200_STAGE_QKV_A = 0,
    DS4B200_STAGE_Q_B = 1,
    DS4B200_STAGE_ATTENTION = 2,
    DS4B200_STAGE_ATTN_OUT = 3,
    DS4B200_STAGE_FFN_UP = 4,
    DS4B200_STAGE_FFN_DOWN = 5
};

typedef struct ds4b200_layer_dims {
    int n_embd;          /* 4096 */
    int n_heads;         /* 64 */
    int head_dim;        /* 512 */
    int n_rot;           /* 64 */
    int q_lora;          /* 1024 */
    int ff_dim;          /* 2048 */
    int top_k;           /* 6 */
    int sinkhorn_iters;  /* 20 */
    int il;              /* layer index: selects the RoPE parameters (cuda/rope.cu:214-250) */
    int glu_fast_exp;    /* 1: the reference epilogue's hardware exp */
    float eps;           /* 1e-6 */
    float clamp;         /* 10 */
} ds4b200_layer_dims;

typedef struct ds4b200_layer_weights {      /* device pointers */
    const uint16_t *hc_attn_fn;             /* f16 [24][4*n_embd] */
    const float *hc_attn_scale, *hc_attn_base;      /* [3], [24] */
    const float *attn_norm, *q_a_norm, *kv_a_norm;  /* [n_embd], [q_lora], [head_dim] */
    const uint16_t *hc_ffn_fn;
    const float *hc_ffn_scale, *hc_ffn_base;
    const float *ffn_norm;                  /* [n_embd] */
} ds4b200_layer_weights;

typedef struct ds4b200_layer_buffers {      /* caller-owned device workspace for T tokens */
    float *x, *x_norm;                      /* [T][n_embd] */
    int8_t *xq;                             /* [T][n_embd] */
    float *xscale;                          /* [T][n_embd/32] */
    float *q_lora, *q_lora_norm;            /* [T][q_lora] */
    float *kv_raw, *raw_rows;               /* [T][head_dim] */
    float *q, *kqv;                         /* [T][n_heads][head_dim] */
    float *attn_out;                        /* [T][n_embd] */
    float *post, *comb;                     /* [T][4], [T][16] */
    float *resid_mid;                       /* [T][4][n_embd] */
    float *sh_gate, *sh_up, *sh_mid;        /* [T][ff_dim] */
    float *gate, *up;                       /* [T][top_k][ff_dim] */
    float *router_w;                        /* [T][top_k] */
    int8_t *mid_q;                          /* [T][top_k][ff_dim] */
    float *mid_scale;                       /* [T][top_k][ff_dim/256] */
    int16_t *mid_bsums;                     /* [T][top_k][ff_dim/256][16] */
    float *moe_out, *shexp_out;             /* [T][n_embd] */
    /* Optional (both or neither): when given, the inverse RoPE leaves its rows as the Q8_0 blocks
     * the grouped out-projection quantises them to (cuda/attn_out.cu:119-145) and kqv is NOT
     * rewritten: ATTN_OUT then reads kqv_q / kqv_scale instead of rotated f32 rows. */
    int8_t *kqv_q;                          /* [T][n_heads][head_dim] */
    float *kqv_scale;                       /* [T][n_heads][head_dim/32] */
    /* Optional: room for the chunk's RoPE angle table (the entries ds4b200_rope_table_rows writes).
     * When given, the KV row chain, which evaluates a token's 32 angles anyway, leaves them here, and
     * the two head-row RoPE stages behind it read them instead of evaluating 32 cos / sin pairs per
     * head row; the rotated rows keep their bits. */
    float *rope_cs;                         /* [T][n_rot/2][2] */
    /* Optional (all three or none; n_embd % 256 == 0): the feed-forward norm also leaves its row as the
     * Q8_K blocks the routed experts' IQ2_XXS gate / up dots read (cuda/moe_iq2_pair.cu:404-421 quantises
     * the row inside that launcher), so FFN_UP needs no quantiser launch of its own. */
    int8_t *ffn_kq;                         /* [T][n_embd] */
    float *ffn_kscale;                      /* [T][n_embd/256] */
    int16_t *ffn_kbsums;                    /* [T][n_embd/256][16] */
    /* Optional (both or neither; ff_dim % 32 == 0): the shared expert's silu(gate) * up leaves as the Q8_0
     * blocks its down projection quantises the row to (cuda/forward_layer.cu:1296, then the quantiser
     * inside the Q8_0 matvec, cuda/dense_q8.cu:122-152) and sh_mid is NOT written. */
    int8_t *sh_q;                           /* [T][ff_dim] */
    float *sh_scale;                        /* [T][ff_dim/32] */
    /* Optional (both or neither; q_lora % 32 == 0): the q_a norm also leaves its row as the Q8_0 blocks
     * the q_b projection quantises it to (cuda/forward_layer.cu:879 through cuda/dense_q8.cu:122-152). */
    int8_t *ql_q;                           /* [T][q_lora] */
    float *ql_scale;                        /* [T][q_lora/32] */
} ds4b200_layer_buffers;

/* Called on the issuing thread between row stages; must enqueue its work on `stream` (or
 * order it with that stream) and return 0.  A non-zero return aborts the layer with that code. */
typedef int (*ds4b200_stage_hook)(void *user, int stage, int64_t n_tokens, void *stream);

/* Enqueues the whole sequence on `stream`.  Nothing is allocated or synchronised.  Returns 0,
 * -EINVAL for a bad argument, -EIO for a launch error, or the hook's own non-zero code. */
int ds4b200_layer_rows_f32(const ds4b200_layer_dims *dims, const ds4b200_layer_weights *w,
                           const ds4b200_layer_buffers *b, const float *resid_in, const int32_t *pos,
                           int64_t n_tokens, float *resid_out, ds4b200_stage_hook hook, void *user,
                           void *stream);

/* The layers of a chunk: the batched counterpart of the layer loop of ds4_forward_chunk
 * (cuda/forward_batch.cu:264-284 run for all T tokens at once instead of token by token).  Layers
 * first_layer .. first_layer + n_layers - 1 run in turn through ds4b200_layer_rows_f32 with weights[i]
 * (an array of n_layers entries) and the RoPE parameters of their index (dims->il is ignored); the
 * residual streams alternate between resid_a (holding the chunk's streams on entry) and resid_b, as the
 * reference's HC ping / pong buffers do (cuda/session_state.cu:12-19).  *resid_final (host, nullable)
 * receives the buffer that holds the streams after the last layer.  The hook gets the layer index. */
typedef int (*ds4b200_chunk_hook)(void *user, int il, int stage, int64_t n_tokens, void *stream);

int ds4b200_chunk_rows_f32(const ds4b200_layer_dims *dims, const ds4b200_layer_weights *weights, int n_layers,
                           int first_layer, const ds4b200_layer_buffers *b, float *resid_a, float *resid_b,
                           const int32_t *pos, int64_t n_tokens, ds4b200_chunk_hook hook, void *user, void *stream,
                           float **resid_final);

#ifdef __cplusplus
}
#endif
#endif /* DS4B200_LAYER_H */
