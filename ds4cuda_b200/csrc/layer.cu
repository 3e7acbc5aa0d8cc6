// layer.cu — host side of ds4b200_layer_rows_f32: the row stages of one layer for a chunk of
// tokens, one launch per stage, with the caller's matvec / attention stages run through a
// hook at the points where ds4_forward_layer calls them (cuda/forward_layer.cu:808-1461).
// Pure sequencing: every stage is one of the batched kernels of this library.
#include <cerrno>

#include "../../include/ds4b200_layer.h"
#include "kernels.cuh"

using ds4b200::set_error;

namespace {

int launch_ok(const char *what) {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : set_error(-EIO, "layer_rows: %s: %s", what, cudaGetErrorString(e));
}

}  // namespace

extern "C" int ds4b200_layer_rows_f32(const ds4b200_layer_dims *d, const ds4b200_layer_weights *w,
                                      const ds4b200_layer_buffers *b, const float *resid_in, const int32_t *pos,
                                      int64_t T, float *resid_out, ds4b200_stage_hook hook, void *user,
                                      void *stream) {
    if (!d || !w || !b || !resid_in || !pos || !resid_out || !hook)
        return set_error(-EINVAL, "layer_rows: null argument");
    if (T <= 0) return T == 0 ? 0 : set_error(-EINVAL, "layer_rows: negative token count");
    if (d->n_embd <= 0 || d->n_embd % 32 || d->n_embd > 8192 || d->n_heads <= 0 || d->head_dim <= 0 ||
        d->head_dim % 4 || d->head_dim > 1024 || d->n_rot <= 0 || d->n_rot % 64 || (d->head_dim - d->n_rot) % 64 ||
        d->q_lora <= 0 || d->ff_dim <= 0 || d->ff_dim % 256 || d->top_k <= 0 || d->sinkhorn_iters <= 0)
        return set_error(-EINVAL, "layer_rows: unsupported geometry");
    const void *need[] = {w->hc_attn_fn, w->hc_attn_scale, w->hc_attn_base, w->attn_norm, w->q_a_norm, w->kv_a_norm,
                          w->hc_ffn_fn, w->hc_ffn_scale, w->hc_ffn_base, w->ffn_norm, b->x, b->x_norm, b->xq,
                          b->xscale, b->q_lora, b->q_lora_norm, b->kv_raw, b->raw_rows, b->q, b->kqv, b->attn_out,
                          b->post, b->comb, b->resid_mid, b->sh_gate, b->sh_up, b->sh_mid, b->gate, b->up,
                          b->router_w, b->mid_q, b->mid_scale, b->mid_bsums, b->moe_out, b->shexp_out};
    for (const void *p : need)
        if (!p) return set_error(-EINVAL, "layer_rows: null weight or buffer");
    if (!b->kqv_q != !b->kqv_scale) return set_error(-EINVAL, "layer_rows: kqv_q and kqv_scale go together");
    if (b->kqv_q && (d->head_dim % 32 || (reinterpret_cast<uintptr_t>(b->kqv) & 15u) ||
                     (reinterpret_cast<uintptr_t>(b->kqv_q) & 3u)))
        return set_error(-EINVAL, "layer_rows: the Q8_0 form of the inverse RoPE needs head_dim % 32 == 0 and aligned rows");

    if (!b->ffn_kq != !b->ffn_kscale || !b->ffn_kq != !b->ffn_kbsums)
        return set_error(-EINVAL, "layer_rows: ffn_kq, ffn_kscale and ffn_kbsums go together");
    if (b->ffn_kq && (d->n_embd % 256 || (reinterpret_cast<uintptr_t>(b->ffn_kq) & 3u) ||
                      (reinterpret_cast<uintptr_t>(b->x) & 15u) || (reinterpret_cast<uintptr_t>(b->x_norm) & 15u) ||
                      (reinterpret_cast<uintptr_t>(w->ffn_norm) & 15u)))
        return set_error(-EINVAL, "layer_rows: the Q8_K form of the ffn norm needs n_embd % 256 == 0 and aligned rows");

    if (!b->sh_q != !b->sh_scale) return set_error(-EINVAL, "layer_rows: sh_q and sh_scale go together");
    if (b->sh_q && (d->ff_dim % 32 || (reinterpret_cast<uintptr_t>(b->sh_q) & 3u) ||
                    (reinterpret_cast<uintptr_t>(b->sh_gate) & 15u) || (reinterpret_cast<uintptr_t>(b->sh_up) & 15u)))
        return set_error(-EINVAL, "layer_rows: the Q8_0 form of the shared expert's rows needs aligned rows");

    auto misaligned = [](const void *p, uintptr_t mask) { return (reinterpret_cast<uintptr_t>(p) & mask) != 0; };
    // the norms that leave Q8_0 blocks run as the vector kernels only: rows and gains on 16 bytes
    if (misaligned(b->x, 15) || misaligned(b->x_norm, 15) || misaligned(w->attn_norm, 15) || misaligned(w->ffn_norm, 15) ||
        misaligned(b->xq, 3))
        return set_error(-EINVAL, "layer_rows: x, x_norm and the norm gains need 16-byte alignment, xq 4-byte");
    if (!b->ql_q != !b->ql_scale) return set_error(-EINVAL, "layer_rows: ql_q and ql_scale go together");
    if (b->ql_q && (d->q_lora % 32 || d->q_lora > 8192 || misaligned(b->ql_q, 3) || misaligned(b->q_lora, 15) ||
                    misaligned(b->q_lora_norm, 15) || misaligned(w->q_a_norm, 15)))
        return set_error(-EINVAL, "layer_rows: the Q8_0 form of the q_a norm needs q_lora % 32 == 0 and aligned rows");

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int n = d->n_embd, hd = d->head_dim;
    ds4b200_rope_params rope;
    ds4b200_rope_params_for_layer(d->il, d->n_rot, &rope);
    auto call = [&](int stage) {
        const int rc = hook(user, stage, T, stream);
        return rc ? set_error(rc, "layer_rows: hook stage %d returned %d", stage, rc) : 0;
    };
    int rc;
    // the chunk's angle table: written by the KV row chain below (one KV row per token evaluates exactly the
    // table's entries), read by the two head-row RoPE stages after it
    const float *cs = (b->rope_cs && d->n_rot <= 64) ? b->rope_cs : nullptr;

    // ---- attention half
    ds4b200::hc_pre_rows(resid_in, w->hc_attn_fn, w->hc_attn_scale, w->hc_attn_base, b->post, b->comb, b->x, T, n,
                         d->sinkhorn_iters, d->eps, s);
    ds4b200::rms_norm_rows(b->x, nullptr, w->attn_norm, n, b->x_norm, nullptr, nullptr, T, n, d->eps, s, b->xq,
                           b->xscale);
    if ((rc = launch_ok("hc attn pre / attn norm"))) return rc;
    if ((rc = call(DS4B200_STAGE_QKV_A))) return rc;
    ds4b200::rms_norm_rows(b->q_lora, nullptr, w->q_a_norm, d->q_lora, b->q_lora_norm, nullptr, nullptr, T, d->q_lora,
                           d->eps, s, b->ql_q, b->ql_scale);
    ds4b200::rope_fp8_store_rows(b->kv_raw, T, hd, d->n_rot, pos, &rope, w->kv_a_norm, d->eps,
                                 DS4B200_FP8_BLOCK64_POW2, nullptr, nullptr, nullptr, nullptr, nullptr, s,
                                 b->raw_rows, nullptr, cs ? b->rope_cs : nullptr);
    if ((rc = launch_ok("q_a norm / kv chain"))) return rc;
    if ((rc = call(DS4B200_STAGE_Q_B))) return rc;
    ds4b200::rope_rows(b->q, b->q, T, d->n_heads, hd, d->n_rot, pos, 0, rope, 0, 1, d->eps, s, nullptr, nullptr, cs);
    if ((rc = launch_ok("q norm + RoPE"))) return rc;
    if ((rc = call(DS4B200_STAGE_ATTENTION))) return rc;
    if (b->kqv_q)      // rotated rows straight into the out-projection's activation blocks, no f32 round trip
        ds4b200::rope_rows(b->kqv, nullptr, T, d->n_heads, hd, d->n_rot, pos, 0, rope, 1, 0, d->eps, s, b->kqv_q,
                           b->kqv_scale, cs);
    else
        ds4b200::rope_rows(b->kqv, b->kqv, T, d->n_heads, hd, d->n_rot, pos, 0, rope, 1, 0, d->eps, s, nullptr,
                           nullptr, cs);
    if ((rc = launch_ok("inverse RoPE"))) return rc;
    if ((rc = call(DS4B200_STAGE_ATTN_OUT))) return rc;
    ds4b200::hc_post_rows(b->attn_out, nullptr, resid_in, b->post, b->comb, nullptr, nullptr, b->resid_mid, T, n, 0,
                          0.0f, s);

    // ---- feed-forward half
    ds4b200::hc_pre_rows(b->resid_mid, w->hc_ffn_fn, w->hc_ffn_scale, w->hc_ffn_base, b->post, b->comb, b->x, T, n,
                         d->sinkhorn_iters, d->eps, s);
    ds4b200::rms_norm_rows(b->x, nullptr, w->ffn_norm, n, b->x_norm, nullptr, nullptr, T, n, d->eps, s, b->xq,
                           b->xscale, b->ffn_kq, b->ffn_kscale, b->ffn_kbsums);
    if ((rc = launch_ok("hc attn post / hc ffn pre / ffn norm"))) return rc;
    if ((rc = call(DS4B200_STAGE_FFN_UP))) return rc;
    if (b->sh_q)       // straight into the shared down projection's activation blocks
        ds4b200::swiglu_q8_0_rows(b->sh_gate, b->sh_up, nullptr, b->sh_q, b->sh_scale, nullptr, T, d->ff_dim,
                                  DS4B200_GLU_PLAIN, 0.0f, 0, s);
    else
        ds4b200::swiglu_rows(b->sh_gate, b->sh_up, nullptr, b->sh_mid, T, 1, d->ff_dim, DS4B200_GLU_PLAIN, 0.0f, 0, 0, s);
    ds4b200::swiglu_q8_K_rows(b->gate, b->up, b->router_w, b->mid_q, b->mid_scale, b->mid_bsums, nullptr,
                              T * d->top_k, d->ff_dim, DS4B200_GLU_CLAMP_REF, d->clamp, d->glu_fast_exp, s);
    if ((rc = launch_ok("shared silu / routed epilogue"))) return rc;
    if ((rc = call(DS4B200_STAGE_FFN_DOWN))) return rc;
    ds4b200::hc_post_rows(b->moe_out, b->shexp_out, b->resid_mid, b->post, b->comb, nullptr, nullptr, resid_out, T, n,
                          0, 0.0f, s);
    return launch_ok("add + hc ffn post");
}

namespace {

struct ChunkHook {
    ds4b200_chunk_hook hook;
    void *user;
    int il;
};

int chunk_stage(void *user, int stage, int64_t n_tokens, void *stream) {
    const ChunkHook *c = static_cast<const ChunkHook *>(user);
    return c->hook(c->user, c->il, stage, n_tokens, stream);
}

}  // namespace

extern "C" int ds4b200_chunk_rows_f32(const ds4b200_layer_dims *dims, const ds4b200_layer_weights *weights,
                                      int n_layers, int first_layer, const ds4b200_layer_buffers *b, float *resid_a,
                                      float *resid_b, const int32_t *pos, int64_t T, ds4b200_chunk_hook hook,
                                      void *user, void *stream, float **resid_final) {
    if (!dims || !weights || !b || !resid_a || !resid_b || !pos || !hook)
        return set_error(-EINVAL, "chunk_rows: null argument");
    if (n_layers < 0 || first_layer < 0) return set_error(-EINVAL, "chunk_rows: negative layer count or index");
    if (resid_a == resid_b) return set_error(-EINVAL, "chunk_rows: resid_a and resid_b are the same buffer");
    if (T < 0) return set_error(-EINVAL, "chunk_rows: negative token count");
    float *cur = resid_a, *next = resid_b;
    for (int i = 0; i < n_layers && T > 0; ++i) {
        ds4b200_layer_dims d = *dims;
        d.il = first_layer + i;
        ChunkHook c{hook, user, d.il};
        const int rc = ds4b200_layer_rows_f32(&d, &weights[i], b, cur, pos, T, next, chunk_stage, &c, stream);
        if (rc) return rc;
        float *t = cur; cur = next; next = t;
    }
    if (resid_final) *resid_final = cur;
    return 0;
}
