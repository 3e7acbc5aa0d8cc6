// ref_layer_shim.cu — drives the reference's own single-token layer (`ds4_forward_layer`,
// cuda/forward_layer.cu) and the matvec / attention launchers it calls, over synthetic weights.
// TEST INFRASTRUCTURE ONLY: compiled together with the reference's sources (where they lie in the
// reference tree) into oracle/_ref/libds4ref.so by oracle/Makefile.  Nothing here is part of the
// product library.
//
// Three things live here:
//   * a tensor table over one device blob, so that `ds4_forward_layer` finds "blk.<il>.*" weights
//     without a GGUF file (the model struct's direct-pointer backend: base + offset);
//   * `extern "C"` names for the launchers a batched caller loops per token between the row stages
//     (attention, router, routed down-projection);
//   * the routed experts' gate / up dot products on their own.  The reference only has them fused
//     with the SwiGLU tail (cuda/moe_iq2_pair.cu:264-373), so a caller that keeps the tail as a
//     separate row stage needs the dots alone; this translation unit includes that source file to
//     use its IQ2_XXS tables and restates the per-lane sum with the same operation order.
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#include <cuda_runtime.h>

#include "moe_iq2_pair.cu"          // the reference's file, compiled in place (tables + fused launcher)

#include "ds4cuda.h"
#include "flash_attn.cuh"
#include "forward_layer.cuh"
#include "moe_q2k_sum6.cuh"
#include "router.cuh"

#define S(s) static_cast<cudaStream_t>(s)

namespace ds4cuda {

// One warp per (row, slot): lane l takes the 32-weight groups l, l+32, ... of the row, as the fused
// kernel does, so the per-lane partial sums and the butterfly see the same values in the same order.
__global__ void test_iq2_pair_dots_kernel(const block_iq2_xxs *__restrict__ w_gate,
                                          const block_iq2_xxs *__restrict__ w_up, const int8_t *__restrict__ xq,
                                          const float *__restrict__ xscale, const int32_t *__restrict__ ids,
                                          float *__restrict__ gate_out, float *__restrict__ up_out, int n_used,
                                          int out_dim, int n_blocks_in, int n_experts) {
    const int slot = blockIdx.y, row = blockIdx.x, lane = threadIdx.x;
    if (slot >= n_used || row >= out_dim) return;
    const int eid = ids[slot];
    if (eid < 0 || eid >= n_experts) return;
    const block_iq2_xxs *g_row = w_gate + ((size_t)eid * out_dim + row) * n_blocks_in;
    const block_iq2_xxs *u_row = w_up + ((size_t)eid * out_dim + row) * n_blocks_in;
    float total_g = 0.0f, total_u = 0.0f;
    for (int grp = lane; grp < n_blocks_in * 8; grp += 32) {
        const int blk = grp >> 3, part = grp & 7;
        const uint16_t *hg = g_row[blk].qs + 4 * part, *hu = u_row[blk].qs + 4 * part;
        const uint32_t idx_g = (uint32_t)hg[0] | ((uint32_t)hg[1] << 16), sgn_g = (uint32_t)hg[2] | ((uint32_t)hg[3] << 16);
        const uint32_t idx_u = (uint32_t)hu[0] | ((uint32_t)hu[1] << 16), sgn_u = (uint32_t)hu[2] | ((uint32_t)hu[3] << 16);
        const int8_t *y = xq + (size_t)blk * 256 + part * 32;
        int isum_g = 0, isum_u = 0;
        for (int o = 0; o < 4; ++o) {
            const uint8_t *vg = (const uint8_t *)(c_pair_grid + ((idx_g >> (8 * o)) & 0xff));
            const uint8_t *vu = (const uint8_t *)(c_pair_grid + ((idx_u >> (8 * o)) & 0xff));
            const uint8_t neg_g = c_pair_ksigns[(sgn_g >> (7 * o)) & 0x7f], neg_u = c_pair_ksigns[(sgn_u >> (7 * o)) & 0x7f];
            for (int j = 0; j < 8; ++j) {
                const int yj = (int)y[8 * o + j];
                isum_g += ((neg_g >> j) & 1 ? -(int)vg[j] : (int)vg[j]) * yj;
                isum_u += ((neg_u >> j) & 1 ? -(int)vu[j] : (int)vu[j]) * yj;
            }
        }
        const float yd = xscale[blk];
        const float ls_g = 0.5f + (float)(sgn_g >> 28), ls_u = 0.5f + (float)(sgn_u >> 28);
        const float dg = fp16_bits_to_fp32(g_row[blk].d) * yd, du = fp16_bits_to_fp32(u_row[blk].d) * yd;
        total_g += dg * (ls_g * (float)isum_g);
        total_u += du * (ls_u * (float)isum_u);
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
        total_g += __shfl_xor_sync(0xffffffff, total_g, offset);
        total_u += __shfl_xor_sync(0xffffffff, total_u, offset);
    }
    if (lane == 0) {
        gate_out[(size_t)slot * out_dim + row] = 0.25f * total_g;
        up_out[(size_t)slot * out_dim + row] = 0.25f * total_u;
    }
}

}  // namespace ds4cuda

using namespace ds4cuda;

namespace {
struct FakeModel {
    ds4_model m;
    std::vector<ds4_tensor> tensors;
    std::vector<std::string> names;
};
}  // namespace

extern "C" {

// A model whose tensor table names byte ranges of one device blob.
void *ds4ref_model_create(const char *const *names, const uint64_t *offsets, const uint64_t *sizes, int n_tensors,
                          void *dev_base, uint64_t total_bytes) {
    FakeModel *f = new FakeModel();
    std::memset(&f->m, 0, sizeof(f->m));
    f->names.assign(names, names + n_tensors);
    f->tensors.resize(n_tensors);
    for (int i = 0; i < n_tensors; ++i) {
        ds4_tensor &t = f->tensors[i];
        std::memset(&t, 0, sizeof(t));
        t.name = f->names[i].c_str();
        t.n_dims = 1;
        t.dims[0] = sizes[i];
        t.abs_offset = offsets[i];
        t.byte_size = sizes[i];
    }
    f->m.fd = -1;
    f->m.mmap_ptr = dev_base;
    f->m.file_size = total_bytes;
    f->m.tensors = f->tensors.data();
    f->m.n_tensors = (size_t)n_tensors;
    ds4_model_set_weight_backend(&f->m, DS4_WEIGHT_BACKEND_MMAP_DIRECT);
    return f;
}
void ds4ref_model_destroy(void *model) { delete static_cast<FakeModel *>(model); }

void *ds4ref_session_create(int max_context) {
    ds4_session_state *s = static_cast<ds4_session_state *>(std::calloc(1, sizeof(ds4_session_state)));
    if (s && ds4_session_state_alloc(s, max_context) != 0) {
        std::free(s);
        return nullptr;
    }
    return s;
}
void ds4ref_session_destroy(void *session) {
    if (!session) return;
    ds4_session_state_free(static_cast<ds4_session_state *>(session));
    std::free(session);
}
int ds4ref_session_n_raw(void *session, int il) { return static_cast<ds4_session_state *>(session)->layers[il].n_raw; }
const float *ds4ref_session_raw_kv(void *session, int il) {
    return static_cast<ds4_session_state *>(session)->layers[il].raw_kv;
}

const float *ds4ref_session_arena(void *session) { return static_cast<ds4_session_state *>(session)->activation_arena; }

// Copies out of session-owned memory into a caller's buffer (device to device, stream-ordered).
int ds4ref_copy_bytes(void *dst, const void *src, uint64_t n_bytes, void *s) {
    return (int)cudaMemcpyAsync(dst, src, n_bytes, cudaMemcpyDeviceToDevice, S(s));
}

// The reference's layer for ONE token, unmodified.
int ds4ref_forward_layer(void *model, void *session, int il, int token_id, int pos, const float *resid_in,
                         float *resid_out, void *s) {
    return ds4_forward_layer(&static_cast<FakeModel *>(model)->m, static_cast<ds4_session_state *>(session), il,
                             token_id, pos, resid_in, resid_out, S(s));
}

void ds4ref_flash_attn_decode_raw_f32(const float *q, const float *k, const float *v, const float *sinks, float *out,
                                      int n_head, int n_kv, int head_dim, void *s) {
    launch_flash_attn_decode_raw_f32(q, k, v, sinks, out, n_head, n_kv, head_dim, S(s));
}
void ds4ref_sqrt_softplus_f32(const float *x, float *y, int n, void *s) { launch_sqrt_softplus_f32(x, y, n, S(s)); }
void ds4ref_hash_router_topk_ids_i32(const int32_t *table, int token_id, int32_t *out, int k, void *s) {
    launch_hash_router_topk_ids_i32(table, token_id, out, k, S(s));
}
void ds4ref_hash_router_topk_w_f32(const float *probs, const int32_t *selected, float *w_out, int k, float scale,
                                   float sum_floor, void *s) {
    launch_hash_router_topk_w_f32(probs, selected, w_out, k, scale, sum_floor, S(s));
}
void ds4ref_routed_moe_pair_swiglu_full_f32_prealloc(const void *w_gate, const void *w_up, const float *x,
                                                     const int32_t *ids, const float *w, float *mid, int n_used,
                                                     int out_dim, int in_dim, int n_experts, float clamp, int8_t *xq,
                                                     float *xscale, int16_t *xbsums, void *s) {
    launch_routed_moe_pair_swiglu_full_f32_prealloc(static_cast<const block_iq2_xxs *>(w_gate),
                                                    static_cast<const block_iq2_xxs *>(w_up), x, ids, w, mid, n_used,
                                                    out_dim, in_dim, n_experts, clamp, xq, xscale, xbsums, S(s));
}
void ds4ref_routed_moe_q2k_sum6_full_f32_prealloc(const void *w_down, const float *mid, const int32_t *ids, float *out,
                                                  int n_used, int out_dim, int in_dim, int n_experts, int8_t *midq,
                                                  float *midscale, int16_t *midbsums, void *s) {
    launch_routed_moe_q2k_sum6_full_f32_prealloc(static_cast<const block_q2_K *>(w_down), mid, ids, out, n_used,
                                                 out_dim, in_dim, n_experts, midq, midscale, midbsums, S(s));
}

// Gate and up dot products of the selected experts for one token: the reference's Q8_K quantiser on
// x, then the dots with the fused kernel's operation order.
void ds4ref_test_iq2_pair_dots(const void *w_gate, const void *w_up, const float *x, const int32_t *ids, float *gate,
                               float *up, int n_used, int out_dim, int in_dim, int n_experts, int8_t *xq,
                               float *xscale, int16_t *xbsums, void *s) {
    const int nb = in_dim / 256;
    launch_quantize_fp32_to_q8_K(x, xq, xscale, xbsums, nb, S(s));
    test_iq2_pair_dots_kernel<<<dim3(out_dim, n_used, 1), 32, 0, S(s)>>>(
        static_cast<const block_iq2_xxs *>(w_gate), static_cast<const block_iq2_xxs *>(w_up), xq, xscale, ids, gate, up,
        n_used, out_dim, nb, n_experts);
}

}  // extern "C"
