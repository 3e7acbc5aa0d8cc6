/* ds4b200_path.h — the T-token prefill pass of the fused elementwise /
 * row-reduction path as one host-side object: it owns the device buffers, a
 * stream and (optionally) a CUDA graph of the per-layer launches, and replays
 * per layer the four fused ops the reference runs as ~20 single-token launches
 * (cuda/forward_layer.cu:808-1461, cuda/forward_token.cu:334-354):
 *
 *   gather   embedding gather (Q8_0 or F16) + residual add + RMSNorm
 *            -> f32 residual + bf16 normed            (ds4b200_embed_gather_rows)
 *   kvstore  tail YaRN RoPE + E4M3FN store into the layer's KV cache
 *                                                      (ds4b200_rope_fp8_store_rows)
 *   swiglu   clamped SwiGLU x router weight, summed over the top-k experts
 *                                                      (ds4b200_swiglu_rows_f32)
 *   hcmix    4x4 Sinkhorn (ds4b200_hc_sinkhorn_rows_f32, one thread per token,
 *            overlapped with the three kernels above) + mix of the 4
 *            hyper-connection streams                  (ds4b200_hc_post_rows_f32)
 *
 * It is the C/C++ host side the benchmark and the end-to-end tests drive; the
 * reference has no counterpart object (its cuda/forward_batch.cu:264-284 loops
 * one token at a time over cuda/forward_layer.cu).
 */
#ifndef DS4B200_PATH_H
#define DS4B200_PATH_H

#include "ds4b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ds4b200_path_config {
    int32_t n_tokens;        /* rows per call, e.g. 4096                       */
    int32_t n_embd;          /* 4096                                            */
    int32_t vocab;           /* 129280                                          */
    int32_t table_dtype;     /* DS4B200_TABLE_*                                 */
    int32_t kv_dim;          /* 512                                             */
    int32_t n_rot;           /* 64                                              */
    int32_t n_slots;         /* KV cache slots per layer, e.g. 65536            */
    int32_t ff_dim;          /* 2048                                            */
    int32_t top_k;           /* 6                                               */
    int32_t max_layers;      /* KV caches allocated, e.g. 43                    */
    int32_t sinkhorn_iters;  /* 20                                              */
    int32_t fp8_scale_mode;  /* DS4B200_FP8_*                                   */
    int32_t glu_mode;        /* DS4B200_GLU_*                                   */
    int32_t glu_fast_exp;    /* 0 / 1                                           */
    int32_t use_graph;       /* replay the layer chain from a CUDA graph        */
    float eps;               /* 1e-6                                            */
    float clamp;             /* 10                                              */
    ds4b200_rope_params rope;
} ds4b200_path_config;

/* Host pointers of one call.  NULL entries are skipped (the device copy keeps
 * its previous content).  Inputs: */
typedef struct ds4b200_path_io {
    const int32_t *ids;        /* [T]                 */
    const int32_t *pos;        /* [T], also the slot  */
    const float *residual;     /* [T][n_embd]         */
    const float *norm_w;       /* [n_embd]            */
    const float *kv;           /* [T][kv_dim]         */
    const float *gate;         /* [T][top_k][ff_dim]  */
    const float *up;           /* [T][top_k][ff_dim]  */
    const float *router_w;     /* [T][top_k]          */
    const float *hc_logits;    /* [T][16]             */
    const float *hc_resid;     /* [T][4][n_embd]      */
    /* outputs (of the last layer run): */
    float *residual_out;       /* [T][n_embd]         */
    uint16_t *normed_bf16;     /* [T][n_embd]         */
    uint8_t *kv_codes;         /* [T][kv_dim], the rows at slots pos[0..T)      */
    float *kv_scales;          /* [T][n_scales]       */
    float *kv_tail;            /* [T][n_rot] (BLOCK64_POW2 only)                */
    float *ffn_out;            /* [T][ff_dim]         */
    float *hc_out;             /* [T][4][n_embd]      */
} ds4b200_path_io;

typedef struct ds4b200_path ds4b200_path;

/* Kernels one layer launches: gather, kvstore, swiglu, hcmix and the Sinkhorn
 * rows that feed hcmix (run on a side stream beside the first three). */
#define DS4B200_PATH_N_KERNELS 5

/* Allocates every device buffer on the current device.  NULL on failure
 * (ds4b200_last_error() says why). */
ds4b200_path *ds4b200_path_create(const ds4b200_path_config *cfg);
void ds4b200_path_destroy(ds4b200_path *p);

/* The embedding table is a weight: uploaded once, not per call. */
int ds4b200_path_upload_table(ds4b200_path *p, const void *host_table, size_t bytes);
/* Range check of the index arrays of a host-side batch: every ids[t] in [0, vocab), every
 * pos[t] in [0, n_slots).  0, or -EINVAL with the first offending index in
 * ds4b200_last_error().  Needs no device.  ds4b200_path_upload, ds4b200_path_run_host and
 * ds4b200_path_run_host_chunked run the same check before their first copy or launch (the
 * kernels index the table and the cache with these values). */
int ds4b200_path_check_io(const ds4b200_path_config *cfg, const ds4b200_path_io *host);
/* Synchronous copy of every non-NULL input of `host` to the device. */
int ds4b200_path_upload(ds4b200_path *p, const ds4b200_path_io *host);
/* Device pointer and size of a named buffer ("table", "ids", "pos", "residual",
 * "norm_w", "kv", "gate", "up", "router_w", "hc_logits", "hc_a", "hc_b",
 * "residual_out", "normed_bf16", "kv_codes", "kv_scales", "kv_tail", "ffn_out"). */
void *ds4b200_path_buffer(ds4b200_path *p, const char *name, int64_t *bytes);
void *ds4b200_path_stream(ds4b200_path *p);

/* Enqueue n_layers replays of the four ops on the path's stream; no sync. */
int ds4b200_path_run_device(ds4b200_path *p, int n_layers);
/* One end-to-end call on host buffers: copy the non-NULL inputs in, run
 * n_layers, copy the non-NULL outputs out, wait.  *ms (nullable) receives the
 * device time of the whole call measured with events on the path's stream. */
int ds4b200_path_run_host(ds4b200_path *p, const ds4b200_path_io *host, int n_layers, float *ms);
/* The same end-to-end call with the token rows cut into n_chunks slices that are
 * pipelined over three streams: while slice k runs the layer chain, slice k+1 is
 * copied in and slice k-1 is copied out (PCIe is full duplex).  Every row is
 * independent, so results equal ds4b200_path_run_host.  Launches are issued
 * eagerly (no graph).  The pos/slot values of different slices must not collide. */
int ds4b200_path_run_host_chunked(ds4b200_path *p, const ds4b200_path_io *host, int n_layers,
                                  int n_chunks, float *ms);
/* Time `steps` back-to-back device runs after `warmup` untimed ones, with
 * events on the path's stream.  *ms_total = time of all timed steps. */
int ds4b200_path_time_device(ds4b200_path *p, int n_layers, int warmup, int steps, float *ms_total);
/* Average device time of one launch of each kernel, measured with events on
 * the path's stream around `reps` back-to-back launches of that kernel alone:
 * ms_per_launch[DS4B200_PATH_N_KERNELS] in the order gather, kvstore, swiglu,
 * hcmix, sinkhorn. */
int ds4b200_path_profile_ops(ds4b200_path *p, int reps, float *ms_per_launch);
/* Kernel launches one device run of n_layers enqueues. */
int ds4b200_path_launches_per_run(ds4b200_path *p, int n_layers);
/* Algorithmic HBM bytes of one launch of kernel i (0 gather, 1 kvstore,
 * 2 swiglu, 3 hcmix, 4 sinkhorn): every input row read once, every output row
 * written once. */
int64_t ds4b200_path_op_bytes(ds4b200_path *p, int op);

#ifdef __cplusplus
}
#endif
#endif /* DS4B200_PATH_H */
