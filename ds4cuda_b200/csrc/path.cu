// path.cu — host side of the T-token prefill pass (see include/ds4b200_path.h):
// device buffers, one stream, an optional CUDA graph of the per-layer launch
// chain, host-buffer entry point with the copies inside, and event timing.
#include <cerrno>
#include <cstring>
#include <map>
#include <tuple>
#include <string>
#include <vector>

#include "../../include/ds4b200_path.h"
#include "kernels.cuh"

using ds4b200::set_error;

struct ds4b200_path {
    ds4b200_path_config cfg{};
    cudaStream_t stream = nullptr;
    int device = 0;
    std::map<std::string, std::pair<void *, int64_t>> buf;   // name -> (device ptr, bytes)
    std::vector<void *> owned;
    int n_scales = 1;
    // typed views
    void *table = nullptr;
    int32_t *ids = nullptr, *pos = nullptr;
    float *residual = nullptr, *norm_w = nullptr, *kv = nullptr, *gate = nullptr, *up = nullptr;
    float *router_w = nullptr, *hc_logits = nullptr, *hc_a = nullptr, *hc_b = nullptr;
    float *residual_out = nullptr, *kv_scales = nullptr, *kv_tail = nullptr, *ffn_out = nullptr;
    uint16_t *normed_bf16 = nullptr;
    uint8_t *kv_codes = nullptr;
    float *comb = nullptr;             // [T][16] Sinkhorn matrices of the layer in flight
    float *gather_scratch = nullptr;   // [T][kv_dim] rows gathered from the cache for D2H
    cudaStream_t side = nullptr;       // the Sinkhorn rows run here, beside the other ops
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    cudaStream_t copy_in = nullptr, copy_out = nullptr;   // chunked host calls: H2D / D2H beside compute
    std::vector<cudaEvent_t> chunk_events;
    // graph cache (one per layer count)
    std::map<int, cudaGraphExec_t> graphs;
    // per row slice of the chunked host entry point: (first row, rows, layers) -> its layer chain
    std::map<std::tuple<int64_t, int64_t, int>, cudaGraphExec_t> slice_graphs;
    std::vector<cudaEvent_t> events;
};

namespace {

#define CUDA_OK(call, what)                                                            \
    do {                                                                               \
        const cudaError_t e_ = (call);                                                 \
        if (e_ != cudaSuccess) return set_error(-EIO, "%s: %s", what, cudaGetErrorString(e_)); \
    } while (0)

template <typename T>
bool alloc(ds4b200_path *p, const char *name, T *&ptr, int64_t bytes) {
    void *d = nullptr;
    if (cudaMalloc(&d, (size_t)bytes) != cudaSuccess) {
        set_error(-ENOMEM, "path_create: cudaMalloc(%s, %lld bytes) failed", name, (long long)bytes);
        return false;
    }
    p->owned.push_back(d);
    p->buf[name] = {d, bytes};
    ptr = static_cast<T *>(d);
    return true;
}

int64_t table_bytes(const ds4b200_path_config &c) {
    const int64_t row = c.table_dtype == DS4B200_TABLE_Q8_0 ? (int64_t)(c.n_embd / 32) * 34
                                                            : (int64_t)c.n_embd * 2;
    return row * c.vocab;
}

// gather the T freshly written cache rows (slot = pos[t]) into a dense buffer
__global__ void gather_rows_kernel(const uint8_t *src, const int32_t *slots, uint8_t *dst,
                                   int row_bytes, int64_t n_rows) {
    const int64_t r = blockIdx.x;
    if (r >= n_rows) return;
    const uint8_t *s = src + (int64_t)slots[r] * row_bytes;
    for (int i = threadIdx.x; i < row_bytes; i += blockDim.x) dst[r * row_bytes + i] = s[i];
}

float *hc_in(ds4b200_path *p, int layer) { return (layer & 1) ? p->hc_b : p->hc_a; }
float *hc_out(ds4b200_path *p, int layer) { return (layer & 1) ? p->hc_a : p->hc_b; }

// The launches of one layer.  `op` < 0 runs all of them, with the Sinkhorn rows
// (which depend only on the logits) and the KV store (10 MB, launch-bound) forked
// onto the side stream so that they overlap the streaming kernels before the mix.
// `op` >= 0 runs one kernel alone on the main stream (profiling).
void enqueue_layer(ds4b200_path *p, int layer, int op, int64_t t0 = 0, int64_t n = -1) {
    const ds4b200_path_config &c = p->cfg;
    const int64_t T = n < 0 ? c.n_tokens : n;          // rows [t0, t0 + T)
    cudaStream_t s = p->stream;
    const int64_t E = c.n_embd;
    float *comb = p->comb + t0 * 16;
    const float *logits = p->hc_logits + t0 * 16;
    auto kvstore = [&](cudaStream_t st) {
        const int64_t l = layer % c.max_layers;
        ds4b200::rope_fp8_store_rows(p->kv + t0 * c.kv_dim, T, c.kv_dim, c.n_rot, p->pos + t0, &c.rope, nullptr,
                                     c.eps, c.fp8_scale_mode, p->pos + t0,
                                     p->kv_codes + l * (int64_t)c.n_slots * c.kv_dim,
                                     p->kv_scales + l * (int64_t)c.n_slots * p->n_scales,
                                     p->kv_tail ? p->kv_tail + l * (int64_t)c.n_slots * c.n_rot : nullptr,
                                     nullptr, st);
    };
    if (op < 0) {
        // side stream: the two small latency-bound kernels (Sinkhorn rows, KV store); they
        // share no buffer with the streaming kernels on the main stream
        cudaEventRecord(p->ev_fork, s);
        cudaStreamWaitEvent(p->side, p->ev_fork, 0);
        ds4b200::hc_sinkhorn_rows(logits, comb, T, c.sinkhorn_iters, c.eps, p->side);
        kvstore(p->side);
        cudaEventRecord(p->ev_join, p->side);
    }
    if (op == 4) ds4b200::hc_sinkhorn_rows(logits, comb, T, c.sinkhorn_iters, c.eps, s);
    if (op == 1) kvstore(s);
    if (op < 0 || op == 0)
        ds4b200::embed_gather_rows(p->table, c.table_dtype, p->ids + t0, 0, T, c.n_embd, p->residual + t0 * E,
                                   p->norm_w, c.eps, p->residual_out + t0 * E, 1, nullptr,
                                   p->normed_bf16 + t0 * E, s);
    if (op < 0 || op == 2)
        ds4b200::swiglu_rows(p->gate + t0 * c.top_k * c.ff_dim, p->up + t0 * c.top_k * c.ff_dim,
                             p->router_w + t0 * c.top_k, p->ffn_out + t0 * c.ff_dim, T, c.top_k, c.ff_dim,
                             c.glu_mode, c.clamp, 1, c.glu_fast_exp, s);
    if (op < 0) cudaStreamWaitEvent(s, p->ev_join, 0);
    if (op < 0 || op == 3)
        ds4b200::hc_post_rows(nullptr, nullptr, hc_in(p, layer) + t0 * 4 * E, nullptr, comb, nullptr, nullptr,
                              hc_out(p, layer) + t0 * 4 * E, T, c.n_embd, 0, 0.0f, s);
}

int enqueue_run(ds4b200_path *p, int n_layers) {
    if (!p->cfg.use_graph) {
        for (int l = 0; l < n_layers; ++l) enqueue_layer(p, l, -1);
        CUDA_OK(cudaGetLastError(), "path_run: launch");
        return 0;
    }
    auto it = p->graphs.find(n_layers);
    if (it == p->graphs.end()) {
        cudaGraph_t g = nullptr;
        cudaGraphExec_t ge = nullptr;
        CUDA_OK(cudaStreamBeginCapture(p->stream, cudaStreamCaptureModeThreadLocal), "path_run: begin capture");
        for (int l = 0; l < n_layers; ++l) enqueue_layer(p, l, -1);
        CUDA_OK(cudaStreamEndCapture(p->stream, &g), "path_run: end capture");
        CUDA_OK(cudaGraphInstantiate(&ge, g, 0), "path_run: graph instantiate");
        cudaGraphDestroy(g);
        it = p->graphs.emplace(n_layers, ge).first;
    }
    CUDA_OK(cudaGraphLaunch(it->second, p->stream), "path_run: graph launch");
    return 0;
}

int ensure_events(ds4b200_path *p, size_t n) {
    while (p->events.size() < n) {
        cudaEvent_t e;
        CUDA_OK(cudaEventCreate(&e), "cudaEventCreate");
        p->events.push_back(e);
    }
    return 0;
}

struct Copy { void *dev; const void *host; int64_t bytes; };

std::vector<Copy> input_copies(ds4b200_path *p, const ds4b200_path_io *h) {
    const ds4b200_path_config &c = p->cfg;
    const int64_t T = c.n_tokens;
    return {
        {p->ids, h->ids, T * 4},
        {p->pos, h->pos, T * 4},
        {p->residual, h->residual, T * c.n_embd * 4},
        {p->norm_w, h->norm_w, (int64_t)c.n_embd * 4},
        {p->kv, h->kv, T * c.kv_dim * 4},
        {p->gate, h->gate, T * c.top_k * c.ff_dim * 4},
        {p->up, h->up, T * c.top_k * c.ff_dim * 4},
        {p->router_w, h->router_w, T * c.top_k * 4},
        {p->hc_logits, h->hc_logits, T * 16 * 4},
        {p->hc_a, h->hc_resid, T * 4 * c.n_embd * 4},
    };
}

// The token ids and positions of a host-side batch index device memory (table rows, cache
// slots), so they are range-checked here, while they are still in host memory.
int check_host_indices(const ds4b200_path_config &c, const ds4b200_path_io *h, const char *who) {
    if (h->ids)
        for (int64_t t = 0; t < c.n_tokens; ++t)
            if (h->ids[t] < 0 || h->ids[t] >= c.vocab)
                return set_error(-EINVAL, "%s: ids[%lld] = %d is outside [0, %d)", who, (long long)t, (int)h->ids[t],
                                 (int)c.vocab);
    if (h->pos)
        for (int64_t t = 0; t < c.n_tokens; ++t)
            if (h->pos[t] < 0 || h->pos[t] >= c.n_slots)
                return set_error(-EINVAL, "%s: pos[%lld] = %d is outside [0, %d)", who, (long long)t, (int)h->pos[t],
                                 (int)c.n_slots);
    return 0;
}

}  // namespace

extern "C" {

ds4b200_path *ds4b200_path_create(const ds4b200_path_config *cfg) {
    if (!cfg) { set_error(-EINVAL, "path_create: null config"); return nullptr; }
    const ds4b200_path_config &c = *cfg;
    const bool ok = c.n_tokens > 0 && c.n_embd > 0 && c.n_embd % 32 == 0 && c.n_embd <= 8192 &&
                    c.vocab > 0 && c.kv_dim > 0 && c.kv_dim % 4 == 0 && c.kv_dim <= 1024 &&
                    c.n_rot >= 0 && c.n_rot % 4 == 0 && c.n_rot <= c.kv_dim &&
                    c.n_slots >= c.n_tokens && c.ff_dim > 0 && c.ff_dim % 4 == 0 && c.top_k > 0 &&
                    c.max_layers > 0 && c.sinkhorn_iters > 0 &&
                    (c.table_dtype == DS4B200_TABLE_F16 || c.table_dtype == DS4B200_TABLE_Q8_0) &&
                    (c.fp8_scale_mode == DS4B200_FP8_ROW_AMAX ||
                     (c.fp8_scale_mode == DS4B200_FP8_BLOCK64_POW2 && (c.kv_dim - c.n_rot) % 64 == 0 &&
                      c.n_rot % 64 == 0));
    if (!ok) { set_error(-EINVAL, "path_create: bad geometry"); return nullptr; }
    ds4b200_path *p = new ds4b200_path;
    p->cfg = c;
    cudaGetDevice(&p->device);
    p->n_scales = c.fp8_scale_mode == DS4B200_FP8_BLOCK64_POW2 ? (c.kv_dim - c.n_rot) / 64 : 1;
    const int64_t T = c.n_tokens, L = c.max_layers;
    bool good = cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking) == cudaSuccess &&
                cudaStreamCreateWithFlags(&p->side, cudaStreamNonBlocking) == cudaSuccess &&
                cudaStreamCreateWithFlags(&p->copy_in, cudaStreamNonBlocking) == cudaSuccess &&
                cudaStreamCreateWithFlags(&p->copy_out, cudaStreamNonBlocking) == cudaSuccess &&
                cudaEventCreateWithFlags(&p->ev_fork, cudaEventDisableTiming) == cudaSuccess &&
                cudaEventCreateWithFlags(&p->ev_join, cudaEventDisableTiming) == cudaSuccess;
    if (!good) set_error(-EIO, "path_create: cudaStreamCreate failed");
    good = good && alloc(p, "table", p->table, table_bytes(c));
    good = good && alloc(p, "ids", p->ids, T * 4) && alloc(p, "pos", p->pos, T * 4);
    good = good && alloc(p, "residual", p->residual, T * c.n_embd * 4);
    good = good && alloc(p, "norm_w", p->norm_w, (int64_t)c.n_embd * 4);
    good = good && alloc(p, "kv", p->kv, T * c.kv_dim * 4);
    good = good && alloc(p, "gate", p->gate, T * c.top_k * c.ff_dim * 4);
    good = good && alloc(p, "up", p->up, T * c.top_k * c.ff_dim * 4);
    good = good && alloc(p, "router_w", p->router_w, T * c.top_k * 4);
    good = good && alloc(p, "hc_logits", p->hc_logits, T * 16 * 4);
    good = good && alloc(p, "hc_a", p->hc_a, T * 4 * c.n_embd * 4);
    good = good && alloc(p, "hc_b", p->hc_b, T * 4 * c.n_embd * 4);
    good = good && alloc(p, "residual_out", p->residual_out, T * c.n_embd * 4);
    good = good && alloc(p, "normed_bf16", p->normed_bf16, T * c.n_embd * 2);
    good = good && alloc(p, "kv_codes", p->kv_codes, L * c.n_slots * c.kv_dim);
    good = good && alloc(p, "kv_scales", p->kv_scales, L * c.n_slots * p->n_scales * 4);
    if (c.fp8_scale_mode == DS4B200_FP8_BLOCK64_POW2)
        good = good && alloc(p, "kv_tail", p->kv_tail, L * c.n_slots * c.n_rot * 4);
    good = good && alloc(p, "ffn_out", p->ffn_out, T * c.ff_dim * 4);
    good = good && alloc(p, "comb", p->comb, T * 16 * 4);
    good = good && alloc(p, "gather_scratch", p->gather_scratch, T * c.kv_dim * 4);
    if (good) {
        // ids default to 0 so a run before the first upload stays inside the table
        good = cudaMemset(p->ids, 0, T * 4) == cudaSuccess && cudaMemset(p->pos, 0, T * 4) == cudaSuccess;
    }
    if (!good) { ds4b200_path_destroy(p); return nullptr; }
    return p;
}

void ds4b200_path_destroy(ds4b200_path *p) {
    if (!p) return;
    if (p->stream) cudaStreamSynchronize(p->stream);
    if (p->side) cudaStreamSynchronize(p->side);
    for (auto &g : p->graphs) cudaGraphExecDestroy(g.second);
    for (auto &g : p->slice_graphs) cudaGraphExecDestroy(g.second);
    if (p->ev_fork) cudaEventDestroy(p->ev_fork);
    if (p->ev_join) cudaEventDestroy(p->ev_join);
    if (p->side) cudaStreamDestroy(p->side);
    for (cudaEvent_t e : p->chunk_events) cudaEventDestroy(e);
    if (p->copy_in) { cudaStreamSynchronize(p->copy_in); cudaStreamDestroy(p->copy_in); }
    if (p->copy_out) { cudaStreamSynchronize(p->copy_out); cudaStreamDestroy(p->copy_out); }
    for (cudaEvent_t e : p->events) cudaEventDestroy(e);
    for (void *d : p->owned) cudaFree(d);
    if (p->stream) cudaStreamDestroy(p->stream);
    delete p;
}

int ds4b200_path_upload_table(ds4b200_path *p, const void *host_table, size_t bytes) {
    if (!p || !host_table) return set_error(-EINVAL, "path_upload_table: null argument");
    if ((int64_t)bytes != table_bytes(p->cfg))
        return set_error(-EINVAL, "path_upload_table: expected %lld bytes", (long long)table_bytes(p->cfg));
    CUDA_OK(cudaMemcpy(p->table, host_table, bytes, cudaMemcpyHostToDevice), "path_upload_table");
    return 0;
}

int ds4b200_path_check_io(const ds4b200_path_config *cfg, const ds4b200_path_io *host) {
    if (!cfg || !host) return set_error(-EINVAL, "path_check_io: null argument");
    return check_host_indices(*cfg, host, "path_check_io");
}

int ds4b200_path_upload(ds4b200_path *p, const ds4b200_path_io *host) {
    if (!p || !host) return set_error(-EINVAL, "path_upload: null argument");
    if (int rc = check_host_indices(p->cfg, host, "path_upload")) return rc;
    for (const Copy &c : input_copies(p, host))
        if (c.host) CUDA_OK(cudaMemcpyAsync(c.dev, c.host, (size_t)c.bytes, cudaMemcpyHostToDevice, p->stream), "path_upload");
    CUDA_OK(cudaStreamSynchronize(p->stream), "path_upload: sync");
    return 0;
}

void *ds4b200_path_buffer(ds4b200_path *p, const char *name, int64_t *bytes) {
    if (!p || !name) return nullptr;
    auto it = p->buf.find(name);
    if (it == p->buf.end()) return nullptr;
    if (bytes) *bytes = it->second.second;
    return it->second.first;
}

void *ds4b200_path_stream(ds4b200_path *p) { return p ? p->stream : nullptr; }

int ds4b200_path_run_device(ds4b200_path *p, int n_layers) {
    if (!p || n_layers < 0) return set_error(-EINVAL, "path_run_device: bad argument");
    return enqueue_run(p, n_layers);
}

int ds4b200_path_run_host(ds4b200_path *p, const ds4b200_path_io *h, int n_layers, float *ms) {
    if (!p || !h || n_layers < 1) return set_error(-EINVAL, "path_run_host: bad argument");
    if (int rc = check_host_indices(p->cfg, h, "path_run_host")) return rc;
    const ds4b200_path_config &c = p->cfg;
    const int64_t T = c.n_tokens;
    cudaStream_t s = p->stream;
    if (int rc = ensure_events(p, 2)) return rc;
    CUDA_OK(cudaEventRecord(p->events[0], s), "path_run_host: event");
    for (const Copy &cp : input_copies(p, h))
        if (cp.host) CUDA_OK(cudaMemcpyAsync(cp.dev, cp.host, (size_t)cp.bytes, cudaMemcpyHostToDevice, s), "path_run_host: H2D");
    if (int rc = enqueue_run(p, n_layers)) return rc;
    const int last = n_layers - 1;
    const int64_t l = last % c.max_layers;
#define D2H(host, dev, bytes) \
    if (host) CUDA_OK(cudaMemcpyAsync(host, dev, (size_t)(bytes), cudaMemcpyDeviceToHost, s), "path_run_host: D2H")
    D2H(h->residual_out, p->residual_out, T * c.n_embd * 4);
    D2H(h->normed_bf16, p->normed_bf16, T * c.n_embd * 2);
    D2H(h->ffn_out, p->ffn_out, T * c.ff_dim * 4);
    D2H(h->hc_out, hc_out(p, last), T * 4 * c.n_embd * 4);
    uint8_t *scratch = reinterpret_cast<uint8_t *>(p->gather_scratch);
    if (h->kv_codes) {
        gather_rows_kernel<<<(unsigned)T, 128, 0, s>>>(p->kv_codes + l * (int64_t)c.n_slots * c.kv_dim,
                                                       p->pos, scratch, c.kv_dim, T);
        D2H(h->kv_codes, scratch, T * c.kv_dim);
    }
    if (h->kv_scales) {
        gather_rows_kernel<<<(unsigned)T, 32, 0, s>>>(
            reinterpret_cast<uint8_t *>(p->kv_scales + l * (int64_t)c.n_slots * p->n_scales), p->pos,
            scratch, p->n_scales * 4, T);
        D2H(h->kv_scales, scratch, T * p->n_scales * 4);
    }
    if (h->kv_tail && p->kv_tail) {
        gather_rows_kernel<<<(unsigned)T, 64, 0, s>>>(
            reinterpret_cast<uint8_t *>(p->kv_tail + l * (int64_t)c.n_slots * c.n_rot), p->pos, scratch,
            c.n_rot * 4, T);
        D2H(h->kv_tail, scratch, T * c.n_rot * 4);
    }
#undef D2H
    CUDA_OK(cudaEventRecord(p->events[1], s), "path_run_host: event");
    CUDA_OK(cudaStreamSynchronize(s), "path_run_host: sync");
    if (ms) CUDA_OK(cudaEventElapsedTime(ms, p->events[0], p->events[1]), "path_run_host: elapsed");
    return 0;
}

int ds4b200_path_run_host_chunked(ds4b200_path *p, const ds4b200_path_io *h, int n_layers, int n_chunks,
                                  float *ms) {
    if (!p || !h || n_layers < 1 || n_chunks < 1) return set_error(-EINVAL, "path_run_host_chunked: bad argument");
    if (int rc = check_host_indices(p->cfg, h, "path_run_host_chunked")) return rc;
    const ds4b200_path_config &c = p->cfg;
    const int64_t T = c.n_tokens, E = c.n_embd;
    if (n_chunks > T) n_chunks = (int)T;
    if (int rc = ensure_events(p, 2)) return rc;
    while (p->chunk_events.size() < (size_t)2 * n_chunks + 1) {
        cudaEvent_t e;
        CUDA_OK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
        p->chunk_events.push_back(e);
    }
    cudaStream_t s = p->stream, in = p->copy_in, out = p->copy_out;
    CUDA_OK(cudaEventRecord(p->events[0], s), "path_run_host_chunked: event");
    CUDA_OK(cudaStreamWaitEvent(in, p->events[0], 0), "path_run_host_chunked: wait");
    CUDA_OK(cudaStreamWaitEvent(out, p->events[0], 0), "path_run_host_chunked: wait");
    const int last = n_layers - 1;
    const int64_t l = last % c.max_layers;
    uint8_t *scratch = reinterpret_cast<uint8_t *>(p->gather_scratch);
#define H2D(dev, host, off, cnt, esz) \
    if (host) CUDA_OK(cudaMemcpyAsync((char *)(dev) + (off) * (esz), (const char *)(host) + (off) * (esz), \
                                      (size_t)((cnt) * (esz)), cudaMemcpyHostToDevice, in), "path_run_host_chunked: H2D")
#define D2H(host, dev, off, cnt, esz) \
    if (host) CUDA_OK(cudaMemcpyAsync((char *)(host) + (off) * (esz), (const char *)(dev) + (off) * (esz), \
                                      (size_t)((cnt) * (esz)), cudaMemcpyDeviceToHost, out), "path_run_host_chunked: D2H")
    // Slice boundaries.  The first slice's copy-in and the last slice's compute and copy-out overlap with
    // nothing, so those two slices are half as long as the others (with four slices or more; a second,
    // finer step of the ramp measured the same).
    std::vector<int64_t> bound(n_chunks + 1);
    {
        auto weight = [&](int k) { return (n_chunks >= 4 && (k == 0 || k == n_chunks - 1)) ? 0.5 : 1.0; };
        double total_w = 0.0;
        for (int k = 0; k < n_chunks; ++k) total_w += weight(k);
        double acc = 0.0;
        bound[0] = 0;
        for (int k = 0; k < n_chunks; ++k) {
            acc += weight(k);
            int64_t b = (int64_t)(T * (acc / total_w) + 0.5);
            if (b <= bound[k]) b = bound[k] + 1;             // every slice has at least one row
            if (b > T - (n_chunks - 1 - k)) b = T - (n_chunks - 1 - k);
            bound[k + 1] = b;
        }
        bound[n_chunks] = T;
    }
    // The small per-token inputs go over once, whole: per copy the engine pays about 10 us whatever the size,
    // and per slice that was six such copies.
    H2D(p->norm_w, h->norm_w, 0, E, 4);
    H2D(p->ids, h->ids, 0, T, 4);
    H2D(p->pos, h->pos, 0, T, 4);
    H2D(p->router_w, h->router_w, 0, T * c.top_k, 4);
    H2D(p->hc_logits, h->hc_logits, 0, T * 16, 4);
    for (int k = 0; k < n_chunks; ++k) {
        const int64_t t0 = bound[k], n = bound[k + 1] - t0;
        cudaEvent_t in_ready = p->chunk_events[2 * k], done = p->chunk_events[2 * k + 1];
        // ---- inputs of this chunk, on the copy-in stream
        H2D(p->residual, h->residual, t0 * E, n * E, 4);
        H2D(p->kv, h->kv, t0 * c.kv_dim, n * c.kv_dim, 4);
        H2D(p->gate, h->gate, t0 * c.top_k * c.ff_dim, n * c.top_k * c.ff_dim, 4);
        H2D(p->up, h->up, t0 * c.top_k * c.ff_dim, n * c.top_k * c.ff_dim, 4);
        H2D(p->hc_a, h->hc_resid, t0 * 4 * E, n * 4 * E, 4);
        CUDA_OK(cudaEventRecord(in_ready, in), "path_run_host_chunked: event");
        // ---- the layer chain over this chunk's rows
        CUDA_OK(cudaStreamWaitEvent(s, in_ready, 0), "path_run_host_chunked: wait");
        if (c.use_graph) {
            // the slice's 43-layer chain is several hundred launches and event calls: replay it
            // from a graph, or the host cannot keep the copy engines and the GPU busy
            const auto key = std::make_tuple(t0, n, n_layers);
            auto it = p->slice_graphs.find(key);
            if (it == p->slice_graphs.end()) {
                cudaGraph_t g = nullptr;
                cudaGraphExec_t ge = nullptr;
                CUDA_OK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal), "path_run_host_chunked: begin capture");
                for (int layer = 0; layer < n_layers; ++layer) enqueue_layer(p, layer, -1, t0, n);
                CUDA_OK(cudaStreamEndCapture(s, &g), "path_run_host_chunked: end capture");
                CUDA_OK(cudaGraphInstantiate(&ge, g, 0), "path_run_host_chunked: graph instantiate");
                cudaGraphDestroy(g);
                it = p->slice_graphs.emplace(key, ge).first;
            }
            CUDA_OK(cudaGraphLaunch(it->second, s), "path_run_host_chunked: graph launch");
        } else {
            for (int layer = 0; layer < n_layers; ++layer) enqueue_layer(p, layer, -1, t0, n);
        }
        CUDA_OK(cudaGetLastError(), "path_run_host_chunked: launch");
        CUDA_OK(cudaEventRecord(done, s), "path_run_host_chunked: event");
        // ---- outputs of this chunk, on the copy-out stream
        CUDA_OK(cudaStreamWaitEvent(out, done, 0), "path_run_host_chunked: wait");
        D2H(h->residual_out, p->residual_out, t0 * E, n * E, 4);
        D2H(h->normed_bf16, p->normed_bf16, t0 * E, n * E, 2);
        D2H(h->ffn_out, p->ffn_out, t0 * c.ff_dim, n * c.ff_dim, 4);
        D2H(h->hc_out, hc_out(p, last), t0 * 4 * E, n * 4 * E, 4);
        if (h->kv_codes) {
            gather_rows_kernel<<<(unsigned)n, 128, 0, out>>>(p->kv_codes + l * (int64_t)c.n_slots * c.kv_dim,
                                                             p->pos + t0, scratch, c.kv_dim, n);
            CUDA_OK(cudaMemcpyAsync(h->kv_codes + t0 * c.kv_dim, scratch, (size_t)(n * c.kv_dim),
                                    cudaMemcpyDeviceToHost, out), "path_run_host_chunked: D2H");
        }
        if (h->kv_scales) {
            gather_rows_kernel<<<(unsigned)n, 32, 0, out>>>(
                reinterpret_cast<uint8_t *>(p->kv_scales + l * (int64_t)c.n_slots * p->n_scales), p->pos + t0,
                scratch, p->n_scales * 4, n);
            CUDA_OK(cudaMemcpyAsync(h->kv_scales + t0 * p->n_scales, scratch, (size_t)(n * p->n_scales * 4),
                                    cudaMemcpyDeviceToHost, out), "path_run_host_chunked: D2H");
        }
        if (h->kv_tail && p->kv_tail) {
            gather_rows_kernel<<<(unsigned)n, 64, 0, out>>>(
                reinterpret_cast<uint8_t *>(p->kv_tail + l * (int64_t)c.n_slots * c.n_rot), p->pos + t0, scratch,
                c.n_rot * 4, n);
            CUDA_OK(cudaMemcpyAsync(h->kv_tail + t0 * c.n_rot, scratch, (size_t)(n * c.n_rot * 4),
                                    cudaMemcpyDeviceToHost, out), "path_run_host_chunked: D2H");
        }
    }
#undef H2D
#undef D2H
    // join: the main stream waits for the last copy-out, then closes the timed region
    cudaEvent_t all_out = p->chunk_events[2 * n_chunks];
    CUDA_OK(cudaEventRecord(all_out, out), "path_run_host_chunked: event");
    CUDA_OK(cudaStreamWaitEvent(s, all_out, 0), "path_run_host_chunked: wait");
    CUDA_OK(cudaEventRecord(p->events[1], s), "path_run_host_chunked: event");
    CUDA_OK(cudaStreamSynchronize(s), "path_run_host_chunked: sync");
    if (ms) CUDA_OK(cudaEventElapsedTime(ms, p->events[0], p->events[1]), "path_run_host_chunked: elapsed");
    return 0;
}

int ds4b200_path_time_device(ds4b200_path *p, int n_layers, int warmup, int steps, float *ms_total) {
    if (!p || n_layers < 1 || warmup < 0 || steps < 1 || !ms_total)
        return set_error(-EINVAL, "path_time_device: bad argument");
    if (int rc = ensure_events(p, 2)) return rc;
    for (int i = 0; i < warmup; ++i)
        if (int rc = enqueue_run(p, n_layers)) return rc;
    CUDA_OK(cudaStreamSynchronize(p->stream), "path_time_device: sync");
    CUDA_OK(cudaEventRecord(p->events[0], p->stream), "path_time_device: event");
    for (int i = 0; i < steps; ++i)
        if (int rc = enqueue_run(p, n_layers)) return rc;
    CUDA_OK(cudaEventRecord(p->events[1], p->stream), "path_time_device: event");
    CUDA_OK(cudaStreamSynchronize(p->stream), "path_time_device: sync");
    CUDA_OK(cudaEventElapsedTime(ms_total, p->events[0], p->events[1]), "path_time_device: elapsed");
    return 0;
}

int ds4b200_path_profile_ops(ds4b200_path *p, int reps, float *ms_per_launch) {
    if (!p || reps < 1 || !ms_per_launch) return set_error(-EINVAL, "path_profile_ops: bad argument");
    if (int rc = ensure_events(p, 2 * DS4B200_PATH_N_KERNELS)) return rc;
    if (int rc = enqueue_run(p, 1)) return rc;        // valid comb / cache contents, warm caches
    for (int op = 0; op < DS4B200_PATH_N_KERNELS; ++op) {
        CUDA_OK(cudaEventRecord(p->events[2 * op], p->stream), "path_profile_ops: event");
        for (int r = 0; r < reps; ++r) enqueue_layer(p, r, op);
        CUDA_OK(cudaEventRecord(p->events[2 * op + 1], p->stream), "path_profile_ops: event");
    }
    CUDA_OK(cudaGetLastError(), "path_profile_ops: launch");
    CUDA_OK(cudaStreamSynchronize(p->stream), "path_profile_ops: sync");
    for (int op = 0; op < DS4B200_PATH_N_KERNELS; ++op) {
        float ms = 0.0f;
        CUDA_OK(cudaEventElapsedTime(&ms, p->events[2 * op], p->events[2 * op + 1]), "path_profile_ops: elapsed");
        ms_per_launch[op] = ms / (float)reps;
    }
    return 0;
}

int ds4b200_path_launches_per_run(ds4b200_path *p, int n_layers) {
    return p ? DS4B200_PATH_N_KERNELS * n_layers : 0;
}

int64_t ds4b200_path_op_bytes(ds4b200_path *p, int op) {
    if (!p) return 0;
    const ds4b200_path_config &c = p->cfg;
    const int64_t T = c.n_tokens;
    const int64_t row = c.table_dtype == DS4B200_TABLE_Q8_0 ? (int64_t)(c.n_embd / 32) * 34 : (int64_t)c.n_embd * 2;
    switch (op) {
    case 0: return T * (row + 4 + (int64_t)c.n_embd * (4 + 4 + 2)) + (int64_t)c.n_embd * 4;
    case 1: return T * ((int64_t)c.kv_dim * 4 + 4 + c.kv_dim + (int64_t)p->n_scales * 4 +
                        (p->kv_tail ? (int64_t)c.n_rot * 4 : 0));
    case 2: return T * ((int64_t)2 * c.top_k * c.ff_dim * 4 + (int64_t)c.top_k * 4 + (int64_t)c.ff_dim * 4);
    case 3: return T * ((int64_t)2 * 4 * c.n_embd * 4 + 64);
    case 4: return T * (int64_t)(64 + 64);
    default: return 0;
    }
}

}  // extern "C"
