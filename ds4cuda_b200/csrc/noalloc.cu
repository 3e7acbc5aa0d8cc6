// noalloc.cu — Sinkhorn mixing for callers that cannot provide (or allocate) the
// intermediate buffer the fast two-kernel path needs.
//
// ds4b200_hc_sinkhorn_mix_rows_f32 is fast only when the caller hands it a
// [n_tokens][16] buffer for the Sinkhorn matrices, which the first kernel writes
// and the second reads.  Some callers have no such buffer and no way to get one:
// an engine whose device memory is one arena carved at start-up and fully spoken
// for (the reference's own session does this and its launchers never allocate),
// a serving loop that bans allocator calls on the token path because cudaMalloc
// stalls the whole device and may fail late, or a binding layer that is handed
// input and output pointers and nothing else.  For them the variant below keeps
// that buffer inside the library, in a fixed array in device global memory.
#include <cerrno>
#include <mutex>

#include "../../include/ds4b200.h"
#include "kernels.cuh"

namespace {

// 16384 tokens x 16 floats = 1 MiB.  Every GPU that loads the library carries
// this array from module load until the process exits.
constexpr int64_t kStaticMaxTokens = DS4B200_STATIC_MAX_TOKENS;
static __device__ __align__(256) float g_comb_scratch[kStaticMaxTokens * 16];

// In host code `g_comb_scratch` is only a handle for the runtime, not a device
// address; the address a kernel can use comes from cudaGetSymbolAddress, asked
// once per device with that device current, and cached here.
constexpr int kMaxDevices = 64;
float *g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

int scratch_on_current_device(float **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return ds4b200::set_error(-EIO, "static scratch: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return ds4b200::set_error(-EINVAL, "static scratch: device %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_addr[dev]) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_comb_scratch);
        if (e != cudaSuccess || !ptr)
            return ds4b200::set_error(-EIO, "static scratch: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_scratch_addr[dev] = static_cast<float *>(ptr);
    }
    *out = g_scratch_addr[dev];
    return 0;
}

}  // namespace

extern "C" int ds4b200_hc_sinkhorn_mix_rows_static_f32(const float *logits, const float *residual_hc,
                                                       float *out_hc, int64_t n_tokens, int n_embd,
                                                       int sinkhorn_iters, float eps, void *stream) {
    if (n_tokens < 0) return ds4b200::set_error(-EINVAL, "hc_sinkhorn_mix_rows_static: n_tokens < 0");
    if (n_tokens == 0) return 0;
    if (n_tokens > kStaticMaxTokens)
        return ds4b200::set_error(-EINVAL,
                                  "hc_sinkhorn_mix_rows_static: %lld tokens exceed the built-in scratch of %lld "
                                  "tokens; split the batch or use ds4b200_hc_sinkhorn_mix_rows_f32 with comb_out",
                                  (long long)n_tokens, (long long)kStaticMaxTokens);
    if (!logits || !residual_hc || !out_hc)
        return ds4b200::set_error(-EINVAL, "hc_sinkhorn_mix_rows_static: null pointer");
    if (n_embd <= 0 || n_embd % 4 != 0 || n_embd > 8192)
        return ds4b200::set_error(-EINVAL, "hc_sinkhorn_mix_rows_static: n_embd must be a multiple of 4, at most 8192");
    if (sinkhorn_iters < 1) return ds4b200::set_error(-EINVAL, "hc_sinkhorn_mix_rows_static: sinkhorn_iters < 1");
    float *comb = nullptr;
    if (int rc = scratch_on_current_device(&comb)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The first kernel overwrites rows [0, n_tokens) of the scratch before the
    // second reads them, so nothing left by an earlier call is ever consumed.
    ds4b200::hc_sinkhorn_rows(logits, comb, n_tokens, sinkhorn_iters, eps, s);
    ds4b200::hc_post_rows(nullptr, nullptr, residual_hc, nullptr, comb, nullptr, nullptr, out_hc, n_tokens,
                          n_embd, 0, 0.0f, s);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return ds4b200::set_error(-EIO, "hc_sinkhorn_mix_rows_static: %s", cudaGetErrorString(e));
    return 0;
}
