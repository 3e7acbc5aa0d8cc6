// embedding.cu — token-embedding row gather for a batch of ids, fused with the
// steps that follow it in the forward pass: dequantise -> (+ residual) ->
// replicate into the hyper-connection streams -> RMSNorm -> f32 / bf16.
//
// Arithmetic: F16 rows are converted exactly (cuda/embedding.cu:27-39,
// cuda/common.cuh:20-24); Q8_0 rows are 34-byte blocks {f16 scale, 32 x int8}
// (cuda/common.cuh:29-33) dequantised with one multiply d*(float)q
// (cuda/dense_q8.cu:60-67).  Both are bit-exact.  The norm is cuda/norm.cu:52-105.
//
// Data movement: one CTA per token.  A Q8_0 row (4352 B for 4096 columns) is a
// run of 2-byte-aligned records, so it is pulled into shared memory with ONE
// 1-D bulk asynchronous copy (TMA) while the threads fetch the residual row with
// 128-bit loads; the decode then reads shared memory.  F16 rows are read with
// 64-bit loads straight into registers.  The dequantised row stays in registers
// through the reduction, so every byte crosses HBM once.
#include "device_utils.cuh"
#include "kernels.cuh"

namespace ds4b200 {
namespace {

__device__ int g_status_word = 0;

constexpr int kThreads = 256;
constexpr int kMaxEmbd = 8192;                       // VPT <= 8 at 256 threads
constexpr int kMaxQ8RowBytes = kMaxEmbd / 32 * 34;   // 8704

struct EmbedArgs {
    const void *table;
    const int32_t *ids;
    int single_id;
    int n_embd;
    const float *residual_in;
    const float *norm_w;
    float eps;
    float *out_rows;
    int n_replicas;
    float *normed_f32;
    uint16_t *normed_bf16;
};

template <int VPT, bool Q8, bool BULK>
__global__ void __launch_bounds__(kThreads) embed_gather_kernel(EmbedArgs a) {
    __shared__ float red[33];
    __shared__ __align__(16) unsigned char raw[Q8 ? kMaxQ8RowBytes : 16];
    __shared__ __align__(8) uint64_t bar;

    const int64_t t = blockIdx.x;
    const int64_t id = a.ids ? a.ids[t] : a.single_id;
    const int n = a.n_embd, n4 = n >> 2, tid = threadIdx.x;
    float4 v[VPT];

    if (Q8) {
        const uint32_t row_bytes = (uint32_t)(n / 32) * 34u;
        const unsigned char *src = static_cast<const unsigned char *>(a.table) + id * row_bytes;
        if (BULK) {
            if (tid == 0) mbar_init(&bar, 1);
            __syncthreads();
            if (tid == 0) bulk_load_1d(raw, src, row_bytes, &bar);
        } else {
            // 2-byte granularity copy for tables or rows that are not 16-byte aligned
            const uint16_t *s16 = reinterpret_cast<const uint16_t *>(src);
            uint16_t *d16 = reinterpret_cast<uint16_t *>(raw);
            for (uint32_t i = tid; i < row_bytes / 2; i += kThreads) d16[i] = __ldg(s16 + i);
        }
    }

    // residual loads are issued before anybody waits on the row
    float4 r[VPT];
    if (a.residual_in) {
        const float *rr = a.residual_in + t * n;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = tid + j * kThreads;
            if (i < n4) r[j] = ld_stream4(rr + 4 * i);
        }
    }

    if (Q8) {
        if (BULK) mbar_wait_bounded(&bar, 0, &g_status_word);
        else __syncthreads();
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = tid + j * kThreads;
            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i >= n4) continue;
            const int e = 4 * i;                       // 4 elements inside one block
            const unsigned char *blk = raw + (e >> 5) * 34;
            const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(blk));
            const uint16_t q01 = *reinterpret_cast<const uint16_t *>(blk + 2 + (e & 31));
            const uint16_t q23 = *reinterpret_cast<const uint16_t *>(blk + 4 + (e & 31));
            v[j].x = d * (float)(int8_t)(q01 & 0xff);
            v[j].y = d * (float)(int8_t)(q01 >> 8);
            v[j].z = d * (float)(int8_t)(q23 & 0xff);
            v[j].w = d * (float)(int8_t)(q23 >> 8);
        }
    } else {
        const uint16_t *src = static_cast<const uint16_t *>(a.table) + id * n;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = tid + j * kThreads;
            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i >= n4) continue;
            const uint2 h = __ldcs(reinterpret_cast<const uint2 *>(src + 4 * i));
            const float2 lo = f16x2_bits_to_f32(h.x), hi = f16x2_bits_to_f32(h.y);
            v[j] = make_float4(lo.x, lo.y, hi.x, hi.y);
        }
    }

    if (a.residual_in) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) v[j] = add4(v[j], (tid + j * kThreads < n4) ? r[j] : make_float4(0.f, 0.f, 0.f, 0.f));
    }
    if (a.out_rows) {
        for (int rep = 0; rep < a.n_replicas; ++rep) {
            float *o = a.out_rows + (t * a.n_replicas + rep) * n;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int i = tid + j * kThreads;
                if (i < n4) st_stream4(o + 4 * i, v[j]);
            }
        }
    }
    if (!a.norm_w) return;

    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) ss += dot4(v[j]);
    ss = block_sum(ss, red);
    const float scale = rms_scale(ss, (float)n, a.eps);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = tid + j * kThreads;
        if (i >= n4) continue;
        const float4 w4 = ld_ro4(a.norm_w + 4 * i);
        const float4 y = make_float4(v[j].x * scale * w4.x, v[j].y * scale * w4.y,
                                     v[j].z * scale * w4.z, v[j].w * scale * w4.w);
        if (a.normed_f32) st_stream4(a.normed_f32 + t * n + 4 * i, y);
        if (a.normed_bf16) st_bf16x4(a.normed_bf16 + t * n + 4 * i, y);
    }
}

// Any n_embd / alignment: scalar loads, row re-read for the second pass.
__global__ void embed_gather_scalar_kernel(EmbedArgs a, int q8) {
    __shared__ float red[33];
    const int64_t t = blockIdx.x;
    const int64_t id = a.ids ? a.ids[t] : a.single_id;
    const int n = a.n_embd;
    auto element = [&](int i) -> float {
        float v;
        if (q8) {
            const unsigned char *blk = static_cast<const unsigned char *>(a.table) +
                                       id * (int64_t)(n / 32) * 34 + (i >> 5) * 34;
            const float d = f16_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
            v = d * (float)(int8_t)blk[2 + (i & 31)];
        } else {
            v = f16_bits_to_f32(static_cast<const uint16_t *>(a.table)[id * n + i]);
        }
        if (a.residual_in) v += a.residual_in[t * n + i];
        return v;
    };
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = element(i);
        if (a.out_rows)
            for (int rep = 0; rep < a.n_replicas; ++rep) a.out_rows[(t * a.n_replicas + rep) * n + i] = v;
        ss += v * v;
    }
    if (!a.norm_w) return;
    ss = block_sum(ss, red);
    const float scale = rms_scale(ss, (float)n, a.eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float y = element(i) * scale * a.norm_w[i];
        if (a.normed_f32) a.normed_f32[t * n + i] = y;
        if (a.normed_bf16) a.normed_bf16[t * n + i] = bf16_bits(y);
    }
}

// One F16 row to f32 and nothing else (the single-token launcher): 64-thread CTAs, one
// 64-bit load and one 128-bit store per thread, so the row is spread over many SMs.
__global__ void embed_f16_row_kernel(const uint16_t *__restrict__ row, float *__restrict__ out, int n4) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const uint2 h = __ldg(reinterpret_cast<const uint2 *>(row + 4 * i));
    const float2 lo = f16x2_bits_to_f32(h.x), hi = f16x2_bits_to_f32(h.y);
    *reinterpret_cast<float4 *>(out + 4 * i) = make_float4(lo.x, lo.y, hi.x, hi.y);
}

template <bool Q8, bool BULK>
void launch_vec(const EmbedArgs &a, int64_t n_tokens, cudaStream_t s) {
    const int vpt = ((a.n_embd >> 2) + kThreads - 1) / kThreads;
    const unsigned grid = (unsigned)n_tokens;
    if (vpt <= 1) embed_gather_kernel<1, Q8, BULK><<<grid, kThreads, 0, s>>>(a);
    else if (vpt <= 2) embed_gather_kernel<2, Q8, BULK><<<grid, kThreads, 0, s>>>(a);
    else if (vpt <= 4) embed_gather_kernel<4, Q8, BULK><<<grid, kThreads, 0, s>>>(a);
    else embed_gather_kernel<8, Q8, BULK><<<grid, kThreads, 0, s>>>(a);
}

}  // namespace

void embed_gather_rows(const void *table, int table_dtype, const int32_t *ids, int single_id,
                       int64_t n_tokens, int n_embd, const float *residual_in,
                       const float *norm_w, float eps, float *out_rows, int n_replicas,
                       float *normed_f32, uint16_t *normed_bf16, cudaStream_t s) {
    if (n_tokens <= 0 || n_embd <= 0) return;
    const EmbedArgs a{table, ids, single_id, n_embd, residual_in, norm_w, eps,
                      out_rows, n_replicas, normed_f32, normed_bf16};
    const bool q8 = table_dtype == DS4B200_TABLE_Q8_0;
    const bool vec = (n_embd & 3) == 0 && n_embd <= kMaxEmbd && (!q8 || (n_embd & 31) == 0) &&
                     aligned16(residual_in) && aligned16(norm_w) && aligned16(out_rows) &&
                     aligned16(normed_f32) && aligned8(normed_bf16) &&
                     (q8 ? (reinterpret_cast<uintptr_t>(table) & 1u) == 0 : aligned8(table));
    if (!vec) {
        embed_gather_scalar_kernel<<<(unsigned)n_tokens, kThreads, 0, s>>>(a, q8 ? 1 : 0);
        return;
    }
    if (!q8 && n_tokens == 1 && !ids && !residual_in && !norm_w && n_replicas == 1) {
        const int n4 = n_embd >> 2;
        embed_f16_row_kernel<<<(n4 + 63) / 64, 64, 0, s>>>(
            static_cast<const uint16_t *>(table) + (int64_t)single_id * n_embd, out_rows, n4);
    } else if (!q8) {
        launch_vec<false, false>(a, n_tokens, s);
    } else if (aligned16(table) && ((n_embd / 32 * 34) & 15) == 0) {
        launch_vec<true, true>(a, n_tokens, s);    // every row starts on 16 B: bulk copy
    } else {
        launch_vec<true, false>(a, n_tokens, s);
    }
}

// A wait that nothing will ever satisfy, with a short poll limit: it must give up, raise
// the status bit and let the kernel end normally.  Used by the self-test of the bounded wait.
__global__ void wait_gives_up_kernel(int max_polls, int *gave_up) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) mbar_init(&bar, 1);
    __syncthreads();
    const bool done = mbar_wait_bounded(&bar, 0, &g_status_word, max_polls);
    if (threadIdx.x == 0) *gave_up = done ? 0 : 1;
}

void selftest_bounded_wait(int max_polls, int *gave_up_dev, cudaStream_t s) {
    wait_gives_up_kernel<<<1, 32, 0, s>>>(max_polls, gave_up_dev);
}

// Device address of the status word on the current device (null on error), for kernels in
// other translation units that make bounded waits.
int *device_status_word() {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return static_cast<int *>(p);
}

int read_and_clear_device_status() {
    int v = 0, zero = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -5;
    if (cudaMemcpyFromSymbol(&v, g_status_word, sizeof v) != cudaSuccess) return -5;
    if (v != 0 && cudaMemcpyToSymbol(g_status_word, &zero, sizeof zero) != cudaSuccess) return -5;
    return v;
}

}  // namespace ds4b200
