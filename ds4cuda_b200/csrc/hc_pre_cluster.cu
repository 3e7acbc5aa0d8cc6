// hc_pre_cluster.cu — the hyper-connection "pre" step for many tokens with the
// 24 x (4*n_embd) f16 matrix resident on chip.
//
// Arithmetic: cuda/hc_sinkhorn.cu:85-305 of the reference (RMS over the token's
// 4*n_embd residual block, 24 dot products with hc_fn, sigmoid gates, weighted
// stream sum); the Sinkhorn sweeps over the 16 comb values run afterwards in
// hc_sinkhorn_rows_kernel.
//
// Why a cluster: per token the step reads 64 KiB of activations but needs all
// 768 KiB of hc_fn.  Re-reading hc_fn per token through L2 costs 12x the HBM
// traffic of the activations.  Here a thread-block cluster of C CTAs splits the
// columns: CTA r keeps the slice hc_fn[:, columns of r], converted once to f32 and
// stored as pairs of output rows (192 KiB), in its shared memory for its whole
// life, so that one 64-bit shared load feeds a packed two-lane FMA
// (fma.rn.f32x2) per token, streams the matching column slice of every
// token through registers exactly once (M tokens at a time, so each weight read
// from shared memory feeds M tokens), and the C partial results per token
// (24 dots + sum of squares) are exchanged over distributed shared memory with
// one cluster barrier per token group.  Every CTA then holds the full sums,
// computes the gates redundantly and writes its own column slice of `out`.
#include <cooperative_groups.h>

#include <mutex>

#include "device_utils.cuh"
#include "kernels.cuh"

namespace cg = cooperative_groups;

namespace ds4b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMixN = 24;
constexpr int kSlots = 32;            // per token: 24 dots, slot 24 = sum of squares, rest unused


// Sum 32 per-lane values across the warp; lane l ends with the total of value l.
__device__ __forceinline__ float warp_transpose_sum32(float (&v)[32]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int half = 16; half >= 1; half >>= 1) {
        const bool upper = (lane & half) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            const float send = upper ? v[i] : v[i + half];
            const float keep = upper ? v[i + half] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
        }
    }
    return v[0];
}

// Packed FMA on two f32 lanes: d = a * b + c per lane, one instruction on sm_100.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    unsigned long long ua = *reinterpret_cast<unsigned long long *>(&a);
    unsigned long long ub = *reinterpret_cast<unsigned long long *>(&b);
    unsigned long long uc = *reinterpret_cast<unsigned long long *>(&c), ud;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(ud) : "l"(ua), "l"(ub), "l"(uc));
    return *reinterpret_cast<float2 *>(&ud);
}

// C: CTAs per cluster.  VC: float2 columns per thread per stream
// (n_embd = C * VC * 512).  M: tokens held in registers together.  S: sub-batches of M
// tokens per exchange over the cluster.
template <int C, int VC, int M, int S>
__global__ void __launch_bounds__(kThreads, 1)
hc_pre_cluster_kernel(const float *__restrict__ residual_hc, const uint16_t *__restrict__ hc_fn,
                      const float *__restrict__ hc_scale, const float *__restrict__ hc_base,
                      float *__restrict__ post_out, float *__restrict__ comb_out,
                      float *__restrict__ out, int64_t n_tokens, int n_embd, float eps) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int kWPairs = (kMixN / 2) * 4 * VC * 2 * kThreads;       // float2 {row 2p, row 2p+1} entries
    float2 *w_s = reinterpret_cast<float2 *>(smem_raw);
    float *part = reinterpret_cast<float *>(w_s + kWPairs);            // [kWarps][S*M][32]
    float *cl_part = part + kWarps * S * M * kSlots;                   // [C][S*M][32]
    float *tot = cl_part + C * S * M * kSlots;                         // [S*M][32]
    float *pre_s = tot + S * M * kSlots;                               // [S*M][4]

    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int64_t cluster_id = blockIdx.x / C, n_clusters = gridDim.x / C;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cols = n_embd / C;                                       // floats per stream owned by this CTA
    const int64_t hc_dim = 4 * (int64_t)n_embd;
    const int col0 = rank * cols;

    // resident slice of hc_fn: entry (((p*4+h)*VC+v)*2+c)*256+tid = rows 2p, 2p+1 at column
    // col0 + 2*(v*256+tid) + c of stream h
    for (int p = 0; p < kMixN / 2; ++p)
#pragma unroll
        for (int h = 0; h < 4; ++h)
#pragma unroll
            for (int v = 0; v < VC; ++v) {
                const int64_t off = (int64_t)h * n_embd + col0 + 2 * (v * kThreads + tid);
                const float2 lo = f16x2_bits_to_f32(__ldg(reinterpret_cast<const uint32_t *>(hc_fn + (2 * p) * hc_dim + off)));
                const float2 hi = f16x2_bits_to_f32(__ldg(reinterpret_cast<const uint32_t *>(hc_fn + (2 * p + 1) * hc_dim + off)));
                w_s[(((p * 4 + h) * VC + v) * 2 + 0) * kThreads + tid] = make_float2(lo.x, hi.x);
                w_s[(((p * 4 + h) * VC + v) * 2 + 1) * kThreads + tid] = make_float2(lo.y, hi.y);
            }
    __syncthreads();

    // A super-group is S sub-batches of M tokens: the dot products run sub-batch by
    // sub-batch (registers hold M tokens), the exchange over the cluster and its barriers
    // happen once per super-group, and the weighted sum re-reads the rows, which are then
    // still in L2 (G * 64 KiB per cluster).
    constexpr int G = S * M;
    const int64_t n_super = (n_tokens + G - 1) / G;
    const int64_t n_sub = n_super * S;                                  // sub-batch index q covers tokens q*M..
    auto x_ptr = [&](int64_t t, int h, int v) {
        return reinterpret_cast<const float2 *>(residual_hc + t * hc_dim + (int64_t)h * n_embd + col0 +
                                                2 * (v * kThreads + tid));
    };
    float2 xn[M][4][VC];
    auto load_sub = [&](int64_t q) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const int64_t t = q * M + m;
#pragma unroll
            for (int h = 0; h < 4; ++h)
#pragma unroll
                for (int v = 0; v < VC; ++v)
                    xn[m][h][v] = (t < n_tokens) ? __ldg(x_ptr(t, h, v)) : make_float2(0.f, 0.f);
        }
    };
    if (cluster_id < n_super) load_sub(cluster_id * S);

    for (int64_t sg = cluster_id; sg < n_super; sg += n_clusters) {
#pragma unroll 1
        for (int sb = 0; sb < S; ++sb) {
            float2 x[M][4][VC];
#pragma unroll
            for (int m = 0; m < M; ++m)
#pragma unroll
                for (int h = 0; h < 4; ++h)
#pragma unroll
                    for (int v = 0; v < VC; ++v) x[m][h][v] = xn[m][h][v];
            // the next sub-batch's loads fly during the math
            const int64_t q_next = (sb + 1 < S) ? sg * S + sb + 1 : (sg + n_clusters) * S;
            if (q_next < n_sub) load_sub(q_next);

            // ---- this thread's partial sums: pair p of token m holds rows 2p and 2p+1
            float2 acc2[M][kMixN / 2];
            float ss[M];
#pragma unroll
            for (int m = 0; m < M; ++m) {
                ss[m] = 0.0f;
#pragma unroll
                for (int p = 0; p < kMixN / 2; ++p) acc2[m][p] = make_float2(0.f, 0.f);
            }
#pragma unroll
            for (int h = 0; h < 4; ++h)
#pragma unroll
                for (int v = 0; v < VC; ++v) {
                    float2 xx[M], xy[M];
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        xx[m] = make_float2(x[m][h][v].x, x[m][h][v].x);
                        xy[m] = make_float2(x[m][h][v].y, x[m][h][v].y);
                        ss[m] += x[m][h][v].x * x[m][h][v].x + x[m][h][v].y * x[m][h][v].y;
                    }
#pragma unroll
                    for (int p = 0; p < kMixN / 2; ++p) {
                        const float2 w0 = w_s[(((p * 4 + h) * VC + v) * 2 + 0) * kThreads + tid];
                        const float2 w1 = w_s[(((p * 4 + h) * VC + v) * 2 + 1) * kThreads + tid];
#pragma unroll
                        for (int m = 0; m < M; ++m) {
                            acc2[m][p] = ffma2(w0, xx[m], acc2[m][p]);
                            acc2[m][p] = ffma2(w1, xy[m], acc2[m][p]);
                        }
                    }
                }
            float acc[M][kSlots];
#pragma unroll
            for (int m = 0; m < M; ++m) {
#pragma unroll
                for (int p = 0; p < kMixN / 2; ++p) { acc[m][2 * p] = acc2[m][p].x; acc[m][2 * p + 1] = acc2[m][p].y; }
                acc[m][kMixN] = ss[m];
#pragma unroll
                for (int k = kMixN + 1; k < kSlots; ++k) acc[m][k] = 0.0f;
            }
#pragma unroll
            for (int m = 0; m < M; ++m)
                part[(warp * G + sb * M + m) * kSlots + lane] = warp_transpose_sum32(acc[m]);
        }
        __syncthreads();

        // ---- CTA totals, pushed into every CTA of the cluster over DSMEM
        for (int i = tid; i < G * kSlots; i += kThreads) {
            float s = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) s += part[w * G * kSlots + i];
            float *mine = cl_part + rank * G * kSlots + i;
#pragma unroll
            for (int r = 0; r < C; ++r) *cluster.map_shared_rank(mine, r) = s;
        }
        cluster.sync();
        for (int i = tid; i < G * kSlots; i += kThreads) {
            float s = 0.0f;
#pragma unroll
            for (int r = 0; r < C; ++r) s += cl_part[r * G * kSlots + i];          // same order everywhere
            tot[i] = s;
        }
        __syncthreads();

        // ---- gates (every CTA, identical results); rank 0 writes the small outputs
        for (int i = tid; i < 4 * G; i += kThreads) {
            const int m = i >> 2, h = i & 3;
            const int64_t t = sg * G + m;
            const float rms = rms_scale(tot[m * kSlots + kMixN], (float)hc_dim, eps);
            const float zp = (tot[m * kSlots + h] * rms) * hc_scale[0] + hc_base[h];
            pre_s[m * 4 + h] = 1.0f / (1.0f + expf(-zp)) + eps;
            if (rank == 0 && t < n_tokens) {
                const float zq = (tot[m * kSlots + 4 + h] * rms) * hc_scale[1] + hc_base[4 + h];
                post_out[t * 4 + h] = 2.0f / (1.0f + expf(-zq));
            }
        }
        if (rank == 0) {
            for (int i = tid; i < 16 * G; i += kThreads) {
                const int m = i >> 4, k = i & 15;
                const int64_t t = sg * G + m;
                if (t < n_tokens) {
                    const float rms = rms_scale(tot[m * kSlots + kMixN], (float)hc_dim, eps);
                    comb_out[t * 16 + k] = (tot[m * kSlots + 8 + k] * rms) * hc_scale[2] + hc_base[8 + k];
                }
            }
        }
        __syncthreads();

        // ---- weighted stream sum for this CTA's columns; the rows come back from L2
#pragma unroll 1
        for (int m0 = 0; m0 < G; m0 += M) {
            float2 xr[M][4][VC];
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const int64_t t = sg * G + m0 + m;
#pragma unroll
                for (int h = 0; h < 4; ++h)
#pragma unroll
                    for (int v = 0; v < VC; ++v)
                        xr[m][h][v] = (t < n_tokens) ? __ldcs(x_ptr(t, h, v)) : make_float2(0.f, 0.f);
            }
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const int64_t t = sg * G + m0 + m;
                if (t >= n_tokens) continue;
                const float *pm = pre_s + (m0 + m) * 4;
                const float p0 = pm[0], p1 = pm[1], p2 = pm[2], p3 = pm[3];
#pragma unroll
                for (int v = 0; v < VC; ++v) {
                    float2 o2;
                    o2.x = xr[m][0][v].x * p0 + xr[m][1][v].x * p1 + xr[m][2][v].x * p2 + xr[m][3][v].x * p3;
                    o2.y = xr[m][0][v].y * p0 + xr[m][1][v].y * p1 + xr[m][2][v].y * p2 + xr[m][3][v].y * p3;
                    __stcs(reinterpret_cast<float2 *>(out + t * n_embd + col0 + 2 * (v * kThreads + tid)), o2);
                }
            }
        }
        cluster.sync();     // cl_part is reused by the next super-group; also the exit barrier
    }
}

template <int C, int VC, int M, int S>
size_t smem_bytes() {
    return sizeof(float2) * (kMixN / 2) * 4 * VC * 2 * kThreads +
           sizeof(float) * (kWarps * S * M * kSlots + C * S * M * kSlots + S * M * kSlots + S * M * 4);
}

// Per device and kernel variant, looked up once: the shared-memory opt-in and how many clusters the
// device holds at once (0: this variant cannot run here).
template <int C, int VC, int M, int S>
int max_clusters_on_this_device() {
    constexpr int kMaxDevices = 64;
    static int cached[kMaxDevices];          // 0 = not asked yet, -1 = cannot run, > 0 = clusters
    static std::mutex mutex;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return -1; }
    std::lock_guard<std::mutex> lock(mutex);
    if (cached[dev] != 0) return cached[dev];
    auto kernel = hc_pre_cluster_kernel<C, VC, M, S>;
    const size_t smem = smem_bytes<C, VC, M, S>();
    cached[dev] = -1;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = C;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.blockDim = dim3(kThreads);
    cfg.gridDim = dim3(C);
    cfg.dynamicSmemBytes = smem;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n < 1) {
        cudaGetLastError();
        return -1;
    }
    return cached[dev] = n;
}

template <int C, int VC, int M, int S>
bool launch(const float *residual_hc, const uint16_t *hc_fn, const float *hc_scale, const float *hc_base,
            float *post, float *comb, float *out, int64_t n_tokens, int n_embd, float eps, cudaStream_t s) {
    const int max_clusters = max_clusters_on_this_device<C, VC, M, S>();
    if (max_clusters < 1) return false;
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = C;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes<C, VC, M, S>();
    cfg.stream = s;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const int64_t n_super = (n_tokens + S * M - 1) / (S * M);
    const int64_t clusters = n_super < max_clusters ? n_super : max_clusters;
    cfg.gridDim = dim3((unsigned)(clusters * C));
    if (cudaLaunchKernelEx(&cfg, hc_pre_cluster_kernel<C, VC, M, S>, residual_hc, hc_fn, hc_scale, hc_base, post, comb,
                           out, n_tokens, n_embd, eps) != cudaSuccess) {
        cudaGetLastError();        // the caller falls back to another kernel: do not leave the error behind
        return false;
    }
    return true;
}

}  // namespace

// Returns false when the shape has no cluster variant or the launch could not
// be configured; the caller then uses the one-CTA-per-token kernel.
bool hc_pre_rows_cluster(const float *residual_hc, const uint16_t *hc_fn, const float *hc_scale,
                         const float *hc_base, float *post, float *comb, float *out, int64_t n_tokens,
                         int n_embd, float eps, cudaStream_t s) {
    if (!aligned8(residual_hc) || !aligned8(out) || (reinterpret_cast<uintptr_t>(hc_fn) & 3u)) return false;
    // the f32 slice is 24 x 2048 x 4 B = 192 KiB per CTA whatever C is: n_embd = C * 512
    // few tokens: one sub-batch per exchange (lowest latency); batches: four
    if (n_embd == 8 * 512)
        return n_tokens <= 64
            ? launch<8, 1, 4, 1>(residual_hc, hc_fn, hc_scale, hc_base, post, comb, out, n_tokens, n_embd, eps, s)
            : launch<8, 1, 4, 4>(residual_hc, hc_fn, hc_scale, hc_base, post, comb, out, n_tokens, n_embd, eps, s);
    if (n_embd == 4 * 512)
        return n_tokens <= 64
            ? launch<4, 1, 4, 1>(residual_hc, hc_fn, hc_scale, hc_base, post, comb, out, n_tokens, n_embd, eps, s)
            : launch<4, 1, 4, 4>(residual_hc, hc_fn, hc_scale, hc_base, post, comb, out, n_tokens, n_embd, eps, s);
    return false;
}

}  // namespace ds4b200
