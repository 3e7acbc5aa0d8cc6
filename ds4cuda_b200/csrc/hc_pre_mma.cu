// hc_pre_mma.cu — the hyper-connection "pre" step for token batches with the 24 dot
// products per token on the tensor cores.
//
// Arithmetic: cuda/hc_sinkhorn.cu:85-305 of the reference (RMS over the token's 4*n_embd
// residual block, 24 dot products with hc_fn, sigmoid gates, weighted stream sum); the
// Sinkhorn sweeps over the 16 comb values run afterwards in hc_sinkhorn_rows_kernel.
//
// Why tensor cores here and nowhere else in this library: per token the step reads 64 KiB
// but needs 2 * 24 * 16384 = 786 k flops, about 10 flop per byte.  At the HBM rate that is
// ~65 Tflop/s of f32 multiply-adds, the whole SIMT peak of the chip, so a CUDA-core
// version is instruction-bound several times over its memory floor.  The dot products are
// a [tokens x 16384] x [16384 x 24] product, which a warp-level MMA does with a fraction
// of the instructions and no cross-lane reduction.
//
// Precision: hc_fn is f16, which TF32 holds exactly.  Each activation is split into
// hi = x with the low 13 mantissa bits cleared (a TF32 value) and lo = x - hi (exact in
// f32, below 2^-10 |x|), cut to TF32 the same way; both parts are multiplied against the
// same weights, so a product carries x to within 2^-20 |x|, less than the rounding of an
// f32 multiply-add chain of this length.  Accumulation is f32; the hi accumulators are
// restarted every 32 columns and added to running sums with ordinary round-to-nearest
// adds, so the tensor core's internal accumulation rounding never compounds over a long
// chain.
//
// Layout: a thread-block cluster of C CTAs splits the columns as in hc_pre_cluster.cu: CTA
// r keeps hc_fn[:, its 4 x 512 columns] in shared memory for its whole life, as f16 pairs in
// the order the MMA B fragments are read (96 KiB; one conflict-free 32-bit load and two
// exact conversions per fragment, shared by the hi and the lo product).  A step is 16
// tokens (one MMA M tile); warp w of 16 takes the w-th block of 32 columns of each stream
// slice.  The activations of a step arrive in four stages, one per stream: 16 row slices of
// 2 KiB fetched by ONE tiled TMA load into a three-stage ring in shared memory (the box is a
// chunk wider than the slice, which pads the rows to 2112 B and keeps the A fragment loads
// free of bank conflicts), so ~96 KiB of loads per SM stay in flight through the reduction
// and the exchange.  The order of the k index inside an MMA is arbitrary as long as A and B
// agree, so a lane reads whole float4s of a row and feeds element j of them to MMA j.  The
// per-CTA sums are exchanged over distributed shared memory once per step with one blocking
// cluster barrier (the second one is split into an arrive right after the values are read
// and a wait a whole MMA phase later).  The weighted stream sum of a step re-reads its 16
// rows from L2 and is spread over the stages of the next step.
//
// Waits: every wait on a copy is bounded (2^22 polls); if one gives up the kernel raises
// the status bit read by ds4b200_device_status(), carries on with whatever is in the stage
// and terminates normally.
#include <cooperative_groups.h>
#include <cuda.h>

#include <mutex>

#include "device_utils.cuh"
#include "kernels.cuh"

namespace cg = cooperative_groups;

namespace ds4b200 {
namespace {

constexpr int kThreads = 512;
constexpr int kMixN = 24;
constexpr int kVals = 25;             // per token: 24 dots + sum of squares
constexpr int kStepTokens = 16;       // one m16 tile
constexpr int kColsPerCta = 512;      // per stream: 16 blocks of 32 columns, one per warp
constexpr int kPartStride = 26;       // floats per token in the partial buffer (even: float2 stores)
constexpr int kStages = 3;
constexpr int kRowBytes = kColsPerCta * 4;           // 2048: one token's slice of one stream
constexpr int kRowStride = kRowBytes + 64;           // 2112 B = 528 words = 16 mod 32 banks
constexpr int kStageBytes = kStepTokens * kRowStride;
constexpr int kWEntries = 64 * 4 * 3 * 32;           // half2 {b0, b1}: [k-block of 32 cols][j][n tile][lane]

// One tiled TMA load of a 4-D box into shared memory; completion is signalled on `bar`.
// The innermost coordinate is always 0 here (TMA wants it on a 16-byte boundary).
__device__ __forceinline__ void tma_load_4d(void *dst_smem, const CUtensorMap *map, int c0, int c1, int c2, int c3,
                                            uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(smem_addr(dst_smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
          "r"(smem_addr(bar)) : "memory");
}

// D += A(16x8, row) * B(8x8, col), TF32 inputs, f32 accumulate.  Fragment layout (g = lane/4,
// t = lane%4): a0=(g,t) a1=(g+8,t) a2=(g,t+4) a3=(g+8,t+4); b0=(k=t,n=g) b1=(k=t+4,n=g);
// d0=(g,2t) d1=(g,2t+1) d2=(g+8,2t) d3=(g+8,2t+1).
__device__ __forceinline__ void mma_tf32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float elem(const float4 &v, int j) {
    return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w));
}

constexpr uint32_t kTf32Mask = 0xffffe000u;          // sign, exponent, 10 mantissa bits

template <int C>
__global__ void __launch_bounds__(kThreads, 1)
hc_pre_mma_kernel(const __grid_constant__ CUtensorMap x_map, const float *__restrict__ residual_hc,
                  const uint16_t *__restrict__ hc_fn,
                  const float *__restrict__ hc_scale, const float *__restrict__ hc_base,
                  float *__restrict__ post_out, float *__restrict__ comb_out,
                  float *__restrict__ out, int64_t n_tokens, float eps, int *status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char *ring = smem_raw;                                                   // [kStages][16][kRowStride]
    uint32_t *w_h = reinterpret_cast<uint32_t *>(smem_raw + kStages * kStageBytes);   // [kb][j][nt][lane] half2
    float *part = reinterpret_cast<float *>(w_h + kWEntries);           // [8][16][kPartStride]
    float *cl_part = part + 8 * kStepTokens * kPartStride;              // [C][16][kVals]
    float *pre_s = cl_part + C * kStepTokens * kVals;                   // [2][16][4]: this step's and the previous step's
    __shared__ __align__(8) uint64_t full[kStages];     // a stage has landed
    __shared__ __align__(8) uint64_t empty[kStages];    // all 16 warps are done with a stage

    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int64_t cluster_id = blockIdx.x / C, n_clusters = gridDim.x / C;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    constexpr int n_embd = C * kColsPerCta;
    constexpr int64_t hc_dim = 4 * (int64_t)n_embd;
    constexpr int kTokensPerRank = kStepTokens / C;   // tokens whose post/comb this CTA writes
    const int col0 = rank * kColsPerCta;
    const int64_t n_steps = (n_tokens + kStepTokens - 1) / kStepTokens;

    // Stage n of this cluster (n = 4 * local step + stream) into ring slot n % kStages: one tiled
    // TMA load of the box {16 floats, 33 chunks, 1 stream, 16 tokens}, issued by one thread.
    // Tokens past the end of the batch are zero-filled by the copy.
    auto issue_stage = [&](int64_t n) {
        const int64_t step = cluster_id + (n >> 2) * n_clusters;
        if (step >= n_steps) return;
        const int slot = (int)(n % kStages);
        mbar_arrive_expect_tx(&full[slot], kStageBytes);
        tma_load_4d(ring + slot * kStageBytes, &x_map, 0, col0 / 16, (int)(n & 3), (int)(step * kStepTokens), &full[slot]);
    };

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kThreads / 32); }
    }
    __syncthreads();
    if (tid == 0) {
#pragma unroll
        for (int n = 0; n < kStages; ++n) issue_stage(n);
    }

    // ---- resident slice of hc_fn in B-fragment order (the first loads fly meanwhile).
    // Reads are coalesced: the lower half of the CTA takes even (row, stream) pairs, the upper
    // half odd ones; a thread takes columns 2c, 2c+1 of its pair, 6 pairs in flight; the two
    // halves then go to their places in the fragment order.
    {
        uint16_t *w16 = reinterpret_cast<uint16_t *>(w_h);
        const int c2 = tid & 255, odd = tid >> 8;
        int idx[2];                                   // half index of the two columns for row 0, stream 0
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int c = 2 * c2 + q, kb16 = c >> 5, within = c & 31;
            const int e = ((kb16 * 4 + (within & 3)) * 3) * 32 + ((within & 15) >> 2);
            idx[q] = 2 * e + (within >> 4);
        }
        for (int r0 = 0; r0 < kMixN * 4; r0 += 12) {
            uint32_t v[6];
#pragma unroll
            for (int u = 0; u < 6; ++u) {
                const int pair = r0 + 2 * u + odd, row = pair >> 2, h = pair & 3;
                v[u] = __ldg(reinterpret_cast<const uint32_t *>(hc_fn + (int64_t)row * hc_dim + (int64_t)h * n_embd + col0) + c2);
            }
#pragma unroll
            for (int u = 0; u < 6; ++u) {
                const int pair = r0 + 2 * u + odd, row = pair >> 2, h = pair & 3;
                // entry e = (((h*16+kb16)*4+j)*3+nt)*32 + g*4+t: add the row and stream terms
                const int add = 2 * ((h * 16 * 4 * 3 + (row >> 3)) * 32 + (row & 7) * 4);
                w16[idx[0] + add] = (uint16_t)(v[u] & 0xffffu);
                w16[idx[1] + add] = (uint16_t)(v[u] >> 16);
            }
        }
    }
    __syncthreads();

    // The weighted stream sum of a step (re-reading its 16 rows from L2) is spread over the
    // four stages of the NEXT step, one token per thread per stage: thread tid covers float4
    // column c4 of token 4 * stage + (tid >> 7).
    const int c4 = tid & 127;
    auto out_load = [&](int64_t st, int i, float4 (&xr)[4]) {
        const int64_t t = st * kStepTokens + 4 * i + (tid >> 7);
        const float *row = residual_hc + t * hc_dim + col0 + 4 * c4;
#pragma unroll
        for (int h = 0; h < 4; ++h)
            xr[h] = (t < n_tokens) ? ld_stream4(row + (int64_t)h * n_embd) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto out_store = [&](int64_t st, int i, const float4 (&xr)[4], const float *pre) {
        const int m = 4 * i + (tid >> 7);
        const int64_t t = st * kStepTokens + m;
        if (t >= n_tokens) return;
        const float p0 = pre[m * 4 + 0], p1 = pre[m * 4 + 1], p2 = pre[m * 4 + 2], p3 = pre[m * 4 + 3];
        float4 o;
        o.x = xr[0].x * p0 + xr[1].x * p1 + xr[2].x * p2 + xr[3].x * p3;
        o.y = xr[0].y * p0 + xr[1].y * p1 + xr[2].y * p2 + xr[3].y * p3;
        o.z = xr[0].z * p0 + xr[1].z * p1 + xr[2].z * p2 + xr[3].z * p3;
        o.w = xr[0].w * p0 + xr[1].w * p1 + xr[2].w * p2 + xr[3].w * p3;
        st_stream4(out + t * n_embd + col0 + 4 * c4, o);
    };

    int64_t n = 0;                                   // stage counter of this cluster
    int64_t prev_step = -1;                          // step whose weighted sum is still owed
    int local = 0;
    for (int64_t step = cluster_id; step < n_steps; step += n_clusters, ++local) {
        float *pre_cur = pre_s + (local & 1) * (4 * kStepTokens);
        const float *pre_prev = pre_s + ((local & 1) ^ 1) * (4 * kStepTokens);
        float sum[3][4];
        float acc_lo[3][4];
        float ss_a = 0.0f, ss_b = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 3; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) { sum[nt][i] = 0.0f; acc_lo[nt][i] = 0.0f; }

#pragma unroll 1
        for (int h = 0; h < 4; ++h, ++n) {
            float4 xo[4];
            if (prev_step >= 0) out_load(prev_step, h, xo);
            const int slot = (int)(n % kStages);
            mbar_wait_bounded(&full[slot], (uint32_t)(n / kStages) & 1u, status);
            // this warp's 32-column block of the stream slice: rows g and g + 8
            const unsigned char *ra = ring + slot * kStageBytes + g * kRowStride + (warp * 32 + 4 * t4) * 4;
            const float4 xa = *reinterpret_cast<const float4 *>(ra);
            const float4 xb = *reinterpret_cast<const float4 *>(ra + 64);
            const float4 xc = *reinterpret_cast<const float4 *>(ra + 8 * kRowStride);
            const float4 xd = *reinterpret_cast<const float4 *>(ra + 8 * kRowStride + 64);
            ss_a += dot4(xa) + dot4(xb);
            ss_b += dot4(xc) + dot4(xd);
            // This warp is done with the slot: its rows are in registers (the sums above consumed
            // all four loads, so they have returned before the arrive can issue).  The slot is
            // refilled by one lane of a warp that changes from stage to stage (issuing a TMA load
            // costs its warp a few hundred cycles), as soon as all 16 warps have said so; the
            // load then has the whole MMA work of this stage and of the next two to land.  The
            // slot of a step's last stage is refilled later: it first serves as scratch below.
            asm volatile("" ::"f"(ss_a), "f"(ss_b) : "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
            if (h != 3 && lane == 0 && warp == (int)((n + kStages) & 15)) {
                mbar_wait_bounded(&empty[slot], (uint32_t)(n / kStages) & 1u, status);
                issue_stage(n + kStages);
            }
            __syncwarp();
            float acc_hi[3][4];
#pragma unroll
            for (int nt = 0; nt < 3; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc_hi[nt][i] = 0.0f;
            const uint32_t *wk = w_h + (((h * 16 + warp) * 4) * 3) * 32 + lane;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float a[4] = {elem(xa, j), elem(xc, j), elem(xb, j), elem(xd, j)};
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    hi[i] = __float_as_uint(a[i]) & kTf32Mask;
                    lo[i] = __float_as_uint(a[i] - __uint_as_float(hi[i])) & kTf32Mask;
                }
#pragma unroll
                for (int nt = 0; nt < 3; ++nt) {
                    const float2 b = f16x2_bits_to_f32(wk[(j * 3 + nt) * 32]);
                    mma_tf32(acc_hi[nt], hi[0], hi[1], hi[2], hi[3], __float_as_uint(b.x), __float_as_uint(b.y));
                    mma_tf32(acc_lo[nt], lo[0], lo[1], lo[2], lo[3], __float_as_uint(b.x), __float_as_uint(b.y));
                }
            }
#pragma unroll
            for (int nt = 0; nt < 3; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) sum[nt][i] += acc_hi[nt][i];
            if (prev_step >= 0) out_store(prev_step, h, xo, pre_prev);
        }

        // ---- the warps' partial sums for the 16 tokens: warps 0-7 store theirs in `part`, warps
        // 8-15 in the ring slot of the step's last stage, which every warp has released by then
        // (they check) and whose refill waits until the sums below have been read.
        ss_a += __shfl_xor_sync(0xffffffffu, ss_a, 1); ss_a += __shfl_xor_sync(0xffffffffu, ss_a, 2);
        ss_b += __shfl_xor_sync(0xffffffffu, ss_b, 1); ss_b += __shfl_xor_sync(0xffffffffu, ss_b, 2);
        const int last_slot = (int)((n - 1) % kStages);
        float *part_hi = reinterpret_cast<float *>(ring + last_slot * kStageBytes);
        if (warp >= 8) mbar_wait_bounded(&empty[last_slot], (uint32_t)((n - 1) / kStages) & 1u, status);
        float *pa = (warp < 8 ? part : part_hi) + ((warp & 7) * kStepTokens + g) * kPartStride;
        float *pb = pa + 8 * kPartStride;
#pragma unroll
        for (int nt = 0; nt < 3; ++nt) {
            *reinterpret_cast<float2 *>(pa + nt * 8 + 2 * t4) =
                make_float2(sum[nt][0] + acc_lo[nt][0], sum[nt][1] + acc_lo[nt][1]);
            *reinterpret_cast<float2 *>(pb + nt * 8 + 2 * t4) =
                make_float2(sum[nt][2] + acc_lo[nt][2], sum[nt][3] + acc_lo[nt][3]);
        }
        if (t4 == 0) { pa[kMixN] = ss_a; pb[kMixN] = ss_b; }
        __syncthreads();

        // ---- CTA totals, pushed into every CTA of the cluster over DSMEM.  The peers must have
        // finished reading the previous step's values: they said so with the arrive below, a
        // whole MMA phase ago, so this wait hardly ever blocks.
        if (local > 0) cluster.barrier_wait();
        if (tid < kStepTokens * kVals) {
            const int m = tid / kVals, k = tid - m * kVals;
            float s = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) s += part[(w * kStepTokens + m) * kPartStride + k];
#pragma unroll
            for (int w = 0; w < 8; ++w) s += part_hi[(w * kStepTokens + m) * kPartStride + k];
            float *mine = cl_part + rank * kStepTokens * kVals + tid;
#pragma unroll
            for (int r = 0; r < C; ++r) *cluster.map_shared_rank(mine, r) = s;
        }
        cluster.sync();
        // every thread has read the scratch slot: order those generic-proxy accesses before the
        // asynchronous copy, then refill the slot with the third stage of the next step
        if (tid == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue_stage(n - 1 + kStages);
        }

        // ---- gates.  Every CTA computes `pre` for the 16 tokens (identical results: the ranks
        // are summed in the same order everywhere); post and comb of a token are written by one
        // CTA, each kind by its own warps so that the three chains run side by side.
        auto total = [&](int m, int k) {
            float s = 0.0f;
#pragma unroll
            for (int r = 0; r < C; ++r) s += cl_part[(r * kStepTokens + m) * kVals + k];
            return s;
        };
        if (tid < 4 * kStepTokens) {
            const int m = tid >> 2, h = tid & 3;
            const float rms = rms_scale(total(m, kMixN), (float)hc_dim, eps);
            const float zp = (total(m, h) * rms) * hc_scale[0] + hc_base[h];
            pre_cur[m * 4 + h] = 1.0f / (1.0f + expf(-zp)) + eps;
        } else if (tid >= 128 && tid < 128 + 4 * kTokensPerRank) {
            const int m = rank * kTokensPerRank + ((tid - 128) >> 2), h = tid & 3;
            const int64_t t = step * kStepTokens + m;
            if (t < n_tokens) {
                const float rms = rms_scale(total(m, kMixN), (float)hc_dim, eps);
                const float zq = (total(m, 4 + h) * rms) * hc_scale[1] + hc_base[4 + h];
                post_out[t * 4 + h] = 2.0f / (1.0f + expf(-zq));
            }
        } else if (tid >= 256 && tid < 256 + 16 * kTokensPerRank) {
            const int m = rank * kTokensPerRank + ((tid - 256) >> 4), k = tid & 15;
            const int64_t t = step * kStepTokens + m;
            if (t < n_tokens) {
                const float rms = rms_scale(total(m, kMixN), (float)hc_dim, eps);
                comb_out[t * 16 + k] = (total(m, 8 + k) * rms) * hc_scale[2] + hc_base[8 + k];
            }
        }
        cluster.barrier_arrive();                    // this thread no longer reads cl_part
        __syncthreads();                             // pre_cur is complete
        prev_step = step;
    }
    if (local > 0) cluster.barrier_wait();           // pairs with the last arrive; nobody writes here any more
    if (prev_step >= 0) {
        const float *pre_last = pre_s + ((local - 1) & 1) * (4 * kStepTokens);
#pragma unroll 1
        for (int h = 0; h < 4; ++h) {
            float4 xo[4];
            out_load(prev_step, h, xo);
            out_store(prev_step, h, xo, pre_last);
        }
    }
}

// The residual block [T][4][n_embd] seen as a 4-D tensor {16 floats, n_embd/16 chunks, 4 streams,
// T tokens}.  A box of 33 chunks x 16 tokens lands in shared memory as 16 rows of 2112 bytes:
// a CTA's 512 columns plus one chunk of padding, which keeps the MMA A-fragment loads free of
// bank conflicts (row stride = 16 mod 32 banks).  The padding chunk is the neighbour's first 16
// columns, or zero fill past the end of the row.
bool encode_rows_map(CUtensorMap *map, const float *residual_hc, int64_t n_tokens, int n_embd) {
    using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            encode = reinterpret_cast<EncodeFn>(fn);
        else
            cudaGetLastError();
    });
    if (!encode) return false;
    const cuuint64_t dims[4] = {16, (cuuint64_t)n_embd / 16, 4, (cuuint64_t)n_tokens};
    const cuuint64_t strides[3] = {64, (cuuint64_t)n_embd * 4, (cuuint64_t)n_embd * 16};
    const cuuint32_t box[4] = {16, kRowStride / 64, 1, kStepTokens};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(residual_hc), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Per device and cluster width, looked up once: the status word's address, the shared-memory opt-in
// and how many clusters the device holds at once.  Only the tensor map is built per call.
struct DeviceSetup { int *status = nullptr; int max_clusters = 0; bool done = false; };
constexpr int kMaxDevices = 64;
DeviceSetup g_setup[kMaxDevices][2];
std::mutex g_setup_mutex;

template <int C>
constexpr size_t smem_bytes() {
    return (size_t)kStages * kStageBytes + sizeof(uint32_t) * kWEntries +
           sizeof(float) * (8 * kStepTokens * kPartStride + C * kStepTokens * kVals + 2 * kStepTokens * 4);
}

template <int C>
void cluster_config(cudaLaunchConfig_t &cfg, cudaLaunchAttribute &attr, unsigned grid, cudaStream_t s) {
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = C;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.blockDim = dim3(kThreads);
    cfg.gridDim = dim3(grid);
    cfg.dynamicSmemBytes = smem_bytes<C>();
    cfg.stream = s;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
}

template <int C>
const DeviceSetup *device_setup() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return nullptr; }
    DeviceSetup &d = g_setup[dev][C == 8 ? 0 : 1];
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (d.done) return &d;
    d.done = true;
    d.status = device_status_word();
    if (!d.status) return &d;
    auto kernel = hc_pre_mma_kernel<C>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<C>()) != cudaSuccess) {
        cudaGetLastError();
        return &d;
    }
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr{};
    cluster_config<C>(cfg, attr, C, nullptr);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
    d.max_clusters = n;
    return &d;
}

template <int C>
bool launch(const float *residual_hc, const uint16_t *hc_fn, const float *hc_scale, const float *hc_base,
            float *post, float *comb, float *out, int64_t n_tokens, float eps, cudaStream_t s) {
    const DeviceSetup *d = device_setup<C>();
    if (!d || !d->status || d->max_clusters < 1) return false;
    CUtensorMap x_map;
    if (!encode_rows_map(&x_map, residual_hc, n_tokens, C * kColsPerCta)) return false;
    const int64_t n_steps = (n_tokens + kStepTokens - 1) / kStepTokens;
    const int64_t clusters = n_steps < d->max_clusters ? n_steps : d->max_clusters;
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr{};
    cluster_config<C>(cfg, attr, (unsigned)(clusters * C), s);
    if (cudaLaunchKernelEx(&cfg, hc_pre_mma_kernel<C>, x_map, residual_hc, hc_fn, hc_scale, hc_base, post, comb, out,
                           n_tokens, eps, d->status) != cudaSuccess) {
        cudaGetLastError();        // the caller falls back to another kernel: do not leave the error behind
        return false;
    }
    return true;
}

}  // namespace

// Returns false when the shape has no variant here or the launch could not be configured.
bool hc_pre_rows_mma(const float *residual_hc, const uint16_t *hc_fn, const float *hc_scale,
                     const float *hc_base, float *post, float *comb, float *out, int64_t n_tokens,
                     int n_embd, float eps, cudaStream_t s) {
    if (!aligned16(residual_hc) || !aligned16(out)) return false;
    if (n_embd == 8 * kColsPerCta) return launch<8>(residual_hc, hc_fn, hc_scale, hc_base, post, comb, out, n_tokens, eps, s);
    if (n_embd == 4 * kColsPerCta) return launch<4>(residual_hc, hc_fn, hc_scale, hc_base, post, comb, out, n_tokens, eps, s);
    return false;
}

}  // namespace ds4b200
