// hc_pre_tc.cu — the hyper-connection "pre" step for token batches with the 24 dot products
// per token on the fifth-generation tensor cores (tcgen05, accumulators in tensor memory).
//
// Arithmetic: cuda/hc_sinkhorn.cu:85-305 of the reference (RMS over the token's 4*n_embd
// residual block, 24 dot products with hc_fn, sigmoid gates, weighted stream sum, Sinkhorn sweeps over
// the 16 comb values).
//
// Shape of the work: per token the step streams 64 KiB once and needs 2*24*16384 flops, 10
// flop per byte: at the HBM rate that is the whole f32 SIMT peak, and as warp-level MMAs it is
// bound by instruction issue (fragment loads, hi/lo split and mma.sync all compete for the
// same issue slots).  tcgen05.mma is issued by one thread and reads its operands itself, so
// the other warps only move data.
//
// Layout.  A cluster of 16 CTAs splits the 16384 columns of a token row: CTA r owns the
// contiguous columns [1024 r, 1024 r + 1024) and keeps hc_fn[:, those columns] resident in
// shared memory as TF32 (f16 is exact in TF32) in the K-major 128-byte-swizzled layout the
// MMA's B operand wants (32 chunks of 24 rows x 32 columns, 96 KiB).  A step is 64 tokens (the last
// one of a cluster may be shorter, so that the clusters finish together), a stage 128 of the CTA's columns.
//   * one thread streams the stages into a 3-slot ring with tiled TMA loads (no cluster
//     broadcast): a box of 132 columns x 64 tokens lands as rows of 528 bytes, the 16 bytes of
//     padding keep row-per-thread reads off each other's banks;
//   * three groups of four warps take the stages in turn; a group's warps cover the four lane
//     quadrants of tensor memory.  A thread reads one token's row 64 bytes at a time and writes
//     the MMA's A operand straight into tensor memory: quadrants 0 and 2 hold the rows
//     themselves (the tensor core drops the low 13 mantissa bits: the TF32 "hi" part),
//     quadrants 1 and 3 hold lo = x - hi (exact in f32).  Both parts of 64 tokens thus form ONE
//     128-row operand, and one MMA per 8 columns multiplies hi and lo against the same weights;
//     hi and lo keep separate accumulator rows.  The hi threads also accumulate sum(x^2);
//   * one thread issues the MMAs (M=128, N=32 of which 24 are real, K=8).  The tensor core
//     accumulates with truncation, so consecutive stages alternate between two accumulator sets
//     (chains of 64 MMAs) and the sets are added with ordinary f32 adds; accumulators are
//     double-buffered across steps;
//   * the groups take turns draining a finished step's accumulators (a stage into the next step,
//     when its MMAs have long completed) and send each token's partial sums to the CTA that owns
//     the token (4 tokens per CTA per step) over distributed shared memory, announced by a
//     remote mbarrier arrival;
//   * sixteen warps per CTA finish the CTA's own tokens: add the 32 partial records in a fixed
//     order, gates, post values, then the weighted stream sum over the whole 4096-wide
//     row, re-read from L2, where the step's rows still are; two of those warps then run the Sinkhorn
//     sweeps of the step's four tokens, 16 lanes per token.
// Every residual row crosses HBM once; nothing is reduced across clusters; every sum has a fixed
// order that does not depend on the token's place in the batch, so two runs agree bit for bit and
// a token's outputs are the same whether it is computed in a batch of 4096 or in a slice of it.
//
// What the tensor-core unit costs here (measured on B200 with single-CTA probes): every tcgen05
// operation — an MMA of any shape up to N=64, a commit, a shared-to-tensor-memory copy — takes
// about 45 cycles of the unit, so with K=8 per TF32 MMA the stacked hi/lo operand (one MMA per 8
// columns per 64 tokens) is what keeps the unit under the memory time; accumulation rounds
// toward zero (error grows with the chain length); TF32 operands read from f32 words are
// truncated, not rounded; a mbarrier hand-off between two warps costs about 180 cycles, so
// stages are as large as tensor memory allows (128 columns: 3 operand entries + 4 accumulator
// sets fill its 512 columns).  A mbarrier arrival may overtake the same warp's pending
// shared-memory loads: a slot is handed back only after an instruction has consumed them.
//
// Waits.  Every wait is bounded by a cycle budget of about a second; a wait that gives up raises
// the status bit read by ds4b200_device_status() and a CTA-wide flag that makes every later wait
// in the CTA return at once, so the kernel always terminates (with invalid results and the bit
// set).  Control flow is the same in every CTA of a cluster, and no CTA waits for another
// cluster.
#include <cuda.h>

#include <mutex>

#include "device_utils.cuh"
#include "kernels.cuh"

namespace ds4b200 {
namespace {

constexpr int kC = 16;                       // CTAs per cluster
constexpr int kMixN = 24;
constexpr int kStepTokens = 64;
constexpr int kTokensPerCta = kStepTokens / kC;   // tokens a CTA finishes per step
constexpr int kColsPerCta = 1024;            // of the 16384 columns of a token's block
constexpr int kChunkCols = 32;               // 128 bytes: one swizzle row
constexpr int kChunks = kColsPerCta / kChunkCols;
constexpr int kStageChunks = 4;              // chunks handed over together (one barrier round per stage)
constexpr int kStageCols = kStageChunks * kChunkCols;
constexpr int kStages = kChunks / kStageChunks;   // per step
constexpr int kRowBytes = kStageCols * 4 + 16;    // a token's slice of a stage in shared memory: 528 B, an odd
                                                  // number of 16-byte units, so 8 consecutive rows never share a bank
constexpr int kSlotBytes = kStepTokens * kRowBytes;
constexpr int kSlots = 3;
constexpr int kWChunkBytes = kMixN * 128;    // 3 KiB
constexpr int kWBytes = kChunks * kWChunkBytes;   // 96 KiB
constexpr int kRec = 28;                     // floats per partial record: 24 dots, sum of squares, padding
constexpr int kXchFloats = kC * 2 * kTokensPerCta * kRec;   // one exchange buffer
constexpr int kAccSets = 2;
constexpr int kARing = 3;                    // operand entries of kStageChunks x 32 columns in tensor memory
constexpr int kAEntryCols = kStageChunks * 32;
constexpr int kTmemCols = 512;               // 2 x 2 x 32 accumulator columns, 3 x 128 operand columns
constexpr int kThreads = 1024;              // warp 0 copies, 1 MMAs, 4-15 operand writers, 16-31 the CTA's own tokens
constexpr int kPrepWarp0 = 4;
constexpr int kPrepGroups = 3;
constexpr int kTailThreads = 512;
constexpr int kTailWarp0 = 16;
constexpr long long kWaitCycles = 1ll << 31; // about a second

constexpr size_t kSmemBytes = (size_t)kWBytes + (size_t)kSlots * kSlotBytes + 2 * kXchFloats * 4;

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_id() { uint32_t r; asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t n_clusters() { uint32_t r; asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_remote4(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void named_bar(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_addr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_addr(bar)) : "memory");
}
// Shared-memory matrix descriptor: K-major rows of 128 bytes, 128-byte swizzle, 8-row groups
// 1024 bytes apart (descriptor version 1 of sm_100).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    return ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61) |
           (uint64_t)((saddr & 0x3FFFFu) >> 4);
}
// D[tmem] (+)= A[tmem] * B[smem]^T, TF32 inputs, f32 accumulate, issued by one thread.
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The mbarrier receives one arrival when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// Bounded waits on an mbarrier phase.  `cluster_scope`: the arrivals come from other CTAs.
// Every poll is a shared-memory transaction that competes with the arrivals it is waiting for,
// so only the two single-thread roles (copy issuer, MMA issuer) poll back to back; everybody else
// backs off between polls.  The first poll is the common case; only a wait that really blocks
// pays for the clock and the abort flag.
__device__ __forceinline__ bool try_phase(uint64_t *bar, uint32_t parity, bool cluster_scope) {
    uint32_t done;
    if (cluster_scope)
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return done != 0;
}
template <bool TIGHT>
__device__ __noinline__ bool wait_phase_slow(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status,
                                             bool cluster_scope) {
    if (*abort_flag) return false;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            if (!TIGHT) __nanosleep(40);
            if (try_phase(bar, parity, cluster_scope)) return true;
        }
        if (*abort_flag || clock64() - t0 > kWaitCycles) {
            *abort_flag = 1;
            atomicOr(status, kStatusBulkCopyTimeout);
            return false;
        }
    }
}
__device__ __forceinline__ bool wait_phase(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status,
                                           bool cluster_scope = false) {
    if (try_phase(bar, parity, cluster_scope)) return true;
    return wait_phase_slow<false>(bar, parity, abort_flag, status, cluster_scope);
}
__device__ __forceinline__ bool wait_phase_tight(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status) {
    if (try_phase(bar, parity, false)) return true;
    return wait_phase_slow<true>(bar, parity, abort_flag, status, false);
}

__global__ void __launch_bounds__(kThreads, 1)
hc_pre_tc_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap x_map16,
                 const float *__restrict__ residual_hc,
                 const uint16_t *__restrict__ hc_fn, const float *__restrict__ hc_scale,
                 const float *__restrict__ hc_base, float *__restrict__ post_out, float *__restrict__ comb_out,
                 float *__restrict__ out, int64_t n_tokens, int iters, float eps, int *status) {
    constexpr int n_embd = 4096;
    constexpr int64_t hc_dim = 4 * (int64_t)n_embd;
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char *w_s = smem;                                       // [32 chunks][24 rows][128 B]
    unsigned char *ring = smem + kWBytes;                            // [kSlots][64 tokens][kRowBytes]
    float *xch = reinterpret_cast<float *>(ring + kSlots * kSlotBytes);   // [2][16 src][2 parts][4 tokens][kRec]
    __shared__ __align__(8) uint64_t full[kSlots], slot_free[kSlots];
    __shared__ __align__(8) uint64_t a_full[kARing], a_free[kARing];
    __shared__ __align__(8) uint64_t acc_full[2], acc_free[2];
    __shared__ __align__(8) uint64_t xch_full[2], xch_free[2], ss_ready[2];
    __shared__ float ss_part[2][kPrepGroups][kStepTokens];   // sum(x^2) per token, per stage residue mod 3, per step parity
    static_assert(kStages % kPrepGroups == 2 && kPrepGroups == 3, "the residue a group files its share under assumes 8 = 2 mod 3");
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    __shared__ float tot_s[kTokensPerCta][kRec];
    __shared__ float pre_s[kTokensPerCta][4];
    __shared__ float comb_s[2][kTokensPerCta][16];           // comb values before the Sinkhorn sweeps, per step parity
    __shared__ __align__(8) uint64_t comb_ready[2], comb_free[2];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t rank = cluster_rank();
    // Schedule.  `rounds` full steps of 64 tokens per cluster, taken round robin; what is left (fewer than
    // 64 tokens per cluster) is split evenly over the clusters in multiples of 16 tokens and handled as one
    // last, shorter step each (16-token boxes), so no cluster runs a whole extra step while the others idle.
    const int first_step = (int)cluster_id(), step_stride = (int)n_clusters();
    const int rounds = (int)(n_tokens / ((int64_t)kStepTokens * step_stride));
    const int64_t tail_first = (int64_t)rounds * step_stride * kStepTokens;
    const int64_t tail_all = n_tokens - tail_first;                       // < 64 * clusters
    const int tail_share = tail_all > 0 ? (int)(((tail_all + step_stride - 1) / step_stride + 15) / 16) * 16 : 0;
    const int64_t tail_base = tail_first + (int64_t)first_step * tail_share;
    const int tail_count = tail_base < n_tokens ? tail_share : 0;         // tokens past n_tokens are masked below
    const int my_steps = rounds + (tail_count > 0 ? 1 : 0);
#define DS4B200_STEP_BASE(it) ((it) < rounds ? ((int64_t)first_step + (int64_t)(it) * step_stride) * kStepTokens : tail_base)
#define DS4B200_STEP_COUNT(it) ((it) < rounds ? kStepTokens : tail_count)
    volatile int *abort_flag = &abort_s;

    if (tid == 0) {
        abort_s = 0;
        for (int i = 0; i < kSlots; ++i) { mbar_init(&full[i], 1); mbar_init(&slot_free[i], 4); }
        for (int i = 0; i < kARing; ++i) { mbar_init(&a_full[i], 4); mbar_init(&a_free[i], 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1); mbar_init(&acc_free[i], 4);
            mbar_init(&xch_full[i], kC * 2 * kTokensPerCta); mbar_init(&xch_free[i], kC);
            mbar_init(&ss_ready[i], kPrepGroups * 2);
            mbar_init(&comb_ready[i], 2); mbar_init(&comb_free[i], 2);
        }
    }
    __syncthreads();
    if (warp == 1) {      // tensor memory: the whole SM's 512 columns (one CTA per SM)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)), "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    // resident weights: hc_fn[r][1024 rank + k] -> chunk k/32, row r, swizzled 16-byte unit
    for (int u = tid; u < kMixN * (kColsPerCta / 8); u += kThreads) {
        const int r = u / (kColsPerCta / 8), k8 = u - r * (kColsPerCta / 8);     // 8 halves at column 8*k8
        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(hc_fn + (int64_t)r * hc_dim + rank * kColsPerCta + 8 * k8));
        const int c = k8 >> 2, unit = (k8 & 3) * 2;
        unsigned char *row = w_s + c * kWChunkBytes + (r >> 3) * 1024 + (r & 7) * 128;
        const float2 a = f16x2_bits_to_f32(raw.x), b = f16x2_bits_to_f32(raw.y);
        const float2 e = f16x2_bits_to_f32(raw.z), f = f16x2_bits_to_f32(raw.w);
        *reinterpret_cast<float4 *>(row + ((unit ^ (r & 7)) * 16)) = make_float4(a.x, a.y, b.x, b.y);
        *reinterpret_cast<float4 *>(row + (((unit + 1) ^ (r & 7)) * 16)) = make_float4(e.x, e.y, f.x, f.y);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the tensor core reads w_s through the async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    cluster_sync_all();            // every CTA's barriers exist before anybody arrives on them remotely
    const uint32_t tmem = tmem_base_s;
    const uint32_t acc_base = tmem, a_base = tmem + 2 * kAccSets * 32;
    const int total_stages = my_steps * kStages;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int slot = 0;
            uint32_t use_parity = 1;                     // a fresh barrier passes a wait on parity 1
            int it = 0, sg = 0;
            for (int n = 0; n < total_stages; ++n) {
                wait_phase_tight(&slot_free[slot], use_parity, abort_flag, status);
                const int col = (int)(rank * kColsPerCta + sg * kStageCols);
                if (it < rounds) {
                    mbar_arrive_expect_tx(&full[slot], kSlotBytes);
                    tma_load_2d(ring + slot * kSlotBytes, &x_map, col, (int)DS4B200_STEP_BASE(it), &full[slot]);
                } else {                                 // the short last step: 16 tokens per box
                    mbar_arrive_expect_tx(&full[slot], (uint32_t)(tail_count * kRowBytes));
                    for (int j = 0; j < tail_count; j += 16)
                        tma_load_2d(ring + slot * kSlotBytes + j * kRowBytes, &x_map16, col, (int)(tail_base + j), &full[slot]);
                }
                if (++slot == kSlots) { slot = 0; use_parity ^= 1u; }
                if (++sg == kStages) { sg = 0; ++it; }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            // M = 128, N = 32, TF32 x TF32 -> f32, A from tensor memory, B K-major in shared memory
            constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((32u >> 3) << 17) | ((128u >> 4) << 24);
            const uint64_t w_desc = smem_desc(smem_addr(w_s));
            int ar = 0;
            uint32_t a_parity = 0;
            for (int it = 0; it < my_steps; ++it) {
                const int buf = it & 1;
                wait_phase_tight(&acc_free[buf], (((uint32_t)it >> 1) & 1u) ^ 1u, abort_flag, status);
                tc_fence_after();
                for (int sg = 0; sg < kStages; ++sg) {
                    wait_phase_tight(&a_full[ar], a_parity, abort_flag, status);
                    tc_fence_after();
                    const uint32_t d = acc_base + (uint32_t)(buf * kAccSets * 32 + (sg % kAccSets) * 32);
                    const uint32_t a = a_base + (uint32_t)(ar * kAEntryCols);
                    const uint64_t b = w_desc + (uint64_t)((sg * kStageChunks * kWChunkBytes) >> 4);
#pragma unroll
                    for (int h = 0; h < kStageChunks; ++h)
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            mma_tf32_ts(d, a + (uint32_t)(h * 32 + k * 8), b + (uint64_t)(((h * kWChunkBytes) >> 4) + k * 2), idesc,
                                        (sg >= kAccSets || h > 0 || k > 0) ? 1u : 0u);
                    mma_commit(&a_free[ar]);             // a commit costs the tensor pipe about as much as an MMA
                    if (++ar == kARing) { ar = 0; a_parity ^= 1u; }
                }
                mma_commit(&acc_full[buf]);
            }
        }
    } else if (warp == 2 || warp == 3) {
        // ---------------------------------------------------------------- Sinkhorn sweeps, 16 lanes per token
        // (with the sweeps in two of the finishing warps the call took 133 us instead of 120; here they run
        // beside everything else)
        const int m = (warp - 2) * 2 + (lane >> 4), k = lane & 15;
        for (int it = 0; it < my_steps; ++it) {
            const int buf = it & 1;
            const int in_step = (int)rank * kTokensPerCta + m;                 // this token's index within the step
            const int64_t t = in_step < DS4B200_STEP_COUNT(it) ? DS4B200_STEP_BASE(it) + in_step : n_tokens;
            wait_phase(&comb_ready[buf], ((uint32_t)it >> 1) & 1u, abort_flag, status);
            const float v = comb_s[buf][m][k];
            // the first shuffles of the sweeps consume v, so the load has returned before the buffer is handed back
            const float probe = __shfl_sync(0xffffffffu, v, lane ^ 1);
            __syncwarp();
            if (lane == 0)     // `probe` as an operand keeps the arrival behind the shuffle in the instruction stream
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&comb_free[buf])), "f"(probe) : "memory");
            const float c = sinkhorn_4x4_lanes(v, lane, iters, eps);
            if (t < n_tokens) comb_out[t * 16 + k] = c;
        }
    } else if (warp >= kPrepWarp0 && warp < kTailWarp0) {
        // ---------------------------------------------------------------- operand writers / accumulator drain
        // kPrepGroups groups of four warps take the chunks in turn; a group's four warps cover the
        // four lane quadrants of tensor memory.  The groups also take turns draining a step.
        const int group = (warp - kPrepWarp0) >> 2;
        const int q = warp & 3;                          // tensor-memory lane quadrant of this warp
        const int token = (q >> 1) * 32 + lane;          // this thread's token within the step
        const bool is_lo = q & 1;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        const uint32_t owner = (uint32_t)(token / kTokensPerCta);
        const uint32_t row_off = (uint32_t)(token * kRowBytes);
        int slot = group % kSlots, ar = group % kARing;
        uint32_t slot_parity = 0, ar_parity = 0;         // phases of full[slot] and a_full/a_free of entry ar
        static_assert(kSlots % kPrepGroups == 0 && kARing % kPrepGroups == 0, "a group keeps its own slots and entries");
        int next_drain = group;                          // the step this group drains next
        int cur_step = 0;                                // step of chunk n
        float ss0 = 0.0f, ss1 = 0.0f, ss2 = 0.0f, ss3 = 0.0f;
        for (int n = group; ; n += kPrepGroups) {
            // ---- past the end of a step: publish this group's share of sum(x^2)
            const int n_step = n / kStages < my_steps ? n / kStages : my_steps;
            if (n_step > cur_step) {
                // A step has 8 stages and the groups take chunks in turn, so in step `it` this group had the
                // stages sg with sg % 3 == (group + it) % 3, in rising order.  Filed under that residue, the
                // three shares add up in the same order wherever in the batch the token sits.
                if (!is_lo)
                    ss_part[cur_step & 1][(group + cur_step) % kPrepGroups][token] = (ss0 + ss1) + (ss2 + ss3);
                ss0 = ss1 = ss2 = ss3 = 0.0f;
                __syncwarp();
                if (!is_lo && lane == 0) mbar_arrive(&ss_ready[cur_step & 1]);
                cur_step = n_step;
            }
            // ---- a few chunks into the next step (the MMAs of the finished step have completed by
            // then and the issuer has other operands queued): is it this group's turn to drain?
            const int drain_upto = (n - kPrepGroups) / kStages < my_steps && n < total_stages
                                       ? (n - kPrepGroups) / kStages : my_steps;
            while (next_drain < drain_upto) {
                const int it = next_drain;
                next_drain += kPrepGroups;
                const int buf = it & 1;
                const uint32_t ph = ((uint32_t)it >> 1) & 1u;
                wait_phase(&acc_full[buf], ph, abort_flag, status);
                tc_fence_after();
                float accv[kMixN];
#pragma unroll
                for (int set = 0; set < kAccSets; ++set) {
                    uint32_t r[kMixN];
                    const uint32_t src = acc_base + lane_base + (uint32_t)(buf * kAccSets * 32 + set * 32);
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                                   "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                                   "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                                 : "r"(src));
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                 : "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
                                   "=r"(r[21]), "=r"(r[22]), "=r"(r[23])
                                 : "r"(src + 16u));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < kMixN; ++j) accv[j] = set == 0 ? __uint_as_float(r[j]) : accv[j] + __uint_as_float(r[j]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_free[buf]);
                float ssum = 0.0f;
                if (!is_lo) {
                    wait_phase(&ss_ready[buf], ph, abort_flag, status);
#pragma unroll
                    for (int g = 0; g < kPrepGroups; ++g) ssum += ss_part[buf][g][token];
                }
                wait_phase(&xch_free[buf], ph ^ 1u, abort_flag, status, true);
                const uint32_t rec = smem_addr(xch + buf * kXchFloats +
                                               (((int)rank * 2 + (is_lo ? 1 : 0)) * kTokensPerCta + (token % kTokensPerCta)) * kRec);
                const uint32_t dst = map_to_rank(rec, owner);
                // the accumulator sets are added in order
                static_assert(kAccSets == 2, "the drain below adds two sets");
#define DS4B200_ACC(j) (accv[j])
#pragma unroll
                for (int j = 0; j < kMixN; j += 4)
                    st_remote4(dst + 4 * j, DS4B200_ACC(j), DS4B200_ACC(j + 1), DS4B200_ACC(j + 2), DS4B200_ACC(j + 3));
#undef DS4B200_ACC
                st_remote4(dst + 4 * kMixN, ssum, 0.0f, 0.0f, 0.0f);
                mbar_arrive_remote(map_to_rank(smem_addr(&xch_full[buf]), owner));
            }
            if (n >= total_stages) break;
            // ---- stage n, chunk by chunk: this thread's row -> tensor memory (hi: as is; lo: x - tf32(x))
            wait_phase(&full[slot], slot_parity, abort_flag, status);
            wait_phase(&a_free[ar], ar_parity ^ 1u, abort_flag, status);
            tc_fence_after();
#pragma unroll
            for (int h = 0; h < 2 * kStageChunks; ++h) {         // 16 columns (64 bytes of the row) at a time
                const unsigned char *tile = ring + slot * kSlotBytes + row_off + h * 64;
                uint32_t v[16];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 f = *reinterpret_cast<const float4 *>(tile + j * 16);
                    v[4 * j + 0] = __float_as_uint(f.x); v[4 * j + 1] = __float_as_uint(f.y);
                    v[4 * j + 2] = __float_as_uint(f.z); v[4 * j + 3] = __float_as_uint(f.w);
                }
                if (is_lo) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        v[j] = __float_as_uint(__uint_as_float(v[j]) - __uint_as_float(v[j] & 0xffffe000u));
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        ss0 = fmaf(__uint_as_float(v[j]), __uint_as_float(v[j]), ss0);
                        ss1 = fmaf(__uint_as_float(v[j + 1]), __uint_as_float(v[j + 1]), ss1);
                        ss2 = fmaf(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 2]), ss2);
                        ss3 = fmaf(__uint_as_float(v[j + 3]), __uint_as_float(v[j + 3]), ss3);
                    }
                }
                if (h == 2 * kStageChunks - 1) {
                    // the arithmetic above has consumed the stage's last loads, so they have returned:
                    // hand the slot back
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&slot_free[slot]);
                }
                asm volatile(
                    "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                    ::"r"(a_base + lane_base + (uint32_t)(ar * kAEntryCols + h * 16)),
                      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            // the operand entry is written: one lane says so for the warp
            if (lane == 0) mbar_arrive(&a_full[ar]);
            slot += kPrepGroups; if (slot >= kSlots) { slot -= kSlots; slot_parity ^= 1u; }
            ar += kPrepGroups; if (ar >= kARing) { ar -= kARing; ar_parity ^= 1u; }
        }
    } else if (warp >= kTailWarp0) {
        // ---------------------------------------------------------------- the CTA's own tokens
        const int tt = tid - kTailWarp0 * 32;
        for (int it = 0; it < my_steps; ++it) {
            const int buf = it & 1;
            // one thread watches the exchange buffer fill; the others sleep in the hardware barrier
            if (tt == 0) wait_phase(&xch_full[buf], ((uint32_t)it >> 1) & 1u, abort_flag, status, true);
            named_bar(1, kTailThreads);
            if (tt < kTokensPerCta * 25) {
                const int m = tt / 25, k = tt - m * 25;
                const float *p = xch + buf * kXchFloats + m * kRec + k;
                float s = 0.0f;
#pragma unroll
                for (int src = 0; src < kC; ++src) {
                    s += p[(src * 2 + 0) * kTokensPerCta * kRec];
                    s += p[(src * 2 + 1) * kTokensPerCta * kRec];
                }
                tot_s[m][k] = s;
            }
            named_bar(1, kTailThreads);
            // the exchange buffer has been read: the sources may fill it again
            if (tt < kC) mbar_arrive_remote(map_to_rank(smem_addr(&xch_free[buf]), (uint32_t)tt));
            // this CTA's four tokens of the step; in the short last step the ranks past its end have none
            // (their t0 is then n_tokens, which every guard below treats as "no token")
            const int64_t t0 = (int)rank * kTokensPerCta < DS4B200_STEP_COUNT(it)
                                   ? DS4B200_STEP_BASE(it) + (int64_t)rank * kTokensPerCta : n_tokens;
            // warps 16-17: the four tokens' 16 comb values before the Sinkhorn sweeps, handed to warps 2-3 through
            // shared memory; threads 64-79 the pre gates, 80-95 the post gates
            if (tt < 96) {
                const int m = tt < 64 ? tt >> 4 : (tt & 15) >> 2;
                const int64_t t = t0 + m;
                const float rms = rms_scale(tot_s[m][kMixN], (float)hc_dim, eps);
                if (tt < 64) {
                    const int k = tt & 15;
                    wait_phase(&comb_free[buf], (((uint32_t)it >> 1) & 1u) ^ 1u, abort_flag, status);
                    comb_s[buf][m][k] = (tot_s[m][8 + k] * rms) * hc_scale[2] + hc_base[8 + k];
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&comb_ready[buf]);
                } else if (tt < 80) {
                    const int h = tt & 3;
                    const float z = (tot_s[m][h] * rms) * hc_scale[0] + hc_base[h];
                    pre_s[m][h] = 1.0f / (1.0f + expf(-z)) + eps;
                } else {
                    const int h = tt & 3;
                    const float z = (tot_s[m][4 + h] * rms) * hc_scale[1] + hc_base[4 + h];
                    if (t < n_tokens) post_out[t * 4 + h] = 2.0f / (1.0f + expf(-z));
                }
            }
            named_bar(1, kTailThreads);
            // ---- weighted stream sum over the whole row: float4 columns tt and tt + 512 of each stream, so that
            // every load and store of a warp covers 512 contiguous bytes (two adjacent float4 per thread, each
            // instruction touching half of every sector, measured 126 against 120 us).  The loads keep the
            // streaming policy: the rows are dead after this pass, and evict-first lets L2 drop them before the
            // rows of later steps (with ld.global.cg: 134 us).  The four tokens' 16 stream
            // pieces go through a four-deep register window: a piece's registers are reloaded with the next
            // token's piece as soon as it has been used, so the loads of one token overlap the arithmetic
            // and the stores of the previous one, and no barrier separates the tokens.
            // (Requesting a step's first pieces one iteration ahead, before the wait for its partial sums, changed
            // nothing: these warps wait for the copy-and-MMA pipeline, not the other way round.)
            const float *xrow = residual_hc + t0 * hc_dim + 4 * tt;
            float4 win[4][2];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                if (t0 < n_tokens) {
                    win[h][0] = ld_stream4(xrow + (int64_t)h * n_embd);
                    win[h][1] = ld_stream4(xrow + (int64_t)h * n_embd + 2048);
                }
            }
#pragma unroll
            for (int m = 0; m < kTokensPerCta; ++m) {
                const int64_t t = t0 + m;
                if (t >= n_tokens) continue;
                const bool more = m + 1 < kTokensPerCta && t + 1 < n_tokens;
                const float *nrow = xrow + (int64_t)(m + 1) * hc_dim;
                float4 o[2];
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const float p = pre_s[m][h];
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        // x0*p0 + x1*p1 + x2*p2 + x3*p3 in that association, contracted to multiply-adds
                        if (h == 0) o[i] = make_float4(win[0][i].x * p, win[0][i].y * p, win[0][i].z * p, win[0][i].w * p);
                        else o[i] = make_float4(fmaf(win[h][i].x, p, o[i].x), fmaf(win[h][i].y, p, o[i].y),
                                                fmaf(win[h][i].z, p, o[i].z), fmaf(win[h][i].w, p, o[i].w));
                    }
                    if (more) {
                        win[h][0] = ld_stream4(nrow + (int64_t)h * n_embd);
                        win[h][1] = ld_stream4(nrow + (int64_t)h * n_embd + 2048);
                    }
                }
                st_stream4(out + t * n_embd + 4 * tt, o[0]);
                st_stream4(out + t * n_embd + 4 * tt + 2048, o[1]);
            }
        }
    }
#undef DS4B200_STEP_BASE
#undef DS4B200_STEP_COUNT
    // nobody leaves while a peer may still write into its shared memory
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
    }
}

// The residual block as a 2-D tensor {16384 columns, T tokens}.  A box of 132 columns x 64 tokens (16 for the
// short last step) lands as rows of 528 bytes: the stage's 128 columns plus one 16-byte unit of padding (the next columns,
// or zero fill past the end of the row), which keeps the row-per-thread reads of the operand writers
// free of bank conflicts.  Rows past the end of the batch are zero-filled by the copy.
bool encode_rows_map(CUtensorMap *map, const float *residual_hc, int64_t n_tokens, int box_tokens) {
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
    const cuuint64_t dims[2] = {16384, (cuuint64_t)n_tokens};
    const cuuint64_t strides[1] = {65536};
    const cuuint32_t box[2] = {kRowBytes / 4, (cuuint32_t)box_tokens};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(residual_hc), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Per-device launch facts, looked up once: the status word's address and how many clusters of
// 16 the device can hold at once (0: the kernel cannot run here).
struct DeviceSetup { int *status = nullptr; int max_clusters = 0; bool done = false; };
constexpr int kMaxDevices = 64;
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;

const DeviceSetup *device_setup() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return nullptr; }
    DeviceSetup &d = g_setup[dev];
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (d.done) return &d;
    d.done = true;
    auto kernel = hc_pre_tc_kernel;
    d.status = device_status_word();
    if (!d.status) return &d;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        cudaGetLastError();
        return &d;
    }
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = kC; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.blockDim = dim3(kThreads);
    cfg.gridDim = dim3(kC);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
    d.max_clusters = n;
    return &d;
}

bool launch(const float *residual_hc, const uint16_t *hc_fn, const float *hc_scale, const float *hc_base,
            float *post, float *comb, float *out, int64_t n_tokens, int iters, float eps, cudaStream_t s) {
    const DeviceSetup *d = device_setup();
    if (!d || !d->status || d->max_clusters < 1) return false;
    CUtensorMap x_map, x_map16;
    if (!encode_rows_map(&x_map, residual_hc, n_tokens, kStepTokens) || !encode_rows_map(&x_map16, residual_hc, n_tokens, 16))
        return false;
    // as many clusters as fit, unless the batch is so small that 16 tokens each need fewer
    const int64_t n_groups16 = (n_tokens + 15) / 16;
    const int64_t clusters = n_groups16 < d->max_clusters ? n_groups16 : d->max_clusters;
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = kC; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.blockDim = dim3(kThreads);
    cfg.gridDim = dim3((unsigned)(clusters * kC));
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = s;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, hc_pre_tc_kernel, x_map, x_map16, residual_hc, hc_fn, hc_scale, hc_base, post, comb, out,
                           n_tokens, iters, eps, d->status) != cudaSuccess) {
        cudaGetLastError();        // the caller falls back to another kernel: do not leave the error behind
        return false;
    }
    return true;
}

}  // namespace

// Returns false when the shape has no variant here or the launch could not be configured
// (nothing was launched then).
bool hc_pre_rows_tc(const float *residual_hc, const uint16_t *hc_fn, const float *hc_scale, const float *hc_base,
                    float *post, float *comb, float *out, int64_t n_tokens, int n_embd, int iters, float eps,
                    cudaStream_t s) {
    if (n_embd != 4096 || !aligned16(residual_hc) || !aligned16(out) || !aligned16(hc_fn)) return false;
    return launch(residual_hc, hc_fn, hc_scale, hc_base, post, comb, out, n_tokens, iters, eps, s);
}

}  // namespace ds4b200
