// Streaming matrix product for decode steps, fed by bulk asynchronous copies:
// out[M, N] = x[M, K] . w[N, K]^T with M <= 16 tokens.
//
// The kernel is bound by HBM bandwidth: the weights are read exactly once and everything is arranged so that as many
// bytes as possible are in flight per SM without costing registers or issue slots.
//
// A tile is 16 output features. For small N a thread-block cluster of up to 8 CTAs owns a tile and each CTA takes
// a slice of K; for large N the grid is three CTAs per SM and a CTA walks over many tiles, its copy ring running ahead
// into the next tile while the current one is reduced. A producer warp streams the tile's rows into a ring of shared-memory stages with bulk
// asynchronous copies (cp.async.bulk, one per row and stage, completion counted on an mbarrier); eight consumer
// warps wait for a stage, read weight fragments from it with conflict-free 16-byte loads, multiply them with the
// tokens on mma.sync m16n8k16 (bfloat16 in, float accumulation; the tokens are the 8-wide operand) and hand the
// stage back through a second mbarrier. Bytes in flight per SM = resident CTAs x stages x 16 KB.
// The producer issues its first stages BEFORE the kernel waits for its predecessor (weights have no producer kernel),
// and lets the successor be scheduled at once, so the weight stream continues across kernel boundaries.
//
// Partial tiles of the eight warps are added in shared memory in warp order; across a cluster the first CTA reads the
// other CTAs' sums through distributed shared memory in rank order: no global scratch, no atomics, a result that
// does not depend on timing. Every mbarrier wait is bounded; one that runs out raises the status word.
//
// Lane (g, t) of a warp holds elements [8t, 8t+8) of rows g and g+8 of a 32-element chunk. The two MMAs of a chunk
// pair those elements in an order that differs from the natural k order, identically for weights and activations,
// which leaves every dot product unchanged.
//
// For K <= 1536 a tile is one stage and a lane's fragments of the activations are the same in every tile: they are
// read once per CTA, and the RMSNorm that precedes the product in a decoder layer can be applied to them in
// registers (one pass over the float rows, the sum of squares put together from the warps' shares in warp order).
//
// Epilogues: (0) + bias -> bfloat16 or float; (1) + residual (float, may alias out) -> float; (2) SwiGLU for a
// gate/up matrix whose rows are interleaved in blocks of 8 (rows 16b..16b+7 = gate features 8b..8b+7, rows
// 16b+8..16b+15 = the matching up features): out[m, 8b + r] = silu(gate) * up, bfloat16 [M, N/2].
// K must be a multiple of 8 (16-byte alignment of every row); anything else is refused.
#include "common.cuh"

#include <cooperative_groups.h>

IB_DEFINE_LAST_ERROR()

namespace {

namespace cg = cooperative_groups;
using bf16 = __nv_bfloat16;
constexpr int WARPS = 8;                  // consumer warps; warp 8 is the producer
constexpr int THREADS = (WARPS + 1) * 32;
constexpr int ROWS = 16;
#ifndef IB_GEMV_CTAS_PER_SM
#define IB_GEMV_CTAS_PER_SM 2
#endif
constexpr int KC_MAX = 1536;              // most elements of K per stage and row (3 KB)
constexpr int CPW_MAX = KC_MAX / 32 / WARPS;   // most 32-element chunks per warp and stage
constexpr int NS_MAX = 8;                 // most stages in the ring
constexpr int RING_BYTES = 2 * ROWS * (KC_MAX * 2 + 64);
constexpr int NW_BYTES = KC_MAX * 4;         // the fused norm's weight, behind the ring
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr int STATUS_TIMEOUT = 104;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait (about a second): false if the phase did not complete.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; i++) {
        if (mbar_test(bar, parity)) return true;
        if (i > 2048) __nanosleep(64);
    }
    return false;
}
// Weight rows are read once per step: they are marked to leave L2 first, so that streaming the model through it
// does not push out what is read again soon (activations, cache pages, the kernels' own instructions).
#ifndef IB_WEIGHTS_EVICT_FIRST
#define IB_WEIGHTS_EVICT_FIRST 1
#endif
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
#if IB_WEIGHTS_EVICT_FIRST
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
#else
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
#endif
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#ifdef IB_GEMV_TRACE
// Profiling build: the first consumer thread of the first CTA records the SM clock at the kernel's marks.
__device__ long long ib_gemv_trace[64];
#define IB_GT(k) do { if (blockIdx.x == 0 && threadIdx.x == 0 && (k) < 64) ib_gemv_trace[k] = clock64(); } while (0)
#else
#define IB_GT(k) do {} while (0)
#endif

struct GemvParams {
    const bf16* x;            // [M, K]; or, with norm_w, float rows that are RMS-normalised first (K <= KC_MAX)
    const float* norm_w;      // [K] or null
    float eps;
    const bf16* w;            // [N, K]
    const float* bias;        // [N] or null
    const float* residual;    // [M, N] or null
    void* out;
    int M;
    int64_t N, K;
    int cluster;              // CTAs per tile
    int gate_ring;            // 1: the ring's second slot is requested only after the consumers have requested the activations
    int nw_smem;              // 1: the fused norm's weight is staged in shared memory behind the ring by asynchronous
                              //    copies (up to 8 rows of activations; measured: q/k/v 4.1 -> 3.2 us)
    int kc;                   // elements of K per stage and row: a multiple of 64, at most KC_MAX
    int ns;                   // stages in the ring: 2 .. NS_MAX, ns * ROWS * (kc * 2 + 64) <= RING_BYTES
    int64_t tiles;
    int groups;               // tile walkers in the grid (grid = groups * cluster); a walker takes every groups-th tile
    int* status;
    const void* prefetch;     // weights of a later kernel to pull into L2 meanwhile (or null)
    int64_t prefetch_bytes;
};

template <int NT, int EPI, typename TOut, bool NWS>
__global__ void __launch_bounds__(THREADS, 2)
bulk_gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t stages[];   // [ns][ROWS][pitch]
    __shared__ __align__(8) uint64_t bars[2 * NS_MAX + 1]; // full[ns], empty[ns], activations requested
    __shared__ float red[WARPS][NT][8][ROWS];
    __shared__ float part[NT][8][ROWS];                  // this CTA's sum; read by the cluster's first CTA
    __shared__ float sumsq[WARPS][NT * 8];               // the warps' shares of a row's sum of squares (fused norm)
    __shared__ int failed;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int cluster = p.cluster;
    const int rank = cluster > 1 ? int(blockIdx.x % cluster) : 0;
    const int group = blockIdx.x / cluster;              // this CTA walks tiles group, group + groups, ...
    const int64_t K = p.K, N = p.N;
    const int KC = p.kc, NS = p.ns;
    const int PITCH = KC * 2 + 64;                       // bytes between rows of a stage: consecutive rows start 16 banks apart
    const int STAGE_BYTES = ROWS * PITCH;
    // This CTA's slice of K, in stages of KC elements.
    const int64_t total_stages = (K + KC - 1) / KC;
    const int64_t per_cta = (total_stages + cluster - 1) / cluster;
    const int64_t s_begin = min(total_stages, rank * per_cta), s_end = min(total_stages, s_begin + per_cta);
    const int spt = int(s_end - s_begin);                // stages per tile
    const int64_t my_tiles = group < p.tiles ? (p.tiles - group + p.groups - 1) / p.groups : 0;
    const int64_t n_iter = my_tiles * spt;
    const uint32_t stage0 = smem_u32(stages), bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (NS_MAX + s); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), WARPS); }
        mbar_init(bar0 + 8u * (2 * NS_MAX), WARPS);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Rows beyond N (last tile only) are never copied: start from zeros. A stage that held an earlier tile's rows is
    // harmless there, because those rows' results are not stored.
    if (N % ROWS != 0 && (p.tiles - 1 - group) % p.groups == 0) {     // this CTA takes the last, partial tile
        for (int i = threadIdx.x; i < RING_BYTES / 16; i += THREADS) reinterpret_cast<uint4*>(stages)[i] = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == WARPS) {
        // ---------------------------------------------------------------- producer: lane r copies row r of every stage
        // (ring slot, its use count, stage within the tile and tile are carried along: 64-bit divisions by run-time
        // values would cost more per stage than the copies)
        int s = 0, st = 0;
        uint32_t round = 0;
        int64_t tile = group;
        const uint64_t once = policy_evict_first();
        for (int64_t i = 0; i < n_iter; i++) {
            if (i == 1 && p.gate_ring) {
                // With every SM's ring being filled at once, activations requested after the dependency wait would
                // queue behind megabytes of weights and the consumers would start microseconds late: the second slot
                // waits until the consumers have sent their requests.
                int ok = 1;
                if (lane == 0) ok = mbar_wait(bar0 + 8u * (2 * NS_MAX), 0) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { if (lane == 0) { atomicExch(p.status, STATUS_TIMEOUT); failed = 1; } break; }
            }
            if (i >= NS) {
                int ok = 1;
                if (lane == 0) ok = mbar_wait(empty_bar(s), (round - 1) & 1u) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { if (lane == 0) { atomicExch(p.status, STATUS_TIMEOUT); failed = 1; } break; }
            }
            const int64_t n0 = tile * ROWS;
            const int64_t k0 = (s_begin + st) * KC;
            const int live_rows = int(min(int64_t(ROWS), N - n0));
            const uint32_t bytes = uint32_t(min(int64_t(KC), K - k0) * 2);
            if (lane == 0) mbar_expect_tx(full_bar(s), bytes * uint32_t(live_rows));
            __syncwarp();
            if (lane < live_rows) bulk_load(stage0 + s * STAGE_BYTES + lane * PITCH, p.w + (n0 + lane) * K + k0, bytes, full_bar(s), once);
            if (i == NS - 1 || i == n_iter - 1) ib::pdl_launch_dependents();     // the first ring is on its way
            if (++s == NS) { s = 0; round++; }
            if (++st == spt) { st = 0; tile += p.groups; }
        }
        if (n_iter == 0) ib::pdl_launch_dependents();
        ib::l2_prefetch_share(p.prefetch, p.prefetch_bytes, blockIdx.x, gridDim.x);
        if (cluster > 1) {                               // the cluster barriers below count every thread
            cg::cluster_group cl = cg::this_cluster();
            cl.sync();
            cl.sync();
        }
        return;
    }
    // -------------------------------------------------------------------- consumers (warps 0..7)
    IB_GT(0);
    // The norm's weight does not come from the predecessor: it goes into shared memory behind the ring now (up to 8 rows:
    // with 16 the static arrays leave no room beside a second CTA, and it is fetched into L1 instead).
    float* nw_s = reinterpret_cast<float*>(stages + RING_BYTES);
    constexpr bool NW_SMEM = NWS;              // (a template parameter: as a run-time flag it cost 1 us per kernel)
    if (p.norm_w) {
        if constexpr (NW_SMEM) {
            // asynchronous copies, awaited only where the weight is used: a CTA that starts after its predecessor has
            // finished (most of gate/up's) then has this trip to L2 and the activations' in flight together
            for (int64_t k = threadIdx.x * 4; k < K; k += WARPS * 32 * 4)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(nw_s + k)), "l"(p.norm_w + k) : "memory");
            asm volatile("cp.async.commit_group;" ::: "memory");
        } else {
#pragma unroll
            for (int u = 0; u < CPW_MAX; u++) {
                const int64_t k = (warp + u * WARPS) * 32 + t * 8;
                if (k < K) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.norm_w + k));
            }
        }
    }
    ib::pdl_wait();                                      // activations come from the predecessor
    IB_GT(1);
    bool x_ok[NT];
    const bf16* xr[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        x_ok[nt] = nt * 8 + g < p.M;
        xr[nt] = p.x + int64_t(nt * 8 + g) * K + t * 8;
    }
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    constexpr int CPW = CPW_MAX;                         // warp w takes the 32-element chunks w, w + 8, ... of a stage
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
    const bool active = threadIdx.x < NT * 128;
    const int r = threadIdx.x & 15, col = (threadIdx.x >> 4) & 7, ant = active ? threadIdx.x >> 7 : 0;
    TOut* out = reinterpret_cast<TOut*>(p.out);

    // With one stage per tile a lane multiplies the same fragments of the activations in every tile: they are
    // fetched, and normalised if the kernel is given the float residual stream, once.
    const bool hoist = total_stages == 1;
    uint4 b[CPW][NT];
    bool k_ok[CPW];
    if (hoist && n_iter > 0) {
#pragma unroll
        for (int u = 0; u < CPW; u++) k_ok[u] = (warp + u * WARPS) * 32 < KC && (warp + u * WARPS) * 32 + t * 8 < K;
        if (p.norm_w) {
            const float* h = reinterpret_cast<const float*>(p.x);
            uint4 hi[CPW][NT];                           // b holds the first four floats of a fragment meanwhile, hi the rest
            float ss[NT];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) ss[nt] = 0.0f;
#pragma unroll
            for (int u = 0; u < CPW; u++) {
                const int64_t k = (warp + u * WARPS) * 32 + t * 8;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const uint4* src = reinterpret_cast<const uint4*>(h + int64_t(nt * 8 + g) * K + k);
                    b[u][nt] = (k_ok[u] && x_ok[nt]) ? src[0] : zero;
                    hi[u][nt] = (k_ok[u] && x_ok[nt]) ? src[1] : zero;
                }
            }
            if (lane == 0) mbar_arrive(bar0 + 8u * (2 * NS_MAX));        // the requests are out: the producer may go on
            auto sq = [](float a, uint4 q) {
                a = fmaf(__uint_as_float(q.x), __uint_as_float(q.x), a);
                a = fmaf(__uint_as_float(q.y), __uint_as_float(q.y), a);
                a = fmaf(__uint_as_float(q.z), __uint_as_float(q.z), a);
                return fmaf(__uint_as_float(q.w), __uint_as_float(q.w), a);
            };
#pragma unroll
            for (int u = 0; u < CPW; u++) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++) ss[nt] = sq(sq(ss[nt], b[u][nt]), hi[u][nt]);
            }
            IB_GT(60);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                ss[nt] += __shfl_xor_sync(0xffffffffu, ss[nt], 1);
                ss[nt] += __shfl_xor_sync(0xffffffffu, ss[nt], 2);
                if (t == 0) sumsq[warp][nt * 8 + g] = ss[nt];
            }
            if constexpr (NW_SMEM) asm volatile("cp.async.wait_all;" ::: "memory");      // the norm's weight: visible after the barrier
            asm volatile("bar.sync 1, 256;" ::: "memory");
            IB_GT(61);
            float scale[NT];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                float total = 0.0f;
#pragma unroll
                for (int wi = 0; wi < WARPS; wi++) total += sumsq[wi][nt * 8 + g];   // warp order: the same for every batch
                scale[nt] = rsqrtf(total / float(K) + p.eps);
            }
            auto pack = [](float lo, float hi2) {
                __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi2);
                return *reinterpret_cast<uint32_t*>(&v);
            };
#pragma unroll
            for (int u = 0; u < CPW; u++) {
                const int64_t k = (warp + u * WARPS) * 32 + t * 8;
                float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f), w1 = w0;
                if (k_ok[u]) {
                    if constexpr (NW_SMEM) {
                        w0 = *reinterpret_cast<const float4*>(nw_s + k);
                        w1 = *reinterpret_cast<const float4*>(nw_s + k + 4);
                    } else {
                        w0 = __ldg(reinterpret_cast<const float4*>(p.norm_w + k));
                        w1 = __ldg(reinterpret_cast<const float4*>(p.norm_w + k) + 1);
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const uint4 lo = b[u][nt], up = hi[u][nt];
                    const float sc = scale[nt];
                    b[u][nt] = make_uint4(pack(__uint_as_float(lo.x) * sc * w0.x, __uint_as_float(lo.y) * sc * w0.y),
                                          pack(__uint_as_float(lo.z) * sc * w0.z, __uint_as_float(lo.w) * sc * w0.w),
                                          pack(__uint_as_float(up.x) * sc * w1.x, __uint_as_float(up.y) * sc * w1.y),
                                          pack(__uint_as_float(up.z) * sc * w1.z, __uint_as_float(up.w) * sc * w1.w));
                }
            }
        } else {
#pragma unroll
            for (int u = 0; u < CPW; u++) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
                    b[u][nt] = (k_ok[u] && x_ok[nt]) ? __ldg(reinterpret_cast<const uint4*>(xr[nt] + (warp + u * WARPS) * 32)) : zero;
            }
            if (lane == 0) mbar_arrive(bar0 + 8u * (2 * NS_MAX));
        }
    } else if (lane == 0) {
        mbar_arrive(bar0 + 8u * (2 * NS_MAX));
    }

    IB_GT(2);
    int s = 0, st = 0;
    uint32_t round = 0;
    int64_t tile = group;
    for (int64_t i = 0; i < n_iter; i++) {
        const int64_t k0 = (s_begin + st) * KC;
        IB_GT(4 + 4 * int(i));
        if (!hoist) {
            // activations of this warp's chunks: independent of the weights, so they are loaded before the wait
#pragma unroll
            for (int u = 0; u < CPW; u++) {
                const int64_t k = k0 + (warp + u * WARPS) * 32;
                k_ok[u] = (warp + u * WARPS) * 32 < KC && k + t * 8 < K;
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
                    b[u][nt] = (k_ok[u] && x_ok[nt]) ? __ldg(reinterpret_cast<const uint4*>(xr[nt] + k)) : zero;
            }
        }
        if (!mbar_wait(full_bar(s), round & 1u)) {
            if (lane == 0) { atomicExch(p.status, STATUS_TIMEOUT); failed = 1; }
            break;
        }
        IB_GT(5 + 4 * int(i));
        const uint8_t* stg = stages + s * STAGE_BYTES;
#pragma unroll
        for (int u = 0; u < CPW; u++) {
            const int cb = ((warp + u * WARPS) * 32 + t * 8) * 2;
            const uint4 a0 = k_ok[u] ? *reinterpret_cast<const uint4*>(stg + g * PITCH + cb) : zero;
            const uint4 a1 = k_ok[u] ? *reinterpret_cast<const uint4*>(stg + (g + 8) * PITCH + cb) : zero;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                mma_bf16(acc[nt], a0.x, a1.x, a0.y, a1.y, b[u][nt].x, b[u][nt].y);
                mma_bf16(acc[nt], a0.z, a1.z, a0.w, a1.w, b[u][nt].z, b[u][nt].w);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(s));
        IB_GT(6 + 4 * int(i));
        if (++s == NS) { s = 0; round++; }
        if (++st != spt) continue;
        st = 0;

        // ---------------------------------------------------------------- the tile is complete
        const int64_t this_tile = tile;
        tile += p.groups;
        const int64_t n0 = this_tile * ROWS;
        asm volatile("bar.sync 1, 256;" ::: "memory");   // the previous tile's sums have been read (consumers only)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            red[warp][nt][2 * t][g] = acc[nt][0];
            red[warp][nt][2 * t + 1][g] = acc[nt][1];
            red[warp][nt][2 * t][g + 8] = acc[nt][2];
            red[warp][nt][2 * t + 1][g + 8] = acc[nt][3];
            acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        float v = 0.0f;
        if (active) {
#pragma unroll
            for (int wi = 0; wi < WARPS; wi++) v += red[wi][ant][col][r];
        }
        bool writer = true;
        if (cluster > 1) {
            cg::cluster_group cl = cg::this_cluster();
            if (active) part[ant][col][r] = v;
            cl.sync();
            if (rank == 0 && active) {
                for (int other = 1; other < cluster; other++)
                    v += cl.map_shared_rank(&part[0][0][0], other)[(ant * 8 + col) * ROWS + r];
            }
            cl.sync();                                   // the others' shared memory stays alive until it was read
            writer = rank == 0;
        }
        if (EPI == 2 && writer) {
            if (active) part[ant][col][r] = v;           // the SwiGLU epilogue pairs rows r and r + 8
            asm volatile("bar.sync 1, 256;" ::: "memory");
        }
        const int m = ant * 8 + col;
        IB_GT(7 + 4 * int(i));
        if (!writer || !active || m >= p.M || failed) continue;
        if constexpr (EPI == 2) {
            if (r < 8) {
                const float gate = v, up = part[ant][col][r + 8];
                const int64_t f = this_tile * 8 + r;
                if (f < N / 2) out[int64_t(m) * (N / 2) + f] = ib::from_f32<TOut>(gate / (1.0f + expf(-gate)) * up);
            }
        } else {
            const int64_t n = n0 + r;
            if (n < N) {
                if (p.bias) v += p.bias[n];
                if constexpr (EPI == 1) v += p.residual[int64_t(m) * N + n];
                out[int64_t(m) * N + n] = ib::from_f32<TOut>(v);
            }
        }
    }
}

template <int NT>
int launch(const GemvParams& p, int out_dtype, int epi, int grid_ctas, cudaStream_t stream) {
    const dim3 grid{unsigned(grid_ctas), 1u, 1u};
    const dim3 block{THREADS, 1u, 1u};
    const unsigned cl = unsigned(p.cluster);
#define IB_GEMV_LAUNCH_(EPI_, T_, NWS_)                                                                            \
    do {                                                                                                           \
        static bool configured = false;                                                                            \
        if (!configured) {                                                                                         \
            cudaError_t e = cudaFuncSetAttribute(bulk_gemv_kernel<NT, EPI_, T_, NWS_>,                             \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, RING_BYTES + NW_BYTES); \
            if (e != cudaSuccess) return ib::fail(IB_ERR_CUDA, "linear_skinny_bulk: cannot set shared memory size: %s", cudaGetErrorString(e)); \
            configured = true;                                                                                     \
        }                                                                                                          \
        return ib::launch("linear_skinny_bulk", bulk_gemv_kernel<NT, EPI_, T_, NWS_>, grid, block,                 \
                          size_t(RING_BYTES) + (NWS_ ? size_t(NW_BYTES) : 0), stream, cl, p);                      \
    } while (0)
#define IB_GEMV_LAUNCH(EPI_, T_)                                                                                   \
    do {                                                                                                           \
        if (NT == 1 && p.norm_w && p.nw_smem) IB_GEMV_LAUNCH_(EPI_, T_, true);                                     \
        IB_GEMV_LAUNCH_(EPI_, T_, false);                                                                          \
    } while (0)
    if (epi == 2) {
        if (out_dtype != IB_BF16) return ib::fail(IB_ERR_ARG, "linear_skinny_bulk: the SwiGLU epilogue writes bfloat16");
        IB_GEMV_LAUNCH(2, bf16);
    }
    if (epi == 1) {
        if (out_dtype != IB_F32 || !p.residual) return ib::fail(IB_ERR_ARG, "linear_skinny_bulk: the residual epilogue needs a float residual and output");
        IB_GEMV_LAUNCH(1, float);
    }
    if (out_dtype == IB_F32) IB_GEMV_LAUNCH(0, float);
    if (out_dtype == IB_BF16) IB_GEMV_LAUNCH(0, bf16);
#undef IB_GEMV_LAUNCH
#undef IB_GEMV_LAUNCH_
    return ib::fail(IB_ERR_ARG, "linear_skinny_bulk: unknown output dtype %d", out_dtype);
}

}  // namespace

// x: bfloat16 [M, K]; with norm_w (float [K]) x is float [M, K] and is RMS-normalised (eps norm_eps) on the way in,
// each CTA once for all its tiles (K <= 1536). epi: 0 = (+ bias), 1 = (+ bias) + residual -> float, 2 = SwiGLU over rows interleaved by 8 ->
// bfloat16 [M, N/2]. cluster: CTAs that share a tile's K range (1, 2, 4 or 8); 0 lets the kernel choose from N, K and
// sm_count. status: one int in device memory, raised if a bounded wait runs out.
// What this kernel takes: the most rows of activations, and the longest row that the fused RMSNorm prologue
// normalises in registers. Callers plan with these figures instead of carrying copies of them.
IB_EXPORT int ib_linear_skinny_bulk_limits(int* max_rows, int* max_fused_norm_k) {
    if (max_rows) *max_rows = ROWS;
    if (max_fused_norm_k) *max_fused_norm_k = KC_MAX;
    return IB_OK;
}

IB_EXPORT int ib_linear_skinny_bulk(const void* x, const float* norm_w, float norm_eps, const void* w, const float* bias, const float* residual, void* out,
                                    int64_t M, int64_t N, int64_t K, int out_dtype, int epi, int cluster, int sm_count,
                                    int* status, const void* prefetch, int64_t prefetch_bytes, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IB_OK;
    if (M > 16) return ib::fail(IB_ERR_ARG, "linear_skinny_bulk: at most 16 rows, got %lld", (long long)M);
    if (K <= 0 || K % 8) return ib::fail(IB_ERR_ARG, "linear_skinny_bulk: K = %lld must be a positive multiple of 8", (long long)K);
    if ((uintptr_t(x) & 15) || (uintptr_t(w) & 15)) return ib::fail(IB_ERR_ARG, "linear_skinny_bulk: operands must be 16-byte aligned");
    if (epi == 2 && N % 16) return ib::fail(IB_ERR_ARG, "linear_skinny_bulk: the SwiGLU epilogue needs N to be a multiple of 16");
    if (!status) return ib::fail(IB_ERR_ARG, "linear_skinny_bulk: a status word is required");
    if (norm_w && (K > KC_MAX || (uintptr_t(norm_w) & 15)))
        return ib::fail(IB_ERR_ARG, "linear_skinny_bulk: the fused norm takes K <= %d and a 16-byte aligned weight", KC_MAX);
    if (norm_w && cluster > 1) return ib::fail(IB_ERR_ARG, "linear_skinny_bulk: the fused norm does not share a tile among CTAs");
    const int64_t tiles = (N + ROWS - 1) / ROWS;
    if (tiles > 0x7fffffffLL / 8) return ib::fail(IB_ERR_ARG, "linear_skinny_bulk: N too large");
    const int sms = sm_count > 0 ? sm_count : 148;
    // A stage holds ROWS rows of kc elements: K in as few equal stages as the ring allows (a whole row for K up to
    // KC_MAX), since the cost of a stage (its copies, the barrier round trip) does not depend on its size.
    int64_t n_stages = (K + KC_MAX - 1) / KC_MAX;
    if (cluster == 0) {
        // Share a tile among CTAs while the tiles alone leave SMs idle and every CTA keeps at least three stages of K
        // (measured on B200 for K = 8960: 10.8 us alone, 8.9 us in pairs, 14.4 us in fours; clusters of three or six
        // run slower still).
        cluster = 1;
        while (cluster < 8 && tiles * cluster < 2LL * sms && n_stages >= 6 * cluster) cluster *= 2;
    }
    if (cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) return ib::fail(IB_ERR_ARG, "linear_skinny_bulk: cluster must be 1, 2, 4 or 8");
    n_stages = (n_stages + cluster - 1) / cluster * cluster;     // the same number of stages for every CTA of a cluster
    const int kc = int(((K + n_stages - 1) / n_stages + 63) / 64 * 64);
    int ns = RING_BYTES / (ROWS * (kc * 2 + 64));
    if (ns > NS_MAX) ns = NS_MAX;
    GemvParams p;
    p.x = (const bf16*)x; p.norm_w = norm_w; p.eps = norm_eps; p.w = (const bf16*)w; p.bias = bias; p.residual = residual; p.out = out;
    p.M = int(M); p.N = N; p.K = K; p.cluster = cluster; p.status = status; p.tiles = tiles; p.kc = kc; p.ns = ns;
    // gate the ring's second slot where the whole GPU's rings fill at once (a CTA per half SM) and a tile is one stage
    p.gate_ring = (n_stages == 1 && cluster == 1 && tiles >= 2LL * sms) ? 1 : 0;
    p.nw_smem = norm_w ? 1 : 0;
    p.prefetch = prefetch; p.prefetch_bytes = prefetch_bytes & ~int64_t(15);
    // Two CTAs fit an SM; with more tiles than that, a CTA walks over several and its ring never drains between them.
    constexpr int64_t PER_SM = IB_GEMV_CTAS_PER_SM;
    int64_t groups = cluster > 1 ? tiles : (tiles < PER_SM * sms ? tiles : PER_SM * sms);
    p.groups = int(groups);
    const int grid_ctas = int(groups) * cluster;
    if (M <= 8) return launch<1>(p, out_dtype, epi, grid_ctas, stream);
    return launch<2>(p, out_dtype, epi, grid_ctas, stream);
}

#ifdef IB_GEMV_TRACE
IB_EXPORT int ib_linear_skinny_bulk_trace(long long* host) {
    return cudaMemcpyFromSymbol(host, ib_gemv_trace, sizeof(ib_gemv_trace)) == cudaSuccess ? IB_OK : IB_ERR_CUDA;
}
#endif
