// A chain of skinny matrix products in ONE kernel, for decode steps (M <= 16 tokens):
//
//     phase p:   out_p[M, N_p] = epilogue_p( f_p(x_p)[M, K_p] . w_p[N_p, K_p]^T )        p = 0 .. n-1 (n <= 4)
//
// where each phase reads what an earlier phase wrote (f_p is the identity or an RMSNorm of the float residual
// stream). A decode layer is such a chain: attention output -> o product + residual -> norm -> gate/up product +
// SwiGLU -> down product + residual -> (next layer's) norm -> q/k/v product + bias. Run as separate kernels, each
// product pays a launch, a ramp-up and a tail of several microseconds, during which HBM idles; at batch 8 those
// gaps are most of the step.
//
// Here the grid is launched cooperatively (every CTA resident), and
//   * a producer warp per CTA streams the weight rows of the CTA's tiles, phase after phase, into a ring of
//     shared-memory slots with bulk asynchronous copies (cp.async.bulk + mbarrier). Weights do not depend on
//     anything a phase computes, so the producer never waits for a phase boundary: while the consumers of a CTA sit
//     at the grid barrier, the first tiles of the next phase are already arriving. A slot holds 16 rows of up to
//     1536 elements (a whole row of the weight for K <= 1536: the cost of a stage, its copies and its barrier round
//     trip, does not depend on its size);
//   * eight consumer warps multiply (mma.sync m16n8k16; the tokens are the 8-wide operand). Warp w takes the
//     32-element chunks w, w + 8, ... of a stage. Its fragments of the activations live in registers: for K <= 1536
//     they are the same for every tile of the phase and are fetched (and normalised) once per phase; for longer K
//     they are fetched through L2 one stage ahead. The warps' partial tiles are added in shared memory in warp order
//     and the phase's epilogue runs;
//   * between phases the consumers meet at a grid-wide barrier (an arrival counter in global memory that the last
//     CTA to leave the kernel resets). Activations that another CTA wrote are read with ld.global.cg, past the L1.
//
// A tile is 16 output features, or 8 when a one-stage phase has too few 16-row tiles to give every CTA one.
// Every wait (mbarrier, grid barrier) is bounded; one that runs out raises the status word and an abort flag that
// makes the other CTAs leave as well (the barrier words then have to be zeroed by the host before the next launch).
//
// Epilogues: 0 (+ bias) -> bfloat16; 1 += into the float residual stream (in place); 2 SwiGLU over rows interleaved
// in blocks of 8 (8 gate rows, then the 8 matching up rows; 16-row tiles only) -> bfloat16 [M, N/2].
// The sum of a dot product is formed in an order that depends on K alone, so a token's result does not depend on
// the other rows of the batch.
#include "common.cuh"

IB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;
constexpr int WARPS = 8;                  // consumer warps; warp 8 is the producer
constexpr int THREADS = (WARPS + 1) * 32;
constexpr int KC_MAX = 1536;              // most elements of K per stage and row (3 KB)
constexpr int CPW = KC_MAX / 32 / WARPS;  // most 32-element chunks per warp and stage
constexpr int PITCH = KC_MAX * 2 + 64;    // bytes between rows of a slot: consecutive rows start 16 banks apart
constexpr int SLOT_BYTES = 16 * PITCH;
constexpr int MAX_PHASES = 4;
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr int STATUS_TIMEOUT = 105;
template <int NT> struct Geometry { static constexpr int NS = NT == 1 ? 2 : 4; };   // slots in the ring (2 or 1 CTAs per SM)

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
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t ld_acquire(const unsigned int* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

#ifdef IB_CHAIN_TRACE
// Profiling build: every CTA records the global timer at the marks of each phase (thread 0 only).
constexpr int TRACE_MARKS = 4;            // per phase: barrier passed, activations ready, first stage arrived, tiles done
__device__ long long ib_trace[1024][1 + MAX_PHASES * TRACE_MARKS];
__device__ __forceinline__ long long now_ns() { long long v; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v)); return v; }
#define IB_MARK(phase, mark) do { if (threadIdx.x == 0 && blockIdx.x < 1024) ib_trace[blockIdx.x][1 + (phase) * TRACE_MARKS + (mark)] = now_ns(); } while (0)
#define IB_MARK0() do { if (threadIdx.x == 0 && blockIdx.x < 1024) ib_trace[blockIdx.x][0] = now_ns(); } while (0)
__device__ long long ib_stage_trace[MAX_PHASES][32][8];    // CTA 0: stage entered, weights arrived, multiplied; epilogue marks
#define IB_STAGE_MARK(phase, j, mark) do { if (threadIdx.x == 0 && blockIdx.x == 0 && (j) < 32) ib_stage_trace[phase][j][mark] = clock64(); } while (0)
#else
#define IB_STAGE_MARK(phase, j, mark) do {} while (0)
#define IB_MARK(phase, mark) do {} while (0)
#define IB_MARK0() do {} while (0)
#endif

struct Phase {
    const bf16* w;            // [N, K]
    int64_t N, K;
    int rows;                 // rows per tile: 16, or 8 (one-stage phases only)
    int kc;                   // elements of K per stage: a multiple of 64, at most KC_MAX
    int spt;                  // stages per tile: ceil(K / kc)
    int x_kind;               // 0: bfloat16 activations; 1: RMSNorm of float rows (one-stage phases only)
    const void* x;            // bf16 [M, K] (kind 0) or float [M, K] (kind 1)
    const float* norm_w;      // [K] (kind 1)
    float eps;
    int epi;                  // 0: (+ bias) -> bf16; 1: += float residual stream in place; 2: SwiGLU -> bf16 [M, N/2]
    const float* bias;        // [N] or null
    void* out;                // bf16 [M, N] / float [M, N] (the residual stream) / bf16 [M, N/2]
};

struct ChainParams {
    Phase ph[MAX_PHASES];
    int n_phases;
    int M;
    unsigned int* barrier;    // [0] arrivals, [1] departures, [2] abort flag; all zero before the first launch ever
    int* status;
};

// Grid-wide barrier number `k` of this launch for the consumer threads (256 per CTA; thread 0 does the global
// part). The arrival counter only grows during a launch. Returns false if it gave up.
__device__ __forceinline__ bool grid_barrier(const ChainParams& p, int k, int* failed) {
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (threadIdx.x == 0) {
        const unsigned int target = unsigned(k + 1) * gridDim.x;
        __threadfence();
        atomicAdd(p.barrier, 1u);
        bool ok = false;
        for (uint32_t i = 0; i < SPIN_LIMIT; i++) {
            if (ld_acquire(p.barrier) >= target) { ok = true; break; }
            if ((i & 15) == 15 && ld_acquire(p.barrier + 2) != 0u) break;
            if (i > 4096) __nanosleep(40);
        }
        if (!ok) {
            atomicExch(p.status, STATUS_TIMEOUT);
            atomicExch(p.barrier + 2, 1u);
            *failed = 1;
        }
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    return *reinterpret_cast<volatile int*>(failed) == 0;
}

template <int NT>
__global__ void __launch_bounds__(THREADS, NT == 1 ? 2 : 1)
linear_chain_kernel(const __grid_constant__ ChainParams p) {
    constexpr int NS = Geometry<NT>::NS;
    extern __shared__ __align__(128) uint8_t ring[];     // [NS][16][PITCH]
    __shared__ __align__(8) uint64_t bars[2 * NS];       // full[NS], empty[NS]
    __shared__ float red[WARPS][NT][8][16];
    __shared__ float part[NT][8][16];
    __shared__ float sumsq[WARPS][NT * 8];
    __shared__ int failed;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = gridDim.x, cta = blockIdx.x;
    const uint32_t ring0 = smem_u32(ring), bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (NS + s); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), WARPS); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == WARPS) {
        // ---------------------------------------------------------------- producer: weights of every phase, in order
        int64_t seq = 0;
        for (int pi = 0; pi < p.n_phases; pi++) {
            const Phase& ph = p.ph[pi];
            const int64_t tiles = (ph.N + ph.rows - 1) / ph.rows;
            for (int64_t tile = cta; tile < tiles; tile += G) {
                const int64_t n0 = tile * ph.rows;
                const int live_rows = int(min(int64_t(ph.rows), ph.N - n0));
                for (int i = 0; i < ph.spt; i++, seq++) {
                    const int s = int(seq % NS);
                    if (seq >= NS) {
                        int ok = 1;
                        if (lane == 0) {
                            ok = 0;
                            const uint32_t parity = uint32_t((seq / NS) - 1) & 1u;
                            for (uint32_t it = 0; it < SPIN_LIMIT; it++) {
                                if (mbar_test(empty_bar(s), parity)) { ok = 1; break; }
                                if ((it & 63) == 63 && *reinterpret_cast<volatile int*>(&failed)) break;
                                if (it > 2048) __nanosleep(64);
                            }
                        }
                        ok = __shfl_sync(0xffffffffu, ok, 0);
                        if (!ok) {
                            if (lane == 0 && !*reinterpret_cast<volatile int*>(&failed)) { atomicExch(p.status, STATUS_TIMEOUT); failed = 1; }
                            return;
                        }
                    }
                    const int64_t k0 = int64_t(i) * ph.kc;
                    const uint32_t bytes = uint32_t(min(int64_t(ph.kc), ph.K - k0) * 2);
                    if (lane == 0) mbar_expect_tx(full_bar(s), bytes * uint32_t(live_rows));
                    __syncwarp();
                    if (lane < live_rows) bulk_load(ring0 + s * SLOT_BYTES + lane * PITCH, ph.w + (n0 + lane) * ph.K + k0, bytes, full_bar(s));
                }
            }
        }
        return;
    }

    // -------------------------------------------------------------------- consumers (warps 0..7)
    IB_MARK0();
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const bool active = threadIdx.x < NT * 128;
    const int r = threadIdx.x & 15, col = (threadIdx.x >> 4) & 7, ant = active ? threadIdx.x >> 7 : 0;
    bool x_ok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) x_ok[nt] = nt * 8 + g < p.M;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
    int64_t seq = 0;
    uint4 xcur[CPW][NT], xnext[CPW][NT];                 // this lane's fragments of the activations

    for (int pi = 0; pi < p.n_phases; pi++) {
        const Phase& ph = p.ph[pi];
        const int64_t K = ph.K, N = ph.N;
        const int kc = ph.kc, spt = ph.spt;
        const bool wide = ph.rows == 16;
        const int64_t tiles = (N + ph.rows - 1) / ph.rows;
        const int64_t n_local = cta < tiles ? ((tiles - cta + G - 1) / G) * spt : 0;   // this CTA's stages of the phase
        if (pi > 0 && !grid_barrier(p, pi - 1, &failed)) return; // what this phase reads has been written everywhere
        IB_MARK(pi, 0);
        // ---------------------------------------------------------------- activations of the phase
        const bf16* xg = static_cast<const bf16*>(ph.x);
        auto fetch_x = [&](uint4 (&dst)[CPW][NT], int64_t k0) {
#pragma unroll
            for (int u = 0; u < CPW; u++) {
                const int c = warp + u * WARPS;
                const int64_t k = k0 + c * 32 + t * 8;
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
                    dst[u][nt] = (c * 32 < kc && k < K && x_ok[nt]) ? __ldcg(reinterpret_cast<const uint4*>(xg + int64_t(nt * 8 + g) * K + k)) : zero;
            }
        };
        if (n_local > 0) {
            if (ph.x_kind == 1) {
                // RMSNorm of this lane's fragments: the row's sum of squares is put together from the warps' shares
                // in warp order.
                const float* h = static_cast<const float*>(ph.x);
                // the raw float fragments sit in the registers of xcur (first four) and xnext (last four) meanwhile
                float ss[NT];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) ss[nt] = 0.0f;
#pragma unroll
                for (int u = 0; u < CPW; u++) {
                    const int64_t k = (warp + u * WARPS) * 32 + t * 8;
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        const bool ok = k < K && x_ok[nt];
                        const uint4* src = reinterpret_cast<const uint4*>(h + int64_t(nt * 8 + g) * K + k);
                        xcur[u][nt] = ok ? __ldcg(src) : zero;
                        xnext[u][nt] = ok ? __ldcg(src + 1) : zero;
                    }
                }
                auto sq = [](float acc, uint4 q) {
                    acc = fmaf(__uint_as_float(q.x), __uint_as_float(q.x), acc);
                    acc = fmaf(__uint_as_float(q.y), __uint_as_float(q.y), acc);
                    acc = fmaf(__uint_as_float(q.z), __uint_as_float(q.z), acc);
                    return fmaf(__uint_as_float(q.w), __uint_as_float(q.w), acc);
                };
#pragma unroll
                for (int u = 0; u < CPW; u++) {
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) ss[nt] = sq(sq(ss[nt], xcur[u][nt]), xnext[u][nt]);
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    ss[nt] += __shfl_xor_sync(0xffffffffu, ss[nt], 1);
                    ss[nt] += __shfl_xor_sync(0xffffffffu, ss[nt], 2);
                    if (t == 0) sumsq[warp][nt * 8 + g] = ss[nt];
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
                float scale[NT];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    float total = 0.0f;
#pragma unroll
                    for (int wi = 0; wi < WARPS; wi++) total += sumsq[wi][nt * 8 + g];
                    scale[nt] = rsqrtf(total / float(K) + ph.eps);
                }
#pragma unroll
                for (int u = 0; u < CPW; u++) {
                    const int64_t k = (warp + u * WARPS) * 32 + t * 8;
                    float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f), w1 = w0;
                    if (k < K) {
                        w0 = __ldg(reinterpret_cast<const float4*>(ph.norm_w + k));
                        w1 = __ldg(reinterpret_cast<const float4*>(ph.norm_w + k) + 1);
                    }
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        const uint4 a = xcur[u][nt], b = xnext[u][nt];
                        const float s = scale[nt];
                        xcur[u][nt] = make_uint4(
                            pack_bf16(__uint_as_float(a.x) * s * w0.x, __uint_as_float(a.y) * s * w0.y),
                            pack_bf16(__uint_as_float(a.z) * s * w0.z, __uint_as_float(a.w) * s * w0.w),
                            pack_bf16(__uint_as_float(b.x) * s * w1.x, __uint_as_float(b.y) * s * w1.y),
                            pack_bf16(__uint_as_float(b.z) * s * w1.z, __uint_as_float(b.w) * s * w1.w));
                    }
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");   // the shares have been read before the next phase writes them
            } else if (spt == 1) {
                fetch_x(xcur, 0);
            } else {
                fetch_x(xnext, 0);
            }
        }
        IB_MARK(pi, 1);

        int64_t jl = 0;
        for (int64_t tile = cta; tile < tiles; tile += G) {
            const int64_t n0 = tile * ph.rows;
            for (int i = 0; i < spt; i++, seq++, jl++) {
                const int s = int(seq % NS);
                IB_STAGE_MARK(pi, jl, 0);
                if (spt > 1) {                                   // fragments of this stage; the next stage's set out now
#pragma unroll
                    for (int u = 0; u < CPW; u++) {
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) xcur[u][nt] = xnext[u][nt];
                    }
                    if (jl + 1 < n_local) fetch_x(xnext, int64_t((i + 1) % spt) * kc);
                }
                {
                    bool ok = false;
                    const uint32_t parity = uint32_t(seq / NS) & 1u;
                    for (uint32_t it = 0; it < SPIN_LIMIT; it++) {
                        if (mbar_test(full_bar(s), parity)) { ok = true; break; }
                        if ((it & 63) == 63 && *reinterpret_cast<volatile int*>(&failed)) break;
                        if (it > 2048) __nanosleep(64);
                    }
                    if (!ok) {
                        if (lane == 0 && !*reinterpret_cast<volatile int*>(&failed)) {
                            atomicExch(p.status, STATUS_TIMEOUT);
                            atomicExch(p.barrier + 2, 1u);
                            failed = 1;
                        }
                        return;
                    }
                }
                if (jl == 0) IB_MARK(pi, 2);
                IB_STAGE_MARK(pi, jl, 1);
                const uint8_t* st = ring + s * SLOT_BYTES;
                const int64_t k0 = int64_t(i) * kc;
#pragma unroll
                for (int u = 0; u < CPW; u++) {
                    const int c = warp + u * WARPS;
                    const bool k_ok = c * 32 < kc && k0 + c * 32 + t * 8 < K;
                    const int cb = (c * 32 + t * 8) * 2;
                    const uint4 a0 = k_ok ? *reinterpret_cast<const uint4*>(st + g * PITCH + cb) : zero;
                    const uint4 a1 = (k_ok && wide) ? *reinterpret_cast<const uint4*>(st + (g + 8) * PITCH + cb) : zero;
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        mma_bf16(acc[nt], a0.x, a1.x, a0.y, a1.y, xcur[u][nt].x, xcur[u][nt].y);
                        mma_bf16(acc[nt], a0.z, a1.z, a0.w, a1.w, xcur[u][nt].z, xcur[u][nt].w);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar(s));
                IB_STAGE_MARK(pi, jl, 2);
            }
            // ------------------------------------------------------------ the tile is complete
            IB_STAGE_MARK(pi, jl - 1, 3);
            asm volatile("bar.sync 1, 256;" ::: "memory");       // the previous tile's sums have been read
            IB_STAGE_MARK(pi, jl - 1, 4);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                red[warp][nt][2 * t][g] = acc[nt][0];
                red[warp][nt][2 * t + 1][g] = acc[nt][1];
                red[warp][nt][2 * t][g + 8] = acc[nt][2];
                red[warp][nt][2 * t + 1][g + 8] = acc[nt][3];
                acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            IB_STAGE_MARK(pi, jl - 1, 5);
            float v = 0.0f;
            if (active) {
#pragma unroll
                for (int wi = 0; wi < WARPS; wi++) v += red[wi][ant][col][r];
            }
            if (ph.epi == 2) {
                if (active) part[ant][col][r] = v;               // the SwiGLU epilogue pairs rows r and r + 8
                asm volatile("bar.sync 1, 256;" ::: "memory");
            }
            IB_STAGE_MARK(pi, jl - 1, 6);
            const int m = ant * 8 + col;
            if (active && m < p.M && r < ph.rows) {
                if (ph.epi == 2) {
                    if (r < 8) {
                        const float gate = v, up = part[ant][col][r + 8];
                        const int64_t f = tile * 8 + r;
                        if (f < N / 2)
                            static_cast<bf16*>(ph.out)[int64_t(m) * (N / 2) + f] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
                    }
                } else {
                    const int64_t n = n0 + r;
                    if (n < N) {
                        if (ph.bias) v += ph.bias[n];
                        if (ph.epi == 1) {
                            float* o = static_cast<float*>(ph.out) + int64_t(m) * N + n;
                            *o = __ldcg(o) + v;
                        } else {
                            static_cast<bf16*>(ph.out)[int64_t(m) * N + n] = __float2bfloat16_rn(v);
                        }
                    }
                }
            }
            IB_STAGE_MARK(pi, jl - 1, 7);
        }
        IB_MARK(pi, 3);
    }
    // The last CTA to leave puts the barrier words back to zero for the next launch.
    if (threadIdx.x == 0) {
        if (atomicAdd(p.barrier + 1, 1u) == unsigned(G) - 1) {
            atomicExch(p.barrier, 0u);
            atomicExch(p.barrier + 1, 0u);
        }
    }
}

template <int NT>
int launch_chain(ChainParams& p, int sms, cudaStream_t stream) {
    constexpr size_t smem = size_t(Geometry<NT>::NS) * SLOT_BYTES;
    static bool configured = false;
    static int per_sm = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(linear_chain_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return ib::fail(IB_ERR_CUDA, "linear_chain: cannot set shared memory size: %s", cudaGetErrorString(e));
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, linear_chain_kernel<NT>, THREADS, smem);
        if (e != cudaSuccess || per_sm < 1) return ib::fail(IB_ERR_CUDA, "linear_chain: the kernel does not fit an SM");
        if (per_sm > 2) per_sm = 2;
        configured = true;
    }
    const int grid = per_sm * sms;
    // 8-row tiles where a one-stage phase's 16-row tiles would leave more than half of the CTAs without work
    for (int i = 0; i < p.n_phases; i++) {
        Phase& ph = p.ph[i];
        ph.rows = (ph.epi != 2 && ph.spt == 1 && (ph.N + 15) / 16 * 2 <= grid) ? 8 : 16;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, linear_chain_kernel<NT>, p);
    if (e != cudaSuccess) return ib::fail(IB_ERR_CUDA, "linear_chain: %s", cudaGetErrorString(e));
    return IB_OK;
}

}  // namespace

// One phase of a chain, as the C ABI takes it (an array of these).
struct ib_chain_phase {
    const void* w; int64_t N; int64_t K;
    int x_kind; const void* x; const float* norm_w; float eps;
    int epi; const float* bias; void* out;
};

// Runs phases[0..n_phases) as one cooperative kernel. barrier: three zero-initialised words in device memory, kept
// for the process's lifetime (the kernel leaves them zero for the next launch unless it raised the status word).
// Sizes: M <= 16; every K a multiple of 8; a normalised input (x_kind 1) needs K <= 1536; SwiGLU needs N % 16 == 0.
IB_EXPORT int ib_linear_chain(const ib_chain_phase* phases, int n_phases, int64_t M, int sm_count, unsigned int* barrier,
                              int* status, cudaStream_t stream) {
    if (n_phases <= 0 || M <= 0) return IB_OK;
    if (n_phases > MAX_PHASES) return ib::fail(IB_ERR_ARG, "linear_chain: at most %d phases", MAX_PHASES);
    if (M > 16) return ib::fail(IB_ERR_ARG, "linear_chain: at most 16 rows, got %lld", (long long)M);
    if (!barrier || !status) return ib::fail(IB_ERR_ARG, "linear_chain: barrier words and a status word are required");
    const int sms = sm_count > 0 ? sm_count : 148;
    ChainParams p = {};
    p.n_phases = n_phases; p.M = int(M); p.barrier = barrier; p.status = status;
    for (int i = 0; i < n_phases; i++) {
        const ib_chain_phase& a = phases[i];
        if (a.N <= 0 || a.K <= 0 || a.K % 8) return ib::fail(IB_ERR_ARG, "linear_chain: phase %d: N and K must be positive, K a multiple of 8", i);
        if ((uintptr_t(a.w) & 15) || (uintptr_t(a.x) & 15)) return ib::fail(IB_ERR_ARG, "linear_chain: phase %d: operands must be 16-byte aligned", i);
        if (a.x_kind < 0 || a.x_kind > 1 || a.epi < 0 || a.epi > 2) return ib::fail(IB_ERR_ARG, "linear_chain: phase %d: unknown kind", i);
        if (a.x_kind == 1 && a.K > KC_MAX) return ib::fail(IB_ERR_ARG, "linear_chain: phase %d: a normalised input takes K <= %d", i, KC_MAX);
        if (a.x_kind == 1 && (!a.norm_w || (uintptr_t(a.norm_w) & 15))) return ib::fail(IB_ERR_ARG, "linear_chain: phase %d: a 16-byte aligned norm weight is required", i);
        if (a.epi == 2 && a.N % 16) return ib::fail(IB_ERR_ARG, "linear_chain: phase %d: SwiGLU needs N %% 16 == 0", i);
        Phase& ph = p.ph[i];
        ph.w = (const bf16*)a.w; ph.N = a.N; ph.K = a.K; ph.x_kind = a.x_kind; ph.x = a.x; ph.norm_w = a.norm_w; ph.eps = a.eps;
        ph.epi = a.epi; ph.bias = a.bias; ph.out = a.out;
        // K in as few equal stages as a slot allows
        const int64_t n_stages = (a.K + KC_MAX - 1) / KC_MAX;
        ph.kc = int(((a.K + n_stages - 1) / n_stages + 63) / 64 * 64);
        ph.spt = int((a.K + ph.kc - 1) / ph.kc);
    }
    return M <= 8 ? launch_chain<1>(p, sms, stream) : launch_chain<2>(p, sms, stream);
}

#ifdef IB_CHAIN_TRACE
// Profiling build only: copies the per-CTA timestamps of the last launch to the host ([1024][1 + 4 * 4] int64, then CTA 0's [4][32][3] stage marks).
IB_EXPORT int ib_linear_chain_trace(long long* host) {
    cudaError_t e = cudaMemcpyFromSymbol(host, ib_trace, sizeof(ib_trace));
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(host + sizeof(ib_trace) / 8, ib_stage_trace, sizeof(ib_stage_trace));
    return e == cudaSuccess ? IB_OK : ib::fail(IB_ERR_CUDA, "linear_chain_trace: %s", cudaGetErrorString(e));
}
#endif
