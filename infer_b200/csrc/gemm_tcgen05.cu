// bfloat16 matrix product on the 5th-generation tensor cores of sm_100a:
//   out[M, N] = x[M, K] . w[N, K]^T (+ bias[N]) (+ residual[M, N])
// both operands row-major with K contiguous ("K-major"), float accumulation in tensor memory (TMEM).
//
// Structure of one CTA (192 threads, one 128 x BN output tile, BN in {16, 32, 64, 128}; 256 with K slices):
//   warp 0      one lane issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of 128 x 64 and BN x 64
//               operand tiles into a ring of shared-memory stages, each guarded by a full/empty mbarrier pair;
//   warp 1      allocates BN TMEM columns; one lane issues tcgen05.mma (M=128, N=BN, K=16, kind::f16) four times
//               per stage, then tcgen05.commit to hand the stage back, and at the end to signal the epilogue;
//   warps 2-5   read the accumulator with tcgen05.ld (each warp its 32 TMEM lanes = 32 tile rows), apply the
//               epilogue (bias, residual, conversion) and store to global memory.
//
// Two ways to map the product onto a tile:
//   plain   A = x (tokens on the 128-row side), B = w;  for many tokens (prefill)
//   swap    A = w (output features on the 128-row side), B = x, tokens on the BN side padded to 16/32/64/128;
//           for up to 128 tokens (decode), where the weights are streamed once and the tensor core's M is not wasted.
// With few tiles the K range is cut into `splits` slices. Up to 8 slices of a tile are the CTAs of one thread-block
// cluster (always in the swapped mapping; 2, 4 or 8 in the plain one): every slice pushes each block of columns of
// its float tile into the shared memory of the slice that owns the block, and after one cluster barrier the owner
// adds the slices in ascending order and runs the epilogue. Otherwise (grid.z, up to 16 slices of very few tiles)
// each CTA writes its float tile to a workspace and the CTA that arrives last at the tile's counter adds the slices
// in ascending order. Either way the sum does not depend on arrival order.
// A long K on few tiles (a 512-token portion of a prompt against a down matrix) takes 128 x 256 tiles with 2, 4 or 8
// K slices as a cluster: 128 KB of float tile do not fit behind the ring, so the slices' columns are received in the
// operand ring itself, once a cluster barrier has told every slice that the others' MMAs are done.
// For many tokens a persistent kernel (further down) walks over tiles with two accumulators in tensor memory.
// ib_gemm_tc_plan chooses among these ways with a time model fitted to measurements.
// What is read once per step (the weights' tiles) is loaded with the L2 evict-first policy.
// In the swapped mapping the ring takes up to eight stages (the CTA has the SM to itself and all of its weights
// should be in flight) and the weights' first stages are requested before the kernel waits for its predecessor.
//
// Sizes: any M, N >= 1; K a multiple of 8 (TMA needs 16-byte row pitch); rows beyond M, N and columns beyond K are
// zero-filled by TMA and masked at the store. Everything else is refused with an error.
//
// Every wait on an mbarrier is bounded; a wait that runs out raises the status word, and the CTA drains its
// copies, frees its TMEM and returns.
#include "common.cuh"
#include "tma_map.cuh"

#include <cuda.h>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

IB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;

constexpr int BM = 128;            // tile rows on the A side = TMEM lanes
constexpr int BK = 64;             // bf16 elements per stage row = one 128-byte swizzle line
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

constexpr int STATUS_TIMEOUT_PRODUCER = 101, STATUS_TIMEOUT_MMA = 102, STATUS_TIMEOUT_EPILOGUE = 103;

// ------------------------------------------------------------------------------------------------ PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// Bounded wait (non-blocking probes, short sleeps after the first thousand): false if the phase did not complete
// within the limit, which is of the order of a second.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; i++) {
        if (mbar_test(bar, parity)) return true;
        if (i > 1024) __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_cluster(uint32_t local_smem, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem), "r"(rank));
    return remote;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// Weights are read once per step and never again before the whole model has streamed past: their tiles are marked
// to leave L2 first, so that they do not push out what is read again soon (activations, the residual stream, cache
// pages, and the kernels' own instructions: with the default policy a kernel that runs between other kernels spent
// thousands of cycles in parts of its code it had not touched since its last launch).
#ifndef IB_WEIGHTS_EVICT_FIRST
#define IB_WEIGHTS_EVICT_FIRST 1
#endif
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void tma_load_2d_once(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, uint64_t policy) {
#if IB_WEIGHTS_EVICT_FIRST
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy) : "memory");
#else
    tma_load_2d(dst, map, bar, x, y);
#endif
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has finished (reading smem, writing TMEM).
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile of 128-byte rows in 128-byte swizzle: groups of 8 rows are
// 1024 bytes apart (stride byte offset), the leading offset is unused by swizzled K-major layouts, descriptor
// version 1 (Blackwell), layout type 2 (SWIZZLE_128B). Stepping 16 elements along K adds 32 bytes to the start.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= uint64_t((smem_addr & 0x3FFFF) >> 4);
    d |= uint64_t(1) << 16;
    d |= uint64_t(1024 >> 4) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(2) << 61;
    return d;
}

// Instruction descriptor for kind::f16: D float (bit 4), A and B bfloat16 (bits 7, 10), both K-major (bits 15, 16
// clear), N/8 at bit 17, M/16 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(BM >> 4) << 24);
}

struct GemmParams {
    int64_t rows_a, rows_b, K;           // extents on the 128-row side, the BN side, and the reduction
    int kb_total, kb_per_split, splits;
    int swap;                            // 0: A = x (tokens), B = w (features); 1: A = w, B = x
    int epi;                             // 0: bias/residual; 2: SwiGLU over feature rows interleaved by 8 -> [M, N/2]
    int64_t M, N;                        // logical output [M tokens, N features], leading dimension N
    const float* bias;                   // [N] or null
    const float* residual;               // [M, N] or null (may alias out)
    void* out;
    float* workspace;                    // [splits, tiles, 128, BN] partials (splits > 1)
    unsigned int* counters;              // [tiles], zero between calls
    int* status;
    int stages;                          // stages of the operand ring in use (<= Cfg::MAX_STAGES)
    int cluster_split;                   // 1: the K slices of a tile are the CTAs of one cluster (grid.x) and are added
                                         //    through distributed shared memory; no workspace, no counters
    int early_release;                   // persistent kernel: 1 = the successor is released at the kernel's start (its CTAs
                                         //    set up wherever an SM has room), 0 = after the MMA loop. Early costs where
                                         //    kernels are long (a 2,048-token step at 5120 features: 60 against 57 ms; the
                                         //    waiting CTAs are not free on a power-bound GPU) and is kept for short ones
    int weights_once;                    // persistent kernel: 1 = the weight tiles carry the L2 evict-first policy (a matrix
                                         //    that fits L2 beside the activations; a larger one is evicted between the row
                                         //    tiles' reads: 2 % slower at 3584 and 5120 features)
    int recv_in_ring;                    // 1: the slices' columns are received in the operand ring itself, once every slice
                                         //    of the cluster is done with its ring (one more cluster barrier; for tiles whose
                                         //    float columns would not fit behind the ring)
};

template <int BN> struct Cfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = BN >= 128 ? 3 : (BN >= 64 ? 4 : 5);       // <= ~100 KB: two CTAs per SM
    static constexpr int MAX_STAGES = BN >= 256 ? 4 : (BN >= 128 ? 6 : 8);  // a CTA alone on its SM (decode: all of the ring in flight)
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    static constexpr int SMEM_EXTRA = 1024 /*alignment slack*/ + 256 /*barriers*/;
    static constexpr int RECV_OFFSET = 256;                                 // behind the barriers
    static constexpr int RECV_BYTES = BM * (BN + 8) * 4;                    // cluster split-K: the slices' columns of one owner
    static constexpr int SMEM_BYTES = MAX_STAGES * STAGE_BYTES + SMEM_EXTRA;
    static_assert(BM * BN * 4 <= STAGES * STAGE_BYTES, "a float partial tile must fit the smallest ring");
};

template <typename TOut> __device__ __forceinline__ void store_elem(TOut* p, float v);
template <> __device__ __forceinline__ void store_elem<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_elem<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// Applies bias/residual and stores 16 accumulator values of tile row `r`, tile columns [c0, c0 + 16).
// PRE: the residual's 16 floats were loaded by the caller ahead of time (plain mapping, whole chunk inside N, N % 8 == 0).
template <typename TOut, bool PRE = false>
__device__ __forceinline__ void epilogue_store(const GemmParams& p, const float* v, int64_t a_row, int64_t b_row0, int ncols = 16,
                                               const float4* pre_res = nullptr) {
    TOut* out = reinterpret_cast<TOut*>(p.out);
    if (p.epi == 2) {
        // Feature rows come in blocks of 16: 8 gate rows, then the 8 matching up rows. out[m, 8 blk + r] = silu(g) * u.
        const int64_t half = p.N / 2;
        if (p.swap) {
            // lanes 0-7 and 16-23 of a warp hold gate rows, lanes 8-15 and 24-31 the matching up rows
            // Columns go in pairs: the gate lane finishes column j with its partner's up value, the up lane column j + 1
            // with its partner's gate value, so every lane computes and stores a result (one exchange per pair). No
            // short-circuit operators, the arithmetic outside the condition: a branch per element cost several times it.
            const int64_t n = a_row;
            const bool is_gate = (n & 8) == 0;
            const bool row_ok = n < p.N;
            TOut* dst = out + (n >> 4) * 8 + (n & 7);
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
                const float got = __shfl_xor_sync(0xffffffffu, is_gate ? v[j + 1] : v[j], 8);
                const float gte = is_gate ? v[j] : got, up = is_gate ? got : v[j + 1];
                const int jj = is_gate ? j : j + 1;
                const int64_t m = b_row0 + jj;
                const float act = __fdividef(gte, 1.0f + __expf(-gte)) * up;
                if (row_ok & (m < p.M) & (jj < ncols)) store_elem<TOut>(dst + m * half, act);
            }
        } else {
            const int64_t m = a_row, n0 = b_row0;
            if (m < p.M && n0 < p.N) {
                float act[8];
#pragma unroll
                // the approximate division: an IEEE one made the epilogue of a 128 x 256 tile longer than the tile's MMAs
                // (gate/up of a 2,048-token step: 94 us with it, 86 us without)
                for (int j = 0; j < 8; j++) act[j] = __fdividef(v[j], 1.0f + __expf(-v[j])) * v[j + 8];
                if constexpr (sizeof(TOut) == 2) {
                    if ((half & 7) == 0) {                      // 8 bfloat16 = one 16-byte store
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(act[0], act[1]), h1 = __floats2bfloat162_rn(act[2], act[3]);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(act[4], act[5]), h3 = __floats2bfloat162_rn(act[6], act[7]);
                        uint4 u;
                        u.x = *reinterpret_cast<uint32_t*>(&h0); u.y = *reinterpret_cast<uint32_t*>(&h1);
                        u.z = *reinterpret_cast<uint32_t*>(&h2); u.w = *reinterpret_cast<uint32_t*>(&h3);
                        *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.out) + m * half + (n0 >> 1)) = u;
                        return;
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; j++) store_elem<TOut>(out + m * half + (n0 >> 1) + j, act[j]);
            }
        }
        return;
    }
    if (p.swap) {
        // a_row = output feature n; b rows = tokens m. A warp's 32 lanes hold 32 consecutive features of one token.
        const int64_t n = a_row;
        if (n >= p.N) return;
        const float b = p.bias ? p.bias[n] : 0.0f;
        // The residual may be the output itself, so the compiler keeps every load behind the store before it: written
        // as one loop, a row cost a trip to L2 per token. Each thread reads and writes the same addresses, so all of
        // its residual values can be requested first.
        float res[16];
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const int64_t m = b_row0 + j;
            res[j] = (p.residual && m < p.M && j < ncols) ? p.residual[m * p.N + n] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const int64_t m = b_row0 + j;
            if (m < p.M && j < ncols) store_elem<TOut>(out + m * p.N + n, v[j] + b + res[j]);
        }
    } else {
        const int64_t m = a_row;
        if (m >= p.M) return;
        const int64_t n0 = b_row0;
        if (ncols == 16 && n0 + 16 <= p.N && (p.N & 7) == 0) {
            float x[16];
#pragma unroll
            for (int j = 0; j < 16; j++) x[j] = v[j] + (p.bias ? p.bias[n0 + j] : 0.0f);
            if (p.residual) {
                const float4* r4 = reinterpret_cast<const float4*>(p.residual + m * p.N + n0);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    float4 r;
                    if constexpr (PRE) r = pre_res[j]; else r = r4[j];
                    x[4 * j] += r.x; x[4 * j + 1] += r.y; x[4 * j + 2] += r.z; x[4 * j + 3] += r.w;
                }
            }
            if constexpr (sizeof(TOut) == 4) {
                float4* o4 = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + m * p.N + n0);
#pragma unroll
                for (int j = 0; j < 4; j++) o4[j] = make_float4(x[4 * j], x[4 * j + 1], x[4 * j + 2], x[4 * j + 3]);
            } else {
                uint4* o4 = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.out) + m * p.N + n0);
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(x[8 * j], x[8 * j + 1]);
                    __nv_bfloat162 h1 = __floats2bfloat162_rn(x[8 * j + 2], x[8 * j + 3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(x[8 * j + 4], x[8 * j + 5]);
                    __nv_bfloat162 h3 = __floats2bfloat162_rn(x[8 * j + 6], x[8 * j + 7]);
                    uint4 u;
                    u.x = *reinterpret_cast<uint32_t*>(&h0); u.y = *reinterpret_cast<uint32_t*>(&h1);
                    u.z = *reinterpret_cast<uint32_t*>(&h2); u.w = *reinterpret_cast<uint32_t*>(&h3);
                    o4[j] = u;
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const int64_t n = n0 + j;
                if (n < p.N && j < ncols) {
                    float x = v[j] + (p.bias ? p.bias[n] : 0.0f);
                    if (p.residual) x += p.residual[m * p.N + n];
                    store_elem<TOut>(out + m * p.N + n, x);
                }
            }
        }
    }
}

#ifdef IB_GEMM_TRACE
// Profiling build: the first CTA's producer, MMA and first epilogue thread record the SM clock at their marks.
__device__ long long ib_gemm_trace[32];
#define IB_MT(k) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ib_gemm_trace[k] = clock64(); } while (0)
#else
#define IB_MT(k) do {} while (0)
#endif

template <int BN, typename TOut>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    // Operand stages need 1024-byte alignment for the 128-byte swizzle pattern.
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const int S = p.stages;
    const uint32_t bars = base + S * C::STAGE_BYTES;                          // full[S], empty[S], tmem_full
    volatile uint32_t* slots = reinterpret_cast<volatile uint32_t*>(base_ptr + S * C::STAGE_BYTES + (2 * S + 1) * 8);
    // slots[0] = TMEM base address, slots[1] = abort flag, slots[2] = "this CTA reduces the split-K slices"

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) IB_MT(0);
    // grid (tiles a, tiles b, slices), or with the slices as one cluster: (slices, tiles a, tiles b)
    const int tile_a = p.cluster_split ? blockIdx.y : blockIdx.x, tile_b = p.cluster_split ? blockIdx.z : blockIdx.y;
    const int split = p.cluster_split ? blockIdx.x : blockIdx.z;
    const int kb0 = split * p.kb_per_split;
    const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
    const int n_kb = kb1 - kb0;

    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (S + s); };
    const uint32_t tmem_full_bar = bars + 8u * (2 * S);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(tmem_full_bar, 1);
        slots[1] = 0; slots[2] = 0;
        fence_barrier_init();
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(&slots[0])), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = slots[0];
    if (threadIdx.x == 0) IB_MT(1);
    // The set-up above overlapped the predecessor. Each role waits for it where it first touches what the predecessor
    // may have written: the producer before it loads activations, the epilogue before it reads or writes the output.
    // K slices as a cluster, weights on the rows: the CTA that owns a few of the tile's token columns needs their
    // residual values and its row's bias only after the cluster barrier, at the very end of the kernel; it asks for
    // them as soon as the predecessor is done, so that no trip to L2 is left on the tail.
    float own_res[16], own_bias = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j++) own_res[j] = 0.0f;
    const int own_per = (BN + p.splits - 1) / p.splits;
    const bool own_early = p.cluster_split && p.swap && p.epi == 0 && own_per <= 16;

    // K slices as a cluster: every slice pushes the columns of its float tile to the CTA that owns them, through
    // distributed shared memory; after a cluster barrier the owners add what they received, in slice order, and
    // nobody touches remote memory again. The receive area lies behind the ring (a fast slice may push while the
    // owner's ring is still in use) or, for wide tiles, is the ring itself, after a cluster barrier of its own.
    // Called by the epilogue warps once their accumulator is complete.
    auto push_partials = [&]() {
        const int quad = warp & 3, r = quad * 32 + lane;
        const int per = (BN + p.splits - 1) / p.splits;               // columns per owner
        const uint32_t recv = p.recv_in_ring ? base : base + uint32_t(p.stages) * C::STAGE_BYTES + C::RECV_OFFSET;
        // Where the owners' widths are multiples of four columns the owner's area is [slice][group of four
        // columns][row][4]: a thread sends four columns in one 16-byte store and a warp's stores are contiguous;
        // otherwise [slice][column][row] with single floats.
        const bool vec = (per & 3) == 0;
        const uint32_t mine = vec ? recv + uint32_t(split * (per >> 2) * BM + r) * 16u : recv + uint32_t((split * per) * BM + r) * 4u;
        int owner = 0, lc = 0;                            // (carried along: no division per column)
        uint32_t dst = map_cluster(mine, 0u);
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
            uint32_t raw[16];
            tmem_ld16(tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(c), raw);
            tmem_ld_wait();
            if (vec) {
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    st_cluster_v4(dst, __uint_as_float(raw[4 * g]), __uint_as_float(raw[4 * g + 1]),
                                  __uint_as_float(raw[4 * g + 2]), __uint_as_float(raw[4 * g + 3]));
                    dst += BM * 16u;
                    lc += 4;
                    if (lc == per) { lc = 0; owner++; if (owner < p.splits) dst = map_cluster(mine, uint32_t(owner)); }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (owner < p.splits) st_cluster_f32(dst, __uint_as_float(raw[j]));
                    dst += BM * 4u;
                    if (++lc == per) { lc = 0; owner++; if (owner < p.splits) dst = map_cluster(mine, uint32_t(owner)); }
                }
            }
        }
    };

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane != 0) ib::pdl_launch_dependents();
        if (lane == 0) {
            int issued = 0;
            // With the weights on the A side (decode) their first stages set out before the wait: no kernel writes them.
            const int pre = p.swap ? min(S, n_kb) : 0;
            const uint64_t once = policy_evict_first();
            for (int i = 0; i < pre; i++) {
                mbar_expect_tx(full_bar(i), C::STAGE_BYTES);
                tma_load_2d_once(base + i * C::STAGE_BYTES, &tm_a, full_bar(i), (kb0 + i) * BK, tile_a * BM, once);
            }
            IB_MT(2);
            ib::pdl_wait();
            IB_MT(3);
            for (int i = 0; i < pre; i++)
                tma_load_2d(base + i * C::STAGE_BYTES + C::A_BYTES, &tm_b, full_bar(i), (kb0 + i) * BK, tile_b * BN);
            issued = pre;
            int s = pre % S;                             // (slot and round carried along: S is a run-time value)
            uint32_t round = pre / S;
            for (int i = pre; i < n_kb; i++, s = (s + 1 == S ? 0 : s + 1), round += (s == 0)) {
                if (i >= S && !mbar_wait(empty_bar(s), (round - 1) & 1)) {
                    atomicExch(p.status, STATUS_TIMEOUT_PRODUCER); slots[1] = 1; break;
                }
                if (slots[1]) break;
                const uint32_t a_dst = base + s * C::STAGE_BYTES, b_dst = a_dst + C::A_BYTES;
                mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
                if (p.swap) {
                    tma_load_2d_once(a_dst, &tm_a, full_bar(s), (kb0 + i) * BK, tile_a * BM, once);
                    tma_load_2d(b_dst, &tm_b, full_bar(s), (kb0 + i) * BK, tile_b * BN);
                } else {
                    tma_load_2d(a_dst, &tm_a, full_bar(s), (kb0 + i) * BK, tile_a * BM);
                    tma_load_2d_once(b_dst, &tm_b, full_bar(s), (kb0 + i) * BK, tile_b * BN, once);
                }
                issued = i + 1;
            }
            IB_MT(4);
            if (slots[1]) {
                // Drain: wait (bounded) until every copy this thread started has landed, so that none writes into
                // shared memory after the CTA is gone.
                for (int i = max(0, issued - S); i < issued; i++) mbar_wait(full_bar(i % S), (i / S) & 1);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BN);
            int s = 0;
            uint32_t round = 0;
            for (int i = 0; i < n_kb; i++, s = (s + 1 == S ? 0 : s + 1), round += (s == 0)) {
                if (!mbar_wait(full_bar(s), round & 1)) {
                    atomicExch(p.status, STATUS_TIMEOUT_MMA); slots[1] = 1; break;
                }
                tc_fence_after();
                if (i == 0) IB_MT(5);
                if (i == n_kb / 2) IB_MT(6);
                const uint32_t a_addr = base + s * C::STAGE_BYTES, b_addr = a_addr + C::A_BYTES;
                const uint64_t a_desc = make_desc(a_addr), b_desc = make_desc(b_addr);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; k++) {
                    // 16 elements along K = 32 bytes = 2 units of the descriptor's 16-byte address field
                    umma_f16(tmem_base, a_desc + uint64_t(2 * k), b_desc + uint64_t(2 * k), idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(empty_bar(s));
            }
            umma_commit(tmem_full_bar);
            IB_MT(7);
        }
        ib::pdl_launch_dependents();
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..5)
        const int quad = warp & 3;                                  // this warp may touch TMEM lanes [32 quad, 32 quad + 32)
        const int r = quad * 32 + lane;                             // tile row
        const int64_t a_row = int64_t(tile_a) * BM + r;
        ib::pdl_wait();
        if (own_early && a_row < p.N) {
            const int c_begin = min(BN, split * own_per), n_own = min(BN, c_begin + own_per) - c_begin;
            if (p.bias) own_bias = p.bias[a_row];
            if (p.residual) {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int64_t m = int64_t(tile_b) * BN + c_begin + j;
                    if (j < n_own && m < p.M) own_res[j] = p.residual[m * p.N + a_row];
                }
            }
        }
        bool ok = mbar_wait(tmem_full_bar, 0);
        if (!ok) { atomicExch(p.status, STATUS_TIMEOUT_EPILOGUE); slots[1] = 1; }
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        if (threadIdx.x == 64) IB_MT(8);
        if (ok) {
            const int n_tiles = gridDim.x * gridDim.y;
            const int tile = tile_b * gridDim.x + tile_a;
            if (p.cluster_split) {
                if (!p.recv_in_ring) push_partials();
            } else if (p.splits == 1) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    uint32_t raw[16];
                    tmem_ld16(tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(c), raw);
                    tmem_ld_wait();
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = __uint_as_float(raw[j]);
                    epilogue_store<TOut>(p, v, a_row, int64_t(tile_b) * BN + c);
                }
            } else {
                // Slices are stored column-major within the tile (element (r, col) at col * 128 + r), so that the 32 lanes
                // of a warp, which hold 32 consecutive rows, write and later read 128 contiguous bytes per column.
                float* mine = p.workspace + (int64_t(split) * n_tiles + tile) * (BM * BN) + r;
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    uint32_t raw[16];
                    tmem_ld16(tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(c), raw);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) mine[(c + j) * BM] = __uint_as_float(raw[j]);
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    const unsigned int prev = atomicAdd(p.counters + tile, 1u);
                    slots[2] = (prev == unsigned(p.splits - 1)) ? 1u : 0u;
                    if (prev == unsigned(p.splits - 1)) p.counters[tile] = 0;        // ready for the next call
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (slots[2]) {
                    __threadfence();
#pragma unroll 1
                    for (int c = 0; c < BN; c += 16) {
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; j++) v[j] = 0.0f;
                        // Slices are added in ascending order; the 16 loads of a slice are in flight together, and the
                        // next slice's loads are issued before the current one is added.
                        const float* src = p.workspace + int64_t(tile) * (BM * BN) + int64_t(c) * BM + r;
                        const int64_t zstride = int64_t(n_tiles) * (BM * BN);
                        float cur[16], nxt[16];
#pragma unroll
                        for (int j = 0; j < 16; j++) cur[j] = __ldcg(src + j * BM);
                        for (int z = 0; z < p.splits; z++) {
                            if (z + 1 < p.splits) {
#pragma unroll
                                for (int j = 0; j < 16; j++) nxt[j] = __ldcg(src + (z + 1) * zstride + j * BM);
                            }
#pragma unroll
                            for (int j = 0; j < 16; j++) { v[j] += cur[j]; cur[j] = nxt[j]; }
                        }
                        epilogue_store<TOut>(p, v, a_row, int64_t(tile_b) * BN + c);
                    }
                }
            }
        }
    }
    if (p.cluster_split) {
        if (p.recv_in_ring) {
            __syncwarp();
            cluster_sync();                              // every slice's MMAs are complete: the rings are free
            if (warp >= 2 && !slots[1]) { tc_fence_after(); push_partials(); }
        }
        if (threadIdx.x == 64) IB_MT(11);
        __syncwarp();
        cluster_sync();                                  // every slice's pushes have arrived
        if (threadIdx.x == 64) IB_MT(12);
        if (warp >= 2 && !slots[1]) {
            const int r = (warp & 3) * 32 + lane;
            const int64_t a_row = int64_t(tile_a) * BM + r;
            const int per = (BN + p.splits - 1) / p.splits;
            const int c_begin = min(BN, split * per), c_end = min(BN, c_begin + per);
            const float* recv = reinterpret_cast<const float*>(p.recv_in_ring ? base_ptr : base_ptr + size_t(p.stages) * C::STAGE_BYTES + C::RECV_OFFSET);
            const bool vec = (per & 3) == 0;
            for (int c0 = c_begin; c0 < c_end; c0 += 16) {
                const int ncols = min(16, c_end - c0);
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; j++) v[j] = 0.0f;
                for (int z = 0; z < p.splits; z++) {
                    if (vec) {
                        const float4* src = reinterpret_cast<const float4*>(recv) + (z * (per >> 2) + ((c0 - c_begin) >> 2)) * BM + r;
#pragma unroll
                        for (int g = 0; g < 4; g++) {
                            if (4 * g < ncols) {
                                const float4 f = src[g * BM];
                                v[4 * g] += f.x; v[4 * g + 1] += f.y; v[4 * g + 2] += f.z; v[4 * g + 3] += f.w;
                            }
                        }
                    } else {
                        const float* src = recv + ((z * per) + (c0 - c_begin)) * BM + r;
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (j < ncols) v[j] += src[j * BM];
                    }
                }
                if (own_early) {
                    if (a_row < p.N) {
                        TOut* dst = reinterpret_cast<TOut*>(p.out) + (int64_t(tile_b) * BN + c0) * p.N + a_row;
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (j < ncols && int64_t(tile_b) * BN + c0 + j < p.M) store_elem<TOut>(dst + j * p.N, v[j] + own_bias + own_res[j]);
                    }
                } else {
                    epilogue_store<TOut>(p, v, a_row, int64_t(tile_b) * BN + c0, ncols);
                }
            }
        }
        if (threadIdx.x == 64) IB_MT(13);
    }
    if (threadIdx.x == 64) IB_MT(9);
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 64) IB_MT(10);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}


// ------------------------------------------------------------------------------------------------ persistent kernel
// For many tokens (prefill). The one-tile kernel above reads (128 + 128) rows of operands for a 128 x 128 tile; at
// bfloat16 tensor speed that is more than the path from L2 delivers, so it cannot get far beyond half of the tensor
// peak. Here a CTA owns an SM, walks over 256 x 128 tiles (two M=128 MMAs per k-step share one B tile: a quarter
// less operand traffic per flop) and keeps two accumulators of 256 columns in tensor memory, so that the epilogue
// warps drain one tile while the MMA warp already works on the next; the operand ring runs on across tiles.
// The tile is 256 x 128 with two MMAs per k-step, or (the default) 128 tokens x 256, 192 or 176 features with one,
// whichever width fills the SMs best (a matrix of 1536 features has 6, 8 or 9 column tiles; with 16 row tiles that
// is 96, 128 or 144 CTAs' worth of work for 148 SMs).
#ifndef IB_GEMM_PSTAGES
#define IB_GEMM_PSTAGES 4
#endif
constexpr int PBM = 256, PSTAGES = IB_GEMM_PSTAGES;
constexpr int P_A_BYTES = PBM * BK * 2;
constexpr int P_STAGE_BYTES = P_A_BYTES + 128 * BK * 2;           // sized for the wider tile
constexpr int P_SMEM_BYTES = PSTAGES * P_STAGE_BYTES + 1024 + 256;
constexpr int P_TMEM_COLS = 512;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// The epilogue of the persistent kernels for one thread's accumulator row: COLS columns from tensor memory at `taddr`
// to out[a_row, n_base ...]. Columns go in groups of 64: four tensor-memory loads under one wait, and with a residual
// the group's 64 floats are requested before that wait (the first group's by the caller, before the accumulator is
// even complete, through res_first/res_next), so that a row costs a few memory round trips instead of one per 16 columns.
constexpr int DRAIN_GROUP = 4;
struct ResidualAhead {
    float4 r[DRAIN_GROUP][4];
    bool on;                                                      // the vector path of epilogue_store will be taken
};
template <int COLS>
__device__ __forceinline__ void residual_request(const GemmParams& p, ResidualAhead& ra, int64_t a_row, int64_t n_base, int c) {
    if (!ra.on) return;
    const float* row = p.residual + a_row * p.N + n_base + c;
#pragma unroll
    for (int g = 0; g < DRAIN_GROUP; g++) {
        if (c + 16 * g < COLS && n_base + c + 16 * g + 16 <= p.N) {
            const float4* r4 = reinterpret_cast<const float4*>(row + 16 * g);
#pragma unroll
            for (int j = 0; j < 4; j++) ra.r[g][j] = r4[j];
        }
    }
}
template <typename TOut, int COLS>
__device__ __forceinline__ void drain_row(const GemmParams& p, uint32_t taddr, int64_t a_row, int64_t n_base, ResidualAhead& ra) {
    static_assert(COLS % 16 == 0, "columns come in chunks of 16");
    if (p.epi != 0 || p.residual == nullptr) {
        // nothing to read from memory: chunk by chunk (measured faster than groups for the SwiGLU and bias epilogues)
#pragma unroll 1
        for (int c = 0; c < COLS; c += 16) {
            uint32_t raw[16];
            tmem_ld16(taddr + uint32_t(c), raw);
            tmem_ld_wait();
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; j++) v[j] = __uint_as_float(raw[j]);
            epilogue_store<TOut>(p, v, a_row, n_base + c);
        }
        return;
    }
#pragma unroll 1
    for (int c = 0; c < COLS; c += 16 * DRAIN_GROUP) {
        uint32_t raw[DRAIN_GROUP][16];
#pragma unroll
        for (int g = 0; g < DRAIN_GROUP; g++)
            if (c + 16 * g < COLS) tmem_ld16(taddr + uint32_t(c + 16 * g), raw[g]);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < DRAIN_GROUP; g++) {
            if (c + 16 * g < COLS) {
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; j++) v[j] = __uint_as_float(raw[g][j]);
                const int64_t n0 = n_base + c + 16 * g;
                if (ra.on && n0 + 16 <= p.N) epilogue_store<TOut, true>(p, v, a_row, n0, 16, ra.r[g]);
                else epilogue_store<TOut, false>(p, v, a_row, n0);
            }
        }
        if (c + 16 * DRAIN_GROUP < COLS) residual_request<COLS>(p, ra, a_row, n_base, c + 16 * DRAIN_GROUP);
    }
}

template <int PBN, bool WIDE, typename TOut>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    constexpr int S = PSTAGES;
    // WIDE: 128 tokens x PBN features per tile (PBN up to 256), one M=128 x N=PBN MMA per k-step (the A operand is
    // read once for all columns: less shared-memory traffic per flop); else 256 tokens x PBN features, two M=128 MMAs.
    constexpr int TM = WIDE ? 128 : PBM, TN = PBN;
    static_assert(PBN % 16 == 0 && PBN <= (WIDE ? 256 : 128), "tile width");
    constexpr int A_BYTES = TM * BK * 2, B_BYTES = TN * BK * 2;
    const uint32_t bars = base + S * P_STAGE_BYTES;               // full[S], empty[S], acc_full[2], acc_empty[2]
    volatile uint32_t* slots = reinterpret_cast<volatile uint32_t*>(base_ptr + S * P_STAGE_BYTES + (2 * S + 4) * 8);
    // slots[0] = TMEM base address, slots[1] = abort flag
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = int((p.rows_a + TM - 1) / TM), tiles_n = int((p.rows_b + TN - 1) / TN);
    const int n_tiles = tiles_m * tiles_n;
    const int n_kb = p.kb_total;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (S + s); };
    auto acc_full_bar = [&](int b) { return bars + 8u * (2 * S + b); };
    auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * S + 2 + b); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; b++) { mbar_init(acc_full_bar(b), 1); mbar_init(acc_empty_bar(b), 4); }
        slots[1] = 0;
        fence_barrier_init();
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(&slots[0])), P_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = slots[0];

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (p.early_release && lane != 0) ib::pdl_launch_dependents();
        if (lane == 0) {
            ib::pdl_wait();
            int it = 0, issued = 0;
            const uint64_t once = policy_evict_first();
            for (int tile = blockIdx.x; tile < n_tiles && !slots[1]; tile += gridDim.x) {
                const int tm = tile % tiles_m, tn = tile / tiles_m;    // neighbouring CTAs share the weight tile
                for (int kb = 0; kb < n_kb; kb++, it++) {
                    const int s = it % S;
                    if (it >= S && !mbar_wait(empty_bar(s), ((it / S) - 1) & 1)) {
                        atomicExch(p.status, STATUS_TIMEOUT_PRODUCER); slots[1] = 1; break;
                    }
                    if (slots[1]) break;
                    const uint32_t a_dst = base + s * P_STAGE_BYTES, b_dst = a_dst + A_BYTES;
                    mbar_expect_tx(full_bar(s), A_BYTES + B_BYTES);
                    tma_load_2d(a_dst, &tm_a, full_bar(s), kb * BK, tm * TM);
                    if (p.weights_once) tma_load_2d_once(b_dst, &tm_b, full_bar(s), kb * BK, tn * TN, once);
                    else tma_load_2d(b_dst, &tm_b, full_bar(s), kb * BK, tn * TN);
                    issued = it + 1;
                }
            }
            if (slots[1]) {
                // Drain: wait (bounded) until every copy this thread started has landed.
                for (int i = max(0, issued - S); i < issued; i++) mbar_wait(full_bar(i % S), (i / S) & 1);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(TN);
            int it = 0, lt = 0;
            for (int tile = blockIdx.x; tile < n_tiles && !slots[1]; tile += gridDim.x, lt++) {
                const int b = lt & 1;
                if (lt >= 2 && !mbar_wait(acc_empty_bar(b), ((lt >> 1) - 1) & 1)) {      // the epilogue has drained it
                    atomicExch(p.status, STATUS_TIMEOUT_MMA); slots[1] = 1; break;
                }
                tc_fence_after();
                const uint32_t d0 = tmem_base + uint32_t(b * 256), d1 = d0 + 128u;
                for (int kb = 0; kb < n_kb; kb++, it++) {
                    const int s = it % S;
                    if (!mbar_wait(full_bar(s), (it / S) & 1)) {
                        atomicExch(p.status, STATUS_TIMEOUT_MMA); slots[1] = 1; break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = base + s * P_STAGE_BYTES;
                    const uint64_t a0 = make_desc(a_addr), a1 = make_desc(a_addr + 128 * BK * 2), bd = make_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
                        if constexpr (WIDE) {
                            umma_f16(d0, a0 + uint64_t(2 * k), bd + uint64_t(2 * k), idesc, acc);
                        } else {
                            umma_f16(d0, a0 + uint64_t(2 * k), bd + uint64_t(2 * k), idesc, acc);
                            umma_f16(d1, a1 + uint64_t(2 * k), bd + uint64_t(2 * k), idesc, acc);
                        }
                    }
                    umma_commit(empty_bar(s));
                }
                if (slots[1]) break;
                umma_commit(acc_full_bar(b));
            }
        }
        ib::pdl_launch_dependents();                     // (unless that happened at the start)
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..5)
        const int quad = warp & 3;
        ib::pdl_wait();
        int lt = 0;
        ResidualAhead ra;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, lt++) {
            const int tm = tile % tiles_m, tn = tile / tiles_m;
            const int b = lt & 1;
            const int64_t row0 = int64_t(tm) * TM + quad * 32 + lane, n_base = int64_t(tn) * TN;
            // the first 64 residual values of this thread's row travel while the tile's last MMAs still run
            ra.on = p.epi == 0 && p.residual != nullptr && (p.N & 7) == 0 && row0 < p.M;
            residual_request<TN>(p, ra, row0, n_base, 0);
            bool ok = !slots[1] && mbar_wait(acc_full_bar(b), (lt >> 1) & 1);
            if (!ok && !slots[1]) { atomicExch(p.status, STATUS_TIMEOUT_EPILOGUE); slots[1] = 1; }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(b * 256);
            if constexpr (WIDE) {
                drain_row<TOut, TN>(p, taddr, row0, n_base, ra);
            } else {
                drain_row<TOut, TN>(p, taddr, row0, n_base, ra);
                const int64_t row1 = row0 + 128;
                ra.on = p.epi == 0 && p.residual != nullptr && (p.N & 7) == 0 && row1 < p.M;
                residual_request<TN>(p, ra, row1, n_base, 0);
                drain_row<TOut, TN>(p, taddr + 128u, row1, n_base, ra);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(b));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, P_TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------ host side

using ib::get_map;

template <int BN, typename TOut>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid, cudaStream_t stream) {
    using C = Cfg<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return ib::fail(IB_ERR_CUDA, "gemm_tc: cannot set shared memory size: %s", cudaGetErrorString(e));
        configured = true;
    }
    if (p.stages < 1 || p.stages > C::MAX_STAGES) return ib::fail(IB_ERR_ARG, "gemm_tc: %d stages (at most %d)", p.stages, C::MAX_STAGES);
    const size_t smem = size_t(p.stages) * C::STAGE_BYTES + C::SMEM_EXTRA + (p.cluster_split && !p.recv_in_ring ? C::RECV_BYTES : 0);
    if (smem > size_t(C::SMEM_BYTES)) return ib::fail(IB_ERR_ARG, "gemm_tc: %d stages and the receive area do not fit", p.stages);
    return ib::launch("gemm_tc", gemm_tc_kernel<BN, TOut>, grid, dim3(NUM_THREADS), smem, stream,
                      p.cluster_split ? unsigned(p.splits) : 1u, ma, mb, p);
}

template <int PBN, bool WIDE, typename TOut>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int sm_count, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<PBN, WIDE, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES);
        if (e != cudaSuccess) return ib::fail(IB_ERR_CUDA, "gemm_tc: cannot set shared memory size: %s", cudaGetErrorString(e));
        configured = true;
    }
    const int64_t tiles = WIDE ? ((p.rows_a + 127) / 128) * ((p.rows_b + PBN - 1) / PBN) : ((p.rows_a + PBM - 1) / PBM) * ((p.rows_b + PBN - 1) / PBN);
    const unsigned ctas = unsigned(tiles < sm_count ? tiles : sm_count);
    return ib::launch("gemm_tc", gemm_tc_persistent_kernel<PBN, WIDE, TOut>, dim3(ctas), dim3(NUM_THREADS), size_t(P_SMEM_BYTES), stream, 1u, ma, mb, p);
}

// Stages of the ring: the default leaves room for a second CTA on the SM (prefill: one tile's epilogue overlaps the
// other's main loop); with the weights on the A side a CTA streams them alone, so it takes as many stages as it has
// k-blocks, up to the whole SM.
template <int BN> int pick_stages(const GemmParams& p) {
    using C = Cfg<BN>;
    if (!p.swap) return C::STAGES;
    if (p.cluster_split) {
        // as many stages as the slice has k-blocks and no more: with the receive area a short slice then still fits
        // beside a second CTA, and its neighbours in the stream can start under it
        const int room = (C::SMEM_BYTES - C::SMEM_EXTRA - C::RECV_BYTES) / C::STAGE_BYTES;
        const int most = room < C::MAX_STAGES - 2 ? room : C::MAX_STAGES - 2;
        const int want = p.kb_per_split < 2 ? 2 : p.kb_per_split;
        return want > most ? most : want;
    }
    const int want = p.kb_per_split < C::STAGES ? C::STAGES : p.kb_per_split;
    return want > C::MAX_STAGES ? C::MAX_STAGES : want;
}

}  // namespace

// Plans a product: how tokens and features map onto the tile, the BN to use, the number of K slices, and the
// float workspace and counters it needs. Returns 0, or IB_ERR_ARG if the kernel does not take the sizes.
IB_EXPORT int ib_gemm_tc_plan(int64_t M, int64_t N, int64_t K, int sm_count, int* swap, int* bn, int* splits,
                              int64_t* workspace_floats, int64_t* n_counters) {
    if (M <= 0 || N <= 0 || K <= 0) return ib::fail(IB_ERR_ARG, "gemm_tc: sizes must be positive");
    if (K % 8) return ib::fail(IB_ERR_ARG, "gemm_tc: K = %lld is not a multiple of 8 (TMA needs a 16-byte row pitch)", (long long)K);
    if (M >= (1LL << 31) || N >= (1LL << 31) || K >= (1LL << 31)) return ib::fail(IB_ERR_ARG, "gemm_tc: a size exceeds 2^31");
    const int kb_total = int((K + BK - 1) / BK);
    *swap = M <= 128 ? 1 : 0;
    if (*swap) *bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128)); else *bn = 128;
    const int64_t rows_a = *swap ? N : M, rows_b = *swap ? M : N;
    const int64_t tiles = ((rows_a + BM - 1) / BM) * ((rows_b + *bn - 1) / *bn);
    if ((rows_b + *bn - 1) / *bn > 65535) return ib::fail(IB_ERR_ARG, "gemm_tc: too many tiles on the grid's second axis");
    // Slices of K only when the tiles alone leave most of the GPU idle.
    int s = 1;
    bool cluster = false;                                         // (plain mapping) the slices form a cluster
    if (sm_count > 0 && tiles * 2 < sm_count) {
        if (*swap) {
            // decode: the slices of a tile form a cluster (at most 8 CTAs) and are added through distributed shared
            // memory; each slice keeps at least two k-blocks
            s = int(sm_count / tiles);
            if (s > 8) s = 8;
            if (s > kb_total / 2) s = kb_total / 2 > 0 ? kb_total / 2 : 1;
        } else {
            // each slice keeps at least four k-blocks
            s = int((sm_count + tiles - 1) / tiles);
            if (s > 16) s = 16;
            if (s > kb_total / 4) s = kb_total / 4 > 0 ? kb_total / 4 : 1;
            // 2, 4 or 8 slices meet in the cluster's shared memory like those of the swapped mapping (the most that
            // leaves at most a quarter of the CTAs to a second round)
            // (unless the tiles are so few that even 8 slices each leave half of the GPU idle: then up to 16 through
            // the workspace)
            for (int c = 8; c >= 2 && tiles * 16 > sm_count; c /= 2) {
                const int kper = (kb_total + c - 1) / c;
                if (c <= s * 2 && tiles * c <= sm_count + sm_count / 4 && kper >= 2 && (kb_total + kper - 1) / kper == c) { s = c; cluster = true; break; }
            }
        }
    }
    const int per = (kb_total + s - 1) / s;
    s = (kb_total + per - 1) / per;
    *splits = s;
    // Many tokens and enough 256 x 128 tiles to occupy the GPU: the persistent kernel (bn = 256 stands for it).
    static const bool persistent_on = [] { const char* e = getenv("INFER_B200_GEMM_PERSISTENT"); return !(e && e[0] == '0'); }();
    if (!*swap && s == 1 && persistent_on && sm_count > 0) {
        // bn = 512, 384, 352 stand for tiles of 128 tokens x 256, 192, 176 features (one MMA per k-step), 256 for
        // 256 x 128 (two MMAs). Among the 128-row tiles the one with the least estimated time wins: rounds over the
        // SMs times (width + 224), the constant being what a tile costs beside its columns (operand rows of the
        // A side, the exposed epilogue). A matrix of 1536 features gets 16 x 9 tiles of 176 columns for 148 SMs
        // (measured at 2,048 tokens: down 60 us against 70 with 256 columns, o 21 against 25).
        const int64_t tm = (M + PBM - 1) / PBM, tm128 = (M + 127) / 128;
        const int64_t t128 = tm * ((N + 127) / 128);
        static const bool wide_on = [] { const char* e = getenv("INFER_B200_GEMM_WIDE"); return !(e && e[0] == '0'); }();
        int64_t best = -1, best_tiles = 0;
        int best_code = 256;
        for (int width : {256, 192, 176}) {
            const int64_t t = tm128 * ((N + width - 1) / width);
            const int64_t cost = ((t + sm_count - 1) / sm_count) * (width + 224);
            if (best < 0 || cost < best) { best = cost; best_code = 2 * width; best_tiles = t; }
        }
        // Also where the tiles fill only 40 % of the SMs (a 512-token portion of a prompt at 3584 features: 84 tiles):
        // the one-tile kernel without K slices then reads (128 + 128) operand rows per 128 x 128 outputs on every SM at
        // once and loses to it (down at 7B sizes, 512 tokens: 127 us against 105; q/k/v 28 against 24).
        if (t128 * 2 >= sm_count || (wide_on && best_tiles * 5 >= int64_t(sm_count) * 2)) *bn = wide_on ? best_code : 256;
    }
    // A long K on tiles that leave SMs idle (down at 3584 features, a 512-token portion: 84 tiles of 176 columns, 296
    // k-blocks each; or at 1536 features: 48 tiles of 128 columns in two slices): tiles of 128 x 256 whose K slices form
    // a cluster of 2, 4 or 8 (bn = 768 stands for them), the slices' columns meeting in the owners' operand rings.
    // The ways are compared by a model fitted to measurements (unit: the time of one k-block of a sliced tile, 0.38 us):
    // a CTA of 128 x 128 or of 128 x 256 takes one unit per k-block, the persistent kernel 0.4 + width / 330; beside
    // that a one-tile kernel costs 20 units, a sliced wide one 34 (40 with eight slices: the exchange), the persistent
    // one 10. A grid of clusters runs at once only if it leaves the SMs free that clusters cannot use.
    static const bool sliced_on = [] { const char* e = getenv("INFER_B200_GEMM_SLICED"); return !(e && e[0] == '0'); }();
    if (!*swap && sliced_on && sm_count > 0) {
        auto room = [&](int c) -> int64_t { return c == 1 ? 2 * int64_t(sm_count) : (c == 2 ? sm_count - 4 : sm_count - sm_count / 7); };
        const int64_t tm128 = (M + 127) / 128, t256 = tm128 * ((N + 255) / 256);
        int slices = 0;
        int64_t sliced = 0;                                       // in hundredths of a unit
        for (int c : {2, 4, 8}) {
            if (t256 * c > room(c) || kb_total / c < 16) continue;
            const int64_t est = 100 * (int64_t(kb_total + c - 1) / c) + (c == 8 ? 4000 : 3400);
            if (!slices || est < sliced) { slices = c; sliced = est; }
        }
        if (slices) {
            int64_t other;
            if (*bn >= 256) {                                     // the persistent kernel
                const int64_t width = *bn == 256 ? 256 : *bn / 2, rows = *bn == 256 ? 256 : 128;
                const int64_t t = ((M + rows - 1) / rows) * ((N + (*bn == 256 ? 128 : width) - 1) / (*bn == 256 ? 128 : width));
                other = ((t + sm_count - 1) / sm_count) * kb_total * (40 + width * 100 / 330) + 1000;
            } else {                                              // one 128 x 128 tile per CTA, s slices
                const int64_t ctas = tiles * s, cap = cluster ? room(s) : 2 * int64_t(sm_count);
                other = ((ctas + cap - 1) / cap) * 100 * (int64_t(kb_total + s - 1) / s) + 2000;
            }
            if (sliced * 23 < other * 20) { *bn = 768; s = slices; *splits = s; cluster = true; }
        }
    }
    *workspace_floats = (s > 1 && !*swap && !cluster) ? int64_t(s) * tiles * BM * (*bn) : 0;
    *n_counters = (s > 1 && !*swap && !cluster) ? tiles : 0;
    return IB_OK;
}

// out[M, N] = x[M, K] . w[N, K]^T (+ bias) (+ residual), or with epi = 2 out[M, N/2] = SwiGLU of feature rows
// interleaved in blocks of 8 (8 gate rows, then the 8 matching up rows). x, w bfloat16 with 16-byte aligned bases; out float or
// bfloat16; bias, residual float. swap/bn/splits come from ib_gemm_tc_plan (or a caller's override within the same
// rules); workspace holds splits * tiles * 128 * bn floats and counters `tiles` zeroed words when splits > 1.
// The workspace and counters are shared by every call that passes them: calls on different streams must not overlap.
IB_EXPORT int ib_gemm_tc(const void* x, const void* w, const float* bias, const float* residual, void* out, int64_t M,
                         int64_t N, int64_t K, int out_dtype, int epi, int swap, int bn, int splits, float* workspace,
                         unsigned int* counters, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IB_OK;
    if (K <= 0 || K % 8) return ib::fail(IB_ERR_ARG, "gemm_tc: K = %lld must be a positive multiple of 8", (long long)K);
    if ((uintptr_t(x) & 15) || (uintptr_t(w) & 15)) return ib::fail(IB_ERR_ARG, "gemm_tc: operand bases must be 16-byte aligned");
    if (bn != 16 && bn != 32 && bn != 64 && bn != 128 && bn != 256 && bn != 352 && bn != 384 && bn != 512 && bn != 768)
        return ib::fail(IB_ERR_ARG, "gemm_tc: bn must be 16, 32, 64, 128, or 256 (the persistent kernel on 256 x 128 tiles), 352, 384, 512 (on 128 x 176, 128 x 192, 128 x 256 with one MMA per k-step) or 768 (one 128 x 256 tile per CTA, K slices as a cluster)");
    const bool sliced_wide = bn == 768;
    if (sliced_wide) {
        if (swap || workspace || (splits != 2 && splits != 4 && splits != 8)) return ib::fail(IB_ERR_ARG, "gemm_tc: 128 x 256 tiles with K slices take the plain mapping, 2, 4 or 8 slices and no workspace");
        bn = 256;
    } else if (bn >= 256 && (swap || splits > 1)) return ib::fail(IB_ERR_ARG, "gemm_tc: the persistent kernel takes the plain mapping without K slices");
    if (!status) return ib::fail(IB_ERR_ARG, "gemm_tc: a status word is required");
    if (epi != 0 && epi != 2) return ib::fail(IB_ERR_ARG, "gemm_tc: unknown epilogue %d", epi);
    if (epi == 2 && (N % 16 || bias || residual)) return ib::fail(IB_ERR_ARG, "gemm_tc: the SwiGLU epilogue needs N %% 16 == 0 and no bias or residual");
    GemmParams p;
    p.epi = epi;
    p.swap = swap ? 1 : 0;
    p.M = M; p.N = N; p.K = K;
    p.rows_a = swap ? N : M;
    p.rows_b = swap ? M : N;
    p.kb_total = int((K + BK - 1) / BK);
    if (splits < 1) splits = 1;
    if (splits > p.kb_total) splits = p.kb_total;
    p.kb_per_split = (p.kb_total + splits - 1) / splits;
    p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
    p.cluster_split = (p.splits > 1 && !workspace) ? 1 : 0;
    p.recv_in_ring = sliced_wide ? 1 : 0;
    p.weights_once = 1; p.early_release = 1;
    if (sliced_wide && !p.cluster_split) return ib::fail(IB_ERR_ARG, "gemm_tc: K = %lld is too short for %d slices of 128 x 256 tiles", (long long)K, splits);
    if (p.cluster_split && (p.splits > 8 || (!swap && (BM % p.splits || (BM / p.splits) % 16))))
        return ib::fail(IB_ERR_ARG, "gemm_tc: split-K without a workspace takes at most 8 slices, in the plain mapping 2, 4 or 8 (whole 16-column chunks per owner)");
    if (p.splits > 1 && !p.cluster_split && !counters) return ib::fail(IB_ERR_ARG, "gemm_tc: split-K through the workspace needs counters");
    p.bias = bias; p.residual = residual; p.out = out;
    p.workspace = workspace; p.counters = counters; p.status = status;
    const unsigned ta = unsigned((p.rows_a + BM - 1) / BM), tb = unsigned((p.rows_b + bn - 1) / bn);
    if (tb > 65535 || (p.cluster_split && ta > 65535)) return ib::fail(IB_ERR_ARG, "gemm_tc: too many tiles on a grid axis");
    const dim3 grid = p.cluster_split ? dim3{unsigned(p.splits), ta, tb} : dim3{ta, tb, unsigned(p.splits)};
    const bool f32 = out_dtype == IB_F32;
    if (!f32 && out_dtype != IB_BF16) return ib::fail(IB_ERR_ARG, "gemm_tc: unknown output dtype %d", out_dtype);
    CUtensorMap ma, mb;
    if (bn >= 256 && !sliced_wide) {
        const bool wide = bn >= 352 && bn <= 512;
        int rc = get_map(x, p.rows_a, K, wide ? 128 : PBM, &ma);
        if (rc) return rc;
        rc = get_map(w, p.rows_b, K, wide ? bn / 2 : 128, &mb);
        if (rc) return rc;
        static int sms = 0;
        if (!sms) {
            int dev = 0;
            if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
                return ib::fail(IB_ERR_CUDA, "gemm_tc: cannot read the number of SMs");
        }
        p.splits = 1; p.cluster_split = 0; p.stages = PSTAGES;
        p.weights_once = N * K * 2 <= (64LL << 20) ? 1 : 0;
        {
            // k-blocks a CTA goes through: up to about 300 (120 us) the successor is released at once
            const int64_t tm_rows = wide ? 128 : PBM, tn_cols = wide ? bn / 2 : 128;
            const int64_t n_tiles = ((M + tm_rows - 1) / tm_rows) * ((N + tn_cols - 1) / tn_cols);
            p.early_release = ((n_tiles + sms - 1) / sms) * p.kb_total * (wide ? 1 : 2) <= 300 ? 1 : 0;
        }
        if (bn == 512) return f32 ? launch_persistent<256, true, float>(ma, mb, p, sms, stream) : launch_persistent<256, true, bf16>(ma, mb, p, sms, stream);
        if (bn == 384) return f32 ? launch_persistent<192, true, float>(ma, mb, p, sms, stream) : launch_persistent<192, true, bf16>(ma, mb, p, sms, stream);
        if (bn == 352) return f32 ? launch_persistent<176, true, float>(ma, mb, p, sms, stream) : launch_persistent<176, true, bf16>(ma, mb, p, sms, stream);
        return f32 ? launch_persistent<128, false, float>(ma, mb, p, sms, stream) : launch_persistent<128, false, bf16>(ma, mb, p, sms, stream);
    }
    int rc = get_map(swap ? w : x, p.rows_a, K, BM, &ma);
    if (rc) return rc;
    rc = get_map(swap ? x : w, p.rows_b, K, bn, &mb);
    if (rc) return rc;
    if (sliced_wide) {
        p.stages = p.kb_per_split >= 4 ? 4 : 3;          // the ring also receives the slices' columns: 128 KB
        return f32 ? launch<256, float>(ma, mb, p, grid, stream) : launch<256, bf16>(ma, mb, p, grid, stream);
    }
    p.stages = bn == 16 ? pick_stages<16>(p) : bn == 32 ? pick_stages<32>(p) : bn == 64 ? pick_stages<64>(p) : pick_stages<128>(p);
    switch (bn) {
        case 16: return f32 ? launch<16, float>(ma, mb, p, grid, stream) : launch<16, bf16>(ma, mb, p, grid, stream);
        case 32: return f32 ? launch<32, float>(ma, mb, p, grid, stream) : launch<32, bf16>(ma, mb, p, grid, stream);
        case 64: return f32 ? launch<64, float>(ma, mb, p, grid, stream) : launch<64, bf16>(ma, mb, p, grid, stream);
        default: return f32 ? launch<128, float>(ma, mb, p, grid, stream) : launch<128, bf16>(ma, mb, p, grid, stream);
    }
}

// ================================================================================================
// The variant that allocates nothing (declared and explained in gemm_static.h).
#include "gemm_static.h"

namespace {

// Split-K scratch of ib_gemm_tc_static: [counters: IB_STATIC_COUNTERS words][partial tiles: the rest, as floats].
// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[IB_GEMM_STATIC_SCRATCH_BYTES];
constexpr int64_t IB_STATIC_COUNTERS = 4096;                                    // per-tile arrival counters (16 KiB)
constexpr int IB_STATIC_MAX_DEVICES = 64;

// Device address of g_static_scratch on `device`, looked up once per device with that device current.
int static_scratch(int device, unsigned char** ptr) {
    static unsigned char* addr[IB_STATIC_MAX_DEVICES] = {};
    static std::mutex mu;
    if (device < 0 || device >= IB_STATIC_MAX_DEVICES) return ib::fail(IB_ERR_ARG, "gemm_tc_static: device %d out of range", device);
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[device]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);      // the current device is `device`
        if (e != cudaSuccess) return ib::fail(IB_ERR_CUDA, "gemm_tc_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        addr[device] = static_cast<unsigned char*>(p);
    }
    *ptr = addr[device];
    return IB_OK;
}

}  // namespace

IB_EXPORT int ib_gemm_tc_static(const void* x, const void* w, const float* bias, const float* residual, void* out, int64_t M,
                                int64_t N, int64_t K, int out_dtype, int sm_count, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IB_OK;
    int swap = 0, bn = 0, splits = 1;
    int64_t ws_floats = 0, n_counters = 0;
    int rc = ib_gemm_tc_plan(M, N, K, sm_count > 0 ? sm_count : 148, &swap, &bn, &splits, &ws_floats, &n_counters);
    if (rc) return rc;
    float* workspace = nullptr;
    unsigned int* counters = nullptr;
    // Only a plan that sums its K slices through global memory (ws_floats > 0) gets the array. The other split plans
    // (up to 128 rows, and clusters of 2, 4 or 8 slices) add their slices in the cluster's shared memory and must be
    // given no workspace: with one, ib_gemm_tc would take the global-memory path, whose need the plan did not state.
    if (splits > 1 && ws_floats > 0) {
        const int64_t room = (int64_t(IB_GEMM_STATIC_SCRATCH_BYTES) - IB_STATIC_COUNTERS * 4) / 4;
        if (ws_floats > room || n_counters > IB_STATIC_COUNTERS)
            return ib::fail(IB_ERR_ARG, "gemm_tc_static: M=%lld N=%lld K=%lld needs %lld bytes of split-K scratch and %lld counters; "
                            "the built-in array holds %lld bytes and %lld counters",
                            (long long)M, (long long)N, (long long)K, (long long)(ws_floats * 4), (long long)n_counters,
                            (long long)(room * 4), (long long)IB_STATIC_COUNTERS);
        int device = 0;
        cudaError_t e = cudaGetDevice(&device);
        if (e != cudaSuccess) return ib::fail(IB_ERR_CUDA, "gemm_tc_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
        unsigned char* base = nullptr;
        rc = static_scratch(device, &base);
        if (rc) return rc;
        counters = reinterpret_cast<unsigned int*>(base);
        workspace = reinterpret_cast<float*>(base + IB_STATIC_COUNTERS * 4);
        // The counters must start at zero; earlier calls leave them so, but a call that was cut short would not.
        e = cudaMemsetAsync(counters, 0, size_t(n_counters) * 4, stream);
        if (e != cudaSuccess) return ib::fail(IB_ERR_CUDA, "gemm_tc_static: clearing the counters failed: %s", cudaGetErrorString(e));
    }
    return ib_gemm_tc(x, w, bias, residual, out, M, N, K, out_dtype, 0, swap, bn, splits, workspace, counters, status, stream);
}

#ifdef IB_GEMM_TRACE
IB_EXPORT int ib_gemm_tc_trace(long long* host) {
    return cudaMemcpyFromSymbol(host, ib_gemm_trace, sizeof(ib_gemm_trace)) == cudaSuccess ? IB_OK : IB_ERR_CUDA;
}
#endif
