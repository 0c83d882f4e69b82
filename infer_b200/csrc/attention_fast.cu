// Attention over the paged bfloat16 cache on tensor cores (mma.sync m16n8k16, float accumulation, online softmax
// in float), compiled for one head size: -DIB_HEAD_DIM=<multiple of 16, at most 128>. Pages hold 16 positions.
//
// Two kernels share one launch call; each segment (a request's tokens in this step) goes to one of them:
//
//  decode  (segments of ONE token)   grid (slices, kv heads, segments). The query heads that share a kv head are
//          the 8 columns of one MMA tile and a page's 16 keys its rows (S^T = K Q^T, then O^T = V^T P^T with P^T
//          turned into the B operand by movmatrix), so a key or value is read once for the whole group and a page
//          costs 16 MMAs, not 32: the legacy tensor path issues about one m16n8k16 per 32 cycles and scheduler on
//          sm_100, and that, not bytes, bounds this kernel at short contexts. The key range is cut
//          into slices (flash-decoding); inside a CTA each of the 6 warps walks its own pages (a page is a
//          contiguous 16 x head_dim block per kv head) through a ring of 2 stages that is requested whole before
//          the kernel waits for its predecessor, with its own running maximum, sum and output, merged in shared
//          memory at the end. For head sizes 64 and 128 a page arrives by TMA (cp.async.bulk.tensor, 128-byte
//          swizzle, completion on an mbarrier per stage), otherwise by 16-byte cp.async into padded rows. Six warps
//          and two stages are what measured best inside a decode step at 2,048-token contexts (0.94-0.96 ms at
//          batch 1, 1.04-1.05 at batch 8; four warps and three stages 1.00 / 1.08; anything above about 100 KB of
//          shared memory no longer fits beside a neighbouring product's CTA and loses 15 %). Up to 8 slices form a thread-block cluster
//          and meet through distributed shared memory; for long contexts at small batches several clusters share a
//          (segment, kv head): each leaves (max, sum, unnormalised output) in the workspace and the CTA that arrives
//          last at the (segment, kv head) counter adds the clusters in ascending order and writes the result.
//
//  prefill (segments of 2 or more tokens)   grid (heads, query tiles from the last to the first, segments). 64 queries of one head per CTA,
//          16 per warp; keys in tiles of 64 (4 pages) aligned to absolute multiples of 64, double-buffered with
//          cp.async, causal and window masks applied in registers.
//
// A key j is visible to the query at position p iff max(0, p - window + 1) <= j <= p (window 0: every j <= p).
// Rows of keys or values that are not visible and not yet written are zero-filled in shared memory, so stale
// cache contents can never reach a sum. Page ids outside the pool raise the status word and read as zeros.
#include "common.cuh"
#include "tma_map.cuh"

#include <cooperative_groups.h>

IB_DEFINE_LAST_ERROR()

#ifndef IB_HEAD_DIM
#define IB_HEAD_DIM 128
#endif

namespace {

namespace cg = cooperative_groups;
using bf16 = __nv_bfloat16;

constexpr int HD = IB_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128, "head_dim must be a multiple of 16 in [16, 128]");
constexpr int PAGE = 16;
constexpr int ROW_BYTES = HD * 2 + 16;          // padded row: 8 consecutive rows start in 8 different 16-byte bank groups
constexpr int CHUNKS = HD / 8;                  // 16-byte chunks per row
constexpr int KS = HD / 16;                     // k-steps over the head dimension
constexpr float LOG2E = 1.4426950408889634f;

#ifndef IB_DEC_WARPS
#define IB_DEC_WARPS 6
#endif
#ifndef IB_DEC_STAGES
#define IB_DEC_STAGES 2
#endif
constexpr int DEC_WARPS = IB_DEC_WARPS, DEC_STAGES = IB_DEC_STAGES;
constexpr int MAX_SPLITS = 8;                   // slices of the key range per cluster
constexpr int MAX_SUPER = 32;                   // clusters per (segment, kv head)
constexpr int WS_STRIDE = 16 * HD + 32;         // floats a cluster leaves in the workspace: [16][HD] output, [16][2] max and sum
// The decode kernel's pages arrive by TMA where a row is whole 128-byte swizzle lines (head sizes 64 and 128): one
// tensor copy per 16 rows x 64 elements, 128-byte swizzle, no padding. Other head sizes use 16-byte cp.async into
// padded rows.
#ifndef IB_DEC_TMA
#define IB_DEC_TMA 1
#endif
constexpr bool TMA_PAGES = IB_DEC_TMA && HD % 64 == 0;
constexpr int PAGE_TILE_BYTES = TMA_PAGES ? PAGE * HD * 2 : PAGE * ROW_BYTES;   // K (or V) rows of one page in shared memory
constexpr int DEC_STAGE_BYTES = 2 * PAGE_TILE_BYTES;                        // K page + V page
constexpr int DEC_RING_BYTES = DEC_WARPS * DEC_STAGES * DEC_STAGE_BYTES;
constexpr int DEC_SMEM = DEC_RING_BYTES + (TMA_PAGES ? 1024 : 0);           // swizzled tiles start on 1024-byte boundaries
constexpr int MO_PITCH = HD + 8;                // floats between rows of a warp's partial output: 8-byte stores of a half-warp hit 32 banks
constexpr int DEC_MERGE_BYTES = DEC_WARPS * (16 * MO_PITCH + 32) * 4;
static_assert(DEC_MERGE_BYTES <= DEC_RING_BYTES, "merge area must fit the stage area");

constexpr int PF_BM = 64, PF_BN = 64, PF_WARPS = 4;
constexpr int PF_TILE_BYTES = PF_BN * ROW_BYTES;
constexpr int PF_SMEM = PF_BM * ROW_BYTES + 2 * 2 * PF_TILE_BYTES;          // Q + 2 stages of (K, V)

struct AttnParams {
    const bf16* q; const bf16* k_cache; const bf16* v_cache; bf16* out;
    const bf16* qkv; const float* cos; const float* sin; bf16* k_cache_w; bf16* v_cache_w; int write_cache;   // fused decode
    const void* prefetch; int64_t prefetch_bytes;      // weights of a later kernel to pull into L2 meanwhile
    const int* block_table; int max_blocks;
    const int* seg_start; const int* seg_pos0;
    int n_heads, n_kv, group, window;
    float scale_log2;                      // softmax scale * log2(e)
    int64_t n_pages;
    int n_splits, n_super;
    float* workspace; unsigned int* counters; int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

// 16-byte asynchronous copy; src_bytes = 0 writes zeros.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// Bulk asynchronous copies of whole cache rows, counted on an mbarrier (the decode kernel's page ring).
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
// Bounded wait (about a second): false if the phase did not complete.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 22); i++) {
        if (mbar_test(bar, parity)) return true;
        if (i > 2048) __nanosleep(64);
    }
    return false;
}
// A page of the cache for the decode kernel: a decode step reads every page of its requests once, so the tiles are
// marked to leave L2 first; with the default policy a batch's cache (134 MB per layer at 64 x 2,048 tokens) pushed
// out what the neighbouring kernels read again: their activations and their own instructions (batch 64: 2.21 -> 2.07 ms
// per step; batch 8: 1.033 -> 1.021).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(pol) : "memory");
}
// Byte offset of the 16-byte chunk c of row r inside a page tile of the decode ring: swizzled 128-byte lines in tiles
// of 64 elements (what the tensor copy writes), or padded rows.
__device__ __forceinline__ uint32_t page_chunk(int r, int c) {
    if constexpr (TMA_PAGES) return uint32_t((c >> 3) * (PAGE * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4));
    else return uint32_t(r * ROW_BYTES + c * 16);
}
constexpr int STATUS_PAGE_TIMEOUT = 105;        // a decode warp's wait for a page ran out

__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Online-softmax update of one 16-row tile held across a warp (rows g and g+8 per thread) with NT score tiles of 8
// keys each; s holds raw dot products and is replaced by probabilities. `vis(row_half, key_offset)` tells visibility.
template <int NT, int OT, typename Vis>
__device__ __forceinline__ void softmax_update(float (*s)[4], float* m, float* l, float (*o)[4], float scale_log2, Vis vis) {
    const int t4 = (threadIdx.x & 3) * 2;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; n++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int half = e >> 1, key = n * 8 + t4 + (e & 1);
            s[n][e] = vis(half, key) ? s[n][e] * scale_log2 : -INFINITY;
            mx[half] = fmaxf(mx[half], s[n][e]);
        }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const float m_new = fmaxf(m[h], mx[h]);
        msafe[h] = m_new == -INFINITY ? 0.0f : m_new;
        corr[h] = exp2f(m[h] - msafe[h]);                  // m = -inf gives 0
        m[h] = m_new;
    }
    float sum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int n = 0; n < NT; n++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float p = exp2f(s[n][e] - msafe[e >> 1]);
            s[n][e] = p;
            sum[e >> 1] += p;
        }
#pragma unroll
    for (int h = 0; h < 2; h++) l[h] = l[h] * corr[h] + sum[h];
    // once the running maximum has settled the factors are exactly 1 for every row of the warp: skip the multiplies
    if (__any_sync(0xffffffffu, (corr[0] != 1.0f) | (corr[1] != 1.0f))) {
#pragma unroll
        for (int n = 0; n < OT; n++) {
            o[n][0] *= corr[0]; o[n][1] *= corr[0];
            o[n][2] *= corr[1]; o[n][3] *= corr[1];
        }
    }
}

// S[16 x 8 NT] += Q[16 x HD] . K^T, K rows (keys) at k_smem with ROW_BYTES pitch; qf = A fragments per k-step.
template <int NT>
__device__ __forceinline__ void qk_tile(float (*s)[4], const uint32_t (*qf)[4], uint32_t k_smem) {
    const int lane = threadIdx.x & 31;
    const int n_off = (lane & 7) + ((lane >> 4) << 3), k_off = ((lane >> 3) & 1) << 3;
#pragma unroll
    for (int ks = 0; ks < KS; ks++)
#pragma unroll
        for (int np = 0; np < NT / 2; np++) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4(k_smem + (np * 16 + n_off) * ROW_BYTES + (ks * 16 + k_off) * 2, b0, b1, b2, b3);
            mma_bf16(s[2 * np], qf[ks], b0, b1);
            mma_bf16(s[2 * np + 1], qf[ks], b2, b3);
        }
}

// O[16 x HD] += P[16 x 8 NT] . V, V rows (keys) at v_smem; probabilities in s (C layout) become A fragments.
template <int NT>
__device__ __forceinline__ void pv_tile(float (*o)[4], const float (*s)[4], uint32_t v_smem) {
    const int lane = threadIdx.x & 31;
    const int key_off = (lane & 7) + (((lane >> 3) & 1) << 3), d_off = (lane >> 4) << 3;
#pragma unroll
    for (int kk = 0; kk < NT / 2; kk++) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int j = 0; j < KS; j++) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_trans(v_smem + (kk * 16 + key_off) * ROW_BYTES + (j * 16 + d_off) * 2, b0, b1, b2, b3);
            mma_bf16(o[2 * j], a, b0, b1);
            mma_bf16(o[2 * j + 1], a, b2, b3);
        }
    }
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// Decode tiles, keys on the rows: S^T[16 keys x 8 NH heads] = K[16 x HD] . Q^T, K rows at k_smem (a page tile);
// qf[nh][ks] = B fragments of Q^T (heads nh*8 .. nh*8+7). Even and odd k-steps go to two accumulators, so the chain of
// dependent MMAs is half as long.
template <int NH>
__device__ __forceinline__ void qk_page(float (*s)[4], const uint32_t (*qf)[KS][2], uint32_t k_smem) {
    const int lane = threadIdx.x & 31;
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8, c0 = lane >> 4;
    float s2[NH][4];
#pragma unroll
    for (int nh = 0; nh < NH; nh++) s2[nh][0] = s2[nh][1] = s2[nh][2] = s2[nh][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        uint32_t a[4];
        ldsm_x4(k_smem + page_chunk(row, ks * 2 + c0), a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int nh = 0; nh < NH; nh++) mma_bf16((ks & 1) ? s2[nh] : s[nh], a, qf[nh][ks][0], qf[nh][ks][1]);
    }
#pragma unroll
    for (int nh = 0; nh < NH; nh++)
#pragma unroll
        for (int e = 0; e < 4; e++) s[nh][e] += s2[nh][e];
}

// O^T[HD x 8 NH heads] += V^T[HD x 16 keys] . P^T: V rows (keys) at v_smem are read transposed as the A operand; the
// probabilities in s (C layout: keys on rows, heads on columns) become the B operand through movmatrix.
template <int NH>
__device__ __forceinline__ void pv_page(float (*o)[HD / 16][4], const float (*s)[4], uint32_t v_smem) {
    const int lane = threadIdx.x & 31;
    uint32_t b[NH][2];
#pragma unroll
    for (int nh = 0; nh < NH; nh++) {
        b[nh][0] = movmatrix_trans(pack_bf16(s[nh][0], s[nh][1]));
        b[nh][1] = movmatrix_trans(pack_bf16(s[nh][2], s[nh][3]));
    }
    const int row = (lane & 7) + (lane >> 4) * 8, c0 = (lane >> 3) & 1;
#pragma unroll
    for (int mt = 0; mt < HD / 16; mt++) {
        uint32_t a[4];
        ldsm_x4_trans(v_smem + page_chunk(row, mt * 2 + c0), a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int nh = 0; nh < NH; nh++) mma_bf16(o[nh][mt], a, b[nh][0], b[nh][1]);
    }
}

// Online softmax of one page in that layout. A thread holds, per group of 8 heads, heads 2 t4 and 2 t4 + 1 of keys g
// and g + 8: s[nh] = {(g, h0), (g, h1), (g+8, h0), (g+8, h1)}. The maximum of a head runs over the lanes that share
// t4; l stays a per-thread share of the sum (the shares are added at the end).
template <int NH>
__device__ __forceinline__ void softmax_page(float (*s)[4], float (*m)[2], float (*l)[2], float (*o)[HD / 16][4], float scale_log2,
                                             bool vis0, bool vis1) {
    bool rescale = false;
    float corr[NH][2];
#pragma unroll
    for (int nh = 0; nh < NH; nh++)
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const float v0 = vis0 ? s[nh][c] * scale_log2 : -INFINITY, v1 = vis1 ? s[nh][2 + c] * scale_log2 : -INFINITY;
            float mx = fmaxf(v0, v1);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m[nh][c], mx);
            const float msafe = m_new == -INFINITY ? 0.0f : m_new;
            corr[nh][c] = exp2f(m[nh][c] - msafe);             // m = -inf gives 0
            m[nh][c] = m_new;
            const float p0 = exp2f(v0 - msafe), p1 = exp2f(v1 - msafe);
            s[nh][c] = p0; s[nh][2 + c] = p1;
            l[nh][c] = l[nh][c] * corr[nh][c] + p0 + p1;
            rescale |= corr[nh][c] != 1.0f;
        }
    // once the running maximum has settled the factors are exactly 1 for every head of the warp: skip the multiplies
    if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int nh = 0; nh < NH; nh++)
#pragma unroll
            for (int mt = 0; mt < HD / 16; mt++) {
                o[nh][mt][0] *= corr[nh][0]; o[nh][mt][1] *= corr[nh][1];
                o[nh][mt][2] *= corr[nh][0]; o[nh][mt][3] *= corr[nh][1];
            }
    }
}

// ================================================================================================ decode
//
// Grid (slices, kv heads, segments); the slices of one (segment, kv head) form a thread-block cluster, and their
// partial results (running maximum, sum, unnormalised output per head of the group) are merged through distributed
// shared memory: each CTA of the cluster combines its share of the output elements from all ranks, in rank order.
//
// FUSED: the kernel reads the packed projection rows [q | k | v] itself, rotates q in registers (half-split rotation:
// element j pairs with j + HD/2, both in the same thread's fragments when HD/2 is a multiple of 16), and the warp that
// owns the page of the new position rotates k, puts k and v into its shared-memory copy of the page and into the
// cache: one launch instead of two.

#ifdef IB_ATTN_DEC_TRACE
// Profiling build: thread 0 of the first CTA records the SM clock at the marks of the decode kernel.
__device__ long long ib_dec_trace[32];
#define IB_DT(k) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) ib_dec_trace[k] = clock64(); } while (0)
#else
#define IB_DT(k) do {} while (0)
#endif

template <bool FUSED, int NH>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* smem = TMA_PAGES ? smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u) : smem_raw;
    // This kernel is a chain of latencies and leaves HBM nearly idle: a good time to fetch a later product's weights.
    ib::l2_prefetch_share(p.prefetch, p.prefetch_bytes, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x,
                          gridDim.x * gridDim.y * gridDim.z);
    // Everything this kernel reads before the wait below was written before the step began (segment and block
    // tables, the cache rows of earlier positions): with the rotation and the cache write fused in, the pages of the
    // old keys are requested while the kernel that makes q, k and v is still running.
    IB_DT(0);
    const bool early = FUSED && p.write_cache;
    if (!early) ib::pdl_wait();
    // blockIdx.x = super-slice * cluster size + rank in the cluster: the key range is cut into gridDim.x slices, the
    // n_splits slices of a cluster meet through distributed shared memory, and clusters (n_super > 1: long contexts at
    // small batches, where one cluster per (segment, kv head) would leave most SMs idle) through the workspace
    const int n_splits = p.n_splits;
    const int split = blockIdx.x & (n_splits - 1), slice = blockIdx.x, kvh = blockIdx.y, seg = blockIdx.z;
    const int n_slices = gridDim.x;
    const int t = p.seg_start[seg];
    const bool is_decode = p.seg_start[seg + 1] - t == 1;         // uniform over the cluster
    if (!is_decode) return;
    const int pos = p.seg_pos0[seg];
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int first_page = lo / PAGE, last_page = pos / PAGE;
    const int n_pg = last_page - first_page + 1;
    const int pps = (n_pg + n_slices - 1) / n_slices;
    const int pg_begin = min(last_page + 1, first_page + slice * pps), pg_end = min(last_page + 1, pg_begin + pps);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int* table = p.block_table + int64_t(seg) * p.max_blocks;
    const int G = p.group;
    const int64_t qkv_row = int64_t(t) * (p.n_heads + 2 * p.n_kv) * HD;

    uint8_t* my_ptr = smem + warp * DEC_STAGES * DEC_STAGE_BYTES;
    const uint32_t my_smem = smem_u32(my_ptr);
    const int my_pages = pg_end > pg_begin + warp ? (pg_end - pg_begin - warp + DEC_WARPS - 1) / DEC_WARPS : 0;

    // The ids of this warp's first 32 pages in one load (lane i holds the i-th): a read of the table per page would put
    // a round trip to L2 in front of every copy.
    int lane_page = -1;
    if (lane < my_pages) lane_page = table[pg_begin + warp + lane * DEC_WARPS];
    // A warp's ring of pages. With TMA_PAGES a page is two tensor copies per 64 elements of the head size (K and V,
    // 16 rows x 128 bytes each, 128-byte swizzle) issued by one lane and counted on the stage's mbarrier: sixteen-byte
    // cp.async took sixteen instructions per lane and page, about 900 cycles of a warp that has 600 of arithmetic per
    // page. Rows that are not written yet (beyond the new position; with FUSED the new position itself, which comes
    // from the projections) are zeroed before use, so that what a page held before can never reach a sum: by the
    // copy's zero fill with cp.async, by stores after the tensor copy has landed.
    __shared__ __align__(8) uint64_t page_bar[DEC_WARPS][DEC_STAGES];
    const int copy_limit = (FUSED && p.write_cache) ? pos : pos + 1;       // keys below this are in the cache
    if constexpr (TMA_PAGES) {
        if (lane < DEC_STAGES) mbar_init(smem_u32(&page_bar[warp][lane]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_k) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_v) : "memory");
        }
        __syncwarp();
    }
    auto issue = [&](int i) {
        if (i < my_pages) {
            const int pg = pg_begin + warp + i * DEC_WARPS;
            int page = i < 32 ? __shfl_sync(0xffffffffu, lane_page, i) : table[pg];
            if (page < 0 || page >= p.n_pages) { atomicExch(p.status, 3); page = -1; }
            const uint32_t dst = my_smem + (i % DEC_STAGES) * DEC_STAGE_BYTES;
            if constexpr (TMA_PAGES) {
                // one lane states the bytes to come; the copies (K and V of every 64-element tile) go out from as many
                // lanes at once, since a tensor copy holds up the lane that issues it for about 150 cycles
                const uint32_t bar = smem_u32(&page_bar[warp][i % DEC_STAGES]);
                if (lane == 0) mbar_expect_tx(bar, page < 0 ? 0u : uint32_t(2 * PAGE_TILE_BYTES));
                __syncwarp();
                if (page >= 0 && lane < 2 * (HD / 64)) {
                    const int bx = lane >> 1, is_v = lane & 1;
                    const int y = (page * p.n_kv + kvh) * PAGE;              // row of the [pages * kv heads * 16, HD] view
                    tma_load_2d(dst + is_v * PAGE_TILE_BYTES + bx * (PAGE * 128), is_v ? &tm_v : &tm_k, bar, bx * 64, y);
                }
            } else {
                const int64_t base = page < 0 ? 0 : ((int64_t(page) * p.n_kv + kvh) * PAGE) * HD;
#pragma unroll
                for (int c = lane; c < PAGE * CHUNKS; c += 32) {
                    const int row = c / CHUNKS, col = c % CHUNKS;
                    const int bytes = (page >= 0 && pg * PAGE + row < copy_limit) ? 16 : 0;
                    cp_async16(dst + row * ROW_BYTES + col * 16, p.k_cache + base + row * HD + col * 8, bytes);
                    cp_async16(dst + PAGE * ROW_BYTES + row * ROW_BYTES + col * 16, p.v_cache + base + row * HD + col * 8, bytes);
                }
            }
        }
        if constexpr (!TMA_PAGES) cp_commit();
    };

    float m[NH][2], l[NH][2];
    float o[NH][HD / 16][4];
#pragma unroll
    for (int nh = 0; nh < NH; nh++) {
        m[nh][0] = m[nh][1] = -INFINITY;
        l[nh][0] = l[nh][1] = 0.0f;
#pragma unroll
        for (int mt = 0; mt < HD / 16; mt++) o[nh][mt][0] = o[nh][mt][1] = o[nh][mt][2] = o[nh][mt][3] = 0.0f;
    }

    // The whole ring is requested now, before the wait for the predecessor: a copy costs its issuer hundreds of cycles
    // (about 150 per tensor copy), which are free here and would sit in the chain of dependent work later.
#pragma unroll
    for (int i = 0; i < DEC_STAGES; i++) issue(i);
    if constexpr (FUSED) {                               // the rotation's table rows, on their way meanwhile
        if (lane * 32 < HD / 2) {
            asm volatile("prefetch.global.L1 [%0];" ::"l"(p.cos + int64_t(pos) * (HD / 2) + lane * 32));
            asm volatile("prefetch.global.L1 [%0];" ::"l"(p.sin + int64_t(pos) * (HD / 2) + lane * 32));
        }
    }
    IB_DT(1);
    if (early) ib::pdl_wait();                           // q, k and v of this step come from the predecessor
    IB_DT(2);

    // Query fragments (the B operand: Q^T) straight from global memory: column g of group nh is head nh * 8 + g of
    // this kv head's group, zero beyond it; a thread holds elements 2 t4, 2 t4 + 1 and those 8 further of every k-step.
    uint32_t qf[NH][KS][2];
    if constexpr (FUSED) {
        const bf16* qb = p.qkv + qkv_row + int64_t(kvh) * G * HD;
        const float* cs = p.cos + int64_t(pos) * (HD / 2);
        const float* sn = p.sin + int64_t(pos) * (HD / 2);
#pragma unroll
        for (int nh = 0; nh < NH; nh++)
#pragma unroll
            for (int ks = 0; ks < KS / 2; ks++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int head = nh * 8 + g, d = ks * 16 + t4 * 2 + e * 8;             // d < HD/2
                    if (head < G) {
                        const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(qb + head * HD + d));
                        const float2 x2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(qb + head * HD + d + HD / 2));
                        const float2 c = *reinterpret_cast<const float2*>(cs + d), sv = *reinterpret_cast<const float2*>(sn + d);
                        qf[nh][ks][e] = pack_bf16(x1.x * c.x - x2.x * sv.x, x1.y * c.y - x2.y * sv.y);
                        qf[nh][ks + KS / 2][e] = pack_bf16(x2.x * c.x + x1.x * sv.x, x2.y * c.y + x1.y * sv.y);
                    } else {
                        qf[nh][ks][e] = 0u;
                        qf[nh][ks + KS / 2][e] = 0u;
                    }
                }
    } else {
        const bf16* qb = p.q + (int64_t(t) * p.n_heads + int64_t(kvh) * G) * HD;
#pragma unroll
        for (int nh = 0; nh < NH; nh++)
#pragma unroll
            for (int ks = 0; ks < KS; ks++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int head = nh * 8 + g;
                    qf[nh][ks][e] = head < G ? *reinterpret_cast<const uint32_t*>(qb + head * HD + ks * 16 + t4 * 2 + e * 8) : 0u;
                }
    }
    IB_DT(3);
    // The warp whose page holds the new position rotates k and puts k and v into its shared-memory copy of the page and
    // into the cache. Their values are requested now, so that they have arrived when the warp gets to that page.
    constexpr int NP = (HD / 2 + 31) / 32;
    const bool owns_new = FUSED && p.write_cache && last_page >= pg_begin && last_page < pg_end &&
                          (last_page - pg_begin) % DEC_WARPS == warp;
    float nk1[NP], nk2[NP], ncs[NP], nsn[NP];
    bf16 nv1[NP], nv2[NP];
    if constexpr (FUSED) {
        if (owns_new) {
            const bf16* kb = p.qkv + qkv_row + (int64_t(p.n_heads) + kvh) * HD;
            const bf16* vb = p.qkv + qkv_row + (int64_t(p.n_heads) + p.n_kv + kvh) * HD;
            const float* cs = p.cos + int64_t(pos) * (HD / 2);
            const float* sn = p.sin + int64_t(pos) * (HD / 2);
#pragma unroll
            for (int u = 0; u < NP; u++) {
                const int j = lane + u * 32;
                if (j < HD / 2) {
                    nk1[u] = __bfloat162float(kb[j]); nk2[u] = __bfloat162float(kb[j + HD / 2]);
                    nv1[u] = vb[j]; nv2[u] = vb[j + HD / 2];
                    ncs[u] = cs[j]; nsn[u] = sn[j];
                }
            }
        }
    }
    // Prepares page i of this warp (its stage has landed): zeroes the rows that the tensor copy brought but that are
    // not written yet, and puts the new position's k and v into the page. Returns the first key of the page.
    auto prepare = [&](int i, uint8_t* stage) -> int {
        const int pg = pg_begin + warp + i * DEC_WARPS;
        const int key0 = pg * PAGE;
        if constexpr (TMA_PAGES) {
            const int n_ok = (i < 32 ? __shfl_sync(0xffffffffu, lane_page, i) : table[pg]) < 0 ? 0 : copy_limit - key0;   // rows that hold cache contents
            if (n_ok < PAGE) {
                // a row is whole 128-byte lines of every 64-element tile, wherever the swizzle puts its chunks
                for (int idx = lane; idx < (PAGE - max(n_ok, 0)) * CHUNKS; idx += 32) {
                    const int row = max(n_ok, 0) + idx / CHUNKS, c = idx % CHUNKS;
                    *reinterpret_cast<uint4*>(stage + page_chunk(row, c)) = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(stage + PAGE_TILE_BYTES + page_chunk(row, c)) = make_uint4(0u, 0u, 0u, 0u);
                }
                __syncwarp();
            }
        }
        if constexpr (FUSED) {
            if (owns_new && pg == last_page) {
                const int page = table[pg];
                const int row = pos - key0;
                uint8_t* ks_tile = stage;
                uint8_t* vs_tile = stage + PAGE_TILE_BYTES;
                const bool page_ok = page >= 0 && page < p.n_pages;
                if (!page_ok && lane == 0) atomicExch(p.status, 2);
                const int64_t gbase = page_ok ? ((int64_t(page) * p.n_kv + kvh) * PAGE + row) * HD : 0;
#pragma unroll
                for (int u = 0; u < NP; u++) {
                    const int j = lane + u * 32;
                    if (j < HD / 2) {
                        const bf16 r1 = __float2bfloat16_rn(nk1[u] * ncs[u] - nk2[u] * nsn[u]);
                        const bf16 r2 = __float2bfloat16_rn(nk2[u] * ncs[u] + nk1[u] * nsn[u]);
                        const uint32_t e1 = page_chunk(row, j >> 3) + (j & 7) * 2, e2 = page_chunk(row, (j + HD / 2) >> 3) + (j & 7) * 2;
                        *reinterpret_cast<bf16*>(ks_tile + e1) = r1; *reinterpret_cast<bf16*>(ks_tile + e2) = r2;
                        *reinterpret_cast<bf16*>(vs_tile + e1) = nv1[u]; *reinterpret_cast<bf16*>(vs_tile + e2) = nv2[u];
                        if (page_ok) {
                            p.k_cache_w[gbase + j] = r1; p.k_cache_w[gbase + j + HD / 2] = r2;
                            p.v_cache_w[gbase + j] = nv1[u]; p.v_cache_w[gbase + j + HD / 2] = nv2[u];
                        }
                    }
                }
                __syncwarp();
            }
        }
        return key0;
    };
    bool pages_ok = true;
    for (int i = 0; i < my_pages; i++) {
        // (a wait that runs out raises the status word; the pages already requested are still waited for, so that no
        // copy is in flight when the ring is reused below)
        if constexpr (TMA_PAGES) {
            if (!mbar_wait(smem_u32(&page_bar[warp][i % DEC_STAGES]), uint32_t(i / DEC_STAGES) & 1u)) {
                if (pages_ok && lane == 0) atomicExch(p.status, STATUS_PAGE_TIMEOUT);
                pages_ok = false;
            }
        } else {
            cp_wait<DEC_STAGES - 1>();
        }
        __syncwarp();
        if (i < 8) IB_DT(4 + 2 * i);
        if (pages_ok) {
            uint8_t* stage = my_ptr + (i % DEC_STAGES) * DEC_STAGE_BYTES;
            const int key0 = prepare(i, stage);
            const uint32_t ka = smem_u32(stage), va = ka + PAGE_TILE_BYTES;
            float s[NH][4];
#pragma unroll
            for (int nh = 0; nh < NH; nh++) s[nh][0] = s[nh][1] = s[nh][2] = s[nh][3] = 0.0f;
            qk_page<NH>(s, qf, ka);
            softmax_page<NH>(s, m, l, o, p.scale_log2, (key0 + g >= lo) & (key0 + g <= pos), (key0 + g + 8 >= lo) & (key0 + g + 8 <= pos));
            pv_page<NH>(o, s, va);
            __syncwarp();
        }
        if (pages_ok || !TMA_PAGES) issue(i + DEC_STAGES);       // into the stage that was just read
        if (i < 8) IB_DT(5 + 2 * i);
    }
    if constexpr (!TMA_PAGES) cp_wait<0>();
    IB_DT(20);
    ib::pdl_launch_dependents();                         // (at the kernel's start instead: every batch size slower)
#pragma unroll
    for (int nh = 0; nh < NH; nh++)
#pragma unroll
        for (int c = 0; c < 2; c++) {                    // the lanes that share t4 hold shares of the same heads' sums
            l[nh][c] += __shfl_xor_sync(0xffffffffu, l[nh][c], 4);
            l[nh][c] += __shfl_xor_sync(0xffffffffu, l[nh][c], 8);
            l[nh][c] += __shfl_xor_sync(0xffffffffu, l[nh][c], 16);
        }
    __syncthreads();                                     // every warp is done with its stages: reuse them for the merge
    float* mo = reinterpret_cast<float*>(smem);          // [warp][head][MO_PITCH]: every warp's partial output
    float* mml = mo + DEC_WARPS * 16 * MO_PITCH;         // [warp][head][2]
#pragma unroll
    for (int nh = 0; nh < NH; nh++)
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const int head = nh * 8 + t4 * 2 + c;
            float* b = mo + (warp * 16 + head) * MO_PITCH + g;
#pragma unroll
            for (int mt = 0; mt < HD / 16; mt++) {
                b[mt * 16] = o[nh][mt][c];
                b[mt * 16 + 8] = o[nh][mt][2 + c];
            }
            if (g == 0) {
                mml[(warp * 16 + head) * 2] = m[nh][c];
                mml[(warp * 16 + head) * 2 + 1] = l[nh][c];
            }
        }
    __syncthreads();
    // Merge of the CTA's warps, kept in registers until every thread has read what it needs.
    float cta_val[(16 * HD + DEC_WARPS * 32 - 1) / (DEC_WARPS * 32)];
    float cta_m = -INFINITY, cta_l = 0.0f;
    {
        int e = 0;
        for (int idx = threadIdx.x; idx < G * HD; idx += DEC_WARPS * 32, e++) {
            const int row = idx / HD, d = idx - row * HD;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; w++) M = fmaxf(M, mml[(w * 16 + row) * 2]);
            const float Ms = M == -INFINITY ? 0.0f : M;
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; w++) acc += mo[(w * 16 + row) * MO_PITCH + d] * exp2f(mml[(w * 16 + row) * 2] - Ms);
            cta_val[e] = acc;
        }
        if (threadIdx.x < G) {
            const int row = threadIdx.x;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; w++) cta_m = fmaxf(cta_m, mml[(w * 16 + row) * 2]);
            const float Ms = cta_m == -INFINITY ? 0.0f : cta_m;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; w++) cta_l += mml[(w * 16 + row) * 2 + 1] * exp2f(mml[(w * 16 + row) * 2] - Ms);
        }
    }
    IB_DT(21);
    bf16* out_row = p.out + (int64_t(t) * p.n_heads + int64_t(kvh) * G) * HD;
    if (n_splits == 1) {
        __shared__ float inv_l[16];
        if (threadIdx.x < G) inv_l[threadIdx.x] = cta_l > 0.0f ? 1.0f / cta_l : 0.0f;
        __syncthreads();
        int e = 0;
        for (int idx = threadIdx.x; idx < G * HD; idx += DEC_WARPS * 32, e++) out_row[idx] = __float2bfloat16_rn(cta_val[e] * inv_l[idx / HD]);
        return;
    }
    // The slices of the key range meet through distributed shared memory: every rank owns a share of the G * HD output
    // elements and receives the other ranks' values for them (and every rank's maximum and sum per head) into arrays
    // of its own, apart from the page ring that slower warps of the owner may still be using. One cluster barrier
    // after the pushes; the owner then adds the slices in rank order and nobody touches remote memory again, so the
    // ranks leave independently.
    __shared__ float recv_o[16 * HD];                    // [rank][share]
    __shared__ float recv_ml[MAX_SPLITS][16][2];
    cg::cluster_group cl = cg::this_cluster();
    IB_DT(22);
    const int total = G * HD, share = (total + n_splits - 1) / n_splits;
    {
        int e = 0;
        for (int idx = threadIdx.x; idx < total; idx += DEC_WARPS * 32, e++) {
            const int owner = idx / share;
            cl.map_shared_rank(recv_o, owner)[split * share + (idx - owner * share)] = cta_val[e];
        }
        if (threadIdx.x < G) {
            for (int r = 0; r < n_splits; r++) {
                float* ml = cl.map_shared_rank(&recv_ml[0][0][0], r) + (split * 16 + threadIdx.x) * 2;
                ml[0] = cta_m; ml[1] = cta_l;
            }
        }
    }
    cl.sync();
    IB_DT(23);
    const bool last_level = p.n_super == 1;
    float* ws = last_level ? nullptr : p.workspace + ((int64_t(seg) * p.n_kv + kvh) * p.n_super + blockIdx.x / n_splits) * WS_STRIDE;
    for (int j = threadIdx.x; j < share; j += DEC_WARPS * 32) {
        const int idx = split * share + j;
        if (idx >= total) break;
        const int row = idx / HD;
        float M = -INFINITY;
#pragma unroll
        for (int r = 0; r < MAX_SPLITS; r++) if (r < n_splits) M = fmaxf(M, recv_ml[r][row][0]);
        const float Ms = M == -INFINITY ? 0.0f : M;
        float acc = 0.0f, L = 0.0f;
#pragma unroll
        for (int r = 0; r < MAX_SPLITS; r++) {
            if (r < n_splits) {
                const float w = exp2f(recv_ml[r][row][0] - Ms);
                L += recv_ml[r][row][1] * w;
                acc += recv_o[r * share + j] * w;
            }
        }
        if (last_level) out_row[idx] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
        else ws[idx] = acc;                              // unnormalised, relative to this cluster's maximum of the row
    }
    IB_DT(24);
    if (last_level) return;
    // Clusters beside one another: each leaves its unnormalised share and, per head, its maximum and sum in the
    // workspace; the CTA that arrives last at the (segment, kv head) counter adds the clusters in index order (the
    // result does not depend on who is last) and leaves the counter at zero for the next launch.
    if (split == 0 && threadIdx.x < G) {
        const int row = threadIdx.x;
        float M = -INFINITY, L = 0.0f;
#pragma unroll
        for (int r = 0; r < MAX_SPLITS; r++) if (r < n_splits) M = fmaxf(M, recv_ml[r][row][0]);
        const float Ms = M == -INFINITY ? 0.0f : M;
#pragma unroll
        for (int r = 0; r < MAX_SPLITS; r++) if (r < n_splits) L += recv_ml[r][row][1] * exp2f(recv_ml[r][row][0] - Ms);
        ws[16 * HD + row * 2] = M;
        ws[16 * HD + row * 2 + 1] = L;
    }
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int* counter = p.counters + seg * p.n_kv + kvh;
        const unsigned int prev = atomicAdd(counter, 1u);
        is_last = prev == gridDim.x - 1u;
        if (is_last) *counter = 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float* all = p.workspace + (int64_t(seg) * p.n_kv + kvh) * p.n_super * WS_STRIDE;
    for (int idx = threadIdx.x; idx < total; idx += DEC_WARPS * 32) {
        const int row = idx / HD;
        const float* ml = all + 16 * HD + row * 2;
        float M = -INFINITY;
        // four clusters' values are requested together: one round trip to L2 per four clusters, not three per cluster
        for (int c0 = 0; c0 < p.n_super; c0 += 4) {
            float mm[4];
#pragma unroll
            for (int u = 0; u < 4; u++) mm[u] = c0 + u < p.n_super ? __ldcg(ml + (c0 + u) * WS_STRIDE) : -INFINITY;
#pragma unroll
            for (int u = 0; u < 4; u++) M = fmaxf(M, mm[u]);
        }
        const float Ms = M == -INFINITY ? 0.0f : M;
        float acc = 0.0f, L = 0.0f;
        for (int c0 = 0; c0 < p.n_super; c0 += 4) {
            float mm[4], ll[4], vv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const bool in = c0 + u < p.n_super;
                mm[u] = in ? __ldcg(ml + (c0 + u) * WS_STRIDE) : -INFINITY;
                ll[u] = in ? __ldcg(ml + (c0 + u) * WS_STRIDE + 1) : 0.0f;
                vv[u] = in ? __ldcg(all + (c0 + u) * WS_STRIDE + idx) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const float w = exp2f(mm[u] - Ms);
                L += ll[u] * w;
                acc += vv[u] * w;
            }
        }
        out_row[idx] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
    }
}

// ================================================================================================ prefill

__global__ void __launch_bounds__(PF_WARPS * 32)
attn_prefill_kernel(const AttnParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    ib::pdl_wait();
    // The last query tiles have the most keys to go through: they start first, for every head (heads are the fast
    // grid axis), and the short ones fill the gaps at the end.
    const int qt = gridDim.y - 1 - blockIdx.y, h = blockIdx.x, seg = blockIdx.z;
    const int t0 = p.seg_start[seg];
    const int q_len = p.seg_start[seg + 1] - t0;
    if (q_len == 1 || qt * PF_BM >= q_len) return;
    const int pos0 = p.seg_pos0[seg];
    const int kvh = h / p.group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int* table = p.block_table + int64_t(seg) * p.max_blocks;
    const int q_first = pos0 + qt * PF_BM;                                   // position of tile row 0
    const int q_last = min(pos0 + q_len - 1, q_first + PF_BM - 1);
    const int lo_key = p.window > 0 ? max(0, q_first - p.window + 1) : 0;
    const int kt0 = lo_key / PF_BN, kt1 = q_last / PF_BN;

    const uint32_t q_smem = smem_u32(smem);
    const uint32_t kv_smem = q_smem + PF_BM * ROW_BYTES;

    // Q tile: rows beyond the segment are zero.
    for (int c = threadIdx.x; c < PF_BM * CHUNKS; c += PF_WARPS * 32) {
        const int row = c / CHUNKS, col = c % CHUNKS;
        const int qi = qt * PF_BM + row;
        const bf16* src = p.q + (int64_t(t0 + min(qi, q_len - 1)) * p.n_heads + h) * HD + col * 8;
        cp_async16(q_smem + row * ROW_BYTES + col * 16, src, qi < q_len ? 16 : 0);
    }
    auto issue = [&](int kt, int stage) {
        if (kt <= kt1) {
            const uint32_t k_dst = kv_smem + stage * 2 * PF_TILE_BYTES, v_dst = k_dst + PF_TILE_BYTES;
            for (int c = threadIdx.x; c < PF_BN * CHUNKS; c += PF_WARPS * 32) {
                const int row = c / CHUNKS, col = c % CHUNKS;
                const int key = kt * PF_BN + row;
                int page = -1;
                if (key >= (lo_key / PAGE) * PAGE && key <= q_last) {
                    page = table[key / PAGE];
                    if (page < 0 || page >= p.n_pages) { atomicExch(p.status, 3); page = -1; }
                }
                const int64_t off = page < 0 ? 0 : ((int64_t(page) * p.n_kv + kvh) * PAGE + key % PAGE) * HD + col * 8;
                const int bytes = page >= 0 ? 16 : 0;
                cp_async16(k_dst + row * ROW_BYTES + col * 16, p.k_cache + off, bytes);
                cp_async16(v_dst + row * ROW_BYTES + col * 16, p.v_cache + off, bytes);
            }
        }
        cp_commit();
    };
    issue(kt0, 0);                                                            // group 0: Q and the first key tile

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    const int row_pos[2] = {q_first + warp * 16 + g, q_first + warp * 16 + g + 8};
    int row_lo[2];
#pragma unroll
    for (int hh = 0; hh < 2; hh++) row_lo[hh] = p.window > 0 ? max(0, row_pos[hh] - p.window + 1) : 0;
    const uint32_t q_warp = q_smem + (warp * 16) * ROW_BYTES;
    const int a_row = (lane & 7) + (((lane >> 3) & 1) << 3), a_k = (lane >> 4) << 3;

    for (int kt = kt0; kt <= kt1; kt++) {
        const int stage = (kt - kt0) & 1;
        issue(kt + 1, stage ^ 1);
        cp_wait<1>();
        __syncthreads();
        const uint32_t k_smem = kv_smem + stage * 2 * PF_TILE_BYTES, v_smem = k_smem + PF_TILE_BYTES;
        // Skip tiles that lie entirely above this warp's rows (causal) or entirely before their windows.
        const int warp_last = q_first + warp * 16 + 15, warp_first_lo = p.window > 0 ? max(0, q_first + warp * 16 - p.window + 1) : 0;
        if (kt * PF_BN <= warp_last && kt * PF_BN + PF_BN - 1 >= warp_first_lo) {
            float s[PF_BN / 8][4];
#pragma unroll
            for (int n = 0; n < PF_BN / 8; n++) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
            uint32_t qf[KS][4];
#pragma unroll
            for (int ks = 0; ks < KS; ks++)
                ldsm_x4(q_warp + a_row * ROW_BYTES + (ks * 16 + a_k) * 2, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
            qk_tile<PF_BN / 8>(s, qf, k_smem);
            const int key0 = kt * PF_BN;
            softmax_update<PF_BN / 8, HD / 8>(s, m, l, o, p.scale_log2, [&](int half, int key) {
                return key0 + key <= row_pos[half] && key0 + key >= row_lo[half];
            });
            pv_tile<PF_BN / 8>(o, s, v_smem);
        }
        __syncthreads();
    }
    cp_wait<0>();
    ib::pdl_launch_dependents();
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 1);
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 2);
    }
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
        const int qi = qt * PF_BM + warp * 16 + g + hh * 8;
        if (qi >= q_len) continue;
        const float inv = l[hh] > 0.0f ? 1.0f / l[hh] : 0.0f;
        bf16* dst = p.out + (int64_t(t0 + qi) * p.n_heads + h) * HD + t4 * 2;
#pragma unroll
        for (int n = 0; n < HD / 8; n++)
            *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16(o[n][hh * 2] * inv, o[n][hh * 2 + 1] * inv);
    }
}

}  // namespace

IB_EXPORT int ib_attention_head_dim() { return HD; }

#ifdef IB_ATTN_DEC_TRACE
IB_EXPORT int ib_attention_decode_trace(long long* host) {
    return cudaMemcpyFromSymbol(host, ib_dec_trace, sizeof(ib_dec_trace)) == cudaSuccess ? IB_OK : IB_ERR_CUDA;
}
#endif

namespace {

int check_common(int n_segments, int n_heads, int n_kv, int head_dim, int page_size, int n_splits, const int* status,
                 int n_super = 1, const float* workspace = nullptr, const unsigned int* counters = nullptr) {
    if (n_super < 1 || n_super > MAX_SUPER) return ib::fail(IB_ERR_ARG, "attention_fast: 1 to %d clusters per (segment, kv head), got %d", MAX_SUPER, n_super);
    if (n_super > 1 && (n_splits != MAX_SPLITS || !workspace || !counters))
        return ib::fail(IB_ERR_ARG, "attention_fast: several clusters per (segment, kv head) need 8 slices each, a workspace and counters");
    if (head_dim != HD) return ib::fail(IB_ERR_ARG, "attention_fast: built for head_dim %d, called with %d", HD, head_dim);
    if (page_size != PAGE) return ib::fail(IB_ERR_ARG, "attention_fast: pages must hold %d positions, got %d", PAGE, page_size);
    if (n_kv <= 0 || n_heads % n_kv) return ib::fail(IB_ERR_ARG, "attention_fast: heads %d not a multiple of kv heads %d", n_heads, n_kv);
    if (n_heads / n_kv > 16) return ib::fail(IB_ERR_ARG, "attention_fast: more than 16 query heads per kv head");
    if (n_heads > 65535 || n_segments > 65535) return ib::fail(IB_ERR_ARG, "attention_fast: too many heads or segments");
    if (n_splits != 1 && n_splits != 2 && n_splits != 4 && n_splits != 8) return ib::fail(IB_ERR_ARG, "attention_fast: splits must be 1, 2, 4 or 8");
    if (!status) return ib::fail(IB_ERR_ARG, "attention_fast: a status word is required");
    return IB_OK;
}

// Tensor maps of the K and V pages of one cache entry, seen as matrices [pages * kv heads * 16, HD] (boxes of one page's
// 16 rows x 64 elements). Only the head sizes whose pages arrive by tensor copy need them.
int page_maps(const void* k_cache, const void* v_cache, int64_t n_pages, int n_kv, CUtensorMap* mk, CUtensorMap* mv) {
    if (!TMA_PAGES) return IB_OK;
    if ((uintptr_t(k_cache) & 15) || (uintptr_t(v_cache) & 15)) return ib::fail(IB_ERR_ARG, "attention_fast: the cache must be 16-byte aligned");
    if (n_pages * n_kv * PAGE >= (1LL << 31)) return ib::fail(IB_ERR_ARG, "attention_fast: the cache has too many rows for a tensor map");
    int rc = ib::get_map(k_cache, n_pages * n_kv * PAGE, HD, PAGE, mk);
    if (rc) return rc;
    return ib::get_map(v_cache, n_pages * n_kv * PAGE, HD, PAGE, mv);
}

int configure() {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_decode_kernel<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_decode_kernel<true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_decode_kernel<true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
        if (e != cudaSuccess) return ib::fail(IB_ERR_CUDA, "attention_fast: cannot set shared memory size: %s", cudaGetErrorString(e));
        configured = true;
    }
    return IB_OK;
}

}  // namespace

// Attention for every segment of a step. q/out [tokens, heads*HD] bfloat16; caches [pages, kv_heads, 16, HD] bfloat16;
// seg_start [S+1], seg_pos0 [S], block_table [S, max_blocks] int32. has_decode / max_q_len tell which kernels to
// launch (a kernel skips segments of the other kind). n_splits: slices of the decode kernel's cluster, 1, 2, 4 or 8;
// n_super: clusters per (segment, kv head), more than one only with 8 slices each, a workspace of
// segments * kv_heads * n_super * (16 * HD + 32) floats and segments * kv_heads zeroed counters (left at zero).
IB_EXPORT int ib_attention_fast(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                                int max_blocks, const int* seg_start, const int* seg_pos0, int n_segments, int n_heads,
                                int n_kv, int head_dim, int page_size, int window, float scale, int64_t n_pages,
                                int has_decode, int max_q_len, int n_splits, int* status, cudaStream_t stream,
                                int n_super, float* workspace, unsigned int* counters) {
    if (n_segments <= 0) return IB_OK;
    int rc = check_common(n_segments, n_heads, n_kv, head_dim, page_size, n_splits, status, n_super, workspace, counters);
    if (rc) return rc;
    AttnParams p = {};
    p.q = (const bf16*)q; p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache; p.out = (bf16*)out;
    p.block_table = block_table; p.max_blocks = max_blocks; p.seg_start = seg_start; p.seg_pos0 = seg_pos0;
    p.n_heads = n_heads; p.n_kv = n_kv; p.group = n_heads / n_kv; p.window = window;
    p.scale_log2 = scale * LOG2E; p.n_pages = n_pages; p.n_splits = n_splits; p.status = status;
    p.n_super = n_super; p.workspace = workspace; p.counters = counters;
    if ((rc = configure())) return rc;
    if (has_decode) {
        CUtensorMap mk = {}, mv = {};
        if ((rc = page_maps(k_cache, v_cache, n_pages, n_kv, &mk, &mv))) return rc;
        const dim3 grid{unsigned(n_splits * n_super), unsigned(n_kv), unsigned(n_segments)};
        // the heads of a group are the columns of one MMA tile (up to 8) or of two (up to 16)
        rc = ib::launch("attention_fast (decode)", p.group <= 8 ? attn_decode_kernel<false, 1> : attn_decode_kernel<false, 2>, grid,
                        dim3(DEC_WARPS * 32), size_t(DEC_SMEM), stream, unsigned(n_splits), mk, mv, p);
        if (rc) return rc;
    }
    if (max_q_len > 1) {
        if ((max_q_len + PF_BM - 1) / PF_BM > 65535) return ib::fail(IB_ERR_ARG, "attention_fast: a segment of %lld tokens has too many query tiles", (long long)max_q_len);
        const dim3 grid{unsigned(n_heads), unsigned((max_q_len + PF_BM - 1) / PF_BM), unsigned(n_segments)};
        return ib::launch("attention_fast (prefill)", attn_prefill_kernel, grid, dim3(PF_WARPS * 32), size_t(PF_SMEM), stream, 1u, p);
    }
    return IB_OK;
}

// Decode-only steps (every segment one token): rotation of q and k, the cache write of the new position and the
// attention in one launch. qkv [tokens, (heads + 2 kv_heads) * HD] bfloat16 packed [q | k | v] rows with the bias
// already added; cos/sin float [positions, HD/2]; caches are written (write_cache != 0) and read. HD/2 must be a
// multiple of 16.
IB_EXPORT int ib_attention_decode_fused(const void* qkv, const float* cos_t, const float* sin_t, void* k_cache, void* v_cache,
                                        void* out, const int* block_table, int max_blocks, const int* seg_start,
                                        const int* seg_pos0, int n_segments, int n_heads, int n_kv, int head_dim,
                                        int page_size, int window, float scale, int64_t n_pages, int write_cache,
                                        int n_splits, int* status, const void* prefetch, int64_t prefetch_bytes,
                                        cudaStream_t stream, int n_super, float* workspace, unsigned int* counters) {
    if (n_segments <= 0) return IB_OK;
    int rc = check_common(n_segments, n_heads, n_kv, head_dim, page_size, n_splits, status, n_super, workspace, counters);
    if (rc) return rc;
    if ((HD / 2) % 16) return ib::fail(IB_ERR_ARG, "attention_decode_fused: head_dim/2 must be a multiple of 16, head_dim is %d", HD);
    if (!cos_t || !sin_t) return ib::fail(IB_ERR_ARG, "attention_decode_fused: rotation tables are required");
    AttnParams p = {};
    p.qkv = (const bf16*)qkv; p.cos = cos_t; p.sin = sin_t; p.write_cache = write_cache ? 1 : 0;
    p.prefetch = prefetch; p.prefetch_bytes = prefetch_bytes & ~int64_t(15);
    p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache; p.k_cache_w = (bf16*)k_cache; p.v_cache_w = (bf16*)v_cache;
    p.out = (bf16*)out;
    p.block_table = block_table; p.max_blocks = max_blocks; p.seg_start = seg_start; p.seg_pos0 = seg_pos0;
    p.n_heads = n_heads; p.n_kv = n_kv; p.group = n_heads / n_kv; p.window = window;
    p.scale_log2 = scale * LOG2E; p.n_pages = n_pages; p.n_splits = n_splits; p.status = status;
    p.n_super = n_super; p.workspace = workspace; p.counters = counters;
    if ((rc = configure())) return rc;
    CUtensorMap mk = {}, mv = {};
    if ((rc = page_maps(k_cache, v_cache, n_pages, n_kv, &mk, &mv))) return rc;
    const dim3 grid{unsigned(n_splits * n_super), unsigned(n_kv), unsigned(n_segments)};
    return ib::launch("attention_decode_fused", p.group <= 8 ? attn_decode_kernel<true, 1> : attn_decode_kernel<true, 2>, grid,
                      dim3(DEC_WARPS * 32), size_t(DEC_SMEM), stream, unsigned(n_splits), mk, mv, p);
}
