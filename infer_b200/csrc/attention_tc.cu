// Causal / windowed attention of prompt portions over the paged bfloat16 cache on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory, operands brought in by TMA). Compiled for one head size:
// -DIB_HEAD_DIM=64 or 128. Pages hold 16 positions; a (page, kv head) block of the cache is 16 rows of head_dim.
//
// One CTA (192 threads) serves 128 consecutive queries of one head of one segment and walks over its keys in tiles
// of 128 (8 pages), aligned to absolute multiples of 128:
//   warp 0      lane i issues the TMA loads of page i of a tile (a box of 16 positions x 64 elements per page and half
//               of the head), each into its place of a 128-byte-swizzled operand tile; the page ids of the CTA's key
//               range sit in shared memory. K and V tiles are double-buffered: tile j + 2 is requested as soon as the
//               MMA that read tile j has finished;
//   warp 1      allocates tensor memory; one lane issues S(j) = Q K(j)^T (M=128 queries, N=128 keys, K over the head)
//               two tiles ahead into one of two S buffers, and, when the probabilities of tile j are in shared memory,
//               O += P(j) V(j) (N = head size, K = 128 keys; V is the operand whose contiguous dimension is N,
//               "MN-major": it is used as the cache stores it);
//   warps 2-5   thread r owns query row r: reads its row of S from tensor memory, masks on the diagonal and at the
//               window's edge (select, never arithmetic: unwritten cache rows may hold anything), keeps the running
//               maximum and sum in float, writes bfloat16 probabilities into the swizzled P tile, and at the end
//               divides its row of O. The scale goes into the exponent's multiply-add; exponentials are ex2.approx.
// O stays in tensor memory over all key tiles. Its rows refer to a maximum that is only raised when the true running
// maximum has moved by more than 8 (a factor 256) since: then the row of O is read, scaled and written back
// (tcgen05.ld / tcgen05.st) before the next P V is issued. Probabilities therefore stay below 256, exact in float
// sums. V rows of positions that this step has not written (beyond the segment's last token, or in pages the table
// does not hold) are zeroed in shared memory before P V, so stale cache contents cannot reach a sum.
//
// Where few long query tiles would leave SMs idle (a portion of a prompt behind a long context), the key tiles of a
// query tile are shared among up to four CTAs: each leaves its unnormalised rows of O, their reference maxima and sums
// in a workspace, and the one that arrives last at the tile's counter adds the parts in index order and writes the
// output (the host shares only while all CTAs still run at once: a CTA's start and end cost about three key tiles).
//
// One CTA per SM (193 KB of shared memory, all 512 tensor-memory columns). Query tiles start heaviest first. Measured
// at 2,048 tokens, 12/2 heads of 128: 38 us against 88 us for the mma.sync kernel. A key tile takes about 3,700 cycles,
// the softmax thread's own sequence (wait for S, read it, maximum, 128 exponentials, wait for the previous P V, store P):
// neither two threads per row nor a second MMA-issuing thread shortened it.
// Every mbarrier wait is bounded; one that runs out raises the status word, and the CTA drains its copies,
// frees its tensor memory and returns.
#include <algorithm>

#include "common.cuh"
#include "tma_map.cuh"

IB_DEFINE_LAST_ERROR()

#ifndef IB_HEAD_DIM
#define IB_HEAD_DIM 128
#endif

namespace {

using bf16 = __nv_bfloat16;
constexpr int HD = IB_HEAD_DIM;
static_assert(HD == 64 || HD == 128, "the tensor-memory attention kernel takes head sizes 64 and 128");
constexpr int DB = HD / 64;                 // 64-element (128-byte) blocks of the head dimension
constexpr int PAGE = 16;
#ifndef IB_ATTN_BN
#define IB_ATTN_BN 128
#endif
constexpr int BM = 128, BN = IB_ATTN_BN;    // queries per CTA, keys per tile (64 or 128)
static_assert(BN == 64 || BN == 128, "key tiles of 64 or 128");
constexpr int PB = BN / 64;                 // 64-key (128-byte) blocks of a row of P
constexpr int PAGES_PER_TILE = BN / PAGE;
constexpr int NUM_THREADS = 192;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;        // O's reference maximum follows the running maximum in steps of this (log2)
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr int STATUS_TIMEOUT = 106, STATUS_BAD_PAGE = 3;
constexpr int TAB_MAX = 2048;               // page ids kept in shared memory: 32,768 positions

constexpr int Q_BYTES = DB * BM * 128, K_BYTES = DB * BN * 128, V_BYTES = DB * BN * 128, P_BYTES = PB * BM * 128;
constexpr int SMEM_BYTES = Q_BYTES + 2 * K_BYTES + 2 * V_BYTES + P_BYTES + 1024 /*alignment*/ + 128 /*barriers*/;
constexpr int TMEM_COLS = (2 * BN + HD) > 256 ? 512 : ((2 * BN + HD) > 128 ? 256 : 128);
constexpr int S_COL = 0, O_COL = 2 * BN;    // two S tiles of BN columns each, then O's HD columns

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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; i++) {
        if (mbar_test(bar, parity)) return true;
        if (i > 1024) __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
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
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
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
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void softmax_barrier() {         // the four softmax warps (threads 64..191) among themselves
    asm volatile("bar.sync 1, 128;" ::: "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {        // ex2.approx: 2^-inf = 0, about 2 ulp
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory descriptor of a 128-byte-swizzled operand tile (descriptor version 1, layout type 2).
// K-major (rows of 128 bytes along the reduction, groups of 8 rows 1024 bytes apart): lbo unused, sbo = 1024.
// MN-major (rows of 128 bytes along N, one row per reduction index): sbo = 1024 between groups of 8 reduction rows,
// lbo = distance between blocks of 64 elements of N.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= uint64_t((smem_addr & 0x3FFFF) >> 4);
    d |= uint64_t((lbo >> 4) & 0x3FFF) << 16;
    d |= uint64_t((sbo >> 4) & 0x3FFF) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(2) << 61;
    return d;
}
// kind::f16 instruction descriptor: D float, A and B bfloat16, A K-major; b_mn selects an MN-major B; M = 128.
__host__ __device__ constexpr uint32_t make_idesc(int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | (uint32_t(n >> 3) << 17) | (uint32_t(BM >> 4) << 24);
}

#ifdef IB_ATTN_TRACE
// Profiling build (-DIB_ATTN_TRACE): the first CTA's first softmax thread and its MMA thread record the SM clock per
// key tile: 0 tile entered, 1 S arrived, 2 S read, 3 maximum known, 4 probabilities computed, 5 P handed over;
// 6 Q K^T issued, 7 P V issued. ib_attention_tc_trace copies the marks to the host.
__device__ long long ib_attn_trace[64][8];
#define IB_T(j, k) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x == 64 || threadIdx.x == 32) && (j) < 64) ib_attn_trace[j][k] = clock64(); } while (0)
#else
#define IB_T(j, k) do {} while (0)
#endif

struct Params {
    bf16* out;                              // [tokens, heads * HD]
    const int* block_table; int max_blocks;
    const int* seg_start; const int* seg_pos0;
    int n_heads, n_kv, group, window;
    float scale_log2;
    int64_t n_pages;
    int* status;
    // A query tile's key tiles are shared among up to `split` CTAs (blockIdx.y = query tile x split + part), each with
    // at least PART_MIN_TILES of them: a part leaves its rows of O (unnormalised), their reference maxima and sums in
    // the workspace, and the part that arrives last at the tile's counter adds all parts in index order, divides and
    // writes the output. Few long query tiles (a prompt on few heads, a portion behind a long context) fill the SMs
    // that way, and the heaviest tile of a causal prompt no longer sets the kernel's time alone.
    int early_release;                       // 1: the successor is released at the kernel's start (few CTAs: a short kernel)
    int split;
    float* workspace;                        // [segments of two or more tokens][heads][query tiles][split][PART_FLOATS]
    unsigned int* counters;                  // [segments of two or more tokens][heads][query tiles], zero between launches
};
constexpr int MAX_SPLIT = 4;
constexpr int PART_MIN_TILES = 4;
constexpr int PART_FLOATS = BM * HD + 2 * BM;   // O as [HD][BM] (a warp's rows side by side), then the maxima, then the sums

__global__ void __launch_bounds__(NUM_THREADS)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t q_s = base, k_s = q_s + Q_BYTES, v_s = k_s + 2 * K_BYTES, p_s = v_s + 2 * V_BYTES, bars = p_s + P_BYTES;
    uint8_t* v_ptr = base_ptr + Q_BYTES + 2 * K_BYTES;
    uint8_t* p_ptr = v_ptr + 2 * V_BYTES;
    volatile uint32_t* slots = reinterpret_cast<volatile uint32_t*>(p_ptr + P_BYTES + 112);  // [0] TMEM base, [1] abort
    // k_full, k_empty, v_full, v_empty and s_full come in pairs (two K and two V tiles in shared memory, two S tiles in
    // tensor memory): tile j uses member j & 1, for the (j >> 1)-th time
    const uint32_t q_full = bars, k_full = bars + 8, k_empty = bars + 24, s_full = bars + 40, v_full = bars + 56,
                   v_empty = bars + 72, p_full = bars + 88, o_full = bars + 96;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // The last query tiles have the most keys: they start first, for every head.
    const int n_qt = gridDim.y / p.split;
    const int h = blockIdx.x, qt = n_qt - 1 - int(blockIdx.y) / p.split, part = int(blockIdx.y) % p.split, seg = blockIdx.z;
    const int t0 = p.seg_start[seg];
    const int q_len = p.seg_start[seg + 1] - t0;
    if (q_len <= 1 || qt * BM >= q_len) return;          // one-token segments belong to the decode kernel
    const int pos0 = p.seg_pos0[seg];
    const int kvh = h / p.group;
    const int q_first = pos0 + qt * BM;
    const int last_written = pos0 + q_len - 1;           // the last position whose k and v exist
    const int q_last = min(last_written, q_first + BM - 1);
    const int lo_key = p.window > 0 ? max(0, q_first - p.window + 1) : 0;
    // this CTA's key tiles: all of the query tile's, or one of `n_parts` contiguous shares
    const int all0 = lo_key / BN, all1 = q_last / BN;
    const int n_all = all1 - all0 + 1;
    const int n_parts = max(1, min(p.split, n_all / PART_MIN_TILES));
    if (part >= n_parts) return;
    const int kt0 = all0 + (n_all * part) / n_parts, kt1 = all0 + (n_all * (part + 1)) / n_parts - 1;
    const int n_tiles = kt1 - kt0 + 1;                   // >= PART_MIN_TILES when the tile is shared, >= 1 otherwise
    // Scratch is laid out over the segments that have two or more tokens only (a step may carry dozens of one-token
    // segments beside one portion): this segment's rank among those, counted from the segment table.
    int tile_id = 0;
    if (n_parts > 1) {
        int before = 0;
        for (int s2 = 0; s2 < seg; s2++) before += (p.seg_start[s2 + 1] - p.seg_start[s2] > 1) ? 1 : 0;
        tile_id = (before * p.n_heads + h) * n_qt + qt;
    }
    const int* table = p.block_table + int64_t(seg) * p.max_blocks;
    // The page ids of this CTA's key range, checked, in shared memory (a read of the table in global memory costs the
    // producer a round trip to L2 per page otherwise); ranges longer than the array fall back to the table itself.
    __shared__ int page_tab[TAB_MAX];
    const int tab0 = kt0 * PAGES_PER_TILE, tab_n = (kt1 + 1) * PAGES_PER_TILE - tab0;
    const bool tab_ok = tab_n <= TAB_MAX;
    if (tab_ok) {
        for (int i = threadIdx.x; i < tab_n; i += NUM_THREADS) {
            const int idx = tab0 + i;
            const int page = idx < p.max_blocks ? table[idx] : -1;
            page_tab[i] = (page < 0 || page >= p.n_pages) ? -1 : page;
        }
    }
    auto page_of = [&](int key) -> int {                 // page id of the page that holds `key`, or -1
        const int idx = key / PAGE;
        if (tab_ok) return page_tab[idx - tab0];
        if (idx >= p.max_blocks) return -1;
        const int page = table[idx];
        return (page < 0 || page >= p.n_pages) ? -1 : page;
    };

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int b = 0; b < 2; b++) {
            mbar_init(k_full + 8 * b, 1); mbar_init(k_empty + 8 * b, 1); mbar_init(s_full + 8 * b, 1);
            mbar_init(v_full + 8 * b, 1); mbar_init(v_empty + 8 * b, 1);
        }
        mbar_init(p_full, 4); mbar_init(o_full, 1);
        slots[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(&slots[0])), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = slots[0];
    if (p.early_release) ib::pdl_launch_dependents();    // (pays for short kernels only: see the GEMM's note)
    ib::pdl_wait();                                      // q and this step's cache rows come from the predecessor

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (lane i copies page i of a tile)
        if (lane == 0) {
            mbar_expect_tx(q_full, Q_BYTES);
            for (int db = 0; db < DB; db++) tma_load_2d(q_s + db * (BM * 128), &tm_q, q_full, h * HD + db * 64, t0 + qt * BM);
        }
        int pend_k[2] = {-1, -1}, pend_v[2] = {-1, -1};  // tiles whose copies were issued into each buffer last
        // Loads the K (which = 0) or V (which = 1) pages of tile j. Pages that hold nothing this step may read are
        // skipped (their rows are masked, and zeroed for V).
        auto load_tile = [&](int j, int which) {
            const int key0 = (kt0 + j) * BN;
            const uint32_t full = (which ? v_full : k_full) + 8 * (j & 1);
            const uint32_t dst0 = which ? v_s + (j & 1) * V_BYTES : k_s + (j & 1) * K_BYTES;
            int page = -1;
            if (lane < PAGES_PER_TILE) {
                const int key = key0 + lane * PAGE;
                page = key <= last_written ? page_of(key) : -1;
                if (key <= last_written && key + PAGE - 1 >= lo_key && page < 0) atomicExch(p.status, STATUS_BAD_PAGE);
            }
            const int valid = __popc(__ballot_sync(0xffffffffu, page >= 0));
            if (lane == 0) {
                if (valid == 0) mbar_arrive(full);
                else mbar_expect_tx(full, uint32_t(valid) * DB * (PAGE * 128));
            }
            __syncwarp();
            if (page >= 0) {
                const int row = (page * p.n_kv + kvh) * PAGE;
                for (int db = 0; db < DB; db++)
                    tma_load_2d(dst0 + db * (BN * 128) + lane * (PAGE * 128), which ? &tm_v : &tm_k, full, db * 64, row);
            }
            if (valid > 0) { if (which) pend_v[j & 1] = j; else pend_k[j & 1] = j; }
        };
        auto wait_all = [&](uint32_t bar, uint32_t parity) -> bool {      // lane 0 waits, every lane learns the outcome
            int got = 1;
            if (lane == 0) got = mbar_wait(bar, parity) ? 1 : 0;
            return __shfl_sync(0xffffffffu, got, 0) != 0;
        };
        load_tile(0, 0);
        load_tile(0, 1);
        if (n_tiles > 1) { load_tile(1, 0); load_tile(1, 1); }
        bool failed = false;
        for (int j = 0; j < n_tiles && !failed; j++) {
            if (__shfl_sync(0xffffffffu, int(slots[1]), 0)) { failed = true; break; }
            if (j + 2 < n_tiles) {                       // S(j) is complete: its K buffer takes tile j + 2
                if (!wait_all(k_empty + 8 * (j & 1), (j >> 1) & 1)) { failed = true; break; }
                load_tile(j + 2, 0);
            }
            if (j + 2 < n_tiles) {                       // P(j) V(j) is complete: its V buffer takes tile j + 2
                if (!wait_all(v_empty + 8 * (j & 1), (j >> 1) & 1)) { failed = true; break; }
                load_tile(j + 2, 1);
            }
        }
        if (failed && lane == 0) {
            if (!slots[1]) { atomicExch(p.status, STATUS_TIMEOUT); slots[1] = 1; }
            // Drain: wait (bounded) for the copies that may still be on their way, so that none lands after the CTA is gone.
            mbar_wait(q_full, 0);
            for (int b = 0; b < 2; b++) {
                if (pend_k[b] >= 0) mbar_wait(k_full + 8 * b, (pend_k[b] >> 1) & 1);
                if (pend_v[b] >= 0) mbar_wait(v_full + 8 * b, (pend_v[b] >> 1) & 1);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(BN, false), idesc_o = make_idesc(HD, true);
            const uint32_t o_tmem = tmem_base + O_COL;
            // S(j) = Q K(j)^T into S buffer j & 1
            auto issue_qk = [&](int j) -> bool {
                if (!mbar_wait(k_full + 8 * (j & 1), (j >> 1) & 1)) return false;
                tc_fence_after();
                const uint32_t s_tmem = tmem_base + S_COL + (j & 1) * BN, kb = k_s + (j & 1) * K_BYTES;
#pragma unroll
                for (int db = 0; db < DB; db++) {
                    const uint64_t qd = make_desc(q_s + db * (BM * 128), 16, 1024), kd = make_desc(kb + db * (BN * 128), 16, 1024);
#pragma unroll
                    for (int k = 0; k < 4; k++)          // 16 elements of the head per step = 32 bytes = 2 address units
                        umma_f16(s_tmem, qd + uint64_t(2 * k), kd + uint64_t(2 * k), idesc_s, (db > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(s_full + 8 * (j & 1));
                umma_commit(k_empty + 8 * (j & 1));
                IB_T(j, 6);
                return true;
            };
            bool ok = mbar_wait(q_full, 0) && issue_qk(0) && (n_tiles < 2 || issue_qk(1));
            for (int j = 0; j < n_tiles && ok && !slots[1]; j++) {
                ok = mbar_wait(p_full, j & 1) && mbar_wait(v_full + 8 * (j & 1), (j >> 1) & 1);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < BN / 16; k++) {      // 16 keys per step: 32 bytes along P's rows, 2 groups of 8 rows of V
                    const uint64_t pd = make_desc(p_s + (k / 4) * (BM * 128), 16, 1024) + uint64_t(2 * (k % 4));
                    const uint64_t vd = make_desc(v_s + (j & 1) * V_BYTES + k * (16 * 128), BN * 128, 1024);
                    umma_f16(o_tmem, pd, vd, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(o_full);
                umma_commit(v_empty + 8 * (j & 1));
                IB_T(j, 7);
                // the softmax threads have read S(j) (they wrote P(j) from it): its buffer takes S(j + 2)
                if (j + 2 < n_tiles) ok = issue_qk(j + 2);
            }
            if (!ok) { atomicExch(p.status, STATUS_TIMEOUT); slots[1] = 1; }
        }
    } else {
        // ---------------------------------------------------------------- softmax and epilogue (warps 2..5)
        const int quad = warp & 3;
        const int r = quad * 32 + lane;                  // query row of the tile = TMEM lane
        const uint32_t lane_addr = tmem_base + (uint32_t(quad * 32) << 16);
        const int row_pos = q_first + r;
        const int row_lo = p.window > 0 ? max(0, row_pos - p.window + 1) : 0;
        float m_ref = -INFINITY, l = 0.0f;               // reference maximum of this row's O and P; sum of probabilities
        bool ok = true;
        for (int j = 0; j < n_tiles; j++) {
            const int key0 = (kt0 + j) * BN;
            IB_T(j, 0);
            ok = !slots[1] && mbar_wait(s_full + 8 * (j & 1), (j >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            IB_T(j, 1);
            float s[BN];
#pragma unroll
            for (int c = 0; c < BN; c += 16) tmem_ld16(lane_addr + S_COL + (j & 1) * BN + c, reinterpret_cast<uint32_t*>(s + c));
            tmem_ld_wait();
            IB_T(j, 2);
            const bool full_tile = key0 + BN - 1 <= q_first && key0 >= (p.window > 0 ? max(0, q_first + BM - 1 - p.window + 1) : 0);
            // Raw scores: the scale goes into the exponent's multiply-add below. Most tiles lie wholly below the diagonal
            // and inside the window and need no mask. (Masks are written without short-circuit operators: a branch per
            // element costs more than the arithmetic.)
            float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            const float scale_log2 = p.scale_log2;       // > 0
            if (full_tile) {
#pragma unroll
                for (int c = 0; c < BN; c++) mxs[c & 3] = fmaxf(mxs[c & 3], s[c]);
            } else {
                const int hi = row_pos - key0, lo = row_lo - key0;       // visible: lo <= c <= hi
#pragma unroll
                for (int c = 0; c < BN; c++) {
                    const bool vis = (c <= hi) & (c >= lo);
                    s[c] = vis ? s[c] : -INFINITY;
                    mxs[c & 3] = fmaxf(mxs[c & 3], s[c]);
                }
            }
            const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])) * scale_log2;
            // O and the probabilities refer to m_ref, which follows the running maximum in steps
            const bool raise = mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
            const float alpha = raise ? fast_exp2(m_ref - mx) : 1.0f;   // m_ref = -inf gives 0: nothing was summed yet
            if (raise) { m_ref = mx; l *= alpha; }
            IB_T(j, 3);
            // with no visible key so far every score is -inf: subtracting 0 instead of -inf keeps exp2 at 0, not NaN
            const float m_neg = m_ref == -INFINITY ? 0.0f : -m_ref;
            float sums[2] = {0.0f, 0.0f};
            uint32_t pk[BN / 2];                         // the row of P, packed
#pragma unroll
            for (int c = 0; c < BN; c += 2) {
                const float a = fast_exp2(fmaf(s[c], scale_log2, m_neg)), b = fast_exp2(fmaf(s[c + 1], scale_log2, m_neg));
                __nv_bfloat162 two = __floats2bfloat162_rn(a, b);
                pk[c / 2] = *reinterpret_cast<uint32_t*>(&two);
                sums[(c >> 1) & 1] += a + b;
            }
            l += sums[0] + sums[1];
            IB_T(j, 4);
            if (j > 0) {
                // P(j-1) V(j-1) must be complete before P is overwritten and before O is touched
                ok = mbar_wait(o_full, (j - 1) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (__any_sync(0xffffffffu, raise)) {
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < HD; c += 16) {
                        uint32_t o[16];
                        tmem_ld16(lane_addr + O_COL + c, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 16; e++) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                        tmem_st16(lane_addr + O_COL + c, o);
                    }
                    tmem_st_wait();
                }
            }
            uint8_t* prow0 = p_ptr + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
            for (int c8 = 0; c8 < BN / 8; c8++) {
                uint8_t* prow = prow0 + (c8 >> 3) * (BM * 128);
                *reinterpret_cast<uint4*>(prow + (((c8 & 7) ^ (r & 7)) << 4)) = make_uint4(pk[c8 * 4], pk[c8 * 4 + 1], pk[c8 * 4 + 2], pk[c8 * 4 + 3]);
            }
            // Rows of V that hold nothing this step may read (positions after the segment's last token, pages the table
            // does not hold) become zeros, so that 0 x garbage cannot make a NaN.
            if (key0 + BN - 1 > last_written || key0 < lo_key) {
                ok = mbar_wait(v_full + 8 * (j & 1), (j >> 1) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                for (int u = r; u < BN * DB; u += BM) {
                    const int key_row = u % BN, db = u / BN;
                    const int key = key0 + key_row;
                    if (key > last_written || page_of(key) < 0) {
                        uint4* line = reinterpret_cast<uint4*>(v_ptr + (j & 1) * V_BYTES + db * (BN * 128) + key_row * 128);
#pragma unroll
                        for (int e = 0; e < 8; e++) line[e] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            }
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
            IB_T(j, 5);
        }
        if (ok) {
            ok = mbar_wait(o_full, (n_tiles - 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (!ok && !slots[1]) { atomicExch(p.status, STATUS_TIMEOUT); slots[1] = 1; }
        const int qi = qt * BM + r;
        bf16* dst = p.out + (int64_t(t0 + qi) * p.n_heads + h) * HD;
        auto store16 = [&](int c, const float* v) {      // 16 outputs of this row from column c on
            uint32_t w[8];
#pragma unroll
            for (int e = 0; e < 8; e++) {
                __nv_bfloat162 two = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
                w[e] = *reinterpret_cast<uint32_t*>(&two);
            }
            *reinterpret_cast<uint4*>(dst + c) = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4*>(dst + c + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        };
        if (n_parts == 1) {
            if (ok) {
                tc_fence_after();
                const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll 1
                for (int c = 0; c < HD; c += 16) {
                    uint32_t o[16];
                    tmem_ld16(lane_addr + O_COL + c, o);
                    tmem_ld_wait();
                    float v[16];
#pragma unroll
                    for (int e = 0; e < 16; e++) v[e] = __uint_as_float(o[e]) * inv;
                    if (qi < q_len) store16(c, v);
                }
            }
        } else {
            // Every softmax warp goes through both barriers whatever happened to it, so that a failed wait in one warp
            // (the status word is raised then) cannot leave the others waiting; the counter is always brought back to 0.
            float* parts = p.workspace + int64_t(tile_id) * p.split * PART_FLOATS;
            float* mine = parts + part * PART_FLOATS;
            if (ok) {
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < HD; c += 16) {
                    uint32_t o[16];
                    tmem_ld16(lane_addr + O_COL + c, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 16; e++) __stcg(mine + (c + e) * BM + r, __uint_as_float(o[e]));
                }
                __stcg(mine + HD * BM + r, m_ref);
                __stcg(mine + HD * BM + BM + r, l);
            }
            __threadfence();
            softmax_barrier();
            if (threadIdx.x == 64) slots[2] = atomicAdd(p.counters + tile_id, 1u);
            softmax_barrier();
            if (slots[2] == uint32_t(n_parts - 1)) {     // all parts of this query tile are in the workspace
                __threadfence();
                if (threadIdx.x == 64) p.counters[tile_id] = 0u;
                float m = -INFINITY;
#pragma unroll
                for (int i = 0; i < MAX_SPLIT; i++)
                    if (i < n_parts) m = fmaxf(m, __ldcg(parts + i * PART_FLOATS + HD * BM + r));
                float f[MAX_SPLIT], l_all = 0.0f;
#pragma unroll
                for (int i = 0; i < MAX_SPLIT; i++) {
                    f[i] = 0.0f;
                    if (i < n_parts) {
                        const float mi = __ldcg(parts + i * PART_FLOATS + HD * BM + r);
                        f[i] = mi == -INFINITY ? 0.0f : fast_exp2(mi - m);       // a part with no visible key adds nothing
                        l_all += __ldcg(parts + i * PART_FLOATS + HD * BM + BM + r) * f[i];
                    }
                }
                const float inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
#pragma unroll
                for (int i = 0; i < MAX_SPLIT; i++) f[i] *= inv;
#pragma unroll 1
                for (int c = 0; c < HD; c += 16) {
                    float v[16];
#pragma unroll
                    for (int e = 0; e < 16; e++) v[e] = 0.0f;
#pragma unroll
                    for (int i = 0; i < MAX_SPLIT; i++) {
                        if (i < n_parts) {
#pragma unroll
                            for (int e = 0; e < 16; e++) v[e] = fmaf(__ldcg(parts + i * PART_FLOATS + (c + e) * BM + r), f[i], v[e]);
                        }
                    }
                    if (qi < q_len) store16(c, v);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace

IB_EXPORT int ib_attention_tc_head_dim() { return HD; }

// Attention of the segments with two or more tokens (one-token segments are skipped: the decode kernel serves them).
// q, out: bfloat16 [tokens, heads * HD]; caches bfloat16 [pages, kv heads, 16, HD] holding this step's keys and values
// already; block_table int32 [segments, max_blocks]; seg_start int32 [segments + 1]; seg_pos0 int32 [segments].
// split: up to how many CTAs share the key tiles of one query tile (1: none); it is lowered to what the workspace
// (floats) and the counters (zero before and after) have room for: one slot per segment of two or more tokens
// (n_long_segments of them; 0: assume all), head and query tile.
IB_EXPORT int ib_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                                      int max_blocks, const int* seg_start, const int* seg_pos0, int n_segments, int64_t n_tokens,
                                      int n_heads, int n_kv, int head_dim, int page_size, int window, float scale, int64_t n_pages,
                                      int max_q_len, int* status, cudaStream_t stream, int split, float* workspace,
                                      int64_t workspace_floats, unsigned int* counters, int64_t n_counters, int n_long_segments) {
    if (n_segments <= 0 || max_q_len <= 1) return IB_OK;
    if (head_dim != HD) return ib::fail(IB_ERR_ARG, "attention_tc: built for head_dim %d, called with %d", HD, head_dim);
    if (page_size != PAGE) return ib::fail(IB_ERR_ARG, "attention_tc: pages must hold %d positions, got %d", PAGE, page_size);
    if (n_kv <= 0 || n_heads % n_kv) return ib::fail(IB_ERR_ARG, "attention_tc: heads %d not a multiple of kv heads %d", n_heads, n_kv);
    if (n_heads > 65535 || n_segments > 65535 || (max_q_len + BM - 1) / BM > 65535) return ib::fail(IB_ERR_ARG, "attention_tc: too many heads, segments or query tiles");
    if (!status) return ib::fail(IB_ERR_ARG, "attention_tc: a status word is required");
    if ((uintptr_t(q) | uintptr_t(k_cache) | uintptr_t(v_cache) | uintptr_t(out)) & 15) return ib::fail(IB_ERR_ARG, "attention_tc: buffers must be 16-byte aligned");
    if (n_pages * n_kv * PAGE >= (1LL << 31) || n_tokens >= (1LL << 31)) return ib::fail(IB_ERR_ARG, "attention_tc: the cache or the step is too large for 32-bit tile coordinates");
    CUtensorMap mq, mk, mv;
    int rc = ib::get_map(q, n_tokens, int64_t(n_heads) * HD, BM, &mq);
    if (rc) return rc;
    rc = ib::get_map(k_cache, n_pages * n_kv * PAGE, HD, PAGE, &mk);
    if (rc) return rc;
    rc = ib::get_map(v_cache, n_pages * n_kv * PAGE, HD, PAGE, &mv);
    if (rc) return rc;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return ib::fail(IB_ERR_CUDA, "attention_tc: cannot set shared memory size: %s", cudaGetErrorString(e));
        configured = true;
    }
    Params p = {};
    p.out = (bf16*)out; p.block_table = block_table; p.max_blocks = max_blocks; p.seg_start = seg_start; p.seg_pos0 = seg_pos0;
    p.n_heads = n_heads; p.n_kv = n_kv; p.group = n_heads / n_kv; p.window = window; p.scale_log2 = scale * LOG2E;
    p.n_pages = n_pages; p.status = status;
    // Sharing query tiles needs scratch for every (segment, head, query tile); with less than that, fewer parts.
    if (n_long_segments <= 0 || n_long_segments > n_segments) n_long_segments = n_segments;
    const int64_t n_qt = (max_q_len + BM - 1) / BM, tiles = int64_t(n_long_segments) * n_heads * n_qt;
    split = std::max(1, std::min(split, MAX_SPLIT));
    if (!workspace || !counters || tiles > n_counters) split = 1;
    while (split > 1 && tiles * split * PART_FLOATS > workspace_floats) split--;
    if (n_qt * split > 65535) split = 1;
    p.split = split; p.workspace = workspace; p.counters = counters;
    p.early_release = int64_t(n_segments) * n_heads * n_qt * split <= 296 ? 1 : 0;
    const dim3 grid{unsigned(n_heads), unsigned(n_qt * split), unsigned(n_segments)};
    return ib::launch("attention_tc", attn_prefill_tc_kernel, grid, dim3(NUM_THREADS), size_t(SMEM_BYTES), stream, 1u, mq, mk, mv, p);
}

#ifdef IB_ATTN_TRACE
IB_EXPORT int ib_attention_tc_trace(long long* host) {
    return cudaMemcpyFromSymbol(host, ib_attn_trace, sizeof(ib_attn_trace)) == cudaSuccess ? IB_OK : IB_ERR_CUDA;
}
#endif
