// Skinny matrix product for decode steps: out[M, N] = x[M, K] . w[N, K]^T with M <= 16 tokens.
//
// The weights are read exactly once, straight from global memory into registers with 16-byte loads, and used as
// the 16-row operand of mma.sync m16n8k16 (bfloat16 in, float accumulation); the tokens are the 8-wide operand.
// The kernel is bound by HBM bandwidth, so the tensor-core shape only has to keep the instruction count low.
//
// Work split. A tile is 16 output features. A thread-block cluster of CL CTAs (1, 2, 4 or 8, chosen so that the
// grid fills the GPU even when N is small) owns one tile; each CTA of the cluster takes a contiguous slice of K, each
// of its 8 warps a slice of that. Partial tiles are added in shared memory in warp order, then, across the cluster,
// the first CTA reads the other CTAs' sums through distributed shared memory in rank order. No global scratch, no
// atomics, and a result that does not depend on timing.
//
// Loads are 16 bytes per lane and 64 contiguous bytes per weight row and 32-element chunk: lane (g, t) of a warp
// holds elements [8t, 8t+8) of rows g and g+8. The two MMAs of a chunk pair those elements in an order that differs
// from the natural k order, identically for weights and activations, which leaves every dot product unchanged.
// Weight loads run one iteration (4 chunks) ahead of the MMAs, and the first of them are issued before the kernel
// waits for its predecessor (weights are never written by a kernel), so HBM stays busy across kernel boundaries.
//
// Epilogues: (0) + bias -> bfloat16 or float; (1) + residual (float, may alias out) -> float; (2) SwiGLU for a
// gate/up matrix whose rows are interleaved in blocks of 8 (rows 16b..16b+7 = gate features 8b..8b+7, rows
// 16b+8..16b+15 = the matching up features): out[m, 8b + r] = silu(gate) * up, bfloat16 [M, N/2].
// K must be a multiple of 8 (16-byte loads); anything else is refused.
#include "common.cuh"

#include <cooperative_groups.h>

IB_DEFINE_LAST_ERROR()

namespace {

namespace cg = cooperative_groups;
using bf16 = __nv_bfloat16;
constexpr int WARPS = 8;
constexpr int ROWS = 16;
constexpr int UNROLL = 4;

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One tile step: the MMAs of UNROLL chunks starting at chunk c, weights in (a0, a1), activations loaded here.
template <int NT>
__device__ __forceinline__ void tile_step(float (*acc)[4], const uint4* a0, const uint4* a1, const bf16* const* xr,
                                          const bool* x_ok, int64_t c, int64_t c_end, int64_t K, int t) {
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    uint4 b[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; u++) {
        const int64_t k = (c + u) * 32;
        const bool k_ok = c + u < c_end && k + t * 8 < K;
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
            b[u][nt] = (k_ok && x_ok[nt]) ? __ldg(reinterpret_cast<const uint4*>(xr[nt] + k)) : zero;
    }
#pragma unroll
    for (int u = 0; u < UNROLL; u++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            mma_bf16(acc[nt], a0[u].x, a1[u].x, a0[u].y, a1[u].y, b[u][nt].x, b[u][nt].y);
            mma_bf16(acc[nt], a0[u].z, a1[u].z, a0[u].w, a1[u].w, b[u][nt].z, b[u][nt].w);
        }
}

// WPT = warps per tile: 8 (the CTA's warps split K and add their partial tiles in shared memory; with a cluster,
// CTAs split K further) or 1 (every warp owns a tile and the whole K range: no reduction at all, for very large N).
template <int NT, int EPI, int WPT, typename TOut>
__global__ void __launch_bounds__(WARPS * 32, 2)
skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const float* __restrict__ bias,
              const float* residual, TOut* out, int M, int64_t N, int64_t K, int cluster) {
    __shared__ float red[WPT == 1 ? 1 : WARPS][NT][8][ROWS];
    __shared__ float part[NT][8][ROWS];                  // this CTA's sum; read by the cluster's first CTA
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rank = cluster > 1 ? int(blockIdx.x % cluster) : 0;
    const int64_t tile = WPT == 1 ? int64_t(blockIdx.x) * WARPS + warp : blockIdx.x / cluster;
    const int64_t n0 = tile * ROWS;
    const int64_t chunks = (K + 31) / 32;
    int64_t c_begin = 0, c_end = chunks;
    if (WPT != 1) {
        const int64_t per_cta = (chunks + cluster - 1) / cluster;
        const int64_t cta_begin = rank * per_cta, cta_end = min(chunks, cta_begin + per_cta);
        const int64_t per_warp = (max(int64_t(0), cta_end - cta_begin) + WARPS - 1) / WARPS;
        c_begin = cta_begin + warp * per_warp;
        c_end = min(cta_end, c_begin + per_warp);
    }
    const bool row0_ok = n0 + g < N, row1_ok = n0 + g + 8 < N;
    const bf16* w0 = w + (n0 + g) * K + t * 8;
    const bf16* w1 = w + (n0 + g + 8) * K + t * 8;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    auto load_w = [&](int64_t c, uint4* a0, uint4* a1) {
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int64_t k = (c + u) * 32;
            const bool k_ok = c + u < c_end && k + t * 8 < K;
            a0[u] = (k_ok && row0_ok) ? ld_stream(w0 + k) : zero;
            a1[u] = (k_ok && row1_ok) ? ld_stream(w1 + k) : zero;
        }
    };
    // Two register sets of weights alternate: while one is multiplied, the other is in flight.
    uint4 pa0[UNROLL], pa1[UNROLL], qa0[UNROLL], qa1[UNROLL];
    load_w(c_begin, pa0, pa1);                           // before the wait: weights have no producer kernel
    ib::pdl_wait();

    const bf16* xr[NT];
    bool x_ok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        x_ok[nt] = nt * 8 + g < M;
        xr[nt] = x + int64_t(nt * 8 + g) * K + t * 8;
    }
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;

    for (int64_t c = c_begin; c < c_end; c += 2 * UNROLL) {
        load_w(c + UNROLL, qa0, qa1);
        tile_step<NT>(acc, pa0, pa1, xr, x_ok, c, c_end, K, t);
        load_w(c + 2 * UNROLL, pa0, pa1);
        tile_step<NT>(acc, qa0, qa1, xr, x_ok, c + UNROLL, c_end, K, t);
    }
    ib::pdl_launch_dependents();

    if constexpr (WPT == 1) {
        // The warp's C fragments are the tile: rows g and g+8 (features), columns 2t and 2t+1 (tokens).
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int m = nt * 8 + 2 * t + e;
                if (m >= M) continue;
                if constexpr (EPI == 2) {
                    const float gate = acc[nt][e], up = acc[nt][2 + e];
                    const int64_t f = tile * 8 + g;
                    if (f < N / 2) out[int64_t(m) * (N / 2) + f] = ib::from_f32<TOut>(gate / (1.0f + expf(-gate)) * up);
                } else {
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {
                        const int64_t n = n0 + g + 8 * hh;
                        if (n >= N) continue;
                        float v = acc[nt][2 * hh + e];
                        if (bias) v += bias[n];
                        if constexpr (EPI == 1) v += residual[int64_t(m) * N + n];
                        out[int64_t(m) * N + n] = ib::from_f32<TOut>(v);
                    }
                }
            }
        return;
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        red[warp][nt][2 * t][g] = acc[nt][0];
        red[warp][nt][2 * t + 1][g] = acc[nt][1];
        red[warp][nt][2 * t][g + 8] = acc[nt][2];
        red[warp][nt][2 * t + 1][g + 8] = acc[nt][3];
    }
    __syncthreads();
    const bool active = threadIdx.x < NT * 128;
    const int r = threadIdx.x & 15, col = (threadIdx.x >> 4) & 7, nt = active ? threadIdx.x >> 7 : 0;
    float v = 0.0f;
    if (active) {
#pragma unroll
        for (int wi = 0; wi < WARPS; wi++) v += red[wi][nt][col][r];
    }
    if (cluster > 1) {
        cg::cluster_group cl = cg::this_cluster();
        if (active) part[nt][col][r] = v;
        cl.sync();
        if (rank == 0 && active) {
            for (int other = 1; other < cluster; other++)
                v += cl.map_shared_rank(&part[0][0][0], other)[(nt * 8 + col) * ROWS + r];
        }
        if (rank == 0 && EPI == 2 && active) part[nt][col][r] = v;     // the SwiGLU epilogue pairs rows r and r + 8
        cl.sync();                                       // the others' shared memory stays alive until it was read
        if (rank != 0) return;
    } else if (EPI == 2) {
        if (active) part[nt][col][r] = v;
        __syncthreads();
    }
    if (!active) return;
    const int m = nt * 8 + col;
    if (m >= M) return;
    if constexpr (EPI == 2) {
        if (r >= 8) return;
        const float gate = v, up = part[nt][col][r + 8];
        const int64_t f = tile * 8 + r;
        if (f < N / 2) out[int64_t(m) * (N / 2) + f] = ib::from_f32<TOut>(gate / (1.0f + expf(-gate)) * up);
    } else {
        const int64_t n = n0 + r;
        if (n >= N) return;
        if (bias) v += bias[n];
        if constexpr (EPI == 1) v += residual[int64_t(m) * N + n];
        out[int64_t(m) * N + n] = ib::from_f32<TOut>(v);
    }
}

template <int NT, int WPT>
int launch(const bf16* x, const bf16* w, const float* bias, const float* residual, void* out, int M, int64_t N, int64_t K,
           int out_dtype, int epi, int cluster, cudaStream_t stream) {
    const int64_t tiles = (N + ROWS - 1) / ROWS;
    const dim3 grid{WPT == 1 ? unsigned((tiles + WARPS - 1) / WARPS) : unsigned(tiles) * unsigned(cluster), 1u, 1u};
    const dim3 block{WARPS * 32, 1u, 1u};
    const unsigned cl = unsigned(cluster);
    if (epi == 2) {
        if (out_dtype != IB_BF16) return ib::fail(IB_ERR_ARG, "linear_skinny: the SwiGLU epilogue writes bfloat16");
        return ib::launch("linear_skinny", skinny_kernel<NT, 2, WPT, bf16>, grid, block, 0, stream, cl, x, w,
                          (const float*)nullptr, (const float*)nullptr, (bf16*)out, M, N, K, cluster);
    }
    if (epi == 1) {
        if (out_dtype != IB_F32 || !residual) return ib::fail(IB_ERR_ARG, "linear_skinny: the residual epilogue needs a float residual and output");
        return ib::launch("linear_skinny", skinny_kernel<NT, 1, WPT, float>, grid, block, 0, stream, cl, x, w, bias,
                          residual, (float*)out, M, N, K, cluster);
    }
    if (out_dtype == IB_F32)
        return ib::launch("linear_skinny", skinny_kernel<NT, 0, WPT, float>, grid, block, 0, stream, cl, x, w, bias,
                          (const float*)nullptr, (float*)out, M, N, K, cluster);
    if (out_dtype == IB_BF16)
        return ib::launch("linear_skinny", skinny_kernel<NT, 0, WPT, bf16>, grid, block, 0, stream, cl, x, w, bias,
                          (const float*)nullptr, (bf16*)out, M, N, K, cluster);
    return ib::fail(IB_ERR_ARG, "linear_skinny: unknown output dtype %d", out_dtype);
}

}  // namespace

// epi: 0 = (+ bias), 1 = (+ bias) + residual -> float, 2 = SwiGLU over rows interleaved by 8 -> bfloat16 [M, N/2].
// cluster: CTAs that share a tile's K range (1, 2, 4 or 8); 0 lets the kernel choose from N, K and sm_count, and
// -1 asks for the warp-per-tile mapping (no reduction), which the kernel also chooses by itself for very large N.
IB_EXPORT int ib_linear_skinny(const void* x, const void* w, const float* bias, const float* residual, void* out,
                               int64_t M, int64_t N, int64_t K, int out_dtype, int epi, int cluster, int sm_count,
                               cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IB_OK;
    if (M > 16) return ib::fail(IB_ERR_ARG, "linear_skinny: at most 16 rows, got %lld", (long long)M);
    if (K <= 0 || K % 8) return ib::fail(IB_ERR_ARG, "linear_skinny: K = %lld must be a positive multiple of 8", (long long)K);
    if ((uintptr_t(x) & 15) || (uintptr_t(w) & 15)) return ib::fail(IB_ERR_ARG, "linear_skinny: operands must be 16-byte aligned");
    if (epi == 2 && N % 16) return ib::fail(IB_ERR_ARG, "linear_skinny: the SwiGLU epilogue needs N to be a multiple of 16");
    const int64_t tiles = (N + ROWS - 1) / ROWS;
    if (tiles * 8 > 0x7fffffffLL) return ib::fail(IB_ERR_ARG, "linear_skinny: N too large");
    const int sms = sm_count > 0 ? sm_count : 148;
    if (cluster == 0) {
        if (tiles >= 16LL * WARPS * sms / 4) {
            cluster = -1;                                 // enough tiles for every warp of the GPU to own several
        } else {
            // Fill the GPU about twice over, but leave every warp at least four 32-element chunks of K.
            cluster = 1;
            const int64_t chunks = (K + 31) / 32;
            while (cluster < 8 && tiles * cluster < 2LL * sms && chunks / (cluster * 2) >= 4 * WARPS) cluster *= 2;
        }
    }
    if (cluster == -1) {
        if (M <= 8) return launch<1, 1>((const bf16*)x, (const bf16*)w, bias, residual, out, int(M), N, K, out_dtype, epi, 1, stream);
        return launch<2, 1>((const bf16*)x, (const bf16*)w, bias, residual, out, int(M), N, K, out_dtype, epi, 1, stream);
    }
    if (cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) return ib::fail(IB_ERR_ARG, "linear_skinny: cluster must be 1, 2, 4 or 8");
    if (M <= 8) return launch<1, 8>((const bf16*)x, (const bf16*)w, bias, residual, out, int(M), N, K, out_dtype, epi, cluster, stream);
    return launch<2, 8>((const bf16*)x, (const bf16*)w, bias, residual, out, int(M), N, K, out_dtype, epi, cluster, stream);
}
