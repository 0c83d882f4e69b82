// Streaming matrix product for decode steps: out[M, N] = f(x)[M, K] . w[N, K]^T with M <= 16 tokens, where f is the
// identity (x bfloat16) or a fused RMSNorm (x = the float residual stream, normalised on the fly).
//
// The weights are read exactly once, straight from global memory into registers with 16-byte loads, and used as
// the 16-row operand of mma.sync m16n8k16 (bfloat16 in, float accumulation); the tokens are the 8-wide operand.
// The kernel is bound by HBM bandwidth, so the tensor-core shape only has to keep the instruction count low.
//
// Work split. A tile is 16 output features and one CTA (many small CTAs, eight and more per SM, keep enough loads in
// flight to saturate HBM; a persistent variant with a register ping-pong across tiles measured slower). The CTA's 8
// warps split K and add their partial tiles in shared memory in warp order. For small N a thread-block cluster of 2,
// 4 or 8 CTAs shares each tile, each CTA taking a slice of K, and the cluster's first CTA adds the slices through
// distributed shared memory in rank order: no global scratch, no atomics, a result that does not depend on timing.
// The first weight loads are issued before the kernel waits for its predecessor (weights have no producer kernel).
//
// Fused norm. With norm_w the activations are the float residual stream: each warp normalises rows into shared
// memory, y = x * rsqrt(mean(x^2) + eps) * g in float, rounded to bfloat16 as the separate norm kernel would
// (K <= 4096; padded rows give conflict-free 16-byte reads). Without it activations are read through L1.
//
// Loads are 16 bytes per lane and 64 contiguous bytes per weight row and 32-element chunk: lane (g, t) of a warp
// holds elements [8t, 8t+8) of rows g and g+8. The two MMAs of a chunk pair those elements in an order that differs
// from the natural k order, identically for weights and activations, which leaves every dot product unchanged.
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
constexpr int XS_MAX_K = 4096;            // activations are staged in shared memory up to this K
constexpr int XS_PAD = 64;                // bytes of padding per staged row (rows start 16 banks apart)

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

struct GemvParams {
    const bf16* x;            // [M, K] bfloat16 activations (NORM = false)
    const float* h;           // [M, K] float residual stream (NORM = true)
    const float* norm_w;      // [K]
    float eps;
    const bf16* w;            // [N, K]
    const float* bias;        // [N] or null
    const float* residual;    // [M, N] or null
    void* out;
    int M;
    int64_t N, K, tiles;
    int cluster, groups;      // CTAs per tile; tile groups in the grid (grid = groups * cluster)
    int stage_x;              // activations staged in shared memory
    const void* prefetch;     // weights of a later kernel to pull into L2 meanwhile (or null)
    int64_t prefetch_bytes;
};

// Occupancy matters more than anything else here (resident warps = bytes in flight): 64 registers for up to 8
// tokens, so that four CTAs share an SM.
template <int NT, int EPI, bool NORM, typename TOut>
__global__ void __launch_bounds__(WARPS * 32, NT == 1 ? 4 : 2)
stream_gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(16) uint8_t xs[];        // staged activations [8 NT][K + pad] bfloat16 (fused norm only)
    __shared__ float red[WARPS][NT][8][ROWS];
    __shared__ float part[NT][8][ROWS];                  // this CTA's sum; read by the cluster's first CTA
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int cluster = p.cluster;
    const int rank = cluster > 1 ? int(blockIdx.x % cluster) : 0;
    const int64_t tile = blockIdx.x / cluster;
    const int64_t K = p.K, N = p.N;
    const int64_t n0 = tile * ROWS;
    const int64_t chunks = (K + 31) / 32;
    const int64_t per_cta = (chunks + cluster - 1) / cluster;
    const int64_t cta_begin = rank * per_cta, cta_end = min(chunks, cta_begin + per_cta);
    const int64_t per_warp = (per_cta + WARPS - 1) / WARPS;
    const int64_t c_begin = min(cta_end, cta_begin + warp * per_warp), c_end = min(cta_end, c_begin + per_warp);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const bool row0_ok = n0 + g < N, row1_ok = n0 + g + 8 < N;
    const bf16* w0 = p.w + (n0 + g) * K + t * 8;
    const bf16* w1 = p.w + (n0 + g + 8) * K + t * 8;

    auto load_w = [&](int64_t c, uint4* a0, uint4* a1) {
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int64_t k = (c + u) * 32;
            const bool k_ok = c + u < c_end && k + t * 8 < K;
            a0[u] = (k_ok && row0_ok) ? ld_stream(w0 + k) : zero;
            a1[u] = (k_ok && row1_ok) ? ld_stream(w1 + k) : zero;
        }
    };
    uint4 a0[UNROLL], a1[UNROLL];
    load_w(c_begin, a0, a1);                             // before the wait: weights have no producer kernel
    ib::l2_prefetch_share(p.prefetch, p.prefetch_bytes, blockIdx.x, gridDim.x);
    ib::pdl_launch_dependents();                         // the successor may start its own weight loads as SMs free up
    ib::pdl_wait();

    // ---------------------------------------------------------------- fused RMSNorm: normalised rows in shared memory
    const int64_t xs_pitch = K * 2 + XS_PAD;             // bytes per staged row
    if constexpr (NORM) {
        for (int row = warp; row < p.M; row += WARPS) {
            const float* hr = p.h + int64_t(row) * K;
            float ss = 0.0f;
            for (int64_t i = lane * 4; i < K; i += 128) {
                const float4 v = *reinterpret_cast<const float4*>(hr + i);
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            }
            ss = ib::warp_sum(ss);
            const float scale = rsqrtf(ss / float(K) + p.eps);
            for (int64_t i = lane * 4; i < K; i += 128) {
                const float4 v = *reinterpret_cast<const float4*>(hr + i);
                const float4 gw = *reinterpret_cast<const float4*>(p.norm_w + i);
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * scale * gw.x, v.y * scale * gw.y);
                __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * scale * gw.z, v.w * scale * gw.w);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(xs + row * xs_pitch + i * 2) = pk;
            }
        }
        __syncthreads();
    }
    bool x_ok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) x_ok[nt] = nt * 8 + g < p.M;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;

    for (int64_t c = c_begin; c < c_end; c += UNROLL) {
        if (c != c_begin) load_w(c, a0, a1);
        uint4 b[UNROLL][NT];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int64_t k = (c + u) * 32 + t * 8;
            const bool k_ok = c + u < c_end && k < K;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                if (!(k_ok && x_ok[nt])) b[u][nt] = zero;
                else if (NORM) b[u][nt] = *reinterpret_cast<const uint4*>(xs + (nt * 8 + g) * xs_pitch + k * 2);
                else b[u][nt] = __ldg(reinterpret_cast<const uint4*>(p.x + int64_t(nt * 8 + g) * K + k));
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                mma_bf16(acc[nt], a0[u].x, a1[u].x, a0[u].y, a1[u].y, b[u][nt].x, b[u][nt].y);
                mma_bf16(acc[nt], a0[u].z, a1[u].z, a0[u].w, a1[u].w, b[u][nt].z, b[u][nt].w);
            }
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
        cl.sync();                                       // the others' shared memory stays alive until it was read
        if (rank != 0) return;
    }
    if (EPI == 2) {
        if (active) part[nt][col][r] = v;                // the SwiGLU epilogue pairs rows r and r + 8
        __syncthreads();
    }
    const int m = nt * 8 + col;
    if (!active || m >= p.M) return;
    TOut* out = reinterpret_cast<TOut*>(p.out);
    if constexpr (EPI == 2) {
        if (r >= 8) return;
        const float gate = v, up = part[nt][col][r + 8];
        const int64_t f = tile * 8 + r;
        if (f < N / 2) out[int64_t(m) * (N / 2) + f] = ib::from_f32<TOut>(gate / (1.0f + expf(-gate)) * up);
    } else {
        const int64_t n = n0 + r;
        if (n >= N) return;
        if (p.bias) v += p.bias[n];
        if constexpr (EPI == 1) v += p.residual[int64_t(m) * N + n];
        out[int64_t(m) * N + n] = ib::from_f32<TOut>(v);
    }
}

template <int NT, bool NORM>
int launch(const GemvParams& p, int out_dtype, int epi, int grid_ctas, size_t smem, cudaStream_t stream) {
    const dim3 grid{unsigned(grid_ctas), 1u, 1u};
    const dim3 block{WARPS * 32, 1u, 1u};
    const unsigned cl = unsigned(p.cluster);
#define IB_GEMV_LAUNCH(EPI_, T_)                                                                                   \
    do {                                                                                                           \
        static bool configured = false;                                                                            \
        if (!configured) {                                                                                         \
            cudaError_t e = cudaFuncSetAttribute(stream_gemv_kernel<NT, EPI_, NORM, T_>,                           \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 16 * (XS_MAX_K * 2 + XS_PAD)); \
            if (e != cudaSuccess) return ib::fail(IB_ERR_CUDA, "linear_skinny: cannot set shared memory size: %s", cudaGetErrorString(e)); \
            configured = true;                                                                                     \
        }                                                                                                          \
        return ib::launch("linear_skinny", stream_gemv_kernel<NT, EPI_, NORM, T_>, grid, block, smem, stream, cl, p);  \
    } while (0)
    if (epi == 2) {
        if (out_dtype != IB_BF16) return ib::fail(IB_ERR_ARG, "linear_skinny: the SwiGLU epilogue writes bfloat16");
        IB_GEMV_LAUNCH(2, bf16);
    }
    if (epi == 1) {
        if (out_dtype != IB_F32 || !p.residual) return ib::fail(IB_ERR_ARG, "linear_skinny: the residual epilogue needs a float residual and output");
        IB_GEMV_LAUNCH(1, float);
    }
    if (out_dtype == IB_F32) IB_GEMV_LAUNCH(0, float);
    if (out_dtype == IB_BF16) IB_GEMV_LAUNCH(0, bf16);
#undef IB_GEMV_LAUNCH
    return ib::fail(IB_ERR_ARG, "linear_skinny: unknown output dtype %d", out_dtype);
}

}  // namespace

// x: bfloat16 [M, K], or with norm_w != null the float residual stream [M, K] that is RMS-normalised on the fly
// (y = x * rsqrt(mean(x^2) + eps) * norm_w, K <= 4096). epi: 0 = (+ bias), 1 = (+ bias) + residual -> float,
// 2 = SwiGLU over rows interleaved by 8 -> bfloat16 [M, N/2]. cluster: CTAs that share a tile's K range (1, 2, 4 or
// 8); 0 lets the kernel choose from N, K and sm_count.
IB_EXPORT int ib_linear_skinny(const void* x, const float* norm_w, float eps, const void* w, const float* bias,
                               const float* residual, void* out, int64_t M, int64_t N, int64_t K, int out_dtype, int epi,
                               int cluster, int sm_count, const void* prefetch, int64_t prefetch_bytes,
                               cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IB_OK;
    if (M > 16) return ib::fail(IB_ERR_ARG, "linear_skinny: at most 16 rows, got %lld", (long long)M);
    if (K <= 0 || K % 8) return ib::fail(IB_ERR_ARG, "linear_skinny: K = %lld must be a positive multiple of 8", (long long)K);
    if ((uintptr_t(x) & 15) || (uintptr_t(w) & 15)) return ib::fail(IB_ERR_ARG, "linear_skinny: operands must be 16-byte aligned");
    if (epi == 2 && N % 16) return ib::fail(IB_ERR_ARG, "linear_skinny: the SwiGLU epilogue needs N to be a multiple of 16");
    if (norm_w && (K > XS_MAX_K || (uintptr_t(norm_w) & 15)))
        return ib::fail(IB_ERR_ARG, "linear_skinny: the fused norm takes K <= %d and a 16-byte aligned weight", XS_MAX_K);
    const int64_t tiles = (N + ROWS - 1) / ROWS;
    if (tiles > 0x7fffffffLL / 8) return ib::fail(IB_ERR_ARG, "linear_skinny: N too large");
    const int sms = sm_count > 0 ? sm_count : 148;
    if (cluster == 0) {
        // Share a tile among CTAs while the tiles alone leave SMs idle and every warp keeps at least four chunks of K.
        cluster = 1;
        const int64_t chunks = (K + 31) / 32;
        while (cluster < 8 && tiles * cluster < 2LL * sms && chunks / (cluster * 2) >= 4 * WARPS) cluster *= 2;
    }
    if (cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) return ib::fail(IB_ERR_ARG, "linear_skinny: cluster must be 1, 2, 4 or 8");
    GemvParams p;
    p.x = norm_w ? nullptr : (const bf16*)x;
    p.h = norm_w ? (const float*)x : nullptr;
    p.norm_w = norm_w; p.eps = eps;
    p.w = (const bf16*)w; p.bias = bias; p.residual = residual; p.out = out;
    p.M = int(M); p.N = N; p.K = K; p.tiles = tiles; p.cluster = cluster;
    p.groups = int(tiles);
    p.prefetch = prefetch; p.prefetch_bytes = prefetch_bytes & ~int64_t(15);
    p.stage_x = norm_w ? 1 : 0;
    const int rows_pad = M <= 8 ? 8 : 16;
    const size_t smem = norm_w ? size_t(rows_pad) * size_t(K * 2 + XS_PAD) : 0;
    const int grid_ctas = int(tiles) * cluster;
    if (norm_w) {
        if (M <= 8) return launch<1, true>(p, out_dtype, epi, grid_ctas, smem, stream);
        return launch<2, true>(p, out_dtype, epi, grid_ctas, smem, stream);
    }
    if (M <= 8) return launch<1, false>(p, out_dtype, epi, grid_ctas, smem, stream);
    return launch<2, false>(p, out_dtype, epi, grid_ctas, smem, stream);
}
