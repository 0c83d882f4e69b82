// Skinny matrix product for decode steps: out[M, N] = x[M, K] . w[N, K]^T with M <= 16 tokens.
//
// The weights are read exactly once, straight from global memory into registers with 16-byte loads, and used as
// the 16-row operand of mma.sync m16n8k16 (bfloat16 in, float accumulation); the tokens are the 8-wide operand.
// The kernel is bound by HBM bandwidth, so the tensor-core shape only has to keep the instruction count low.
//
// One CTA of 8 warps owns 16 output features and the whole K range; each warp takes a contiguous slice of K and the
// eight partial tiles are added in shared memory in warp order, so a result does not depend on timing.
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

IB_DEFINE_LAST_ERROR()

namespace {

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

template <int NT, int EPI, typename TOut>
__global__ void __launch_bounds__(WARPS * 32)
skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const float* __restrict__ bias,
              const float* residual, TOut* out, int M, int64_t N, int64_t K) {
    __shared__ float red[WARPS][NT][8][ROWS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t n0 = int64_t(blockIdx.x) * ROWS;
    const int64_t chunks = (K + 31) / 32;
    const int64_t per_warp = (chunks + WARPS - 1) / WARPS;
    const int64_t c_begin = warp * per_warp, c_end = min(chunks, c_begin + per_warp);

    const bool row0_ok = n0 + g < N, row1_ok = n0 + g + 8 < N;
    const bf16* w0 = w + (n0 + g) * K + t * 8;
    const bf16* w1 = w + (n0 + g + 8) * K + t * 8;
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
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    for (int64_t c = c_begin; c < c_end; c += UNROLL) {
        uint4 a0[UNROLL], a1[UNROLL], b[UNROLL][NT];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int64_t k = (c + u) * 32;
            const bool k_ok = c + u < c_end && k + t * 8 < K;
            a0[u] = (k_ok && row0_ok) ? ld_stream(w0 + k) : zero;
            a1[u] = (k_ok && row1_ok) ? ld_stream(w1 + k) : zero;
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
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        red[warp][nt][2 * t][g] = acc[nt][0];
        red[warp][nt][2 * t + 1][g] = acc[nt][1];
        red[warp][nt][2 * t][g + 8] = acc[nt][2];
        red[warp][nt][2 * t + 1][g + 8] = acc[nt][3];
    }
    __syncthreads();
    if (threadIdx.x >= NT * 128) return;
    const int r = threadIdx.x & 15, col = (threadIdx.x >> 4) & 7, nt = threadIdx.x >> 7;
    const int m = nt * 8 + col;
    if (m >= M) return;
    if constexpr (EPI == 2) {
        if (r >= 8) return;
        float gate = 0.0f, up = 0.0f;
#pragma unroll
        for (int wi = 0; wi < WARPS; wi++) { gate += red[wi][nt][col][r]; up += red[wi][nt][col][r + 8]; }
        const int64_t f = int64_t(blockIdx.x) * 8 + r;
        if (f < N / 2) out[int64_t(m) * (N / 2) + f] = ib::from_f32<TOut>(gate / (1.0f + expf(-gate)) * up);
    } else {
        const int64_t n = n0 + r;
        if (n >= N) return;
        float v = 0.0f;
#pragma unroll
        for (int wi = 0; wi < WARPS; wi++) v += red[wi][nt][col][r];
        if (bias) v += bias[n];
        if constexpr (EPI == 1) v += residual[int64_t(m) * N + n];
        out[int64_t(m) * N + n] = ib::from_f32<TOut>(v);
    }
}

template <int NT>
int launch(const bf16* x, const bf16* w, const float* bias, const float* residual, void* out, int M, int64_t N, int64_t K,
           int out_dtype, int epi, cudaStream_t stream) {
    const unsigned grid = unsigned((N + ROWS - 1) / ROWS);
    if (epi == 2) {
        if (out_dtype != IB_BF16) return ib::fail(IB_ERR_ARG, "linear_skinny: the SwiGLU epilogue writes bfloat16");
        skinny_kernel<NT, 2, bf16><<<grid, WARPS * 32, 0, stream>>>(x, w, nullptr, nullptr, (bf16*)out, M, N, K);
    } else if (epi == 1) {
        if (out_dtype != IB_F32 || !residual) return ib::fail(IB_ERR_ARG, "linear_skinny: the residual epilogue needs a float residual and output");
        skinny_kernel<NT, 1, float><<<grid, WARPS * 32, 0, stream>>>(x, w, bias, residual, (float*)out, M, N, K);
    } else if (out_dtype == IB_F32) {
        skinny_kernel<NT, 0, float><<<grid, WARPS * 32, 0, stream>>>(x, w, bias, nullptr, (float*)out, M, N, K);
    } else if (out_dtype == IB_BF16) {
        skinny_kernel<NT, 0, bf16><<<grid, WARPS * 32, 0, stream>>>(x, w, bias, nullptr, (bf16*)out, M, N, K);
    } else {
        return ib::fail(IB_ERR_ARG, "linear_skinny: unknown output dtype %d", out_dtype);
    }
    return ib::check_launch("linear_skinny");
}

}  // namespace

// epi: 0 = (+ bias), 1 = (+ bias) + residual -> float, 2 = SwiGLU over rows interleaved by 8 -> bfloat16 [M, N/2].
IB_EXPORT int ib_linear_skinny(const void* x, const void* w, const float* bias, const float* residual, void* out,
                               int64_t M, int64_t N, int64_t K, int out_dtype, int epi, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IB_OK;
    if (M > 16) return ib::fail(IB_ERR_ARG, "linear_skinny: at most 16 rows, got %lld", (long long)M);
    if (K <= 0 || K % 8) return ib::fail(IB_ERR_ARG, "linear_skinny: K = %lld must be a positive multiple of 8", (long long)K);
    if ((uintptr_t(x) & 15) || (uintptr_t(w) & 15)) return ib::fail(IB_ERR_ARG, "linear_skinny: operands must be 16-byte aligned");
    if (epi == 2 && N % 16) return ib::fail(IB_ERR_ARG, "linear_skinny: the SwiGLU epilogue needs N to be a multiple of 16");
    if ((N + ROWS - 1) / ROWS > 0x7fffffffLL) return ib::fail(IB_ERR_ARG, "linear_skinny: N too large");
    if (M <= 8) return launch<1>((const bf16*)x, (const bf16*)w, bias, residual, out, int(M), N, K, out_dtype, epi, stream);
    return launch<2>((const bf16*)x, (const bf16*)w, bias, residual, out, int(M), N, K, out_dtype, epi, stream);
}
