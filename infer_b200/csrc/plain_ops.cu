// Plain kernels: one simple, batch-invariant kernel per operation of the model.
//
// They serve two purposes. With float storage they ARE the true 32-bit path of the engine: FFMA
// accumulation in a fixed order, no tensor cores, no reduced-precision matrix mode. With bfloat16
// storage (float arithmetic inside) they are the reference that each fast kernel is tested against,
// and the path for shapes a fast kernel refuses.
//
// Batch invariance: every output element is reduced in an order that depends only on the
// reduction length and the absolute position of what is reduced, never on the number of rows,
// the composition of the batch, or where pages lie.
//
// The operations and their formulas follow the reference engine: kernels/ops/embedding.cu:6-12,
// kernels/ops/rmsnorm.cu:9-28, kernels/ops/gemm.cu:25-75, kernels/ops/batch.cu:207-237 (rotary +
// cache write), kernels/ops/batch.cu:250-316 (attention over a block table),
// kernels/ops/elementwise.cu:6-16, kernels/ops/batch.cu:450-478 (sampling).
#include "common.cuh"
#include <cooperative_groups.h>

IB_DEFINE_LAST_ERROR()

// Launch on `stream` with the library's launch attributes; a failure returns from the calling entry point.
#define IB_LAUNCH(kernel, grid, block, smem, ...)                                                              \
    do {                                                                                                       \
        const int rc_ = ib::launch(#kernel, kernel, dim3(grid), dim3(block), size_t(smem), stream, 1u, __VA_ARGS__); \
        if (rc_) return rc_;                                                                                   \
    } while (0)

namespace {

using bf16 = __nv_bfloat16;

// ------------------------------------------------------------------------------------------------
// Embedding: out[t, :] = float(table[ids[t], :]) * scale (scale 1 for architectures without one). Ids are validated on the host; an id outside the
// table writes zeros and raises the status word rather than reading out of bounds. An id of -1 stands for "the
// token sampled last for this request", which the sampling kernel left in feedback[slot of the request].
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids, int64_t n_tokens,
                                 int64_t hidden, int64_t vocab, float* __restrict__ out, int* status,
                                 const int* __restrict__ feedback, const int* __restrict__ token_seg,
                                 const int* __restrict__ seg_slot, float scale) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_tokens * hidden) return;
    const int64_t t = i / hidden, c = i - t * hidden;
    int id = ids[t];
    // id -1: the token that was sampled last for this token's request, still on the device (feedback[slot])
    if (id == -1 && feedback) id = feedback[seg_slot[token_seg[t]]];
    if (id < 0 || id >= vocab) {
        out[i] = 0.0f;
        if (status) atomicExch(status, 1);
        return;
    }
    const float v = ib::to_f32(table[int64_t(id) * hidden + c]);
    out[i] = scale == 1.0f ? v : v * scale;
}

// ------------------------------------------------------------------------------------------------
// RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, eps inside the root, after the mean.
// One block per output row; `rows` optionally gathers input rows (out[i] = norm(x[rows[i]])).
template <typename TOut>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps, int64_t hidden,
                               const int* __restrict__ rows, TOut* __restrict__ out) {
    ib::pdl_launch_dependents();                          // the successor may set up (and request its weights) meanwhile
    ib::pdl_wait();
    __shared__ float red[32];
    const int64_t r_out = blockIdx.x;
    const int64_t r_in = rows ? rows[r_out] : r_out;
    const float* xr = x + r_in * hidden;
    float ss = 0.0f;
    for (int64_t i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = ib::block_sum(ss, red);
    const float scale = rsqrtf(ss / float(hidden) + eps);
    for (int64_t i = threadIdx.x; i < hidden; i += blockDim.x)
        out[r_out * hidden + i] = ib::from_f32<TOut>(xr[i] * scale * w[i]);
}

// The same norm for rows whose length is a multiple of 4 and whose buffers are 16-byte aligned: a block of four warps
// per row, 16-byte loads kept in registers between the two passes (rows of up to 6144 elements; longer rows read the
// row a second time, from L1). The sum of squares is put together in thread, lane and warp order, whatever the number
// of rows is.
constexpr int NORM_THREADS = 128, NORM_KEEP = 12;
template <typename TOut>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps, int64_t hidden,
                   const int* __restrict__ rows, TOut* __restrict__ out) {
    ib::pdl_launch_dependents();                          // the successor may set up (and request its weights) meanwhile
    ib::pdl_wait();
    __shared__ float red[NORM_THREADS / 32];
    const int64_t r_out = blockIdx.x;
    const int64_t r_in = rows ? rows[r_out] : r_out;
    const float4* xr = reinterpret_cast<const float4*>(x + r_in * hidden);
    const float4* wr = reinterpret_cast<const float4*>(w);
    const int64_t n4 = hidden / 4;
    float4 keep[NORM_KEEP];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < NORM_KEEP; j++) {
        const int64_t i = threadIdx.x + int64_t(j) * NORM_THREADS;
        keep[j] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < NORM_KEEP; j++) {
        const float4 v = keep[j];
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    for (int64_t i = threadIdx.x + int64_t(NORM_KEEP) * NORM_THREADS; i < n4; i += NORM_THREADS) {
        const float4 v = xr[i];
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = ib::warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < NORM_THREADS / 32; i++) total += red[i];
    const float scale = rsqrtf(total / float(hidden) + eps);
    auto emit = [&](int64_t i, float4 v) {
        const float4 g = wr[i];
        const float a = v.x * scale * g.x, b = v.y * scale * g.y, c = v.z * scale * g.z, d = v.w * scale * g.w;
        if constexpr (sizeof(TOut) == 4) {
            reinterpret_cast<float4*>(out + r_out * hidden)[i] = make_float4(a, b, c, d);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
            uint2 u;
            u.x = *reinterpret_cast<uint32_t*>(&lo);
            u.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(out + r_out * hidden)[i] = u;
        }
    };
#pragma unroll
    for (int j = 0; j < NORM_KEEP; j++) {
        const int64_t i = threadIdx.x + int64_t(j) * NORM_THREADS;
        if (i < n4) emit(i, keep[j]);
    }
    for (int64_t i = threadIdx.x + int64_t(NORM_KEEP) * NORM_THREADS; i < n4; i += NORM_THREADS) emit(i, xr[i]);
}

// ------------------------------------------------------------------------------------------------
// Linear: out[m, n] = sum_k x[m, k] * w[n, k] (+ bias[n]) (+ residual[m, n]).
// 64x64 output tile, 16-wide k steps, 4x4 outputs per thread. Each output's sum runs over k in
// ascending order in float, whatever M is.
constexpr int LT = 64, LK = 16;

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
linear_kernel(const TIn* __restrict__ x, const TIn* __restrict__ w, const float* __restrict__ bias,
              const float* residual, TOut* out, int64_t M, int64_t N, int64_t K) {
    ib::pdl_wait();
    __shared__ float xs[LK][LT + 1];
    __shared__ float ws[LK][LT + 1];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int64_t m0 = int64_t(blockIdx.y) * LT, n0 = int64_t(blockIdx.x) * LT;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    for (int64_t k0 = 0; k0 < K; k0 += LK) {
        // 64 rows x 16 k of each operand: 1024 elements, 4 per thread.
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int idx = tid + e * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int64_t k = k0 + kk;
            xs[kk][r] = (m0 + r < M && k < K) ? ib::to_f32(x[(m0 + r) * K + k]) : 0.0f;
            ws[kk][r] = (n0 + r < N && k < K) ? ib::to_f32(w[(n0 + r) * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < LK; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int64_t m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int64_t n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            if (residual) v += residual[m * N + n];
            out[m * N + n] = ib::from_f32<TOut>(v);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Rotary positions + cache write. Input rows are [q heads | k heads | v heads] of one token.
// q is rotated into q_out; k is rotated and stored at the token's place in the paged cache; v is
// stored as it is. Rotation pairs element j with j + head_dim/2:
//   x1' = x1*cos - x2*sin ; x2' = x2*cos + x1*sin, angles from float tables [max_pos, head_dim/2].
// A page is [kv_heads, page_size, head_dim]; the token's page is block_table[seg, pos / page_size].
// cos == nullptr skips the rotation (positions are encoded elsewhere, or not at all).
template <typename T>
__global__ void rope_kv_write_kernel(const T* __restrict__ qkv, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, const int* __restrict__ positions,
                                     const int* __restrict__ token_seg, const int* __restrict__ block_table,
                                     int64_t max_blocks, T* __restrict__ q_out, T* __restrict__ k_cache,
                                     T* __restrict__ v_cache, int64_t n_tokens, int n_heads, int n_kv, int head_dim,
                                     int page_size, int write_cache, int64_t n_pages, int* status) {
    ib::pdl_launch_dependents();                          // the successor may set up (and request its weights) meanwhile
    ib::pdl_wait();
    const int half = head_dim / 2;
    const int units = (n_heads + 2 * n_kv) * half;   // one unit = one (head, j) pair
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_tokens * units) return;
    const int64_t t = i / units;
    const int u = int(i - t * units);
    const int head = u / half, j = u - head * half;
    const int pos = positions[t];
    const T* row = qkv + t * int64_t(n_heads + 2 * n_kv) * head_dim + int64_t(head) * head_dim;
    float x1 = ib::to_f32(row[j]), x2 = ib::to_f32(row[j + half]);
    const bool is_v = head >= n_heads + n_kv;
    if (!is_v && cos_t) {
        const float c = cos_t[int64_t(pos) * half + j], s = sin_t[int64_t(pos) * half + j];
        const float r1 = x1 * c - x2 * s;
        const float r2 = x2 * c + x1 * s;
        x1 = r1;
        x2 = r2;
    }
    if (head < n_heads) {
        T* o = q_out + t * int64_t(n_heads) * head_dim + int64_t(head) * head_dim;
        o[j] = ib::from_f32<T>(x1);
        o[j + half] = ib::from_f32<T>(x2);
        return;
    }
    if (!write_cache) return;
    const int kvh = is_v ? head - n_heads - n_kv : head - n_heads;
    const int page = block_table[int64_t(token_seg[t]) * max_blocks + pos / page_size];
    if (page < 0 || page >= n_pages) {
        if (status) atomicExch(status, 2);
        return;
    }
    T* base = (is_v ? v_cache : k_cache) +
              ((int64_t(page) * n_kv + kvh) * page_size + pos % page_size) * head_dim;
    base[j] = ib::from_f32<T>(x1);
    base[j + half] = ib::from_f32<T>(x2);
}

// The same for bfloat16 with head_dim a multiple of 16 and 16-byte aligned buffers: a thread takes 8 consecutive
// pairs (two 16-byte loads, two 16-byte stores); every element goes through the arithmetic above.
__global__ void __launch_bounds__(256)
rope_kv_write_vec_kernel(const bf16* __restrict__ qkv, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                         const int* __restrict__ positions, const int* __restrict__ token_seg,
                         const int* __restrict__ block_table, int64_t max_blocks, bf16* __restrict__ q_out,
                         bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int64_t n_tokens, int n_heads, int n_kv,
                         int head_dim, int page_size, int write_cache, int64_t n_pages, int* status) {
    ib::pdl_launch_dependents();                          // the successor may set up (and request its weights) meanwhile
    ib::pdl_wait();
    const int half = head_dim / 2, groups = half / 8;
    const int units = (n_heads + 2 * n_kv) * groups;
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_tokens * units) return;
    const int64_t t = i / units;
    const int u = int(i - t * units);
    const int head = u / groups, j = (u - head * groups) * 8;
    const int pos = positions[t];
    const bf16* row = qkv + t * int64_t(n_heads + 2 * n_kv) * head_dim + int64_t(head) * head_dim;
    uint4 a = *reinterpret_cast<const uint4*>(row + j), b = *reinterpret_cast<const uint4*>(row + j + half);
    const bool is_v = head >= n_heads + n_kv;
    if (!is_v && cos_t) {
        const float4* c4 = reinterpret_cast<const float4*>(cos_t + int64_t(pos) * half + j);
        const float4* s4 = reinterpret_cast<const float4*>(sin_t + int64_t(pos) * half + j);
        const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        bf16* pa = reinterpret_cast<bf16*>(&a);
        bf16* pb = reinterpret_cast<bf16*>(&b);
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float x1 = __bfloat162float(pa[e]), x2 = __bfloat162float(pb[e]);
            pa[e] = __float2bfloat16_rn(x1 * c[e] - x2 * sn[e]);
            pb[e] = __float2bfloat16_rn(x2 * c[e] + x1 * sn[e]);
        }
    }
    bf16* dst;
    if (head < n_heads) {
        dst = q_out + t * int64_t(n_heads) * head_dim + int64_t(head) * head_dim;
    } else {
        if (!write_cache) return;
        const int kvh = is_v ? head - n_heads - n_kv : head - n_heads;
        const int page = block_table[int64_t(token_seg[t]) * max_blocks + pos / page_size];
        if (page < 0 || page >= n_pages) {
            if (status) atomicExch(status, 2);
            return;
        }
        dst = (is_v ? v_cache : k_cache) + ((int64_t(page) * n_kv + kvh) * page_size + pos % page_size) * head_dim;
    }
    *reinterpret_cast<uint4*>(dst + j) = a;
    *reinterpret_cast<uint4*>(dst + j + half) = b;
}

// ------------------------------------------------------------------------------------------------
// Attention over the paged cache, one block of 128 threads per (token, query head).
// The query at position p of its request reads keys lo..p, lo = max(0, p - window + 1) (window 0 =
// all), from the pages of its request's block-table row. Keys are taken in tiles of 128 positions
// aligned to absolute multiples of 128, softmax is computed online over the tiles, so the result
// depends on (lo, p) only.
constexpr int AT = 128;

template <typename T>
__global__ void __launch_bounds__(AT)
attention_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                 const int* __restrict__ block_table, int64_t max_blocks, const int* __restrict__ token_seg,
                 const int* __restrict__ positions, T* __restrict__ out, int n_heads, int n_kv, int head_dim,
                 int page_size, int window, float scale, int64_t n_pages, int* status) {
    ib::pdl_wait();
    extern __shared__ float smem[];
    float* qs = smem;                      // [head_dim]
    float* ps = qs + head_dim;             // [AT]
    int64_t* rowoff = reinterpret_cast<int64_t*>(ps + AT);   // [AT] element offset of each key row
    __shared__ float red[32];

    const int64_t t = blockIdx.x;
    const int h = blockIdx.y;
    const int g = h / (n_heads / n_kv);
    const int tid = threadIdx.x;
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* table = block_table + int64_t(token_seg[t]) * max_blocks;

    for (int d = tid; d < head_dim; d += AT) qs[d] = ib::to_f32(q[(t * n_heads + h) * head_dim + d]);
    float m = -INFINITY, l = 0.0f, acc0 = 0.0f, acc1 = 0.0f;
    __syncthreads();

    for (int tile = (lo / AT) * AT; tile <= pos; tile += AT) {
        const int j = tile + tid;
        const bool valid = j >= lo && j <= pos;
        float s = -INFINITY;
        if (valid) {
            const int page = table[j / page_size];
            if (page < 0 || page >= n_pages) {
                if (status) atomicExch(status, 3);
                rowoff[tid] = 0;
            } else {
                const int64_t off = ((int64_t(page) * n_kv + g) * page_size + j % page_size) * head_dim;
                rowoff[tid] = off;
                const T* kr = k_cache + off;
                float dot = 0.0f;
                for (int d = 0; d < head_dim; d++) dot = fmaf(qs[d], ib::to_f32(kr[d]), dot);
                s = dot * scale;
            }
        }
        const float tile_max = ib::block_max(s, red);
        const float m_new = fmaxf(m, tile_max);
        const float p = valid && s > -INFINITY ? expf(s - m_new) : 0.0f;
        ps[tid] = p;
        const float tile_sum = ib::block_sum(p, red);   // contains __syncthreads: ps and rowoff are visible
        const float corr = m == -INFINITY ? 0.0f : expf(m - m_new);
        l = l * corr + tile_sum;
        acc0 *= corr;
        acc1 *= corr;
        const int jj0 = max(lo, tile) - tile, jj1 = min(pos, tile + AT - 1) - tile;
        for (int jj = jj0; jj <= jj1; jj++) {
            const float pj = ps[jj];
            const T* vr = v_cache + rowoff[jj];
            if (tid < head_dim) acc0 = fmaf(pj, ib::to_f32(vr[tid]), acc0);
            if (tid + AT < head_dim) acc1 = fmaf(pj, ib::to_f32(vr[tid + AT]), acc1);
        }
        m = m_new;
        __syncthreads();
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    T* o = out + (t * n_heads + h) * head_dim;
    if (tid < head_dim) o[tid] = ib::from_f32<T>(acc0 * inv);
    if (tid + AT < head_dim) o[tid + AT] = ib::from_f32<T>(acc1 * inv);
}

// ------------------------------------------------------------------------------------------------
// SwiGLU: out[t, i] = silu(gate) * up, silu(g) = g / (1 + exp(-g)); input rows are [gate | up], or with
// `interleave8` blocks of 16: gate features 8b..8b+7, then up features 8b..8b+7.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int64_t n_tokens, int64_t inter,
                              int interleave8) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_tokens * inter) return;
    const int64_t t = i / inter, c = i - t * inter;
    const int64_t gi = interleave8 ? (c >> 3) * 16 + (c & 7) : c;
    const int64_t ui = interleave8 ? gi + 8 : inter + c;
    const float g = ib::to_f32(gate_up[t * 2 * inter + gi]);
    const float u = ib::to_f32(gate_up[t * 2 * inter + ui]);
    out[i] = ib::from_f32<T>(g / (1.0f + expf(-g)) * u);
}

// ------------------------------------------------------------------------------------------------
// Sampling: temperature 0 -> first index of the maximum. Otherwise argmax of logit/T + Gumbel noise,
// the noise a hash of (seed, step, index): an exact sample of softmax(logits/T) that needs no state
// and does not depend on the batch (kernels/ops/ops.cuh:26-38, kernels/ops/batch.cu:450-478).
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float hash_uniform(uint64_t seed, uint64_t step, uint64_t v) {
    uint64_t x = mix64(seed + 0x9E3779B97F4A7C15ull * (step + 1));
    x = mix64(x ^ (v + 0x632BE59BD9B4E019ull));
    return (float((x >> 40) & 0xFFFFFF) + 0.5f) / 16777216.0f;
}

// A row is shared by a thread-block cluster of SAMPLE_CLUSTER CTAs (each takes a contiguous slice of the vocabulary);
// every CTA leaves its best (value, index) in the first CTA's shared memory, which picks among them. The maximum
// with ties to the lowest index is the same in whatever order the candidates meet.
constexpr int SAMPLE_CLUSTER = 8;
constexpr int SAMPLE_THREADS = 512;

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int64_t vocab, const float* __restrict__ temperature,
              const int64_t* __restrict__ seed, const int64_t* __restrict__ step,
              int* __restrict__ out, int* feedback, const int64_t* __restrict__ slots) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float sv[SAMPLE_THREADS / 32];
    __shared__ int si[SAMPLE_THREADS / 32];
    __shared__ float cv[SAMPLE_CLUSTER];                    // candidates of the cluster's CTAs (used in the first CTA)
    __shared__ int ci[SAMPLE_CLUSTER];
    const int rank = int(cluster.block_rank());
    const int b = blockIdx.x / SAMPLE_CLUSTER;
    ib::pdl_wait();
    const float* row = logits + int64_t(b) * vocab;
    const float T = temperature[b];
    const uint64_t sd = uint64_t(seed[b]), stp = uint64_t(step[b]);
    float best = -INFINITY;
    int besti = 0x7fffffff;
    auto take = [&](float x, int64_t v) {
        if (T > 0.0f) x = x / T - logf(-logf(hash_uniform(sd, stp, uint64_t(v))));
        if (x > best || (x == best && v < besti)) { best = x; besti = int(v); }
    };
    if ((vocab & 3) == 0) {
        // rows are 16-byte aligned: four logits per load, two loads in flight per thread
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const int64_t n4 = vocab >> 2, per = (n4 + SAMPLE_CLUSTER - 1) / SAMPLE_CLUSTER;
        const int64_t lo = per * rank, hi = lo + per < n4 ? lo + per : n4;
        int64_t i = lo + threadIdx.x;
        for (; i + blockDim.x < hi; i += 2 * blockDim.x) {
            const float4 a = row4[i], c = row4[i + blockDim.x];
            take(a.x, 4 * i); take(a.y, 4 * i + 1); take(a.z, 4 * i + 2); take(a.w, 4 * i + 3);
            const int64_t j = i + blockDim.x;
            take(c.x, 4 * j); take(c.y, 4 * j + 1); take(c.z, 4 * j + 2); take(c.w, 4 * j + 3);
        }
        if (i < hi) {
            const float4 a = row4[i];
            take(a.x, 4 * i); take(a.y, 4 * i + 1); take(a.z, 4 * i + 2); take(a.w, 4 * i + 3);
        }
    } else {
        const int64_t per = (vocab + SAMPLE_CLUSTER - 1) / SAMPLE_CLUSTER;
        const int64_t lo = per * rank, hi = lo + per < vocab ? lo + per : vocab;
        for (int64_t v = lo + threadIdx.x; v < hi; v += blockDim.x) take(row[v], v);
    }
    auto better = [](float ov, int oi, float v, int i) { return ov > v || (ov == v && oi < i); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (better(ov, oi, best, besti)) { best = ov; besti = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = besti; }
    __syncthreads();
    if (warp == 0) {
        best = lane < SAMPLE_THREADS / 32 ? sv[lane] : -INFINITY;
        besti = lane < SAMPLE_THREADS / 32 ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
            if (better(ov, oi, best, besti)) { best = ov; besti = oi; }
        }
        if (lane == 0) {
            *cluster.map_shared_rank(&cv[rank], 0) = best;
            *cluster.map_shared_rank(&ci[rank], 0) = besti;
        }
    }
    cluster.sync();                                          // every CTA's candidate has arrived in the first CTA
    if (rank == 0 && threadIdx.x == 0) {
        best = cv[0]; besti = ci[0];
        for (int r = 1; r < SAMPLE_CLUSTER; r++)
            if (better(cv[r], ci[r], best, besti)) { best = cv[r]; besti = ci[r]; }
        const int tok = besti == 0x7fffffff ? 0 : besti;
        out[b] = tok;
        if (feedback) feedback[slots[b]] = tok;          // stays on the device for the request's next step
    }
}

// Sampling with top-k / top-p filters (src/sampler.cpp:8-63): x = logit / T; keep the k largest x; among
// those keep the smallest set of largest probabilities whose mass reaches top_p; sample among the kept
// by argmax of x + Gumbel noise. Both thresholds are found by bisection over an order-preserving integer
// image of x, each probe a fixed-order block reduction, so the result is the same on every run.
__device__ __forceinline__ uint32_t ordered_key(float x) {
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(1024)
sample_filtered_kernel(const float* __restrict__ logits, int64_t vocab, const float* __restrict__ temperature,
                       const int64_t* __restrict__ seed, const int64_t* __restrict__ step,
                       const int64_t* __restrict__ top_k, const float* __restrict__ top_p, int* __restrict__ out,
                       int* feedback, const int64_t* __restrict__ slots) {
    ib::pdl_wait();
    __shared__ float red[32];
    __shared__ float sv[1024];
    __shared__ int si[1024];
    const int b = blockIdx.x;
    const float* row = logits + int64_t(b) * vocab;
    const float T = temperature[b];
    const float invT = T > 0.0f ? 1.0f / T : 1.0f;
    uint32_t thr = 0u;                                   // keep keys >= thr
    float mx = -INFINITY;
    for (int64_t v = threadIdx.x; v < vocab; v += blockDim.x) mx = fmaxf(mx, row[v] * invT);
    mx = ib::block_max(mx, red);
    if (T > 0.0f) {
        const int64_t k = top_k[b];
        if (k > 0 && k < vocab) {
            uint32_t lo = 0u, hi = 0xFFFFFFFFu;
            while (lo < hi) {
                const uint32_t mid = lo + (hi - lo) / 2u + ((hi - lo) & 1u);
                float cnt = 0.0f;
                for (int64_t v = threadIdx.x; v < vocab; v += blockDim.x) cnt += ordered_key(row[v] * invT) >= mid ? 1.0f : 0.0f;
                cnt = ib::block_sum(cnt, red);
                if (cnt >= float(k)) lo = mid; else hi = mid - 1u;
            }
            thr = lo;
        }
        const float p = top_p[b];
        if (p < 1.0f) {
            float Z = 0.0f;
            for (int64_t v = threadIdx.x; v < vocab; v += blockDim.x) {
                const float x = row[v] * invT;
                if (ordered_key(x) >= thr) Z += expf(x - mx);
            }
            Z = ib::block_sum(Z, red);
            const float want = p * Z;
            uint32_t lo = thr, hi = 0xFFFFFFFFu;
            while (lo < hi) {
                const uint32_t mid = lo + (hi - lo) / 2u + ((hi - lo) & 1u);
                float mass = 0.0f;
                for (int64_t v = threadIdx.x; v < vocab; v += blockDim.x) {
                    const float x = row[v] * invT;
                    if (ordered_key(x) >= mid) mass += expf(x - mx);
                }
                mass = ib::block_sum(mass, red);
                if (mass >= want) lo = mid; else hi = mid - 1u;
            }
            thr = lo;
        }
    }
    float best = -INFINITY;
    int besti = 0x7fffffff;
    for (int64_t v = threadIdx.x; v < vocab; v += blockDim.x) {
        float x = row[v] * invT;
        if (T > 0.0f) {
            if (ordered_key(x) < thr) continue;
            x = row[v] / T - logf(-logf(hash_uniform(uint64_t(seed[b]), uint64_t(step[b]), uint64_t(v))));
        } else {
            x = row[v];
        }
        if (x > best || (x == best && v < besti)) { best = x; besti = int(v); }
    }
    sv[threadIdx.x] = best;
    si[threadIdx.x] = besti;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = sv[threadIdx.x + s];
            const int oi = si[threadIdx.x + s];
            if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) {
                sv[threadIdx.x] = ov;
                si[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const int tok = si[0] == 0x7fffffff ? 0 : si[0];
        out[b] = tok;
        if (feedback) feedback[slots[b]] = tok;          // stays on the device for the request's next step
    }
}

inline unsigned blocks_for(int64_t n, int threads) { return unsigned((n + threads - 1) / threads); }

}  // namespace

// ================================================================================================
// C entry points. dtype arguments: 0 = float, 1 = bfloat16.

IB_EXPORT int ib_embedding(const void* table, int table_dtype, const int* ids, int64_t n_tokens, int64_t hidden,
                           int64_t vocab, float* out, int* status, const int* feedback, const int* token_seg,
                           const int* seg_slot, float scale, cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    const int64_t n = n_tokens * hidden;
    if (table_dtype == IB_F32)
        IB_LAUNCH(embedding_kernel<float>, blocks_for(n, 256), 256, 0, (const float*)table, ids, n_tokens, hidden, vocab, out, status, feedback, token_seg, seg_slot, scale);
    else if (table_dtype == IB_BF16)
        IB_LAUNCH(embedding_kernel<bf16>, blocks_for(n, 256), 256, 0, (const bf16*)table, ids, n_tokens, hidden, vocab, out, status, feedback, token_seg, seg_slot, scale);
    else
        return ib::fail(IB_ERR_ARG, "ib_embedding: unknown table dtype %d", table_dtype);
    return ib::check_launch("ib_embedding");
}

IB_EXPORT int ib_rmsnorm(const float* x, const float* w, float eps, int64_t n_rows, int64_t hidden, const int* rows,
                         void* out, int out_dtype, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (hidden <= 0) return ib::fail(IB_ERR_ARG, "ib_rmsnorm: hidden must be positive");
    const int threads = hidden >= 1024 ? 256 : 128;
    // (the choice does not look at the number of rows: a row's result must not depend on what else is in the step)
    if (hidden % 4 == 0 && !((uintptr_t(x) | uintptr_t(w) | uintptr_t(out)) & 15)) {
        if (out_dtype == IB_F32)
            IB_LAUNCH(rmsnorm_vec_kernel<float>, unsigned(n_rows), NORM_THREADS, 0, x, w, eps, hidden, rows, (float*)out);
        else if (out_dtype == IB_BF16)
            IB_LAUNCH(rmsnorm_vec_kernel<bf16>, unsigned(n_rows), NORM_THREADS, 0, x, w, eps, hidden, rows, (bf16*)out);
        else
            return ib::fail(IB_ERR_ARG, "ib_rmsnorm: unknown output dtype %d", out_dtype);
        return ib::check_launch("ib_rmsnorm");
    }
    if (out_dtype == IB_F32)
        IB_LAUNCH(rmsnorm_kernel<float>, unsigned(n_rows), threads, 0, x, w, eps, hidden, rows, (float*)out);
    else if (out_dtype == IB_BF16)
        IB_LAUNCH(rmsnorm_kernel<bf16>, unsigned(n_rows), threads, 0, x, w, eps, hidden, rows, (bf16*)out);
    else
        return ib::fail(IB_ERR_ARG, "ib_rmsnorm: unknown output dtype %d", out_dtype);
    return ib::check_launch("ib_rmsnorm");
}

IB_EXPORT int ib_linear_plain(const void* x, const void* w, const float* bias, const float* residual, void* out,
                              int64_t M, int64_t N, int64_t K, int in_dtype, int out_dtype, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IB_OK;
    if (K <= 0) return ib::fail(IB_ERR_ARG, "ib_linear_plain: K must be positive");
    const dim3 grid{unsigned((N + LT - 1) / LT), unsigned((M + LT - 1) / LT), 1u};
    if (grid.y > 65535) return ib::fail(IB_ERR_ARG, "ib_linear_plain: too many rows (%lld)", (long long)M);
    if (in_dtype == IB_F32 && out_dtype == IB_F32)
        IB_LAUNCH((linear_kernel<float, float>), grid, 256, 0, (const float*)x, (const float*)w, bias, residual, (float*)out, M, N, K);
    else if (in_dtype == IB_BF16 && out_dtype == IB_BF16)
        IB_LAUNCH((linear_kernel<bf16, bf16>), grid, 256, 0, (const bf16*)x, (const bf16*)w, bias, residual, (bf16*)out, M, N, K);
    else if (in_dtype == IB_BF16 && out_dtype == IB_F32)
        IB_LAUNCH((linear_kernel<bf16, float>), grid, 256, 0, (const bf16*)x, (const bf16*)w, bias, residual, (float*)out, M, N, K);
    else
        return ib::fail(IB_ERR_ARG, "ib_linear_plain: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
    return ib::check_launch("ib_linear_plain");
}

IB_EXPORT int ib_rope_kv_write(const void* qkv, const float* cos_t, const float* sin_t, const int* positions,
                               const int* token_seg, const int* block_table, int64_t max_blocks, void* q_out,
                               void* k_cache, void* v_cache, int64_t n_tokens, int n_heads, int n_kv, int head_dim,
                               int page_size, int write_cache, int64_t n_pages, int dtype, int* status,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    if (head_dim <= 0 || head_dim % 2) return ib::fail(IB_ERR_ARG, "ib_rope_kv_write: head_dim %d must be even", head_dim);
    if (n_heads <= 0 || n_kv <= 0 || page_size <= 0) return ib::fail(IB_ERR_ARG, "ib_rope_kv_write: bad sizes");
    const int64_t n = n_tokens * (n_heads + 2 * n_kv) * (head_dim / 2);
    const uintptr_t bases = uintptr_t(qkv) | uintptr_t(q_out) | uintptr_t(k_cache) | uintptr_t(v_cache) | uintptr_t(cos_t) | uintptr_t(sin_t);
    if (dtype == IB_BF16 && head_dim % 16 == 0 && !(bases & 15)) {
        IB_LAUNCH(rope_kv_write_vec_kernel, blocks_for(n / 8, 256), 256, 0, (const bf16*)qkv, cos_t, sin_t, positions, token_seg, block_table, max_blocks,
            (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, n_tokens, n_heads, n_kv, head_dim, page_size, write_cache, n_pages, status);
        return ib::check_launch("ib_rope_kv_write");
    }
    if (dtype == IB_F32)
        IB_LAUNCH(rope_kv_write_kernel<float>, blocks_for(n, 256), 256, 0, (const float*)qkv, cos_t, sin_t, positions, token_seg, block_table, max_blocks, (float*)q_out,
            (float*)k_cache, (float*)v_cache, n_tokens, n_heads, n_kv, head_dim, page_size, write_cache, n_pages, status);
    else if (dtype == IB_BF16)
        IB_LAUNCH(rope_kv_write_kernel<bf16>, blocks_for(n, 256), 256, 0, (const bf16*)qkv, cos_t, sin_t, positions, token_seg, block_table, max_blocks, (bf16*)q_out,
            (bf16*)k_cache, (bf16*)v_cache, n_tokens, n_heads, n_kv, head_dim, page_size, write_cache, n_pages, status);
    else
        return ib::fail(IB_ERR_ARG, "ib_rope_kv_write: unknown dtype %d", dtype);
    return ib::check_launch("ib_rope_kv_write");
}

// The largest head size the plain attention kernel takes (parts ask at construction, so that a configuration the
// kernels cannot serve is refused when the model is built, not at its first step).
IB_EXPORT int ib_attention_plain_max_head_dim() { return 2 * AT; }

IB_EXPORT int ib_attention_plain(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                 int64_t max_blocks, const int* token_seg, const int* positions, void* out,
                                 int64_t n_tokens, int n_heads, int n_kv, int head_dim, int page_size, int window,
                                 float scale, int64_t n_pages, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    if (head_dim <= 0 || head_dim > 2 * AT)
        return ib::fail(IB_ERR_ARG, "ib_attention_plain: head_dim %d is outside 1..%d", head_dim, 2 * AT);
    if (n_kv <= 0 || n_heads % n_kv) return ib::fail(IB_ERR_ARG, "ib_attention_plain: heads %d not a multiple of kv heads %d", n_heads, n_kv);
    if (n_heads > 65535) return ib::fail(IB_ERR_ARG, "ib_attention_plain: too many heads");
    const dim3 grid{unsigned(n_tokens), unsigned(n_heads), 1u};
    const size_t smem = size_t(head_dim + AT) * sizeof(float) + AT * sizeof(int64_t) + 8;
    if (dtype == IB_F32)
        IB_LAUNCH(attention_kernel<float>, grid, AT, smem, (const float*)q, (const float*)k_cache, (const float*)v_cache,
            block_table, max_blocks, token_seg, positions, (float*)out, n_heads, n_kv, head_dim, page_size, window, scale, n_pages, status);
    else if (dtype == IB_BF16)
        IB_LAUNCH(attention_kernel<bf16>, grid, AT, smem, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
            block_table, max_blocks, token_seg, positions, (bf16*)out, n_heads, n_kv, head_dim, page_size, window, scale, n_pages, status);
    else
        return ib::fail(IB_ERR_ARG, "ib_attention_plain: unknown dtype %d", dtype);
    return ib::check_launch("ib_attention_plain");
}

IB_EXPORT int ib_swiglu(const void* gate_up, void* out, int64_t n_tokens, int64_t inter, int dtype, int interleave8,
                        cudaStream_t stream) {
    if (n_tokens <= 0 || inter <= 0) return IB_OK;
    if (interleave8 && inter % 8) return ib::fail(IB_ERR_ARG, "ib_swiglu: interleaved rows need a multiple of 8 features");
    const int64_t n = n_tokens * inter;
    if (dtype == IB_F32)
        IB_LAUNCH(swiglu_kernel<float>, blocks_for(n, 256), 256, 0, (const float*)gate_up, (float*)out, n_tokens, inter, interleave8);
    else if (dtype == IB_BF16)
        IB_LAUNCH(swiglu_kernel<bf16>, blocks_for(n, 256), 256, 0, (const bf16*)gate_up, (bf16*)out, n_tokens, inter, interleave8);
    else
        return ib::fail(IB_ERR_ARG, "ib_swiglu: unknown dtype %d", dtype);
    return ib::check_launch("ib_swiglu");
}

IB_EXPORT int ib_sample(const float* logits, int64_t n_rows, int64_t vocab, const float* temperature,
                        const int64_t* seed, const int64_t* step, int* out, int* feedback, const int64_t* slots,
                        cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (vocab <= 0 || vocab >= 0x7fffffff) return ib::fail(IB_ERR_ARG, "ib_sample: vocabulary %lld out of range", (long long)vocab);
    const int rc = ib::launch("sample_kernel", sample_kernel, dim3(unsigned(n_rows) * SAMPLE_CLUSTER), dim3(SAMPLE_THREADS), 0, stream,
                              unsigned(SAMPLE_CLUSTER), logits, vocab, temperature, seed, step, out, feedback, slots);
    if (rc) return rc;
    return ib::check_launch("ib_sample");
}

IB_EXPORT int ib_sample_filtered(const float* logits, int64_t n_rows, int64_t vocab, const float* temperature,
                                 const int64_t* seed, const int64_t* step, const int64_t* top_k, const float* top_p,
                                 int* out, int* feedback, const int64_t* slots, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (vocab <= 0 || vocab >= 0x7fffffff) return ib::fail(IB_ERR_ARG, "ib_sample_filtered: vocabulary %lld out of range", (long long)vocab);
    IB_LAUNCH(sample_filtered_kernel, unsigned(n_rows), 1024, 0, logits, vocab, temperature, seed, step, top_k, top_p, out, feedback, slots);
    return ib::check_launch("ib_sample_filtered");
}
