// Blocks whose sublayers all read one norm's rows and whose results enter the stream in one sum.
//
// stream_add: h += coef * sum_i t_i / sqrt(mean(t_i^2) + eps) * w_i + sum_j p_j   (h float32, in place),
//             up to two normed terms (a pair of mixers side by side) and up to three plain ones; the new
//             stream also leaves in bfloat16 where the next product wants it so.
// polynorm:   a N(z) + b N(z^2) + c N(z^3) + e over a row, N(y) = y / sqrt(mean(y^2) + eps), powers element
//             by element; one pass gathers the three sums of squares, one writes.
// side_gate:  gelu_tanh(u) * table[token]: the gate of a per-token input.
//
// stream_inject: h[t] += e[t] + r: a second stream and one row for all tokens (either may be absent), float32.
//
// sum_partials: the planes of a split-K product added up and rounded once (for readers that take no partial sums).
//
// Sums, norms and the stream are float32 whatever the terms' dtype.  Every term may arrive as float32 partial sums
// [splits][T][width] of a split-K product (planes `plane` elements apart); the kernels add the planes up as they read.
#include "common.cuh"

namespace {

constexpr int MAX_NORMED = 2, MAX_PLAIN = 3;

__device__ __forceinline__ float block_sum(float v, float* part) {
    // part: 33 floats of shared memory
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) part[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? part[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) part[32] = t;
    }
    __syncthreads();
    return part[32];
}

__device__ __forceinline__ float load_as(const void* p, int dtype, size_t at) {
    return dtype == TL_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[at]) : reinterpret_cast<const float*>(p)[at];
}

// the sum over the planes of a split-K product (or the one plane there is)
__device__ __forceinline__ float load_sum(const void* p, int dtype, int splits, long long plane, size_t at) {
    float v = load_as(p, dtype, at);
    for (int s = 1; s < splits; ++s) v += reinterpret_cast<const float*>(p)[(size_t)s * plane + at];
    return v;
}

struct SumParams {
    float* h;                         // [T][dim]
    const void* normed[MAX_NORMED];   // [T][dim] each
    const float* weight[MAX_NORMED];  // [dim] each
    int normed_dtype[MAX_NORMED], normed_splits[MAX_NORMED];
    long long normed_plane[MAX_NORMED];
    const void* plain[MAX_PLAIN];     // [T][dim] each
    int plain_dtype[MAX_PLAIN], plain_splits[MAX_PLAIN];
    long long plain_plane[MAX_PLAIN];
    int n_normed, n_plain, dim;
    float coef, eps;
    __nv_bfloat16* rows;              // [T][dim] or null
};

// a CTA per token
__global__ void stream_add_kernel(const SumParams p) {
    __shared__ float part[33];
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t base = (size_t)blockIdx.x * p.dim;
    float r[MAX_NORMED];
#pragma unroll
    for (int i = 0; i < MAX_NORMED; ++i) {
        r[i] = 0.f;
        if (i < p.n_normed) {
            float ssq = 0.f;
            for (int d = threadIdx.x; d < p.dim; d += blockDim.x) {
                const float v = load_sum(p.normed[i], p.normed_dtype[i], p.normed_splits[i], p.normed_plane[i], base + d);
                ssq = fmaf(v, v, ssq);
            }
            r[i] = rsqrtf(block_sum(ssq, part) / (float)p.dim + p.eps);
        }
    }
    for (int d = threadIdx.x; d < p.dim; d += blockDim.x) {
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_NORMED; ++i)
            if (i < p.n_normed)
                m += load_sum(p.normed[i], p.normed_dtype[i], p.normed_splits[i], p.normed_plane[i], base + d) * r[i] * p.weight[i][d];
        float v = p.h[base + d] + p.coef * m;
#pragma unroll
        for (int i = 0; i < MAX_PLAIN; ++i)
            if (i < p.n_plain) v += load_sum(p.plain[i], p.plain_dtype[i], p.plain_splits[i], p.plain_plane[i], base + d);
        p.h[base + d] = v;
        if (p.rows != nullptr) p.rows[base + d] = __float2bfloat16_rn(v);
    }
}

template <typename TI, typename TO>
__global__ void polynorm_kernel(const TI* __restrict__ z, int splits, long long plane, const float* __restrict__ coef,
                                TO* __restrict__ out, int width, float eps) {
    __shared__ float part[33];
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t base = (size_t)blockIdx.x * width;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float v = to_float(z[base + d]);
        for (int sp = 1; sp < splits; ++sp) v += to_float(z[(size_t)sp * plane + base + d]);
        const float v2 = v * v, v3 = v2 * v;
        s2 += v2;
        s4 = fmaf(v2, v2, s4);
        s6 = fmaf(v3, v3, s6);
    }
    const float inv = 1.f / (float)width;
    const float r1 = rsqrtf(block_sum(s2, part) * inv + eps);
    const float r2 = rsqrtf(block_sum(s4, part) * inv + eps);
    const float r3 = rsqrtf(block_sum(s6, part) * inv + eps);
    const float a = coef[0] * r1, b = coef[1] * r2, c = coef[2] * r3, e = coef[3];
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float v = to_float(z[base + d]);
        for (int sp = 1; sp < splits; ++sp) v += to_float(z[(size_t)sp * plane + base + d]);
        const float v2 = v * v;
        out[base + d] = from_float<TO>(a * v + b * v2 + c * (v2 * v) + e);
    }
}

template <typename TI, typename TT, typename TO>
__global__ void side_gate_kernel(const TI* __restrict__ u, int splits, long long plane, const int* __restrict__ token_ids,
                                 const TT* __restrict__ table, TO* __restrict__ out, long long total, int width, int vocab) {
    grid_launch_dependents();
    grid_dependency_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / width;
        const int c = (int)(i - t * width);
        int tok = token_ids[t];
        if (!TL_CHECK(tok >= 0 && tok < vocab, TL_DBG_TOKEN_ID)) tok = 0;
        float x = to_float(u[i]);
        for (int sp = 1; sp < splits; ++sp) x += to_float(u[(size_t)sp * plane + i]);
        const float g = 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
        out[i] = from_float<TO>(g * to_float(table[(size_t)tok * width + c]));
    }
}

__global__ void stream_inject_kernel(float* __restrict__ h, const float* __restrict__ rows, const float* __restrict__ row,
                                     long long total, int width) {
    grid_launch_dependents();
    grid_dependency_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float v = h[i];
        if (rows != nullptr) v += rows[i];
        if (row != nullptr) v += row[i % width];
        h[i] = v;
    }
}

template <typename TO>
__global__ void sum_partials_kernel(const float* __restrict__ parts, int splits, long long plane, TO* __restrict__ out, long long total) {
    grid_launch_dependents();
    grid_dependency_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float v = parts[i];
        for (int sp = 1; sp < splits; ++sp) v += parts[(size_t)sp * plane + i];
        out[i] = from_float<TO>(v);
    }
}

// threads of a CTA that owns a row: few rows (a decode step, whose terms are often many planes of partial sums) are
// all the parallelism there is, so a row gets as many threads as it has pairs of columns
int row_threads(int width, int n_rows) {
    if (n_rows <= 64) {
        const int t = ((width / 2 + 31) / 32) * 32;
        return t > 1024 ? 1024 : t < 128 ? 128 : t;
    }
    return width >= 2048 ? 512 : width >= 512 ? 256 : 128;
}

}  // namespace

// h: float32 [n_tokens][dim], updated in place; normed / plain: arrays of n_normed (<= 2) / n_plain (<= 3) pointers to
// [splits][n_tokens][dim] tensors with their dtype codes, plane counts (1: no partial sums; more only in float32) and
// the planes' distance in elements; weights: n_normed pointers to float32 [dim]; rows: bfloat16 [n_tokens][dim] or null.
extern "C" int tl_stream_add(float* h, const void* const* normed, const int* normed_dtype, const int* normed_splits,
                             const long long* normed_plane, const float* const* weights, int n_normed, const void* const* plain,
                             const int* plain_dtype, const int* plain_splits, const long long* plain_plane, int n_plain, float coef,
                             float eps, void* rows, int n_tokens, int dim, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (dim <= 0 || n_normed < 0 || n_normed > MAX_NORMED || n_plain < 0 || n_plain > MAX_PLAIN) return TL_BAD_SIZE;
    SumParams p = {};
    p.h = h; p.n_normed = n_normed; p.n_plain = n_plain; p.dim = dim; p.coef = coef; p.eps = eps;
    p.rows = reinterpret_cast<__nv_bfloat16*>(rows);
    for (int i = 0; i < n_normed; ++i) {
        if (normed_dtype[i] != TL_F32 && normed_dtype[i] != TL_BF16) return TL_BAD_DTYPE;
        if (normed_splits[i] < 1 || (normed_splits[i] > 1 && normed_dtype[i] != TL_F32)) return TL_BAD_SIZE;
        p.normed[i] = normed[i]; p.normed_dtype[i] = normed_dtype[i]; p.weight[i] = weights[i];
        p.normed_splits[i] = normed_splits[i]; p.normed_plane[i] = normed_plane[i];
    }
    for (int i = 0; i < n_plain; ++i) {
        if (plain_dtype[i] != TL_F32 && plain_dtype[i] != TL_BF16) return TL_BAD_DTYPE;
        if (plain_splits[i] < 1 || (plain_splits[i] > 1 && plain_dtype[i] != TL_F32)) return TL_BAD_SIZE;
        p.plain[i] = plain[i]; p.plain_dtype[i] = plain_dtype[i]; p.plain_splits[i] = plain_splits[i]; p.plain_plane[i] = plain_plane[i];
    }
    return (int)tl_launch(stream_add_kernel, dim3(n_tokens), dim3(row_threads(dim, n_tokens)), 0, (cudaStream_t)stream, p);
}

// z: [splits][n_tokens][width]; coef: float32 [4] = (a, b, c, e); out: [n_tokens][width].
extern "C" int tl_polynorm(const void* z, int in_dtype, int splits, long long plane, const float* coef, void* out, int out_dtype,
                           int n_tokens, int width, float eps, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (width <= 0 || splits < 1 || (splits > 1 && in_dtype != TL_F32)) return TL_BAD_SIZE;
    const dim3 grid(n_tokens), block(row_threads(width, n_tokens));
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == TL_F32 && out_dtype == TL_F32)
        return (int)tl_launch(polynorm_kernel<float, float>, grid, block, 0, s, (const float*)z, splits, plane, coef, (float*)out, width, eps);
    if (in_dtype == TL_F32 && out_dtype == TL_BF16)
        return (int)tl_launch(polynorm_kernel<float, __nv_bfloat16>, grid, block, 0, s, (const float*)z, splits, plane, coef, (__nv_bfloat16*)out, width, eps);
    if (in_dtype == TL_BF16 && out_dtype == TL_BF16)
        return (int)tl_launch(polynorm_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)z, splits, plane, coef,
                              (__nv_bfloat16*)out, width, eps);
    return TL_BAD_DTYPE;
}

// u: [splits][n_tokens][width] of u_dtype (float32 where splits > 1); table: [vocab][width] and out: [n_tokens][width] of dtype.
extern "C" int tl_side_gate(const void* u, int u_dtype, int splits, long long plane, const int* token_ids, const void* table, void* out,
                            int dtype, int n_tokens, int width, int vocab, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (width <= 0 || vocab <= 0 || splits < 1 || (splits > 1 && u_dtype != TL_F32)) return TL_BAD_SIZE;
    const long long total = (long long)n_tokens * width;
    const dim3 grid((unsigned)((total + 255) / 256 > 148 * 8 ? 148 * 8 : (total + 255) / 256)), block(256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == TL_F32 && u_dtype == TL_F32)
        return (int)tl_launch(side_gate_kernel<float, float, float>, grid, block, 0, s, (const float*)u, splits, plane, token_ids,
                              (const float*)table, (float*)out, total, width, vocab);
    if (dtype == TL_BF16 && u_dtype == TL_F32)
        return (int)tl_launch(side_gate_kernel<float, __nv_bfloat16, __nv_bfloat16>, grid, block, 0, s, (const float*)u, splits, plane,
                              token_ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, total, width, vocab);
    if (dtype == TL_BF16 && u_dtype == TL_BF16)
        return (int)tl_launch(side_gate_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)u,
                              splits, plane, token_ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, total, width, vocab);
    return TL_BAD_DTYPE;
}

// parts: float32 [splits][total], planes `plane` elements apart; out: [total] of out_dtype.
extern "C" int tl_sum_partials(const float* parts, int splits, long long plane, void* out, int out_dtype, long long total, void* stream) {
    if (total <= 0) return TL_OK;
    if (splits < 1) return TL_BAD_SIZE;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    const dim3 grid((unsigned)blocks), block(256);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == TL_F32) return (int)tl_launch(sum_partials_kernel<float>, grid, block, 0, s, parts, splits, plane, (float*)out, total);
    if (out_dtype == TL_BF16)
        return (int)tl_launch(sum_partials_kernel<__nv_bfloat16>, grid, block, 0, s, parts, splits, plane, (__nv_bfloat16*)out, total);
    return TL_BAD_DTYPE;
}

// h: float32 [n_tokens][width], updated in place; rows: float32 [n_tokens][width] or null; row: float32 [width] or null
extern "C" int tl_stream_inject(float* h, const float* rows, const float* row, int n_tokens, int width, void* stream) {
    if (n_tokens <= 0 || width <= 0) return TL_OK;
    const long long total = (long long)n_tokens * width;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    return (int)tl_launch(stream_inject_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, h, rows, row, total, width);
}
