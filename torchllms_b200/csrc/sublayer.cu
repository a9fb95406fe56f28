// What stands between the matrix products of a layer whose norms sit on the sublayers' outputs:
//
// embed_positions:  h[t] = table[id[t]] * scale + positions[p[t]]       (float32 stream; optionally
//                   the same rows in bfloat16 for the first product)
// stream_rows:      the float32 stream in bfloat16
// norm_add:         d = sum of delta's planes;  h[t] += d / sqrt(mean(d^2) + eps) * w   (float32),
//                   and the new h[t] in bfloat16 for the sublayer that reads the stream next
// glu_clamped:      g = min(gate, limit), u = clamp(up, -limit, limit);
//                   y = g * sigmoid(alpha * g) * (u + up_offset)        (float32 arithmetic)
// project_store:    a row of a stacked projection [q | k | v | extra]: bias added, q and k each
//                   RMS-normed over their *whole* width (where they have a weight), k and v written
//                   into their pages, q and sigmoid(extra) returned
//
// Every sum, norm and activation is float32; rows are rounded once, where they leave.
#include "common.cuh"

namespace {

__device__ __forceinline__ float block_sum(float v, float* part) {
    // part: 33 floats of shared memory
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    __syncthreads();            // part may still be read from an earlier call
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

template <typename T>
__global__ void embed_positions_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                       const T* __restrict__ table, const T* __restrict__ pos_table, float scale,
                                       float* __restrict__ out, __nv_bfloat16* __restrict__ rows_out, int dim,
                                       int vocab, int n_positions) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    (void)TL_CHECK(id >= 0 && id < vocab, TL_DBG_TOKEN_ID);
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);   // the host rejects such ids; stay in bounds anyway
    const T* src = table + (size_t)id * dim;
    const T* pos = nullptr;
    if (pos_table != nullptr) {
        int p = positions[t];
        (void)TL_CHECK(p >= 0 && p < n_positions, TL_DBG_POSITION);
        p = p < 0 ? 0 : (p >= n_positions ? n_positions - 1 : p);
        pos = pos_table + (size_t)p * dim;
    }
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float v = to_float(src[d]) * scale;
        if (pos != nullptr) v += to_float(pos[d]);
        out[(size_t)t * dim + d] = v;
        if (rows_out != nullptr) rows_out[(size_t)t * dim + d] = __float2bfloat16_rn(v);
    }
}

__global__ void stream_rows_kernel(const float* __restrict__ h, __nv_bfloat16* __restrict__ out, long long n) {
    grid_launch_dependents();
    grid_dependency_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16_rn(h[i]);
}

template <typename T>
__global__ void gate_mul_kernel(const T* __restrict__ x, const T* __restrict__ gate, T* __restrict__ out, long long n) {
    grid_launch_dependents();
    grid_dependency_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_float<T>(to_float(x[i]) * to_float(gate[i]));
}

// One CTA per row.  The summed delta is kept in shared memory between the two passes.
template <typename TD>
__global__ void norm_add_kernel(float* __restrict__ h, const TD* __restrict__ delta, int splits, long long plane, const float* __restrict__ bias,
                                const float* __restrict__ weight, __nv_bfloat16* __restrict__ rows_out, int dim,
                                float eps) {
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float part[33];
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t base = (size_t)blockIdx.x * dim;
    float ssq = 0.f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float v = bias != nullptr ? bias[d] : 0.f;
        for (int s = 0; s < splits; ++s) v += to_float(delta[(size_t)s * plane + base + d]);
        row_buf[d] = v;
        ssq = fmaf(v, v, ssq);
    }
    const float total = block_sum(ssq, part);
    const float r = rsqrtf(total / (float)dim + eps);
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        const float v = h[base + d] + row_buf[d] * r * weight[d];
        h[base + d] = v;
        if (rows_out != nullptr) rows_out[base + d] = __float2bfloat16_rn(v);
    }
}

template <typename TI, typename TO>
__global__ void glu_clamped_kernel(const TI* __restrict__ in, int splits, long long plane, TO* __restrict__ out,
                                   long long n_tokens, int hidden, float limit, float alpha, float up_offset) {
    grid_launch_dependents();
    grid_dependency_wait();
    const long long total = n_tokens * hidden;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / hidden;
        const int f = (int)(i - t * hidden);
        const size_t at = (size_t)t * 2 * hidden + f;
        float g = 0.f, u = 0.f;
        for (int s = 0; s < splits; ++s) {
            g += to_float(in[(size_t)s * plane + at]);
            u += to_float(in[(size_t)s * plane + at + hidden]);
        }
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        out[i] = from_float<TO>(g / (1.f + expf(-alpha * g)) * (u + up_offset));
    }
}

struct ProjectParams {
    const void* proj;       // [splits][T][width]
    int splits;
    long long plane;
    const float* bias;      // [width] or null
    const float* q_norm;    // [n_q] or null
    const float* k_norm;    // [n_k] or null
    float eps;
    int n_q, n_k, n_v, n_extra;
    void* q_out;            // [T, n_q]
    void* extra_out;        // [T, n_extra]
    void* k_pages;          // [pages, kv_heads, page_size, k_dim] or null
    void* v_pages;          // [pages, kv_heads, page_size, v_dim] or null
    const int* slot_mapping;
    int page_size, n_kv_heads, k_dim, v_dim;
    int norm_head;          // > 0: q and k are normed head by head, heads of this size, the weights [norm_head] shared by all heads
};

// the scale of every head of q and k (shared memory behind the row: (n_q + n_k) / norm_head floats), a warp per head
__device__ __forceinline__ void head_scales(const ProjectParams& p, const float* row, float* scales) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int heads = (p.n_q + p.n_k) / p.norm_head;
    for (int h = warp; h < heads; h += n_warps) {
        float ssq = 0.f;
        for (int d = lane; d < p.norm_head; d += 32) {
            const float v = row[h * p.norm_head + d];
            ssq = fmaf(v, v, ssq);
        }
        ssq = warp_sum(ssq);
        if (lane == 0) scales[h] = rsqrtf(ssq / (float)p.norm_head + p.eps);
    }
}

// One CTA per token; the row in shared memory as float32.
template <typename TI, typename TO>
__global__ void project_store_kernel(const ProjectParams p) {
    extern __shared__ __align__(16) float row[];
    __shared__ float part[33];
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x;
    const int width = p.n_q + p.n_k + p.n_v + p.n_extra;
    const TI* in = reinterpret_cast<const TI*>(p.proj) + (size_t)t * width;
    float ssq_q = 0.f, ssq_k = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < p.splits; ++s) v += to_float(in[(size_t)s * p.plane + c]);
        if (p.bias != nullptr) v += p.bias[c];
        row[c] = v;
        if (c < p.n_q) ssq_q = fmaf(v, v, ssq_q);
        else if (c < p.n_q + p.n_k) ssq_k = fmaf(v, v, ssq_k);
    }
    float rq = 1.f, rk = 1.f;
    if (p.q_norm != nullptr) rq = rsqrtf(block_sum(ssq_q, part) / (float)p.n_q + p.eps);
    if (p.k_norm != nullptr && p.n_k > 0) rk = rsqrtf(block_sum(ssq_k, part) / (float)p.n_k + p.eps);
    __syncthreads();
    const int nh = p.norm_head;
    const float* hs = row + width;
    if (nh > 0) {
        head_scales(p, row, row + width);
        __syncthreads();
    }

    TO* q_out = reinterpret_cast<TO*>(p.q_out) + (size_t)t * p.n_q;
    for (int c = threadIdx.x; c < p.n_q; c += blockDim.x) {
        float v = row[c];
        if (p.q_norm != nullptr) v *= nh > 0 ? hs[c / nh] * p.q_norm[c % nh] : rq * p.q_norm[c];
        q_out[c] = from_float<TO>(v);
    }

    if (p.k_pages != nullptr && p.n_k > 0) {
        const int slot = p.slot_mapping[t];
        if (TL_CHECK(slot >= 0, TL_DBG_SLOT) && tl_check_page(slot / p.page_size)) {
            const size_t page = slot / p.page_size, off = slot % p.page_size;
            TO* kp = reinterpret_cast<TO*>(p.k_pages);
            const float* k = row + p.n_q;
            for (int c = threadIdx.x; c < p.n_k; c += blockDim.x) {
                const int head = c / p.k_dim, d = c - head * p.k_dim;
                float v = k[c];
                if (p.k_norm != nullptr) v *= nh > 0 ? hs[(p.n_q + c) / nh] * p.k_norm[c % nh] : rk * p.k_norm[c];
                kp[((page * p.n_kv_heads + head) * p.page_size + off) * p.k_dim + d] = from_float<TO>(v);
            }
            if (p.v_pages != nullptr && p.n_v > 0) {
                TO* vp = reinterpret_cast<TO*>(p.v_pages);
                const float* v = row + p.n_q + p.n_k;
                for (int c = threadIdx.x; c < p.n_v; c += blockDim.x) {
                    const int head = c / p.v_dim, d = c - head * p.v_dim;
                    vp[((page * p.n_kv_heads + head) * p.page_size + off) * p.v_dim + d] = from_float<TO>(v[c]);
                }
            }
        }
    }
    if (p.n_extra > 0) {
        TO* e_out = reinterpret_cast<TO*>(p.extra_out) + (size_t)t * p.n_extra;
        const float* e = row + p.n_q + p.n_k + p.n_v;
        for (int c = threadIdx.x; c < p.n_extra; c += blockDim.x) e_out[c] = from_float<TO>(1.f / (1.f + expf(-e[c])));
    }
}


// ---- four columns at a time (widths that are multiples of 4, rows that start on 16 bytes)
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&a);
    raw.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}
// the sum over the planes of a split-K product (or the one plane there is), four columns
template <typename T>
__device__ __forceinline__ float4 sum_planes4(const T* p, int splits, long long plane) {
    float4 v = ld4(p);
#pragma unroll 4
    for (int s = 1; s < splits; ++s) {
        const float4 w = ld4(p + (size_t)s * plane);
        v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
    }
    return v;
}

template <typename TD>
__global__ void norm_add_vec_kernel(float* __restrict__ h, const TD* __restrict__ delta, int splits, long long plane, const float* __restrict__ bias,
                                    const float* __restrict__ weight, __nv_bfloat16* __restrict__ rows_out, int dim,
                                    float eps) {
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float part[33];
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t base = (size_t)blockIdx.x * dim;
    float ssq = 0.f;
    for (int d = threadIdx.x * 4; d < dim; d += blockDim.x * 4) {
        float4 v = sum_planes4(delta + base + d, splits, plane);
        if (bias != nullptr) { const float4 bb = ld4(bias + d); v.x += bb.x; v.y += bb.y; v.z += bb.z; v.w += bb.w; }
        st4(row_buf + d, v);
        ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float r = rsqrtf(block_sum(ssq, part) / (float)dim + eps);
    for (int d = threadIdx.x * 4; d < dim; d += blockDim.x * 4) {
        const float4 x = ld4(row_buf + d), w = ld4(weight + d);
        float4 v = ld4(h + base + d);
        v.x += x.x * r * w.x; v.y += x.y * r * w.y; v.z += x.z * r * w.z; v.w += x.w * r * w.w;
        st4(h + base + d, v);
        if (rows_out != nullptr) st4(rows_out + base + d, v);
    }
}

// bfloat16 in and out, one plane, hidden a multiple of 8: eight gates and eight ups per thread and turn
__global__ void glu_clamped_bf16x8_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                          long long n_chunks, int chunks_per_row, float limit, float alpha, float up_offset) {
    grid_launch_dependents();
    grid_dependency_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_chunks; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / chunks_per_row;
        const int c = (int)(i - t * chunks_per_row);
        const size_t hidden = (size_t)chunks_per_row * 8;
        const __nv_bfloat16* g = in + (size_t)t * 2 * hidden + (size_t)c * 8;
        Vec16<__nv_bfloat16> gv, uv, ov;
        gv.load(g);
        uv.load(g + hidden);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float a = fminf(gv.get(e), limit);
            const float u = fminf(fmaxf(uv.get(e), -limit), limit);
            ov.set(e, __fdividef(a, 1.f + __expf(-alpha * a)) * (u + up_offset));
        }
        ov.store(out + (size_t)t * hidden + (size_t)c * 8);
    }
}

// project_store, four columns at a time: every part of the row ([q | k | v | extra]) and every head's
// share of it is a multiple of 4 wide
template <typename TI, typename TO>
__global__ void project_store_vec_kernel(const ProjectParams p) {
    extern __shared__ __align__(16) float row[];
    __shared__ float part[33];
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x;
    const int width = p.n_q + p.n_k + p.n_v + p.n_extra;
    const TI* in = reinterpret_cast<const TI*>(p.proj) + (size_t)t * width;
    float ssq_q = 0.f, ssq_k = 0.f;
    for (int c = threadIdx.x * 4; c < width; c += blockDim.x * 4) {
        float4 v = sum_planes4(in + c, p.splits, p.plane);
        if (p.bias != nullptr) {
            const float4 b = ld4(p.bias + c);
            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
        }
        st4(row + c, v);
        const float sq = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        if (c < p.n_q) ssq_q += sq;
        else if (c < p.n_q + p.n_k) ssq_k += sq;
    }
    float rq = 1.f, rk = 1.f;
    if (p.q_norm != nullptr) rq = rsqrtf(block_sum(ssq_q, part) / (float)p.n_q + p.eps);
    if (p.k_norm != nullptr && p.n_k > 0) rk = rsqrtf(block_sum(ssq_k, part) / (float)p.n_k + p.eps);
    __syncthreads();
    const int nh = p.norm_head;
    const float* hs = row + width;
    if (nh > 0) {
        head_scales(p, row, row + width);
        __syncthreads();
    }

    TO* q_out = reinterpret_cast<TO*>(p.q_out) + (size_t)t * p.n_q;
    for (int c = threadIdx.x * 4; c < p.n_q; c += blockDim.x * 4) {
        float4 v = ld4(row + c);
        if (p.q_norm != nullptr) {
            const float4 w = ld4(p.q_norm + (nh > 0 ? c % nh : c));
            if (nh > 0) rq = hs[c / nh];
            v.x *= rq * w.x; v.y *= rq * w.y; v.z *= rq * w.z; v.w *= rq * w.w;
        }
        st4(q_out + c, v);
    }
    if (p.k_pages != nullptr && p.n_k > 0) {
        const int slot = p.slot_mapping[t];
        if (TL_CHECK(slot >= 0, TL_DBG_SLOT) && tl_check_page(slot / p.page_size)) {
            const size_t page = slot / p.page_size, off = slot % p.page_size;
            TO* kp = reinterpret_cast<TO*>(p.k_pages);
            const float* k = row + p.n_q;
            for (int c = threadIdx.x * 4; c < p.n_k; c += blockDim.x * 4) {
                const int head = c / p.k_dim, d = c - head * p.k_dim;
                float4 v = ld4(k + c);
                if (p.k_norm != nullptr) {
                    const float4 w = ld4(p.k_norm + (nh > 0 ? c % nh : c));
                    if (nh > 0) rk = hs[(p.n_q + c) / nh];
                    v.x *= rk * w.x; v.y *= rk * w.y; v.z *= rk * w.z; v.w *= rk * w.w;
                }
                st4(kp + ((page * p.n_kv_heads + head) * p.page_size + off) * p.k_dim + d, v);
            }
            if (p.v_pages != nullptr && p.n_v > 0) {
                TO* vp = reinterpret_cast<TO*>(p.v_pages);
                const float* vv = row + p.n_q + p.n_k;
                for (int c = threadIdx.x * 4; c < p.n_v; c += blockDim.x * 4) {
                    const int head = c / p.v_dim, d = c - head * p.v_dim;
                    st4(vp + ((page * p.n_kv_heads + head) * p.page_size + off) * p.v_dim + d, ld4(vv + c));
                }
            }
        }
    }
    if (p.n_extra > 0) {
        TO* e_out = reinterpret_cast<TO*>(p.extra_out) + (size_t)t * p.n_extra;
        const float* e = row + p.n_q + p.n_k + p.n_v;
        for (int c = threadIdx.x * 4; c < p.n_extra; c += blockDim.x * 4) {
            const float4 v = ld4(e + c);
            st4(e_out + c, make_float4(1.f / (1.f + expf(-v.x)), 1.f / (1.f + expf(-v.y)), 1.f / (1.f + expf(-v.z)),
                                       1.f / (1.f + expf(-v.w))));
        }
    }
}

// A thread to four columns, in whole warps: at most 1,024 threads for the few rows of a decode step (a row is
// a CTA: the row's latency is the kernel's), at most 256 where rows are many (several CTAs share an SM and the
// block-wide sums cost less).
inline int vec_threads(int cols, int n_rows) {
    int t = ((cols / 4 + 31) / 32) * 32;
    const int most = n_rows > 256 ? 256 : 1024;
    return t < 64 ? 64 : (t > most ? most : t);
}

inline int row_threads(int dim) { return dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128); }

}  // namespace

// table and pos_table have one dtype; positions and pos_table may be null (no position table);
// rows_out (bfloat16) may be null.
extern "C" int tl_embed_positions(const int* ids, const int* positions, const void* table, const void* pos_table,
                                  int table_dtype, float scale, float* out, void* rows_out, int n_tokens, int dim,
                                  int vocab, int n_positions, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (dim <= 0 || vocab <= 0 || (pos_table != nullptr && (positions == nullptr || n_positions <= 0))) return TL_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (table_dtype == TL_F32)
        e = tl_launch(embed_positions_kernel<float>, dim3(n_tokens), dim3(row_threads(dim)), 0, s, ids, positions,
                      (const float*)table, (const float*)pos_table, scale, out, (__nv_bfloat16*)rows_out, dim, vocab,
                      n_positions);
    else if (table_dtype == TL_BF16)
        e = tl_launch(embed_positions_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(row_threads(dim)), 0, s, ids, positions,
                      (const __nv_bfloat16*)table, (const __nv_bfloat16*)pos_table, scale, out, (__nv_bfloat16*)rows_out,
                      dim, vocab, n_positions);
    else
        return TL_BAD_DTYPE;
    return (int)e;
}

extern "C" int tl_stream_rows(const float* h, void* out, long long n, void* stream) {
    if (n <= 0) return TL_OK;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    return (int)tl_launch(stream_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, h,
                          (__nv_bfloat16*)out, n);
}

// out = x * gate element by element (float32 product); x, gate and out of one dtype, n elements
extern "C" int tl_gate_mul(const void* x, const void* gate, void* out, int dtype, long long n, void* stream) {
    if (n <= 0) return TL_OK;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == TL_F32)
        return (int)tl_launch(gate_mul_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, (const float*)x, (const float*)gate, (float*)out, n);
    if (dtype == TL_BF16)
        return (int)tl_launch(gate_mul_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, s, (const __nv_bfloat16*)x,
                              (const __nv_bfloat16*)gate, (__nv_bfloat16*)out, n);
    return TL_BAD_DTYPE;
}

// delta: [splits][n_rows][dim] in delta_dtype, planes `plane` elements apart; rows_out (bfloat16) may be null.
// bias: float32 [dim] or null, added to the summed delta before its norm.
extern "C" int tl_norm_add(float* h, const void* delta, int delta_dtype, int splits, long long plane, const float* bias,
                           const float* weight, void* rows_out, int n_rows, int dim, float eps, void* stream) {
    if (n_rows <= 0) return TL_OK;
    if (dim <= 0 || splits < 1) return TL_BAD_SIZE;
    const size_t smem = (size_t)dim * sizeof(float);
    if (smem > 200 * 1024) return TL_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    const bool vec = dim % 4 == 0 && plane % 4 == 0 && aligned16(h) && aligned16(delta) && aligned16(weight) && aligned16(bias) &&
                     (rows_out == nullptr || aligned16(rows_out)) && smem <= 48 * 1024;
    if (vec && delta_dtype == TL_F32)
        return (int)tl_launch(norm_add_vec_kernel<float>, dim3(n_rows), dim3(vec_threads(dim, n_rows)), smem, s, h, (const float*)delta,
                              splits, plane, bias, weight, (__nv_bfloat16*)rows_out, dim, eps);
    if (vec && delta_dtype == TL_BF16)
        return (int)tl_launch(norm_add_vec_kernel<__nv_bfloat16>, dim3(n_rows), dim3(vec_threads(dim, n_rows)), smem, s, h,
                              (const __nv_bfloat16*)delta, splits, plane, bias, weight, (__nv_bfloat16*)rows_out, dim, eps);
    if (delta_dtype == TL_F32) {
        static int raised = 0;
        if (smem > 48 * 1024 && (int)smem > raised) {
            e = cudaFuncSetAttribute(norm_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            raised = (int)smem;
        }
        e = tl_launch(norm_add_kernel<float>, dim3(n_rows), dim3(row_threads(dim)), smem, s, h, (const float*)delta, splits,
                      plane, bias, weight, (__nv_bfloat16*)rows_out, dim, eps);
    } else if (delta_dtype == TL_BF16) {
        static int raised = 0;
        if (smem > 48 * 1024 && (int)smem > raised) {
            e = cudaFuncSetAttribute(norm_add_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            raised = (int)smem;
        }
        e = tl_launch(norm_add_kernel<__nv_bfloat16>, dim3(n_rows), dim3(row_threads(dim)), smem, s, h,
                      (const __nv_bfloat16*)delta, splits, plane, bias, weight, (__nv_bfloat16*)rows_out, dim, eps);
    } else {
        return TL_BAD_DTYPE;
    }
    return (int)e;
}

// in: [splits][n_tokens][2 * hidden] (gate columns first); out: [n_tokens][hidden].
extern "C" int tl_glu_clamped(const void* in, int in_dtype, int splits, long long plane, void* out, int out_dtype,
                              int n_tokens, int hidden, float limit, float alpha, float up_offset, void* stream) {
    if ((long long)n_tokens * hidden <= 0) return TL_OK;
    if (splits < 1) return TL_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    long long blocks = ((long long)n_tokens * hidden + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    const dim3 grid((unsigned)blocks), block(256);
    cudaError_t e;
    if (in_dtype == TL_BF16 && out_dtype == TL_BF16 && splits == 1 && hidden % 8 == 0 && aligned16(in) && aligned16(out)) {
        const long long n_chunks = (long long)n_tokens * (hidden / 8);
        long long b8 = (n_chunks + 255) / 256;
        if (b8 > 148 * 16) b8 = 148 * 16;
        return (int)tl_launch(glu_clamped_bf16x8_kernel, dim3((unsigned)b8), block, 0, s, (const __nv_bfloat16*)in,
                              (__nv_bfloat16*)out, n_chunks, hidden / 8, limit, alpha, up_offset);
    }
    if (in_dtype == TL_F32 && out_dtype == TL_F32)
        e = tl_launch(glu_clamped_kernel<float, float>, grid, block, 0, s, (const float*)in, splits, plane, (float*)out,
                      (long long)n_tokens, hidden, limit, alpha, up_offset);
    else if (in_dtype == TL_F32 && out_dtype == TL_BF16)
        e = tl_launch(glu_clamped_kernel<float, __nv_bfloat16>, grid, block, 0, s, (const float*)in, splits, plane,
                      (__nv_bfloat16*)out, (long long)n_tokens, hidden, limit, alpha, up_offset);
    else if (in_dtype == TL_BF16 && out_dtype == TL_BF16)
        e = tl_launch(glu_clamped_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)in, splits,
                      plane, (__nv_bfloat16*)out, (long long)n_tokens, hidden, limit, alpha, up_offset);
    else
        return TL_BAD_DTYPE;
    return (int)e;
}

extern "C" int tl_project_store(const void* proj, int in_dtype, int splits, long long plane, const float* bias,
                                const float* q_norm, const float* k_norm, float eps, int n_q, int n_k, int n_v,
                                int n_extra, void* q_out, void* extra_out, int out_dtype, void* k_pages, void* v_pages,
                                const int* slot_mapping, int page_size, int n_kv_heads, int k_dim, int v_dim,
                                int n_tokens, int norm_head, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (n_q < 0 || n_k < 0 || n_v < 0 || n_extra < 0 || splits < 1) return TL_BAD_SIZE;
    const int width = n_q + n_k + n_v + n_extra;
    if (width <= 0) return TL_BAD_SIZE;
    if (k_pages != nullptr && n_k > 0 &&
        (slot_mapping == nullptr || page_size <= 0 || n_kv_heads <= 0 || k_dim <= 0 || n_k != n_kv_heads * k_dim))
        return TL_BAD_SIZE;
    if (k_pages != nullptr && v_pages != nullptr && n_v > 0 && (v_dim <= 0 || n_v != n_kv_heads * v_dim)) return TL_BAD_SIZE;
    if (norm_head < 0 || (norm_head > 0 && (n_q % norm_head != 0 || n_k % norm_head != 0))) return TL_BAD_SIZE;
    const size_t smem = (size_t)(width + (norm_head > 0 ? (n_q + n_k) / norm_head : 0)) * sizeof(float);
    if (smem > 200 * 1024) return TL_TOO_LARGE;
    ProjectParams p;
    p.norm_head = norm_head;
    p.proj = proj; p.splits = splits; p.plane = plane; p.bias = bias; p.q_norm = q_norm; p.k_norm = k_norm; p.eps = eps;
    p.n_q = n_q; p.n_k = n_k; p.n_v = n_v; p.n_extra = n_extra; p.q_out = q_out; p.extra_out = extra_out;
    p.k_pages = k_pages; p.v_pages = v_pages; p.slot_mapping = slot_mapping; p.page_size = page_size;
    p.n_kv_heads = n_kv_heads; p.k_dim = k_dim; p.v_dim = v_dim;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    const bool vec = n_q % 4 == 0 && n_k % 4 == 0 && n_v % 4 == 0 && n_extra % 4 == 0 && plane % 4 == 0 && norm_head % 4 == 0 &&
                     (k_pages == nullptr || n_k == 0 || (k_dim % 4 == 0 && aligned16(k_pages))) &&
                     (v_pages == nullptr || n_v == 0 || (v_dim % 4 == 0 && aligned16(v_pages))) && aligned16(proj) &&
                     aligned16(q_out) && (extra_out == nullptr || aligned16(extra_out)) && (bias == nullptr || aligned16(bias)) &&
                     (q_norm == nullptr || aligned16(q_norm)) && (k_norm == nullptr || aligned16(k_norm)) && smem <= 48 * 1024;
    if (vec) {
        const dim3 grid(n_tokens), block(vec_threads(width, n_tokens));
        if (in_dtype == TL_F32 && out_dtype == TL_F32) return (int)tl_launch(project_store_vec_kernel<float, float>, grid, block, smem, s, p);
        if (in_dtype == TL_F32 && out_dtype == TL_BF16) return (int)tl_launch(project_store_vec_kernel<float, __nv_bfloat16>, grid, block, smem, s, p);
        if (in_dtype == TL_BF16 && out_dtype == TL_BF16) return (int)tl_launch(project_store_vec_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, smem, s, p);
        return TL_BAD_DTYPE;
    }
#define TL_PROJECT_LAUNCH(TI, TO)                                                                                      \
    do {                                                                                                               \
        static int raised = 0;                                                                                         \
        if (smem > 48 * 1024 && (int)smem > raised) {                                                                  \
            e = cudaFuncSetAttribute(project_store_kernel<TI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                       \
            raised = (int)smem;                                                                                        \
        }                                                                                                              \
        e = tl_launch(project_store_kernel<TI, TO>, dim3(n_tokens), dim3(row_threads(width)), smem, s, p);             \
    } while (0)
    if (in_dtype == TL_F32 && out_dtype == TL_F32) TL_PROJECT_LAUNCH(float, float);
    else if (in_dtype == TL_F32 && out_dtype == TL_BF16) TL_PROJECT_LAUNCH(float, __nv_bfloat16);
    else if (in_dtype == TL_BF16 && out_dtype == TL_BF16) TL_PROJECT_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return TL_BAD_DTYPE;
#undef TL_PROJECT_LAUNCH
    return (int)e;
}

// ---------------------------------------------------------------------------------------------
// Layers with a norm in front of each sublayer and another on its output, gated and plain
// activations by name, an average over the results of all layers so far, and the combination of
// two attention maps:
//
// norm_add_norm:   d = sum of delta's planes;  h[t] += d / sqrt(mean(d^2) + eps) * w   (float32), and
//                  out[t] = h[t] / sqrt(mean(h[t]^2) + eps2) * w2: the output norm of one sublayer, the
//                  residual sum and the input norm of the next sublayer in one pass over the row
// depth_mix:       out = sum_j c[j] * level_j over the first n levels of [levels][tokens][dim]
// gated_act:       act(gate) * up for a row [gate | up];  activation: act(x)      (float32 arithmetic)
// differential_combine:  per (token, head): o = a1 - lambda a2 over the head's values, then
//                  o / sqrt(mean(o^2) + eps) * out_scale * gate[token, head]
namespace {

enum : int { ACT_SILU = 0, ACT_GELU_TANH = 1, ACT_RELU2 = 2 };

__device__ __forceinline__ float act_apply(float x, int act) {
    if (act == ACT_SILU) return x / (1.f + expf(-x));
    if (act == ACT_GELU_TANH) return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    const float r = fmaxf(x, 0.f);
    return r * r;
}

// One CTA per row; the row is kept in shared memory between the passes.  VEC: four columns per thread and turn.
template <typename TD, typename TO, bool VEC>
__global__ void norm_add_norm_kernel(float* __restrict__ h, const TD* __restrict__ delta, int splits, long long plane, const float* __restrict__ bias,
                                     const float* __restrict__ weight, const float* __restrict__ weight2,
                                     TO* __restrict__ out, int dim, float eps, float eps2) {
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float part[33];
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t base = (size_t)blockIdx.x * dim;
    float ssq = 0.f;
    if (VEC) {
        for (int d = threadIdx.x * 4; d < dim; d += blockDim.x * 4) {
            float4 v = sum_planes4(delta + base + d, splits, plane);
            if (bias != nullptr) { const float4 bb = ld4(bias + d); v.x += bb.x; v.y += bb.y; v.z += bb.z; v.w += bb.w; }
            st4(row_buf + d, v);
            ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            float v = bias != nullptr ? bias[d] : 0.f;
            for (int s = 0; s < splits; ++s) v += to_float(delta[(size_t)s * plane + base + d]);
            row_buf[d] = v;
            ssq = fmaf(v, v, ssq);
        }
    }
    const float r = rsqrtf(block_sum(ssq, part) / (float)dim + eps);
    float ssq2 = 0.f;
    if (VEC) {
        for (int d = threadIdx.x * 4; d < dim; d += blockDim.x * 4) {
            const float4 x = ld4(row_buf + d), w = ld4(weight + d);
            float4 v = ld4(h + base + d);
            v.x += x.x * r * w.x; v.y += x.y * r * w.y; v.z += x.z * r * w.z; v.w += x.w * r * w.w;
            st4(h + base + d, v);
            st4(row_buf + d, v);
            ssq2 += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            const float v = h[base + d] + row_buf[d] * r * weight[d];
            h[base + d] = v;
            row_buf[d] = v;
            ssq2 = fmaf(v, v, ssq2);
        }
    }
    const float r2 = rsqrtf(block_sum(ssq2, part) / (float)dim + eps2);
    if (VEC) {
        for (int d = threadIdx.x * 4; d < dim; d += blockDim.x * 4) {
            const float4 x = ld4(row_buf + d), w = ld4(weight2 + d);
            st4(out + base + d, make_float4(x.x * r2 * w.x, x.y * r2 * w.y, x.z * r2 * w.z, x.w * r2 * w.w));
        }
    } else {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) out[base + d] = from_float<TO>(row_buf[d] * r2 * weight2[d]);
    }
}

template <bool VEC>
__global__ void depth_mix_kernel(const float* __restrict__ levels, long long level_stride, const float* __restrict__ coef,
                                 int n, float* __restrict__ out, long long count) {
    grid_launch_dependents();
    grid_dependency_wait();
    const long long step = (long long)gridDim.x * blockDim.x;
    if (VEC) {
        for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < count; i += step * 4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < n; ++j) {
                const float c = __ldg(coef + j);
                const float4 v = ld4(levels + j * level_stride + i);
                acc.x = fmaf(c, v.x, acc.x); acc.y = fmaf(c, v.y, acc.y); acc.z = fmaf(c, v.z, acc.z); acc.w = fmaf(c, v.w, acc.w);
            }
            st4(out + i, acc);
        }
    } else {
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += step) {
            float acc = 0.f;
            for (int j = 0; j < n; ++j) acc = fmaf(__ldg(coef + j), levels[j * level_stride + i], acc);
            out[i] = acc;
        }
    }
}

// The same average, a row per CTA, with the RMS norm of the result under weight / eps beside it (the input norm of
// the layer that reads the average next): the row stays in shared memory between the two passes.
template <typename TO>
__global__ void depth_mix_norm_kernel(const float* __restrict__ levels, long long level_stride, const float* __restrict__ coef,
                                      int n, float* __restrict__ out, const float* __restrict__ weight, TO* __restrict__ normed,
                                      int dim, float eps) {
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float part[33];
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t base = (size_t)blockIdx.x * dim;
    float ssq = 0.f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < n; ++j) acc = fmaf(__ldg(coef + j), levels[j * level_stride + base + d], acc);
        out[base + d] = acc;
        row_buf[d] = acc;
        ssq = fmaf(acc, acc, ssq);
    }
    const float r = rsqrtf(block_sum(ssq, part) / (float)dim + eps);
    for (int d = threadIdx.x; d < dim; d += blockDim.x) normed[base + d] = from_float<TO>(row_buf[d] * r * weight[d]);
}

// in: [splits][n_tokens][(gated ? 2 : 1) * hidden]; out: [n_tokens][hidden]
template <typename TI, typename TO>
__global__ void act_kernel(const TI* __restrict__ in, int splits, long long plane, TO* __restrict__ out,
                           long long n_tokens, int hidden, int act, int gated) {
    grid_launch_dependents();
    grid_dependency_wait();
    const long long total = n_tokens * hidden;
    const int width = gated ? 2 * hidden : hidden;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / hidden;
        const int f = (int)(i - t * hidden);
        const size_t at = (size_t)t * width + f;
        float g = 0.f, u = 0.f;
        for (int s = 0; s < splits; ++s) {
            g += to_float(in[(size_t)s * plane + at]);
            if (gated) u += to_float(in[(size_t)s * plane + at + hidden]);
        }
        const float a = act_apply(g, act);
        out[i] = from_float<TO>(gated ? a * u : a);
    }
}

// bfloat16 in and out, one plane, hidden a multiple of 8: eight values (and eight ups) per thread and turn
__global__ void act_bf16x8_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n_chunks,
                                  int chunks_per_row, int act, int gated) {
    grid_launch_dependents();
    grid_dependency_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_chunks; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / chunks_per_row;
        const int c = (int)(i - t * chunks_per_row);
        const size_t hidden = (size_t)chunks_per_row * 8;
        const __nv_bfloat16* g = in + (size_t)t * (gated ? 2 : 1) * hidden + (size_t)c * 8;
        Vec16<__nv_bfloat16> gv, uv, ov;
        gv.load(g);
        if (gated) uv.load(g + hidden);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float a = act_apply(gv.get(e), act);
            ov.set(e, gated ? a * uv.get(e) : a);
        }
        ov.store(out + (size_t)t * hidden + (size_t)c * 8);
    }
}

// maps: float32 [T][2 H][dv], all first maps before all second maps; a warp per (token, head)
template <typename TO>
__global__ void differential_combine_kernel(const float* __restrict__ maps, const TO* __restrict__ gate,
                                            TO* __restrict__ out, long long n_rows, int n_heads, int dv, float lam,
                                            float eps, float out_scale) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);   // token * H + head
    if (row >= n_rows) return;
    const long long t = row / n_heads;
    const int hd = (int)(row - t * n_heads);
    const float* a1 = maps + ((size_t)t * 2 * n_heads + hd) * dv;
    const float* a2 = a1 + (size_t)n_heads * dv;
    float ssq = 0.f;
    for (int d = lane; d < dv; d += 32) {
        const float o = a1[d] - lam * a2[d];
        ssq = fmaf(o, o, ssq);
    }
    ssq = warp_sum(ssq);
    float f = rsqrtf(ssq / (float)dv + eps) * out_scale;
    if (gate != nullptr) f *= to_float(gate[row]);
    for (int d = lane; d < dv; d += 32) out[(size_t)row * dv + d] = from_float<TO>((a1[d] - lam * a2[d]) * f);
}

}  // namespace

// As tl_norm_add, and out = norm of the new h under weight2 / eps2, in out_dtype.
extern "C" int tl_norm_add_norm(float* h, const void* delta, int delta_dtype, int splits, long long plane, const float* bias,
                                const float* weight, const float* weight2, void* out, int out_dtype, int n_rows, int dim,
                                float eps, float eps2, void* stream) {
    if (n_rows <= 0) return TL_OK;
    if (dim <= 0 || splits < 1) return TL_BAD_SIZE;
    const size_t smem = (size_t)dim * sizeof(float);
    if (smem > 200 * 1024) return TL_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = dim % 4 == 0 && plane % 4 == 0 && aligned16(h) && aligned16(delta) && aligned16(weight) && aligned16(bias) &&
                     aligned16(weight2) && aligned16(out);
    const dim3 grid(n_rows), block(vec ? vec_threads(dim, n_rows) : row_threads(dim));
#define TL_NAN_LAUNCH(TD, TO, V)                                                                                     \
    do {                                                                                                             \
        static int raised = 0;                                                                                       \
        if (smem > 48 * 1024 && (int)smem > raised) {                                                                \
            cudaError_t e = cudaFuncSetAttribute(norm_add_norm_kernel<TD, TO, V>,                                    \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
            if (e != cudaSuccess) return (int)e;                                                                     \
            raised = (int)smem;                                                                                      \
        }                                                                                                            \
        return (int)tl_launch(norm_add_norm_kernel<TD, TO, V>, grid, block, smem, s, h, (const TD*)delta, splits,    \
                              plane, bias, weight, weight2, (TO*)out, dim, eps, eps2);                               \
    } while (0)
#define TL_NAN_PICK(TD, TO) do { if (vec) TL_NAN_LAUNCH(TD, TO, true); else TL_NAN_LAUNCH(TD, TO, false); } while (0)
    if (delta_dtype == TL_F32 && out_dtype == TL_F32) TL_NAN_PICK(float, float);
    if (delta_dtype == TL_F32 && out_dtype == TL_BF16) TL_NAN_PICK(float, __nv_bfloat16);
    if (delta_dtype == TL_BF16 && out_dtype == TL_BF16) TL_NAN_PICK(__nv_bfloat16, __nv_bfloat16);
#undef TL_NAN_PICK
#undef TL_NAN_LAUNCH
    return TL_BAD_DTYPE;
}

// levels: float32 [>= n][count] with level_stride elements between levels; out: [count] (may be a later level)
extern "C" int tl_depth_mix(const float* levels, long long level_stride, const float* coef, int n, float* out,
                            long long count, void* stream) {
    if (count <= 0) return TL_OK;
    if (n < 1) return TL_BAD_SIZE;
    const bool vec = count % 4 == 0 && level_stride % 4 == 0 && aligned16(levels) && aligned16(out);
    long long blocks = ((vec ? count / 4 : count) + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (vec) return (int)tl_launch(depth_mix_kernel<true>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, levels,
                                   level_stride, coef, n, out, count);
    return (int)tl_launch(depth_mix_kernel<false>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, levels,
                          level_stride, coef, n, out, count);
}

// As tl_depth_mix for rows of `dim` elements ([n_rows][dim] per level), and normed = out / sqrt(mean(out^2) + eps) * weight
// in out_dtype.
extern "C" int tl_depth_mix_norm(const float* levels, long long level_stride, const float* coef, int n, float* out,
                                 const float* weight, void* normed, int out_dtype, int n_rows, int dim, float eps, void* stream) {
    if (n_rows <= 0) return TL_OK;
    if (n < 1 || dim <= 0) return TL_BAD_SIZE;
    const size_t smem = (size_t)dim * sizeof(float);
    if (smem > 48 * 1024) return TL_TOO_LARGE;
    const dim3 grid(n_rows), block(row_threads(dim));
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == TL_F32)
        return (int)tl_launch(depth_mix_norm_kernel<float>, grid, block, smem, s, levels, level_stride, coef, n, out, weight,
                              (float*)normed, dim, eps);
    if (out_dtype == TL_BF16)
        return (int)tl_launch(depth_mix_norm_kernel<__nv_bfloat16>, grid, block, smem, s, levels, level_stride, coef, n, out, weight,
                              (__nv_bfloat16*)normed, dim, eps);
    return TL_BAD_DTYPE;
}

// gated: in is [splits][n_tokens][2 * hidden] (gate columns first) and out = act(gate) * up; else in is
// [splits][n_tokens][hidden] and out = act(in).  act: 0 silu, 1 gelu (tanh form), 2 squared relu.
extern "C" int tl_act(const void* in, int in_dtype, int splits, long long plane, void* out, int out_dtype, int n_tokens,
                      int hidden, int act, int gated, void* stream) {
    if ((long long)n_tokens * hidden <= 0) return TL_OK;
    if (splits < 1 || act < 0 || act > 2) return TL_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    long long blocks = ((long long)n_tokens * hidden + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    const dim3 grid((unsigned)blocks), block(256);
    if (in_dtype == TL_BF16 && out_dtype == TL_BF16 && splits == 1 && hidden % 8 == 0 && aligned16(in) && aligned16(out)) {
        const long long n_chunks = (long long)n_tokens * (hidden / 8);
        long long b8 = (n_chunks + 255) / 256;
        if (b8 > 148 * 16) b8 = 148 * 16;
        return (int)tl_launch(act_bf16x8_kernel, dim3((unsigned)b8), block, 0, s, (const __nv_bfloat16*)in, (__nv_bfloat16*)out,
                              n_chunks, hidden / 8, act, gated);
    }
    if (in_dtype == TL_F32 && out_dtype == TL_F32)
        return (int)tl_launch(act_kernel<float, float>, grid, block, 0, s, (const float*)in, splits, plane, (float*)out,
                              (long long)n_tokens, hidden, act, gated);
    if (in_dtype == TL_F32 && out_dtype == TL_BF16)
        return (int)tl_launch(act_kernel<float, __nv_bfloat16>, grid, block, 0, s, (const float*)in, splits, plane,
                              (__nv_bfloat16*)out, (long long)n_tokens, hidden, act, gated);
    if (in_dtype == TL_BF16 && out_dtype == TL_BF16)
        return (int)tl_launch(act_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)in, splits,
                              plane, (__nv_bfloat16*)out, (long long)n_tokens, hidden, act, gated);
    return TL_BAD_DTYPE;
}

// maps: float32 [n_tokens][2 * n_heads][dv]; gate: [n_tokens][n_heads] in out_dtype or null; out: [n_tokens][n_heads * dv]
extern "C" int tl_differential_combine(const float* maps, const void* gate, void* out, int out_dtype, int n_tokens,
                                       int n_heads, int dv, float lam, float eps, float out_scale, void* stream) {
    const long long rows = (long long)n_tokens * n_heads;
    if (rows <= 0) return TL_OK;
    if (dv <= 0) return TL_BAD_SIZE;
    const dim3 grid((unsigned)((rows + 3) / 4)), block(128);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == TL_F32)
        return (int)tl_launch(differential_combine_kernel<float>, grid, block, 0, s, maps, (const float*)gate, (float*)out, rows,
                              n_heads, dv, lam, eps, out_scale);
    if (out_dtype == TL_BF16)
        return (int)tl_launch(differential_combine_kernel<__nv_bfloat16>, grid, block, 0, s, maps, (const __nv_bfloat16*)gate,
                              (__nv_bfloat16*)out, rows, n_heads, dv, lam, eps, out_scale);
    return TL_BAD_DTYPE;
}
