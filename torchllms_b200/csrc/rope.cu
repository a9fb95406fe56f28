// Rotary encoding of q and k fused with the write of k and v into their cache pages.
//
// Input is the packed projection row [q heads | k heads | v heads] of every token.  q and k are
// rotated in float32 with (cos, sin) gathered from a float32 table at the token's absolute
// position; v is copied.  Reference: torchllms/models/networks.py:332-352 (rotation of adjacent
// lanes) and :551-553 (k is stored after rotation, v as it is).  `interleaved` pairs lanes
// (2i, 2i+1); otherwise lanes (i, i + head_dim/2) are paired.
//
// Pages are laid out [page, kv_head, slot_in_page, head_dim]; slot_mapping[t] = page * page_size + slot.
//
// The projection's input may have been weighted for an RMS norm but not normalised yet; then every
// value of a token's row is first multiplied by rsqrt(sum_p ssq[token, p] * inv_dim + eps)
// (the norm of torchllms/models/networks.py:195-200, applied after the product instead of before it).
#include "common.cuh"

// qkv holds `splits` planes `plane` elements apart (partial sums of a split-K product), summed first
template <typename TI, typename T>
__global__ void rope_kv_write_kernel(const TI* __restrict__ qkv, int splits, long long plane,
                                     const int* __restrict__ positions,
                                     const float* __restrict__ table, const int* __restrict__ slot_mapping,
                                     T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     int n_heads, int n_kv_heads, int head_dim, int page_size,
                                     int table_rows, int interleaved, const RowScale rs) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x;
    const float sc = warp_row_scale(rs, t);        // (a CTA's threads all work on token t)
    const int half = head_dim >> 1;
    const int heads_per_cta = (n_heads + 2 * n_kv_heads + gridDim.y - 1) / gridDim.y;
    const int head_lo = blockIdx.y * heads_per_cta;
    const int head_hi = min(n_heads + 2 * n_kv_heads, head_lo + heads_per_cta);
    int pos = positions[t];
    (void)TL_CHECK(pos >= 0 && pos < table_rows, TL_DBG_POSITION);
    pos = pos < 0 ? 0 : (pos >= table_rows ? table_rows - 1 : pos);  // the host keeps positions inside the table
    const float* cs = table + (size_t)pos * head_dim;                 // [half][2]
    const int row = (n_heads + 2 * n_kv_heads) * head_dim;
    const TI* src = qkv + (size_t)t * row;
    const int n_rot_pairs = (n_heads + n_kv_heads) * half;
    const int n_pairs = head_hi * half;
    int page = 0, slot = 0;
    bool write = k_pages != nullptr;
    if (write) {
        const int sm = slot_mapping[t];
        page = sm / page_size;
        slot = sm - page * page_size;
        if (!(TL_CHECK(sm >= 0, TL_DBG_SLOT) && tl_check_page(page))) write = false;    // (debug builds: nothing is written there)
    }
    for (int p = head_lo * half + threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int head = p / half;       // 0 .. H + 2 KV - 1 over the packed row
        const int i = p - head * half;
        const int l0 = interleaved ? 2 * i : i;
        const int l1 = interleaved ? 2 * i + 1 : i + half;
        float x0 = to_float(src[head * head_dim + l0]);
        float x1 = to_float(src[head * head_dim + l1]);
        for (int sp = 1; sp < splits; ++sp) {
            x0 += to_float(src[sp * plane + head * head_dim + l0]);
            x1 += to_float(src[sp * plane + head * head_dim + l1]);
        }
        x0 *= sc;
        x1 *= sc;
        if (p < n_rot_pairs) {
            const float c = cs[2 * i], s = cs[2 * i + 1];
            const float y0 = x0 * c - x1 * s;
            const float y1 = x1 * c + x0 * s;
            x0 = y0;
            x1 = y1;
        }
        if (head < n_heads) {
            T* dst = q_out + ((size_t)t * n_heads + head) * head_dim;
            dst[l0] = from_float<T>(x0);
            dst[l1] = from_float<T>(x1);
        } else if (write) {
            const bool is_k = head < n_heads + n_kv_heads;
            const int kvh = is_k ? head - n_heads : head - n_heads - n_kv_heads;
            T* base = is_k ? k_pages : v_pages;
            T* dst = base + (((size_t)page * n_kv_heads + kvh) * page_size + slot) * head_dim;
            dst[l0] = from_float<T>(x0);
            dst[l1] = from_float<T>(x1);
        }
    }
}

// eight consecutive elements as floats
__device__ __forceinline__ void load8(const float* p, float (&x)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&x)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void store8(float* p, const float (&x)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(x[4], x[5], x[6], x[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&x)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

// The adjacent-lane pairing with 16-byte accesses: a thread takes eight consecutive lanes (four
// pairs) of one head.  Same arithmetic as the kernel above.
template <typename TI, typename T>
__global__ void rope_kv_write_vec_kernel(const TI* __restrict__ qkv, int splits, long long plane,
                                         const int* __restrict__ positions, const float* __restrict__ table,
                                         const int* __restrict__ slot_mapping, T* __restrict__ q_out,
                                         T* __restrict__ k_pages, T* __restrict__ v_pages, int n_heads, int n_kv_heads,
                                         int head_dim, int page_size, int table_rows, const RowScale rs) {
    grid_launch_dependents();
    // positions, cache slots and the rotation table do not come from the kernel before this one (the
    // step's index data were uploaded before its first kernel): they are fetched before waiting for it
    const int t = blockIdx.x;
    const int heads = n_heads + 2 * n_kv_heads;
    const int per_head = head_dim >> 3;
    int pos = positions[t];
    (void)TL_CHECK(pos >= 0 && pos < table_rows, TL_DBG_POSITION);
    pos = pos < 0 ? 0 : (pos >= table_rows ? table_rows - 1 : pos);
    const float* cs = table + (size_t)pos * head_dim;
    const TI* src = qkv + (size_t)t * heads * head_dim;
    bool write = k_pages != nullptr;
    int page = 0, slot = 0;
    if (write) {
        const int sm = slot_mapping[t];
        page = sm / page_size;
        slot = sm - page * page_size;
        if (!(TL_CHECK(sm >= 0, TL_DBG_SLOT) && tl_check_page(page))) write = false;    // (debug builds: nothing is written there)
    }
    const int c_first = blockIdx.y * blockDim.x + threadIdx.x;
    float r_first[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (c_first < heads * per_head && c_first / per_head < n_heads + n_kv_heads)
        load8(cs + ((c_first - (c_first / per_head) * per_head) << 3), r_first);
    grid_dependency_wait();
    const float sc = warp_row_scale(rs, t);        // (a CTA's threads all work on token t)
    for (int c = c_first; c < heads * per_head; c += gridDim.y * blockDim.x) {
        const int head = c / per_head;
        const int off = (c - head * per_head) << 3;
        float x[8];
        load8(src + head * head_dim + off, x);
        for (int sp = 1; sp < splits; ++sp) {
            float y[8];
            load8(src + sp * plane + head * head_dim + off, y);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] += y[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] *= sc;
        if (head < n_heads + n_kv_heads) {
            float r[8];
            if (c == c_first) {
#pragma unroll
                for (int i = 0; i < 8; ++i) r[i] = r_first[i];
            } else {
                load8(cs + off, r);      // (cos, sin) of the four pairs
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float a = x[2 * i], b = x[2 * i + 1], co = r[2 * i], si = r[2 * i + 1];
                x[2 * i] = a * co - b * si;
                x[2 * i + 1] = b * co + a * si;
            }
        }
        if (head < n_heads) {
            store8(q_out + ((size_t)t * n_heads + head) * head_dim + off, x);
        } else if (write) {
            const bool is_k = head < n_heads + n_kv_heads;
            const int kvh = is_k ? head - n_heads : head - n_heads - n_kv_heads;
            T* base = is_k ? k_pages : v_pages;
            store8(base + (((size_t)page * n_kv_heads + kvh) * page_size + slot) * head_dim + off, x);
        }
    }
}

// k_pages / v_pages may both be null: then only q is produced (a run that reads another run's cache).
// qkv: [splits, n_tokens, row] of in_dtype (splits > 1 only for float32 partial sums); q, pages: dtype.
// in_ssq may be null; else [n_tokens, in_parts] floats give every token's row scale (see the top of the file).
extern "C" int tl_rope_kv_write(const void* qkv, int in_dtype, int splits, const int* positions, const float* table,
                                const int* slot_mapping, void* q_out, void* k_pages, void* v_pages,
                                int dtype, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                int page_size, int table_rows, int interleaved,
                                const float* in_ssq, int in_parts, float in_inv_dim, float in_eps, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (in_ssq != nullptr && in_parts < 1) return TL_BAD_SIZE;
    const RowScale rs = {in_ssq, in_parts, in_inv_dim, in_eps};
    if (head_dim <= 0 || (head_dim & 1) || n_heads <= 0 || n_kv_heads <= 0 || page_size <= 0 || table_rows <= 0 || splits < 1)
        return TL_BAD_SIZE;
    if ((k_pages == nullptr) != (v_pages == nullptr)) return TL_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int heads = n_heads + 2 * n_kv_heads;
    // few tokens (decoding): spread a token's heads over several CTAs
    int per_cta = n_tokens >= 256 ? heads : (4 * 128 + head_dim / 2 - 1) / (head_dim / 2);
    if (per_cta > heads) per_cta = heads;
    const int chunks = (heads + per_cta - 1) / per_cta;
    const int pairs = per_cta * (head_dim / 2);
    const int threads = pairs >= 1024 ? 256 : 128;
    const long long plane = (long long)n_tokens * (n_heads + 2 * n_kv_heads) * head_dim;
    if (interleaved && head_dim % 8 == 0 && aligned16(qkv) && aligned16(q_out) && aligned16(table) &&
        (k_pages == nullptr || (aligned16(k_pages) && aligned16(v_pages)))) {
        const int chunks8 = heads * (head_dim / 8);
        const int vthreads = 128;
        int by = (chunks8 + vthreads - 1) / vthreads;
        if (n_tokens >= 256 && by > 2) by = 2;        // many tokens: fewer, fatter CTAs
#define TL_ROPE_VEC(TI, T)                                                                                      \
    tl_launch(rope_kv_write_vec_kernel<TI, T>, dim3(n_tokens, by), dim3(vthreads), 0, s,                        \
              (const TI*)qkv, splits, plane, positions, table, slot_mapping, (T*)q_out, (T*)k_pages, (T*)v_pages, \
              n_heads, n_kv_heads, head_dim, page_size, table_rows, rs)
        if (in_dtype == TL_F32 && dtype == TL_F32) return (int)TL_ROPE_VEC(float, float);
        if (in_dtype == TL_BF16 && dtype == TL_BF16) return (int)TL_ROPE_VEC(__nv_bfloat16, __nv_bfloat16);
        if (in_dtype == TL_F32 && dtype == TL_BF16) return (int)TL_ROPE_VEC(float, __nv_bfloat16);
#undef TL_ROPE_VEC
        return TL_BAD_DTYPE;
    }
#define TL_ROPE_LAUNCH(TI, T)                                                                                   \
    tl_launch(rope_kv_write_kernel<TI, T>, dim3(n_tokens, chunks), dim3(threads), 0, s,                         \
              (const TI*)qkv, splits, plane, positions, table, slot_mapping, (T*)q_out, (T*)k_pages, (T*)v_pages, \
              n_heads, n_kv_heads, head_dim, page_size, table_rows, interleaved, rs)
    if (in_dtype == TL_F32 && dtype == TL_F32) return (int)TL_ROPE_LAUNCH(float, float);
    if (in_dtype == TL_BF16 && dtype == TL_BF16) return (int)TL_ROPE_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    if (in_dtype == TL_F32 && dtype == TL_BF16) return (int)TL_ROPE_LAUNCH(float, __nv_bfloat16);
#undef TL_ROPE_LAUNCH
    return TL_BAD_DTYPE;
}

// ---------------------------------------------------------------------------------------------
// The general form: a row [q heads | k heads | v heads | extra] in which keys and values have head
// counts and sizes of their own, only the first rot_dims coordinates of a q or k head are rotated
// (the table has rot_dims / 2 (cos, sin) pairs a position), and the extra columns leave as their
// sigmoids (gates that ride in the same projection).  k_pages: [pages, n_k_heads, page_size,
// head_dim]; v_pages: [pages, n_v_heads, page_size, v_head_dim].  One CTA per token.
template <typename TI, typename T>
__global__ void rope_store_kernel(const TI* __restrict__ proj, int splits, long long plane, const float* __restrict__ bias,
                                  const int* __restrict__ positions, const float* __restrict__ table,
                                  const int* __restrict__ slot_mapping, T* __restrict__ q_out, T* __restrict__ extra_out,
                                  T* __restrict__ k_pages, T* __restrict__ v_pages, int n_q_heads, int n_k_heads,
                                  int n_v_heads, int head_dim, int v_head_dim, int rot_dims, int n_extra, int page_size,
                                  int table_rows, int interleaved) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x;
    const int half = rot_dims >> 1;
    int pos = positions[t];
    (void)TL_CHECK(pos >= 0 && pos < table_rows, TL_DBG_POSITION);
    pos = pos < 0 ? 0 : (pos >= table_rows ? table_rows - 1 : pos);
    const float* cs = table + (size_t)pos * rot_dims;      // [half][2]
    const int qk_heads = n_q_heads + n_k_heads;
    const int n_qk = qk_heads * head_dim, n_v = n_v_heads * v_head_dim;
    const int width = n_qk + n_v + n_extra;
    const TI* src = proj + (size_t)t * width;
    int page = 0, slot = 0;
    bool write = k_pages != nullptr && n_k_heads > 0;
    if (write) {
        const int sm = slot_mapping[t];
        page = sm / page_size;
        slot = sm - page * page_size;
        if (!(TL_CHECK(sm >= 0, TL_DBG_SLOT) && tl_check_page(page))) write = false;
    }
    auto value = [&](int c) {
        float x = bias != nullptr ? bias[c] : 0.f;
        for (int sp = 0; sp < splits; ++sp) x += to_float(src[(size_t)sp * plane + c]);
        return x;
    };
    auto put_qk = [&](int head, int d, float x) {
        if (head < n_q_heads) q_out[((size_t)t * n_q_heads + head) * head_dim + d] = from_float<T>(x);
        else if (write)
            k_pages[(((size_t)page * n_k_heads + (head - n_q_heads)) * page_size + slot) * head_dim + d] = from_float<T>(x);
    };
    // a head's work items: `half` rotated pairs, then the coordinates that pass
    const int per_head = head_dim - half;
    const int first = blockIdx.y * blockDim.x + threadIdx.x, step = gridDim.y * blockDim.x;    // a token's work may be spread over CTAs
    for (int w = first; w < qk_heads * per_head; w += step) {
        const int head = w / per_head, i = w - head * per_head;
        if (i < half) {
            const int l0 = interleaved ? 2 * i : i, l1 = interleaved ? 2 * i + 1 : i + half;
            const float x0 = value(head * head_dim + l0), x1 = value(head * head_dim + l1);
            const float c = cs[2 * i], s = cs[2 * i + 1];
            put_qk(head, l0, x0 * c - x1 * s);
            put_qk(head, l1, x1 * c + x0 * s);
        } else {
            const int d = i + half;
            put_qk(head, d, value(head * head_dim + d));
        }
    }
    if (write && v_pages != nullptr) {
        for (int c = first; c < n_v; c += step) {
            const int head = c / v_head_dim, d = c - head * v_head_dim;
            v_pages[(((size_t)page * n_v_heads + head) * page_size + slot) * v_head_dim + d] = from_float<T>(value(n_qk + c));
        }
    }
    for (int c = first; c < n_extra; c += step)
        extra_out[(size_t)t * n_extra + c] = from_float<T>(1.f / (1.f + expf(-value(n_qk + n_v + c))));
}

// proj: [splits, n_tokens, width] of in_dtype, width = (n_q_heads + n_k_heads) * head_dim + n_v_heads * v_head_dim
// + n_extra; n_k_heads = n_v_heads = 0 for a run that reads another run's cache (pages may then be null);
// table: float32 [table_rows, rot_dims / 2, 2]; q_out [n_tokens, n_q_heads, head_dim], extra_out [n_tokens, n_extra]
// and the pages in dtype.  bias: float32 [width] or null, added to the row before anything else.
extern "C" int tl_rope_store(const void* proj, int in_dtype, int splits, const float* bias, const int* positions, const float* table,
                             const int* slot_mapping, void* q_out, void* extra_out, void* k_pages, void* v_pages, int dtype,
                             int n_tokens, int n_q_heads, int n_k_heads, int n_v_heads, int head_dim, int v_head_dim,
                             int rot_dims, int n_extra, int page_size, int table_rows, int interleaved, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (head_dim <= 0 || n_q_heads <= 0 || n_k_heads < 0 || n_v_heads < 0 || v_head_dim < 0 || n_extra < 0 || splits < 1 ||
        rot_dims < 0 || (rot_dims & 1) || rot_dims > head_dim || page_size <= 0 || table_rows <= 0)
        return TL_BAD_SIZE;
    if (n_k_heads > 0 && k_pages != nullptr && (slot_mapping == nullptr || (n_v_heads > 0 && v_pages == nullptr))) return TL_BAD_SIZE;
    if (n_extra > 0 && extra_out == nullptr) return TL_BAD_SIZE;
    const long long width = (long long)(n_q_heads + n_k_heads) * head_dim + (long long)n_v_heads * v_head_dim + n_extra;
    const long long plane = (long long)n_tokens * width;
    const int threads = width >= 2048 ? 256 : 128;
    // few tokens (decoding): a token's row is spread over several CTAs
    int by = 1;
    if (n_tokens < 256) {
        by = (int)((width + 2 * threads - 1) / (2 * threads));
        if (by > 16) by = 16;
    }
    cudaStream_t s = (cudaStream_t)stream;
#define TL_ROPE_STORE(TI, T)                                                                                          \
    tl_launch(rope_store_kernel<TI, T>, dim3(n_tokens, by), dim3(threads), 0, s, (const TI*)proj, splits, plane, bias, positions, \
              table, slot_mapping, (T*)q_out, (T*)extra_out, (T*)k_pages, (T*)v_pages, n_q_heads, n_k_heads, n_v_heads, \
              head_dim, v_head_dim, rot_dims, n_extra, page_size, table_rows, interleaved)
    if (in_dtype == TL_F32 && dtype == TL_F32) return (int)TL_ROPE_STORE(float, float);
    if (in_dtype == TL_BF16 && dtype == TL_BF16) return (int)TL_ROPE_STORE(__nv_bfloat16, __nv_bfloat16);
    if (in_dtype == TL_F32 && dtype == TL_BF16) return (int)TL_ROPE_STORE(float, __nv_bfloat16);
#undef TL_ROPE_STORE
    return TL_BAD_DTYPE;
}

// ---------------------------------------------------------------------------------------------
// What follows the stacked input projection of a latent-attention mixer whose row is
// [q latent | kv latent | rotated key part | extra]: both latents are RMS-normed under weights of their own
// (float32), the key part (all of its n_rot coordinates) is rotated by the position, [kv latent | key part]
// goes into the token's place of the one-headed pages ([pages, 1, page_size, n_latent + n_rot]), and the normed
// q latent and the sigmoids of the extra columns leave as tensors.  One CTA per token; the row is summed
// over the split-K planes twice (for the sums of squares, then for the results), which costs less than
// keeping it.
namespace {

__device__ __forceinline__ float block_sum_2(float v, float* part) {      // part: 33 floats of shared memory
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

template <typename TI, typename T>
__global__ void latent_store_kernel(const TI* __restrict__ proj, int splits, long long plane, const int* __restrict__ positions,
                                    const float* __restrict__ table, const int* __restrict__ slot_mapping,
                                    const float* __restrict__ q_norm, const float* __restrict__ latent_norm, float eps,
                                    T* __restrict__ q_out, T* __restrict__ extra_out, T* __restrict__ pages, int n_q, int n_latent,
                                    int n_rot, int n_extra, int page_size, int table_rows, int interleaved) {
    __shared__ float part[33];
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x;
    const int width = n_q + n_latent + n_rot + n_extra;
    const TI* src = proj + (size_t)t * width;
    auto value = [&](int c) {
        float x = 0.f;
        for (int sp = 0; sp < splits; ++sp) x += to_float(src[(size_t)sp * plane + c]);
        return x;
    };
    float sq = 0.f, sc = 0.f;
    for (int c = threadIdx.x; c < n_q + n_latent; c += blockDim.x) {
        const float v = value(c);
        if (c < n_q) sq = fmaf(v, v, sq);
        else sc = fmaf(v, v, sc);
    }
    const float rq = n_q > 0 ? rsqrtf(block_sum_2(sq, part) / (float)n_q + eps) : 0.f;
    const float rc = rsqrtf(block_sum_2(sc, part) / (float)n_latent + eps);
    int pos = positions[t];
    (void)TL_CHECK(pos >= 0 && pos < table_rows, TL_DBG_POSITION);
    pos = pos < 0 ? 0 : (pos >= table_rows ? table_rows - 1 : pos);
    const float* cs = table + (size_t)pos * n_rot;      // [n_rot / 2][2]
    const int sm = slot_mapping[t];
    const int page = sm / page_size, slot = sm - page * page_size;
    const bool write = pages != nullptr && TL_CHECK(sm >= 0, TL_DBG_SLOT) && tl_check_page(page);
    T* dst = pages + ((size_t)page * page_size + slot) * (n_latent + n_rot);
    for (int c = threadIdx.x; c < n_q; c += blockDim.x) q_out[(size_t)t * n_q + c] = from_float<T>(value(c) * rq * q_norm[c]);
    if (write) {
        for (int c = threadIdx.x; c < n_latent; c += blockDim.x) dst[c] = from_float<T>(value(n_q + c) * rc * latent_norm[c]);
        const int half = n_rot >> 1;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const int l0 = interleaved ? 2 * i : i, l1 = interleaved ? 2 * i + 1 : i + half;
            const float x0 = value(n_q + n_latent + l0), x1 = value(n_q + n_latent + l1);
            const float c = cs[2 * i], s = cs[2 * i + 1];
            dst[n_latent + l0] = from_float<T>(x0 * c - x1 * s);
            dst[n_latent + l1] = from_float<T>(x1 * c + x0 * s);
        }
    }
    for (int c = threadIdx.x; c < n_extra; c += blockDim.x)
        extra_out[(size_t)t * n_extra + c] = from_float<T>(1.f / (1.f + expf(-value(n_q + n_latent + n_rot + c))));
}

// out[t, h, o_off + d] = the first `rot` coordinates from x[t, h, x_off ...] rotated by the token's position; a thread per pair
template <typename T>
__global__ void rope_segment_kernel(const T* __restrict__ x, long long ldx, long long hsx, T* __restrict__ out, long long ldo,
                                    long long hso, const int* __restrict__ positions, const float* __restrict__ table,
                                    int table_rows, long long total, int n_heads, int rot, int interleaved) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int half = rot >> 1;
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(w % half);
        const long long th = w / half;
        const int h = (int)(th % n_heads);
        const long long t = th / n_heads;
        int pos = positions[t];
        (void)TL_CHECK(pos >= 0 && pos < table_rows, TL_DBG_POSITION);
        pos = pos < 0 ? 0 : (pos >= table_rows ? table_rows - 1 : pos);
        const float c = table[((size_t)pos * half + i) * 2], s = table[((size_t)pos * half + i) * 2 + 1];
        const int l0 = interleaved ? 2 * i : i, l1 = interleaved ? 2 * i + 1 : i + half;
        const T* src = x + t * ldx + h * hsx;
        T* dst = out + t * ldo + h * hso;
        const float x0 = to_float(src[l0]), x1 = to_float(src[l1]);
        dst[l0] = from_float<T>(x0 * c - x1 * s);
        dst[l1] = from_float<T>(x1 * c + x0 * s);
    }
}

}  // namespace

// proj: [splits, n_tokens, n_q + n_latent + n_rot + n_extra] of in_dtype; table: float32 [table_rows, n_rot / 2, 2];
// q_norm [n_q], latent_norm [n_latent]: float32; q_out [n_tokens, n_q], extra_out [n_tokens, n_extra] and pages
// [pages, 1, page_size, n_latent + n_rot] in dtype.
extern "C" int tl_latent_store(const void* proj, int in_dtype, int splits, const int* positions, const float* table,
                               const int* slot_mapping, const float* q_norm, const float* latent_norm, float eps, void* q_out,
                               void* extra_out, void* pages, int dtype, int n_tokens, int n_q, int n_latent, int n_rot,
                               int n_extra, int page_size, int table_rows, int interleaved, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (n_q < 0 || n_latent <= 0 || n_rot < 0 || (n_rot & 1) || n_extra < 0 || splits < 1 || page_size <= 0 || table_rows <= 0)
        return TL_BAD_SIZE;
    if ((n_extra > 0 && extra_out == nullptr) || (n_q > 0 && (q_out == nullptr || q_norm == nullptr)) || slot_mapping == nullptr)
        return TL_BAD_SIZE;
    const long long width = (long long)n_q + n_latent + n_rot + n_extra;
    const long long plane = (long long)n_tokens * width;
    const int threads = width >= 2048 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
#define TL_LATENT_STORE(TI, T)                                                                                              \
    tl_launch(latent_store_kernel<TI, T>, dim3(n_tokens), dim3(threads), 0, s, (const TI*)proj, splits, plane, positions, table, \
              slot_mapping, q_norm, latent_norm, eps, (T*)q_out, (T*)extra_out, (T*)pages, n_q, n_latent, n_rot, n_extra,      \
              page_size, table_rows, interleaved)
    if (in_dtype == TL_F32 && dtype == TL_F32) return (int)TL_LATENT_STORE(float, float);
    if (in_dtype == TL_BF16 && dtype == TL_BF16) return (int)TL_LATENT_STORE(__nv_bfloat16, __nv_bfloat16);
    if (in_dtype == TL_F32 && dtype == TL_BF16) return (int)TL_LATENT_STORE(float, __nv_bfloat16);
#undef TL_LATENT_STORE
    return TL_BAD_DTYPE;
}

// x, out: [n_tokens] rows of pitches ldx, ldo (elements), every head hsx, hso further on; the pointers name the first
// rotated coordinate of head 0 of token 0.  table: float32 [table_rows, rot / 2, 2].
extern "C" int tl_rope_segment(const void* x, long long ldx, long long hsx, void* out, long long ldo, long long hso, int dtype,
                               const int* positions, const float* table, int table_rows, int n_tokens, int n_heads, int rot,
                               int interleaved, void* stream) {
    if (n_tokens <= 0 || n_heads <= 0 || rot == 0) return TL_OK;
    if (rot < 0 || (rot & 1) || table_rows <= 0) return TL_BAD_SIZE;
    const long long total = (long long)n_tokens * n_heads * (rot / 2);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == TL_F32)
        return (int)tl_launch(rope_segment_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, (const float*)x, ldx, hsx, (float*)out,
                              ldo, hso, positions, table, table_rows, total, n_heads, rot, interleaved);
    if (dtype == TL_BF16)
        return (int)tl_launch(rope_segment_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, s, (const __nv_bfloat16*)x, ldx,
                              hsx, (__nv_bfloat16*)out, ldo, hso, positions, table, table_rows, total, n_heads, rot, interleaved);
    return TL_BAD_DTYPE;
}
