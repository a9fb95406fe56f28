// Feed-forwards made of many small experts of which every token uses a few, routed on the device.
//
// logits:   z = W_router x (float32; W_router may carry one more row, the shared expert's gate), a warp per
//           (token, row) for the few tokens of a decode step
// select:   s = softmax(z) over the experts (or sigmoid(z), each expert by itself), the `top` experts with the
//           largest s + correction are chosen (the lower index wins a tie), their weights are s * scale
//           (divided by their sum + renorm_eps first when renormalising); the extra row leaves as sigmoid(z).
//           With groups the experts form n_groups equal groups of neighbours, a group's score is the sum of
//           its group_top largest s + correction, and only experts of the keep_groups best groups can be chosen.
// plan:     the (token, choice) pairs sorted by expert, stably: for every expert where its rows
//           start, the sorted order and its inverse, and the list of row tiles (expert, first
//           row, rows) that the grouped products walk.  One CTA; nothing goes back to the host,
//           so a step's launches depend on its token count only.
// grouped product:  C[r, :] = act(W[e] A[src(r), :]) for the rows r of a tile, W[e] the tile's
//           expert; float32 multiply-adds on the CUDA cores, operands float32 or bfloat16.
// combine:  out[t] = sum_k weight[t, k] * Y[place(t, k)]  (+ gate[t] * shared[t]), summed in the
//           order of the choices, so a token's result does not depend on what else is in the batch.
#include "common.cuh"
#include <math.h>

namespace {

enum : int { ACT_NONE = -1, ACT_SILU = 0, ACT_GELU_TANH = 1, ACT_RELU2 = 2, ACT_CLAMPED_SWISH = 3 };

// the gated forms: act(gate) * up, or, clamped: g * sigmoid(alpha g) * (u + offset) with g = min(gate, limit), u = clamp(up, +-limit)
struct GateParams { float limit, alpha, up_offset; };

__device__ __forceinline__ float act_apply(float x, int act) {
    if (act == ACT_NONE) return x;
    if (act == ACT_SILU) return x / (1.f + expf(-x));
    if (act == ACT_GELU_TANH) return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    const float r = fmaxf(x, 0.f);
    return r * r;
}

__device__ __forceinline__ float gated_apply(float gate, float up, int act, const GateParams& gp) {
    if (act == ACT_CLAMPED_SWISH) {
        const float g = fminf(gate, gp.limit), u = fminf(fmaxf(up, -gp.limit), gp.limit);
        return g / (1.f + expf(-gp.alpha * g)) * (u + gp.up_offset);
    }
    return act_apply(gate, act) * up;
}

// Router logits of few tokens: grid (tokens, chunks of rows); the token's row in shared memory as float32,
// a warp per router row, sixteen bytes of the row per lane and turn.
template <typename T>
__global__ void __launch_bounds__(256) moe_logits_kernel(const T* __restrict__ x, const float* __restrict__ w_router,
                                                         float* __restrict__ logits, int dim, int n_rows) {
    extern __shared__ __align__(16) float xs[];
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) xs[d] = to_float(x[(size_t)t * dim + d]);
    __syncthreads();
    const int e = blockIdx.y * n_warps + warp;
    if (e >= n_rows) return;
    const float* wr = w_router + (size_t)e * dim;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (dim % 4 == 0 && (((size_t)w_router) & 15u) == 0) {
        int d = lane * 4;
        for (; d + 3 * 128 < dim; d += 4 * 128) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 w = *reinterpret_cast<const float4*>(wr + d + j * 128);
                const float4 v = *reinterpret_cast<const float4*>(xs + d + j * 128);
                acc[j] = fmaf(v.x, w.x, fmaf(v.y, w.y, fmaf(v.z, w.z, fmaf(v.w, w.w, acc[j]))));
            }
        }
        for (; d < dim; d += 128) {
            const float4 w = *reinterpret_cast<const float4*>(wr + d);
            const float4 v = *reinterpret_cast<const float4*>(xs + d);
            acc[0] = fmaf(v.x, w.x, fmaf(v.y, w.y, fmaf(v.z, w.z, fmaf(v.w, w.w, acc[0]))));
        }
    } else {
        for (int d = lane; d < dim; d += 32) acc[0] = fmaf(xs[d], wr[d], acc[0]);
    }
    const float total = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
    if (lane == 0) logits[(size_t)t * n_rows + e] = total;
}

// From the logits to the choice: a warp per token.  Shared memory per warp: scores, then what the choice looks at.
__global__ void __launch_bounds__(128) moe_select_kernel(const float* __restrict__ logits, const float* __restrict__ correction,
                                                         const float* __restrict__ logit_bias, int* __restrict__ chosen, float* __restrict__ weights,
                                                         float* __restrict__ gate, int n_tokens, int n_experts, int n_rows,
                                                         int top, float scale, int renormalize, int sigmoid_scores,
                                                         int n_groups, int keep_groups, int group_top, float renorm_eps) {
    extern __shared__ float sm[];
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= n_tokens) return;
    float* sc = sm + (size_t)warp * 2 * n_experts;
    float* ch = sc + n_experts;
    const float* z = logits + (size_t)t * n_rows;
    float mx = -INFINITY;
    // (the logits with their bias pass through ch[] on the way to the scores)
    for (int e = lane; e < n_experts; e += 32) {
        const float v = z[e] + (logit_bias != nullptr ? logit_bias[e] : 0.f);
        ch[e] = v;
        mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < n_experts; e += 32) sum += expf(ch[e] - mx);
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int e = lane; e < n_experts; e += 32) {
        const float s = sigmoid_scores ? 1.f / (1.f + expf(-ch[e])) : expf(ch[e] - mx) * inv;
        sc[e] = s;
        ch[e] = s + (correction != nullptr ? correction[e] : 0.f);
    }
    if (lane == 0 && gate != nullptr) gate[t] = 1.f / (1.f + expf(-z[n_experts]));
    __syncwarp();
    if (n_groups > 1) {
        // a lane per group (in turns): the sum of the group's group_top largest values; then the best groups are
        // marked one by one (the lower index wins a tie) and the experts of all others leave the choice
        const int per = n_experts / n_groups;
        float* gsc = sm + (size_t)(blockDim.x >> 5) * 2 * n_experts + (size_t)warp * n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float total_g = 0.f;
            float below = INFINITY;        // values are taken in falling order: (value, index) strictly after the last taken
            int below_at = -1;
            for (int k = 0; k < group_top && k < per; ++k) {
                float best = -INFINITY;
                int at = -1;
                for (int e = 0; e < per; ++e) {
                    const float v = ch[g * per + e];
                    const bool after = v < below || (v == below && e > below_at);
                    if (after && v > best) { best = v; at = e; }
                }
                if (at < 0) break;
                total_g += best;
                below = best;
                below_at = at;
            }
            gsc[g] = total_g;
        }
        __syncwarp();
        if (lane == 0) {
            // keep_groups rounds of selection; a kept group's score becomes +inf so that it is told from the rest below
            for (int k = 0; k < keep_groups; ++k) {
                float best = -INFINITY;
                int at = -1;
                for (int g = 0; g < n_groups; ++g) {
                    const float v = gsc[g];
                    if (v != INFINITY && (at < 0 || v > best)) { best = v; at = g; }
                }
                if (at >= 0) gsc[at] = INFINITY;
            }
        }
        __syncwarp();
        for (int e = lane; e < n_experts; e += 32)
            if (gsc[e / per] != INFINITY) ch[e] = -INFINITY;
        __syncwarp();
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = ch[e];
            if (v > best) { best = v; at = e; }       // (a lane walks upwards: the lower index stays on a tie)
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= n_experts) at = 0;                  // (all scores NaN: stay in bounds)
        if (lane == 0) {
            chosen[(size_t)t * top + k] = at;
            weights[(size_t)t * top + k] = sc[at];
            ch[at] = -INFINITY;
        }
        total += sc[at];
        __syncwarp();
    }
    if (lane == 0) {
        const float f = renormalize ? scale / (total + renorm_eps) : scale;
        for (int k = 0; k < top; ++k) weights[(size_t)t * top + k] *= f;
    }
}

// One CTA.  counts/offsets live in shared memory ([n_experts + 1] ints each).
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ chosen, int n_pairs, int n_experts, int tile_rows,
                                                        int* __restrict__ order, int* __restrict__ place,
                                                        int* __restrict__ tiles, int max_tiles, int* __restrict__ ends) {
    extern __shared__ int ism[];
    int* counts = ism;                    // [n_experts]
    int* offsets = ism + n_experts;       // [n_experts + 1]
    grid_launch_dependents();
    grid_dependency_wait();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int a = threadIdx.x; a < n_pairs; a += blockDim.x) {
        const int e = chosen[a];
        if (e >= 0 && e < n_experts) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0, n_tiles = 0;
        for (int e = 0; e < n_experts; ++e) {
            offsets[e] = off;
            for (int r = 0; r < counts[e] && n_tiles < max_tiles; r += tile_rows) {
                tiles[1 + 3 * n_tiles] = e;
                tiles[2 + 3 * n_tiles] = off + r;
                tiles[3 + 3 * n_tiles] = min(tile_rows, counts[e] - r);
                ++n_tiles;
            }
            off += counts[e];
            if (ends != nullptr) ends[e] = off;
        }
        offsets[n_experts] = off;
        tiles[0] = n_tiles;
    }
    __syncthreads();
    // stable placement: a warp per expert walks the pairs in order
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int e = warp; e < n_experts; e += n_warps) {
        if (counts[e] == 0) continue;
        int at = offsets[e];
        for (int a0 = 0; a0 < n_pairs; a0 += 32) {
            const int a = a0 + lane;
            const bool mine = a < n_pairs && chosen[a] == e;
            const unsigned m = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int pos = at + __popc(m & ((1u << lane) - 1u));
                order[pos] = a;
                place[a] = pos;
            }
            at += __popc(m);
        }
    }
}

constexpr int BN = 64, BK = 16, PAD = 4, NT = 256;

// grid: (N slabs, tiles).  BM rows of one expert per CTA (16 or 64), 64 columns, K walked 16 at a time.
template <typename T, typename TO, int BM>
__global__ void __launch_bounds__(NT) moe_gemm_kernel(const T* __restrict__ A, const T* __restrict__ W, TO* __restrict__ C,
                                                      const int* __restrict__ tiles, const int* __restrict__ order,
                                                      int gather_div, int N, int K, int act, long long w_expert, long long ldw) {
    constexpr int TM = BM / 16;
    __shared__ float As[BK][BM + PAD];
    __shared__ float Ws[BK][BN + PAD];
    __shared__ int src[BM];
    grid_launch_dependents();
    grid_dependency_wait();
    const int tile = blockIdx.y;
    if (tile >= tiles[0]) return;
    const int e = tiles[1 + 3 * tile], row0 = tiles[2 + 3 * tile], n_rows = tiles[3 + 3 * tile];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int n0 = blockIdx.x * BN;
    for (int r = tid; r < BM; r += NT) src[r] = r < n_rows ? (gather_div > 0 ? order[row0 + r] / gather_div : row0 + r) : -1;
    __syncthreads();
    W += (size_t)e * w_expert;
    const int lrow = tid >> 2, lk = (tid & 3) * 4;       // loads: a row (of 64) and four k
    float acc[TM][4];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        const int gn = n0 + lrow;
        const int srow = lrow < BM ? src[lrow] : -1;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int gk = k0 + lk + q;
            if (lrow < BM) As[lk + q][lrow] = (srow >= 0 && gk < K) ? to_float(A[(size_t)srow * K + gk]) : 0.f;
            Ws[lk + q][lrow] = (gn < N && gk < K) ? to_float(W[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 w4 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            const float w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int i = 0; i < TM; ++i) {
                const float a = As[k][ty * TM + i];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a, w[j], acc[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = ty * TM + i;
        if (r >= n_rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)(row0 + r) * N + gn] = from_float<TO>(act_apply(acc[i][j], act));
        }
    }
}

// One CTA per token.  y: [pairs][dim] in sorted order; shared: [splits][T][dim] or null.  The token's places and
// weights are fetched once; VEC: sixteen bytes of a row per thread and turn, four choices' loads in flight.
constexpr int COMBINE_TOP = 64;
template <typename T, typename TS, bool VEC>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights,
                                   const TS* __restrict__ shared, int shared_splits, long long shared_plane,
                                   const float* __restrict__ gate, T* __restrict__ out, int dim, int top) {
    __shared__ int pl[COMBINE_TOP];
    __shared__ float wt[COMBINE_TOP];
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x;
    if (threadIdx.x < top) {
        pl[threadIdx.x] = place[(size_t)t * top + threadIdx.x];
        wt[threadIdx.x] = weights[(size_t)t * top + threadIdx.x];
    }
    __syncthreads();
    const float g = gate != nullptr ? gate[t] : 1.f;
    if (VEC) {
        constexpr int N = Vec16<T>::N;
        for (int d = threadIdx.x * N; d < dim; d += blockDim.x * N) {
            float acc[N];
#pragma unroll
            for (int e = 0; e < N; ++e) acc[e] = 0.f;
            int k = 0;
            for (; k + 4 <= top; k += 4) {
                Vec16<T> v[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i].load(y + (size_t)pl[k + i] * dim + d);
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int e = 0; e < N; ++e) acc[e] = fmaf(wt[k + i], v[i].get(e), acc[e]);
            }
            for (; k < top; ++k) {
                Vec16<T> v;
                v.load(y + (size_t)pl[k] * dim + d);
#pragma unroll
                for (int e = 0; e < N; ++e) acc[e] = fmaf(wt[k], v.get(e), acc[e]);
            }
            if (shared != nullptr) {
#pragma unroll
                for (int e = 0; e < N; ++e) {
                    float sh = 0.f;
                    for (int sp = 0; sp < shared_splits; ++sp) sh += to_float(shared[(size_t)sp * shared_plane + (size_t)t * dim + d + e]);
                    acc[e] = fmaf(g, sh, acc[e]);
                }
            }
            Vec16<T> o;
#pragma unroll
            for (int e = 0; e < N; ++e) o.set(e, acc[e]);
            o.store(out + (size_t)t * dim + d);
        }
    } else {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            float acc = 0.f;
            for (int k = 0; k < top; ++k) acc = fmaf(wt[k], to_float(y[(size_t)pl[k] * dim + d]), acc);
            if (shared != nullptr) {
                float sh = 0.f;
                for (int s = 0; s < shared_splits; ++s) sh += to_float(shared[(size_t)s * shared_plane + (size_t)t * dim + d]);
                acc = fmaf(g, sh, acc);
            }
            out[(size_t)t * dim + d] = from_float<T>(acc);
        }
    }
}

// out[r] = x[order[r] / top]: every (token, choice) pair's input row, in sorted order
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ order, T* __restrict__ out, int dim, int top) {
    grid_launch_dependents();
    grid_dependency_wait();
    const T* src = x + (size_t)(order[blockIdx.x] / top) * dim;
    T* dst = out + (size_t)blockIdx.x * dim;
    constexpr int VEC = Vec16<T>::N;
    if (dim % VEC == 0 && (((size_t)x | (size_t)out) & 15u) == 0) {
        for (int d = threadIdx.x * VEC; d < dim; d += blockDim.x * VEC) {
            Vec16<T> v;
            v.load(src + d);
            v.store(dst + d);
        }
    } else {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = src[d];
    }
}

// All experts' hidden rows of a few tokens at once: u is [splits][T][n_experts * hidden + extra] (the product of
// the tokens with every expert's up matrix, stacked, and `extra` more columns of a shared expert); a column of
// expert e leaves as act(u) * weight(t, e), zero where the token did not choose e, an extra column as
// act(u) * gate[t] (or act(u)).
template <typename TI, typename TO>
__global__ void moe_scale_act_kernel(const TI* __restrict__ u, int splits, long long plane, const int* __restrict__ chosen,
                                     const float* __restrict__ weights, const float* __restrict__ gate, TO* __restrict__ out,
                                     int n_experts, int hidden, int extra, int top, int act, int gated, GateParams gp,
                                     GateParams gp_extra) {
    extern __shared__ float wexp[];      // [n_experts]: this token's weight per expert
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x, width = n_experts * hidden + extra;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) wexp[e] = 0.f;
    __syncthreads();
    if (threadIdx.x < top) wexp[chosen[(size_t)t * top + threadIdx.x]] = weights[(size_t)t * top + threadIdx.x];
    __syncthreads();
    const float g = gate != nullptr ? gate[t] : 1.f;
    if (gated) {
        // an expert's columns of u are [gate | up], hidden each, and after all experts a shared expert's [gate | up], extra
        // each; out has hidden columns per expert, gated(gate, up) * weight, and extra more, gated(gate, up) * g
        for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
            const bool own = c < n_experts * hidden;
            const int e = own ? c / hidden : n_experts, f = own ? c - e * hidden : c - n_experts * hidden;
            const float w = own ? wexp[e] : g;
            float v = 0.f;
            if (w != 0.f) {
                const size_t at = (size_t)t * 2 * width + (size_t)e * 2 * hidden + f;
                const int up_at = own ? hidden : extra;
                float a = 0.f, b = 0.f;
                for (int sp = 0; sp < splits; ++sp) {
                    a += to_float(u[(size_t)sp * plane + at]);
                    b += to_float(u[(size_t)sp * plane + at + up_at]);
                }
                v = gated_apply(a, b, act, own ? gp : gp_extra) * w;
            }
            out[(size_t)t * width + c] = from_float<TO>(v);
        }
        return;
    }
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
        const float w = c < n_experts * hidden ? wexp[c / hidden] : g;
        float v = 0.f;
        if (w != 0.f) {
            for (int sp = 0; sp < splits; ++sp) v += to_float(u[(size_t)sp * plane + (size_t)t * width + c]);
            v = act_apply(v, act) * w;
        }
        out[(size_t)t * width + c] = from_float<TO>(v);
    }
}

}  // namespace

// out[r] = x[order[r] / top] for the n_pairs sorted rows; x: [n_tokens][dim]
extern "C" int tl_moe_gather(const void* x, int dtype, const int* order, void* out, int n_pairs, int dim, int top, void* stream) {
    if (n_pairs <= 0) return TL_OK;
    if (dim <= 0 || top <= 0) return TL_BAD_SIZE;
    const dim3 grid(n_pairs), block(dim >= 2048 ? 256 : 128);
    if (dtype == TL_F32) return (int)tl_launch(moe_gather_kernel<float>, grid, block, 0, (cudaStream_t)stream, (const float*)x, order, (float*)out, dim, top);
    if (dtype == TL_BF16) return (int)tl_launch(moe_gather_kernel<__nv_bfloat16>, grid, block, 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, order, (__nv_bfloat16*)out, dim, top);
    return TL_BAD_DTYPE;
}

// u: [splits][n_tokens][n_experts * hidden + extra] of in_dtype; out: the same row shape in out_dtype.  gated != 0
// u is [splits][n_tokens][n_experts * 2 * hidden + 2 * extra], an expert's columns [gate | up] and last a shared
// expert's [gate | up], and out [n_tokens][n_experts * hidden + extra] holds gated(gate, up) * weight (or * gate[t]).
// act 3 (gated only): the clamped form with (limit, alpha, up_offset) for the experts and extra_limit for the extra columns.
extern "C" int tl_moe_scale_act(const void* u, int in_dtype, int splits, long long plane, const int* chosen, const float* weights,
                                const float* gate, void* out, int out_dtype, int n_tokens, int n_experts, int hidden, int extra,
                                int top, int act, int gated, float limit, float alpha, float up_offset, float extra_limit,
                                void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (n_experts <= 0 || hidden <= 0 || extra < 0 || top <= 0 || top > 1024 || splits < 1 || act < -1 || act > 3) return TL_BAD_SIZE;
    if (act == ACT_CLAMPED_SWISH && !gated) return TL_BAD_SIZE;
    const GateParams gp = {limit, alpha, up_offset}, gp_extra = {extra_limit, alpha, up_offset};
    const size_t smem = (size_t)n_experts * sizeof(float);
    if (smem > 48 * 1024) return TL_TOO_LARGE;
    const int width = n_experts * hidden + extra;
    int by = (width + 256 * 8 - 1) / (256 * 8);
    if (by < 1) by = 1;
    const dim3 grid(n_tokens, by), block(256);
    cudaStream_t s = (cudaStream_t)stream;
#define TL_MOE_SA(TI, TO)                                                                                             \
    tl_launch(moe_scale_act_kernel<TI, TO>, grid, block, smem, s, (const TI*)u, splits, plane, chosen, weights, gate, (TO*)out, \
              n_experts, hidden, extra, top, act, gated, gp, gp_extra)
    if (in_dtype == TL_F32 && out_dtype == TL_F32) return (int)TL_MOE_SA(float, float);
    if (in_dtype == TL_F32 && out_dtype == TL_BF16) return (int)TL_MOE_SA(float, __nv_bfloat16);
    if (in_dtype == TL_BF16 && out_dtype == TL_BF16) return (int)TL_MOE_SA(__nv_bfloat16, __nv_bfloat16);
#undef TL_MOE_SA
    return TL_BAD_DTYPE;
}

// Router logits of few tokens: x [n_tokens][dim] of dtype against w_router float32 [n_rows][dim], float32 out.
// (Many tokens take the float32 product of gemm_simt instead, which reads the router once per 64 tokens.)
extern "C" int tl_moe_logits(const void* x, int dtype, const float* w_router, float* logits, int n_tokens, int dim, int n_rows,
                             void* stream) {
    if (n_tokens <= 0 || n_rows <= 0) return TL_OK;
    if (dim <= 0) return TL_BAD_SIZE;
    const size_t smem = (size_t)dim * sizeof(float);
    if (smem > 48 * 1024) return TL_TOO_LARGE;
    const dim3 grid(n_tokens, (n_rows + 7) / 8), block(256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == TL_F32) return (int)tl_launch(moe_logits_kernel<float>, grid, block, smem, s, (const float*)x, w_router, logits, dim, n_rows);
    if (dtype == TL_BF16)
        return (int)tl_launch(moe_logits_kernel<__nv_bfloat16>, grid, block, smem, s, (const __nv_bfloat16*)x, w_router, logits, dim, n_rows);
    return TL_BAD_DTYPE;
}

// logits: float32 [n_tokens][n_rows], n_rows = n_experts (+ 1 with gate != null: the shared expert's gate);
// correction, logit_bias (added to the logits before anything else): float32 [n_experts] or null; chosen: int32 [n_tokens][top]; weights: float32 [n_tokens][top];
// gate: float32 [n_tokens] or null.
// sigmoid_scores != 0: every expert's score is the sigmoid of its own logit.  n_groups > 1: see the top of this file
// (n_groups divides n_experts; keep_groups * n_experts / n_groups >= top).
extern "C" int tl_moe_select(const float* logits, const float* correction, const float* logit_bias, int* chosen, float* weights,
                             float* gate, int n_tokens, int n_experts, int top, float scale, int renormalize, int sigmoid_scores,
                             int n_groups, int keep_groups, int group_top, float renorm_eps, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (n_experts <= 0 || top <= 0 || top > n_experts) return TL_BAD_SIZE;
    if (n_groups < 1 || n_experts % n_groups != 0 || keep_groups < 1 || keep_groups > n_groups || group_top < 1 ||
        (long long)keep_groups * (n_experts / n_groups) < top)
        return TL_BAD_SIZE;
    const int n_rows = n_experts + (gate != nullptr ? 1 : 0);
    const size_t smem = (size_t)4 * (2 * n_experts + n_groups) * sizeof(float);
    if (smem > 48 * 1024) return TL_TOO_LARGE;
    return (int)tl_launch(moe_select_kernel, dim3((n_tokens + 3) / 4), dim3(128), smem, (cudaStream_t)stream, logits, correction,
                          logit_bias, chosen, weights, gate, n_tokens, n_experts, n_rows, top, scale, renormalize, sigmoid_scores,
                          n_groups, keep_groups, group_top, renorm_eps);
}

// rows of a tile for this many (token, choice) pairs, and how many tiles there can be at most
extern "C" int tl_moe_tile_rows(int n_pairs) { return n_pairs <= 512 ? 16 : 64; }
extern "C" int tl_moe_max_tiles(int n_pairs, int n_experts) {
    const int rows = tl_moe_tile_rows(n_pairs);
    const long long most = (long long)(n_pairs + rows - 1) / rows + n_experts;
    return (int)(most < n_pairs ? most : n_pairs);
}

// chosen: int32 [n_pairs]; order, place: int32 [n_pairs]; tiles: int32 [1 + 3 * max_tiles] (count, then
// expert, first row, rows of every tile)
// ends: int32 [n_experts] or null: where every expert's rows end in the sorted order
extern "C" int tl_moe_plan(const int* chosen, int n_pairs, int n_experts, int* order, int* place, int* tiles, int* ends,
                           void* stream) {
    if (n_pairs <= 0) return TL_OK;
    if (n_experts <= 0 || n_experts > 4096) return TL_BAD_SIZE;
    const size_t smem = (size_t)(2 * n_experts + 1) * sizeof(int);
    return (int)tl_launch(moe_plan_kernel, dim3(1), dim3(1024), smem, (cudaStream_t)stream, chosen, n_pairs, n_experts,
                          tl_moe_tile_rows(n_pairs), order, place, tiles, tl_moe_max_tiles(n_pairs, n_experts), ends);
}

// The experts' products over the sorted rows.  A: [rows][K]; with gather_div > 0 row r of the sorted order
// reads A[order[r] / gather_div] (a token's row for each of its choices), else A[r].  W: expert e's [N][K]
// matrix starts w_expert elements after expert e - 1's and its rows lie ldw elements apart;
// C: [n_pairs][N] in sorted order.  act: -1 none, 0 silu, 1 gelu (tanh form), 2 squared relu.
extern "C" int tl_moe_gemm(const void* A, const void* W, void* C, int dtype, const int* tiles, const int* order,
                           int gather_div, int n_pairs, int n_experts, int N, int K, int act, long long w_expert,
                           long long ldw, void* stream) {
    if (n_pairs <= 0 || N <= 0) return TL_OK;
    if (K <= 0 || act < -1 || act > 2) return TL_BAD_SIZE;
    const int max_tiles = tl_moe_max_tiles(n_pairs, n_experts);
    if (max_tiles > 65535) return TL_BAD_SIZE;
    const dim3 grid((N + BN - 1) / BN, max_tiles), block(NT);
    cudaStream_t s = (cudaStream_t)stream;
    const bool small = tl_moe_tile_rows(n_pairs) == 16;
#define TL_MOE_GEMM(T, BM) \
    tl_launch(moe_gemm_kernel<T, T, BM>, grid, block, 0, s, (const T*)A, (const T*)W, (T*)C, tiles, order, gather_div, N, K, act, w_expert, ldw)
    if (dtype == TL_F32) return (int)(small ? TL_MOE_GEMM(float, 16) : TL_MOE_GEMM(float, 64));
    if (dtype == TL_BF16) return (int)(small ? TL_MOE_GEMM(__nv_bfloat16, 16) : TL_MOE_GEMM(__nv_bfloat16, 64));
#undef TL_MOE_GEMM
    return TL_BAD_DTYPE;
}

// y: [n_tokens * top][dim] of dtype in sorted order; shared: [shared_splits][n_tokens][dim] of shared_dtype or
// null; gate: float32 [n_tokens] or null; out: [n_tokens][dim] of dtype.
extern "C" int tl_moe_combine(const void* y, int dtype, const int* place, const float* weights, const void* shared,
                              int shared_dtype, int shared_splits, long long shared_plane, const float* gate, void* out,
                              int n_tokens, int dim, int top, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (dim <= 0 || top <= 0 || top > COMBINE_TOP) return TL_BAD_SIZE;
    const int n16 = dtype == TL_F32 ? 4 : 8;          // elements in sixteen bytes
    const bool vec = dim % n16 == 0 && aligned16(y) && aligned16(out);
    int threads = vec ? ((dim / n16 + 31) / 32) * 32 : (dim >= 1024 ? 256 : 128);
    threads = threads < 64 ? 64 : (threads > 256 ? 256 : threads);
    const dim3 grid(n_tokens), block(threads);
    cudaStream_t s = (cudaStream_t)stream;
#define TL_MOE_COMBINE(T, TS)                                                                                          \
    (vec ? tl_launch(moe_combine_kernel<T, TS, true>, grid, block, 0, s, (const T*)y, place, weights, (const TS*)shared,   \
                     shared_splits, shared_plane, gate, (T*)out, dim, top)                                             \
         : tl_launch(moe_combine_kernel<T, TS, false>, grid, block, 0, s, (const T*)y, place, weights, (const TS*)shared,  \
                     shared_splits, shared_plane, gate, (T*)out, dim, top))
    if (dtype == TL_F32 && (shared == nullptr || shared_dtype == TL_F32)) return (int)TL_MOE_COMBINE(float, float);
    if (dtype == TL_BF16 && (shared == nullptr || shared_dtype == TL_BF16)) return (int)TL_MOE_COMBINE(__nv_bfloat16, __nv_bfloat16);
    if (dtype == TL_BF16 && shared_dtype == TL_F32) return (int)TL_MOE_COMBINE(__nv_bfloat16, float);
#undef TL_MOE_COMBINE
    return TL_BAD_DTYPE;
}
