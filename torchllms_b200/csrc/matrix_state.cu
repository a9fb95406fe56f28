// Mixers whose per-request state is a matrix per head, and what stands around them.
//
// short_conv:        causal convolution over time on every channel, a few taps; a request's last
//                    taps - 1 inputs are its state.  out_t = sum_j w[c][j] x_(t - taps + 1 + j)
//                    (+ x_t), then an optional silu.
// recurrence_prep:   q or k of a recurrence in float32: rotated by position (coordinate i with
//                    i + rot/2) or made a unit vector per head, then scaled.
// linear_recurrence: per head a dk x dv matrix S in float32 that every token updates and reads:
//                      fixed decay:  S <- d_h S + k v^T
//                      delta rule:   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T
//                    and o = S^T q.  Tokens are walked in order, so a result does not depend on how
//                    a request was cut into portions.
// head_norm_gate:    every head of o divided by its root mean square, times a weight shared by the
//                    heads (or none), times silu(gate).
//
// All arithmetic is float32; inputs that come from a product may be bfloat16 and may be column
// ranges of a wider row (a row pitch goes with every such pointer).  State rows may be fields of a
// wider per-request row too (a slot pitch goes with the state pointer).
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 8;
constexpr int CONV_TOKENS = 8;     // tokens a thread of the convolution walks
constexpr int NT = 128;

struct ConvParams {
    const void* x;           // [T] rows of pitch ldx, C channels used
    long long ldx;
    const float* w;          // [C][taps], the last column the current token's
    const float* bias;       // [C] or null: added to the sum before the activation
    float* state;            // [slots] rows of pitch state_pitch, each [taps - 1][C]; null with taps == 1
    long long state_pitch;
    const int* q_start;      // [B + 1]
    const int* state_slot;   // [B]
    const int* fresh;        // [B]
    void* out;               // [T][C]
    int C, taps, act, residual, n_chunks;
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

// the input `rel` places from the portion's start (negative: from the state, zero for a fresh request)
template <typename TI>
__device__ __forceinline__ float conv_input(const ConvParams& p, const TI* x, int start, int rel, int c, const float* st, bool fresh) {
    if (rel >= 0) return to_float(x[(size_t)(start + rel) * p.ldx + c]);
    if (fresh || st == nullptr) return 0.f;
    return st[(size_t)(p.taps - 1 + rel) * p.C + c];
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(NT) short_conv_kernel(const ConvParams p) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int c = blockIdx.x * NT + threadIdx.x;
    const int chunk = blockIdx.y, b = blockIdx.z;
    if (c >= p.C) return;
    const int start = p.q_start[b], len = p.q_start[b + 1] - start;
    const int r0 = chunk * CONV_TOKENS, n = min(len - r0, CONV_TOKENS);
    if (n <= 0) return;
    const bool fresh = p.fresh[b] != 0;
    float* st = p.state != nullptr ? p.state + (size_t)p.state_slot[b] * p.state_pitch : nullptr;
    const TI* x = reinterpret_cast<const TI*>(p.x);
    float in[CONV_TOKENS + MAX_TAPS - 1], w[MAX_TAPS];
    const int back = p.taps - 1;
#pragma unroll
    for (int i = 0; i < CONV_TOKENS + MAX_TAPS - 1; ++i)
        in[i] = (i < n + back) ? conv_input<TI>(p, x, start, r0 - back + i, c, st, fresh) : 0.f;
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) w[j] = j < p.taps ? p.w[(size_t)c * p.taps + j] : 0.f;
    TO* out = reinterpret_cast<TO*>(p.out);
    const float cb = p.bias != nullptr ? p.bias[c] : 0.f;
#pragma unroll
    for (int i = 0; i < CONV_TOKENS; ++i) {
        if (i < n) {
            float acc = cb;
#pragma unroll
            for (int j = 0; j < MAX_TAPS; ++j)
                if (j < p.taps) acc = fmaf(w[j], in[i + j], acc);
            if (p.residual) acc += in[i + back];
            if (p.act == 1) acc = silu_f(acc);
            out[(size_t)(start + r0 + i) * p.C + c] = from_float<TO>(acc);
        }
    }
    // a step of short portions only: this thread is the only one that reads or writes its channel's state
    if (p.n_chunks == 1 && st != nullptr) {
#pragma unroll
        for (int i = 0; i < CONV_TOKENS + MAX_TAPS - 1; ++i) {       // in[] holds the places -back .. n - 1: its last `back` are the state
            const int r = i - n;
            if (r >= 0 && r < back) st[(size_t)r * p.C + c] = in[i];
        }
    }
}

// the state after a step with longer portions: every (request, channel) by one thread, reads before writes
template <typename TI>
__global__ void __launch_bounds__(NT) short_conv_state_kernel(const ConvParams p) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int c = blockIdx.x * NT + threadIdx.x, b = blockIdx.z;
    if (c >= p.C) return;
    const int start = p.q_start[b], len = p.q_start[b + 1] - start;
    if (len <= 0) return;
    const bool fresh = p.fresh[b] != 0;
    float* st = p.state + (size_t)p.state_slot[b] * p.state_pitch;
    const TI* x = reinterpret_cast<const TI*>(p.x);
    const int back = p.taps - 1;
    float keep[MAX_TAPS - 1];
#pragma unroll
    for (int r = 0; r < MAX_TAPS - 1; ++r) keep[r] = r < back ? conv_input<TI>(p, x, start, len - back + r, c, st, fresh) : 0.f;
#pragma unroll
    for (int r = 0; r < MAX_TAPS - 1; ++r)
        if (r < back) st[(size_t)r * p.C + c] = keep[r];
}

struct PrepParams {
    const void* x;           // [T] rows of pitch ldx, n_heads * head_dim columns used
    long long ldx;
    float* out;              // [T][n_heads * head_dim]
    const int* positions;    // [T] or null
    const float* table;      // [positions][rot / 2][2] (cos, sin) or null
    int table_rows;
    int n_heads, head_dim, rot, unit;
    float scale, unit_eps;
    long long n_rows;        // T * n_heads
};

// a warp per (token, head)
template <typename TI>
__global__ void __launch_bounds__(NT) recurrence_prep_kernel(const PrepParams p) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (NT / 32) + (threadIdx.x >> 5);
    if (row >= p.n_rows) return;
    const long long t = row / p.n_heads;
    const int h = (int)(row - t * p.n_heads);
    const TI* x = reinterpret_cast<const TI*>(p.x) + (size_t)t * p.ldx + (size_t)h * p.head_dim;
    float* out = p.out + (size_t)row * p.head_dim;
    if (p.unit) {
        float ssq = 0.f;
        for (int d = lane; d < p.head_dim; d += 32) {
            const float v = to_float(x[d]);
            ssq = fmaf(v, v, ssq);
        }
        const float r = rsqrtf(warp_sum(ssq) + p.unit_eps) * p.scale;
        for (int d = lane; d < p.head_dim; d += 32) out[d] = to_float(x[d]) * r;
        return;
    }
    const int half = p.rot / 2;
    int pos = p.positions != nullptr ? p.positions[t] : 0;
    if (!TL_CHECK(pos >= 0 && pos < p.table_rows, TL_DBG_POSITION)) pos = 0;
    const float* cs = p.table != nullptr ? p.table + (size_t)pos * half * 2 : nullptr;
    for (int d = lane; d < p.head_dim; d += 32) {
        float v = to_float(x[d]);
        if (d < p.rot && cs != nullptr) {
            const int i = d < half ? d : d - half;
            const float c = cs[2 * i], s = cs[2 * i + 1];
            const float other = to_float(x[d < half ? d + half : d - half]);
            v = d < half ? v * c - other * s : v * c + other * s;
        }
        out[d] = v * p.scale;
    }
}

struct HeadNormParams {
    const float* o;          // [T][H * hd]
    const void* gate;        // [T] rows of pitch ldg, H * hd columns
    long long ldg;
    const float* weight;     // [hd] or null
    void* out;               // [T][H * hd]
    int n_heads, head_dim;
    float eps;
    long long n_rows;
};

template <typename TI, typename TO>
__global__ void __launch_bounds__(NT) head_norm_gate_kernel(const HeadNormParams p) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (NT / 32) + (threadIdx.x >> 5);
    if (row >= p.n_rows) return;
    const long long t = row / p.n_heads;
    const int h = (int)(row - t * p.n_heads);
    const float* o = p.o + (size_t)row * p.head_dim;
    const TI* g = reinterpret_cast<const TI*>(p.gate) + (size_t)t * p.ldg + (size_t)h * p.head_dim;
    TO* out = reinterpret_cast<TO*>(p.out) + (size_t)row * p.head_dim;
    float ssq = 0.f;
    for (int d = lane; d < p.head_dim; d += 32) ssq = fmaf(o[d], o[d], ssq);
    const float r = rsqrtf(warp_sum(ssq) / (float)p.head_dim + p.eps);
    for (int d = lane; d < p.head_dim; d += 32) {
        float v = o[d] * r;
        if (p.weight != nullptr) v *= p.weight[d];
        out[d] = from_float<TO>(v * silu_f(to_float(g[d])));
    }
}


constexpr int RC_TOKENS = 16;      // tokens fetched into shared memory at a time

struct RecurrenceParams {
    const float* q;          // [T][G * dk]
    const float* k;          // [T][G * dk]
    const void* v;           // [T] rows of pitch ldv, H * dv columns
    long long ldv;
    const void* beta;        // [T] rows of pitch ldg, H columns (delta rule) or null
    const void* gate;        // [T] rows of pitch ldg, H columns (delta rule)
    long long ldg;
    const float* decay;      // [H]: the fixed decay, or (delta rule) exp(A_log)
    const float* decay_bias; // [H] (delta rule)
    float* state;            // [slots] rows of pitch state_pitch, each [H][dv][dk]: a column's keys lie side by side
    long long state_pitch;
    const int* q_start;
    const int* state_slot;
    const int* fresh;
    float* out;              // [T][H * dv]
    int H, G, dk, dv;
};

// A CTA of 4 warps per (4 * 32 / KS columns, head, request); a warp's lanes are 32 / KS columns x KS slices of the key
// size: lane (jj, s) keeps S[s R + r][j] for r < R in registers (KS R >= dk; rows past dk stay zero).  The state is
// stored with a column's keys side by side, so a lane's slice is one run of R floats.  q and k of 16 tokens lie in
// shared memory, a slice's R floats followed by 4 unused ones (slices then start in different banks), zeros past
// dk, so a lane reads its slice four floats at a time and nothing in the loop over tokens asks where dk ends; the
// next 16 tokens are on their way from global memory into registers meanwhile.  The more slices, the more warps a
// head gives and the shorter a lane's chain per token, at one more shuffle per doubling.
//
// Both sums over the key size that a token needs are taken from the state as the token finds it, in one pass and one
// round of shuffles, because the state it leaves differs by a rank-one term whose share is known beforehand:
//     decay:  o = S_t^T q = d (S^T q) + v (k . q)
//     delta:  S^T k and S^T q of the decayed state are g (S^T k) and g (S^T q);  u = beta (v - g S^T k);
//             o = g (S^T q) + u (k . q)
// with S the state before the token and k . q taken once per token when its rows arrive.  That leaves one
// dependent chain per token (the update of S) instead of two reductions one after the other.
template <int R, int KS, bool DELTA, typename TV>
__global__ void __launch_bounds__(NT) linear_recurrence_kernel(const RecurrenceParams p) {
    extern __shared__ __align__(16) float smem[];
    grid_launch_dependents();
    grid_dependency_wait();
    constexpr int SLOT = R + 4;                          // a slice in shared memory
    constexpr int PITCH = KS * SLOT;
    constexpr int COLS = 4 * (32 / KS);                  // columns of a CTA
    constexpr int XN = (PITCH + 31) / 32;                // places of a row that a lane brings
    constexpr int TPW = RC_TOKENS / (NT / 32);           // tokens of the 16 that a warp brings
    constexpr int V_EACH = (RC_TOKENS * COLS + NT - 1) / NT;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int s = lane & (KS - 1), jj = lane / KS;
    const int h = blockIdx.y, b = blockIdx.z;
    const int jl = warp * (32 / KS) + jj, j = blockIdx.x * COLS + jl;
    const bool live = j < p.dv;
    const int g = h / (p.H / p.G);
    const int start = p.q_start[b], len = p.q_start[b + 1] - start;
    if (len <= 0) return;
    float* sq = smem;                                   // [RC_TOKENS][PITCH]
    float* sk = sq + RC_TOKENS * PITCH;                 // [RC_TOKENS][PITCH]
    float* sv = sk + RC_TOKENS * PITCH;                 // [RC_TOKENS][COLS]
    float* sg = sv + RC_TOKENS * COLS;                  // [RC_TOKENS]: the token's decay
    float* sb = sg + RC_TOKENS;                         // [RC_TOKENS]: the token's beta
    float* skq = sb + RC_TOKENS;                        // [RC_TOKENS]: k . q
    float* st = p.state + (size_t)p.state_slot[b] * p.state_pitch + ((size_t)h * p.dv + (live ? j : 0)) * p.dk;
    float S[R];
    const bool fresh = p.fresh[b] != 0;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = s * R + r;
        S[r] = (!fresh && live && i < p.dk) ? st[i] : 0.f;
    }
    const float fixed = DELTA ? 0.f : p.decay[h];
    const float rate = DELTA ? p.decay[h] : 0.f, dbias = DELTA ? p.decay_bias[h] : 0.f;
    const TV* v = reinterpret_cast<const TV*>(p.v);
    const int qk_row = p.G * p.dk;
    // a warp brings whole rows (tokens warp, warp + 4, ...), a lane the places lane, lane + 32, ... of each: which
    // coordinate of the head a place holds (-1: the unused floats behind a slice, and what lies past dk) is the same
    // for every token
    int coord[XN];
#pragma unroll
    for (int it = 0; it < XN; ++it) {
        const int x = lane + 32 * it, sl = x / SLOT, r = x - sl * SLOT, d = sl * R + r;
        coord[it] = (x < PITCH && r < R && d < p.dk) ? d : -1;
    }
    float fq[TPW * XN], fk[TPW * XN], fv[V_EACH], fa = 0.f, fb = 0.f;
    // the rows of the 16 tokens from t0 on, into registers (zeros past the portion's end)
    auto fetch = [&](int t0) {
        const int n = min(len - t0, RC_TOKENS);
#pragma unroll
        for (int w = 0; w < TPW; ++w) {
            const int tt = warp + (NT / 32) * w;
            const size_t row = (size_t)(start + t0 + tt) * qk_row + (size_t)g * p.dk;
#pragma unroll
            for (int it = 0; it < XN; ++it) {
                const bool in = tt < n && coord[it] >= 0;
                fq[w * XN + it] = in ? p.q[row + coord[it]] : 0.f;
                fk[w * XN + it] = in ? p.k[row + coord[it]] : 0.f;
            }
        }
#pragma unroll
        for (int i = 0; i < V_EACH; ++i) {
            const int e = threadIdx.x + i * NT, tt = e / COLS, c = e - tt * COLS, col = blockIdx.x * COLS + c;
            fv[i] = (tt < n && col < p.dv) ? to_float(v[(size_t)(start + t0 + tt) * p.ldv + (size_t)h * p.dv + col]) : 0.f;
        }
        if (DELTA && threadIdx.x < n) {
            const size_t at = (size_t)(start + t0 + threadIdx.x) * p.ldg + h;
            fa = to_float(reinterpret_cast<const TV*>(p.gate)[at]);
            fb = to_float(reinterpret_cast<const TV*>(p.beta)[at]);
        }
    };
    fetch(0);
    for (int t0 = 0; t0 < len; t0 += RC_TOKENS) {
        const int n = min(len - t0, RC_TOKENS);
        __syncthreads();                                // the tokens before have been used
#pragma unroll
        for (int w = 0; w < TPW; ++w) {
            const int tt = warp + (NT / 32) * w;
            float acc = 0.f;                            // k . q of the token, from the registers that hold its rows
#pragma unroll
            for (int it = 0; it < XN; ++it) {
                const int x = lane + 32 * it;
                if (x < PITCH) {
                    sq[tt * PITCH + x] = fq[w * XN + it];
                    sk[tt * PITCH + x] = fk[w * XN + it];
                }
                acc = fmaf(fq[w * XN + it], fk[w * XN + it], acc);
            }
            acc = warp_sum(acc);
            if (lane == 0) skq[tt] = acc;
        }
#pragma unroll
        for (int i = 0; i < V_EACH; ++i)
            if (threadIdx.x + i * NT < RC_TOKENS * COLS) sv[threadIdx.x + i * NT] = fv[i];
        if (DELTA && threadIdx.x < n) {
            const float a = fa + dbias;
            const float soft = a > 20.f ? a : log1pf(expf(a));
            sg[threadIdx.x] = expf(-rate * soft);
            sb[threadIdx.x] = 1.f / (1.f + expf(-fb));
        }
        __syncthreads();
        if (t0 + RC_TOKENS < len) fetch(t0 + RC_TOKENS);  // in flight while these tokens are walked
        for (int tt = 0; tt < n; ++tt) {
            const float4* kt = reinterpret_cast<const float4*>(sk + tt * PITCH + s * SLOT);
            const float4* qt = reinterpret_cast<const float4*>(sq + tt * PITCH + s * SLOT);
            const float vt = sv[tt * COLS + jl], kq = skq[tt];
            float4 kv[R / 4];
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f, o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int r = 0; r < R / 4; ++r) {
                kv[r] = kt[r];
                const float4 qv = qt[r];
                o0 = fmaf(S[4 * r], qv.x, o0);
                o1 = fmaf(S[4 * r + 1], qv.y, o1);
                o2 = fmaf(S[4 * r + 2], qv.z, o2);
                o3 = fmaf(S[4 * r + 3], qv.w, o3);
                if (DELTA) {
                    d0 = fmaf(S[4 * r], kv[r].x, d0);
                    d1 = fmaf(S[4 * r + 1], kv[r].y, d1);
                    d2 = fmaf(S[4 * r + 2], kv[r].z, d2);
                    d3 = fmaf(S[4 * r + 3], kv[r].w, d3);
                }
            }
            float oq = (o0 + o1) + (o2 + o3), dot = (d0 + d1) + (d2 + d3);
#pragma unroll
            for (int off = 1; off < KS; off <<= 1) {
                oq += __shfl_xor_sync(0xffffffffu, oq, off);
                if (DELTA) dot += __shfl_xor_sync(0xffffffffu, dot, off);
            }
            float o;
            if (DELTA) {
                const float gt = sg[tt];
                const float u = sb[tt] * (vt - gt * dot);
                o = fmaf(u, kq, gt * oq);
#pragma unroll
                for (int r = 0; r < R / 4; ++r) {
                    S[4 * r] = fmaf(kv[r].x, u, gt * S[4 * r]);
                    S[4 * r + 1] = fmaf(kv[r].y, u, gt * S[4 * r + 1]);
                    S[4 * r + 2] = fmaf(kv[r].z, u, gt * S[4 * r + 2]);
                    S[4 * r + 3] = fmaf(kv[r].w, u, gt * S[4 * r + 3]);
                }
            } else {
                o = fmaf(vt, kq, fixed * oq);
#pragma unroll
                for (int r = 0; r < R / 4; ++r) {
                    S[4 * r] = fmaf(fixed, S[4 * r], kv[r].x * vt);
                    S[4 * r + 1] = fmaf(fixed, S[4 * r + 1], kv[r].y * vt);
                    S[4 * r + 2] = fmaf(fixed, S[4 * r + 2], kv[r].z * vt);
                    S[4 * r + 3] = fmaf(fixed, S[4 * r + 3], kv[r].w * vt);
                }
            }
            if (s == 0 && live) p.out[(size_t)(start + t0 + tt) * p.H * p.dv + (size_t)h * p.dv + j] = o;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = s * R + r;
        if (live && i < p.dk) st[i] = S[r];
    }
}

}  // namespace

// x: [n_tokens] rows of pitch ldx (elements of in_dtype), `channels` used; w: float32 [channels][taps]; state: float32
// rows of pitch state_pitch per slot, [taps - 1][channels] each (null with taps == 1); out: [n_tokens][channels].
// act: 0 none, 1 silu.  residual: x_t is added to the sum before the activation.  bias: float32 [channels] or null,
// added to the sum as well.
extern "C" int tl_short_conv(const void* x, int in_dtype, long long ldx, const float* w, const float* bias, float* state, long long state_pitch,
                             const int* q_start, const int* state_slot, const int* fresh, void* out, int out_dtype,
                             int n_tokens, int n_seqs, int channels, int taps, int max_q_len, int act, int residual,
                             void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return TL_OK;
    if (channels <= 0 || taps < 1 || taps > MAX_TAPS || max_q_len <= 0 || n_seqs > 65535 || act < 0 || act > 1) return TL_BAD_SIZE;
    if (taps > 1 && state == nullptr) return TL_BAD_SIZE;
    ConvParams p;
    p.x = x; p.ldx = ldx; p.w = w; p.bias = bias; p.state = taps > 1 ? state : nullptr; p.state_pitch = state_pitch;
    p.q_start = q_start; p.state_slot = state_slot; p.fresh = fresh; p.out = out;
    p.C = channels; p.taps = taps; p.act = act; p.residual = residual;
    p.n_chunks = (max_q_len + CONV_TOKENS - 1) / CONV_TOKENS;
    if (p.n_chunks > 65535) return TL_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((channels + NT - 1) / NT, p.n_chunks, n_seqs), block(NT);
    cudaError_t e;
#define TL_CONV(TI, TO)                                                                                        \
    do {                                                                                                       \
        e = tl_launch(short_conv_kernel<TI, TO>, grid, block, 0, s, p);                                        \
        if (e == cudaSuccess && p.n_chunks > 1 && p.state != nullptr)                                          \
            e = tl_launch(short_conv_state_kernel<TI>, dim3(grid.x, 1, n_seqs), block, 0, s, p);               \
    } while (0)
    if (in_dtype == TL_F32 && out_dtype == TL_F32) TL_CONV(float, float);
    else if (in_dtype == TL_F32 && out_dtype == TL_BF16) TL_CONV(float, __nv_bfloat16);
    else if (in_dtype == TL_BF16 && out_dtype == TL_BF16) TL_CONV(__nv_bfloat16, __nv_bfloat16);
    else return TL_BAD_DTYPE;
#undef TL_CONV
    return (int)e;
}

// x: [n_tokens] rows of pitch ldx, n_heads * head_dim columns used; out: float32 [n_tokens][n_heads * head_dim].
// unit != 0: every head becomes x / sqrt(sum(x^2) + unit_eps).  Otherwise, with a table ([table_rows][rot / 2][2] of
// (cos, sin)), the first `rot` coordinates of every head turn by the token's position.  Then times scale.
extern "C" int tl_recurrence_prep(const void* x, int in_dtype, long long ldx, float* out, const int* positions,
                                  const float* table, int table_rows, int n_tokens, int n_heads, int head_dim, int rot,
                                  int unit, float unit_eps, float scale, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (n_heads <= 0 || head_dim <= 0 || rot < 0 || rot > head_dim || rot % 2 != 0) return TL_BAD_SIZE;
    if (!unit && rot > 0 && (table == nullptr || positions == nullptr || table_rows <= 0)) return TL_BAD_SIZE;
    PrepParams p;
    p.x = x; p.ldx = ldx; p.out = out; p.positions = positions; p.table = rot > 0 ? table : nullptr; p.table_rows = table_rows;
    p.n_heads = n_heads; p.head_dim = head_dim; p.rot = rot; p.unit = unit; p.scale = scale; p.unit_eps = unit_eps;
    p.n_rows = (long long)n_tokens * n_heads;
    const dim3 grid((unsigned)((p.n_rows + NT / 32 - 1) / (NT / 32))), block(NT);
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == TL_F32) return (int)tl_launch(recurrence_prep_kernel<float>, grid, block, 0, s, p);
    if (in_dtype == TL_BF16) return (int)tl_launch(recurrence_prep_kernel<__nv_bfloat16>, grid, block, 0, s, p);
    return TL_BAD_DTYPE;
}

// q, k: float32 [n_tokens][qk_heads * dk]; v: rows of pitch ldv, heads * dv columns; state: float32, per slot a row of
// pitch state_pitch holding [heads][dv][dk] (the matrix of a head with a column's keys side by side); out: float32 [n_tokens][heads * dv].  delta == 0: decay is [heads], the
// fixed decay.  delta != 0: beta and gate are rows of pitch ldg with `heads` columns (of v's dtype), decay is
// exp(A_log) per head and decay_bias the bias inside the softplus.
extern "C" int tl_linear_recurrence(const float* q, const float* k, const void* v, int v_dtype, long long ldv, const void* beta,
                                    const void* gate, long long ldg, const float* decay, const float* decay_bias, float* state,
                                    long long state_pitch, const int* q_start, const int* state_slot, const int* fresh,
                                    float* out, int n_tokens, int n_seqs, int heads, int qk_heads, int dk, int dv, int delta,
                                    void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return TL_OK;
    if (heads <= 0 || qk_heads <= 0 || heads % qk_heads != 0 || dk <= 0 || dk > 256 || dv <= 0 || n_seqs > 65535 || heads > 65535)
        return TL_BAD_SIZE;
    if (decay == nullptr || (delta && (beta == nullptr || gate == nullptr || decay_bias == nullptr))) return TL_BAD_SIZE;
    RecurrenceParams p;
    p.q = q; p.k = k; p.v = v; p.ldv = ldv; p.beta = beta; p.gate = gate; p.ldg = ldg; p.decay = decay; p.decay_bias = decay_bias;
    p.state = state; p.state_pitch = state_pitch; p.q_start = q_start; p.state_slot = state_slot; p.fresh = fresh; p.out = out;
    p.H = heads; p.G = qk_heads; p.dk = dk; p.dv = dv;
    // slices of the key size per column (TORCHLLMS_B200_REC_SLICES=4|8|16 overrides the choice, for comparisons), and a
    // lane's share of it (a multiple of 4)
    static int forced = -1;
    if (forced < 0) {
        const char* e = getenv("TORCHLLMS_B200_REC_SLICES");
        forced = e != nullptr ? atoi(e) : 0;
    }
    int ks = dk > 128 ? 16 : dk > 32 ? 8 : 4;
    if ((forced == 4 && dk <= 128) || (forced == 8 && dk <= 128) || forced == 16) ks = forced;
    const int share = (dk + ks - 1) / ks;
    const int rows = share <= 8 ? 8 : share <= 12 ? 12 : share <= 16 ? 16 : share <= 24 ? 24 : 32;
    const int cols = 4 * (32 / ks);
    const size_t smem = ((size_t)2 * RC_TOKENS * ks * (rows + 4) + RC_TOKENS * cols + 3 * RC_TOKENS) * sizeof(float);
    const dim3 grid((dv + cols - 1) / cols, heads, n_seqs), block(NT);
    cudaStream_t s = (cudaStream_t)stream;
#define TL_REC(R, KS, TV)                                                                                           \
    (delta ? tl_launch(linear_recurrence_kernel<R, KS, true, TV>, grid, block, smem, s, p)                          \
           : tl_launch(linear_recurrence_kernel<R, KS, false, TV>, grid, block, smem, s, p))
#define TL_REC_SIZES(TV)                                                                                            \
    (ks == 4 ? (rows == 8 ? TL_REC(8, 4, TV) : rows <= 16 ? TL_REC(16, 4, TV) : rows == 24 ? TL_REC(24, 4, TV) : TL_REC(32, 4, TV)) \
     : ks == 8 ? (rows == 8 ? TL_REC(8, 8, TV) : rows == 12 ? TL_REC(12, 8, TV) : TL_REC(16, 8, TV))                \
               : (rows == 8 ? TL_REC(8, 16, TV) : rows == 12 ? TL_REC(12, 16, TV) : TL_REC(16, 16, TV)))
    if (v_dtype == TL_F32) return (int)TL_REC_SIZES(float);
    if (v_dtype == TL_BF16) return (int)TL_REC_SIZES(__nv_bfloat16);
#undef TL_REC_SIZES
#undef TL_REC
    return TL_BAD_DTYPE;
}

// o: float32 [n_tokens][n_heads * head_dim]; gate: rows of pitch ldg, n_heads * head_dim columns; weight: float32
// [head_dim] or null; out: [n_tokens][n_heads * head_dim] of out_dtype.
extern "C" int tl_head_norm_gate(const float* o, const void* gate, int gate_dtype, long long ldg, const float* weight, void* out,
                                 int out_dtype, int n_tokens, int n_heads, int head_dim, float eps, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (n_heads <= 0 || head_dim <= 0) return TL_BAD_SIZE;
    HeadNormParams p;
    p.o = o; p.gate = gate; p.ldg = ldg; p.weight = weight; p.out = out; p.n_heads = n_heads; p.head_dim = head_dim; p.eps = eps;
    p.n_rows = (long long)n_tokens * n_heads;
    const dim3 grid((unsigned)((p.n_rows + NT / 32 - 1) / (NT / 32))), block(NT);
    cudaStream_t s = (cudaStream_t)stream;
    if (gate_dtype == TL_F32 && out_dtype == TL_F32) return (int)tl_launch(head_norm_gate_kernel<float, float>, grid, block, 0, s, p);
    if (gate_dtype == TL_F32 && out_dtype == TL_BF16) return (int)tl_launch(head_norm_gate_kernel<float, __nv_bfloat16>, grid, block, 0, s, p);
    if (gate_dtype == TL_BF16 && out_dtype == TL_BF16) return (int)tl_launch(head_norm_gate_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, s, p);
    return TL_BAD_DTYPE;
}
