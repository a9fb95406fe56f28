// Selective scan: a diagonal state-space recurrence whose step sizes, inputs and read-outs the token chooses.
//
// Per request, channel c and state index n (S float32, kept per request between steps):
//     dt_c   = softplus(dt_in[t, c] + dt_bias[c])
//     S[c,n] <- exp(dt_c * A[c, n]) * S[c, n] + dt_c * x[t, c] * B[t, n]
//     y[t,c] = sum_n S[c, n] * C[t, n] + D[c] * x[t, c]
//     out    = y * silu(z[t, c])
// Tokens are walked in order from the state that the request's slot holds (zeros for a request that
// starts), so a result does not depend on how a prompt was cut into portions, nor on what else is in
// the batch.  Everything here is float32: the step sizes with their softplus, the decays with their
// exponentials (taken as 2^(dt * A * log2 e), a lane's rates multiplied by log2 e once when it loads them),
// the state and every product into it.  x, dt_in, B, C and z come from matrix products and
// may be bfloat16 and column ranges of wider rows (a row pitch goes with each).
//
// Work split: a CTA of 128 threads takes one request and 128 / L channels, L lanes sharing a channel
// and each holding NS of its state numbers in registers (n = lane + j * L).  Tokens come in chunks of
// 16: dt (after softplus), x, z of the CTA's channels and B, C of the chunk are staged in shared
// memory as float32 (through registers, the next chunk's loads in flight while this one is walked), then
// every token is one pass over the lane's NS numbers; the sums over the L lanes are taken for the whole
// chunk at once, and the chunk's outputs leave together.  Per state number the arithmetic is one chain of
// multiply-adds in token order whatever the chunks, so a prompt, its portions and its decoded tokens agree
// to the bit.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int NT = 128;
constexpr float LOG2E = 1.4426950408889634f;

struct ScanParams {
    const void* x;   long long ldx;      // [T] rows, C channels used
    const void* dt;  long long lddt;     // [T] rows, C channels
    const void* B;   long long ldb;      // [T] rows, N numbers
    const void* Cm;  long long ldc;      // [T] rows, N numbers
    const void* z;   long long ldz;      // [T] rows, C channels
    const float* A;                      // [C][N], negative rates (not yet times log2 e)
    const float* D;                      // [C]
    const float* dt_bias;                // [C]
    float* state;    long long state_pitch;   // [slots] rows, each [C][N]
    const int* q_start;                  // [B + 1]
    const int* state_slot;               // [B]
    const int* fresh;                    // [B]
    void* out;                           // [T][C]
    int C, N;
};

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

template <typename TI, typename TO, int NS, int L, int TT>
__global__ void __launch_bounds__(NT) selective_scan_kernel(const ScanParams p) {
    constexpr int CH = NT / L;                          // channels per CTA
    constexpr int CI = (TT * CH + NT - 1) / NT;         // (token, channel) items of a chunk per thread
    constexpr int BI = (TT * NS * L + NT - 1) / NT;     // (token, state index) items of a chunk per thread, at most
    extern __shared__ __align__(16) float sm[];
    float* s_dt = sm;                     // [TT][CH]
    float* s_x = s_dt + TT * CH;          // [TT][CH]
    float* s_z = s_x + TT * CH;           // [TT][CH]
    float* s_y = s_z + TT * CH;           // [TT][CH]
    constexpr int NP = NS * L;            // a row of B or C in shared memory: N numbers and zeros up to NS * L
    float* s_B = s_y + TT * CH;           // [TT][NP]
    float* s_C = s_B + TT * NP;           // [TT][NP]
    grid_launch_dependents();
    grid_dependency_wait();
    const int b = blockIdx.y;
    const int start = p.q_start[b], len = p.q_start[b + 1] - start;
    if (len <= 0) return;
    const int tid = threadIdx.x;
    const int lane = tid % L, cl = tid / L;
    const int c0 = blockIdx.x * CH, c = c0 + cl;
    const bool live = c < p.C;
    const int N = p.N;
    float* st = p.state + (size_t)p.state_slot[b] * p.state_pitch;
    const bool fresh = p.fresh[b] != 0;

    float S[NS], A2[NS];
#pragma unroll
    for (int j = 0; j < NS; ++j) {
        const int n = lane + j * L;
        const bool ok = live && n < N;
        S[j] = (ok && !fresh) ? st[(size_t)c * N + n] : 0.f;
        A2[j] = ok ? p.A[(size_t)c * N + n] * LOG2E : 0.f;
    }
    const float Dc = live ? p.D[c] : 0.f;

    const TI* x = reinterpret_cast<const TI*>(p.x);
    const TI* dt = reinterpret_cast<const TI*>(p.dt);
    const TI* Bm = reinterpret_cast<const TI*>(p.B);
    const TI* Cm = reinterpret_cast<const TI*>(p.Cm);
    const TI* z = reinterpret_cast<const TI*>(p.z);
    TO* out = reinterpret_cast<TO*>(p.out);

    // The chunk's inputs travel global memory -> registers -> shared memory, the next chunk's loads being issued before
    // this chunk's tokens are walked.  Item k of a thread is (token tid / CH + k * (NT / CH), channel tid % CH): always
    // the same channel, whose step-size bias it keeps.
    const int my_cc = tid % CH, my_ch = c0 + my_cc, my_t0 = tid / CH;
    const bool my_live = my_ch < p.C;
    const float my_bias = my_live ? p.dt_bias[my_ch] : 0.f;
    TI r_dt[CI], r_x[CI], r_z[CI], r_B[BI], r_C[BI];
    auto fetch = [&](int t0, int nt) {
#pragma unroll
        for (int k = 0; k < CI; ++k) {
            const int tt = my_t0 + k * (NT / CH);
            if (tt < nt && my_live) {
                const size_t row = (size_t)(start + t0 + tt);
                r_dt[k] = dt[row * p.lddt + my_ch];
                r_x[k] = x[row * p.ldx + my_ch];
                r_z[k] = z[row * p.ldz + my_ch];
            }
        }
#pragma unroll
        for (int k = 0; k < BI; ++k) {
            const int i = tid + k * NT;
            const int tt = i / NP, n = i - tt * NP;
            if (tt < nt && n < N) {
                const size_t row = (size_t)(start + t0 + tt);
                r_B[k] = Bm[row * p.ldb + n];
                r_C[k] = Cm[row * p.ldc + n];
            }
        }
    };
    // (places without a token or a state number hold zeros: a step of size zero leaves the state as it is)
    auto stage = [&](int nt) {
#pragma unroll
        for (int k = 0; k < CI; ++k) {
            const int tt = my_t0 + k * (NT / CH);
            if (tt < TT) {
                const int i = tt * CH + my_cc;
                const bool ok = my_live && tt < nt;
                s_dt[i] = ok ? softplus_f(to_float(r_dt[k]) + my_bias) : 0.f;
                s_x[i] = ok ? to_float(r_x[k]) : 0.f;
                s_z[i] = ok ? to_float(r_z[k]) : 0.f;
            }
        }
#pragma unroll
        for (int k = 0; k < BI; ++k) {
            const int i = tid + k * NT;
            const int tt = i / NP, n = i - tt * NP;
            if (tt < TT) {
                const bool ok = tt < nt && n < N;
                s_B[i] = ok ? to_float(r_B[k]) : 0.f;
                s_C[i] = ok ? to_float(r_C[k]) : 0.f;
            }
        }
    };

    fetch(0, min(TT, len));
    for (int t0 = 0; t0 < len; t0 += TT) {
        const int nt = min(TT, len - t0);
        __syncthreads();      // the chunk before has been walked and its outputs have left shared memory
        stage(nt);
        __syncthreads();
        if (t0 + TT < len) fetch(t0 + TT, min(TT, len - t0 - TT));
        if (nt == TT) {
            // A whole chunk, without a branch: the only chain from token to token is one multiply-add per state
            // number; decays and inputs of later tokens are worked out beside it, and the sums over a channel's
            // lanes wait until the chunk's tokens are done, so that their shuffles do not stand in that chain.
            float acc[TT];
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) {
                const float d = s_dt[tt * CH + cl];
                const float dx = d * s_x[tt * CH + cl];
                float a = 0.f;
#pragma unroll
                for (int j = 0; j < NS; ++j) {
                    const int n = lane + j * L;
                    S[j] = fmaf(exp2f(d * A2[j]), S[j], dx * s_B[tt * NP + n]);
                    a = fmaf(S[j], s_C[tt * NP + n], a);
                }
                acc[tt] = a;
            }
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) {
#pragma unroll
                for (int o = L / 2; o > 0; o >>= 1) acc[tt] += __shfl_xor_sync(0xffffffffu, acc[tt], o);
                if (lane == 0) s_y[tt * CH + cl] = fmaf(Dc, s_x[tt * CH + cl], acc[tt]);
            }
        } else {
            // the last tokens of a portion, a decode step: the same arithmetic, token by token
            for (int tt = 0; tt < nt; ++tt) {
                const float d = s_dt[tt * CH + cl];
                const float dx = d * s_x[tt * CH + cl];
                float a = 0.f;
#pragma unroll
                for (int j = 0; j < NS; ++j) {
                    const int n = lane + j * L;
                    S[j] = fmaf(exp2f(d * A2[j]), S[j], dx * s_B[tt * NP + n]);
                    a = fmaf(S[j], s_C[tt * NP + n], a);
                }
#pragma unroll
                for (int o = L / 2; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                if (lane == 0) s_y[tt * CH + cl] = fmaf(Dc, s_x[tt * CH + cl], a);
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < CI; ++k) {
            const int tt = my_t0 + k * (NT / CH);
            if (tt < nt && my_live) {
                const int i = tt * CH + my_cc;
                const float zv = s_z[i];
                out[(size_t)(start + t0 + tt) * p.C + my_ch] = from_float<TO>(s_y[i] * (zv / (1.f + expf(-zv))));
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NS; ++j) {
        const int n = lane + j * L;
        if (live && n < N) st[(size_t)c * N + n] = S[j];
    }
}

template <typename TI, typename TO, int NS, int L, int TT>
int launch(const ScanParams& p, int n_seqs, cudaStream_t s) {
    constexpr int CH = NT / L;
    const size_t smem = (size_t)(4 * TT * CH + 2 * TT * NS * L) * sizeof(float);
    if (smem > 48 * 1024) return TL_TOO_LARGE;
    const dim3 grid((p.C + CH - 1) / CH, n_seqs);
    return (int)tl_launch(selective_scan_kernel<TI, TO, NS, L, TT>, grid, dim3(NT), smem, s, p);
}

// lanes per channel, state numbers per lane and tokens per chunk for a state of N numbers.  Few numbers a lane mean
// many warps, which is what hides the latencies of a walk that is serial in the tokens, and more work per token that
// all lanes of a channel repeat: two numbers a lane up to 32 measured best (TORCHLLMS_B200_SCAN_PER_LANE = 1 or 4 asks
// for another split, for comparisons), four where a warp's 32 lanes no longer reach, more beyond (and shorter chunks, so that a chunk's inputs still fit a thread's registers)
static int scan_per_lane() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("TORCHLLMS_B200_SCAN_PER_LANE");
        v = (e != nullptr && (e[0] == '1' || e[0] == '4')) ? e[0] - '0' : 2;
    }
    return v;
}

template <typename TI, typename TO>
int launch_n(const ScanParams& p, int n_seqs, cudaStream_t s) {
    const int N = p.N;
    const int per = scan_per_lane();
    if (per == 1) {
        if (N <= 1) return launch<TI, TO, 1, 1, 16>(p, n_seqs, s);
        if (N <= 2) return launch<TI, TO, 1, 2, 16>(p, n_seqs, s);
        if (N <= 4) return launch<TI, TO, 1, 4, 16>(p, n_seqs, s);
        if (N <= 8) return launch<TI, TO, 1, 8, 16>(p, n_seqs, s);
        if (N <= 16) return launch<TI, TO, 1, 16, 16>(p, n_seqs, s);
        if (N <= 32) return launch<TI, TO, 1, 32, 16>(p, n_seqs, s);
    } else if (per == 2) {
        if (N <= 2) return launch<TI, TO, 2, 1, 16>(p, n_seqs, s);
        if (N <= 4) return launch<TI, TO, 2, 2, 16>(p, n_seqs, s);
        if (N <= 8) return launch<TI, TO, 2, 4, 16>(p, n_seqs, s);
        if (N <= 16) return launch<TI, TO, 2, 8, 16>(p, n_seqs, s);
        if (N <= 32) return launch<TI, TO, 2, 16, 16>(p, n_seqs, s);
    }
    if (N <= 4) return launch<TI, TO, 4, 1, 16>(p, n_seqs, s);
    if (N <= 8) return launch<TI, TO, 4, 2, 16>(p, n_seqs, s);
    if (N <= 16) return launch<TI, TO, 4, 4, 16>(p, n_seqs, s);
    if (N <= 32) return launch<TI, TO, 4, 8, 16>(p, n_seqs, s);
    if (N <= 64) return launch<TI, TO, 2, 32, 16>(p, n_seqs, s);
    if (N <= 128) return launch<TI, TO, 4, 32, 16>(p, n_seqs, s);
    if (N <= 256) return launch<TI, TO, 8, 32, 8>(p, n_seqs, s);
    if (N <= 512) return launch<TI, TO, 16, 32, 4>(p, n_seqs, s);
    return TL_BAD_SIZE;
}

}  // namespace

// x, dt, z: [n_tokens] rows of their pitches with n_channels columns; B, C: rows with n_state columns; all of
// in_dtype.  A: float32 [n_channels][n_state]; D, dt_bias: float32 [n_channels]; state: float32, slot s at
// state + s * state_pitch, [n_channels][n_state]; out: [n_tokens][n_channels] of out_dtype.
extern "C" int tl_selective_scan(const void* x, long long ldx, const void* dt, long long lddt, const void* B, long long ldb,
                                 const void* C, long long ldc, const void* z, long long ldz, int in_dtype, const float* A,
                                 const float* D, const float* dt_bias, float* state, long long state_pitch,
                                 const int* q_start, const int* state_slot, const int* fresh, void* out, int out_dtype,
                                 int n_tokens, int n_seqs, int n_channels, int n_state, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return TL_OK;
    if (n_channels <= 0 || n_state <= 0 || n_seqs > 65535) return TL_BAD_SIZE;
    ScanParams p;
    p.x = x; p.ldx = ldx; p.dt = dt; p.lddt = lddt; p.B = B; p.ldb = ldb; p.Cm = C; p.ldc = ldc; p.z = z; p.ldz = ldz;
    p.A = A; p.D = D; p.dt_bias = dt_bias; p.state = state; p.state_pitch = state_pitch;
    p.q_start = q_start; p.state_slot = state_slot; p.fresh = fresh; p.out = out;
    p.C = n_channels; p.N = n_state;
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == TL_F32 && out_dtype == TL_F32) return launch_n<float, float>(p, n_seqs, s);
    if (in_dtype == TL_BF16 && out_dtype == TL_BF16) return launch_n<__nv_bfloat16, __nv_bfloat16>(p, n_seqs, s);
    if (in_dtype == TL_F32 && out_dtype == TL_BF16) return launch_n<float, __nv_bfloat16>(p, n_seqs, s);
    return TL_BAD_DTYPE;
}
