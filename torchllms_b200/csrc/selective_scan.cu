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
// memory as float32, then every token is one pass over the lane's NS numbers, a shuffle sum over the
// L lanes, and the chunk's outputs leave together.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int NT = 128;
constexpr int TT = 16;       // tokens per chunk
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

template <typename TI, typename TO, int NS, int L>
__global__ void __launch_bounds__(NT) selective_scan_kernel(const ScanParams p) {
    constexpr int CH = NT / L;            // channels per CTA
    extern __shared__ __align__(16) float sm[];
    float* s_dt = sm;                     // [TT][CH]
    float* s_x = s_dt + TT * CH;          // [TT][CH]
    float* s_z = s_x + TT * CH;           // [TT][CH]
    float* s_y = s_z + TT * CH;           // [TT][CH]
    float* s_B = s_y + TT * CH;           // [TT][N]
    float* s_C = s_B + TT * p.N;          // [TT][N]
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

    for (int t0 = 0; t0 < len; t0 += TT) {
        const int nt = min(TT, len - t0);
        __syncthreads();      // the chunk before has been read (and its outputs written)
        for (int i = tid; i < nt * CH; i += NT) {
            const int tt = i / CH, cc = i - tt * CH;
            const int ch = c0 + cc;
            float vdt = 0.f, vx = 0.f, vz = 0.f;
            if (ch < p.C) {
                const size_t row = (size_t)(start + t0 + tt);
                vdt = softplus_f(to_float(dt[row * p.lddt + ch]) + p.dt_bias[ch]);
                vx = to_float(x[row * p.ldx + ch]);
                vz = to_float(z[row * p.ldz + ch]);
            }
            s_dt[i] = vdt; s_x[i] = vx; s_z[i] = vz;
        }
        for (int i = tid; i < nt * N; i += NT) {
            const int tt = i / N, n = i - tt * N;
            const size_t row = (size_t)(start + t0 + tt);
            s_B[i] = to_float(Bm[row * p.ldb + n]);
            s_C[i] = to_float(Cm[row * p.ldc + n]);
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float d = s_dt[tt * CH + cl], xv = s_x[tt * CH + cl];
            const float dx = d * xv;
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < NS; ++j) {
                const int n = lane + j * L;
                if (n < N) {
                    S[j] = fmaf(exp2f(d * A2[j]), S[j], dx * s_B[tt * N + n]);
                    acc = fmaf(S[j], s_C[tt * N + n], acc);
                }
            }
#pragma unroll
            for (int o = L / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) s_y[tt * CH + cl] = fmaf(Dc, xv, acc);
        }
        __syncthreads();
        for (int i = tid; i < nt * CH; i += NT) {
            const int tt = i / CH, cc = i - tt * CH;
            const int ch = c0 + cc;
            if (ch < p.C) {
                const float zv = s_z[i];
                out[(size_t)(start + t0 + tt) * p.C + ch] = from_float<TO>(s_y[i] * (zv / (1.f + expf(-zv))));
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NS; ++j) {
        const int n = lane + j * L;
        if (live && n < N) st[(size_t)c * N + n] = S[j];
    }
}

template <typename TI, typename TO, int NS, int L>
int launch(const ScanParams& p, int n_seqs, cudaStream_t s) {
    constexpr int CH = NT / L;
    const size_t smem = (size_t)(4 * TT * CH + 2 * TT * p.N) * sizeof(float);
    if (smem > 48 * 1024) return TL_TOO_LARGE;
    const dim3 grid((p.C + CH - 1) / CH, n_seqs);
    return (int)tl_launch(selective_scan_kernel<TI, TO, NS, L>, grid, dim3(NT), smem, s, p);
}

// lanes per channel and state numbers per lane for a state of N numbers: four numbers a lane while a warp's
// 32 lanes reach, more beyond
template <typename TI, typename TO>
int launch_n(const ScanParams& p, int n_seqs, cudaStream_t s) {
    const int N = p.N;
    if (N <= 4) return launch<TI, TO, 4, 1>(p, n_seqs, s);
    if (N <= 8) return launch<TI, TO, 4, 2>(p, n_seqs, s);
    if (N <= 16) return launch<TI, TO, 4, 4>(p, n_seqs, s);
    if (N <= 32) return launch<TI, TO, 4, 8>(p, n_seqs, s);
    if (N <= 64) return launch<TI, TO, 4, 16>(p, n_seqs, s);
    if (N <= 128) return launch<TI, TO, 4, 32>(p, n_seqs, s);
    if (N <= 256) return launch<TI, TO, 8, 32>(p, n_seqs, s);
    if (N <= 512) return launch<TI, TO, 16, 32>(p, n_seqs, s);
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
