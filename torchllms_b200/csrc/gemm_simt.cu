// C[M, N] = A[M, K] . W[N, K]^T with float32 multiply-adds on the CUDA cores (no tensor cores,
// hence no reduced-precision matrix mode): the projection kernel of the true 32-bit path, and a
// fallback for bfloat16 operands.  Both operands are K-major as stored: activations row-major and
// weights in the [out, in] layout of nn.Linear (torchllms/models/networks.py:474-493, :600-602).
//
// 64 x 64 output tile per CTA, K walked 16 at a time through shared memory, 4 x 4 outputs per
// thread; every edge is guarded, so M, N and K may be anything.  The K loop order is the same
// for every row, so a row's result does not depend on which other rows share the launch.
//
// The batched form takes one product per blockIdx.z with strides of its own for the rows of A and
// C and between the batches: a head's slice of [tokens, heads, K] rows against that head's own
// [N, K] matrix, written into its slice of [tokens, heads, N].
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4, NT = 256;

template <typename T, typename TO>
__global__ void __launch_bounds__(NT) gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ W,
                                                       TO* __restrict__ C, int M, int N, int K,
                                                       long long lda, long long ldc, long long a_batch,
                                                       long long w_batch, long long c_batch,
                                                       const TO* __restrict__ gate = nullptr, long long ldg = 0, long long g_batch = 0) {
    A += blockIdx.z * a_batch;
    W += blockIdx.z * w_batch;
    C += blockIdx.z * c_batch;
    if (gate != nullptr) gate += blockIdx.z * g_batch;
    __shared__ float As[BK][BM + PAD];
    __shared__ float Ws[BK][BN + PAD];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lrow = tid >> 2;         // 0..63: tile row this thread loads
    const int lk = (tid & 3) * 4;      // 0, 4, 8, 12: first of its four k
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        {
            const int gm = m0 + lrow, gn = n0 + lrow;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int gk = k0 + lk + e;
                As[lk + e][lrow] = (gm < M && gk < K) ? to_float(A[(size_t)gm * lda + gk]) : 0.f;
                Ws[lk + e][lrow] = (gn < N && gk < K) ? to_float(W[(size_t)gn * K + gk]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 w4 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            const float a[4] = {a4.x, a4.y, a4.z, a4.w};
            const float w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = from_float<TO>(gate != nullptr ? acc[i][j] * to_float(gate[(size_t)gm * ldg + gn]) : acc[i][j]);
        }
    }
}

template <typename T, typename TO>
int launch(const void* A, const void* W, void* C, int M, int N, int K, cudaStream_t s, int batches = 1,
           long long lda = -1, long long ldc = -1, long long a_batch = 0, long long w_batch = 0, long long c_batch = 0,
           const void* gate = nullptr, long long ldg = 0, long long g_batch = 0) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, batches);
    if (grid.y > 65535 || batches > 65535) return TL_BAD_SIZE;
    gemm_simt_kernel<T, TO><<<grid, NT, 0, s>>>((const T*)A, (const T*)W, (TO*)C, M, N, K, lda < 0 ? K : lda,
                                                ldc < 0 ? N : ldc, a_batch, w_batch, c_batch, (const TO*)gate, ldg, g_batch);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

}  // namespace

extern "C" int tl_gemm_simt(const void* A, const void* W, void* C, int in_dtype, int out_dtype,
                            int M, int N, int K, void* stream) {
    if (M <= 0 || N <= 0) return TL_OK;
    if (K <= 0) return TL_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == TL_F32 && out_dtype == TL_F32) return launch<float, float>(A, W, C, M, N, K, s);
    if (in_dtype == TL_BF16 && out_dtype == TL_BF16) return launch<__nv_bfloat16, __nv_bfloat16>(A, W, C, M, N, K, s);
    if (in_dtype == TL_BF16 && out_dtype == TL_F32) return launch<__nv_bfloat16, float>(A, W, C, M, N, K, s);
    return TL_BAD_DTYPE;
}

namespace {

// Few rows (decode steps): a CTA per (head, token); the token's K inputs in shared memory as float32,
// a thread per output column walking that column's K weights 16 bytes at a time where K allows.
template <typename T>
__global__ void __launch_bounds__(128) head_linear_rows_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                               T* __restrict__ out, int n_heads, int N, int K,
                                                               long long ldx, long long hsx, long long ldo, long long hso,
                                                               const T* __restrict__ gate) {
    extern __shared__ __align__(16) float xs[];
    const int h = blockIdx.x, t = blockIdx.y;
    const T* xr = x + (size_t)t * ldx + (size_t)h * hsx;
    for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_float(xr[k]);
    __syncthreads();
    constexpr int VEC = Vec16<T>::N;
    const bool vec = K % VEC == 0 && ((size_t)w & 15u) == 0;
    for (int n = threadIdx.x; n < N; n += blockDim.x) {
        const T* wr = w + ((size_t)h * N + n) * K;
        float acc = 0.f;
        if (vec) {
            for (int k = 0; k < K; k += VEC) {
                Vec16<T> v;
                v.load(wr + k);
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc = fmaf(v.get(e), xs[k + e], acc);
            }
        } else {
            for (int k = 0; k < K; ++k) acc = fmaf(to_float(wr[k]), xs[k], acc);
        }
        if (gate != nullptr) acc *= to_float(gate[((size_t)t * n_heads + h) * N + n]);
        out[(size_t)t * ldo + (size_t)h * hso + n] = from_float<T>(acc);
    }
}

}  // namespace

// One product per head: x [tokens, heads, K] against w [heads, N, K] gives out [tokens, heads, N],
// out[t, h, :] = w[h] x[t, h, :]; x, w and out have one dtype.
// The extended form: token t's head h reads x + t * ldx + h * hsx (K numbers) and writes out + t * ldo + h * hso
// (N numbers), so either may be a part of every head of wider rows; gate ([tokens, heads, N], dense, or null)
// multiplies the result.
extern "C" int tl_head_linear_ex(const void* x, const void* w, void* out, const void* gate, int dtype, int n_tokens, int n_heads,
                                 int N, int K, long long ldx, long long hsx, long long ldo, long long hso, void* stream) {
    if (n_tokens <= 0 || n_heads <= 0 || N <= 0) return TL_OK;
    if (K <= 0) return TL_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (n_tokens <= 16 && n_heads <= 65535 && (size_t)K * sizeof(float) <= 48 * 1024) {
        const dim3 grid(n_heads, n_tokens);
        if (dtype == TL_F32)
            head_linear_rows_kernel<float><<<grid, 128, (size_t)K * sizeof(float), s>>>((const float*)x, (const float*)w, (float*)out,
                                                                                         n_heads, N, K, ldx, hsx, ldo, hso, (const float*)gate);
        else if (dtype == TL_BF16)
            head_linear_rows_kernel<__nv_bfloat16><<<grid, 128, (size_t)K * sizeof(float), s>>>(
                (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, n_heads, N, K, ldx, hsx, ldo, hso,
                (const __nv_bfloat16*)gate);
        else
            return TL_BAD_DTYPE;
        TL_LAUNCH_CHECK();
        return TL_OK;
    }
    const long long ldg = (long long)n_heads * N;
    if (dtype == TL_F32)
        return launch<float, float>(x, w, out, n_tokens, N, K, s, n_heads, ldx, ldo, hsx, (long long)N * K, hso, gate, ldg, N);
    if (dtype == TL_BF16)
        return launch<__nv_bfloat16, __nv_bfloat16>(x, w, out, n_tokens, N, K, s, n_heads, ldx, ldo, hsx, (long long)N * K, hso, gate, ldg, N);
    return TL_BAD_DTYPE;
}

extern "C" int tl_head_linear(const void* x, const void* w, void* out, int dtype, int n_tokens, int n_heads,
                              int N, int K, void* stream) {
    if (n_tokens <= 0 || n_heads <= 0 || N <= 0) return TL_OK;
    if (K <= 0) return TL_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (n_tokens <= 16 && n_heads <= 65535 && (size_t)K * sizeof(float) <= 48 * 1024) {
        const dim3 grid(n_heads, n_tokens);
        if (dtype == TL_F32)
            head_linear_rows_kernel<float><<<grid, 128, (size_t)K * sizeof(float), s>>>((const float*)x, (const float*)w, (float*)out,
                                                                                         n_heads, N, K, (long long)n_heads * K, K, (long long)n_heads * N, N, nullptr);
        else if (dtype == TL_BF16)
            head_linear_rows_kernel<__nv_bfloat16><<<grid, 128, (size_t)K * sizeof(float), s>>>(
                (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, n_heads, N, K, (long long)n_heads * K, K,
                (long long)n_heads * N, N, nullptr);
        else
            return TL_BAD_DTYPE;
        TL_LAUNCH_CHECK();
        return TL_OK;
    }
    const long long lda = (long long)n_heads * K, ldc = (long long)n_heads * N;
    if (dtype == TL_F32)
        return launch<float, float>(x, w, out, n_tokens, N, K, s, n_heads, lda, ldc, K, (long long)N * K, N);
    if (dtype == TL_BF16)
        return launch<__nv_bfloat16, __nv_bfloat16>(x, w, out, n_tokens, N, K, s, n_heads, lda, ldc, K, (long long)N * K, N);
    return TL_BAD_DTYPE;
}
