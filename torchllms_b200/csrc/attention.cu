// Causal grouped-query attention over paged keys and values, for any mix of prompt portions
// and single decoded tokens (the general kernel: float32 and bfloat16, any head size up to 512
// for keys and, separately, for values, any number of heads and groups, optional sliding window).
//
// Options that a design may switch on, all off by default:
//   keep_first   with a window: the first so many keys of a request stay visible for ever
//   rel, bucket  a learned bias added to the scaled score: rel[bucket[p - k], head], the row of the
//                [rows, heads] table chosen by a tabulated function of the distance
//   gate         the result is multiplied by a gate value, one per (token, head) or one per element
//   v_head_dim   values of another size than keys; v_pages may be the very tensor k_pages (a mixer
//                that attends over one stored vector as key and value)
//   n_v_heads    fewer value heads than key heads: key head j goes with value head j % n_v_heads
//                (several attention maps with keys of their own over one set of values)
//   out_f32      the result is written as float32 whatever q's dtype (for a caller that still
//                combines maps before anything is rounded)
//   softcap      c > 0: the scaled score s becomes c * tanh(s / c) (before any bias)
//   sinks        a learned number per query head, [n_heads] float32: the softmax's denominator also holds
//                exp(sinks[h]); it stands for a key without a value, counts once, and is neither scaled nor capped
//   v_stride     elements from one stored value to the next when that is not v_head_dim: with v_pages being
//                k_pages and v_stride = head_dim, a value is the first v_head_dim coordinates of a stored key
//
// What it computes, per query token at absolute position p of request b and query head h
// (kv head h / (H / KV)):   o = softmax_k( q . k_k * scale ) v_k   over keys k <= p
// (and k > p - window when a window is set), as torchllms/models/networks.py:355-397 does for
// whole sequences; the query's position is kv_len[b] - q_len[b] + its index in the portion, the
// bottom-right aligned mask the reference relies on for a suffix after a cached prefix
// (torchllms/models/networks.py:435-445).  Scores, the running maximum and sum, and the output
// accumulator are float32.
//
// Work split: one CTA takes up to 16 rows, a row being (token, query head of one kv group), so
// the heads of a group share every key and value it loads.  Keys are walked in tiles of 32
// through shared memory with the streaming-softmax update.  When the batch offers too few CTAs
// (decoding a few long requests), the key range is cut into splits whose partial (max, sum,
// accumulator) go to a float32 workspace that tl_attention_merge combines.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int R = 16;    // rows per CTA
constexpr int TK = 32;   // keys per tile
constexpr int NT = 128;  // threads per CTA: 8 threads per row
constexpr int TARGET_CTAS = 296;
constexpr int MIN_SPLIT = 128;

struct AttnParams {
    const void* q;
    const void* k_pages;
    const void* v_pages;
    void* out;
    const int* block_table;
    const int* q_start;
    const int* kv_len;
    float* part_o;   // [T * H, n_splits, v_head_dim]
    float* part_ml;  // [T * H, n_splits, 2]
    const float* rel;    // [rows, n_heads] or null
    const int* bucket;   // [n_bucket]: row of rel for a distance (distances beyond the table take its last entry)
    const void* gate;    // [T, n_heads] (gate_mode 1) or [T, n_heads * v_head_dim] (gate_mode 2), in q's dtype
    int gate_mode, n_bucket, keep_first;
    int n_v_heads, out_f32;
    int v_stride;        // elements between stored values (v_head_dim unless values are parts of wider vectors)
    float softcap;       // 0: none
    const float* sinks;  // [n_heads] or null
    int table_stride;
    int n_heads, n_kv_heads, head_dim, v_head_dim, page_size;
    int group, gchunk, n_gchunks, tokens_per_tile;
    int window;  // 0: none
    int n_splits;
    float scale;
};

template <typename T, int HD_MAX>
__global__ void __launch_bounds__(NT) paged_attention_kernel(const AttnParams p) {
    extern __shared__ float smem[];
    const int hd = p.head_dim, dv = p.v_head_dim;
    const int qpitch = hd + 1;
    float* Qs = smem;                 // [R][hd + 1]
    float* Ks = Qs + R * qpitch;      // [TK][hd + 1]
    float* Vs = Ks + TK * qpitch;     // [TK][dv]
    float* Ss = Vs + TK * dv;         // [R][TK + 1]

    const int b = blockIdx.z;
    const int qs = p.q_start[b];
    const int ql = p.q_start[b + 1] - qs;
    const int kl = p.kv_len[b];
    const int tile = blockIdx.x / p.n_splits;
    const int split = blockIdx.x - tile * p.n_splits;
    const int tok0 = tile * p.tokens_per_tile;
    if (tok0 >= ql) return;
    const int ntok = min(p.tokens_per_tile, ql - tok0);
    const int kvh = blockIdx.y / p.n_gchunks;
    const int g0 = (blockIdx.y - kvh * p.n_gchunks) * p.gchunk;
    const int ng = min(p.gchunk, p.group - g0);
    const int n_rows = ntok * ng;

    const int tid = threadIdx.x;
    const int rr = tid >> 3;  // row of this thread
    const int c = tid & 7;

    const T* q = reinterpret_cast<const T*>(p.q);
    const T* k_pages = reinterpret_cast<const T*>(p.k_pages);
    const T* v_pages = reinterpret_cast<const T*>(p.v_pages);

    // ---- queries of the tile, as float
    for (int i = tid; i < R * hd; i += NT) {
        const int r = i / hd, d = i - r * hd;
        float v = 0.f;
        if (r < n_rows) {
            const int tok = qs + tok0 + r / ng;
            const int head = kvh * p.group + g0 + r % ng;
            v = to_float(q[((size_t)tok * p.n_heads + head) * hd + d]);
        }
        Qs[r * qpitch + d] = v;
    }

    const int qpos_min = kl - ql + tok0;
    const int qpos_max = qpos_min + ntok - 1;
    const int my_qpos = rr < n_rows ? qpos_min + rr / ng : -1;
    const int my_head = kvh * p.group + g0 + (rr < n_rows ? rr % ng : 0);
    // The keys this tile's queries can see: the window's (or all up to the last query), and ahead of
    // them the kept first keys that the window has passed.  They are walked as one run u = 0 .. n_vis - 1,
    // u < n_kept being key u and the rest key win_lo + (u - n_kept).
    const int win_lo = p.window > 0 ? max(0, qpos_min - p.window + 1) : 0;
    const int n_kept = min(p.keep_first, win_lo);
    const int n_vis = n_kept + max(qpos_max + 1 - win_lo, 0);
    int k_lo = 0, k_hi = n_vis;
    if (p.n_splits > 1) {
        // every request cuts its own visible keys evenly, in whole tiles, so the launch shape
        // depends on the batch only and not on how long the requests have grown
        const int chunk = ((n_vis + p.n_splits - 1) / p.n_splits + TK - 1) / TK * TK;
        k_lo = split * chunk;
        k_hi = min(k_hi, k_lo + chunk);
    }

    float m = -INFINITY, l = 0.f;
    float acc[HD_MAX / 8];
#pragma unroll
    for (int j = 0; j < HD_MAX / 8; ++j) acc[j] = 0.f;

    constexpr int VEC = Vec16<T>::N;
    const bool vec_ok = hd % VEC == 0 && dv % VEC == 0 && p.v_stride % VEC == 0;      // every stored vector starts on 16 bytes
    const int k_vecs = hd / VEC, v_vecs = dv / VEC;
    const int* table = p.block_table + (size_t)b * p.table_stride;
    const int vh = kvh % p.n_v_heads;        // the value head that goes with this key head

    for (int k0 = k_lo; k0 < k_hi; k0 += TK) {
        __syncthreads();  // the previous tile's Ks / Vs / Ss are no longer read (and Qs is written)
        if (vec_ok) {
            for (int i = tid; i < TK * (k_vecs + v_vecs); i += NT) {
                const int j = i / (k_vecs + v_vecs), v = i - j * (k_vecs + v_vecs);
                const bool is_k = v < k_vecs;
                const int u = k0 + j;
                const int kpos = u < n_kept ? u : win_lo + (u - n_kept);
                float* dst = is_k ? Ks + j * qpitch + v * VEC : Vs + j * dv + (v - k_vecs) * VEC;
                if (u < k_hi && tl_check_page(table[kpos / p.page_size])) {     // (debug builds: a bad page reads as zeros)
                    const int page = table[kpos / p.page_size];
                    const size_t at = ((size_t)page * p.n_kv_heads + kvh) * p.page_size + kpos % p.page_size;
                    const size_t vat = ((size_t)page * p.n_v_heads + vh) * p.page_size + kpos % p.page_size;
                    Vec16<T> x;
                    x.load(is_k ? k_pages + at * hd + v * VEC : v_pages + vat * p.v_stride + (v - k_vecs) * VEC);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) dst[e] = x.get(e);
                } else {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) dst[e] = 0.f;
                }
            }
        } else {
            for (int i = tid; i < TK * (hd + dv); i += NT) {
                const int j = i / (hd + dv), d = i - j * (hd + dv);
                const bool is_k = d < hd;
                const int u = k0 + j;
                const int kpos = u < n_kept ? u : win_lo + (u - n_kept);
                float x = 0.f;
                if (u < k_hi && tl_check_page(table[kpos / p.page_size])) {
                    const int page = table[kpos / p.page_size];
                    const size_t at = ((size_t)page * p.n_kv_heads + kvh) * p.page_size + kpos % p.page_size;
                    const size_t vat = ((size_t)page * p.n_v_heads + vh) * p.page_size + kpos % p.page_size;
                    x = to_float(is_k ? k_pages[at * hd + d] : v_pages[vat * p.v_stride + (d - hd)]);
                }
                if (is_k) Ks[j * qpitch + d] = x;
                else Vs[j * dv + (d - hd)] = x;
            }
        }
        __syncthreads();

        // ---- scores of row rr against keys c, c + 8, c + 16, c + 24
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        const float* qrow = Qs + rr * qpitch;
        for (int d = 0; d < hd; ++d) {
            const float qv = qrow[d];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) s[jj] = fmaf(qv, Ks[(c + 8 * jj) * qpitch + d], s[jj]);
        }
        float tile_max = -INFINITY;
        bool ok[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int u = k0 + c + 8 * jj;
            const int kpos = u < n_kept ? u : win_lo + (u - n_kept);
            ok[jj] = u < k_hi && kpos <= my_qpos && (p.window <= 0 || kpos > my_qpos - p.window || kpos < p.keep_first);
            s[jj] *= p.scale;
            if (p.softcap > 0.f) s[jj] = p.softcap * tanhf(s[jj] / p.softcap);
            if (ok[jj] && p.rel != nullptr) s[jj] += p.rel[(size_t)p.bucket[min(my_qpos - kpos, p.n_bucket - 1)] * p.n_heads + my_head];
            if (ok[jj]) tile_max = fmaxf(tile_max, s[jj]);
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
        const float m_new = fmaxf(m, tile_max);
        float alpha = 1.f, row_sum = 0.f;
        float pr[4] = {0.f, 0.f, 0.f, 0.f};
        if (m_new != -INFINITY) {
            alpha = expf(m - m_new);  // m = -inf gives 0
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                pr[jj] = ok[jj] ? expf(s[jj] - m_new) : 0.f;
                row_sum += pr[jj];
            }
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) row_sum += __shfl_xor_sync(0xffffffffu, row_sum, o);
        l = l * alpha + row_sum;
        m = m_new;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) Ss[rr * (TK + 1) + c + 8 * jj] = pr[jj];
#pragma unroll
        for (int j = 0; j < HD_MAX / 8; ++j) acc[j] *= alpha;
        __syncthreads();

        // ---- accumulate probabilities times values; this thread owns lanes c, c + 8, ...
        const float* prow = Ss + rr * (TK + 1);
        for (int j = 0; j < TK; ++j) {
            const float pj = prow[j];
            const float* vrow = Vs + j * dv + c;
#pragma unroll
            for (int jd = 0; jd < HD_MAX / 8; ++jd)
                if (c + jd * 8 < dv) acc[jd] = fmaf(pj, vrow[jd * 8], acc[jd]);
        }
    }

    if (rr >= n_rows) return;
    const int tok = qs + tok0 + rr / ng;
    const int head = kvh * p.group + g0 + rr % ng;
    const size_t row = (size_t)tok * p.n_heads + head;
    if (p.n_splits == 1) {
        T* o = reinterpret_cast<T*>(p.out) + row * dv;
        float* o32 = reinterpret_cast<float*>(p.out) + row * dv;
        if (p.sinks != nullptr) {
            // one more term of the denominator: exp(sink - M) with M = max(m, sink), everything else rescaled to M
            const float sink = p.sinks[head];
            const float M = fmaxf(m, sink);
            const float a = expf(m - M);           // m = -inf (no visible key) gives 0
            l = l * a + expf(sink - M);
#pragma unroll
            for (int jd = 0; jd < HD_MAX / 8; ++jd) acc[jd] *= a;
        }
        float inv = l > 0.f ? 1.f / l : 0.f;
        const T* gate = reinterpret_cast<const T*>(p.gate);
        if (p.gate_mode == 1) inv *= to_float(gate[row]);
#pragma unroll
        for (int jd = 0; jd < HD_MAX / 8; ++jd)
            if (c + jd * 8 < dv) {
                const float v = acc[jd] * inv * (p.gate_mode == 2 ? to_float(gate[row * dv + c + jd * 8]) : 1.f);
                if (p.out_f32) o32[c + jd * 8] = v;
                else o[c + jd * 8] = from_float<T>(v);
            }
    } else {
        float* o = p.part_o + (row * p.n_splits + split) * dv;
#pragma unroll
        for (int jd = 0; jd < HD_MAX / 8; ++jd)
            if (c + jd * 8 < dv) o[c + jd * 8] = acc[jd];
        if (c == 0) {
            float* ml = p.part_ml + (row * p.n_splits + split) * 2;
            ml[0] = m;
            ml[1] = l;
        }
    }
}

// out[row, d] = sum_i e^{m_i - M} o_i[d] / sum_i e^{m_i - M} l_i,  M = max_i m_i
template <typename T>
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       T* __restrict__ out, int n_splits, int head_dim,
                                       const T* __restrict__ gate, int gate_mode, int out_f32,
                                       const float* __restrict__ sinks, int n_heads) {
    const size_t row = blockIdx.x;
    const float* ml = part_ml + row * n_splits * 2;
    float M = -INFINITY;
    for (int i = 0; i < n_splits; ++i) M = fmaxf(M, ml[2 * i]);
    const float sink = sinks != nullptr ? sinks[row % n_heads] : -INFINITY;
    M = fmaxf(M, sink);
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float num = 0.f, den = 0.f;
        for (int i = 0; i < n_splits; ++i) {
            const float mi = ml[2 * i];
            if (mi == -INFINITY) continue;
            const float w = expf(mi - M);
            num = fmaf(w, part_o[(row * n_splits + i) * head_dim + d], num);
            den = fmaf(w, ml[2 * i + 1], den);
        }
        if (sinks != nullptr) den += expf(sink - M);
        float o = den > 0.f ? num / den : 0.f;
        if (gate_mode == 1) o *= to_float(gate[row]);
        else if (gate_mode == 2) o *= to_float(gate[row * head_dim + d]);
        if (out_f32) reinterpret_cast<float*>(out)[row * head_dim + d] = o;
        else out[row * head_dim + d] = from_float<T>(o);
    }
}

struct Plan {
    int gchunk, n_gchunks, tokens_per_tile, n_q_tiles, n_splits;
};

Plan make_plan(int n_seqs, int n_heads, int n_kv_heads, int max_q_len, int max_kv_len, int allow_split,
               int window = 0, int keep_first = 0) {
    // what a query tile can see at most: behind a window the context's length does not matter
    if (window > 0 && max_kv_len > (long long)window + keep_first + max_q_len) max_kv_len = window + keep_first + max_q_len;
    Plan pl;
    const int group = n_heads / n_kv_heads;
    pl.gchunk = group < R ? group : R;
    pl.n_gchunks = (group + pl.gchunk - 1) / pl.gchunk;
    pl.tokens_per_tile = R / pl.gchunk;
    pl.n_q_tiles = (max_q_len + pl.tokens_per_tile - 1) / pl.tokens_per_tile;
    pl.n_splits = 1;
    const long long base = (long long)pl.n_q_tiles * n_kv_heads * pl.n_gchunks * n_seqs;
    if (allow_split && base < TARGET_CTAS && max_kv_len >= 2 * MIN_SPLIT) {
        const int want = (int)((TARGET_CTAS + base - 1) / base);
        const int most = max_kv_len / MIN_SPLIT;
        pl.n_splits = want < most ? want : most;
        if (pl.n_splits < 1) pl.n_splits = 1;
    }
    return pl;
}

size_t smem_bytes(int hd, int dv) { return (size_t)(R * (hd + 1) + TK * (hd + 1) + TK * dv + R * (TK + 1)) * sizeof(float); }

template <typename T, int HD_MAX>
int launch(const AttnParams& p, dim3 grid, cudaStream_t s) {
    const size_t smem = smem_bytes(p.head_dim, p.v_head_dim);
    auto kern = paged_attention_kernel<T, HD_MAX>;
    static int raised = 0;         // per instantiation: the largest limit set so far
    if (smem > 48 * 1024 && (int)smem > raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = (int)smem;
    }
    kern<<<grid, NT, smem, s>>>(p);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

template <typename T>
int launch_hd(const AttnParams& p, dim3 grid, cudaStream_t s) {
    const int widest = p.head_dim > p.v_head_dim ? p.head_dim : p.v_head_dim;
    if (widest <= 64) return launch<T, 64>(p, grid, s);
    if (widest <= 128) return launch<T, 128>(p, grid, s);
    if (widest <= 256) return launch<T, 256>(p, grid, s);
    return launch<T, 512>(p, grid, s);
}

}  // namespace

// What a call may switch on beyond plain causal (windowed) attention; see the top of this file.
// Zeros and nulls mean "off"; v_head_dim 0 means "as head_dim".
struct TlAttentionOptions {
    int v_head_dim;
    int keep_first;
    const float* rel;       // [rows, n_heads]
    const int* bucket;      // [n_bucket]
    int n_bucket;
    const void* gate;       // in q's dtype
    int gate_mode;          // 0: none, 1: [tokens, n_heads], 2: [tokens, n_heads * v_head_dim]
    int n_v_heads;          // 0: as n_kv_heads; else it divides n_kv_heads, and v_pages has so many heads
    int out_f32;            // 1: out is float32 whatever q's dtype
    float softcap;          // 0: none
    const float* sinks;     // [n_heads] or null
    int v_stride;           // 0: as v_head_dim
};

// How many key splits the general kernel would use for this batch, and how many float32 words of
// workspace (partials and their max / sum) the caller must provide.  n_splits == 1 needs none.
extern "C" int tl_attention_plan_ex(int n_tokens, int n_seqs, int n_heads, int n_kv_heads, int head_dim,
                                    int v_head_dim, int max_q_len, int max_kv_len, int window, int keep_first,
                                    int allow_split, int* n_splits, long long* workspace_floats) {
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return TL_BAD_SIZE;
    if (v_head_dim <= 0) v_head_dim = head_dim;
    if (head_dim <= 0 || head_dim > 512 || v_head_dim > 512) return TL_BAD_SIZE;
    const Plan pl = make_plan(n_seqs, n_heads, n_kv_heads, max_q_len, max_kv_len, allow_split, window, keep_first);
    *n_splits = pl.n_splits;
    *workspace_floats = pl.n_splits > 1 ? (long long)n_tokens * n_heads * pl.n_splits * (v_head_dim + 2) : 0;
    return TL_OK;
}

extern "C" int tl_attention_plan(int n_tokens, int n_seqs, int n_heads, int n_kv_heads, int head_dim,
                                 int max_q_len, int max_kv_len, int allow_split,
                                 int* n_splits, long long* workspace_floats) {
    return tl_attention_plan_ex(n_tokens, n_seqs, n_heads, n_kv_heads, head_dim, head_dim, max_q_len, max_kv_len, 0, 0,
                                allow_split, n_splits, workspace_floats);
}

// q: [n_tokens, n_heads, head_dim]; out: [n_tokens, n_heads, v_head_dim]; k_pages: [n_pages, n_kv_heads,
// page_size, head_dim]; v_pages: the same with v_head_dim; block_table: [n_seqs, table_stride]; q_start:
// [n_seqs + 1]; kv_len: [n_seqs] (length after this step's tokens were appended).  workspace: float32, as
// large as tl_attention_plan_ex said for the same window and keep_first (may be null when it said 0).
// window <= 0 means no window.
extern "C" int tl_paged_attention_ex(const void* q, const void* k_pages, const void* v_pages, void* out,
                                     const int* block_table, int table_stride, const int* q_start,
                                     const int* kv_len, float* workspace, int dtype, int n_tokens, int n_seqs,
                                     int n_heads, int n_kv_heads, int head_dim, int page_size, int max_q_len,
                                     int max_kv_len, int window, float scale, int allow_split,
                                     const TlAttentionOptions* opt, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return TL_OK;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || page_size <= 0) return TL_BAD_SIZE;
    TlAttentionOptions o = {};
    if (opt != nullptr) o = *opt;
    if (o.v_head_dim <= 0) o.v_head_dim = head_dim;
    if (window <= 0) window = 0;
    if (head_dim <= 0 || head_dim > 512 || o.v_head_dim > 512) return TL_BAD_SIZE;
    if (max_q_len <= 0 || max_kv_len <= 0) return TL_BAD_SIZE;
    if (o.keep_first < 0 || (o.keep_first > 0 && window == 0)) return TL_BAD_SIZE;
    if (o.rel != nullptr && (o.bucket == nullptr || o.n_bucket <= 0)) return TL_BAD_SIZE;
    if (o.gate_mode < 0 || o.gate_mode > 2 || (o.gate_mode != 0 && o.gate == nullptr)) return TL_BAD_SIZE;
    if (o.n_v_heads <= 0) o.n_v_heads = n_kv_heads;
    if (o.v_stride <= 0) o.v_stride = o.v_head_dim;
    if (o.v_stride < o.v_head_dim || o.softcap < 0.f) return TL_BAD_SIZE;
    if (n_kv_heads % o.n_v_heads != 0 || (o.n_v_heads != n_kv_heads && v_pages == k_pages)) return TL_BAD_SIZE;
    if (!aligned16(q) || !aligned16(k_pages) || !aligned16(v_pages) || !aligned16(out)) return TL_BAD_ALIGN;
    const Plan pl = make_plan(n_seqs, n_heads, n_kv_heads, max_q_len, max_kv_len, allow_split, window, o.keep_first);
    if (pl.n_splits > 1 && workspace == nullptr) return TL_BAD_SIZE;
    if (n_seqs > 65535 || (long long)n_kv_heads * pl.n_gchunks > 65535) return TL_BAD_SIZE;
    if (smem_bytes(head_dim, o.v_head_dim) > 200 * 1024) return TL_TOO_LARGE;

    AttnParams p;
    p.q = q; p.k_pages = k_pages; p.v_pages = v_pages; p.out = out;
    p.block_table = block_table; p.q_start = q_start; p.kv_len = kv_len;
    p.table_stride = table_stride;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.v_head_dim = o.v_head_dim;
    p.page_size = page_size;
    p.group = n_heads / n_kv_heads; p.gchunk = pl.gchunk; p.n_gchunks = pl.n_gchunks;
    p.tokens_per_tile = pl.tokens_per_tile;
    p.window = window;
    p.keep_first = o.keep_first;
    p.rel = o.rel; p.bucket = o.bucket; p.n_bucket = o.n_bucket;
    p.gate = o.gate; p.gate_mode = o.gate_mode;
    p.n_v_heads = o.n_v_heads; p.out_f32 = o.out_f32;
    p.v_stride = o.v_stride; p.softcap = o.softcap; p.sinks = o.sinks;
    p.n_splits = pl.n_splits;
    p.scale = scale;
    p.part_o = workspace;
    p.part_ml = workspace ? workspace + (size_t)n_tokens * n_heads * pl.n_splits * o.v_head_dim : nullptr;

    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(pl.n_q_tiles * pl.n_splits, n_kv_heads * pl.n_gchunks, n_seqs);
    int rc;
    if (dtype == TL_F32) rc = launch_hd<float>(p, grid, s);
    else if (dtype == TL_BF16) rc = launch_hd<__nv_bfloat16>(p, grid, s);
    else return TL_BAD_DTYPE;
    if (rc != TL_OK) return rc;
    if (pl.n_splits > 1) {
        const int threads = o.v_head_dim >= 128 ? 128 : 64;
        const unsigned rows = (unsigned)n_tokens * n_heads;
        if (dtype == TL_F32)
            attention_merge_kernel<float><<<rows, threads, 0, s>>>(p.part_o, p.part_ml, (float*)out, pl.n_splits, o.v_head_dim,
                                                                    (const float*)o.gate, o.gate_mode, o.out_f32, o.sinks, n_heads);
        else
            attention_merge_kernel<__nv_bfloat16><<<rows, threads, 0, s>>>(p.part_o, p.part_ml, (__nv_bfloat16*)out, pl.n_splits,
                                                                            o.v_head_dim, (const __nv_bfloat16*)o.gate, o.gate_mode, o.out_f32,
                                                                            o.sinks, n_heads);
        TL_LAUNCH_CHECK();
    }
    return TL_OK;
}

// The plain form: keys and values of one size (a multiple of 16), no options.
extern "C" int tl_paged_attention(const void* q, const void* k_pages, const void* v_pages, void* out,
                                  const int* block_table, int table_stride, const int* q_start,
                                  const int* kv_len, float* workspace, int dtype, int n_tokens, int n_seqs,
                                  int n_heads, int n_kv_heads, int head_dim, int page_size, int max_q_len,
                                  int max_kv_len, int window, float scale, int allow_split, void* stream) {
    if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 256) return TL_BAD_SIZE;
    // (tl_attention_plan does not look at the window, so it never asks for less workspace than this call uses)
    TlAttentionOptions o = {};
    return tl_paged_attention_ex(q, k_pages, v_pages, out, block_table, table_stride, q_start, kv_len, workspace, dtype,
                                 n_tokens, n_seqs, n_heads, n_kv_heads, head_dim, page_size, max_q_len, max_kv_len, window,
                                 scale, allow_split, &o, stream);
}

// ---------------------------------------------------------------------------------------------
// The same attention for callers that may not allocate: the split-KV partials live in a fixed
// array inside this library instead of a workspace the caller brings.  See
// attention_static_scratch.h for who needs this and for the rules of use.
#include "attention_static_scratch.h"

namespace {

// Part of the library image: present on every device that loads it, until the process ends.
static __device__ __align__(256) float tl_static_scratch[TL_STATIC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
float* static_scratch_address[MAX_DEVICES] = {};   // per device, asked for once

// In host code the array's name is only a handle for the runtime, not a pointer a kernel could
// use; the device address has to be asked for, with the right device current.
int static_scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return TL_STATIC_SCRATCH_NO_ADDRESS;
    if (static_scratch_address[dev] == nullptr) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, tl_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (ptr == nullptr) return TL_STATIC_SCRATCH_NO_ADDRESS;
        static_scratch_address[dev] = ptr;
    }
    *out = static_scratch_address[dev];
    return TL_OK;
}

}  // namespace

extern "C" int tl_paged_attention_static_scratch(const void* q, const void* k_pages, const void* v_pages, void* out,
                                                 const int* block_table, int table_stride, const int* q_start,
                                                 const int* kv_len, int dtype, int n_tokens, int n_seqs, int n_heads,
                                                 int n_kv_heads, int head_dim, int page_size, int max_q_len,
                                                 int max_kv_len, int window, float scale, int allow_split, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return TL_OK;
    int n_splits = 0;
    long long floats = 0;
    int rc = tl_attention_plan(n_tokens, n_seqs, n_heads, n_kv_heads, head_dim, max_q_len, max_kv_len, allow_split,
                               &n_splits, &floats);
    if (rc != TL_OK) return rc;
    if (floats > (long long)TL_STATIC_SCRATCH_FLOATS) return TL_STATIC_SCRATCH_TOO_SMALL;   // nothing was launched
    float* scratch = nullptr;
    rc = static_scratch_for_current_device(&scratch);
    if (rc != TL_OK) return rc;
    // Every (row, split) cell that the merge reads is written by the attention kernel of this same
    // call first, so what an earlier call left in the array does not matter and nothing is cleared.
    return tl_paged_attention(q, k_pages, v_pages, out, block_table, table_stride, q_start, kv_len, scratch, dtype,
                              n_tokens, n_seqs, n_heads, n_kv_heads, head_dim, page_size, max_q_len, max_kv_len,
                              window, scale, allow_split, stream);
}

extern "C" const char* tl_static_scratch_strerror(int code) {
    switch (code) {
        case TL_OK: return "ok";
        case TL_STATIC_SCRATCH_TOO_SMALL:
            return "this step needs more split-KV scratch than the 8 MiB array built into the library holds; "
                   "use fewer tokens, heads or splits per call, or tl_paged_attention with a workspace of your own";
        case TL_STATIC_SCRATCH_NO_ADDRESS:
            return "the runtime gave no device address for the built-in scratch array on the current device";
        default: return "see the status codes of tl_paged_attention";
    }
}
