// Causal grouped-query attention over paged bfloat16 keys and values on the tensor cores
// (mma.sync m16n8k16, float32 accumulation), for head_dim 16, 32, 64 and 128.  Same contract as
// the general kernel in attention.cu: any mix of prompt portions and decoded tokens, bottom-right
// aligned causal mask, optional sliding window, block tables, scores / running maximum / sums /
// output accumulators in float32 (torchllms/models/networks.py:355-397 is the formula).
//
// Rows are (token, query head of one kv group) pairs, 16 to a warp, so the heads of a group
// share every key and value tile.  Keys and values come in tiles of 64 through a two-stage
// cp.async pipeline in shared memory (rows padded by 16 bytes: ldmatrix without bank conflicts).
//
// Two shapes of work, one kernel body:
//   row split  (prompt portions): a CTA owns 64 rows, 16 per warp; every warp walks all keys.
//   key split  (decoding and very short portions: a request's rows fit one 16-row tile): the four
//              warps share the 16 rows and each takes a quarter of every key tile; their partial
//              (max, sum, accumulator) are merged through shared memory.  The key range may also be
//              cut over several CTAs; those partials go to a float32 workspace and are combined
//              by merge_partials_kernel (same layout as the general kernel's).
//
// The extended form (template flag EXT, a separate entry point) also takes what the general
// kernel's options describe: keys and values of sizes of their own (multiples of 8 up to the
// instantiated size, the tiles' spare columns zero-filled), one stored vector read as key and as
// value (the value tile is the key tile), a window that keeps a request's first keys visible (they
// are walked as tiles of their own ahead of the window's), a bias by bucketed distance added to the
// scaled score, an output gate per head or per element, a cap on the scaled score (c * tanh(s / c)), a learned
// sink per head in the softmax's denominator, and values that are the first coordinates of the stored keys; and
// it multiplies probabilities as three bfloat16 terms, which add up to the float32 probability exactly.
#include "common.cuh"
#include <limits.h>
#include <math.h>

namespace {

constexpr int BN = 64;       // keys per tile
constexpr int NW = 4;        // warps per CTA
constexpr int NT = NW * 32;
constexpr int TARGET_CTAS = 148 * 3;   // three CTAs of the key-split shape fit an SM
constexpr int MIN_SPLIT = 128;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct MmaParams {
    const __nv_bfloat16* q;
    const __nv_bfloat16* k_pages;
    const __nv_bfloat16* v_pages;
    __nv_bfloat16* out;
    const int* block_table;
    const int* q_start;
    const int* kv_len;
    float* part_o;   // [T * H, n_splits, head_dim]
    float* part_ml;  // [T * H, n_splits, 2]
    int table_stride;
    int n_heads, n_kv_heads, page_size;
    int page_shift;             // log2(page_size) when it is a power of two, else -1
    int group, ng, n_gchunks;   // ng: heads of a group per 16-row tile
    int tpw;                    // tokens per 16-row tile
    int window;
    int n_splits;
    float scale_log2;           // scale * log2(e)
    // ---- the extended form only
    int hd, dv;                 // true sizes of a key and of a value
    int shared_kv;              // 1: v_pages is k_pages, a tile is loaded once
    int keep_first;
    const float* rel;           // [rows, n_heads] or null
    const int* bucket;          // [n_bucket]
    int n_bucket;
    const __nv_bfloat16* gate;
    int gate_mode;              // 0: none, 1: [T, n_heads], 2: [T, n_heads * dv]
    int bias_cols;              // row split: the bias of so many distances (from 0) is tabulated in shared memory per head of the tile
    int n_v_heads;              // value heads of v_pages; key head j goes with value head j % n_v_heads
    int out_f32;                // 1: out holds float32
    float cap_log2;             // softcap * log2(e); 0: scores are not capped
    float scale_over_cap;       // scale / softcap
    const float* sinks;         // [n_heads] or null (natural-log scale, as stored)
};

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {     // 2^x, one instruction; 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

template <int HD, bool KEY_SPLIT, bool EXT>
__global__ void __launch_bounds__(NT, KEY_SPLIT ? 4 : 2) attention_mma_kernel(const MmaParams p) {
    const int hd = EXT ? p.hd : HD, dv = EXT ? p.dv : HD;
    constexpr int PITCH = HD + 8;                 // bf16 elements per shared-memory row
    constexpr int QROWS = KEY_SPLIT ? 16 : 16 * NW;
    constexpr int KG = KEY_SPLIT ? 1 : 4;         // 16-key groups of a tile that one warp handles
    constexpr int KSTEPS = HD / 16;
    constexpr int CHUNKS = HD / 8;                // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);    // [QROWS][PITCH]
    __nv_bfloat16* Ks = Qs + QROWS * PITCH;                            // [2][BN][PITCH]
    __nv_bfloat16* Vs = Ks + 2 * BN * PITCH;                           // [2][BN][PITCH]
    float* Bs = reinterpret_cast<float*>(Vs + 2 * BN * PITCH);         // [ng][bias_cols] (EXT, row split, with a bias)

    const int b = blockIdx.z;
    const int qs = p.q_start[b];
    const int ql = p.q_start[b + 1] - qs;
    const int kl = p.kv_len[b];
    // (prompt portions in the extended form: the last query tiles, which see the most keys, start first,
    // so that the short walks of a portion's first tiles fill the end of the launch)
    const int tile = (EXT && !KEY_SPLIT) ? (int)(gridDim.x / p.n_splits) - 1 - (int)(blockIdx.x / p.n_splits)
                                         : (int)(blockIdx.x / p.n_splits);
    const int split = blockIdx.x % p.n_splits;
    const int tokens_per_cta = KEY_SPLIT ? p.tpw : p.tpw * NW;
    const int tok0 = tile * tokens_per_cta;
    if (tok0 >= ql) return;
    const int kvh = blockIdx.y / p.n_gchunks;
    const int g0 = (blockIdx.y - kvh * p.n_gchunks) * p.ng;
    const int ng = min(p.ng, p.group - g0);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    // ---- queries into shared memory (zero rows where the tile has no row)
    for (int c = tid; c < QROWS * CHUNKS; c += NT) {
        const int r = c / CHUNKS, part = c - r * CHUNKS;
        const int wtile = KEY_SPLIT ? 0 : r >> 4;        // which warp's 16-row tile
        const int rr = r & 15;
        const int tok = tok0 + wtile * p.tpw + rr / ng;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (rr < p.tpw * ng && tok < ql && part * 8 < hd) {
            const int head = kvh * p.group + g0 + rr % ng;
            v = *reinterpret_cast<const uint4*>(p.q + ((size_t)(qs + tok) * p.n_heads + head) * hd + part * 8);
        }
        *reinterpret_cast<uint4*>(Qs + r * PITCH + part * 8) = v;
    }

    // ---- the bias by distance of the tile's heads, on the base-2 scale (a prompt's CTA asks for the same few
    // hundred distances tens of thousands of times)
    const int bias_cols = (EXT && !KEY_SPLIT && p.rel != nullptr) ? p.bias_cols : 0;
    for (int c = tid; c < ng * bias_cols; c += NT) {
        const int hl = c / bias_cols, d = c - hl * bias_cols;
        Bs[c] = __ldg(p.rel + (size_t)__ldg(p.bucket + min(d, p.n_bucket - 1)) * p.n_heads + kvh * p.group + g0 + hl) * LOG2E;
    }

    // ---- which keys this CTA walks
    const int cta_tok_hi = min(ql, tok0 + tokens_per_cta);              // exclusive
    const int qpos_base = kl - ql;
    // The window's keys start at win_lo; ahead of them, in tiles of their own, the kept first keys
    // that the window of the CTA's earliest query has passed (none unless EXT).  Tile i of the walk
    // starts at key tile_k0(i) and ends before tile_hi(i).
    const int win_lo = p.window > 0 ? max(0, qpos_base + tok0 - p.window + 1) : 0;
    const int win_hi = qpos_base + cta_tok_hi;                           // last query's position + 1
    const int n_kept = EXT ? min(p.keep_first, win_lo) : 0;
    const int kept_tiles = (n_kept + BN - 1) / BN;
    int t_lo = 0, t_hi = kept_tiles + (win_hi > win_lo ? (win_hi - win_lo + BN - 1) / BN : 0);
    if (p.n_splits > 1) {
        // every request cuts its own visible keys evenly, in whole tiles, so the launch shape
        // depends on the batch size only and not on how long the requests have grown
        const int per = (t_hi + p.n_splits - 1) / p.n_splits;
        t_lo = split * per;
        t_hi = min(t_hi, t_lo + per);
    }
    auto tile_k0 = [&](int i) { return i < kept_tiles ? i * BN : win_lo + (i - kept_tiles) * BN; };
    auto tile_hi = [&](int i) { return i < kept_tiles ? n_kept : win_hi; };

    // rows of this thread: g and g + 8 of the warp's tile
    const int wtile = KEY_SPLIT ? 0 : warp;
    int qpos[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int rr = g + 8 * i;
        const int tok = tok0 + wtile * p.tpw + rr / ng;
        qpos[i] = (rr < p.tpw * ng && tok < ql) ? qpos_base + tok : -1;
    }
    const int warp_qmax = __reduce_max_sync(0xffffffffu, max(qpos[0], qpos[1]));
    // smallest position among the warp's real rows (rows without a query are never stored)
    const int warp_qmin = __reduce_min_sync(0xffffffffu, min(qpos[0] < 0 ? INT_MAX : qpos[0], qpos[1] < 0 ? INT_MAX : qpos[1]));

    const int* table = p.block_table + (size_t)b * p.table_stride;
    // A thread always copies the same 16-byte column of a row: chunk c = tid + i * NT covers key
    // (tid / CHUNKS) + i * (NT / CHUNKS), column tid % CHUNKS.
    const int ld_part = (tid % CHUNKS) * 8;
    const int ld_key0 = tid / CHUNKS;
    constexpr int LD_STEP = NT / CHUNKS;          // keys between two chunks of one thread
    constexpr int LD_ITERS = BN / LD_STEP;
    const size_t page_stride_k = (size_t)p.n_kv_heads * p.page_size * hd;
    const int n_vh = EXT ? p.n_v_heads : p.n_kv_heads;
    const size_t page_stride_v = (size_t)n_vh * p.page_size * dv;
    const size_t head_off_k = (size_t)kvh * p.page_size * hd + ld_part;
    const size_t head_off_v = (size_t)(kvh % n_vh) * p.page_size * dv + ld_part;
    const bool k_real = ld_part < hd, v_real = ld_part < dv && !(EXT && p.shared_kv);
    auto load_tile = [&](int stage, int k0, int k_end) {
        __nv_bfloat16* kd = Ks + stage * BN * PITCH + ld_part;
        __nv_bfloat16* vd = Vs + stage * BN * PITCH + ld_part;
#pragma unroll
        for (int i = 0; i < LD_ITERS; ++i) {
            const int j = ld_key0 + i * LD_STEP;
            const int kpos = k0 + j;
            bool k_done = false, v_done = false;
            if (kpos < k_end) {   // kpos >= the walk's first key always: pages behind a window may be gone and are never touched
                int blk, slot;
                if (p.page_shift >= 0) {
                    blk = kpos >> p.page_shift;
                    slot = kpos & (p.page_size - 1);
                } else {
                    blk = kpos / p.page_size;
                    slot = kpos - blk * p.page_size;
                }
                const size_t page = (size_t)(tl_check_page(table[blk]) ? table[blk] : 0);   // (debug builds: a bad page is reported, page 0 read in its place)
                if (k_real) {
                    cp_async16(kd + j * PITCH, p.k_pages + page * page_stride_k + head_off_k + (size_t)slot * hd);
                    k_done = true;
                }
                if (v_real) {
                    cp_async16(vd + j * PITCH, p.v_pages + page * page_stride_v + head_off_v + (size_t)slot * dv);
                    v_done = true;
                }
            }
            if (!k_done) *reinterpret_cast<uint4*>(kd + j * PITCH) = make_uint4(0u, 0u, 0u, 0u);
            if (!v_done && !(EXT && p.shared_kv)) *reinterpret_cast<uint4*>(vd + j * PITCH) = make_uint4(0u, 0u, 0u, 0u);
        }
    };

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    unsigned qf[KSTEPS][4];

    const int n_tiles = max(t_hi - t_lo, 0);
    if (n_tiles > 0) load_tile(0, tile_k0(t_lo), tile_hi(t_lo));
    cp_async_commit();
    __syncthreads();   // Qs is complete
#pragma unroll
    for (int kd = 0; kd < KSTEPS; ++kd) {
        const int mi = lane >> 3;
        const int row = (KEY_SPLIT ? 0 : warp * 16) + (lane & 7) + ((mi & 1) ? 8 : 0);
        ldmatrix_x4(qf[kd], Qs + row * PITCH + kd * 16 + ((mi & 2) ? 8 : 0));
    }

    for (int it = 0; it < n_tiles; ++it) {
        const int k0 = tile_k0(t_lo + it), k_hi = tile_hi(t_lo + it);
        if (it + 1 < n_tiles) load_tile((it + 1) & 1, tile_k0(t_lo + it + 1), tile_hi(t_lo + it + 1));
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* kt = Ks + (it & 1) * BN * PITCH;
        const __nv_bfloat16* vt = (EXT && p.shared_kv) ? kt : Vs + (it & 1) * BN * PITCH;
        const int key_off = KEY_SPLIT ? warp * 16 : 0;
        if (k0 + key_off <= warp_qmax) {     // else every key of this warp's share lies beyond its queries
            float s[2 * KG][4];
#pragma unroll
            for (int i = 0; i < 2 * KG; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int kd = 0; kd < KSTEPS; ++kd) {
#pragma unroll
                for (int np = 0; np < KG; ++np) {
                    unsigned kf[4];
                    const int mi = lane >> 3;
                    const int key = key_off + np * 16 + (lane & 7) + ((mi & 2) ? 8 : 0);
                    ldmatrix_x4(kf, kt + key * PITCH + kd * 16 + ((mi & 1) ? 8 : 0));
                    mma_bf16(s[2 * np], qf[kd], kf[0], kf[1]);
                    mma_bf16(s[2 * np + 1], qf[kd], kf[2], kf[3]);
                }
            }
            // ---- mask, streaming softmax (base 2; the scale is folded into the exponent)
            float mx[2] = {-INFINITY, -INFINITY};
            const int share_lo = k0 + key_off, share_hi = share_lo + 16 * KG;   // this warp's keys of the tile
            const bool biased = EXT && p.rel != nullptr;
            const bool capped = EXT && p.cap_log2 > 0.f;        // (never together with a bias: the host sends those elsewhere)
            if (capped) {
                // c * tanh(score * scale / c), on the base-2 scale; hidden keys are masked below as usual
#pragma unroll
                for (int nt = 0; nt < 2 * KG; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[nt][e] = p.cap_log2 * tanhf(s[nt][e] * p.scale_over_cap);
            }
            const float sl = (biased || capped) ? 1.f : p.scale_log2;       // biased and capped scores are on the base-2 scale already
            const bool all_visible = share_hi <= k_hi && share_hi - 1 <= warp_qmin &&
                                     (p.window <= 0 || share_lo > warp_qmax - p.window);
            if (biased && all_visible && warp_qmax - share_lo < bias_cols) {
                // every key of the share counts for every row and every distance is in the table
                const float* brow[2] = {Bs + (g % ng) * bias_cols + (qpos[0] - share_lo - 2 * t),
                                        Bs + ((g + 8) % ng) * bias_cols + (qpos[1] - share_lo - 2 * t)};
                if (qpos[0] < 0) brow[0] = brow[1];          // a row without a query: any valid address (it is never stored)
                if (qpos[1] < 0) brow[1] = brow[0];
#pragma unroll
                for (int nt = 0; nt < 2 * KG; ++nt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        s[nt][e] = fmaf(s[nt][e], p.scale_log2, brow[e >> 1][-(nt * 8 + (e & 1))]);
                }
            } else if (biased) {
                // score * scale + rel[bucket[distance], head], on the base-2 scale; hidden keys get -inf
                int head[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) head[i] = kvh * p.group + g0 + (g + 8 * i) % ng;
#pragma unroll
                for (int nt = 0; nt < 2 * KG; ++nt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = e >> 1;
                        const int kpos = share_lo + nt * 8 + 2 * t + (e & 1);
                        const bool ok = kpos <= qpos[i] && kpos < k_hi &&
                                        (p.window <= 0 || kpos > qpos[i] - p.window || kpos < p.keep_first);
                        float v = -INFINITY;
                        if (ok) {
                            const int dist = qpos[i] - kpos;
                            float bias;
                            if (dist < bias_cols) {
                                bias = Bs[((g + 8 * i) % ng) * bias_cols + dist];
                            } else {
                                const int row = __ldg(p.bucket + min(dist, p.n_bucket - 1));
                                bias = __ldg(p.rel + (size_t)row * p.n_heads + head[i]) * LOG2E;
                            }
                            v = fmaf(s[nt][e], p.scale_log2, bias);
                        }
                        s[nt][e] = v;
                    }
                }
            } else if (!all_visible) {      // else every key counts for every row: no per-element tests
#pragma unroll
                for (int nt = 0; nt < 2 * KG; ++nt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = e >> 1;
                        const int kpos = share_lo + nt * 8 + 2 * t + (e & 1);
                        const bool ok = kpos <= qpos[i] && kpos < k_hi &&
                                        (p.window <= 0 || kpos > qpos[i] - p.window || (EXT && kpos < p.keep_first));
                        if (!ok) s[nt][e] = -INFINITY;
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < 2 * KG; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
            float alpha[2], m_safe[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                const float m_new = fmaxf(m[i], mx[i] * sl);       // maxima live on the base-2 scale
                m_safe[i] = (m_new == -INFINITY) ? 0.f : m_new;                // no key seen yet: keep exponents finite
                alpha[i] = ex2(m[i] - m_safe[i]);
                m[i] = m_new;
                l[i] *= alpha[i];
            }
#pragma unroll
            for (int nt = 0; nt < 2 * KG; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = ex2(fmaf(s[nt][e], sl, -m_safe[e >> 1]));
                    s[nt][e] = pv;
                    l[e >> 1] += pv;
                }
            }
            if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {   // the maximum moved for some row
#pragma unroll
                for (int i = 0; i < HD / 8; ++i) {
                    o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                    o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
                }
            }
            // ---- accumulate probabilities times values.  A probability is split into two bfloat16
            // numbers (value and remainder) and multiplied twice, so the product keeps 16 bits of
            // it: rounding probabilities to 8 bits would depend on the running maximum, hence
            // on how the keys fall into tiles and the prompt into steps.
#pragma unroll
            // The extended form serves designs that ask for 32-bit attention weights: there a third term takes
            // what the first two leave, and the three bfloat16 numbers (8 + 8 + 8 bits) add up to the float32
            // probability exactly, so the product is the one of float32 weights with bfloat16 values.
            for (int kk = 0; kk < KG; ++kk) {
                unsigned ph[4], pl[4], pt[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float a = s[2 * kk + (r >> 1)][(r & 1) * 2], c = s[2 * kk + (r >> 1)][(r & 1) * 2 + 1];
                    const __nv_bfloat162 hi = __floats2bfloat162_rn(a, c);
                    const float2 back = __bfloat1622float2(hi);
                    ph[r] = *reinterpret_cast<const unsigned*>(&hi);
                    const float ra = a - back.x, rc = c - back.y;
                    const __nv_bfloat162 mid = __floats2bfloat162_rn(ra, rc);
                    pl[r] = *reinterpret_cast<const unsigned*>(&mid);
                    if (EXT) {
                        const float2 back2 = __bfloat1622float2(mid);
                        pt[r] = pack_bf16(ra - back2.x, rc - back2.y);
                    }
                }
#pragma unroll
                for (int dp = 0; dp < HD / 16; ++dp) {
                    unsigned vf[4];
                    const int mi = lane >> 3;
                    const int key = key_off + kk * 16 + (lane & 7) + ((mi & 1) ? 8 : 0);
                    ldmatrix_x4_trans(vf, vt + key * PITCH + dp * 16 + ((mi & 2) ? 8 : 0));
                    mma_bf16(o[2 * dp], ph, vf[0], vf[1]);
                    mma_bf16(o[2 * dp + 1], ph, vf[2], vf[3]);
                    mma_bf16(o[2 * dp], pl, vf[0], vf[1]);
                    mma_bf16(o[2 * dp + 1], pl, vf[2], vf[3]);
                    if (EXT) {
                        mma_bf16(o[2 * dp], pt, vf[0], vf[1]);
                        mma_bf16(o[2 * dp + 1], pt, vf[2], vf[3]);
                    }
                }
            }
        }
        __syncthreads();   // this stage may be overwritten by the load after next
    }
    cp_async_wait<0>();

    // the sums are per thread so far: add up the four lanes that share a row
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }

    if (!KEY_SPLIT) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (qpos[i] < 0) continue;
            const int rr = g + 8 * i;
            const int tok = qs + tok0 + warp * p.tpw + rr / ng;
            const int head = kvh * p.group + g0 + rr % ng;
            const size_t row = (size_t)tok * p.n_heads + head;
            __nv_bfloat16* dst = p.out + row * dv;
            if (EXT && p.sinks != nullptr) {
                // one more term of the denominator, without a value: everything is rescaled to max(m, sink)
                const float sink2 = p.sinks[head] * LOG2E;
                const float M = fmaxf(m[i], sink2);
                const float a = ex2(m[i] - M);
                l[i] = l[i] * a + ex2(sink2 - M);
#pragma unroll
                for (int nt = 0; nt < HD / 8; ++nt) { o[nt][2 * i] *= a; o[nt][2 * i + 1] *= a; }
            }
            float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
            if (EXT && p.gate_mode == 1) inv *= __bfloat162float(p.gate[row]);
#pragma unroll
            for (int nt = 0; nt < HD / 8; ++nt) {
                if (EXT && nt * 8 >= dv) break;
                float a = o[nt][2 * i] * inv, c = o[nt][2 * i + 1] * inv;
                if (EXT && p.gate_mode == 2) {
                    const float2 gv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p.gate + row * dv + nt * 8 + 2 * t));
                    a *= gv.x;
                    c *= gv.y;
                }
                if (EXT && p.out_f32) *reinterpret_cast<float2*>(reinterpret_cast<float*>(p.out) + row * dv + nt * 8 + 2 * t) = make_float2(a, c);
                else *reinterpret_cast<unsigned*>(dst + nt * 8 + 2 * t) = pack_bf16(a, c);
            }
        }
        return;
    }

    // ---- key split: merge the four warps' partials through shared memory (reusing the tile buffers)
    __syncthreads();
    float* Om = reinterpret_cast<float*>(smem_raw);       // [NW][16][HD]
    float* Mm = Om + NW * 16 * HD;                        // [NW][16]
    float* Lm = Mm + NW * 16;                             // [NW][16]
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int rr = g + 8 * i;
#pragma unroll
        for (int nt = 0; nt < HD / 8; ++nt) {
            Om[(warp * 16 + rr) * HD + nt * 8 + 2 * t] = o[nt][2 * i];
            Om[(warp * 16 + rr) * HD + nt * 8 + 2 * t + 1] = o[nt][2 * i + 1];
        }
        if (t == 0) {
            Mm[warp * 16 + rr] = m[i];
            Lm[warp * 16 + rr] = l[i];
        }
    }
    __syncthreads();
    const int n_rows = min(p.tpw, ql - tok0) * ng;
    for (int idx = tid; idx < n_rows * HD; idx += NT) {
        const int rr = idx / HD, d = idx - rr * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, Mm[w * 16 + rr]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float mw = Mm[w * 16 + rr];
            if (mw == -INFINITY) continue;
            const float f = exp2f(mw - M);
            num = fmaf(f, Om[(w * 16 + rr) * HD + d], num);
            den = fmaf(f, Lm[w * 16 + rr], den);
        }
        const int tok = qs + tok0 + rr / ng;
        const int head = kvh * p.group + g0 + rr % ng;
        const size_t row = (size_t)tok * p.n_heads + head;
        if (EXT && d >= dv) continue;
        if (p.n_splits == 1) {
            if (EXT && p.sinks != nullptr) {
                const float sink2 = p.sinks[head] * LOG2E;
                const float M2 = fmaxf(M, sink2);
                const float f = exp2f(M - M2);          // M = -inf (no key seen) gives 0
                num *= f;
                den = den * f + exp2f(sink2 - M2);
            }
            float v = den > 0.f ? num / den : 0.f;
            if (EXT && p.gate_mode == 1) v *= __bfloat162float(p.gate[row]);
            else if (EXT && p.gate_mode == 2) v *= __bfloat162float(p.gate[row * dv + d]);
            if (EXT && p.out_f32) reinterpret_cast<float*>(p.out)[row * dv + d] = v;
            else p.out[row * dv + d] = __float2bfloat16_rn(v);
        } else {
            p.part_o[(row * p.n_splits + split) * dv + d] = num;
            if (d == 0) {
                p.part_ml[(row * p.n_splits + split) * 2] = (M == -INFINITY) ? -INFINITY : M * LN2;   // natural-log scale
                p.part_ml[(row * p.n_splits + split) * 2 + 1] = den;
            }
        }
    }
}

// out[row, d] = sum_i e^{m_i - M} o_i[d] / sum_i e^{m_i - M} l_i,  M = max_i m_i.
// One CTA per row: the weights e^{m_i - M} are computed once (lanes over splits) into shared
// memory, then every thread sums its head_dim lanes over the splits in order.
constexpr int MERGE_MAX_SPLITS = 256;
__global__ void merge_partials_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      __nv_bfloat16* __restrict__ out, int n_splits, int head_dim,
                                      const __nv_bfloat16* __restrict__ gate = nullptr, int gate_mode = 0, int out_f32 = 0,
                                      const float* __restrict__ sinks = nullptr, int n_heads = 1) {
    __shared__ float wgt[MERGE_MAX_SPLITS];
    __shared__ float red[2];
    const size_t row = blockIdx.x;
    const float* ml = part_ml + row * n_splits * 2;
    if (threadIdx.x < 32) {
        float M = -INFINITY;
        for (int i = threadIdx.x; i < n_splits; i += 32) M = fmaxf(M, ml[2 * i]);
        M = warp_max(M);
        const float sink = sinks != nullptr ? sinks[row % n_heads] : -INFINITY;
        M = fmaxf(M, sink);
        float den = threadIdx.x == 0 && sinks != nullptr ? __expf(sink - M) : 0.f;
        for (int i = threadIdx.x; i < n_splits; i += 32) {
            const float mi = ml[2 * i];
            const float w = (mi == -INFINITY) ? 0.f : __expf(mi - M);
            wgt[i] = w;
            den = fmaf(w, ml[2 * i + 1], den);
        }
        den = warp_sum(den);
        if (threadIdx.x == 0) red[0] = den;
    }
    __syncthreads();
    const float den = red[0];
    const float inv = den > 0.f ? 1.f / den : 0.f;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float num = 0.f;
        for (int i = 0; i < n_splits; ++i) num = fmaf(wgt[i], part_o[(row * n_splits + i) * head_dim + d], num);
        float v = num * inv;
        if (gate_mode == 1) v *= __bfloat162float(gate[row]);
        else if (gate_mode == 2) v *= __bfloat162float(gate[row * head_dim + d]);
        if (out_f32) reinterpret_cast<float*>(out)[row * head_dim + d] = v;
        else out[row * head_dim + d] = __float2bfloat16_rn(v);
    }
}

struct Plan {
    int ng, n_gchunks, tpw, key_split, n_q_tiles, n_splits;
};

Plan make_plan(int n_seqs, int n_heads, int n_kv_heads, int max_q_len, int max_kv_len, int allow_split,
               int window = 0, int keep_first = 0) {
    Plan pl;
    // (the extended form tells its window: behind one, what a query tile sees does not grow with the context)
    if (window > 0 && max_kv_len > (long long)window + keep_first + max_q_len) max_kv_len = window + keep_first + max_q_len;
    const int group = n_heads / n_kv_heads;
    pl.ng = group < 16 ? group : 16;
    pl.n_gchunks = (group + pl.ng - 1) / pl.ng;
    pl.tpw = 16 / pl.ng;
    pl.key_split = max_q_len <= pl.tpw;
    const int tokens_per_cta = pl.key_split ? pl.tpw : pl.tpw * NW;
    pl.n_q_tiles = (max_q_len + tokens_per_cta - 1) / tokens_per_cta;
    pl.n_splits = 1;
    if (pl.key_split && allow_split && max_kv_len >= 2 * MIN_SPLIT) {
        // CTAs run in waves of TARGET_CTAS; with s splits a CTA does 1/s of the keys.  Pick the s
        // that makes (waves / s), the time in units of one unsplit CTA, smallest, charging each
        // split a little for its partial results and the merge.
        const long long base = (long long)pl.n_q_tiles * n_kv_heads * pl.n_gchunks * n_seqs;
        // (behind a window the keys are few: a split may be as short as one tile)
        int most = max_kv_len / (window > 0 ? BN : MIN_SPLIT);
        if (most > MERGE_MAX_SPLITS) most = MERGE_MAX_SPLITS;
        if (most > 64) most = 64;
        double best = 1e30;
        for (int sp = 1; sp <= most; ++sp) {
            const long long waves = (base * sp + TARGET_CTAS - 1) / TARGET_CTAS;
            const double cost = (double)waves / sp + 0.01 * sp;
            if (cost < best - 1e-9) {
                best = cost;
                pl.n_splits = sp;
            }
        }
    }
    return pl;
}

template <int HD, bool KEY_SPLIT, bool EXT = false>
int launch(const MmaParams& p, dim3 grid, cudaStream_t s) {
    constexpr int PITCH = HD + 8;
    constexpr int QROWS = KEY_SPLIT ? 16 : 16 * NW;
    size_t smem = (size_t)(QROWS + 4 * BN) * PITCH * sizeof(__nv_bfloat16);
    if (EXT && !KEY_SPLIT && p.rel != nullptr) smem += (size_t)p.ng * p.bias_cols * sizeof(float);
    const size_t merge = KEY_SPLIT ? (size_t)(NW * 16 * (HD + 2)) * sizeof(float) : 0;
    if (merge > smem) smem = merge;
    auto kern = attention_mma_kernel<HD, KEY_SPLIT, EXT>;
    static size_t raised = 48 * 1024;    // per instantiation: the largest limit set so far (one device per process)
    if (smem > raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = smem;
    }
    kern<<<grid, NT, smem, s>>>(p);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

template <int HD>
int launch_mode(const MmaParams& p, dim3 grid, bool key_split, cudaStream_t s) {
    return key_split ? launch<HD, true>(p, grid, s) : launch<HD, false>(p, grid, s);
}

template <int HD>
int launch_mode_ext(const MmaParams& p, dim3 grid, bool key_split, cudaStream_t s) {
    return key_split ? launch<HD, true, true>(p, grid, s) : launch<HD, false, true>(p, grid, s);
}

// the instantiated size that holds keys of hd and values of dv elements (0: none does)
int ext_size(int hd, int dv) {
    const int widest = hd > dv ? hd : dv;
    if (hd <= 0 || dv <= 0 || hd % 8 != 0 || dv % 8 != 0 || widest > 128) return 0;
    return widest <= 16 ? 16 : widest <= 32 ? 32 : widest <= 64 ? 64 : 128;
}

bool supported_head_dim(int hd) { return hd == 16 || hd == 32 || hd == 64 || hd == 128; }

}  // namespace

// 1 if this kernel takes the head size, else 0 (the caller then uses the general kernel).
extern "C" int tl_attention_mma_supports(int head_dim) { return supported_head_dim(head_dim) ? 1 : 0; }

extern "C" int tl_attention_mma_plan(int n_tokens, int n_seqs, int n_heads, int n_kv_heads, int head_dim,
                                     int max_q_len, int max_kv_len, int allow_split,
                                     int* n_splits, long long* workspace_floats) {
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || !supported_head_dim(head_dim)) return TL_BAD_SIZE;
    const Plan pl = make_plan(n_seqs, n_heads, n_kv_heads, max_q_len, max_kv_len, allow_split);
    *n_splits = pl.n_splits;
    *workspace_floats = pl.n_splits > 1 ? (long long)n_tokens * n_heads * pl.n_splits * (head_dim + 2) : 0;
    return TL_OK;
}

// Same arguments as tl_paged_attention, bfloat16 only.
extern "C" int tl_paged_attention_mma(const void* q, const void* k_pages, const void* v_pages, void* out,
                                      const int* block_table, int table_stride, const int* q_start,
                                      const int* kv_len, float* workspace, int n_tokens, int n_seqs,
                                      int n_heads, int n_kv_heads, int head_dim, int page_size, int max_q_len,
                                      int max_kv_len, int window, float scale, int allow_split, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return TL_OK;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || page_size <= 0) return TL_BAD_SIZE;
    if (!supported_head_dim(head_dim) || max_q_len <= 0 || max_kv_len <= 0) return TL_BAD_SIZE;
    if (!aligned16(q) || !aligned16(k_pages) || !aligned16(v_pages) || !aligned16(out)) return TL_BAD_ALIGN;
    const Plan pl = make_plan(n_seqs, n_heads, n_kv_heads, max_q_len, max_kv_len, allow_split);
    if (pl.n_splits > 1 && workspace == nullptr) return TL_BAD_SIZE;
    if (n_seqs > 65535 || (long long)n_kv_heads * pl.n_gchunks > 65535) return TL_BAD_SIZE;

    MmaParams p;
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.out = (__nv_bfloat16*)out;
    p.block_table = block_table; p.q_start = q_start; p.kv_len = kv_len; p.table_stride = table_stride;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
    p.page_shift = -1;
    for (int sh = 0; sh < 31; ++sh)
        if ((1 << sh) == page_size) p.page_shift = sh;
    p.group = n_heads / n_kv_heads; p.ng = pl.ng; p.n_gchunks = pl.n_gchunks; p.tpw = pl.tpw;
    p.window = window > 0 ? window : 0;
    p.n_splits = pl.n_splits;
    p.scale_log2 = scale * LOG2E;
    p.part_o = workspace;
    p.part_ml = workspace ? workspace + (size_t)n_tokens * n_heads * pl.n_splits * head_dim : nullptr;
    p.hd = p.dv = head_dim; p.shared_kv = 0; p.keep_first = 0; p.rel = nullptr; p.bucket = nullptr; p.n_bucket = 0; p.n_v_heads = n_kv_heads; p.out_f32 = 0;
    p.gate = nullptr; p.gate_mode = 0; p.bias_cols = 0; p.cap_log2 = 0.f; p.scale_over_cap = 0.f; p.sinks = nullptr;

    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(pl.n_q_tiles * pl.n_splits, n_kv_heads * pl.n_gchunks, n_seqs);
    int rc;
    switch (head_dim) {
        case 16: rc = launch_mode<16>(p, grid, pl.key_split, s); break;
        case 32: rc = launch_mode<32>(p, grid, pl.key_split, s); break;
        case 64: rc = launch_mode<64>(p, grid, pl.key_split, s); break;
        default: rc = launch_mode<128>(p, grid, pl.key_split, s); break;
    }
    if (rc != TL_OK) return rc;
    if (pl.n_splits > 1) {
        merge_partials_kernel<<<dim3((unsigned)n_tokens * (unsigned)n_heads), dim3(head_dim >= 128 ? 128u : 64u), 0, s>>>(
            p.part_o, p.part_ml, p.out, pl.n_splits, head_dim);
        TL_LAUNCH_CHECK();
    }
    return TL_OK;
}

// ---- the extended form (see the top of this file).  Options as for the general kernel's
// tl_paged_attention_ex; the struct is the same.
struct TlAttentionOptions {
    int v_head_dim;
    int keep_first;
    const float* rel;       // [rows, n_heads]
    const int* bucket;      // [n_bucket]
    int n_bucket;
    const void* gate;       // bfloat16
    int gate_mode;          // 0: none, 1: [tokens, n_heads], 2: [tokens, n_heads * v_head_dim]
    int n_v_heads;          // 0: as n_kv_heads; else it divides n_kv_heads, and v_pages has so many heads
    int out_f32;            // 1: out is float32
    float softcap;          // c > 0: the scaled score s becomes c * tanh(s / c); not together with rel
    const float* sinks;     // [n_heads] or null: exp(sinks[h]) joins the softmax's denominator
    int v_stride;           // 0, or head_dim with v_pages == k_pages: a value is the first v_head_dim coordinates of a key
};

// 1 if the extended form takes keys of head_dim and values of v_head_dim elements, else 0.
extern "C" int tl_attention_mma_ex_supports(int head_dim, int v_head_dim) { return ext_size(head_dim, v_head_dim) ? 1 : 0; }

extern "C" int tl_attention_mma_plan_ex(int n_tokens, int n_seqs, int n_heads, int n_kv_heads, int head_dim, int v_head_dim,
                                        int max_q_len, int max_kv_len, int window, int keep_first, int allow_split,
                                        int* n_splits, long long* workspace_floats) {
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || !ext_size(head_dim, v_head_dim)) return TL_BAD_SIZE;
    const Plan pl = make_plan(n_seqs, n_heads, n_kv_heads, max_q_len, max_kv_len, allow_split, window, keep_first);
    *n_splits = pl.n_splits;
    *workspace_floats = pl.n_splits > 1 ? (long long)n_tokens * n_heads * pl.n_splits * (v_head_dim + 2) : 0;
    return TL_OK;
}

// q: [n_tokens, n_heads, head_dim]; out: [n_tokens, n_heads, v_head_dim]; v_pages may be k_pages itself
// (then a value is the first v_head_dim coordinates of a stored key).  bfloat16 only.
extern "C" int tl_paged_attention_mma_ex(const void* q, const void* k_pages, const void* v_pages, void* out,
                                         const int* block_table, int table_stride, const int* q_start,
                                         const int* kv_len, float* workspace, int n_tokens, int n_seqs,
                                         int n_heads, int n_kv_heads, int head_dim, int page_size, int max_q_len,
                                         int max_kv_len, int window, float scale, int allow_split,
                                         const TlAttentionOptions* opt, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return TL_OK;
    if (opt == nullptr) return TL_BAD_SIZE;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || page_size <= 0) return TL_BAD_SIZE;
    const TlAttentionOptions o = *opt;
    const int dv = o.v_head_dim > 0 ? o.v_head_dim : head_dim;
    const int size = ext_size(head_dim, dv);
    if (!size || max_q_len <= 0 || max_kv_len <= 0) return TL_BAD_SIZE;
    if (window <= 0) window = 0;
    if (o.keep_first < 0 || (o.keep_first > 0 && window == 0)) return TL_BAD_SIZE;
    if (o.rel != nullptr && (o.bucket == nullptr || o.n_bucket <= 0)) return TL_BAD_SIZE;
    if (o.gate_mode < 0 || o.gate_mode > 2 || (o.gate_mode != 0 && o.gate == nullptr)) return TL_BAD_SIZE;
    if (v_pages == k_pages && dv > head_dim) return TL_BAD_SIZE;
    if (o.v_stride != 0 && !(v_pages == k_pages && o.v_stride == head_dim)) return TL_BAD_SIZE;
    if (o.softcap < 0.f || (o.softcap > 0.f && o.rel != nullptr)) return TL_BAD_SIZE;
    const int n_v_heads = o.n_v_heads > 0 ? o.n_v_heads : n_kv_heads;
    if (n_kv_heads % n_v_heads != 0 || (n_v_heads != n_kv_heads && v_pages == k_pages)) return TL_BAD_SIZE;
    if (!aligned16(q) || !aligned16(k_pages) || !aligned16(v_pages) || !aligned16(out)) return TL_BAD_ALIGN;
    const Plan pl = make_plan(n_seqs, n_heads, n_kv_heads, max_q_len, max_kv_len, allow_split, window, o.keep_first);
    if (pl.n_splits > 1 && workspace == nullptr) return TL_BAD_SIZE;
    if (n_seqs > 65535 || (long long)n_kv_heads * pl.n_gchunks > 65535) return TL_BAD_SIZE;

    MmaParams p;
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.out = (__nv_bfloat16*)out;
    p.block_table = block_table; p.q_start = q_start; p.kv_len = kv_len; p.table_stride = table_stride;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
    p.page_shift = -1;
    for (int sh = 0; sh < 31; ++sh)
        if ((1 << sh) == page_size) p.page_shift = sh;
    p.group = n_heads / n_kv_heads; p.ng = pl.ng; p.n_gchunks = pl.n_gchunks; p.tpw = pl.tpw;
    p.window = window;
    p.n_splits = pl.n_splits;
    p.scale_log2 = scale * LOG2E;
    p.part_o = workspace;
    p.part_ml = workspace ? workspace + (size_t)n_tokens * n_heads * pl.n_splits * dv : nullptr;
    p.hd = head_dim; p.dv = dv; p.shared_kv = v_pages == k_pages ? 1 : 0;
    p.keep_first = o.keep_first; p.rel = o.rel; p.bucket = o.bucket; p.n_bucket = o.n_bucket;
    p.gate = (const __nv_bfloat16*)o.gate; p.gate_mode = o.gate_mode;
    p.n_v_heads = n_v_heads; p.out_f32 = o.out_f32 ? 1 : 0;
    p.cap_log2 = o.softcap > 0.f ? o.softcap * LOG2E : 0.f;
    p.scale_over_cap = o.softcap > 0.f ? scale / o.softcap : 0.f;
    p.sinks = o.sinks;
    // distances a row-split CTA meets inside its window (all of them when there is no window), as far as
    // 20 KB of shared memory hold them for the heads of a tile
    p.bias_cols = 0;
    if (o.rel != nullptr && !pl.key_split) {
        long long cols = window > 0 ? (long long)window + pl.tpw * NW : max_kv_len;
        if (cols > o.n_bucket) cols = o.n_bucket;
        if (cols > 5120 / pl.ng) cols = 5120 / pl.ng;
        p.bias_cols = (int)cols;
    }

    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(pl.n_q_tiles * pl.n_splits, n_kv_heads * pl.n_gchunks, n_seqs);
    int rc;
    switch (size) {
        case 16: rc = launch_mode_ext<16>(p, grid, pl.key_split, s); break;
        case 32: rc = launch_mode_ext<32>(p, grid, pl.key_split, s); break;
        case 64: rc = launch_mode_ext<64>(p, grid, pl.key_split, s); break;
        default: rc = launch_mode_ext<128>(p, grid, pl.key_split, s); break;
    }
    if (rc != TL_OK) return rc;
    if (pl.n_splits > 1) {
        merge_partials_kernel<<<dim3((unsigned)n_tokens * (unsigned)n_heads), dim3(dv >= 128 ? 128u : 64u), 0, s>>>(
            p.part_o, p.part_ml, p.out, pl.n_splits, dv, p.gate, p.gate_mode, p.out_f32, p.sinks, n_heads);
        TL_LAUNCH_CHECK();
    }
    return TL_OK;
}
