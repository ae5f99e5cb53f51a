// Attention over a sliding window of tokens plus one pooled key and value per block of P tokens
// that lies wholly before the window, with sigmoid weights that are not normalised over the keys.
//
// A query at position p sees token j if 0 <= p - j < window, and pooled block e (the tokens
// e P .. e P + P - 1) if e P + P - 1 <= p - window.  The weight of a visible key is
// sigmoid(q . k * scale + bias[head]); out = sum over the visible keys of weight * value, times
// sigmoid(gate) per output element where a gate is given.  Because nothing is normalised the keys
// can be cut into ranges whose results simply add.
//
// Storage: token keys and values in the paged cache ([pages][kv heads][64][head size], the
// cache's dtype); the pooled ones in a second paged store of 32-bit values whose "token" e is block
// e (64 blocks a page), filled by pool_blocks as soon as a block's last token is cached: the
// mean, summed in token order, of the keys and values as the cache holds them.
//
// Kernels: qk_norm_append (root-mean-square norm over the WHOLE query projection and the whole key
// projection of a token, with weights; queries to their buffer, keys and values to the cache),
// pool_blocks, attention_pool (AP_TQ query tokens of a sequence x one head x one key range per
// block; scores, weights and sums in 32-bit FP32-pipe code; serves prompts and single tokens, both
// precisions), pool_combine (adds the key ranges, applies the gate).
#include "api.h"
#include "common.cuh"

#define AP_THREADS 128
#define AP_TQ 16            // query tokens a block serves
#define AP_TK 32            // keys staged at a time
#define AP_MAX_DIM 256      // head sizes up to this (keys and values)

// ------------------------------------------------------------------------------------------------ qk_norm_append
template <typename TQ, typename TC>
__global__ void __launch_bounds__(256)
qk_norm_append_kernel(const float* __restrict__ proj, long long ldp, const float* __restrict__ qw, const float* __restrict__ kw,
                      float eps, TQ* __restrict__ q_out, long long ldq, TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                      const int* __restrict__ page_table, int pt_width, const int* __restrict__ tok_seq,
                      const int* __restrict__ positions, int H, int G, int d, int dv, int n_pages, int append, int* status) {
    pdl_trigger();
    pdl_wait();
    proj = pdl_fresh(proj);
    __shared__ float scratch[33];
    const int t = blockIdx.x, tid = threadIdx.x;
    const int nq = H * d, nk = G * d, nv = G * dv;
    const float* pq = proj + (size_t)t * ldp;
    const float* pk = pq + nq;
    const float* pv = pk + nk;
    float rq = 1.0f, rk = 1.0f;
    if (qw != nullptr) {
        float ss = 0.0f;
        for (int i = tid; i < nq; i += 256) ss = fmaf(pq[i], pq[i], ss);
        ss = block_sum(ss, scratch);
        rq = 1.0f / sqrtf(ss / (float)nq + eps);
    }
    if (kw != nullptr && append) {
        float ss = 0.0f;
        for (int i = tid; i < nk; i += 256) ss = fmaf(pk[i], pk[i], ss);
        ss = block_sum(ss, scratch);
        rk = 1.0f / sqrtf(ss / (float)nk + eps);
    }
    TQ* qo = q_out + (size_t)t * ldq;
    for (int i = tid; i < nq; i += 256) qo[i] = from_f32<TQ>(qw != nullptr ? pq[i] * rq * qw[i] : pq[i]);
    if (!append) return;
    const int p = positions[t], b = tok_seq[t];
    const int lp = p / HB_PAGE_TOKENS;
    const int page = lp < pt_width ? page_table[(size_t)b * pt_width + lp] : -1;
    if (page < 0 || page >= n_pages) {          // the host's bookkeeping is at fault: note it, write nothing
        if (tid == 0) hb_note(status, HB_STATUS_PAGE, 1 + b);
        return;
    }
    for (int i = tid; i < nk; i += 256) {
        const int g = i / d, c = i - g * d;
        k_cache[cache_offset(page, g, p, G, d) + c] = from_f32<TC>(kw != nullptr ? pk[i] * rk * kw[i] : pk[i]);
    }
    for (int i = tid; i < nv; i += 256) {
        const int g = i / dv, c = i - g * dv;
        v_cache[cache_offset(page, g, p, G, dv) + c] = from_f32<TC>(pv[i]);
    }
}

extern "C" int hb_qk_norm_append(const float* proj, long long ldp, const float* q_weight, const float* k_weight, float eps,
                                 void* q_out, int q_dtype, long long ldq, void* k_cache, void* v_cache, int cache_dtype,
                                 const int* page_table, int pt_width, const int* tok_seq, const int* positions, int n_tokens,
                                 int n_heads, int n_kv_heads, int head_dim, int v_dim, int n_pages, int append, int* status,
                                 void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0 && v_dim > 0 && n_pages > 0, "qk_norm_append: bad sizes");
    HB_REQUIRE(ldp >= (long long)n_heads * head_dim + (long long)n_kv_heads * (head_dim + v_dim), "qk_norm_append: projection rows are too short");
    cudaStream_t s = (cudaStream_t)stream;
#define HB_QKN(TQ, TC)                                                                                                              \
    hb_launch(qk_norm_append_kernel<TQ, TC>, dim3(n_tokens), dim3(256), 0, s, proj, ldp, q_weight, k_weight, eps, (TQ*)q_out, ldq, \
              (TC*)k_cache, (TC*)v_cache, page_table, pt_width, tok_seq, positions, n_heads, n_kv_heads, head_dim, v_dim, n_pages, \
              append, status)
    if (q_dtype == HB_BF16 && cache_dtype == HB_BF16) HB_QKN(bf16, bf16);
    else if (q_dtype == HB_F32 && cache_dtype == HB_F32) HB_QKN(float, float);
    else return hb_fail("qk_norm_append: unsupported dtypes q %d cache %d", q_dtype, cache_dtype);
#undef HB_QKN
    return hb_check_launch("qk_norm_append");
}

// ------------------------------------------------------------------------------------------------ pool_blocks
// Blocks whose last token this step cached: e from pos0 / P to len / P - 1 per sequence.
template <typename TC>
__global__ void __launch_bounds__(128)
pool_blocks_kernel(const TC* __restrict__ k_cache, const TC* __restrict__ v_cache, float* __restrict__ pk_cache,
                   float* __restrict__ pv_cache, const int* __restrict__ pt_tok, const int* __restrict__ pt_pool, int pt_width,
                   const int* __restrict__ seq_pos0, const int* __restrict__ seq_len, int P, int G, int d, int dv, int n_pages_tok,
                   int n_pages_pool, int* status) {
    pdl_trigger();
    pdl_wait();
    k_cache = pdl_fresh(k_cache);
    v_cache = pdl_fresh(v_cache);
    const int b = blockIdx.y;
    const int e = seq_pos0[b] / P + blockIdx.x;
    if (e >= seq_len[b] / P) return;
    const int lpp = e / HB_PAGE_TOKENS;
    const int ppage = lpp < pt_width ? pt_pool[(size_t)b * pt_width + lpp] : -1;
    if (ppage < 0 || ppage >= n_pages_pool) {
        if (threadIdx.x == 0) hb_note(status, HB_STATUS_PAGE, 1 + b);
        return;
    }
    const int per = d + dv, g = blockIdx.z;
    for (int c = threadIdx.x; c < per; c += 128) {
        float sum = 0.0f;
        bool ok = true;
#pragma unroll 4
        for (int j = 0; j < P; j++) {
            const int pos = e * P + j;
            const int lp = pos / HB_PAGE_TOKENS;
            const int page = lp < pt_width ? pt_tok[(size_t)b * pt_width + lp] : -1;
            if (page < 0 || page >= n_pages_tok) {
                ok = false;
                continue;
            }
            sum += c < d ? to_f32(k_cache[cache_offset(page, g, pos, G, d) + c]) : to_f32(v_cache[cache_offset(page, g, pos, G, dv) + (c - d)]);
        }
        if (!ok) hb_note(status, HB_STATUS_PAGE, 1 + b);
        const float mean = sum / (float)P;
        if (c < d) pk_cache[cache_offset(ppage, g, e, G, d) + c] = mean;
        else pv_cache[cache_offset(ppage, g, e, G, dv) + (c - d)] = mean;
    }
}

extern "C" int hb_pool_blocks(const void* k_cache, const void* v_cache, int cache_dtype, float* pk_cache, float* pv_cache,
                              const int* pt_tok, const int* pt_pool, int pt_width, const int* seq_pos0, const int* seq_len,
                              int n_seqs, int max_new, int pool, int n_kv_heads, int head_dim, int v_dim, int n_pages_tok,
                              int n_pages_pool, int* status, void* stream) {
    if (n_seqs == 0) return 0;
    HB_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && max_new >= 1 && pool >= 1 && n_kv_heads > 0 && head_dim > 0 && v_dim > 0, "pool_blocks: bad sizes");
    HB_REQUIRE(n_kv_heads <= 65535, "pool_blocks: too many key/value heads");
    dim3 grid(max_new / pool + 1, n_seqs, n_kv_heads);
    cudaStream_t s = (cudaStream_t)stream;
    if (cache_dtype == HB_BF16)
        hb_launch(pool_blocks_kernel<bf16>, dim3(grid), dim3(128), 0, s, (const bf16*)k_cache, (const bf16*)v_cache, pk_cache, pv_cache, pt_tok,
                  pt_pool, pt_width, seq_pos0, seq_len, pool, n_kv_heads, head_dim, v_dim, n_pages_tok, n_pages_pool, status);
    else if (cache_dtype == HB_F32)
        hb_launch(pool_blocks_kernel<float>, dim3(grid), dim3(128), 0, s, (const float*)k_cache, (const float*)v_cache, pk_cache, pv_cache, pt_tok,
                  pt_pool, pt_width, seq_pos0, seq_len, pool, n_kv_heads, head_dim, v_dim, n_pages_tok, n_pages_pool, status);
    else return hb_fail("pool_blocks: unsupported cache dtype %d", cache_dtype);
    return hb_check_launch("pool_blocks");
}

// ------------------------------------------------------------------------------------------------ attention_pool
// Shared memory (floats): queries [AP_TQ][d], keys [AP_TK][d + 1], values [AP_TK][dv], weights [AP_TQ][AP_TK].
static size_t ap_smem_bytes(int d, int dv) { return sizeof(float) * ((size_t)AP_TQ * d + (size_t)AP_TK * (d + 1) + (size_t)AP_TK * dv + AP_TQ * AP_TK); }

// Stages up to AP_TK rows of `width` values (row kk at cache row k0 + kk of its page, kv head g) into shared memory as 32-bit
// values, row stride ld_dst; rows beyond nk or without a page become zeros.  With rows of whole 16-byte chunks every thread
// has four chunk loads in flight at a time; other widths go element by element.
template <typename T>
__device__ __forceinline__ void ap_stage(const T* __restrict__ cache, const int* pages, int nk, int k0, int g, int G, int width,
                                         float* dst, int ld_dst, int tid) {
    constexpr int EPC = 16 / (int)sizeof(T);
    if (width % EPC == 0) {
        const int cpr = width / EPC, total = AP_TK * cpr;
        for (int base = 0; base < total; base += AP_THREADS * 4) {
            uint4 raw[4];
            int at[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = base + u * AP_THREADS + tid;
                raw[u] = make_uint4(0u, 0u, 0u, 0u);
                at[u] = -1;
                if (i < total) {
                    const int kk = i / cpr, ch = i - kk * cpr;
                    at[u] = kk * ld_dst + ch * EPC;
                    if (kk < nk && pages[kk] >= 0)
                        raw[u] = *reinterpret_cast<const uint4*>(cache + cache_offset(pages[kk], g, k0 + kk, G, width) + ch * EPC);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (at[u] < 0) continue;
                const T* v = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
                for (int e = 0; e < EPC; e++) dst[at[u] + e] = to_f32(v[e]);
            }
        }
        return;
    }
    for (int i = tid; i < AP_TK * width; i += AP_THREADS) {
        const int kk = i / width, c = i - kk * width;
        float v = 0.0f;
        if (kk < nk && pages[kk] >= 0) v = to_f32(cache[cache_offset(pages[kk], g, k0 + kk, G, width) + c]);
        dst[kk * ld_dst + c] = v;
    }
}

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(AP_THREADS)
attention_pool_kernel(const TQ* __restrict__ q, long long ldq, const TC* __restrict__ k_cache, const TC* __restrict__ v_cache,
                      const float* __restrict__ pk_cache, const float* __restrict__ pv_cache, const int* __restrict__ pt_tok,
                      const int* __restrict__ pt_pool, int pt_width, const int* __restrict__ seq_start,
                      const int* __restrict__ seq_pos0, int n_seqs, const float* __restrict__ head_bias,
                      const float* __restrict__ gate, long long ldg, TO* __restrict__ out, long long ldo, float* __restrict__ partial,
                      int n_tokens, int H, int G, int d, int dv, float scale, int window, int P, int n_pages_tok, int n_pages_pool,
                      int splits, int part, int grouped, int* status) {
    pdl_trigger();
    extern __shared__ float ap_smem[];
    float* Qs = ap_smem;
    float* Ks = Qs + AP_TQ * d;
    float* Vs = Ks + AP_TK * (d + 1);
    float* Ps = Vs + AP_TK * dv;
    __shared__ int pages[AP_TK];
    // grouped (steps of one token per sequence): a block serves the query heads of ONE key/value head as its rows, so the
    // group's keys and values are staged once instead of once per head; else its rows are up to AP_TQ tokens of one head
    const int R = H / G;
    const int tid = threadIdx.x, split = blockIdx.z;
    const int g = grouped ? (int)blockIdx.y : (int)blockIdx.y / R;
    const int h0 = grouped ? g * R : (int)blockIdx.y;          // the head of row 0
    // which sequence and which of its query tiles (the step's metadata was copied before the step's first kernel)
    int b = 0, tile = blockIdx.x;
    for (; b < n_seqs; b++) {
        const int tiles = (seq_start[b + 1] - seq_start[b] + AP_TQ - 1) / AP_TQ;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (b >= n_seqs) return;
    const int t0 = seq_start[b] + tile * AP_TQ;
    const int nq = grouped ? R : min(AP_TQ, seq_start[b + 1] - t0);
    const int p_first = seq_pos0[b] + tile * AP_TQ, p_last = grouped ? p_first : p_first + nq - 1;
    pdl_wait();
    q = pdl_fresh(q);
    k_cache = pdl_fresh(k_cache);
    v_cache = pdl_fresh(v_cache);
    pk_cache = pdl_fresh(pk_cache);
    pv_cache = pdl_fresh(pv_cache);
    gate = pdl_fresh(gate);
    for (int i = tid; i < AP_TQ * d; i += AP_THREADS) {
        const int qi = i / d, c = i - qi * d;
        Qs[i] = qi < nq ? to_f32(q[(size_t)(grouped ? t0 : t0 + qi) * ldq + (size_t)(grouped ? h0 + qi : h0) * d + c]) : 0.0f;
    }
    // the keys of this tile, as one list: pooled blocks 0 .. nb - 1, then tokens j_lo .. p_last, in tiles of AP_TK
    const int nb = (P > 0 && window > 0 && p_last - window + 1 >= P) ? (p_last - window + 1) / P : 0;
    const int j_lo = window > 0 ? max(0, p_first - window + 1) : 0;
    const int pool_tiles = (nb + AP_TK - 1) / AP_TK;
    const int tok_tiles = part == 1 ? 0 : (p_last - j_lo + 1 + AP_TK - 1) / AP_TK;      // part 1: the pooled blocks alone
    const int all_tiles = pool_tiles + tok_tiles;
    const int per_split = (all_tiles + splits - 1) / splits;
    const int tile_lo = split * per_split, tile_hi = min(all_tiles, tile_lo + per_split);

    const int qg = tid >> 5, lane = tid & 31;          // PV: queries qg * 4 .. + 3, columns lane + 32 m
    float acc[4][AP_MAX_DIM / 32];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int m = 0; m < AP_MAX_DIM / 32; m++) acc[a][m] = 0.0f;

    for (int kt = tile_lo; kt < tile_hi; kt++) {
        const bool pooled = kt < pool_tiles;
        const int k0 = pooled ? kt * AP_TK : j_lo + (kt - pool_tiles) * AP_TK;      // first key of the tile (block or position)
        const int k_end = pooled ? nb : p_last + 1;
        const int nk = min(AP_TK, k_end - k0);
        __syncthreads();                               // the last tile's weights and values have been read
        if (tid < AP_TK) {
            int page = -1;
            if (tid < nk) {
                const int lp = (k0 + tid) / HB_PAGE_TOKENS;
                page = lp < pt_width ? (pooled ? pt_pool : pt_tok)[(size_t)b * pt_width + lp] : -1;
                if (page >= (pooled ? n_pages_pool : n_pages_tok)) page = -1;
                if (page < 0) {
                    // a page that some query of the tile may need is missing; tokens before the tile's first window
                    // edge are never staged (j_lo), so every staged key is visible to at least the last query
                    hb_note(status, HB_STATUS_PAGE, 1 + b);
                }
            }
            pages[tid] = page;
        }
        __syncthreads();
        if (pooled) {
            ap_stage<float>(pk_cache, pages, nk, k0, g, G, d, Ks, d + 1, tid);
            ap_stage<float>(pv_cache, pages, nk, k0, g, G, dv, Vs, dv, tid);
        } else {
            ap_stage<TC>(k_cache, pages, nk, k0, g, G, d, Ks, d + 1, tid);
            ap_stage<TC>(v_cache, pages, nk, k0, g, G, dv, Vs, dv, tid);
        }
        __syncthreads();
        // weights: key `lane`, queries qg, qg + 4, qg + 8, qg + 12
#pragma unroll
        for (int a = 0; a < AP_TQ / 4; a++) {
            const int qi = qg + 4 * a;
            float wgt = 0.0f;
            if (qi < nq && lane < nk && pages[lane] >= 0) {
                const int p = grouped ? p_first : p_first + qi, key = k0 + lane;
                const bool seen = pooled ? (key * P + P - 1 <= p - window) : (key <= p && (window <= 0 || p - key < window));
                if (seen) {
                    const float* qr = Qs + qi * d;
                    const float* kr = Ks + lane * (d + 1);
                    float dot = 0.0f;
                    for (int c = 0; c < d; c++) dot = fmaf(qr[c], kr[c], dot);
                    const float bias = head_bias != nullptr ? head_bias[grouped ? h0 + qi : h0] : 0.0f;
                    wgt = 1.0f / (1.0f + expf(-(dot * scale + bias)));
                }
            }
            Ps[qi * AP_TK + lane] = wgt;
        }
        __syncthreads();
        // sums: queries qg * 4 + a, columns lane + 32 m
        for (int kk = 0; kk < nk; kk++) {
            float pw[4];
#pragma unroll
            for (int a = 0; a < 4; a++) pw[a] = Ps[(qg * 4 + a) * AP_TK + kk];
            if (pw[0] == 0.0f && pw[1] == 0.0f && pw[2] == 0.0f && pw[3] == 0.0f) continue;
#pragma unroll
            for (int m = 0; m < AP_MAX_DIM / 32; m++) {
                const int c = lane + 32 * m;
                if (c < dv) {
                    const float v = Vs[kk * dv + c];
#pragma unroll
                    for (int a = 0; a < 4; a++) acc[a][m] = fmaf(pw[a], v, acc[a][m]);
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < 4; a++) {
        const int qi = qg * 4 + a;
        if (qi >= nq) continue;
        const int t = grouped ? t0 : t0 + qi;
#pragma unroll
        for (int m = 0; m < AP_MAX_DIM / 32; m++) {
            const int c = lane + 32 * m;
            if (c >= dv) continue;
            const size_t col = (size_t)(grouped ? h0 + qi : h0) * dv + c;
            if (splits == 1 && part == 0) {
                float v = acc[a][m];
                if (gate != nullptr) v *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + col]));
                out[(size_t)t * ldo + col] = from_f32<TO>(v);
            } else {
                partial[((size_t)split * n_tokens + t) * ((size_t)H * dv) + col] = acc[a][m];
            }
        }
    }
}

template <typename TO>
__global__ void __launch_bounds__(256)
pool_combine_kernel(const float* __restrict__ partial, const float* __restrict__ gate, long long ldg, TO* __restrict__ out,
                    long long ldo, int n_tokens, int width, int splits) {
    pdl_trigger();
    pdl_wait();
    partial = pdl_fresh(partial);
    gate = pdl_fresh(gate);
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += 256) {
        float v = 0.0f;
        for (int s = 0; s < splits; s++) v += partial[((size_t)s * n_tokens + t) * width + c];
        if (gate != nullptr) v *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + c]));
        out[(size_t)t * ldo + c] = from_f32<TO>(v);
    }
}

extern "C" int hb_attention_pool_supported(int head_dim, int v_dim) {
    return head_dim >= 1 && head_dim <= AP_MAX_DIM && v_dim >= 1 && v_dim <= AP_MAX_DIM;
}

extern "C" int hb_attention_pool(const void* q, int q_dtype, long long ldq, const void* k_cache, const void* v_cache, int cache_dtype,
                                 const float* pk_cache, const float* pv_cache, const int* pt_tok, const int* pt_pool, int pt_width,
                                 const int* seq_start, const int* seq_pos0, int n_seqs, int q_tiles, const float* head_bias,
                                 const float* gate, long long ldg, void* out, int out_dtype, long long ldo, float* partial,
                                 int n_tokens, int n_heads, int n_kv_heads, int head_dim, int v_dim, float scale, int window,
                                 int pool, int n_pages_tok, int n_pages_pool, int splits, int part, int grouped, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_seqs > 0 && q_tiles > 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attention_pool: bad sizes");
    HB_REQUIRE(hb_attention_pool_supported(head_dim, v_dim), "attention_pool: head sizes %d / %d (up to %d are built)", head_dim, v_dim, AP_MAX_DIM);
    HB_REQUIRE(n_heads <= 65535 && splits >= 1 && splits <= 65535, "attention_pool: too many heads or key ranges");
    HB_REQUIRE(pool == 0 || (pk_cache != nullptr && pv_cache != nullptr && pt_pool != nullptr && window > 0), "attention_pool: pooled blocks need their store and a window");
    HB_REQUIRE((splits == 1 && part == 0) || partial != nullptr, "attention_pool: key ranges need a buffer for their sums");
    HB_REQUIRE(part == 0 || (part == 1 && splits == 1 && pool > 0), "attention_pool: the pooled blocks alone are one range");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = ap_smem_bytes(head_dim, v_dim);
    HB_REQUIRE(!grouped || (n_heads / n_kv_heads <= AP_TQ && q_tiles == n_seqs && n_tokens == n_seqs), "attention_pool: rows by key/value head need one token per sequence and groups of up to %d heads", AP_TQ);
    dim3 grid(q_tiles, grouped ? n_kv_heads : n_heads, splits);
#define HB_AP(TQ, TC, TO)                                                                                                                  \
    do {                                                                                                                                   \
        static bool done[HB_MAX_DEVICES] = {};                                                                                             \
        const int slot = hb_device_slot();                                                                                                 \
        if (!done[slot]) {                                                                                                                 \
            cudaError_t e = cudaFuncSetAttribute(attention_pool_kernel<TQ, TC, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                                 (int)ap_smem_bytes(AP_MAX_DIM, AP_MAX_DIM));                                              \
            if (e != cudaSuccess) return hb_fail("attention_pool: shared memory: %s", cudaGetErrorString(e));                              \
            done[slot] = true;                                                                                                             \
        }                                                                                                                                  \
        hb_launch(attention_pool_kernel<TQ, TC, TO>, dim3(grid), dim3(AP_THREADS), smem, s, (const TQ*)q, ldq, (const TC*)k_cache,         \
                  (const TC*)v_cache, pk_cache, pv_cache, pt_tok, pt_pool, pt_width, seq_start, seq_pos0, n_seqs, head_bias, gate, ldg,    \
                  (TO*)out, ldo, partial, n_tokens, n_heads, n_kv_heads, head_dim, v_dim, scale, window, pool, n_pages_tok, n_pages_pool,  \
                  splits, part, grouped, status);                                                                                          \
    } while (0)
    if (q_dtype == HB_BF16 && cache_dtype == HB_BF16 && out_dtype == HB_BF16) HB_AP(bf16, bf16, bf16);
    else if (q_dtype == HB_F32 && cache_dtype == HB_F32 && out_dtype == HB_F32) HB_AP(float, float, float);
    else return hb_fail("attention_pool: unsupported dtypes q %d cache %d out %d", q_dtype, cache_dtype, out_dtype);
#undef HB_AP
    if (hb_check_launch("attention_pool")) return 1;
    if (splits > 1) {
        const int width = n_heads * v_dim;
        if (out_dtype == HB_BF16)
            hb_launch(pool_combine_kernel<bf16>, dim3(n_tokens), dim3(256), 0, s, (const float*)partial, gate, ldg, (bf16*)out, ldo, n_tokens, width, splits);
        else
            hb_launch(pool_combine_kernel<float>, dim3(n_tokens), dim3(256), 0, s, (const float*)partial, gate, ldg, (float*)out, ldo, n_tokens, width, splits);
        return hb_check_launch("pool_combine");
    }
    return 0;
}
