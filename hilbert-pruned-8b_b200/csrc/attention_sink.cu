// Attention with a sliding window that keeps the sequence's first tokens, key and value heads
// of different sizes, and softmax weights that are mixed between the heads.
//
// Three kernels:
//  * qkv_prepare: per token, adds the projections' biases, turns the queries and keys by the
//    step's rotation table, divides each head by its root mean square (optional), writes the
//    queries to their buffer and the keys and values into the paged cache.  Values can be mixed
//    with the values an earlier layer made for the same token: v <- (1 - l) v + l v_first.
//  * attention_sink: one block per (token, query head).  Query at position p sees key s if
//    s <= p and (p - s < window or s < keep_first); window 0 means every earlier key.  Softmax
//    in float32 with a running maximum.  With all_values the weights of a head are applied to
//    the values of EVERY key/value head (the mixing of weights between heads needs them), else
//    to the head's own.  The results are float32.
//  * head_mix: out[t, h] = sum_g mix[h, g] * partial[t, g, kv(h)]: a mix of the heads' softmax
//    weights, applied to the values, is the same mix of their weighted value sums.
#include "api.h"
#include "common.cuh"

#define QP_THREADS 128
#define QP_MAX_HD 512

// blocks (token, slot): slots 0..nh-1 query heads, nh..nh+nkv-1 key heads, then nkv value heads
template <typename TP, typename TQ, typename TC>
__global__ void __launch_bounds__(QP_THREADS)
qkv_prepare_kernel(const TP* __restrict__ proj, long long ldp, const float* __restrict__ bias, const float2* __restrict__ table,
                   int rot, int nh, int nkv, int hd, int vd, int unit_norm, float eps, TQ* __restrict__ q_out, long long ldq,
                   TC* __restrict__ k_cache, TC* __restrict__ v_cache, const int* __restrict__ page_table, int pt_width,
                   const int* __restrict__ tok_seq, const int* __restrict__ positions, int n_pages, int append,
                   const float* __restrict__ v_lambda, float* __restrict__ v_first, int v_mode, int* status) {
    pdl_trigger();
    __shared__ float xs[QP_MAX_HD];
    __shared__ float scratch[33];
    const int t = blockIdx.x, slot = blockIdx.y, tid = threadIdx.x;
    const int pos = positions[t];
    const bool is_q = slot < nh, is_k = !is_q && slot < nh + nkv;
    int page = -1;
    if (!is_q) {
        const int lp = pos / HB_PAGE_TOKENS;
        page = lp < pt_width ? page_table[(size_t)tok_seq[t] * pt_width + lp] : -1;
        if (page < 0 || page >= n_pages) {
            if (append && tid == 0) hb_note(status, HB_STATUS_PAGE, 1 + tok_seq[t]);
            page = -1;
        }
    }
    pdl_wait();
    proj = pdl_fresh(proj);
    table = pdl_fresh(table);
    if (is_q || is_k) {
        const int col0 = is_q ? slot * hd : nh * hd + (slot - nh) * hd;
        const TP* row = proj + (size_t)t * ldp + col0;
        for (int d = tid; d < hd; d += QP_THREADS) xs[d] = to_f32(row[d]) + (bias ? bias[col0 + d] : 0.0f);
        __syncthreads();
        const int half = rot >> 1;
        float ss = 0.0f;
        for (int d = tid; d < hd; d += QP_THREADS) {
            float y = xs[d];
            if (d < rot) {
                const int i = d < half ? d : d - half;
                const float2 cs = table[(size_t)t * half + i];
                float y1, y2;
                rope_pair(xs[i], xs[i + half], cs.x, cs.y, y1, y2);
                y = d < half ? y1 : y2;
            }
            ss = fmaf(y, y, ss);
        }
        // second pass with the factor (recomputes the rotation: xs still holds the inputs)
        float inv = 1.0f;
        if (unit_norm) {
            ss = block_sum(ss, scratch);
            inv = 1.0f / sqrtf(ss / (float)hd + eps);
        }
        for (int d = tid; d < hd; d += QP_THREADS) {
            float y = xs[d];
            if (d < rot) {
                const int i = d < half ? d : d - half;
                const float2 cs = table[(size_t)t * half + i];
                float y1, y2;
                rope_pair(xs[i], xs[i + half], cs.x, cs.y, y1, y2);
                y = d < half ? y1 : y2;
            }
            y *= inv;
            if (is_q) q_out[(size_t)t * ldq + col0 + d] = from_f32<TQ>(y);
            else if (append && page >= 0) k_cache[cache_offset(page, slot - nh, pos, nkv, hd) + d] = from_f32<TC>(y);
        }
    } else {
        const int g = slot - nh - nkv;
        const int col0 = (nh + nkv) * hd + g * vd;
        const TP* row = proj + (size_t)t * ldp + col0;
        const float lam = v_mode == 2 ? v_lambda[0] : 0.0f;
        float* vf = v_first ? pdl_fresh(v_first) + (size_t)t * nkv * vd + (size_t)g * vd : nullptr;
        for (int d = tid; d < vd; d += QP_THREADS) {
            float v = to_f32(row[d]) + (bias ? bias[col0 + d] : 0.0f);
            if (v_mode == 1) vf[d] = v;
            else if (v_mode == 2) v = (1.0f - lam) * v + lam * vf[d];
            if (append && page >= 0) v_cache[cache_offset(page, g, pos, nkv, vd) + d] = from_f32<TC>(v);
        }
    }
}

extern "C" int hb_qkv_prepare(const void* proj, int proj_dtype, long long ldp, const float* bias, const float* table, int rot,
                              int n_heads, int n_kv_heads, int head_dim, int v_dim, int unit_norm, float eps, void* q_out,
                              int q_dtype, long long ldq, void* k_cache, void* v_cache, int cache_dtype, const int* page_table,
                              int pt_width, const int* tok_seq, const int* positions, int n_tokens, int n_pages, int append,
                              const float* v_lambda, float* v_first, int v_mode, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0 && v_dim > 0, "qkv_prepare: bad sizes");
    HB_REQUIRE(head_dim <= QP_MAX_HD, "qkv_prepare: head size %d is larger than %d", head_dim, QP_MAX_HD);
    HB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= head_dim, "qkv_prepare: %d rotated dimensions of %d", rot, head_dim);
    HB_REQUIRE(rot == 0 || table != nullptr, "qkv_prepare: no rotation table");
    HB_REQUIRE(v_mode >= 0 && v_mode <= 2 && (v_mode == 0 || v_first != nullptr) && (v_mode != 2 || v_lambda != nullptr),
               "qkv_prepare: value mixing needs its buffers");
    HB_REQUIRE(n_heads + 2 * n_kv_heads <= 65535, "qkv_prepare: too many heads");
    const bool cache_same = (q_dtype == cache_dtype);
    HB_REQUIRE(cache_same, "qkv_prepare: queries and cache must have one dtype");
    dim3 grid(n_tokens, n_heads + (append ? 2 * n_kv_heads : 0));
    cudaStream_t s = (cudaStream_t)stream;
#define HB_QP_LAUNCH(TP, TQ)                                                                                                   \
    hb_launch(qkv_prepare_kernel<TP, TQ, TQ>, dim3(grid), dim3(QP_THREADS), 0, s, (const TP*)proj, ldp, bias, (const float2*)table, rot,  \
              n_heads, n_kv_heads, head_dim, v_dim, unit_norm, eps, (TQ*)q_out, ldq, (TQ*)k_cache, (TQ*)v_cache, page_table,       \
              pt_width, tok_seq, positions, n_pages, append, v_lambda, v_first, v_mode, status)
    if (proj_dtype == HB_F32 && q_dtype == HB_F32) HB_QP_LAUNCH(float, float);
    else if (proj_dtype == HB_F32 && q_dtype == HB_BF16) HB_QP_LAUNCH(float, bf16);
    else if (proj_dtype == HB_BF16 && q_dtype == HB_BF16) HB_QP_LAUNCH(bf16, bf16);
    else return hb_fail("qkv_prepare: unsupported dtypes %d -> %d", proj_dtype, q_dtype);
#undef HB_QP_LAUNCH
    return hb_check_launch("qkv_prepare");
}

// ---------------------------------------------------------------------------------------------
#define AS_THREADS 128
#define AS_MAX_HD 512
#define AS_MAX_ACC 16         // value columns per thread: (value heads served) * v_dim <= 128 * 16

template <typename TQ, typename TC>
__global__ void __launch_bounds__(AS_THREADS)
attention_sink_kernel(const TQ* __restrict__ q, long long ldq, const TC* __restrict__ k_cache, const TC* __restrict__ v_cache,
                      const int* __restrict__ page_table, int pt_width, const int* __restrict__ tok_seq,
                      const int* __restrict__ positions, float* __restrict__ out, int nh, int nkv, int hd, int vd, float scale,
                      int window, int keep_first, int all_values, int n_pages, int* status) {
    pdl_trigger();
    pdl_wait();
    q = pdl_fresh(q);
    k_cache = pdl_fresh(k_cache);
    v_cache = pdl_fresh(v_cache);
    __shared__ float qs[AS_MAX_HD];
    __shared__ float ps[AS_THREADS];
    __shared__ int key_of[AS_THREADS];
    __shared__ int page_of[AS_THREADS];
    __shared__ float scratch[33];
    const int t = blockIdx.x, j = blockIdx.y, tid = threadIdx.x;
    const int g = j / (nh / nkv);
    const int p = positions[t];
    const int* pt = page_table + (size_t)tok_seq[t] * pt_width;
    // the keys this query sees: [0, kept) and [lo, p]
    const int lo_w = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int kept = min(min(keep_first, lo_w), p + 1);
    const int lo = max(lo_w, kept);
    const int total = kept + (p - lo + 1);
    const TQ* qr = q + (size_t)t * ldq + (size_t)j * hd;
    for (int d = tid; d < hd; d += AS_THREADS) qs[d] = to_f32(qr[d]);
    __syncthreads();

    const int n_val = all_values ? nkv : 1;
    const int n_out = n_val * vd;
    float m = -INFINITY, l = 0.0f;
    float acc[AS_MAX_ACC];
#pragma unroll
    for (int i = 0; i < AS_MAX_ACC; i++) acc[i] = 0.0f;

    for (int v0 = 0; v0 < total; v0 += AS_THREADS) {
        const int vi = v0 + tid;
        const bool valid = vi < total;
        float sc = -INFINITY;
        int s = 0, page = -1;
        if (valid) {
            s = vi < kept ? vi : lo + (vi - kept);
            const int lp = s / HB_PAGE_TOKENS;
            page = lp < pt_width ? pt[lp] : -1;
            if (page >= n_pages) page = -1;
            if (page < 0) hb_note(status, HB_STATUS_PAGE, 1 + tok_seq[t]);
            if (page >= 0) {
                const TC* kr = k_cache + cache_offset(page, g, s, nkv, hd);
                float dot = 0.0f;
                for (int d = 0; d < hd; d++) dot = fmaf(qs[d], to_f32(kr[d]), dot);
                sc = dot * scale;
            }
        }
        key_of[tid] = s;
        page_of[tid] = page;
        const float tmax = block_max(sc, scratch);
        const float m_new = fmaxf(m, tmax);
        const float pr = (sc == -INFINITY) ? 0.0f : expf(sc - m_new);
        ps[tid] = pr;
        const float tsum = block_sum(pr, scratch);          // also orders the writes above before the reads below
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        l = l * corr + tsum;
        const int n_in_tile = min(AS_THREADS, total - v0);
#pragma unroll
        for (int i = 0; i < AS_MAX_ACC; i++) {
            const int e = tid + i * AS_THREADS;
            if (e < n_out) {
                const int c = all_values ? e / vd : g, d = all_values ? e - (e / vd) * vd : e;
                float a = acc[i] * corr;
                for (int x = 0; x < n_in_tile; x++) {
                    const float pe = ps[x];
                    if (pe != 0.0f) a = fmaf(pe, to_f32(v_cache[cache_offset(page_of[x], c, key_of[x], nkv, vd) + d]), a);
                }
                acc[i] = a;
            }
        }
        m = m_new;
        __syncthreads();
    }
    float* o = out + ((size_t)t * nh + j) * n_out;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < AS_MAX_ACC; i++) {
        const int e = tid + i * AS_THREADS;
        if (e < n_out) o[e] = acc[i] * inv;
    }
}

extern "C" int hb_attention_sink(const void* q, int q_dtype, long long ldq, const void* k_cache, const void* v_cache,
                                 int cache_dtype, const int* page_table, int pt_width, const int* tok_seq,
                                 const int* positions, float* out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                 int v_dim, float scale, int window, int keep_first, int all_values, int n_pages,
                                 int* status, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0 && v_dim > 0 && n_pages > 0, "attention: bad sizes");
    HB_REQUIRE(n_heads % n_kv_heads == 0, "attention: %d heads are no multiple of %d kv heads", n_heads, n_kv_heads);
    HB_REQUIRE(head_dim <= AS_MAX_HD, "attention: head size %d is larger than %d", head_dim, AS_MAX_HD);
    HB_REQUIRE((all_values ? n_kv_heads : 1) * v_dim <= AS_THREADS * AS_MAX_ACC,
               "attention: %d value columns per query head are more than %d", (all_values ? n_kv_heads : 1) * v_dim, AS_THREADS * AS_MAX_ACC);
    HB_REQUIRE(n_heads <= 65535 && window >= 0 && keep_first >= 0, "attention: bad head count, window or kept tokens");
    dim3 grid(n_tokens, n_heads);
    cudaStream_t s = (cudaStream_t)stream;
#define HB_AS_LAUNCH(TQ, TC)                                                                                                  \
    hb_launch(attention_sink_kernel<TQ, TC>, dim3(grid), dim3(AS_THREADS), 0, s, (const TQ*)q, ldq, (const TC*)k_cache, (const TC*)v_cache, \
              page_table, pt_width, tok_seq, positions, out, n_heads, n_kv_heads, head_dim, v_dim, scale, window, keep_first,      \
              all_values, n_pages, status)
    if (q_dtype == HB_F32 && cache_dtype == HB_F32) HB_AS_LAUNCH(float, float);
    else if (q_dtype == HB_BF16 && cache_dtype == HB_BF16) HB_AS_LAUNCH(bf16, bf16);
    else return hb_fail("attention: unsupported dtypes q %d cache %d", q_dtype, cache_dtype);
#undef HB_AS_LAUNCH
    return hb_check_launch("attention_sink");
}

// out[t, h*vd + d] = sum_g mix[h, g] * partial[t, g, c(h), d], c(h) = h / (nh / nkv) when the partial
// results hold all value heads (n_val == nkv), else partial[t, g, 0, d] is taken as it is (no mixing
// possible: mix must be null).  `ones` more columns follow the heads: a one and zeros, by which the
// product behind adds its bias as one more column of its weight.
template <typename TO>
__global__ void __launch_bounds__(256)
head_mix_kernel(const float* __restrict__ partial, const float* __restrict__ mix, TO* __restrict__ out, long long ldo, int nh,
                int nkv, int vd, int n_val, int ones) {
    pdl_trigger();
    pdl_wait();
    partial = pdl_fresh(partial);
    const int t = blockIdx.x;
    const float* pr = partial + (size_t)t * nh * n_val * vd;
    TO* o = out + (size_t)t * ldo;
    const int group = nh / nkv;
    for (int e = threadIdx.x; e < nh * vd; e += blockDim.x) {
        const int h = e / vd, d = e - h * vd;
        float a;
        if (mix != nullptr) {
            const int c = n_val == nkv ? h / group : 0;
            a = 0.0f;
            for (int g = 0; g < nh; g++) a = fmaf(mix[h * nh + g], pr[((size_t)g * n_val + c) * vd + d], a);
        } else {
            a = pr[(size_t)h * n_val * vd + d];
        }
        o[e] = from_f32<TO>(a);
    }
    for (int e = threadIdx.x; e < ones; e += blockDim.x) o[nh * vd + e] = from_f32<TO>(e == 0 ? 1.0f : 0.0f);
}

extern "C" int hb_head_mix(const float* partial, const float* mix, void* out, int out_dtype, long long ldo, int n_tokens,
                           int n_heads, int n_kv_heads, int v_dim, int n_val, int ones, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv_heads > 0 && v_dim > 0 && ones >= 0, "head_mix: bad sizes");
    HB_REQUIRE(n_val == 1 || n_val == n_kv_heads, "head_mix: partial results hold %d value heads, 1 or %d expected", n_val, n_kv_heads);
    HB_REQUIRE(mix == nullptr || n_val == n_kv_heads, "head_mix: mixing needs the partial results of every value head");
    HB_REQUIRE(ldo >= (long long)n_heads * v_dim + ones, "head_mix: output rows are too short");
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == HB_BF16)
        hb_launch(head_mix_kernel<bf16>, dim3(n_tokens), dim3(256), 0, s, partial, mix, (bf16*)out, ldo, n_heads, n_kv_heads, v_dim, n_val, ones);
    else if (out_dtype == HB_F32)
        hb_launch(head_mix_kernel<float>, dim3(n_tokens), dim3(256), 0, s, partial, mix, (float*)out, ldo, n_heads, n_kv_heads, v_dim, n_val, ones);
    else return hb_fail("head_mix: unsupported output dtype %d", out_dtype);
    return hb_check_launch("head_mix");
}
