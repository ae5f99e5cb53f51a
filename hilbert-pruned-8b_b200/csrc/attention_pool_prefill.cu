// The window part of attention_pool (attention_pool.cu) on the tensor cores, for steps that bring many tokens:
// bfloat16, key head size and value head size 64 or 128.
//
// One CTA = 64 consecutive new tokens of one sequence x one query head; each of its 4 warps owns 16 query rows
// (mma.sync m16n8k16).  The window's keys are walked page by page (64 keys) through a cp.async pipeline into swizzled
// shared memory.  Scores are 32-bit accumulators; the weight of a key is sigmoid(score * scale + bias[head]) in 32-bit,
// zero outside the window; there is no maximum and no sum to carry, since nothing is normalised.  Every weight enters
// the second product as two bfloat16 terms (hi + lo, exact to 16 mantissa bits).  The epilogue adds the pooled blocks'
// share (`pooled`, 32-bit, made by attention_pool's FP32 kernel in its pooled-only mode), multiplies by sigmoid(gate)
// and rounds once.
#include "api.h"
#include "mma.cuh"

#define APP_THREADS 128
#define APP_ROWS 64
#define APP_STAGES 2

template <int HD, int DV>
__global__ void __launch_bounds__(APP_THREADS)
attention_pool_prefill_kernel(const bf16* __restrict__ q, long long q_stride, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                              const int* __restrict__ page_table, int pt_width, const int* __restrict__ seq_start,
                              const int* __restrict__ seq_pos0, const float* __restrict__ head_bias, const float* __restrict__ pooled,
                              const float* __restrict__ gate, long long ldg, bf16* __restrict__ out, long long out_stride, int n_seqs,
                              int nh, int nkv, float scale, int window, int n_pages, int* status) {
    pdl_trigger();
    pdl_wait();
    q = pdl_fresh(q);
    kc = pdl_fresh(kc);
    vc = pdl_fresh(vc);
    pooled = pdl_fresh(pooled);
    gate = pdl_fresh(gate);
    constexpr int K_ROW = HD * 2, V_ROW = DV * 2;
    constexpr int K_TILE = HB_PAGE_TOKENS * K_ROW, V_TILE = HB_PAGE_TOKENS * V_ROW, STAGE = K_TILE + V_TILE;
    constexpr int KSTEPS = HD / 16;
    extern __shared__ __align__(128) uint8_t app_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = blockIdx.x, g = head / (nh / nkv);
    // blocks are taken from the back and the heads are the fast grid index (the longest blocks start first)
    int b = 0, blk = gridDim.y - 1 - blockIdx.y;
    for (; b < n_seqs; b++) {
        const int nb = (seq_start[b + 1] - seq_start[b] + APP_ROWS - 1) / APP_ROWS;
        if (blk < nb) break;
        blk -= nb;
    }
    if (b >= n_seqs) return;
    const int t_begin = seq_start[b], n_new = seq_start[b + 1] - t_begin, pos0 = seq_pos0[b];
    const int row_base = blk * APP_ROWS;
    const int rows_here = min(APP_ROWS, n_new - row_base);
    const int* pt = page_table + (size_t)b * pt_width;
    const float bias = head_bias != nullptr ? head_bias[head] : 0.0f;

    const int r0 = row_base + warp * 16 + (lane >> 2), r1 = r0 + 8;
    const int p0 = pos0 + r0, p1 = pos0 + r1;
    const bool v0 = r0 < n_new, v1 = r1 < n_new;
    uint32_t qf[KSTEPS][4];
    {
        const int c = (lane & 3) * 2;
        const bf16* q0 = q + (size_t)(t_begin + r0) * q_stride + (size_t)head * HD;
        const bf16* q1 = q + (size_t)(t_begin + r1) * q_stride + (size_t)head * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            qf[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + c) : 0u;
            qf[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + c) : 0u;
            qf[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + c + 8) : 0u;
            qf[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + c + 8) : 0u;
        }
    }
    const int first_pos = pos0 + row_base, last_pos = pos0 + row_base + rows_here - 1;
    const int lo_cta = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
    const int p_begin = lo_cta / HB_PAGE_TOKENS, p_end = last_pos / HB_PAGE_TOKENS + 1;
    const int lo0 = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
    const int lo1 = (window > 0 && p1 - window + 1 > 0) ? p1 - window + 1 : 0;
    const int w_first = pos0 + row_base + warp * 16, w_last = w_first + 15;
    const int w_lo = (window > 0 && w_first - window + 1 > 0) ? w_first - window + 1 : 0;

    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(app_smem);
    bool bad_page = false;
    auto load_page = [&](int stage, int page_idx) {
        if (page_idx < p_end) {
            int page = page_idx < pt_width ? pt[page_idx] : -1;
            if (page < 0 || page >= n_pages) {          // every page of [p_begin, p_end) holds a key that a row of this CTA sees
                bad_page = true;
                page = 0;
            }
            const uint8_t* ksrc = (const uint8_t*)(kc + ((size_t)page * nkv + g) * HB_PAGE_TOKENS * HD);
            const uint8_t* vsrc = (const uint8_t*)(vc + ((size_t)page * nkv + g) * HB_PAGE_TOKENS * DV);
            const uint32_t kdst = smem_base + stage * STAGE, vdst = kdst + K_TILE;
            for (int i = tid; i < HB_PAGE_TOKENS * (K_ROW / 16); i += APP_THREADS)
                cp_async_16(kdst + swizzled<K_ROW>(i / (K_ROW / 16), i % (K_ROW / 16)), ksrc + (size_t)i * 16);
            for (int i = tid; i < HB_PAGE_TOKENS * (V_ROW / 16); i += APP_THREADS)
                cp_async_16(vdst + swizzled<V_ROW>(i / (V_ROW / 16), i % (V_ROW / 16)), vsrc + (size_t)i * 16);
        }
        cp_async_commit();
    };

    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

#pragma unroll
    for (int s = 0; s < APP_STAGES - 1; s++) load_page(s, p_begin + s);

    for (int pi = p_begin; pi < p_end; pi++) {
        const int it = pi - p_begin;
        cp_async_wait<APP_STAGES - 2>();
        __syncthreads();
        load_page((it + APP_STAGES - 1) % APP_STAGES, pi + APP_STAGES - 1);
        const int page_first = pi * HB_PAGE_TOKENS, page_last = page_first + HB_PAGE_TOKENS - 1;
        if (page_first > w_last || page_last < w_lo) continue;          // nothing for this warp's rows here
        const uint32_t kt = smem_base + (it % APP_STAGES) * STAGE, vt = kt + K_TILE;

        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
            for (int kq = 0; kq < 4; kq++) {
                uint32_t kf[4];
                const int key_row = kq * 16 + ((lane >> 4) << 3) + (lane & 7);
                ldmatrix_x4(kf, kt + swizzled<K_ROW>(key_row, 2 * ks + ((lane >> 3) & 1)));
                mma_bf16_16816(s[2 * kq], qf[ks], kf[0], kf[1]);
                mma_bf16_16816(s[2 * kq + 1], qf[ks], kf[2], kf[3]);
            }
        }
        const bool edge = page_last > w_first || page_first < ((window > 0) ? w_last - window + 1 : 0);
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float w = __fdividef(1.0f, 1.0f + __expf(-(s[nt][e] * scale + bias)));
                if (edge) {
                    const int key = page_first + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const int pp = (e >> 1) ? p1 : p0, ll = (e >> 1) ? lo1 : lo0;
                    if (key > pp || key < ll) w = 0.0f;
                }
                s[nt][e] = w;
            }
#pragma unroll
        for (int kq = 0; kq < 4; kq++) {
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int f = 0; f < 4; f++) {
                const float a = s[2 * kq + (f >> 1)][(f & 1) * 2], c = s[2 * kq + (f >> 1)][(f & 1) * 2 + 1];
                const bf16 ah = __float2bfloat16_rn(a), ch = __float2bfloat16_rn(c);
                hi[f] = pack_bf16(a, c);
                lo[f] = pack_bf16(a - __bfloat162float(ah), c - __bfloat162float(ch));
            }
            const int v_row = kq * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
            for (int dn = 0; dn < DV / 16; dn++) {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, vt + swizzled<V_ROW>(v_row, 2 * dn + (lane >> 4)));
                mma_bf16_16816(o[2 * dn], hi, vf[0], vf[1]);
                mma_bf16_16816(o[2 * dn + 1], hi, vf[2], vf[3]);
                mma_bf16_16816(o[2 * dn], lo, vf[0], vf[1]);
                mma_bf16_16816(o[2 * dn + 1], lo, vf[2], vf[3]);
            }
        }
    }
    cp_async_wait<0>();
    if (bad_page && tid == 0) hb_note(status, HB_STATUS_PAGE, 1 + b);

    const int c = (lane & 3) * 2;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        if (!(h ? v1 : v0)) continue;
        const size_t t = (size_t)(t_begin + (h ? r1 : r0));
        const size_t col0 = (size_t)head * DV + c;
        bf16* dst = out + t * out_stride + col0;
#pragma unroll
        for (int i = 0; i < DV / 8; i++) {
            float a = o[i][2 * h], d = o[i][2 * h + 1];
            if (pooled != nullptr) {
                a += pooled[t * ((size_t)nh * DV) + col0 + i * 8];
                d += pooled[t * ((size_t)nh * DV) + col0 + i * 8 + 1];
            }
            if (gate != nullptr) {
                a *= 1.0f / (1.0f + expf(-gate[t * ldg + col0 + i * 8]));
                d *= 1.0f / (1.0f + expf(-gate[t * ldg + col0 + i * 8 + 1]));
            }
            *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(a, d);
        }
    }
}

extern "C" int hb_attention_pool_prefill_supported(int head_dim, int v_dim) {
    return (head_dim == 64 || head_dim == 128) && (v_dim == 64 || v_dim == 128);
}

template <int HD, int DV>
static int app_launch(const void* q, long long q_stride, const void* kc, const void* vc, const int* page_table, int pt_width,
                      const int* seq_start, const int* seq_pos0, const float* head_bias, const float* pooled, const float* gate, long long ldg,
                      void* out, long long out_stride, int n_seqs, int q_blocks, int nh, int nkv, float scale, int window, int n_pages,
                      int* status, cudaStream_t s) {
    constexpr int SMEM = APP_STAGES * HB_PAGE_TOKENS * (HD + DV) * 2;
    static bool attr_done[HB_MAX_DEVICES] = {};
    bool& attr_set = attr_done[hb_device_slot()];
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attention_pool_prefill_kernel<HD, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return hb_fail("attention_pool_prefill: cannot reserve %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    dim3 grid(nh, q_blocks);
    hb_launch(attention_pool_prefill_kernel<HD, DV>, dim3(grid), dim3(APP_THREADS), SMEM, s, (const bf16*)q, q_stride, (const bf16*)kc,
              (const bf16*)vc, page_table, pt_width, seq_start, seq_pos0, head_bias, pooled, gate, ldg, (bf16*)out, out_stride, n_seqs, nh, nkv,
              scale, window, n_pages, status);
    return hb_check_launch("attention_pool_prefill");
}

// q_blocks = sum over sequences of ceil(new tokens / 64); pooled: float32 [tokens][heads * v_dim] or null
extern "C" int hb_attention_pool_prefill(const void* q, long long q_stride, const void* k_cache, const void* v_cache, const int* page_table,
                                         int pt_width, const int* seq_start, const int* seq_pos0, const float* head_bias,
                                         const float* pooled, const float* gate, long long ldg, void* out, long long out_stride, int n_seqs,
                                         int q_blocks, int n_heads, int n_kv_heads, int head_dim, int v_dim, float scale, int window,
                                         int n_pages, int* status, void* stream) {
    if (n_seqs == 0 || q_blocks == 0) return 0;
    HB_REQUIRE(hb_attention_pool_prefill_supported(head_dim, v_dim), "attention_pool_prefill: head sizes %d / %d are not built (64 or 128)", head_dim, v_dim);
    HB_REQUIRE(n_seqs > 0 && q_blocks > 0 && q_blocks <= 65535 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attention_pool_prefill: bad sizes");
    HB_REQUIRE(q_stride % 2 == 0 && out_stride % 2 == 0 && ((uintptr_t)q & 3) == 0 && ((uintptr_t)out & 3) == 0,
               "attention_pool_prefill: queries and output must be 4-byte aligned");
    HB_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0, "attention_pool_prefill: cache must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
#define HB_APP(HD, DV) return app_launch<HD, DV>(q, q_stride, k_cache, v_cache, page_table, pt_width, seq_start, seq_pos0, head_bias, pooled, gate, \
                                                 ldg, out, out_stride, n_seqs, q_blocks, n_heads, n_kv_heads, scale, window, n_pages, status, s)
    if (head_dim == 64 && v_dim == 64) HB_APP(64, 64);
    if (head_dim == 64 && v_dim == 128) HB_APP(64, 128);
    if (head_dim == 128 && v_dim == 64) HB_APP(128, 64);
    HB_APP(128, 128);
#undef HB_APP
}
