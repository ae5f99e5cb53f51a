// The matrix memory of the mLSTM mixer: a recurrent layer whose per-head state is a matrix
// S [d, dv], a vector n [d] and the running maximum m of the log gates.
//
// Per token and head, with log input gate i and log forget gate f (both capped, see below):
//   m' = max(f + m, i);  a = exp(f + m - m');  b = exp(i - m')
//   S' = a S + b k v^T;  n' = a n + b k
//   o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
// Gates from the pre-activations z_i, z_f: i = cap tanh(z_i / cap), f = logsigmoid(cap tanh(z_f / cap)).
// S, n and m start at zero.  Everything here is float32; q, k, v and the gates' pre-activations
// are read from the row of projections [q | k | v | gate | z_i | z_f] of each token.
//
// mlstm_scan: one block per (32 value columns, head, sequence) walks the sequence's tokens of the
// step in order.  The columns of S are independent of one another, so each block keeps its
// [d, 32] slice of S in shared memory; n and m are small and every block keeps its own copy
// (the block of the first columns writes them back).
// mlstm_output: o of each head divided by its root mean square, times the norm's weight, times
// sigmoid(gate).
#include "api.h"
#include "common.cuh"

#define ML_VS 32              // value columns per block
#define ML_WARPS 4
#define ML_MAX_D 512
#define ML_NR (ML_MAX_D / 32)

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

template <typename TP>
__global__ void __launch_bounds__(ML_VS * ML_WARPS)
mlstm_scan_kernel(const TP* __restrict__ proj, long long ldp, const float* __restrict__ gate_bias, float cap, float q_scale,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ state_slots,
                  const int* __restrict__ seq_start, float* __restrict__ out, int nh, int d, int dv) {
    pdl_trigger();
    extern __shared__ float smem[];
    float* S = smem;                              // [d][ML_VS]
    float* qs = S + (size_t)d * ML_VS;            // [d]
    float* ks = qs + d;                           // [d]
    float* red = ks + d;                          // [ML_WARPS][ML_VS]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int v0 = blockIdx.x * ML_VS, h = blockIdx.y, b = blockIdx.z;
    const int col = v0 + lane;
    const bool has_col = col < dv;
    const int start = seq_start[b], n_tok = seq_start[b + 1] - start;
    // state of a (sequence, head): S [nh][d][dv], then n [nh][d], then m [nh]
    float* base = state + (size_t)state_slots[b] * state_stride;
    float* gS = base + (size_t)h * d * dv;
    float* gn = base + (size_t)nh * d * dv + (size_t)h * d;
    float* gm = base + (size_t)nh * d * dv + (size_t)nh * d + h;
    const float bi = gate_bias ? gate_bias[h] : 0.0f, bf = gate_bias ? gate_bias[nh + h] : 0.0f;
    const int off_k = nh * d, off_v = 2 * nh * d, off_i = 2 * nh * d + 2 * nh * dv, off_f = off_i + nh;
    pdl_wait();
    proj = pdl_fresh(proj);
    base = pdl_fresh(base);
    for (int r = warp; r < d; r += ML_WARPS) S[r * ML_VS + lane] = has_col ? gS[(size_t)r * dv + col] : 0.0f;
    float nreg[ML_NR];
#pragma unroll
    for (int r = 0; r < ML_NR; r++) nreg[r] = (lane + 32 * r < d) ? gn[lane + 32 * r] : 0.0f;
    float m = gm[0];

    for (int t = 0; t < n_tok; t++) {
        const TP* row = proj + (size_t)(start + t) * ldp;
        for (int r = threadIdx.x; r < d; r += ML_VS * ML_WARPS) {
            qs[r] = to_f32(row[h * d + r]) * q_scale;
            ks[r] = to_f32(row[off_k + h * d + r]);
        }
        const float v = has_col ? to_f32(row[off_v + h * dv + col]) : 0.0f;
        const float zi = to_f32(row[off_i + h]) + bi, zf = to_f32(row[off_f + h]) + bf;
        const float li = cap * tanhf(zi / cap);
        const float lf = log_sigmoid(cap * tanhf(zf / cap));
        const float m_new = fmaxf(lf + m, li);
        const float keep = expf(lf + m - m_new), take = expf(li - m_new);
        m = m_new;
        __syncthreads();
        // every warp keeps the whole of n (the same arithmetic in each, so the same values)
        float nq = 0.0f;
#pragma unroll
        for (int r = 0; r < ML_NR; r++) {
            if (lane + 32 * r < d) {
                nreg[r] = fmaf(take, ks[lane + 32 * r], keep * nreg[r]);
                nq = fmaf(nreg[r], qs[lane + 32 * r], nq);
            }
        }
        nq = warp_sum(nq);
        const float tv = take * v;
        float num = 0.0f;
        for (int r = warp; r < d; r += ML_WARPS) {
            const float s = fmaf(ks[r], tv, keep * S[r * ML_VS + lane]);
            S[r * ML_VS + lane] = s;
            num = fmaf(s, qs[r], num);
        }
        red[warp * ML_VS + lane] = num;
        __syncthreads();
        if (warp == 0 && has_col) {
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < ML_WARPS; w++) total += red[w * ML_VS + lane];
            const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
            out[(size_t)(start + t) * nh * dv + (size_t)h * dv + col] = total / den;
        }
    }
    __syncthreads();
    if (n_tok > 0) {
        for (int r = warp; r < d; r += ML_WARPS)
            if (has_col) gS[(size_t)r * dv + col] = S[r * ML_VS + lane];
        if (blockIdx.x == 0 && warp == 0) {
#pragma unroll
            for (int r = 0; r < ML_NR; r++)
                if (lane + 32 * r < d) gn[lane + 32 * r] = nreg[r];
            if (lane == 0) gm[0] = m;
        }
    }
}

extern "C" int hb_mlstm_scan(const void* proj, int proj_dtype, long long ldp, const float* gate_bias, float cap, float q_scale,
                             float* state, long long state_stride, const int* state_slots, const int* seq_start, float* out,
                             int n_seqs, int n_heads, int d, int dv, void* stream) {
    if (n_seqs == 0) return 0;
    HB_REQUIRE(n_seqs > 0 && n_heads > 0 && d > 0 && dv > 0, "mlstm: bad sizes");
    HB_REQUIRE(d <= ML_MAX_D, "mlstm: key size %d is larger than %d", d, ML_MAX_D);
    HB_REQUIRE(n_heads <= 65535 && n_seqs <= 65535, "mlstm: too many heads or sequences");
    HB_REQUIRE(cap > 0.0f, "mlstm: the gates' cap must be positive");
    const size_t smem = ((size_t)d * ML_VS + 2 * (size_t)d + ML_WARPS * ML_VS) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((dv + ML_VS - 1) / ML_VS, n_heads, n_seqs);
    if (proj_dtype == HB_F32) {
        static bool done[HB_MAX_DEVICES];
        if (!done[hb_device_slot()]) {
            cudaFuncSetAttribute(mlstm_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(((size_t)ML_MAX_D * ML_VS + 2 * ML_MAX_D + ML_WARPS * ML_VS) * sizeof(float)));
            done[hb_device_slot()] = true;
        }
        hb_launch(mlstm_scan_kernel<float>, dim3(grid), dim3(ML_VS * ML_WARPS), smem, s, (const float*)proj, ldp, gate_bias, cap, q_scale, state,
                  state_stride, state_slots, seq_start, out, n_heads, d, dv);
    } else {
        return hb_fail("mlstm: the projections must be float32 (the gates enter the recurrence unrounded)");
    }
    return hb_check_launch("mlstm_scan");
}

// mlstm_chunks: the same recurrence for steps that bring many tokens, L tokens at a time.  Inside a chunk that starts
// from (S0, n0, m0), with F_j the sum of the log forget gates up to token j, a_s = i_s - F_s and
// A_j = max(m0, max_{s<=j} a_s):   m_j = F_j + A_j,
//   S_j = exp(m0 - A_j) S0 + sum_{s<=j} exp(a_s - A_j) k_s v_s^T      (n_j likewise with k_s alone),
// which is the recurrence unrolled, so
//   S_j^T q_j = exp(m0 - A_j) S0^T q_j + sum_{s<=j} exp(a_s - A_j) (q_j . k_s) v_s,
//   n_j . q_j = exp(m0 - A_j) n0 . q_j + sum_{s<=j} exp(a_s - A_j) (q_j . k_s).
// The tokens of a chunk no longer wait for one another: one pass over S0 serves L tokens, and the state moves once
// per chunk.  All in float32.  One block per (32 value columns, head, sequence), 4 warps, lane = value column.
#define MC_L 32
#define MC_WARPS 16           // sixteen warps: two tokens of a chunk each; the kernel waits on shared memory, more warps hide it
template <typename TP>
__global__ void __launch_bounds__(ML_VS * MC_WARPS)
mlstm_chunks_kernel(const TP* __restrict__ proj, long long ldp, const float* __restrict__ gate_bias, float cap, float q_scale,
                    float* __restrict__ state, long long state_stride, const int* __restrict__ state_slots,
                    const int* __restrict__ seq_start, float* __restrict__ out, int nh, int d, int dv, int L) {
    pdl_trigger();
    extern __shared__ float smem[];
    const int dp = d + 1;                               // padded rows: threads that read different tokens' rows hit different banks
    float* S = smem;                                    // [d][32]
    float* qs = S + (size_t)d * ML_VS;                  // [L][dp]
    float* ks = qs + (size_t)L * dp;                    // [L][dp]
    float* vs = ks + (size_t)L * dp;                    // [L][32]
    float* W = vs + L * ML_VS;                          // [L][L]: exp(a_s - A_j) (q_j . k_s) for s <= j, else 0
    float* ns = W + L * L;                              // [d]
    float* li_s = ns + d;                               // [L] and the following: per-token scalars of the chunk
    float* lf_s = li_s + L;
    float* g_s = lf_s + L;                              // exp(m0 - A_j)
    float* em_s = g_s + L;                              // exp(-m_j)
    float* A_s = em_s + L;
    float* a_s = A_s + L;
    float* Dl_s = a_s + L;                              // exp(a_s - A_last)
    __shared__ float m_shared;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int v0 = blockIdx.x * ML_VS, h = blockIdx.y, b = blockIdx.z;
    const int col = v0 + lane;
    const bool has_col = col < dv;
    const int start = seq_start[b], n_tok = seq_start[b + 1] - start;
    float* base = state + (size_t)state_slots[b] * state_stride;
    float* gS = base + (size_t)h * d * dv;
    float* gn = base + (size_t)nh * d * dv + (size_t)h * d;
    float* gm = base + (size_t)nh * d * dv + (size_t)nh * d + h;
    const float bi = gate_bias ? gate_bias[h] : 0.0f, bf = gate_bias ? gate_bias[nh + h] : 0.0f;
    const int off_k = nh * d, off_v = 2 * nh * d, off_i = 2 * nh * d + 2 * nh * dv, off_f = off_i + nh;
    pdl_wait();
    proj = pdl_fresh(proj);
    base = pdl_fresh(base);
    for (int r = warp; r < d; r += MC_WARPS) S[r * ML_VS + lane] = has_col ? gS[(size_t)r * dv + col] : 0.0f;
    for (int r = tid; r < d; r += ML_VS * MC_WARPS) ns[r] = gn[r];
    if (tid == 0) m_shared = gm[0];
    __syncthreads();

    for (int c0 = 0; c0 < n_tok; c0 += L) {
        const int nc = min(L, n_tok - c0);
        const float m0 = m_shared;
        // 1. the chunk's q (scaled), k, v and gates.  Two token rows per warp at a time, four values of q and of k
        // per lane and row: sixteen loads in flight per thread before the first is stored.
        for (int j0 = 2 * warp; j0 < nc; j0 += 2 * MC_WARPS) {
            for (int r0 = lane; r0 < d; r0 += 128) {
                float qv[2][4], kv[2][4];
#pragma unroll
                for (int jj = 0; jj < 2; jj++) {
                    const TP* row = proj + (size_t)(start + c0 + min(j0 + jj, nc - 1)) * ldp;
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int r = min(r0 + 32 * u, d - 1);
                        qv[jj][u] = to_f32(row[h * d + r]);
                        kv[jj][u] = to_f32(row[off_k + h * d + r]);
                    }
                }
#pragma unroll
                for (int jj = 0; jj < 2; jj++) {
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int r = r0 + 32 * u;
                        if (j0 + jj < nc && r < d) {
                            qs[(j0 + jj) * dp + r] = qv[jj][u] * q_scale;
                            ks[(j0 + jj) * dp + r] = kv[jj][u];
                        }
                    }
                }
            }
        }
        {
            float vv[MC_L / MC_WARPS];
#pragma unroll
            for (int i = 0; i < MC_L / MC_WARPS; i++) {
                const int j = min(warp + i * MC_WARPS, nc - 1);
                vv[i] = has_col ? to_f32(proj[(size_t)(start + c0 + j) * ldp + off_v + h * dv + col]) : 0.0f;
            }
#pragma unroll
            for (int i = 0; i < MC_L / MC_WARPS; i++) {
                const int j = warp + i * MC_WARPS;
                if (j < nc) vs[j * ML_VS + lane] = vv[i];
            }
        }
        if (tid < nc) {
            const TP* row = proj + (size_t)(start + c0 + tid) * ldp;
            const float zi = to_f32(row[off_i + h]) + bi, zf = to_f32(row[off_f + h]) + bf;
            li_s[tid] = cap * tanhf(zi / cap);
            lf_s[tid] = log_sigmoid(cap * tanhf(zf / cap));
        }
        __syncthreads();
        // 2. warp 0, lane = token: prefix sums of the forget gates, prefix maxima of a
        if (warp == 0) {
            float F = lane < nc ? lf_s[lane] : 0.0f;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, F, o);
                if (lane >= o) F += up;
            }
            const float a = lane < nc ? li_s[lane] - F : -INFINITY;
            float A = fmaxf(a, lane == 0 ? m0 : -INFINITY);
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, A, o);
                if (lane >= o) A = fmaxf(A, up);
            }
            const float A_last = __shfl_sync(0xffffffffu, A, nc - 1);
            if (lane < nc) {
                a_s[lane] = a;
                A_s[lane] = A;
                g_s[lane] = expf(m0 - A);
                em_s[lane] = expf(-(F + A));
                Dl_s[lane] = expf(a - A_last);
                if (lane == nc - 1) m_shared = F + A;        // read again only behind the barriers below
            }
        }
        __syncthreads();
        // 3. W[j][s]
        for (int i = tid; i < nc * nc; i += ML_VS * MC_WARPS) {
            const int j = i / nc, sidx = i - j * nc;
            float w = 0.0f;
            if (sidx <= j) {
                const float* qr = qs + j * dp;
                const float* kr = ks + sidx * dp;
                float dot = 0.0f;
                for (int r = 0; r < d; r++) dot = fmaf(qr[r], kr[r], dot);
                w = dot * expf(a_s[sidx] - A_s[j]);
            }
            W[j * L + sidx] = w;
        }
        __syncthreads();
        // 4. outputs: warp w takes the tokens w, w + 16
        {
            float acc[MC_L / MC_WARPS], nq[MC_L / MC_WARPS];
#pragma unroll
            for (int i = 0; i < MC_L / MC_WARPS; i++) acc[i] = 0.0f, nq[i] = 0.0f;
            for (int r = 0; r < d; r++) {
                const float sv = S[r * ML_VS + lane];
#pragma unroll
                for (int i = 0; i < MC_L / MC_WARPS; i++) {
                    const int j = warp + i * MC_WARPS;
                    if (j < nc) acc[i] = fmaf(sv, qs[j * dp + r], acc[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < MC_L / MC_WARPS; i++) {
                const int j = warp + i * MC_WARPS;
                if (j < nc) {
                    float p = 0.0f;
                    for (int r = lane; r < d; r += 32) p = fmaf(ns[r], qs[j * dp + r], p);
                    const float rowsum = lane < nc ? W[j * L + lane] : 0.0f;      // zero beyond the token itself
                    nq[i] = g_s[j] * warp_sum(p) + warp_sum(rowsum);
                    acc[i] *= g_s[j];
                }
            }
            for (int sidx = 0; sidx < nc; sidx++) {
                const float vv = vs[sidx * ML_VS + lane];
#pragma unroll
                for (int i = 0; i < MC_L / MC_WARPS; i++) {
                    const int j = warp + i * MC_WARPS;
                    if (j < nc) acc[i] = fmaf(W[j * L + sidx], vv, acc[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < MC_L / MC_WARPS; i++) {
                const int j = warp + i * MC_WARPS;
                if (j < nc && has_col) {
                    const float den = fmaxf(fabsf(nq[i]), em_s[j]) + 1e-6f;
                    out[(size_t)(start + c0 + j) * nh * dv + (size_t)h * dv + col] = acc[i] / den;
                }
            }
        }
        __syncthreads();
        // 5. the state at the chunk's end
        {
            const float g_last = g_s[nc - 1];
            float wv[MC_L];
#pragma unroll
            for (int sidx = 0; sidx < MC_L; sidx++) wv[sidx] = sidx < nc ? Dl_s[sidx] * vs[sidx * ML_VS + lane] : 0.0f;
            for (int r = warp; r < d; r += MC_WARPS) {
                float sv = g_last * S[r * ML_VS + lane];
#pragma unroll
                for (int sidx = 0; sidx < MC_L; sidx++)
                    if (sidx < nc) sv = fmaf(ks[sidx * dp + r], wv[sidx], sv);
                S[r * ML_VS + lane] = sv;
            }
            for (int r = tid; r < d; r += ML_VS * MC_WARPS) {
                float nv = g_last * ns[r];
                for (int sidx = 0; sidx < nc; sidx++) nv = fmaf(Dl_s[sidx], ks[sidx * dp + r], nv);
                ns[r] = nv;
            }
        }
        __syncthreads();
    }
    if (n_tok > 0) {
        for (int r = warp; r < d; r += MC_WARPS)
            if (has_col) gS[(size_t)r * dv + col] = S[r * ML_VS + lane];
        if (blockIdx.x == 0) {
            for (int r = tid; r < d; r += ML_VS * MC_WARPS) gn[r] = ns[r];
            if (tid == 0) gm[0] = m_shared;
        }
    }
}

static size_t mc_smem_bytes(int d, int L) {
    return ((size_t)d * ML_VS + 2 * (size_t)L * (d + 1) + (size_t)L * ML_VS + (size_t)L * L + d + 7 * (size_t)L) * sizeof(float);
}

extern "C" int hb_mlstm_chunks(const void* proj, int proj_dtype, long long ldp, const float* gate_bias, float cap, float q_scale,
                               float* state, long long state_stride, const int* state_slots, const int* seq_start, float* out,
                               int n_seqs, int n_heads, int d, int dv, void* stream) {
    if (n_seqs == 0) return 0;
    HB_REQUIRE(n_seqs > 0 && n_heads > 0 && d > 0 && dv > 0, "mlstm: bad sizes");
    HB_REQUIRE(d <= ML_MAX_D, "mlstm: key size %d is larger than %d", d, ML_MAX_D);
    HB_REQUIRE(n_heads <= 65535 && n_seqs <= 65535, "mlstm: too many heads or sequences");
    HB_REQUIRE(cap > 0.0f, "mlstm: the gates' cap must be positive");
    HB_REQUIRE(proj_dtype == HB_F32, "mlstm: the projections must be float32 (the gates enter the recurrence unrounded)");
    int L = MC_L;
    while (L > 4 && mc_smem_bytes(d, L) > 200 * 1024) L /= 2;
    const size_t smem = mc_smem_bytes(d, L);
    static bool done[HB_MAX_DEVICES];
    if (!done[hb_device_slot()]) {
        cudaError_t e = cudaFuncSetAttribute(mlstm_chunks_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return hb_fail("mlstm: %s", cudaGetErrorString(e));
        done[hb_device_slot()] = true;
    }
    dim3 grid((dv + ML_VS - 1) / ML_VS, n_heads, n_seqs);
    hb_launch(mlstm_chunks_kernel<float>, dim3(grid), dim3(ML_VS * MC_WARPS), smem, (cudaStream_t)stream, (const float*)proj, ldp, gate_bias,
              cap, q_scale, state, state_stride, state_slots, seq_start, out, n_heads, d, dv, L);
    return hb_check_launch("mlstm_chunks");
}

// out[t, h*dv + c] = o / sqrt(mean_c(o^2) + eps) * w[h*dv + c] * sigmoid(gate[t, h*dv + c])
template <typename TP, typename TO>
__global__ void __launch_bounds__(128)
mlstm_output_kernel(const float* __restrict__ o, const TP* __restrict__ gate, long long ldg, const float* __restrict__ w, float eps,
                    TO* __restrict__ out, long long ldo, int nh, int dv) {
    pdl_trigger();
    pdl_wait();
    o = pdl_fresh(o);
    gate = pdl_fresh(gate);
    __shared__ float scratch[33];
    const int t = blockIdx.x, h = blockIdx.y;
    const float* orow = o + ((size_t)t * nh + h) * dv;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) ss = fmaf(orow[c], orow[c], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        const float z = to_f32(gate[(size_t)t * ldg + h * dv + c]);
        out[(size_t)t * ldo + h * dv + c] = from_f32<TO>(orow[c] * inv * w[h * dv + c] / (1.0f + expf(-z)));
    }
}

extern "C" int hb_mlstm_output(const float* o, const void* gate, int gate_dtype, long long ldg, const float* w, float eps, void* out,
                               int out_dtype, long long ldo, int n_tokens, int n_heads, int dv, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && dv > 0 && n_heads <= 65535, "mlstm_output: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, n_heads);
    if (gate_dtype == HB_F32 && out_dtype == HB_F32)
        hb_launch(mlstm_output_kernel<float, float>, dim3(grid), dim3(128), 0, s, o, (const float*)gate, ldg, w, eps, (float*)out, ldo, n_heads, dv);
    else if (gate_dtype == HB_F32 && out_dtype == HB_BF16)
        hb_launch(mlstm_output_kernel<float, bf16>, dim3(grid), dim3(128), 0, s, o, (const float*)gate, ldg, w, eps, (bf16*)out, ldo, n_heads, dv);
    else return hb_fail("mlstm_output: unsupported dtypes %d -> %d", gate_dtype, out_dtype);
    return hb_check_launch("mlstm_output");
}
