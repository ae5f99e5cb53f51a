// Selective state-space scan (Mamba) and the short causal convolution in front of it.
//
// conv_act: u[t][c] = act(b[c] + sum_j w[c][j] x[t - taps + 1 + j][c]) per channel, zeros before a
// sequence's first token; the last taps - 1 inputs of every sequence are its state
// ([slot][taps - 1][C] floats), read by the step's first tokens and brought up to date.  x is a
// column range of a wider 32-bit matrix (row stride ldx).
//
// selective_scan: per token t, channel c, state index n (all 32-bit):
//   dt_c = softplus(dt_raw[t][c] + bdt[c]),  A[c][n] = -exp(A_log[c][n])        (dt_raw: the step-size projection's result)
//   S[c][n] <- exp(dt_c A[c][n]) S[c][n] + dt_c u[t][c] B[t][n]      (evaluated as S + expm1(dt A) S + dt u B)
//   y[t][c] = sum_n S[c][n] C[t][n] + D[c] u[t][c];   out[t][c] = y silu(z[t][c])
// with [B | C] the rows of one 32-bit matrix (columns of the result of the projection of u).  A group
// of SS_LANES threads owns a channel (state index n = lane, lane + SS_LANES, ...); a block owns
// SS_CH channels of one sequence and walks its tokens in order, SS_TOK tokens of inputs staged
// in shared memory at a time.  The state is read once and written once per step.
#include "api.h"
#include "common.cuh"

#define CA_CH 32
#define CA_TL 8
#define CA_RUN 256
#define CA_MAX_TAPS 16

template <typename TO>
__global__ void __launch_bounds__(CA_CH * CA_TL)
conv_act_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ cw, const float* __restrict__ cb, int taps,
                float* __restrict__ state, long long state_stride, const int* __restrict__ state_slots,
                const int* __restrict__ seq_start, TO* __restrict__ out, long long ldo, int C, int act) {
    pdl_trigger();
    const int c = blockIdx.x * CA_CH + (threadIdx.x & (CA_CH - 1));
    const int tl = threadIdx.x / CA_CH;
    const int b = blockIdx.y;
    const bool live = c < C;
    const int hist = taps - 1;
    float w[CA_MAX_TAPS], st[CA_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CA_MAX_TAPS; j++) w[j] = (live && j < taps) ? cw[(size_t)c * taps + j] : 0.0f;
    const float bias = (live && cb != nullptr) ? cb[c] : 0.0f;
    const int start = seq_start[b], n = seq_start[b + 1] - start;
    const int t_begin = blockIdx.z * CA_RUN, t_end = min(n, t_begin + CA_RUN);
    if (t_begin >= n) return;
    const bool first = blockIdx.z == 0;        // only a sequence's first run looks back beyond the step and owns the state
    float* srow = state + (size_t)state_slots[b] * state_stride;
    pdl_wait();
    x = pdl_fresh(x);
    srow = pdl_fresh(srow);
#pragma unroll
    for (int j = 0; j < CA_MAX_TAPS; j++) st[j] = (first && live && j < hist) ? srow[(size_t)j * C + c] : 0.0f;
    __syncthreads();                           // every thread has the old state before anyone writes the new one
    auto input = [&](int src) -> float {       // the sequence's input `src` of this step, or of an earlier step (src < 0)
        if (src < 0) {
            float v = 0.0f;
#pragma unroll
            for (int j = 0; j < CA_MAX_TAPS; j++) v = (j == hist + src) ? st[j] : v;
            return v;
        }
        return x[(size_t)(start + src) * ldx + c];
    };
    if (!live) return;
    for (int t = t_begin + tl; t < t_end; t += CA_TL) {
        float acc = bias;
#pragma unroll
        for (int j = 0; j < CA_MAX_TAPS; j++)
            if (j < taps) acc = fmaf(w[j], input(t - hist + j), acc);
        if (act == 1) acc = acc / (1.0f + expf(-acc));
        out[(size_t)(start + t) * ldo + c] = from_f32<TO>(acc);
    }
    if (first && tl == 0)
        for (int j = 0; j < hist; j++) srow[(size_t)j * C + c] = input(n - hist + j);
}

extern "C" int hb_conv_act(const float* x, long long ldx, const float* conv_w, const float* conv_b, int taps, float* state,
                           long long state_stride, const int* state_slots, const int* seq_start, void* out, int out_dtype,
                           long long ldo, int n_seqs, int max_new, int C, int act, void* stream) {
    if (n_seqs == 0) return 0;
    HB_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && C > 0 && ldx >= C && ldo >= C && max_new >= 1, "conv_act: bad sizes");
    HB_REQUIRE(taps >= 1 && taps <= CA_MAX_TAPS, "conv_act: %d taps (1..%d are built)", taps, CA_MAX_TAPS);
    static_assert(CA_RUN >= CA_MAX_TAPS - 1, "a sequence's first run holds every token that looks back beyond the step");
    HB_REQUIRE((max_new + CA_RUN - 1) / CA_RUN <= 65535, "conv_act: too many tokens in one sequence's step");
    HB_REQUIRE(act == 0 || act == 1, "conv_act: activation %d (0 none, 1 silu)", act);
    dim3 grid((C + CA_CH - 1) / CA_CH, n_seqs, (max_new + CA_RUN - 1) / CA_RUN), block(CA_CH * CA_TL);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == HB_BF16)
        hb_launch(conv_act_kernel<bf16>, dim3(grid), dim3(block), 0, s, x, ldx, conv_w, conv_b, taps, state, state_stride, state_slots, seq_start,
                  (bf16*)out, ldo, C, act);
    else if (out_dtype == HB_F32)
        hb_launch(conv_act_kernel<float>, dim3(grid), dim3(block), 0, s, x, ldx, conv_w, conv_b, taps, state, state_stride, state_slots, seq_start,
                  (float*)out, ldo, C, act);
    else return hb_fail("conv_act: unsupported output dtype %d", out_dtype);
    return hb_check_launch("conv_act");
}

// ------------------------------------------------------------------------------------------------ selective_scan
#define SS_THREADS 256
#define SS_TOK 32           // tokens of inputs staged at a time
#define SS_MAX_PER 8        // state values a thread holds: state sizes up to SS_MAX_PER * lanes

__device__ __forceinline__ float ss_softplus(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

template <typename TU, typename TO, int LANES>
__global__ void __launch_bounds__(SS_THREADS)
selective_scan_kernel(const TU* __restrict__ u, long long ldu, const float* __restrict__ bc, long long ldb,
                      const float* __restrict__ z, long long ldz, const float* __restrict__ dt_raw, long long lddt,
                      const float* __restrict__ b_dt, const float* __restrict__ a_log, const float* __restrict__ dvec,
                      float* __restrict__ state, long long state_stride, const int* __restrict__ state_slots,
                      const int* __restrict__ seq_start, TO* __restrict__ out, long long ldo, int I, int N) {
    pdl_trigger();
    constexpr int CH = SS_THREADS / LANES;             // channels per block
    extern __shared__ float ss_smem[];
    float* rows = ss_smem;                             // [SS_TOK][2 N]: B | C of the staged tokens
    float* us = rows + SS_TOK * 2 * N;                 // [SS_TOK][CH]
    float* zs = us + SS_TOK * CH;                      // [SS_TOK][CH]: silu(z)
    float* ds = zs + SS_TOK * CH;                      // [SS_TOK][CH]: the step sizes
    const int tid = threadIdx.x, lane = tid % LANES, ch = tid / LANES;
    const int c = blockIdx.x * CH + ch, b = blockIdx.y;
    const bool live = c < I;
    const int start = seq_start[b], n_all = seq_start[b + 1] - start;
    const int wrow = 2 * N;
    float A[SS_MAX_PER], S[SS_MAX_PER];
#pragma unroll
    for (int k = 0; k < SS_MAX_PER; k++) {
        const int n = lane + k * LANES;
        A[k] = (live && n < N) ? -expf(a_log[(size_t)c * N + n]) : 0.0f;
    }
    const float D = live ? dvec[c] : 0.0f;
    pdl_wait();
    u = pdl_fresh(u);
    bc = pdl_fresh(bc);
    z = pdl_fresh(z);
    dt_raw = pdl_fresh(dt_raw);
    state = pdl_fresh(state);
    float* srow = state + (size_t)state_slots[b] * state_stride + (size_t)(live ? c : 0) * N;
#pragma unroll
    for (int k = 0; k < SS_MAX_PER; k++) {
        const int n = lane + k * LANES;
        S[k] = (live && n < N) ? srow[n] : 0.0f;
    }
    for (int base = 0; base < n_all; base += SS_TOK) {
        const int nt = min(SS_TOK, n_all - base);
        __syncthreads();
        for (int i = tid; i < nt * wrow; i += SS_THREADS) {
            const int j = i / wrow, r = i - j * wrow;
            rows[j * wrow + r] = bc[(size_t)(start + base + j) * ldb + r];
        }
        for (int i = tid; i < nt * CH; i += SS_THREADS) {
            const int j = i / CH, k = i - j * CH, cc = blockIdx.x * CH + k;
            const size_t t = (size_t)(start + base + j);
            // what depends on (token, channel) alone is made here, once and by all threads, not in the walk below
            us[i] = cc < I ? to_f32(u[t * ldu + cc]) : 0.0f;
            const float zv = cc < I ? z[t * ldz + cc] : 0.0f;
            zs[i] = zv / (1.0f + expf(-zv));
            ds[i] = cc < I ? ss_softplus(dt_raw[t * lddt + cc] + b_dt[cc]) : 0.0f;
        }
        __syncthreads();
#pragma unroll 4
        for (int j = 0; j < nt; j++) {
            const float* row = rows + j * wrow;
            const float dt = ds[j * CH + ch];
            const float uv = us[j * CH + ch];
            const float dtu = dt * uv;
            float y = 0.0f;
#pragma unroll
            for (int k = 0; k < SS_MAX_PER; k++) {
                const int n = lane + k * LANES;
                if (n < N) {
                    // S <- S + (exp(dt A) - 1) S + dt u B: with decays close to one, exp() rounded to 32 bits is off by up to
                    // 6e-8 of 1, i.e. by percents of the distance to one, and that error would grow with every token
                    S[k] = fmaf(expm1f(dt * A[k]), S[k], fmaf(dtu, row[n], S[k]));
                    y = fmaf(S[k], row[N + n], y);
                }
            }
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o, LANES);
            if (lane == 0 && live) {
                out[(size_t)(start + base + j) * ldo + c] = from_f32<TO>((y + D * uv) * zs[j * CH + ch]);
            }
        }
    }
    if (live) {
#pragma unroll
        for (int k = 0; k < SS_MAX_PER; k++) {
            const int n = lane + k * LANES;
            if (n < N) srow[n] = S[k];
        }
    }
}

static int ss_lanes(int N) { return N <= 4 ? 4 : N <= 8 ? 8 : N <= 16 ? 16 : 32; }

extern "C" int hb_selective_scan(const void* u, int u_dtype, long long ldu, const float* bc, long long ldb, const float* z, long long ldz,
                                 const float* dt_raw, long long lddt, const float* b_dt, const float* a_log, const float* dvec, float* state,
                                 long long state_stride, const int* state_slots, const int* seq_start, void* out, int out_dtype,
                                 long long ldo, int n_seqs, int inner, int n_state, void* stream) {
    if (n_seqs == 0) return 0;
    HB_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && inner > 0 && n_state > 0, "selective_scan: bad sizes");
    HB_REQUIRE(n_state <= SS_MAX_PER * 32, "selective_scan: state size %d (up to %d is built)", n_state, SS_MAX_PER * 32);
    HB_REQUIRE(ldb >= 2 * n_state && ldu >= inner && ldz >= inner && lddt >= inner && ldo >= inner && state_stride >= (long long)inner * n_state,
               "selective_scan: rows are too short");
    HB_REQUIRE(u_dtype == out_dtype && (u_dtype == HB_BF16 || u_dtype == HB_F32), "selective_scan: unsupported dtypes %d -> %d", u_dtype, out_dtype);
    const int lanes = ss_lanes(n_state), ch = SS_THREADS / lanes;
    const size_t smem = sizeof(float) * ((size_t)SS_TOK * 2 * n_state + 3 * SS_TOK * ch);
    dim3 grid((inner + ch - 1) / ch, n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
#define HB_SS(TU, TO, L)                                                                                                                  \
    hb_launch(selective_scan_kernel<TU, TO, L>, dim3(grid), dim3(SS_THREADS), smem, s, (const TU*)u, ldu, bc, ldb, z, ldz, dt_raw, lddt,  \
              b_dt, a_log, dvec, state, state_stride, state_slots, seq_start, (TO*)out, ldo, inner, n_state)
#define HB_SS_L(TU, TO)                                                                          \
    switch (lanes) {                                                                             \
        case 4: HB_SS(TU, TO, 4); break;                                                         \
        case 8: HB_SS(TU, TO, 8); break;                                                         \
        case 16: HB_SS(TU, TO, 16); break;                                                       \
        default: HB_SS(TU, TO, 32); break;                                                       \
    }
    if (u_dtype == HB_BF16) { HB_SS_L(bf16, bf16) } else { HB_SS_L(float, float) }
#undef HB_SS_L
#undef HB_SS
    return hb_check_launch("selective_scan");
}
