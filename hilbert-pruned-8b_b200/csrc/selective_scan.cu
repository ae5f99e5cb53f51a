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
//
// Steps that bring many tokens to a sequence cut its tokens into chunks of `chunk_len` and run three launches, so that the
// chunks run side by side instead of one block walking thousands of tokens: (1) every chunk from a zero state, without
// outputs: its final state L and the sum of its step sizes; (2) scan_carry: chunk by chunk, S_start[k + 1] = exp(A sum dt_k)
// S_start[k] + L_k (the recurrence is linear in S, and the product of a chunk's decays is the exponential of the sum), which
// also leaves the sequence's new state; (3) every chunk again from its S_start, with outputs.  Same sums, another order.
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
    constexpr int PER = CA_RUN / CA_TL, TOP = CA_MAX_TAPS - 1;
    const int t0 = t_begin + tl * PER, t1 = min(t_end, t0 + PER);
    if (n <= CA_TL) {
        // a handful of tokens (decode steps): one token a thread, its inputs read tap by tap
        const int t = t_begin + tl;
        if (t < t_end) {
            float acc = bias;
#pragma unroll
            for (int j = 0; j < CA_MAX_TAPS; j++)
                if (j < taps) acc = fmaf(w[j], input(t - hist + j), acc);
            if (act == 1) acc = acc / (1.0f + expf(-acc));
            out[(size_t)(start + t) * ldo + c] = from_f32<TO>(acc);
        }
    } else if (t0 < t1) {
        // a thread walks CA_RUN / CA_TL consecutive tokens and keeps the last inputs in registers, newest at the top: one load
        // per token; the taps sit at the top of their array likewise, zeros below them
        float win[CA_MAX_TAPS], wr[CA_MAX_TAPS];
        float w_now = 0.0f;
#pragma unroll
        for (int j = 0; j < CA_MAX_TAPS; j++) {
            const int back = TOP - j + 1;                  // win[j] is the input `back` tokens before the current one
            win[j] = back <= hist ? input(t0 - back) : 0.0f;
            float wv = 0.0f;
#pragma unroll
            for (int k = 0; k < CA_MAX_TAPS; k++) wv = (k == hist - back) ? w[k] : wv;
            wr[j] = back <= hist ? wv : 0.0f;
            w_now = (j == hist) ? w[j] : w_now;
        }
        for (int t = t0; t < t1; t++) {
            const float xin = x[(size_t)(start + t) * ldx + c];
            float acc = fmaf(w_now, xin, bias);
#pragma unroll
            for (int j = 0; j < CA_MAX_TAPS; j++) acc = fmaf(wr[j], win[j], acc);
            if (act == 1) acc = acc / (1.0f + expf(-acc));
            out[(size_t)(start + t) * ldo + c] = from_f32<TO>(acc);
#pragma unroll
            for (int j = 0; j < TOP; j++) win[j] = win[j + 1];
            win[TOP] = xin;
        }
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
// exp(x) - 1 for x <= 0.  FAST (the bfloat16 path): six terms of the series near zero (remainder below 1e-9 of x), the hardware's
// exp2 elsewhere, where the decay is far from one and an error of 2e-7 of it does not build up; else the library's expm1.
template <bool FAST>
__device__ __forceinline__ float ss_expm1(float x) {
    if (!FAST) return expm1f(x);
    if (x > -0.125f) {
        float p = fmaf(x, 1.0f / 720.0f, 1.0f / 120.0f);
        p = fmaf(p, x, 1.0f / 24.0f);
        p = fmaf(p, x, 1.0f / 6.0f);
        p = fmaf(p, x, 0.5f);
        p = fmaf(p, x, 1.0f);
        return p * x;
    }
    return __expf(x) - 1.0f;
}

template <typename TU, typename TO, int LANES>
__global__ void __launch_bounds__(SS_THREADS)
selective_scan_kernel(const TU* __restrict__ u, long long ldu, const float* __restrict__ bc, long long ldb,
                      const float* __restrict__ z, long long ldz, const float* __restrict__ dt_raw, long long lddt,
                      const float* __restrict__ b_dt, const float* __restrict__ a_log, const float* __restrict__ dvec,
                      float* __restrict__ state, long long state_stride, const int* __restrict__ state_slots,
                      const int* __restrict__ seq_start, TO* __restrict__ out, long long ldo, int I, int N, int mode, int chunk_len,
                      int max_chunks, float* __restrict__ carry_L, float* __restrict__ carry_dt, const float* __restrict__ carry_S0) {
    // mode 0: the whole step from the sequence's state; 1: chunk blockIdx.z from zeros, no outputs, L and sum dt out;
    // 3: chunk blockIdx.z from carry_S0, with outputs (the state was written by scan_carry)
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
    const int n_seq = seq_start[b + 1] - seq_start[b];
    const int t_lo = mode == 0 ? 0 : (int)blockIdx.z * chunk_len;
    if (t_lo >= n_seq && mode != 0) return;
    const int start = seq_start[b] + t_lo, n_all = mode == 0 ? n_seq : min(chunk_len, n_seq - t_lo);
    const size_t carry_at = ((size_t)b * max_chunks + blockIdx.z) * I + (c < I ? c : 0);
    const int wrow = 2 * N;
    float A[SS_MAX_PER], S[SS_MAX_PER];
    float sum_dt = 0.0f;
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
    carry_S0 = pdl_fresh(carry_S0);
    float* srow = state + (size_t)state_slots[b] * state_stride + (size_t)(live ? c : 0) * N;
#pragma unroll
    for (int k = 0; k < SS_MAX_PER; k++) {
        const int n = lane + k * LANES;
        S[k] = 0.0f;
        if (live && n < N && mode != 1) S[k] = mode == 0 ? srow[n] : carry_S0[carry_at * N + n];
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
            sum_dt += dt;
            float y = 0.0f;
#pragma unroll
            for (int k = 0; k < SS_MAX_PER; k++) {
                const int n = lane + k * LANES;
                if (n < N) {
                    // S <- S + (exp(dt A) - 1) S + dt u B: with decays close to one, exp() rounded to 32 bits is off by up to
                    // 6e-8 of 1, i.e. by percents of the distance to one, and that error would grow with every token
                    S[k] = fmaf(ss_expm1<sizeof(TU) == 2>(dt * A[k]), S[k], fmaf(dtu, row[n], S[k]));
                    y = fmaf(S[k], row[N + n], y);
                }
            }
            if (mode == 1) continue;                   // only the chunk's final state is wanted
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o, LANES);
            if (lane == 0 && live) {
                out[(size_t)(start + base + j) * ldo + c] = from_f32<TO>((y + D * uv) * zs[j * CH + ch]);
            }
        }
    }
    if (live && mode != 3) {
#pragma unroll
        for (int k = 0; k < SS_MAX_PER; k++) {
            const int n = lane + k * LANES;
            if (n < N) (mode == 0 ? srow : carry_L + carry_at * N)[n] = S[k];
        }
        if (mode == 1 && lane == 0) carry_dt[carry_at] = sum_dt;
    }
}

// S_start of every chunk and the sequence's new state: one thread per (sequence, channel, state index)
__global__ void __launch_bounds__(256)
scan_carry_kernel(const float* __restrict__ a_log, const float* __restrict__ carry_L, const float* __restrict__ carry_dt,
                  float* __restrict__ carry_S0, float* __restrict__ state, long long state_stride, const int* __restrict__ state_slots,
                  const int* __restrict__ seq_start, int I, int N, int chunk_len, int max_chunks) {
    pdl_trigger();
    pdl_wait();
    carry_L = pdl_fresh(carry_L);
    carry_dt = pdl_fresh(carry_dt);
    state = pdl_fresh(state);
    const int b = blockIdx.y;
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long long)I * N) return;
    const int c = (int)(i / N);
    const int chunks = (seq_start[b + 1] - seq_start[b] + chunk_len - 1) / chunk_len;
    const float A = -expf(a_log[i]);
    float* sp = state + (size_t)state_slots[b] * state_stride + i;
    float S = *sp;
    for (int k = 0; k < chunks; k++) {
        const size_t at = ((size_t)b * max_chunks + k) * I;
        carry_S0[at * N + i] = S;
        S = fmaf(expm1f(A * carry_dt[at + c]), S, S) + carry_L[at * N + i];
    }
    *sp = S;
}

// Lanes per channel: four state values a thread where the state is large enough (fewer instructions per channel: the loads,
// the loop and the shuffle sum are shared by a thread's values), but more lanes while the grid has fewer than two blocks per
// SM: a block's walk is a chain of dependent steps and of staging loads that nothing hides but other blocks (measured at
// 8192 channels of 16 state values, 2048 tokens: 1.33 ms with 16 lanes and 512 blocks, 1.77 ms with 4 lanes and 128 blocks).
static int ss_lanes(int N, int inner, long long grids) {
    int full = N <= 4 ? 4 : N <= 8 ? 8 : N <= 16 ? 16 : 32;               // one value a lane (up to SS_MAX_PER beyond 32)
    int lanes = full / 4 < 4 ? 4 : full / 4;
    while (lanes * SS_MAX_PER < N) lanes *= 2;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, hb_device_slot());
    while (lanes < full && (long long)((inner + SS_THREADS / lanes - 1) / (SS_THREADS / lanes)) * grids < 2 * sms) lanes *= 2;
    return lanes;
}

extern "C" int hb_selective_scan(const void* u, int u_dtype, long long ldu, const float* bc, long long ldb, const float* z, long long ldz,
                                 const float* dt_raw, long long lddt, const float* b_dt, const float* a_log, const float* dvec, float* state,
                                 long long state_stride, const int* state_slots, const int* seq_start, void* out, int out_dtype,
                                 long long ldo, int n_seqs, int inner, int n_state, int chunk_len, int max_chunks, float* carry,
                                 long long carry_floats, void* stream) {
    if (n_seqs == 0) return 0;
    HB_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && inner > 0 && n_state > 0, "selective_scan: bad sizes");
    HB_REQUIRE(n_state <= SS_MAX_PER * 32, "selective_scan: state size %d (up to %d is built)", n_state, SS_MAX_PER * 32);
    HB_REQUIRE(ldb >= 2 * n_state && ldu >= inner && ldz >= inner && lddt >= inner && ldo >= inner && state_stride >= (long long)inner * n_state,
               "selective_scan: rows are too short");
    HB_REQUIRE(u_dtype == out_dtype && (u_dtype == HB_BF16 || u_dtype == HB_F32), "selective_scan: unsupported dtypes %d -> %d", u_dtype, out_dtype);
    const long long per = (long long)n_seqs * max_chunks * inner;               // (sequence, chunk, channel) triples
    HB_REQUIRE(chunk_len == 0 || (chunk_len > 0 && max_chunks > 0 && max_chunks <= 65535 && carry != nullptr && carry_floats >= per * (2 * n_state + 1)),
               "selective_scan: chunks need (2 * state + 1) floats per sequence, chunk and channel");
    float* carry_L = carry;
    float* carry_S0 = carry ? carry + per * n_state : nullptr;
    float* carry_dt = carry ? carry + 2 * per * n_state : nullptr;
    const int lanes = ss_lanes(n_state, inner, (long long)n_seqs * (chunk_len ? max_chunks : 1)), ch = SS_THREADS / lanes;
    const size_t smem = sizeof(float) * ((size_t)SS_TOK * 2 * n_state + 3 * SS_TOK * ch);
    HB_REQUIRE(smem <= 200 * 1024, "selective_scan: state size %d needs too much shared memory", n_state);
    cudaStream_t s = (cudaStream_t)stream;
#define HB_SS(TU, TO, L, MODE)                                                                                                            \
    if (smem > 48 * 1024) {                                                                                                               \
        static bool done[HB_MAX_DEVICES] = {};                                                                                            \
        const int slot = hb_device_slot();                                                                                                \
        if (!done[slot]) {                                                                                                                \
            cudaError_t e = cudaFuncSetAttribute(selective_scan_kernel<TU, TO, L>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return hb_fail("selective_scan: shared memory: %s", cudaGetErrorString(e));                             \
            done[slot] = true;                                                                                                            \
        }                                                                                                                                 \
    }                                                                                                                                     \
    hb_launch(selective_scan_kernel<TU, TO, L>, dim3((inner + ch - 1) / ch, n_seqs, MODE == 0 ? 1 : max_chunks), dim3(SS_THREADS), smem, s,  \
              (const TU*)u, ldu, bc, ldb, z, ldz, dt_raw, lddt, b_dt, a_log, dvec, state, state_stride, state_slots, seq_start, (TO*)out,    \
              ldo, inner, n_state, MODE, chunk_len, max_chunks, carry_L, carry_dt, (const float*)carry_S0)
#define HB_SS_L(TU, TO, MODE)                                                                    \
    switch (lanes) {                                                                             \
        case 4: HB_SS(TU, TO, 4, MODE); break;                                                   \
        case 8: HB_SS(TU, TO, 8, MODE); break;                                                   \
        case 16: HB_SS(TU, TO, 16, MODE); break;                                                 \
        default: HB_SS(TU, TO, 32, MODE); break;                                                 \
    }
#define HB_SS_M(MODE)                                                                            \
    do {                                                                                         \
        if (u_dtype == HB_BF16) { HB_SS_L(bf16, bf16, MODE) } else { HB_SS_L(float, float, MODE) } \
    } while (0)
    if (chunk_len == 0) {
        HB_SS_M(0);
        return hb_check_launch("selective_scan");
    }
    HB_SS_M(1);
    if (hb_check_launch("selective_scan (chunks from zero)")) return 1;
    const long long elems = (long long)inner * n_state;
    hb_launch(scan_carry_kernel, dim3((unsigned)((elems + 255) / 256), n_seqs), dim3(256), 0, s, a_log, (const float*)carry_L,
              (const float*)carry_dt, carry_S0, state, state_stride, state_slots, seq_start, inner, n_state, chunk_len, max_chunks);
    if (hb_check_launch("scan_carry")) return 1;
    HB_SS_M(3);
#undef HB_SS_M
#undef HB_SS_L
#undef HB_SS
    return hb_check_launch("selective_scan (chunks with outputs)");
}
