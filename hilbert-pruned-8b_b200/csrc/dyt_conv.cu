// Dynamic-tanh norm, the short causal convolution over time with its per-sequence state, and
// the squared-ReLU activation.
//
// Dynamic tanh: y = tanh(alpha * x) * w + b with a scalar alpha; no statistic of x is taken.
// Short convolution: out[t] = h[t] + sum_j cw[c][j] * h[t - taps + 1 + j] per channel c, zeros
// before a sequence's first token; the last taps - 1 inputs h of every sequence are its state
// and carry over from step to step.  The convolution kernel can apply the norm to its input
// itself (x is then the residual stream and h = dyt(x)), so that norm and convolution are one
// pass over x.  Everything is computed in float32; only the result is rounded to the output type.
#include "api.h"
#include "common.cuh"

#define HB_MAX_TAPS 16

template <typename TO>
__global__ void __launch_bounds__(256)
dyt_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
           const float* __restrict__ alpha, TO* __restrict__ out, long long ldo, const int* __restrict__ rows, int C) {
    pdl_trigger();
    const float a = alpha[0];
    pdl_wait();
    x = pdl_fresh(x);
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const float* xr = x + (size_t)src * C;
    TO* o = out + (size_t)r * ldo;
    for (int i = threadIdx.x; i < C; i += blockDim.x) o[i] = from_f32<TO>(fmaf(tanhf(a * xr[i]), w[i], b[i]));
}

extern "C" int hb_dyt(const float* x, const float* w, const float* b, const float* alpha, void* out, int out_dtype,
                      long long ldo, const int* rows, int n_rows, int C, void* stream) {
    if (n_rows == 0) return 0;
    HB_REQUIRE(n_rows > 0 && C > 0 && ldo >= C, "dyt: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == HB_BF16) hb_launch(dyt_kernel<bf16>, dim3(n_rows), dim3(256), 0, s, x, w, b, alpha, (bf16*)out, ldo, rows, C);
    else if (out_dtype == HB_F32) hb_launch(dyt_kernel<float>, dim3(n_rows), dim3(256), 0, s, x, w, b, alpha, (float*)out, ldo, rows, C);
    else return hb_fail("dyt: unsupported output dtype %d", out_dtype);
    return hb_check_launch("dyt");
}

// Blocks (channel chunk of 32, sequence, run of SC_RUN tokens): 32 channel lanes x 8 token lanes.  Only
// the block of a sequence's first run touches the state: it reads the old state first (the only tokens
// that look back beyond the step are in its run, SC_RUN >= taps - 1), walks its tokens, and at its end
// replaces the state by the last taps - 1 inputs of the sequence (old ones where the step brought
// fewer), which it makes from x again.  No other block reads or writes this (sequence, channel) state,
// so the barrier between its reads and its writes is all the ordering needed.
#define SC_CH 32
#define SC_TL 8
#define SC_RUN 256
template <typename TO, bool NORM>
__global__ void __launch_bounds__(SC_CH * SC_TL)
short_conv_kernel(const float* __restrict__ x, const float* __restrict__ nw, const float* __restrict__ nb,
                  const float* __restrict__ nalpha, const float* __restrict__ cw, int taps, float* __restrict__ state,
                  long long state_stride, const int* __restrict__ state_slots, const int* __restrict__ seq_start,
                  TO* __restrict__ out, long long ldo, int C) {
    pdl_trigger();
    const int c = blockIdx.x * SC_CH + (threadIdx.x & (SC_CH - 1));
    const int tl = threadIdx.x / SC_CH;
    const int b = blockIdx.y;
    const bool live = c < C;
    const int hist = taps - 1;
    float w[HB_MAX_TAPS], st[HB_MAX_TAPS];
    float a = 0.0f, gw = 0.0f, gb = 0.0f;
#pragma unroll
    for (int j = 0; j < HB_MAX_TAPS; j++) w[j] = (live && j < taps) ? cw[(size_t)c * taps + j] : 0.0f;
    if (NORM) {
        a = nalpha[0];
        gw = live ? nw[c] : 0.0f;
        gb = live ? nb[c] : 0.0f;
    }
    const int start = seq_start[b], n = seq_start[b + 1] - start;
    const int t_begin = blockIdx.z * SC_RUN, t_end = min(n, t_begin + SC_RUN);
    if (t_begin >= n) return;
    const bool first = blockIdx.z == 0;
    float* srow = state + (size_t)state_slots[b] * state_stride;
    pdl_wait();
    x = pdl_fresh(x);
    srow = pdl_fresh(srow);
#pragma unroll
    for (int j = 0; j < HB_MAX_TAPS - 1; j++) st[j] = (first && live && j < hist) ? srow[(size_t)j * C + c] : 0.0f;
    __syncthreads();
    auto input = [&](int src) -> float {            // h of the sequence's token `src` of this step, or of an earlier step
        if (src < 0) {
            float v = 0.0f;
#pragma unroll
            for (int j = 0; j < HB_MAX_TAPS - 1; j++) v = (j == hist + src) ? st[j] : v;
            return v;
        }
        const float xv = x[(size_t)(start + src) * C + c];
        return NORM ? fmaf(tanhf(a * xv), gw, gb) : xv;
    };
    if (live) {
        for (int t = t_begin + tl; t < t_end; t += SC_TL) {
            float acc = 0.0f, h = 0.0f;
#pragma unroll
            for (int j = 0; j < HB_MAX_TAPS; j++) {
                if (j < taps) {
                    h = input(t - hist + j);
                    acc = fmaf(w[j], h, acc);
                }
            }
            out[(size_t)(start + t) * ldo + c] = from_f32<TO>(h + acc);
        }
        if (first && tl == 0) {
            for (int j = 0; j < hist; j++) srow[(size_t)j * C + c] = input(n - hist + j);
        }
    }
}

// The same with the number of taps known at compile time (1..8): a thread walks SC_RUN / SC_TL consecutive tokens and
// keeps the last TAPS inputs in registers, so every input is normed once (the general kernel above norms it once per tap).
template <typename TO, bool NORM, int TAPS>
__global__ void __launch_bounds__(SC_CH * SC_TL)
short_conv_taps_kernel(const float* __restrict__ x, const float* __restrict__ nw, const float* __restrict__ nb,
                       const float* __restrict__ nalpha, const float* __restrict__ cw, float* __restrict__ state,
                       long long state_stride, const int* __restrict__ state_slots, const int* __restrict__ seq_start,
                       TO* __restrict__ out, long long ldo, int C) {
    pdl_trigger();
    constexpr int HIST = TAPS - 1, PER = SC_RUN / SC_TL;
    const int c = blockIdx.x * SC_CH + (threadIdx.x & (SC_CH - 1));
    const int tl = threadIdx.x / SC_CH;
    const int b = blockIdx.y;
    const bool live = c < C;
    float w[TAPS], st[TAPS];            // st[HIST] unused: arrays of TAPS - 1 elements would be empty for one tap
    float a = 0.0f, gw = 0.0f, gb = 0.0f;
#pragma unroll
    for (int j = 0; j < TAPS; j++) w[j] = live ? cw[(size_t)c * TAPS + j] : 0.0f;
    if (NORM) {
        a = nalpha[0];
        gw = live ? nw[c] : 0.0f;
        gb = live ? nb[c] : 0.0f;
    }
    const int start = seq_start[b], n = seq_start[b + 1] - start;
    const int t_begin = blockIdx.z * SC_RUN, t_end = min(n, t_begin + SC_RUN);
    if (t_begin >= n) return;
    const bool first = blockIdx.z == 0;
    float* srow = state + (size_t)state_slots[b] * state_stride;
    pdl_wait();
    x = pdl_fresh(x);
    srow = pdl_fresh(srow);
#pragma unroll
    for (int j = 0; j < TAPS; j++) st[j] = (first && live && j < HIST) ? srow[(size_t)j * C + c] : 0.0f;
    __syncthreads();
    auto input = [&](int src) -> float {
        if (src < 0) {
            float v = 0.0f;
#pragma unroll
            for (int j = 0; j < TAPS; j++) v = (j == HIST + src) ? st[j] : v;
            return v;
        }
        const float xv = x[(size_t)(start + src) * C + c];
        return NORM ? fmaf(tanhf(a * xv), gw, gb) : xv;
    };
    if (!live) return;
    const int t0 = t_begin + tl * PER, t1 = min(t_end, t0 + PER);
    if (t0 < t1) {
        float win[TAPS];
#pragma unroll
        for (int j = 0; j < HIST; j++) win[j] = input(t0 - HIST + j);
        for (int t = t0; t < t1; t++) {
            const float h = input(t);
            win[HIST] = h;
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < TAPS; j++) acc = fmaf(w[j], win[j], acc);
            out[(size_t)(start + t) * ldo + c] = from_f32<TO>(h + acc);
#pragma unroll
            for (int j = 0; j < HIST; j++) win[j] = win[j + 1];
        }
    }
    if (first && tl == 0) {
#pragma unroll
        for (int j = 0; j < HIST; j++) srow[(size_t)j * C + c] = input(n - HIST + j);
    }
}

template <typename TO, bool NORM>
static void short_conv_taps_launch(int taps, dim3 grid, dim3 block, cudaStream_t s, const float* x, const float* nw, const float* nb,
                                   const float* na, const float* cw, float* state, long long state_stride, const int* state_slots,
                                   const int* seq_start, void* out, long long ldo, int C) {
#define HB_SCT(T) case T: hb_launch(short_conv_taps_kernel<TO, NORM, T>, dim3(grid), dim3(block), 0, s, x, nw, nb, na, cw, state, state_stride,   \
                                    state_slots, seq_start, (TO*)out, ldo, C); break;
    switch (taps) { HB_SCT(1) HB_SCT(2) HB_SCT(3) HB_SCT(4) HB_SCT(5) HB_SCT(6) HB_SCT(7) HB_SCT(8) }
#undef HB_SCT
}

extern "C" int hb_short_conv(const float* x, const float* norm_w, const float* norm_b, const float* norm_alpha,
                             const float* conv_w, int taps, float* state, long long state_stride, const int* state_slots,
                             const int* seq_start, void* out, int out_dtype, long long ldo, int n_seqs, int max_new, int C,
                             void* stream) {
    if (n_seqs == 0) return 0;
    HB_REQUIRE(n_seqs > 0 && C > 0 && ldo >= C && max_new >= 1, "short_conv: bad sizes");
    static_assert(SC_RUN >= HB_MAX_TAPS - 1, "a sequence's first run holds every token that looks back beyond the step");
    HB_REQUIRE(taps >= 1 && taps <= HB_MAX_TAPS, "short_conv: %d taps (1..%d are built)", taps, HB_MAX_TAPS);
    HB_REQUIRE(n_seqs <= 65535, "short_conv: too many sequences");
    cudaStream_t s = (cudaStream_t)stream;
    HB_REQUIRE((max_new + SC_RUN - 1) / SC_RUN <= 65535, "short_conv: too many tokens in one sequence's step");
    dim3 grid((C + SC_CH - 1) / SC_CH, n_seqs, (max_new + SC_RUN - 1) / SC_RUN), block(SC_CH * SC_TL);
#define HB_SC_LAUNCH(TO, NORM)                                                                                              \
    hb_launch(short_conv_kernel<TO, NORM>, dim3(grid), dim3(block), 0, s, x, norm_w, norm_b, norm_alpha, conv_w, taps, state,           \
              state_stride, state_slots, seq_start, (TO*)out, ldo, C)
    const bool norm = norm_w != nullptr;
    if (taps <= 8 && (out_dtype == HB_BF16 || out_dtype == HB_F32)) {
        if (out_dtype == HB_BF16) {
            if (norm) short_conv_taps_launch<bf16, true>(taps, grid, block, s, x, norm_w, norm_b, norm_alpha, conv_w, state, state_stride, state_slots, seq_start, out, ldo, C);
            else short_conv_taps_launch<bf16, false>(taps, grid, block, s, x, norm_w, norm_b, norm_alpha, conv_w, state, state_stride, state_slots, seq_start, out, ldo, C);
        } else {
            if (norm) short_conv_taps_launch<float, true>(taps, grid, block, s, x, norm_w, norm_b, norm_alpha, conv_w, state, state_stride, state_slots, seq_start, out, ldo, C);
            else short_conv_taps_launch<float, false>(taps, grid, block, s, x, norm_w, norm_b, norm_alpha, conv_w, state, state_stride, state_slots, seq_start, out, ldo, C);
        }
        return hb_check_launch("short_conv");
    }
    if (out_dtype == HB_BF16) { if (norm) HB_SC_LAUNCH(bf16, true); else HB_SC_LAUNCH(bf16, false); }
    else if (out_dtype == HB_F32) { if (norm) HB_SC_LAUNCH(float, true); else HB_SC_LAUNCH(float, false); }
    else return hb_fail("short_conv: unsupported output dtype %d", out_dtype);
#undef HB_SC_LAUNCH
    return hb_check_launch("short_conv");
}

// out = max(x, 0)^2, the square taken in float32
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
relu2_kernel(const TI* __restrict__ in, long long ldi, TO* __restrict__ out, long long ldo, int n) {
    pdl_trigger();
    pdl_wait();
    in = pdl_fresh(in);
    const TI* ir = in + (size_t)blockIdx.y * ldi;
    TO* o = out + (size_t)blockIdx.y * ldo;
    if (sizeof(TI) == 4 && ((n | ldi | ldo) & 3) == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
        // four values per thread: 16-byte loads, 8- or 16-byte stores
        for (int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += gridDim.x * blockDim.x * 4) {
            const float4 x = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(ir) + i);
            const float a = fmaxf(x.x, 0.0f), b = fmaxf(x.y, 0.0f), c = fmaxf(x.z, 0.0f), d = fmaxf(x.w, 0.0f);
            TO r[4] = {from_f32<TO>(a * a), from_f32<TO>(b * b), from_f32<TO>(c * c), from_f32<TO>(d * d)};
            if (sizeof(TO) == 4) *reinterpret_cast<float4*>(o + i) = *reinterpret_cast<const float4*>(r);
            else *reinterpret_cast<uint2*>(o + i) = *reinterpret_cast<const uint2*>(r);
        }
        return;
    }
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = fmaxf(to_f32(ir[i]), 0.0f);
        o[i] = from_f32<TO>(v * v);
    }
}

extern "C" int hb_relu2(const void* in, int in_dtype, long long ldi, void* out, int out_dtype, long long ldo, int n_rows,
                        int n, void* stream) {
    if (n_rows == 0 || n == 0) return 0;
    HB_REQUIRE(n_rows > 0 && n > 0 && n_rows <= 65535 * 32, "relu2: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    HB_REQUIRE(n_rows <= 65535, "relu2: too many rows");
    dim3 grid(min((n + 1023) / 1024, 64), n_rows);
    if (in_dtype == HB_F32 && out_dtype == HB_F32)
        hb_launch(relu2_kernel<float, float>, dim3(grid), dim3(256), 0, s, (const float*)in, ldi, (float*)out, ldo, n);
    else if (in_dtype == HB_F32 && out_dtype == HB_BF16)
        hb_launch(relu2_kernel<float, bf16>, dim3(grid), dim3(256), 0, s, (const float*)in, ldi, (bf16*)out, ldo, n);
    else if (in_dtype == HB_BF16 && out_dtype == HB_BF16)
        hb_launch(relu2_kernel<bf16, bf16>, dim3(grid), dim3(256), 0, s, (const bf16*)in, ldi, (bf16*)out, ldo, n);
    else return hb_fail("relu2: unsupported dtypes %d -> %d", in_dtype, out_dtype);
    return hb_check_launch("relu2");
}
