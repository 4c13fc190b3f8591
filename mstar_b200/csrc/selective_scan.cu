// Selective scan (the Mamba mixer): a short causal convolution per channel with SiLU, and a
// diagonal linear recurrence per channel whose step size and input/output maps depend on the
// token.  Per-request state in a slot: the convolution's last taps-1 inputs [taps-1][inner],
// then S [inner][state], all float.
//
//   conv   xc[t, c] = silu(b_c + sum_k w[c, k] x[t - (taps-1) + k, c]), inputs before the
//          portion's start from the slot, zeros before the sequence's start (a fresh slot).
//   scan   dt = softplus(W_dt dt_in + b_dt);  S[c, n] = exp(dt_c A[c, n]) S[c, n] + dt_c xc_c B_n;
//          y_c = sum_n S[c, n] C_n + D_c xc_c;  out = y * silu(z).
//
// Step sizes, decays, their exponentials, the state and its sums are float for both
// activation types; a channel's arithmetic does not depend on the rest of the batch.
#include "common.cuh"

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// ------------------------------------------------------------------ convolution + SiLU
// xz: [tokens] rows of ld elements, x in columns [0, inner).  One thread per (token, channel).
template <typename A, typename W>
__global__ void conv_silu_kernel(const A* __restrict__ xz, int ld, const W* __restrict__ w,
                                 const W* __restrict__ bias, const int* __restrict__ token_req,
                                 const int* __restrict__ qo_indptr, const int* __restrict__ slots,
                                 const float* __restrict__ state, long long state_stride,
                                 A* __restrict__ out, int tokens, int inner, int taps) {
    xz = pdl_after(xz, pdl_wait());
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)tokens * inner) return;
    const int t = (int)(idx / inner), c = (int)(idx - (size_t)t * inner);
    const int e = token_req[t];
    const int start = qo_indptr[e], local = t - start;
    const float* past = state + (size_t)slots[e] * state_stride;   // [taps-1][inner]
    float acc = to_float(bias[c]);
    for (int k = 0; k < taps; ++k) {
        const int src = local - (taps - 1) + k;
        const float v = src >= 0 ? to_float(xz[(size_t)(start + src) * ld + c])
                                 : past[(size_t)(taps - 1 + src) * inner + c];
        acc = fmaf(to_float(w[(size_t)c * taps + k]), v, acc);
    }
    out[idx] = from_float<A>(silu_f(acc));
}

MSTAR_API int mstar_conv_silu(const void* xz, int ld, const void* w, const void* bias,
                              int weight_dtype, const int* token_req, const int* qo_indptr,
                              const int* slots, const float* state, long long state_stride,
                              void* out, int act_dtype, int tokens, int inner, int taps,
                              void* stream) {
    if (tokens <= 0) return 0;
    if (inner <= 0 || taps <= 0) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)tokens * inner;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
#define GO(A, W)                                                                                  \
    mstar_launch((conv_silu_kernel<A, W>), dim3(blocks), dim3(threads), 0, s, (const A*)xz, ld,   \
                 (const W*)w, (const W*)bias, token_req, qo_indptr, slots, state, state_stride,   \
                 (A*)out, tokens, inner, taps)
    if (act_dtype == MSTAR_F32) {
        if (weight_dtype == MSTAR_F32) { GO(float, float); } else { GO(float, bf16); }
    } else {
        if (weight_dtype == MSTAR_F32) { GO(bf16, float); } else { GO(bf16, bf16); }
    }
#undef GO
    return launch_status();
}

// ------------------------------------------------------------------ the recurrence
#define SS_CH 32          // channels of a block
#define SS_TC 16          // tokens staged at a time
#define SS_NPER 16        // most states a lane holds

struct ScanArgs {
    int inner, n_state, rank, taps, ld_xz, entries;
    long long state_stride;
};

// A block takes one batch entry and SS_CH channels; LANES lanes share a channel: lane s
// holds states s, s + LANES, ...  Tokens come in chunks of SS_TC: the chunk's [dt_in | B | C]
// rows, conv outputs and gates are staged in shared memory, the step sizes of the chunk are
// made for all its tokens at once (W_dt read once a chunk), then the chain runs token by
// token.  At the end the state goes back to the slot and the convolution's window moves on.
template <typename A, int LANES>
__global__ void __launch_bounds__(SS_CH * LANES)
selective_scan_kernel(const A* __restrict__ xc, const A* __restrict__ xz,
                      const float* __restrict__ proj, const float* __restrict__ w_dt,
                      const float* __restrict__ dt_bias, const float* __restrict__ a_neg,
                      const float* __restrict__ d_skip, const int* __restrict__ qo_indptr,
                      const int* __restrict__ slots, float* __restrict__ state,
                      A* __restrict__ out, ScanArgs a) {
    extern __shared__ float sm[];
    const int row = a.rank + 2 * a.n_state;
    float* rows = sm;                                  // [SS_TC][row]
    float* xs = rows + SS_TC * row;                    // [SS_TC][SS_CH]
    float* zs = xs + SS_TC * SS_CH;                    // [SS_TC][SS_CH]
    const int e = blockIdx.x;
    const int tid = threadIdx.x, sub = tid % LANES, ch = tid / LANES;
    const int c = blockIdx.y * SS_CH + ch;
    const bool live = c < a.inner;
    const int cc = live ? c : a.inner - 1;
    const unsigned long long waited = pdl_wait();
    xc = pdl_after(xc, waited);
    xz = pdl_after(xz, waited);
    proj = pdl_after(proj, waited);
    const int start = qo_indptr[e], n_tok = qo_indptr[e + 1] - start;
    float* slot = state + (size_t)slots[e] * a.state_stride;
    float* s_slot = slot + (size_t)(a.taps - 1) * a.inner + (size_t)cc * a.n_state;

    float S[SS_NPER], An[SS_NPER];
#pragma unroll
    for (int i = 0; i < SS_NPER; ++i) {
        const int n = sub + LANES * i;
        S[i] = n < a.n_state ? s_slot[n] : 0.f;
        An[i] = n < a.n_state ? a_neg[(size_t)cc * a.n_state + n] : 0.f;
    }
    const float bias = dt_bias[cc], dsk = d_skip[cc];
    const float* wrow = w_dt + (size_t)cc * a.rank;

    for (int t0 = 0; t0 < n_tok; t0 += SS_TC) {
        const int nt = min(SS_TC, n_tok - t0);
        __syncthreads();
        for (int i = tid; i < nt * row; i += SS_CH * LANES) {
            const int k = i / row, r = i - k * row;
            rows[k * row + r] = proj[(size_t)(start + t0 + k) * row + r];
        }
        for (int i = tid; i < nt * SS_CH; i += SS_CH * LANES) {
            const int k = i / SS_CH, j = i - k * SS_CH;
            const int col = min(blockIdx.y * SS_CH + j, a.inner - 1);
            xs[i] = to_float(xc[(size_t)(start + t0 + k) * a.inner + col]);
            zs[i] = to_float(xz[(size_t)(start + t0 + k) * a.ld_xz + a.inner + col]);
        }
        __syncthreads();
        // step sizes of the chunk
        float dt[SS_TC];
#pragma unroll
        for (int k = 0; k < SS_TC; ++k) dt[k] = 0.f;
        for (int r = sub; r < a.rank; r += LANES) {
            const float w = wrow[r];
#pragma unroll
            for (int k = 0; k < SS_TC; ++k) dt[k] = fmaf(w, rows[k * row + r], dt[k]);
        }
#pragma unroll
        for (int k = 0; k < SS_TC; ++k) {
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) dt[k] += __shfl_xor_sync(0xffffffffu, dt[k], o);
            dt[k] = softplus_f(dt[k] + bias);
        }
        // the chain
#pragma unroll
        for (int k = 0; k < SS_TC; ++k) {
            if (k < nt) {
                const float x = xs[k * SS_CH + ch];
                const float dx = dt[k] * x;
                const float* B = rows + k * row + a.rank;
                const float* C = B + a.n_state;
                float y = 0.f;
#pragma unroll
                for (int i = 0; i < SS_NPER; ++i) {
                    const int n = sub + LANES * i;
                    if (n < a.n_state) {
                        S[i] = fmaf(expf(dt[k] * An[i]), S[i], dx * B[n]);
                        y = fmaf(S[i], C[n], y);
                    }
                }
#pragma unroll
                for (int o = LANES / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
                if (sub == 0 && live) {
                    y = fmaf(dsk, x, y);
                    out[(size_t)(start + t0 + k) * a.inner + c] =
                        from_float<A>(y * silu_f(zs[k * SS_CH + ch]));
                }
            }
        }
    }
    if (!live) return;
#pragma unroll
    for (int i = 0; i < SS_NPER; ++i) {
        const int n = sub + LANES * i;
        if (n < a.n_state) s_slot[n] = S[i];
    }
    if (sub == 0 && n_tok > 0) {
        // the window of the convolution: the last taps-1 inputs of [old window | this portion]
        for (int j = 0; j < a.taps - 1; ++j) {
            const int at = n_tok + j;                  // index into the joined sequence
            slot[(size_t)j * a.inner + c] =
                at < a.taps - 1 ? slot[(size_t)at * a.inner + c]
                                : to_float(xz[(size_t)(start + at - (a.taps - 1)) * a.ld_xz + c]);
        }
    }
}

// xc: [tokens, inner] conv outputs; xz: [tokens] rows of ld_xz elements, x then z; proj: float
// [tokens, rank + 2 n_state]; w_dt float [inner, rank]; a_neg float [inner, n_state] = -exp(A_log);
// out [tokens, inner].  Returns 0, a CUDA error code, or -1 when the shape is refused.
MSTAR_API int mstar_selective_scan(const void* xc, const void* xz, int ld_xz, const float* proj,
                                   const float* w_dt, const float* dt_bias, const float* a_neg,
                                   const float* d_skip, const int* qo_indptr, const int* slots,
                                   float* state, long long state_stride, void* out, int act_dtype,
                                   int entries, int inner, int n_state, int rank, int taps,
                                   void* stream) {
    if (entries <= 0) return 0;
    if (inner <= 0 || n_state <= 0 || rank <= 0 || taps <= 0 || n_state > 16 * SS_NPER) return -1;
    const size_t smem = sizeof(float) * ((size_t)SS_TC * (rank + 2 * n_state) + 2 * SS_TC * SS_CH);
    if (smem > 200 * 1024) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    ScanArgs a{inner, n_state, rank, taps, ld_xz, entries, state_stride};
    dim3 grid(entries, (inner + SS_CH - 1) / SS_CH);
#define GO(A, LANES)                                                                              \
    {                                                                                             \
        static size_t configured = 0;                                                             \
        if (smem > 48 * 1024 && smem > configured) {                                              \
            cudaFuncSetAttribute(selective_scan_kernel<A, LANES>,                                 \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
            configured = smem;                                                                    \
        }                                                                                         \
        mstar_launch((selective_scan_kernel<A, LANES>), grid, dim3(SS_CH * LANES), smem, s,       \
                     (const A*)xc, (const A*)xz, proj, w_dt, dt_bias, a_neg, d_skip, qo_indptr,   \
                     slots, state, (A*)out, a);                                                   \
    }
    if (n_state <= 4 * SS_NPER) {
        if (act_dtype == MSTAR_F32) GO(float, 4) else GO(bf16, 4)
    } else {
        if (act_dtype == MSTAR_F32) GO(float, 16) else GO(bf16, 16)
    }
#undef GO
    return launch_status();
}
