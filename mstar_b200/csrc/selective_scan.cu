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
// xz: [tokens] rows of ld elements, x in columns [0, inner).  One thread per (token, channel):
// a block row of the grid is a token, so neighbours in a warp are neighbouring channels.
template <typename A, typename W>
__global__ void conv_silu_kernel(const A* __restrict__ xz, int ld, const W* __restrict__ w,
                                 const W* __restrict__ bias, const int* __restrict__ token_req,
                                 const int* __restrict__ qo_indptr, const int* __restrict__ slots,
                                 const float* __restrict__ state, long long state_stride,
                                 A* __restrict__ out, int t_first, int inner, int taps) {
    xz = pdl_after(xz, pdl_wait());
    const int t = t_first + blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= inner) return;
    const size_t idx = (size_t)t * inner + c;
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

// The same for 8 channels a thread with 16-byte accesses: weights transposed to float
// [taps][inner], bias float; inner and ld multiples of 8.
template <typename A>
__global__ void conv_silu_vec_kernel(const A* __restrict__ xz, int ld, const float* __restrict__ wt,
                                     const float* __restrict__ bias, const int* __restrict__ token_req,
                                     const int* __restrict__ qo_indptr, const int* __restrict__ slots,
                                     const float* __restrict__ state, long long state_stride,
                                     A* __restrict__ out, int t_first, int inner, int taps) {
    xz = pdl_after(xz, pdl_wait());
    const int t = t_first + blockIdx.y, c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= inner) return;
    const int e = token_req[t];
    const int start = qo_indptr[e], local = t - start;
    const float* past = state + (size_t)slots[e] * state_stride;
    float acc[8];
    load8(bias + c, acc);
    for (int k = 0; k < taps; ++k) {
        const int src = local - (taps - 1) + k;
        float v[8], w[8];
        if (src >= 0) load8(xz + (size_t)(start + src) * ld + c, v);
        else load8(past + (size_t)(taps - 1 + src) * inner + c, v);
        load8(wt + (size_t)k * inner + c, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[i], v[i], acc[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = silu_f(acc[i]);
    store8(out + (size_t)t * inner + c, acc);
}

MSTAR_API int mstar_conv_silu_vec(const void* xz, int ld, const float* wt, const float* bias,
                                  const int* token_req, const int* qo_indptr, const int* slots,
                                  const float* state, long long state_stride, void* out,
                                  int act_dtype, int tokens, int inner, int taps, void* stream) {
    if (tokens <= 0) return 0;
    if (inner <= 0 || taps <= 0 || inner % 8 || ld % 8 || state_stride % 4) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const int lanes = inner / 8;
    const int threads = lanes >= 128 ? 128 : 32;
    for (int t0 = 0; t0 < tokens; t0 += 65535) {
        const dim3 blocks((lanes + threads - 1) / threads, tokens - t0 < 65535 ? tokens - t0 : 65535);
        if (act_dtype == MSTAR_F32)
            mstar_launch((conv_silu_vec_kernel<float>), blocks, dim3(threads), 0, s, (const float*)xz,
                         ld, wt, bias, token_req, qo_indptr, slots, state, state_stride, (float*)out,
                         t0, inner, taps);
        else
            mstar_launch((conv_silu_vec_kernel<bf16>), blocks, dim3(threads), 0, s, (const bf16*)xz,
                         ld, wt, bias, token_req, qo_indptr, slots, state, state_stride, (bf16*)out,
                         t0, inner, taps);
    }
    return launch_status();
}

MSTAR_API int mstar_conv_silu(const void* xz, int ld, const void* w, const void* bias,
                              int weight_dtype, const int* token_req, const int* qo_indptr,
                              const int* slots, const float* state, long long state_stride,
                              void* out, int act_dtype, int tokens, int inner, int taps,
                              void* stream) {
    if (tokens <= 0) return 0;
    if (inner <= 0 || taps <= 0) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = inner >= 256 ? 256 : 64;
#define GO(A, W)                                                                                  \
    mstar_launch((conv_silu_kernel<A, W>), blocks, dim3(threads), 0, s, (const A*)xz, ld,         \
                 (const W*)w, (const W*)bias, token_req, qo_indptr, slots, state, state_stride,   \
                 (A*)out, t0, inner, taps)
    // (a grid's second dimension ends at 65,535: longer batches go in slices)
    for (int t0 = 0; t0 < tokens; t0 += 65535) {
        const dim3 blocks((inner + threads - 1) / threads, tokens - t0 < 65535 ? tokens - t0 : 65535);
        if (act_dtype == MSTAR_F32) {
            if (weight_dtype == MSTAR_F32) { GO(float, float); } else { GO(float, bf16); }
        } else {
            if (weight_dtype == MSTAR_F32) { GO(bf16, float); } else { GO(bf16, bf16); }
        }
    }
#undef GO
    return launch_status();
}

// ------------------------------------------------------------------ the recurrence
#define SS_THREADS 64     // threads of a block: SS_THREADS / LANES channels
#define SS_TC 16          // tokens staged at a time

// 4 bytes global -> shared, asynchronously (rows of floats have no wider alignment)
__device__ __forceinline__ void cp_async_4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(
                     (uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_all_done() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}

struct ScanArgs {
    int inner, n_state, rank, taps, ld_xz, entries;
    long long state_stride;
    // a long portion is cut into pieces of `piece` tokens (0: not cut) that run side by side:
    // pass 1 walks every piece but the last from a zero state and leaves its end state and the
    // sum of its step sizes in scratch (the recurrence is linear: the state after a piece is
    // exp(A sum dt) times the state before it, plus that end state); pass 2 starts every piece
    // from the state so joined and writes the outputs
    int piece, pass, max_pieces;
    float* piece_state;   // [entries][max_pieces][inner][n_state]
    float* piece_dt;      // [entries][max_pieces][inner]
    // W_dt dt_in of every token and channel, made by a product of its own [tokens][inner]
    // (long portions), or nullptr: the kernel makes it from the staged rows
    const float* dt_pre;
};

// A block takes one batch entry and SS_THREADS / LANES channels; LANES lanes share a channel:
// lane s holds states s, s + LANES, ... (NPER of them).  Tokens come in chunks of SS_TC: the
// chunk's [dt_in | B | C] rows, conv outputs and gates stand in shared memory, and the next
// chunk's are on their way (the rows by asynchronous copies into the other buffer, x and z
// in registers) while this one is walked.  The step sizes of a chunk
// are made for all its tokens at once (W_dt read once a chunk), then the chain runs token by
// token: one multiply-add per state on the chain, the decays' exponentials beside it.  At the
// end the state goes back to the slot and the convolution's window moves on.
template <typename A, int LANES, int NPER>
__global__ void __launch_bounds__(SS_THREADS, 8)
selective_scan_kernel(const A* __restrict__ xc, const A* __restrict__ xz,
                      const float* __restrict__ proj, const float* __restrict__ w_dt,
                      const float* __restrict__ dt_bias, const float* __restrict__ a_neg,
                      const float* __restrict__ d_skip, const int* __restrict__ qo_indptr,
                      const int* __restrict__ slots, float* __restrict__ state,
                      A* __restrict__ out, ScanArgs a) {
    constexpr int CH = SS_THREADS / LANES;
    extern __shared__ float sm[];
    const int row = a.rank + 2 * a.n_state;
    const int buf_floats = SS_TC * row + 3 * SS_TC * CH;   // rows, then x, z, and W_dt dt_in
    const int e = blockIdx.x;
    const int tid = threadIdx.x, sub = tid % LANES, ch = tid / LANES;
    const int c = blockIdx.y * CH + ch;
    const bool live = c < a.inner;
    const int cc = live ? c : a.inner - 1;
    const unsigned long long waited = pdl_wait();
    xc = pdl_after(xc, waited);
    xz = pdl_after(xz, waited);
    proj = pdl_after(proj, waited);
    const int e_start = qo_indptr[e], e_tok = qo_indptr[e + 1] - e_start;
    // this block's piece of the entry's tokens
    const int piece = blockIdx.z;
    const int pieces = a.piece > 0 ? max(1, (e_tok + a.piece - 1) / a.piece) : 1;
    if (piece >= pieces || (a.pass == 1 && piece == pieces - 1)) return;
    const int start = e_start + piece * (a.piece > 0 ? a.piece : 0);
    const int n_tok = a.piece > 0 ? min(a.piece, e_tok - piece * a.piece) : e_tok;
    const bool last_piece = piece == pieces - 1;
    float* slot = state + (size_t)slots[e] * a.state_stride;
    float* s_slot = slot + (size_t)(a.taps - 1) * a.inner + (size_t)cc * a.n_state;

    float S[NPER], An[NPER];
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
        const int n = sub + LANES * i;
        S[i] = 0.f;
        // A in units of log2(e): the decays are then 2^(dt A), one exponential instruction
        An[i] = n < a.n_state ? a_neg[(size_t)cc * a.n_state + n] * 1.4426950408889634f : 0.f;
    }
    // The state the portion starts from.  Cut into pieces, the last piece puts the new state
    // into the slot while others may not have started: so pass 1 leaves a copy of the old one
    // in the scratch entry of the last piece (which pass 1 does not walk), and pass 2 reads that.
    float* kept_start = a.piece_state + (((size_t)e * a.max_pieces + pieces - 1) * a.inner + cc) * a.n_state;
    const float* s_from = (a.pass == 2 && pieces > 1) ? kept_start : s_slot;
    if (a.pass == 1 && piece == 0 && live) {
#pragma unroll
        for (int i = 0; i < NPER; ++i) {
            const int n = sub + LANES * i;
            if (n < a.n_state) kept_start[n] = s_slot[n];
        }
    }
    if (a.pass != 1) {
#pragma unroll
        for (int i = 0; i < NPER; ++i) {
            const int n = sub + LANES * i;
            if (n < a.n_state) S[i] = s_from[n];
        }
    }
    if (a.pass == 2) {
        // the state before this piece: the slot's, carried over the pieces before it
        for (int j = 0; j < piece; ++j) {
            const size_t at = (size_t)e * a.max_pieces + j;
            const float sdt = a.piece_dt[at * a.inner + cc];
            const float* E = a.piece_state + (at * a.inner + cc) * a.n_state;
#pragma unroll
            for (int i = 0; i < NPER; ++i) {
                const int n = sub + LANES * i;
                if (n < a.n_state) S[i] = fmaf(exp2f(sdt * An[i]), S[i], E[n]);
            }
        }
    }
    float dt_sum = 0.f;
    const float bias = dt_bias[cc], dsk = d_skip[cc];
    const float* wrow = w_dt + (size_t)cc * a.rank;

    // what a thread fetches of a chunk: its share of the rows, and of the x and z values
    const int row_items = SS_TC * row, xz_items = SS_TC * CH;
    float pf_x[(SS_TC * CH + SS_THREADS - 1) / SS_THREADS],
        pf_z[(SS_TC * CH + SS_THREADS - 1) / SS_THREADS],
        pf_d[(SS_TC * CH + SS_THREADS - 1) / SS_THREADS];
    const float* dt_pre = pdl_after(a.dt_pre, waited);
    auto fetch = [&](float* buf, int t0, int nt) {
        const float* src = proj + (size_t)(start + t0) * row;
        for (int i = tid; i < nt * row; i += SS_THREADS) cp_async_4(buf + i, src + i);
#pragma unroll
        for (int k = 0; k < (xz_items + SS_THREADS - 1) / SS_THREADS; ++k) {
            const int i = tid + k * SS_THREADS;
            const int tk = i / CH, j = i - tk * CH;
            const int col = min(blockIdx.y * CH + j, a.inner - 1);
            const bool ok = i < xz_items && tk < nt;
            pf_x[k] = ok ? to_float(xc[(size_t)(start + t0 + tk) * a.inner + col]) : 0.f;
            pf_z[k] = ok ? to_float(xz[(size_t)(start + t0 + tk) * a.ld_xz + a.inner + col]) : 0.f;
            pf_d[k] = (ok && a.dt_pre != nullptr) ? dt_pre[(size_t)(start + t0 + tk) * a.inner + col] : 0.f;
        }
    };
    auto stash = [&](float* buf) {
        cp_async_all_done();
#pragma unroll
        for (int k = 0; k < (xz_items + SS_THREADS - 1) / SS_THREADS; ++k) {
            const int i = tid + k * SS_THREADS;
            if (i < xz_items) {
                buf[row_items + i] = pf_x[k];
                buf[row_items + xz_items + i] = pf_z[k];
                buf[row_items + 2 * xz_items + i] = pf_d[k];
            }
        }
    };

    if (n_tok > 0) {
        fetch(sm, 0, min(SS_TC, n_tok));
        stash(sm);
    }
    __syncthreads();
    int which = 0;
    for (int t0 = 0; t0 < n_tok; t0 += SS_TC, which ^= 1) {
        const int nt = min(SS_TC, n_tok - t0);
        const bool more = t0 + SS_TC < n_tok;
        if (more) fetch(sm + (which ^ 1) * buf_floats, t0 + SS_TC, min(SS_TC, n_tok - t0 - SS_TC));
        const float* rows = sm + which * buf_floats;
        const float* xs = rows + row_items;
        const float* zs = xs + xz_items;
        const float* ds = zs + xz_items;
        if (nt < SS_TC) {
            // a short portion, or a portion's tail: token by token
            for (int k = 0; k < nt; ++k) {
                float d = 0.f;
                if (a.dt_pre != nullptr) {
                    d = ds[k * CH + ch];
                } else {
                    for (int r = sub; r < a.rank; r += LANES) d = fmaf(wrow[r], rows[k * row + r], d);
#pragma unroll
                    for (int o = LANES / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                }
                d = softplus_f(d + bias);
                dt_sum += d;
                const float x = xs[k * CH + ch];
                const float dx = d * x;
                const float* B = rows + k * row + a.rank;
                const float* C = B + a.n_state;
                float y = 0.f;
#pragma unroll
                for (int i = 0; i < NPER; ++i) {
                    const int n = sub + LANES * i;
                    if (n < a.n_state) {
                        S[i] = fmaf(exp2f(d * An[i]), S[i], dx * B[n]);
                        y = fmaf(S[i], C[n], y);
                    }
                }
#pragma unroll
                for (int o = LANES / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
                if (sub == 0 && live && a.pass != 1)
                    out[(size_t)(start + t0 + k) * a.inner + c] =
                        from_float<A>(fmaf(dsk, x, y) * silu_f(zs[k * CH + ch]));
            }
        } else {
            // step sizes of the chunk
            float dt[SS_TC];
            if (a.dt_pre != nullptr) {
                // the softplus of a channel's 16 step sizes is dealt out among its lanes (in
                // place in the staged values), not made by each of them
                float* dsw = sm + which * buf_floats + row_items + 2 * xz_items;
#pragma unroll
                for (int j = 0; j < SS_TC / LANES; ++j) {
                    const int k = sub + LANES * j;
                    dsw[k * CH + ch] = softplus_f(dsw[k * CH + ch] + bias);
                }
                __syncwarp();
#pragma unroll
                for (int k = 0; k < SS_TC; ++k) {
                    dt[k] = ds[k * CH + ch];
                    dt_sum += dt[k];
                }
            } else {
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
                    for (int o = LANES / 2; o > 0; o >>= 1)
                        dt[k] += __shfl_xor_sync(0xffffffffu, dt[k], o);
                }
#pragma unroll
                for (int k = 0; k < SS_TC; ++k) {
                    dt[k] = softplus_f(dt[k] + bias);
                    dt_sum += dt[k];
                }
            }
            // the chain, SUB tokens at a time: first everything that does not depend on the
            // state (decays exp(dt A), inputs dt x B), then one multiply-add per state and token
            // on the chain with the output sums beside it, then the sums of the lanes and the
            // gated outputs, the tokens dealt out among the lanes of a channel
            constexpr int SUB = NPER <= 1 ? SS_TC : (NPER <= 4 ? 8 : 2);
#pragma unroll
            for (int k0 = 0; k0 < SS_TC; k0 += SUB) {
                float da[SUB][NPER], db[SUB][NPER], yk[SUB];
#pragma unroll
                for (int kk = 0; kk < SUB; ++kk) {
                    const int k = k0 + kk;
                    const float dx = dt[k] * xs[k * CH + ch];
                    const float* B = rows + k * row + a.rank;
#pragma unroll
                    for (int i = 0; i < NPER; ++i) {
                        const int n = sub + LANES * i;
                        const bool use = n < a.n_state;
                        da[kk][i] = use ? exp2f(dt[k] * An[i]) : 1.f;
                        db[kk][i] = use ? dx * B[use ? n : 0] : 0.f;
                    }
                }
#pragma unroll
                for (int kk = 0; kk < SUB; ++kk) {
                    const float* C = rows + (k0 + kk) * row + a.rank + a.n_state;
                    float y = 0.f;
#pragma unroll
                    for (int i = 0; i < NPER; ++i) {
                        const int n = sub + LANES * i;
                        S[i] = fmaf(da[kk][i], S[i], db[kk][i]);
                        y = fmaf(S[i], n < a.n_state ? C[n] : 0.f, y);
                    }
                    yk[kk] = y;
                }
                if (a.pass != 1) {
#pragma unroll
                    for (int kk = 0; kk < SUB; ++kk) {
#pragma unroll
                        for (int o = LANES / 2; o > 0; o >>= 1)
                            yk[kk] += __shfl_xor_sync(0xffffffffu, yk[kk], o);
                    }
#pragma unroll
                    for (int kk = 0; kk < SUB; ++kk) {
                        const int k = k0 + kk;
                        if (kk % LANES == sub && live) {
                            const float y = fmaf(dsk, xs[k * CH + ch], yk[kk]);
                            out[(size_t)(start + t0 + k) * a.inner + c] =
                                from_float<A>(y * silu_f(zs[k * CH + ch]));
                        }
                    }
                }
            }
        }
        if (more) stash(sm + (which ^ 1) * buf_floats);
        __syncthreads();
    }
    if (!live) return;
    if (a.pass == 1) {                         // this piece alone, for the pieces after it
        const size_t at = (size_t)e * a.max_pieces + piece;
        float* E = a.piece_state + (at * a.inner + c) * a.n_state;
#pragma unroll
        for (int i = 0; i < NPER; ++i) {
            const int n = sub + LANES * i;
            if (n < a.n_state) E[n] = S[i];
        }
        if (sub == 0) a.piece_dt[at * a.inner + c] = dt_sum;
        return;
    }
    if (!last_piece) return;
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
        const int n = sub + LANES * i;
        if (n < a.n_state) s_slot[n] = S[i];
    }
    if (sub == 0 && e_tok > 0) {
        // the window of the convolution: the last taps-1 inputs of [old window | this portion]
        for (int j = 0; j < a.taps - 1; ++j) {
            const int at = e_tok + j;                  // index into the joined sequence
            slot[(size_t)j * a.inner + c] =
                at < a.taps - 1 ? slot[(size_t)at * a.inner + c]
                                : to_float(xz[(size_t)(e_start + at - (a.taps - 1)) * a.ld_xz + c]);
        }
    }
}

// xc: [tokens, inner] conv outputs; xz: [tokens] rows of ld_xz elements, x then z; proj: float
// [tokens, rank + 2 n_state]; w_dt float [inner, rank]; a_neg float [inner, n_state] = -exp(A_log);
// out [tokens, inner].  piece > 0: portions are cut into pieces of that many tokens (a multiple
// of the token chunk) that run side by side in two passes; max_pieces bounds the pieces of any
// entry, piece_state is float scratch [entries, max_pieces, inner, n_state], piece_dt
// [entries, max_pieces, inner].  dt_pre: nullptr, or float [tokens, inner] = dt_in W_dt^T made by
// the caller.  Returns 0, a CUDA error code, or -1 when the shape is refused.
MSTAR_API int mstar_selective_scan(const void* xc, const void* xz, int ld_xz, const float* proj,
                                   const float* w_dt, const float* dt_bias, const float* a_neg,
                                   const float* d_skip, const int* qo_indptr, const int* slots,
                                   float* state, long long state_stride, void* out, int act_dtype,
                                   int entries, int inner, int n_state, int rank, int taps,
                                   int piece, int max_pieces, float* piece_state, float* piece_dt,
                                   const float* dt_pre, void* stream) {
    if (entries <= 0) return 0;
    if (inner <= 0 || n_state <= 0 || rank <= 0 || taps <= 0 || n_state > 256) return -1;
    if (piece < 0 || (piece > 0 && (max_pieces < 1 || piece_state == nullptr || piece_dt == nullptr)))
        return -1;
    cudaStream_t s = (cudaStream_t)stream;
    ScanArgs a{inner, n_state, rank, taps, ld_xz, entries, state_stride, piece, 0,
               piece > 0 ? max_pieces : 1, piece_state, piece_dt, dt_pre};
#define GO(A, LANES, NPER)                                                                        \
    {                                                                                             \
        constexpr int CH = SS_THREADS / LANES;                                                    \
        const size_t smem = sizeof(float) * 2 * ((size_t)SS_TC * (rank + 2 * n_state) + 3 * SS_TC * CH); \
        if (smem > 200 * 1024) return -1;                                                         \
        static size_t configured = 0;                                                             \
        if (smem > 48 * 1024 && smem > configured) {                                              \
            cudaFuncSetAttribute(selective_scan_kernel<A, LANES, NPER>,                           \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
            configured = smem;                                                                    \
        }                                                                                         \
        dim3 grid(entries, (inner + CH - 1) / CH, a.max_pieces);                                  \
        for (int pass = (piece > 0 ? 1 : 0); pass <= (piece > 0 ? 2 : 0); ++pass) {               \
            a.pass = pass;                                                                        \
            mstar_launch((selective_scan_kernel<A, LANES, NPER>), grid, dim3(SS_THREADS), smem, s, \
                         (const A*)xc, (const A*)xz, proj, w_dt, dt_bias, a_neg, d_skip,          \
                         qo_indptr, slots, state, (A*)out, a);                                    \
        }                                                                                         \
    }
#define PICK(A)                                                                                   \
    if (n_state <= 4) GO(A, 4, 1)                                                                 \
    else if (n_state <= 16) GO(A, 4, 4)                                                           \
    else if (n_state <= 64) GO(A, 4, 16)                                                          \
    else GO(A, 16, 16)
    if (act_dtype == MSTAR_F32) { PICK(float) } else { PICK(bf16) }
#undef PICK
#undef GO
    return launch_status();
}
