// Matrix-memory recurrence (the mLSTM cell) for any mix of prompt portions and decoded
// tokens, carried in per-request state slots.
//
// Per head, with log input gate i_t and log forget gate f_t and a running maximum m (0 at
// the start of a sequence):
//     m_t = max(f_t + m_{t-1}, i_t)
//     S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T       [dim x vdim]
//     n_t = the same with k_t alone                                           [dim]
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + floor)
// The gates come in as float pre-activations z (a product's float output): i = cap *
// tanh((z_i + b_i) / cap), f = logsigmoid(cap * tanh((z_f + b_f) / cap)).  Everything of the
// recurrence is float: gates, decays, the state and the sums; q, k and v are read in the
// activation type as their products left them.
//
// The scan walks a sequence token by token.  A block owns 32 (or 8) value columns of one head of
// one batch entry; a column's `dim` state rows are spread over 8 lanes (row d on lane d % 8), so a
// step costs dim / 8 multiply-adds per thread and three shuffles; q, k, v and the gates come
// through shared memory 16 tokens at a time, the next 16 copied (cp.async) while these are
// walked.  The arithmetic of a token does not
// depend on how the sequence was cut into steps or on what else is in the batch.
//
// State slot layout (floats): S^T [heads][vdim][dim], then n [heads][dim], then m [heads].
//
// The second kernel finishes the cell: each head's output is divided by its root mean
// square, scaled by a weight and gated by sigmoid(g).
#include "common.cuh"
#include "mma_util.cuh"

#define MM_CHUNK 16

struct MemArgs {
    int heads, dim, vdim;
    int ld;              // elements between tokens of the q/k/v product
    int k_off, v_off;    // column of the first k / v feature (q starts at 0)
    float cap, q_scale, floor;
    long long state_stride;  // floats per slot
};

__device__ __forceinline__ float soft_cap(float z, float cap) { return cap * tanhf(z / cap); }
// log(sigmoid(x)) without overflow
__device__ __forceinline__ float log_sigmoid(float x) {
    return fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
}

// Copies `n` consecutive elements (n a multiple of the 16-byte vector) global -> shared.
template <typename A>
__device__ __forceinline__ void stage_vec(A* dst, const A* src, int n, int first, int step) {
    constexpr int V = 16 / (int)sizeof(A);
    for (int c = first; c < n / V; c += step) cp_async_16(smem_u32(dst + c * V), src + c * V, 16);
}

// MM_COLS x CT value columns a block (CT columns a thread), a column's rows on MM_LANES lanes.
template <typename A, int R, int MM_COLS, int MM_LANES, int CT>
__global__ void __launch_bounds__(MM_COLS * MM_LANES)
matrix_memory_scan_kernel(const A* __restrict__ qkv, const float* __restrict__ gates,
                          const float* __restrict__ bias, const int* __restrict__ qo_indptr,
                          const int* __restrict__ slots, float* __restrict__ state,
                          float* __restrict__ out, MemArgs a) {
    constexpr int MM_THREADS = MM_COLS * MM_LANES;
    constexpr int BCOLS = MM_COLS * CT;                   // columns of the block
    constexpr int V = 16 / (int)sizeof(A);
    // two stages of a chunk's q, k (this head) and v (this block's columns) as they are in
    // memory, and of its gates: the next chunk is copied while this one is walked
    extern __shared__ __align__(16) unsigned char smem_raw[];
    A* q_s = reinterpret_cast<A*>(smem_raw);              // [2][CHUNK][dim]
    A* k_s = q_s + 2 * MM_CHUNK * a.dim;                  // [2][CHUNK][dim]
    A* v_s = k_s + 2 * MM_CHUNK * a.dim;                  // [2][CHUNK][BCOLS]
    float* i_s = reinterpret_cast<float*>(v_s + 2 * MM_CHUNK * BCOLS);   // [2][CHUNK]
    float* f_s = i_s + 2 * MM_CHUNK;                      // [2][CHUNK]

    const int entry = blockIdx.z, head = blockIdx.y;
    const int tid = threadIdx.x, lane = tid % MM_LANES, colb = tid / MM_LANES;
    const int col0 = blockIdx.x * BCOLS;
    const int t0 = qo_indptr[entry], t1 = qo_indptr[entry + 1];
    // the state is an earlier step's, but the slot may have been zeroed just now: everything
    // but the step's index arrays is read after the wait
    const unsigned long long waited = pdl_wait();
    qkv = pdl_after(qkv, waited);
    gates = pdl_after(gates, waited);
    state = pdl_after(state, waited);
    float* slot = state + (size_t)slots[entry] * a.state_stride;
    float* n_g = slot + (size_t)a.heads * a.vdim * a.dim + (size_t)head * a.dim;
    float* m_g = n_g + (size_t)a.heads * a.dim - (size_t)head * a.dim + head;
    float* S_g[CT];
    bool col_ok[CT];
#pragma unroll
    for (int c = 0; c < CT; ++c) {
        const int col = col0 + colb * CT + c;
        col_ok[c] = col < a.vdim;
        S_g[c] = slot + ((size_t)head * a.vdim + (col_ok[c] ? col : 0)) * a.dim;
    }

    // 16-byte copies where rows and columns start on 16-byte boundaries, else element by element
    const bool base_ok = ((uintptr_t)qkv & 15) == 0 && a.ld % V == 0;
    const bool qk_vec = base_ok && a.dim % V == 0 && a.k_off % V == 0;
    const bool v_vec = base_ok && (a.v_off + head * a.vdim + col0) % V == 0 && col0 + BCOLS <= a.vdim &&
                       BCOLS % V == 0;

    auto stage = [&](int buf, int base, int cnt) {
        A* qd = q_s + buf * MM_CHUNK * a.dim;
        A* kd = k_s + buf * MM_CHUNK * a.dim;
        A* vd = v_s + buf * MM_CHUNK * BCOLS;
        if (qk_vec) {
            const int per = a.dim / V;
            for (int idx = tid; idx < cnt * per; idx += MM_THREADS) {
                const int t = idx / per, c = idx - t * per;
                const A* row = qkv + (size_t)(base + t) * a.ld + (size_t)head * a.dim + c * V;
                cp_async_16(smem_u32(qd + t * a.dim + c * V), row, 16);
                cp_async_16(smem_u32(kd + t * a.dim + c * V), row + a.k_off, 16);
            }
        } else {
            for (int idx = tid; idx < cnt * a.dim; idx += MM_THREADS) {
                const int t = idx / a.dim, d = idx - t * a.dim;
                const A* row = qkv + (size_t)(base + t) * a.ld + (size_t)head * a.dim + d;
                qd[idx] = row[0];
                kd[idx] = row[a.k_off];
            }
        }
        if (v_vec) {
            constexpr int per = BCOLS / V > 0 ? BCOLS / V : 1;
            for (int idx = tid; idx < cnt * per; idx += MM_THREADS) {
                const int t = idx / per, c = idx - t * per;
                cp_async_16(smem_u32(vd + t * BCOLS + c * V),
                            qkv + (size_t)(base + t) * a.ld + a.v_off + (size_t)head * a.vdim + col0 + c * V, 16);
            }
        } else {
            for (int idx = tid; idx < cnt * BCOLS; idx += MM_THREADS) {
                const int t = idx / BCOLS, c = idx - t * BCOLS;
                vd[idx] = col0 + c < a.vdim ? qkv[(size_t)(base + t) * a.ld + a.v_off +
                                                  (size_t)head * a.vdim + col0 + c]
                                            : from_float<A>(0.f);
            }
        }
    };
    auto gate_values = [&](float zi, float zf, float& ig, float& fg) {
        ig = soft_cap(zi + bias[head], a.cap);
        fg = log_sigmoid(soft_cap(zf + bias[a.heads + head], a.cap));
    };

    float S[CT][R], n[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = lane + MM_LANES * r;
#pragma unroll
        for (int c = 0; c < CT; ++c) S[c][r] = (col_ok[c] && d < a.dim) ? S_g[c][d] : 0.f;
        n[r] = d < a.dim ? n_g[d] : 0.f;
    }
    float m = *m_g;

    const int chunks = (t1 - t0 + MM_CHUNK - 1) / MM_CHUNK;
    stage(0, t0, min(MM_CHUNK, t1 - t0));
    cp_async_commit();
    if (tid < min(MM_CHUNK, t1 - t0)) {
        const float* g = gates + (size_t)(t0 + tid) * 2 * a.heads;
        gate_values(g[head], g[a.heads + head], i_s[tid], f_s[tid]);
    }
    for (int ch = 0; ch < chunks; ++ch) {
        const int buf = ch & 1, base = t0 + ch * MM_CHUNK;
        const int cnt = min(MM_CHUNK, t1 - base);
        const int cnt_next = min(MM_CHUNK, t1 - base - MM_CHUNK);     // <= 0 after the last chunk
        if (cnt_next > 0) stage(buf ^ 1, base + MM_CHUNK, cnt_next);
        cp_async_commit();
        float zi = 0.f, zf = 0.f;                      // the next chunk's gates: asked for now,
        if (tid < cnt_next) {                          // used after this chunk's tokens
            const float* g = gates + (size_t)(base + MM_CHUNK + tid) * 2 * a.heads;
            zi = g[head];
            zf = g[a.heads + head];
        }
        cp_async_wait<1>();
        __syncthreads();
        const A* kb = k_s + buf * MM_CHUNK * a.dim;
        const A* qb = q_s + buf * MM_CHUNK * a.dim;
        const A* vb = v_s + buf * MM_CHUNK * BCOLS;
        for (int t = 0; t < cnt; ++t) {
            const float fg = f_s[buf * MM_CHUNK + t], ig = i_s[buf * MM_CHUNK + t];
            const float m_new = fmaxf(fg + m, ig);
            const float keep = expf(fg + m - m_new), take = expf(ig - m_new);
            m = m_new;
            float v[CT], num[CT];
#pragma unroll
            for (int c = 0; c < CT; ++c) {
                v[c] = to_float(vb[t * BCOLS + colb * CT + c]);
                num[c] = 0.f;
            }
            const A* kq = kb + t * a.dim;
            const A* qq = qb + t * a.dim;
            float nq = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int d = lane + MM_LANES * r;
                if (d < a.dim) {
                    const float tk = take * to_float(kq[d]), qd = to_float(qq[d]);
                    n[r] = fmaf(keep, n[r], tk);
                    nq = fmaf(n[r], qd, nq);
#pragma unroll
                    for (int c = 0; c < CT; ++c) {
                        S[c][r] = fmaf(keep, S[c][r], tk * v[c]);
                        num[c] = fmaf(S[c][r], qd, num[c]);
                    }
                }
            }
#pragma unroll
            for (int o = 1; o < MM_LANES; o <<= 1) {
                nq += __shfl_xor_sync(0xffffffffu, nq, o);
#pragma unroll
                for (int c = 0; c < CT; ++c) num[c] += __shfl_xor_sync(0xffffffffu, num[c], o);
            }
            if (lane == 0) {
                // q carries the scale dim^-1/2: applied to the sums instead of to every q
                const float den = fmaxf(fabsf(nq * a.q_scale), expf(-m)) + a.floor;
                float* orow = out + (size_t)(base + t) * a.heads * a.vdim + (size_t)head * a.vdim +
                              col0 + colb * CT;
#pragma unroll
                for (int c = 0; c < CT; ++c)
                    if (col_ok[c]) orow[c] = num[c] * a.q_scale / den;
            }
        }
        if (tid < cnt_next)
            gate_values(zi, zf, i_s[(buf ^ 1) * MM_CHUNK + tid], f_s[(buf ^ 1) * MM_CHUNK + tid]);
        __syncthreads();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = lane + MM_LANES * r;
        if (d < a.dim) {
#pragma unroll
            for (int c = 0; c < CT; ++c)
                if (col_ok[c]) S_g[c][d] = S[c][r];
            if (blockIdx.x == 0 && colb == 0) n_g[d] = n[r];
        }
    }
    if (blockIdx.x == 0 && tid == 0) *m_g = m;
}

// Returns 0, a CUDA error code, or -1 when the shape is refused (dim > 512).
MSTAR_API int mstar_matrix_memory_scan(const void* qkv, int act_dtype, int ld, int k_off, int v_off,
                                       const float* gates, const float* bias,
                                       const int* qo_indptr, const int* slots, float* state,
                                       long long state_stride, float* out, int entries, int heads,
                                       int dim, int vdim, float cap, float q_scale, float floor,
                                       void* stream) {
    if (entries <= 0) return 0;
    if (heads <= 0 || dim <= 0 || vdim <= 0 || dim > 512) return -1;
    if (state_stride < (long long)heads * ((long long)dim * vdim + dim + 1)) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    MemArgs a{heads, dim, vdim, ld, k_off, v_off, cap, q_scale, floor, state_stride};
    // Where the batch fills the GPU twice over: 32 columns a block, a column's rows on 8 lanes.
    // Else (a few long sequences): 8 columns a block and a whole warp per column, so that the
    // chains spread over four times as many SMs, a step is a quarter of the instructions, and
    // the eight warps of a block hide one another's latencies.  (Four columns a thread, which
    // share the loads of q and k and the sums of n, were tried there: a third of the
    // instructions per column, but a quarter of the blocks, and 1.70 instead of 1.49 ms for a
    // prompt of 2,048 tokens at 4 heads of 256 x 512: what counts is the latency of a token's
    // chain and how many warps there are to hide it.)
    const bool wide = (long long)((vdim + 31) / 32) * heads * entries >= 2LL * device_sm_count();
    const int cols = wide ? 32 : 8;
    const size_t elem = act_dtype == MSTAR_F32 ? 4 : 2;
    const size_t smem = 2 * elem * ((size_t)2 * MM_CHUNK * dim + MM_CHUNK * cols) + sizeof(float) * 4 * MM_CHUNK;
    dim3 grid((vdim + cols - 1) / cols, heads, entries);
#define LAUNCH(A, R, C, L, CT)                                                                   \
    {                                                                                            \
        static size_t configured = 0; /* largest dynamic shared memory set so far */             \
        if (smem > 48 * 1024 && smem > configured) {                                             \
            cudaFuncSetAttribute(matrix_memory_scan_kernel<A, R, C, L, CT>,                      \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
            configured = smem;                                                                   \
        }                                                                                        \
        mstar_launch((matrix_memory_scan_kernel<A, R, C, L, CT>), grid, dim3(C * L), smem, s,    \
                     (const A*)qkv, gates, bias, qo_indptr, slots, state, out, a);               \
    }
#define PICK(A, C, L, CT)                                                                        \
    if (dim <= 64) { LAUNCH(A, 64 / L, C, L, CT); }                                              \
    else if (dim <= 128) { LAUNCH(A, 128 / L, C, L, CT); }                                       \
    else if (dim <= 256) { LAUNCH(A, 256 / L, C, L, CT); }                                       \
    else { LAUNCH(A, 512 / L, C, L, CT); }
    if (act_dtype == MSTAR_F32) {
        if (wide) { PICK(float, 32, 8, 1) } else { PICK(float, 8, 32, 1) }
    } else {
        if (wide) { PICK(bf16, 32, 8, 1) } else { PICK(bf16, 8, 32, 1) }
    }
#undef PICK
#undef LAUNCH
    return launch_status();
}

// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * weight[h, :] * sigmoid(gate[t, h, :]); one warp
// per (token, head) where there are many, a block of four warps where there are few; float sums.
template <typename A, bool BLOCK>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const A* __restrict__ gate, int ldg,
                                      const float* __restrict__ weight, A* __restrict__ out,
                                      int pairs, int heads, int vdim, float eps) {
    __shared__ float scratch[32];
    const unsigned long long waited = pdl_wait();
    o = pdl_after(o, waited);
    gate = pdl_after(gate, waited);
    const int pair = BLOCK ? blockIdx.x : blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= pairs) return;
    const int first = BLOCK ? threadIdx.x : (threadIdx.x & 31), step = BLOCK ? blockDim.x : 32;
    const int t = pair / heads, h = pair - t * heads;
    const float* row = o + (size_t)pair * vdim;
    float ss = 0.f;
    for (int j = first; j < vdim; j += step) ss = fmaf(row[j], row[j], ss);
    const float total = BLOCK ? block_sum(ss, scratch) : warp_sum(ss);
    const float inv = rsqrtf(total / (float)vdim + eps);
    const A* g = gate + (size_t)t * ldg + (size_t)h * vdim;
    for (int j = first; j < vdim; j += step) {
        const float gv = to_float(g[j]);
        out[(size_t)pair * vdim + j] =
            from_float<A>(row[j] * inv * weight[(size_t)h * vdim + j] / (1.f + expf(-gv)));
    }
}

MSTAR_API int mstar_head_norm_gate(const float* o, const void* gate, int ldg, const float* weight,
                                   void* out, int act_dtype, int tokens, int heads, int vdim,
                                   float eps, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int pairs = tokens * heads, warps = 4;
    const bool few = pairs < 4 * device_sm_count();
    dim3 grid(few ? pairs : (pairs + warps - 1) / warps);
#define LAUNCH(A, B)                                                                              \
    mstar_launch((head_norm_gate_kernel<A, B>), grid, dim3(32 * warps), 0, s, o, (const A*)gate, ldg, \
                 weight, (A*)out, pairs, heads, vdim, eps)
    if (act_dtype == MSTAR_F32) {
        if (few) LAUNCH(float, true); else LAUNCH(float, false);
    } else {
        if (few) LAUNCH(bf16, true); else LAUNCH(bf16, false);
    }
#undef LAUNCH
    return launch_status();
}
