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
// The scan walks a sequence token by token.  A block owns 32 value columns of one head of one
// batch entry; a column's `dim` state rows are spread over 8 lanes (row d on lane d % 8), so a
// step costs dim / 8 multiply-adds per thread and three shuffles, and a step's q, k, v and
// gates are staged in shared memory 16 tokens at a time.  The arithmetic of a token does not
// depend on how the sequence was cut into steps or on what else is in the batch.
//
// State slot layout (floats): S^T [heads][vdim][dim], then n [heads][dim], then m [heads].
//
// The second kernel finishes the cell: each head's output is divided by its root mean
// square, scaled by a weight and gated by sigmoid(g).
#include "common.cuh"

#define MM_COLS 32
#define MM_LANES 8
#define MM_THREADS (MM_COLS * MM_LANES)
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

template <typename A, int R>
__global__ void __launch_bounds__(MM_THREADS)
matrix_memory_scan_kernel(const A* __restrict__ qkv, const float* __restrict__ gates,
                          const float* __restrict__ bias, const int* __restrict__ qo_indptr,
                          const int* __restrict__ slots, float* __restrict__ state,
                          float* __restrict__ out, MemArgs a) {
    extern __shared__ float smem[];
    float* q_s = smem;                         // [CHUNK][dim]
    float* k_s = q_s + MM_CHUNK * a.dim;       // [CHUNK][dim]
    float* v_s = k_s + MM_CHUNK * a.dim;       // [CHUNK][COLS]
    float* i_s = v_s + MM_CHUNK * MM_COLS;     // [CHUNK]
    float* f_s = i_s + MM_CHUNK;               // [CHUNK]

    const int entry = blockIdx.z, head = blockIdx.y;
    const int tid = threadIdx.x, lane = tid % MM_LANES, colb = tid / MM_LANES;
    const int col = blockIdx.x * MM_COLS + colb;
    const bool col_ok = col < a.vdim;
    const int t0 = qo_indptr[entry], t1 = qo_indptr[entry + 1];
    // the state is an earlier step's, but the slot may have been zeroed just now: everything
    // but the step's index arrays is read after the wait
    const unsigned long long waited = pdl_wait();
    qkv = pdl_after(qkv, waited);
    gates = pdl_after(gates, waited);
    state = pdl_after(state, waited);
    float* slot = state + (size_t)slots[entry] * a.state_stride;
    float* S_g = slot + ((size_t)head * a.vdim + (col_ok ? col : 0)) * a.dim;
    float* n_g = slot + (size_t)a.heads * a.vdim * a.dim + (size_t)head * a.dim;
    float* m_g = n_g + (size_t)a.heads * a.dim - (size_t)head * a.dim + head;

    float S[R], n[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = lane + MM_LANES * r;
        S[r] = (col_ok && d < a.dim) ? S_g[d] : 0.f;
        n[r] = d < a.dim ? n_g[d] : 0.f;
    }
    float m = *m_g;

    for (int base = t0; base < t1; base += MM_CHUNK) {
        const int cnt = min(MM_CHUNK, t1 - base);
        __syncthreads();
        for (int idx = tid; idx < cnt * a.dim; idx += MM_THREADS) {
            const int t = idx / a.dim, d = idx - t * a.dim;
            const A* row = qkv + (size_t)(base + t) * a.ld + (size_t)head * a.dim + d;
            q_s[t * a.dim + d] = to_float(row[0]) * a.q_scale;
            k_s[t * a.dim + d] = to_float(row[a.k_off]);
        }
        for (int idx = tid; idx < cnt * MM_COLS; idx += MM_THREADS) {
            const int t = idx / MM_COLS, c = idx - t * MM_COLS;
            const int gc = blockIdx.x * MM_COLS + c;
            v_s[idx] = gc < a.vdim ? to_float(qkv[(size_t)(base + t) * a.ld + a.v_off +
                                                  (size_t)head * a.vdim + gc])
                                   : 0.f;
        }
        if (tid < cnt) {
            const float* g = gates + (size_t)(base + tid) * 2 * a.heads;
            i_s[tid] = soft_cap(g[head] + bias[head], a.cap);
            f_s[tid] = log_sigmoid(soft_cap(g[a.heads + head] + bias[a.heads + head], a.cap));
        }
        __syncthreads();
        for (int t = 0; t < cnt; ++t) {
            const float fg = f_s[t], ig = i_s[t];
            const float m_new = fmaxf(fg + m, ig);
            const float keep = expf(fg + m - m_new), take = expf(ig - m_new);
            m = m_new;
            const float tv = take * v_s[t * MM_COLS + colb];
            const float* kq = k_s + t * a.dim;
            const float* qq = q_s + t * a.dim;
            float num = 0.f, nq = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int d = lane + MM_LANES * r;
                if (d < a.dim) {
                    const float kd = kq[d], qd = qq[d];
                    S[r] = fmaf(keep, S[r], kd * tv);
                    n[r] = fmaf(keep, n[r], take * kd);
                    num = fmaf(S[r], qd, num);
                    nq = fmaf(n[r], qd, nq);
                }
            }
#pragma unroll
            for (int o = 1; o < MM_LANES; o <<= 1) {
                num += __shfl_xor_sync(0xffffffffu, num, o);
                nq += __shfl_xor_sync(0xffffffffu, nq, o);
            }
            if (lane == 0 && col_ok) {
                const float den = fmaxf(fabsf(nq), expf(-m)) + a.floor;
                out[(size_t)(base + t) * a.heads * a.vdim + (size_t)head * a.vdim + col] = num / den;
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = lane + MM_LANES * r;
        if (d < a.dim) {
            if (col_ok) S_g[d] = S[r];
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
    const size_t smem = sizeof(float) * ((size_t)2 * MM_CHUNK * dim + MM_CHUNK * MM_COLS + 2 * MM_CHUNK);
    dim3 grid((vdim + MM_COLS - 1) / MM_COLS, heads, entries);
#define LAUNCH(A, R)                                                                             \
    mstar_launch((matrix_memory_scan_kernel<A, R>), grid, dim3(MM_THREADS), smem, s, (const A*)qkv, \
                 gates, bias, qo_indptr, slots, state, out, a)
#define PICK(A)                                                                                  \
    if (dim <= 64) { LAUNCH(A, 8); }                                                             \
    else if (dim <= 128) { LAUNCH(A, 16); }                                                      \
    else if (dim <= 256) { LAUNCH(A, 32); }                                                      \
    else { LAUNCH(A, 64); }
    if (act_dtype == MSTAR_F32) { PICK(float) } else { PICK(bf16) }
#undef PICK
#undef LAUNCH
    return launch_status();
}

// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * weight[h, :] * sigmoid(gate[t, h, :]); one warp
// per (token, head), float sums.
template <typename A>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const A* __restrict__ gate, int ldg,
                                      const float* __restrict__ weight, A* __restrict__ out,
                                      int pairs, int heads, int vdim, float eps) {
    const unsigned long long waited = pdl_wait();
    o = pdl_after(o, waited);
    gate = pdl_after(gate, waited);
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= pairs) return;
    const int lane = threadIdx.x & 31;
    const int t = pair / heads, h = pair - t * heads;
    const float* row = o + (size_t)pair * vdim;
    float ss = 0.f;
    for (int j = lane; j < vdim; j += 32) ss = fmaf(row[j], row[j], ss);
    const float inv = rsqrtf(warp_sum(ss) / (float)vdim + eps);
    const A* g = gate + (size_t)t * ldg + (size_t)h * vdim;
    for (int j = lane; j < vdim; j += 32) {
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
    dim3 grid((pairs + warps - 1) / warps);
    if (act_dtype == MSTAR_F32)
        mstar_launch((head_norm_gate_kernel<float>), grid, dim3(32 * warps), 0, s, o, (const float*)gate,
                     ldg, weight, (float*)out, pairs, heads, vdim, eps);
    else
        mstar_launch((head_norm_gate_kernel<bf16>), grid, dim3(32 * warps), 0, s, o, (const bf16*)gate,
                     ldg, weight, (bf16*)out, pairs, heads, vdim, eps);
    return launch_status();
}
