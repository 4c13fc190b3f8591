// Routed experts: choosing the experts of a token, and the experts' gated feed-forwards on
// the rows that chose them.
//
//   scores  s = sigmoid(z) or softmax(z) over a token's float router logits z
//   chosen  the `top` largest scores (the lower index wins a tie), weight w = s, or s divided
//           by the sum of the chosen scores when `renormalize`
//   expert  y = W_down (silu(W_gate u) * (W_up u)),  u = w x (`scale_input`) or u = x with
//           w multiplying y
//   out[t] = sum over the chosen experts (+ `add[t]`, the shared expert's output)
//
// Expert matrices are stacked expert after expert: gate_up [experts][2 * ff][width] (gate
// rows first), down [experts][width][ff].
//
// These are the kernels for a step's rows as they come (token by token, each row streaming
// the weights of its experts): dot products on CUDA cores, float sums in a fixed order, so a
// row's result does not depend on what else is in the batch.  Scaling the input by w is done
// on the sums (W (w x) = w (W x)), which is the same number without rounding w x first.
#include "common.cuh"

// ------------------------------------------------------------------ choice
__global__ void route_topk_kernel(const float* __restrict__ logits, int* __restrict__ chosen,
                                  float* __restrict__ weight, int tokens, int experts, int top,
                                  int softmax, int renormalize) {
    logits = pdl_after(logits, pdl_wait());
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tokens) return;
    const float* z = logits + (size_t)t * experts;
    float zmax = -INFINITY, denom = 1.f;
    if (softmax) {
        for (int e = 0; e < experts; ++e) zmax = fmaxf(zmax, z[e]);
        denom = 0.f;
        for (int e = 0; e < experts; ++e) denom += expf(z[e] - zmax);
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        // the largest logit not chosen yet: scores are monotone in the logits
        int best = -1;
        float bz = -INFINITY;
        for (int e = 0; e < experts; ++e) {
            bool taken = false;
            for (int j = 0; j < k; ++j) taken |= chosen[(size_t)t * top + j] == e;
            if (!taken && (best < 0 || z[e] > bz)) {
                best = e;
                bz = z[e];
            }
        }
        const float s = softmax ? expf(bz - zmax) / denom : 1.f / (1.f + expf(-bz));
        chosen[(size_t)t * top + k] = best;
        weight[(size_t)t * top + k] = s;
        total += s;
    }
    if (renormalize)
        for (int k = 0; k < top; ++k) weight[(size_t)t * top + k] /= total;
}

MSTAR_API int mstar_route_topk(const float* logits, int* chosen, float* weight, int tokens,
                               int experts, int top, int softmax, int renormalize, void* stream) {
    if (tokens <= 0) return 0;
    if (experts <= 0 || top <= 0 || top > experts) return -1;
    mstar_launch(route_topk_kernel, dim3((tokens + 127) / 128), dim3(128), 0, (cudaStream_t)stream,
                 logits, chosen, weight, tokens, experts, top, softmax, renormalize);
    return launch_status();
}

// ------------------------------------------------------------------ gate / up
// One block per (row = token x choice, slice of 32 hidden units); a warp per hidden unit,
// lanes along the width.
#define RE_THREADS 256
#define RE_UNITS 32

template <typename A>
__global__ void __launch_bounds__(RE_THREADS)
expert_gate_up_kernel(const A* __restrict__ x, const A* __restrict__ w_gate_up,
                      const int* __restrict__ chosen, const float* __restrict__ weight,
                      float* __restrict__ act, int width, int ff, int top, int scale_input) {
    extern __shared__ float xs[];            // [width]
    const int row = blockIdx.x, t = row / top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned long long waited = pdl_wait();
    x = pdl_after(x, waited);
    chosen = pdl_after(chosen, waited);
    weight = pdl_after(weight, waited);
    for (int i = threadIdx.x; i < width; i += RE_THREADS) xs[i] = to_float(x[(size_t)t * width + i]);
    __syncthreads();
    const int e = chosen[row];
    const float w = scale_input ? weight[row] : 1.f;
    const A* base = w_gate_up + (size_t)e * 2 * ff * width;
    for (int u = blockIdx.y * RE_UNITS + warp; u < min(ff, (int)(blockIdx.y + 1) * RE_UNITS);
         u += RE_THREADS / 32) {
        const A* g = base + (size_t)u * width;
        const A* p = base + (size_t)(ff + u) * width;
        float sg = 0.f, su = 0.f;
        for (int i = lane; i < width; i += 32) {
            sg = fmaf(to_float(g[i]), xs[i], sg);
            su = fmaf(to_float(p[i]), xs[i], su);
        }
        sg = warp_sum(sg) * w;
        su = warp_sum(su) * w;
        if (lane == 0) act[(size_t)row * ff + u] = sg / (1.f + expf(-sg)) * su;
    }
}

// ------------------------------------------------------------------ down (+ sum, + shared)
template <typename A>
__global__ void __launch_bounds__(RE_THREADS)
expert_down_kernel(const float* __restrict__ act, const A* __restrict__ w_down,
                   const int* __restrict__ chosen, const float* __restrict__ weight,
                   const A* __restrict__ add, A* __restrict__ out, int width, int ff, int top,
                   int scale_input) {
    extern __shared__ float as[];            // [top][ff]
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned long long waited = pdl_wait();
    act = pdl_after(act, waited);
    add = pdl_after(add, waited);
    for (int i = threadIdx.x; i < top * ff; i += RE_THREADS) as[i] = act[(size_t)t * top * ff + i];
    __syncthreads();
    for (int c = blockIdx.y * RE_UNITS + warp; c < min(width, (int)(blockIdx.y + 1) * RE_UNITS);
         c += RE_THREADS / 32) {
        float total = 0.f;
        for (int k = 0; k < top; ++k) {
            const int e = chosen[(size_t)t * top + k];
            const A* wrow = w_down + ((size_t)e * width + c) * ff;
            float s = 0.f;
            for (int j = lane; j < ff; j += 32) s = fmaf(to_float(wrow[j]), as[k * ff + j], s);
            s = warp_sum(s);
            total += scale_input ? s : s * weight[(size_t)t * top + k];
        }
        if (lane == 0) {
            if (add != nullptr) total += to_float(add[(size_t)t * width + c]);
            out[(size_t)t * width + c] = from_float<A>(total);
        }
    }
}

// x [tokens, width], chosen / weight [tokens, top]; `act`: float scratch [tokens * top, ff];
// `add`: nullptr or [tokens, width]; out [tokens, width].  Returns 0, a CUDA error code, or
// -1 when a row does not fit shared memory.
MSTAR_API int mstar_experts_by_row(const void* x, const void* w_gate_up, const void* w_down,
                                   const int* chosen, const float* weight, float* act,
                                   const void* add, void* out, int act_dtype, int tokens,
                                   int width, int ff, int top, int scale_input, void* stream) {
    if (tokens <= 0) return 0;
    if (width <= 0 || ff <= 0 || top <= 0) return -1;
    if ((size_t)width * 4 > 48 * 1024 || (size_t)top * ff * 4 > 48 * 1024) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 g1(tokens * top, (ff + RE_UNITS - 1) / RE_UNITS), g2(tokens, (width + RE_UNITS - 1) / RE_UNITS);
    if (act_dtype == MSTAR_F32) {
        mstar_launch((expert_gate_up_kernel<float>), g1, dim3(RE_THREADS), sizeof(float) * width, s,
                     (const float*)x, (const float*)w_gate_up, chosen, weight, act, width, ff, top,
                     scale_input);
        mstar_launch((expert_down_kernel<float>), g2, dim3(RE_THREADS), sizeof(float) * top * ff, s,
                     (const float*)act, (const float*)w_down, chosen, weight, (const float*)add,
                     (float*)out, width, ff, top, scale_input);
    } else {
        mstar_launch((expert_gate_up_kernel<bf16>), g1, dim3(RE_THREADS), sizeof(float) * width, s,
                     (const bf16*)x, (const bf16*)w_gate_up, chosen, weight, act, width, ff, top,
                     scale_input);
        mstar_launch((expert_down_kernel<bf16>), g2, dim3(RE_THREADS), sizeof(float) * top * ff, s,
                     (const float*)act, (const bf16*)w_down, chosen, weight, (const bf16*)add,
                     (bf16*)out, width, ff, top, scale_input);
    }
    return launch_status();
}
