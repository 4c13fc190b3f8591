// Routed experts: choosing the experts of a token, and the experts' gated feed-forwards on
// the rows that chose them.
//
//   scores  s = sigmoid(z) or softmax(z) over a token's float router logits z
//   chosen  the `top` largest scores (the lower index wins a tie), weight w = s, or s divided
//           by the sum of the chosen scores when `renormalize`
//           With a `choice_bias` the largest of s + bias are chosen; the weights stay s.
//   expert  y = W_down (silu(W_gate u) * (W_up u)),  u = w x (`scale_input`) or u = x with
//           w multiplying y; without a gate (`gated` 0) y = W_down relu(W_up u)^2
//   out[t] = sum over the chosen experts (+ `add[t]`, the shared expert's output)
// A chosen index at or beyond `real` (the experts that have matrices) is an identity
// expert: it adds w x[t].
//
// Expert matrices are stacked expert after expert: gate_up [experts][2 * ff][width] (gate
// rows first; [experts][ff][width] without a gate), down [experts][width][ff].
//
// These are the kernels for a step's rows as they come (token by token, each row streaming
// the weights of its experts): dot products on CUDA cores, float sums in a fixed order, so a
// row's result does not depend on what else is in the batch.  Scaling the input by w is done
// on the sums (W (w x) = w (W x)), which is the same number without rounding w x first.
#include "common.cuh"

// ------------------------------------------------------------------ choice
// A warp per token: lane l holds the logits of experts l, l + 32, ... (up to 32 of them, so up
// to 1,024 experts); the largest logit not chosen yet is found `top` times by a warp-wide
// comparison of (value, index), the lower index winning a tie.  Scores are monotone in the
// logits, so the choice is made on the logits.
#define RT_PER_LANE 32

__global__ void route_topk_kernel(const float* __restrict__ logits, const float* __restrict__ choice_bias,
                                  int* __restrict__ chosen,
                                  float* __restrict__ weight, int tokens, int experts, int top,
                                  int softmax, int renormalize) {
    logits = pdl_after(logits, pdl_wait());
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= tokens) return;
    const float* z = logits + (size_t)t * experts;
    float zmax = -INFINITY, denom = 1.f;
    if (softmax) {
        for (int e = lane; e < experts; e += 32) zmax = fmaxf(zmax, z[e]);
        zmax = warp_max(zmax);
        denom = 0.f;
        for (int e = lane; e < experts; e += 32) denom += expf(z[e] - zmax);
        denom = warp_sum(denom);
    }
    unsigned taken = 0u;                       // bit i: expert lane + 32 i is chosen
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float bz = -INFINITY;
        int be = 0x7fffffff;
        for (int i = 0; i < RT_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e >= experts) break;
            if (!((taken >> i) & 1u)) {
                // scores are monotone in the logits; with a bias the choice needs the scores
                float v = z[e];
                if (choice_bias != nullptr)
                    v = (softmax ? expf(v - zmax) / denom : 1.f / (1.f + expf(-v))) + choice_bias[e];
                if (be == 0x7fffffff || v > bz) {
                    bz = v;
                    be = e;
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float oz = __shfl_xor_sync(0xffffffffu, bz, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (oe != 0x7fffffff && (be == 0x7fffffff || oz > bz || (oz == bz && oe < be))) {
                bz = oz;
                be = oe;
            }
        }
        if ((be & 31) == lane) taken |= 1u << (be >> 5);
        const float zb = z[be];
        const float s = softmax ? expf(zb - zmax) / denom : 1.f / (1.f + expf(-zb));
        total += s;
        if (lane == 0) {
            chosen[(size_t)t * top + k] = be;
            weight[(size_t)t * top + k] = s;
        }
    }
    if (renormalize && lane == 0)
        for (int k = 0; k < top; ++k) weight[(size_t)t * top + k] /= total;
}

MSTAR_API int mstar_route_topk(const float* logits, const float* choice_bias, int* chosen,
                               float* weight, int tokens, int experts, int top, int softmax,
                               int renormalize, void* stream) {
    if (tokens <= 0) return 0;
    if (experts <= 0 || top <= 0 || top > experts || experts > 32 * RT_PER_LANE) return -1;
    mstar_launch(route_topk_kernel, dim3((tokens + 3) / 4), dim3(128), 0, (cudaStream_t)stream,
                 logits, choice_bias, chosen, weight, tokens, experts, top, softmax, renormalize);
    return launch_status();
}

// ------------------------------------------------------------------ gate / up
// One block per (row = token x choice, slice of 32 hidden units); a warp per hidden unit,
// lanes along the width.
#define RE_THREADS 256
#define RE_UNITS 32

template <typename A, bool GATED>
__global__ void __launch_bounds__(RE_THREADS)
expert_gate_up_kernel(const A* __restrict__ x, const A* __restrict__ w_gate_up,
                      const int* __restrict__ chosen, const float* __restrict__ weight,
                      float* __restrict__ act, int width, int ff, int top, int scale_input,
                      int real) {
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
    if (e >= real) return;                     // an identity expert has no hidden units
    const float w = scale_input ? weight[row] : 1.f;
    const A* base = w_gate_up + (size_t)e * (GATED ? 2 : 1) * ff * width;
    // rows start at multiples of `width` elements: 8-element loads where that is aligned
    const bool vec = width % 8 == 0 && ((uintptr_t)w_gate_up & 31) == 0;
    // a warp takes four hidden units at a time: eight rows of weights stream side by side
    const int u_end = min(ff, (int)(blockIdx.y + 1) * RE_UNITS);
    for (int u0 = blockIdx.y * RE_UNITS + warp * 4; u0 < u_end; u0 += (RE_THREADS / 32) * 4) {
        float sg[4] = {0.f, 0.f, 0.f, 0.f}, su[4] = {0.f, 0.f, 0.f, 0.f};
        if (vec) {
            for (int c = lane; c < (width >> 3); c += 32) {
                float a8[4][8], b8[4][8];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int u = min(u0 + k, ff - 1);          // a unit past the end repeats the last
                    load8(base + (size_t)u * width + 8 * c, a8[k]);
                    if (GATED) load8(base + (size_t)(ff + u) * width + 8 * c, b8[k]);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float xv = xs[8 * c + i];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        sg[k] = fmaf(a8[k][i], xv, sg[k]);
                        if (GATED) su[k] = fmaf(b8[k][i], xv, su[k]);
                    }
                }
            }
        } else {
            for (int i = lane; i < width; i += 32) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int u = min(u0 + k, ff - 1);
                    sg[k] = fmaf(to_float(base[(size_t)u * width + i]), xs[i], sg[k]);
                    if (GATED) su[k] = fmaf(to_float(base[(size_t)(ff + u) * width + i]), xs[i], su[k]);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float g = warp_sum(sg[k]) * w;
            float v;
            if (GATED) {
                const float up = warp_sum(su[k]) * w;
                v = g / (1.f + expf(-g)) * up;
            } else {
                const float r = fmaxf(g, 0.f);
                v = r * r;
            }
            if (lane == 0 && u0 + k < u_end) act[(size_t)row * ff + u0 + k] = v;
        }
    }
}

// ------------------------------------------------------------------ down (+ sum, + shared)
template <typename A>
__global__ void __launch_bounds__(RE_THREADS)
expert_down_kernel(const float* __restrict__ act, const A* __restrict__ w_down,
                   const int* __restrict__ chosen, const float* __restrict__ weight,
                   const A* __restrict__ add, A* __restrict__ out, int width, int ff, int top,
                   int scale_input, const A* __restrict__ x, int real) {
    extern __shared__ float as[];            // [top][ff]
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned long long waited = pdl_wait();
    act = pdl_after(act, waited);
    add = pdl_after(add, waited);
    x = pdl_after(x, waited);
    for (int i = threadIdx.x; i < top * ff; i += RE_THREADS)
        as[i] = chosen[(size_t)t * top + i / ff] < real ? act[(size_t)t * top * ff + i] : 0.f;
    __syncthreads();
    const bool vec = ff % 8 == 0 && ((uintptr_t)w_down & 31) == 0;
    const int c_end = min(width, (int)(blockIdx.y + 1) * RE_UNITS);
    for (int c0 = blockIdx.y * RE_UNITS + warp * 4; c0 < c_end; c0 += (RE_THREADS / 32) * 4) {
        float total[4] = {0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < top; ++k) {
            const int e = chosen[(size_t)t * top + k];
            if (e >= real) {                   // identity expert: w x[t]
                const float wk = weight[(size_t)t * top + k];
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    total[q] += wk * to_float(x[(size_t)t * width + min(c0 + q, width - 1)]);
                continue;
            }
            const A* wexp = w_down + (size_t)e * width * ff;
            float s4[4] = {0.f, 0.f, 0.f, 0.f};
            if (vec) {
                for (int c2 = lane; c2 < (ff >> 3); c2 += 32) {
                    float a8[4][8];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        load8(wexp + (size_t)min(c0 + q, width - 1) * ff + 8 * c2, a8[q]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float av = as[k * ff + 8 * c2 + i];
#pragma unroll
                        for (int q = 0; q < 4; ++q) s4[q] = fmaf(a8[q][i], av, s4[q]);
                    }
                }
            } else {
                for (int j = lane; j < ff; j += 32) {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        s4[q] = fmaf(to_float(wexp[(size_t)min(c0 + q, width - 1) * ff + j]), as[k * ff + j], s4[q]);
                }
            }
            const float wk = scale_input ? 1.f : weight[(size_t)t * top + k];
#pragma unroll
            for (int q = 0; q < 4; ++q) total[q] += warp_sum(s4[q]) * wk;
        }
        if (lane == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int c = c0 + q;
                if (c < c_end) {
                    float v = total[q];
                    if (add != nullptr) v += to_float(add[(size_t)t * width + c]);
                    out[(size_t)t * width + c] = from_float<A>(v);
                }
            }
        }
    }
}

// x [tokens, width], chosen / weight [tokens, top]; `act`: float scratch [tokens * top, ff];
// `add`: nullptr or [tokens, width]; out [tokens, width].  Returns 0, a CUDA error code, or
// -1 when a row does not fit shared memory.
MSTAR_API int mstar_experts_by_row(const void* x, const void* w_gate_up, const void* w_down,
                                   const int* chosen, const float* weight, float* act,
                                   const void* add, void* out, int act_dtype, int tokens,
                                   int width, int ff, int top, int scale_input, int gated,
                                   int real, void* stream) {
    if (tokens <= 0) return 0;
    if (width <= 0 || ff <= 0 || top <= 0) return -1;
    if ((size_t)width * 4 > 48 * 1024 || (size_t)top * ff * 4 > 48 * 1024) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 g1(tokens * top, (ff + RE_UNITS - 1) / RE_UNITS), g2(tokens, (width + RE_UNITS - 1) / RE_UNITS);
#define GO(A, GATED)                                                                              \
    mstar_launch((expert_gate_up_kernel<A, GATED>), g1, dim3(RE_THREADS), sizeof(float) * width, s, \
                 (const A*)x, (const A*)w_gate_up, chosen, weight, act, width, ff, top,            \
                 scale_input, real)
    if (act_dtype == MSTAR_F32) {
        if (gated) { GO(float, true); } else { GO(float, false); }
        mstar_launch((expert_down_kernel<float>), g2, dim3(RE_THREADS), sizeof(float) * top * ff, s,
                     (const float*)act, (const float*)w_down, chosen, weight, (const float*)add,
                     (float*)out, width, ff, top, scale_input, (const float*)x, real);
    } else {
        if (gated) { GO(bf16, true); } else { GO(bf16, false); }
        mstar_launch((expert_down_kernel<bf16>), g2, dim3(RE_THREADS), sizeof(float) * top * ff, s,
                     (const float*)act, (const bf16*)w_down, chosen, weight, (const bf16*)add,
                     (bf16*)out, width, ff, top, scale_input, (const bf16*)x, real);
    }
#undef GO
    return launch_status();
}

// ====================================================================== grouped by expert
// For many rows (prompt portions) the rows are sorted by expert, and every expert's rows go
// through its matrices as tiles of a tensor-core GEMM (bfloat16 mma.sync, float sums):
//   1. experts_sort: counting sort of the rows (token x choice) by expert; the list of row
//      tiles (expert, first sorted row), one per 64 (or 128) rows of a group.
//   2. grouped GEMM, gated: act[p] = silu(w G) * (w U), G and U the products of the gathered
//      token rows with the expert's gate and up rows (bfloat16 out, sorted order).
//   3. grouped GEMM, plain: y[p] = act[p] W_down[e]^T (float out, sorted order).
//   4. experts_combine: out[t] = sum over a token's choices, in the order of the choices,
//      of (w) y[pos] (+ add[t]).
// A row's numbers depend on its own inputs only: the position of a row in its tile changes
// nothing, so the order inside a group need not be stable.
#include "mma_util.cuh"

#define GG_BN 64
#define GG_BK 32
#define GG_LD 40          // bf16 elements between rows of a shared tile (80 bytes: no bank conflicts)
#define GG_STAGES 3

// `experts`: all router outputs; tiles are made for the first `real` of them only.
__global__ void experts_sort_kernel(const int* __restrict__ chosen, int rows, int experts, int real, int tile_rows,
                                    int* __restrict__ order, int* __restrict__ pos,
                                    int* __restrict__ offsets, int* __restrict__ tile_expert,
                                    int* __restrict__ tile_first, int* __restrict__ num_tiles) {
    extern __shared__ int sh[];               // counts[experts], cursor[experts]
    int* counts = sh;
    int* cursor = sh + experts;
    chosen = pdl_after(chosen, pdl_wait());
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int r = threadIdx.x; r < rows; r += blockDim.x) atomicAdd(&counts[chosen[r]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < experts; ++e) {
            offsets[e] = at;
            cursor[e] = at;
            for (int p = at; e < real && p < at + counts[e]; p += tile_rows) {
                tile_expert[tiles] = e;
                tile_first[tiles] = p;
                ++tiles;
            }
            at += counts[e];
        }
        offsets[experts] = at;
        *num_tiles = tiles;
    }
    __syncthreads();
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
        const int p = atomicAdd(&cursor[chosen[r]], 1);
        order[p] = r;
        pos[r] = p;
    }
}

// C tile [GG_BM x 64] of one expert's group (a warp per 32 x 32 of it).  GATED: A rows are x[order[p] / top], B rows are
// the expert's gate rows n0.. and up rows ff + n0..; out = silu(w G) * (w U) as bfloat16.
// Plain: A rows are act[p], B rows the expert's down rows n0..; out float.
// MODE 0: plain (down), 1: gated gate/up with SiLU, 2: up alone with relu^2 (A rows gathered
// like the gated form, one block of B rows, bfloat16 out).
template <int MODE, int GG_BM>
__global__ void __launch_bounds__(GG_BM * 2)
grouped_gemm_kernel(const bf16* __restrict__ a_src, const bf16* __restrict__ w, void* __restrict__ out,
                    const int* __restrict__ order, const float* __restrict__ weight,
                    const int* __restrict__ offsets, const int* __restrict__ tile_expert,
                    const int* __restrict__ tile_first, const int* __restrict__ num_tiles,
                    int N, int K, int top, int scale_input) {
    constexpr bool GATED = MODE == 1;
    constexpr bool GATHER = MODE != 0;
    constexpr int BROWS = GATED ? 2 * GG_BN : GG_BN;
    constexpr int GG_THREADS = GG_BM * 2;             // a warp per 32 x 32 of the tile
    extern __shared__ __align__(16) unsigned char gg_smem[];
    bf16 (*As)[GG_BM * GG_LD] = reinterpret_cast<bf16 (*)[GG_BM * GG_LD]>(gg_smem);
    bf16 (*Bs)[BROWS * GG_LD] = reinterpret_cast<bf16 (*)[BROWS * GG_LD]>(
        gg_smem + sizeof(bf16) * GG_STAGES * GG_BM * GG_LD);
    int* src_row = reinterpret_cast<int*>(gg_smem + sizeof(bf16) * GG_STAGES * (GG_BM + BROWS) * GG_LD);

    const unsigned long long waited = pdl_wait();
    a_src = pdl_after(a_src, waited);
    order = pdl_after(order, waited);
    num_tiles = pdl_after(num_tiles, waited);
    if ((int)blockIdx.y >= *num_tiles) return;
    const int e = tile_expert[blockIdx.y], p0 = tile_first[blockIdx.y];
    const int p_end = offsets[e + 1];
    const int n0 = blockIdx.x * GG_BN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;

    if (tid < GG_BM) {
        const int p = p0 + tid;
        src_row[tid] = p < p_end ? (GATHER ? order[p] / top : p) : -1;
    }
    __syncthreads();
    const bf16* wbase = w + (size_t)e * (GATED ? 2 : 1) * N * K;

    auto load_stage = [&](int stage, int k0) {
        // A: 64 rows x 4 chunks of 8
        for (int c = tid; c < GG_BM * 4; c += GG_THREADS) {
            const int r = c >> 2, kc = (c & 3) * 8;
            const int src = src_row[r];
            const bool ok = src >= 0 && k0 + kc < K;
            const bf16* g = a_src + (ok ? (size_t)src * K + k0 + kc : 0);
            cp_async_16(smem_u32(&As[stage][r * GG_LD + kc]), g, ok ? 16 : 0);
        }
        for (int c = tid; c < BROWS * 4; c += GG_THREADS) {
            const int r = c >> 2, kc = (c & 3) * 8;
            const int n = n0 + (r % GG_BN);
            const bool ok = n < N && k0 + kc < K;
            const size_t wrow = (GATED && r >= GG_BN) ? (size_t)N + n : (size_t)n;
            const bf16* g = wbase + (ok ? wrow * K + k0 + kc : 0);
            cp_async_16(smem_u32(&Bs[stage][r * GG_LD + kc]), g, ok ? 16 : 0);
        }
    };

    float acc[GATED ? 2 : 1][2][4][4];
#pragma unroll
    for (int s = 0; s < (GATED ? 2 : 1); ++s)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[s][i][j][q] = 0.f;

    const int k_tiles = (K + GG_BK - 1) / GG_BK;
#pragma unroll
    for (int s = 0; s < GG_STAGES - 1; ++s) {
        if (s < k_tiles) load_stage(s, s * GG_BK);
        cp_async_commit();
    }
    for (int kt = 0; kt < k_tiles; ++kt) {
        cp_async_wait<GG_STAGES - 2>();
        __syncthreads();
        const int next = kt + GG_STAGES - 1;
        if (next < k_tiles) load_stage(next % GG_STAGES, next * GG_BK);
        cp_async_commit();
        const bf16* At = As[kt % GG_STAGES];
        const bf16* Bt = Bs[kt % GG_STAGES];
#pragma unroll
        for (int kk = 0; kk < GG_BK; kk += 16) {
            uint32_t af[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                ldmatrix_x4(af[i], smem_u32(&At[(wm + i * 16 + (lane & 15)) * GG_LD + kk + (lane >> 4) * 8]));
#pragma unroll
            for (int s = 0; s < (GATED ? 2 : 1); ++s) {
#pragma unroll
                for (int jp = 0; jp < 2; ++jp) {
                    uint32_t bfr[4];
                    const int brow = s * GG_BN + wn + jp * 16 + (lane & 7) + (lane >> 4) * 8;
                    ldmatrix_x4(bfr, smem_u32(&Bt[brow * GG_LD + kk + ((lane >> 3) & 1) * 8]));
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        mma_bf16_16816(acc[s][i][jp * 2], af[i], bfr[0], bfr[1]);
                        mma_bf16_16816(acc[s][i][jp * 2 + 1], af[i], bfr[2], bfr[3]);
                    }
                }
            }
        }
    }
    cp_async_wait<0>();

    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm + i * 16 + g + half * 8;
            const int p = p0 + r;
            if (p >= p_end) continue;
            float wgt = 1.f;
            if (GATHER && scale_input) wgt = weight[order[p]];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + wn + j * 8 + 2 * t4;
                if (n >= N) continue;
                if (GATED) {
                    const float g0 = acc[0][i][j][half * 2] * wgt, g1 = acc[0][i][j][half * 2 + 1] * wgt;
                    const float u0 = acc[GATED ? 1 : 0][i][j][half * 2] * wgt;
                    const float u1 = acc[GATED ? 1 : 0][i][j][half * 2 + 1] * wgt;
                    bf16* o = (bf16*)out + (size_t)p * N + n;
                    o[0] = __float2bfloat16_rn(g0 / (1.f + expf(-g0)) * u0);
                    if (n + 1 < N) o[1] = __float2bfloat16_rn(g1 / (1.f + expf(-g1)) * u1);
                } else if (MODE == 2) {
                    const float r0 = fmaxf(acc[0][i][j][half * 2] * wgt, 0.f);
                    const float r1 = fmaxf(acc[0][i][j][half * 2 + 1] * wgt, 0.f);
                    bf16* o = (bf16*)out + (size_t)p * N + n;
                    o[0] = __float2bfloat16_rn(r0 * r0);
                    if (n + 1 < N) o[1] = __float2bfloat16_rn(r1 * r1);
                } else {
                    float* o = (float*)out + (size_t)p * N + n;
                    o[0] = acc[0][i][j][half * 2];
                    if (n + 1 < N) o[1] = acc[0][i][j][half * 2 + 1];
                }
            }
        }
    }
}

template <typename A>
__global__ void experts_combine_kernel(const float* __restrict__ y, const int* __restrict__ pos,
                                       const float* __restrict__ weight, const A* __restrict__ add,
                                       A* __restrict__ out, int width, int top, int scale_input,
                                       const int* __restrict__ chosen, const A* __restrict__ x,
                                       int real) {
    const unsigned long long waited = pdl_wait();
    y = pdl_after(y, waited);
    pos = pdl_after(pos, waited);
    add = pdl_after(add, waited);
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float total = 0.f;
        for (int k = 0; k < top; ++k) {
            if (chosen[(size_t)t * top + k] >= real) {     // identity expert: w x[t]
                total += weight[(size_t)t * top + k] * to_float(x[(size_t)t * width + c]);
                continue;
            }
            const float v = y[(size_t)pos[(size_t)t * top + k] * width + c];
            total += scale_input ? v : v * weight[(size_t)t * top + k];
        }
        if (add != nullptr) total += to_float(add[(size_t)t * width + c]);
        out[(size_t)t * width + c] = from_float<A>(total);
    }
}

// bfloat16 only.  `ints`: scratch of 2 * rows + experts + 2 + 2 * (rows / 64 + experts) ints;
// `act`: bfloat16 [rows, ff]; `y`: float [rows, width] (rows = tokens * top).  Returns 0, a CUDA
// error code, or -1 when the shape is refused (width or ff no multiple of 8, over 1024 experts).
MSTAR_API int mstar_experts_grouped(const void* x, const void* w_gate_up, const void* w_down,
                                    const int* chosen, const float* weight, int* ints, void* act,
                                    float* y, const void* add, void* out, int tokens, int width,
                                    int ff, int top, int experts, int scale_input, int gated,
                                    int real, void* stream) {
    if (tokens <= 0) return 0;
    if (width % 8 != 0 || ff % 8 != 0 || experts <= 0 || experts > 1024 || top <= 0) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const int rows = tokens * top;
    // tiles of 128 rows where an expert's group fills them on average, else of 64
    const int bm = rows / experts >= 128 ? 128 : 64;
    const int max_tiles = rows / bm + experts;
    int* order = ints;
    int* pos = order + rows;
    int* offsets = pos + rows;
    int* num_tiles = offsets + experts + 1;
    int* tile_expert = num_tiles + 1;
    int* tile_first = tile_expert + (rows / 64 + experts);
    mstar_launch(experts_sort_kernel, dim3(1), dim3(1024), sizeof(int) * 2 * experts, s, chosen, rows,
                 experts, real, bm, order, pos, offsets, tile_expert, tile_first, num_tiles);
#define GG_SMEM(BM, BROWS) (sizeof(bf16) * GG_STAGES * ((BM) + (BROWS)) * GG_LD + sizeof(int) * (BM))
#define GG_GO(MODE, BM, BROWS, GRIDX, ...)                                                        \
    {                                                                                             \
        static bool configured = false;                                                           \
        const size_t bytes = GG_SMEM(BM, BROWS);                                                  \
        if (!configured && bytes > 48 * 1024) {                                                   \
            cudaFuncSetAttribute(grouped_gemm_kernel<MODE, BM>,                                   \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);        \
            configured = true;                                                                    \
        }                                                                                         \
        mstar_launch((grouped_gemm_kernel<MODE, BM>), dim3(GRIDX, max_tiles), dim3((BM) * 2), bytes, s, \
                     __VA_ARGS__);                                                                \
    }
    const int gx1 = (ff + GG_BN - 1) / GG_BN, gx2 = (width + GG_BN - 1) / GG_BN;
#define GG_UP(BM)                                                                                 \
    if (gated)                                                                                    \
        GG_GO(1, BM, 2 * GG_BN, gx1, (const bf16*)x, (const bf16*)w_gate_up, act, order, weight,  \
              offsets, tile_expert, tile_first, num_tiles, ff, width, top, scale_input)           \
    else                                                                                          \
        GG_GO(2, BM, GG_BN, gx1, (const bf16*)x, (const bf16*)w_gate_up, act, order, weight,      \
              offsets, tile_expert, tile_first, num_tiles, ff, width, top, scale_input)
    if (bm == 128) {
        GG_UP(128)
        GG_GO(0, 128, GG_BN, gx2, (const bf16*)act, (const bf16*)w_down, (void*)y, order, weight,
              offsets, tile_expert, tile_first, num_tiles, width, ff, top, scale_input)
    } else {
        GG_UP(64)
        GG_GO(0, 64, GG_BN, gx2, (const bf16*)act, (const bf16*)w_down, (void*)y, order, weight,
              offsets, tile_expert, tile_first, num_tiles, width, ff, top, scale_input)
    }
#undef GG_UP
#undef GG_GO
#undef GG_SMEM
    mstar_launch((experts_combine_kernel<bf16>), dim3(tokens), dim3(256), 0, s, (const float*)y, pos,
                 weight, (const bf16*)add, (bf16*)out, width, top, scale_input, chosen,
                 (const bf16*)x, real);
    return launch_status();
}
