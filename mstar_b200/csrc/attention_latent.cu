// Attention over a paged cache of latent rows, for any mix of prompt portions and decoded
// tokens, in float arithmetic on CUDA cores.
//
// A token's cache row holds `rank` latent features c (normalised) followed by `rot` rotated
// key features r that all heads share: [pages, 1, 1, page_size, rank + rot].  With the key
// up-projection folded into the query (a = W_uk[h]^T q_plain, float, made by the caller),
// head h scores key j as (a . c_j + q_rot . r_j) * scale, takes a softmax over the keys the
// token sees (lo..p, lo = max(0, p - window + 1), window 0: lo = 0), and returns the
// probability-weighted sum of the latents, sum_j p_j c_j (float, [tokens, heads, rank]); the
// caller applies the value up-projection W_uv[h] to it.  Scores, softmax statistics,
// probabilities and the output sum are float for both activation types.
//
// Every head reads the same rows, so a block takes one token and a group of heads and
// streams the rows through shared memory once, 32 keys at a time, anchored at the token's
// own first visible key: what a token computes does not depend on the batch it is in.
//
// The first kernel fills the cache: it normalises the latent part of the down-projection
// (RMS, plain weight), rotates the shared key part and the rotated part of every query head
// (pairs (2i, 2i+1), angle = position * freq_i in double precision), and writes the row.
#include "common.cuh"

#define LAT_TILE 32
#define LAT_THREADS 128
#define LAT_MAX_ACC 32

struct LatentArgs {
    int heads, group, rank, rot, page_size, bt_stride, window;
    int ldq;      // elements between tokens of the rotated query part
    int q_head;   // elements between heads of the rotated query part
    float scale;
};

template <typename A>
__global__ void __launch_bounds__(LAT_THREADS)
latent_attention_kernel(const float* __restrict__ q_abs, const A* __restrict__ q_rot,
                        float* __restrict__ out, const A* __restrict__ cache,
                        const int* __restrict__ block_table, const int* __restrict__ token_req,
                        const int* __restrict__ cache_pos, LatentArgs a) {
    extern __shared__ float smem[];
    const int t = blockIdx.x, h0 = blockIdx.y * a.group;
    const int G = min(a.group, a.heads - h0);
    const int D = a.rank + a.rot, ldk = D + 1;
    float* qs = smem;                         // [group][D]
    float* tile = qs + a.group * D;           // [TILE][D+1]
    float* sc = tile + LAT_TILE * ldk;        // [group][TILE]
    float* m_s = sc + a.group * LAT_TILE;     // [group]
    float* l_s = m_s + a.group;
    float* alpha_s = l_s + a.group;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned long long waited = pdl_wait();
    q_abs = pdl_after(q_abs, waited);
    q_rot = pdl_after(q_rot, waited);
    cache = pdl_after(cache, waited);

    const int hi = cache_pos[t] + 1;
    const int lo = (a.window > 0 && hi > a.window) ? hi - a.window : 0;
    const int* bt = block_table + (size_t)token_req[t] * a.bt_stride;

    for (int i = tid; i < G * D; i += LAT_THREADS) {
        const int g = i / D, d = i - g * D;
        qs[i] = d < a.rank ? q_abs[((size_t)t * a.heads + h0 + g) * a.rank + d]
                           : to_float(q_rot[(size_t)t * a.ldq + (size_t)(h0 + g) * a.q_head + (d - a.rank)]);
    }
    for (int i = tid; i < G; i += LAT_THREADS) {
        m_s[i] = -INFINITY;
        l_s[i] = 0.f;
    }
    float acc[LAT_MAX_ACC];
#pragma unroll
    for (int k = 0; k < LAT_MAX_ACC; ++k) acc[k] = 0.f;
    const int n_out = G * a.rank;
    __syncthreads();

    for (int base = lo; base < hi; base += LAT_TILE) {
        for (int idx = tid; idx < LAT_TILE * D; idx += LAT_THREADS) {
            const int j = idx / D, d = idx - j * D;
            const int key = base + j;
            float v = 0.f;
            if (key < hi) {
                const int page = bt[key / a.page_size];
                const int slot = key % a.page_size;
                v = to_float(cache[((size_t)page * a.page_size + slot) * D + d]);
            }
            tile[j * ldk + d] = v;
        }
        __syncthreads();
        for (int idx = tid; idx < G * LAT_TILE; idx += LAT_THREADS) {
            const int g = idx / LAT_TILE, j = idx - g * LAT_TILE;
            float s = -INFINITY;
            if (base + j < hi) {
                const float* qv = qs + g * D;
                const float* kv = tile + j * ldk;
                float dot = 0.f;
                for (int d = 0; d < D; ++d) dot = fmaf(qv[d], kv[d], dot);
                s = dot * a.scale;
            }
            sc[idx] = s;
        }
        __syncthreads();
        for (int g = warp; g < G; g += LAT_THREADS / 32) {
            const float s = sc[g * LAT_TILE + lane];
            const float m_old = m_s[g];
            const float m_new = fmaxf(m_old, warp_max(s));   // key `base` is always valid
            const float p = expf(s - m_new);
            const float psum = warp_sum(p);
            sc[g * LAT_TILE + lane] = p;
            if (lane == 0) {
                const float al = expf(m_old - m_new);
                alpha_s[g] = al;
                l_s[g] = l_s[g] * al + psum;
                m_s[g] = m_new;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < LAT_MAX_ACC; ++k) {
            const int o = tid + k * LAT_THREADS;
            if (o < n_out) {
                const int g = o / a.rank, d = o - g * a.rank;
                const float* p = sc + g * LAT_TILE;
                float sum = acc[k] * alpha_s[g];
#pragma unroll 8
                for (int j = 0; j < LAT_TILE; ++j) sum = fmaf(p[j], tile[j * ldk + d], sum);
                acc[k] = sum;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int k = 0; k < LAT_MAX_ACC; ++k) {
        const int o = tid + k * LAT_THREADS;
        if (o < n_out) {
            const int g = o / a.rank, d = o - g * a.rank;
            out[((size_t)t * a.heads + h0 + g) * a.rank + d] = acc[k] / l_s[g];
        }
    }
}

// Returns 0, a CUDA error code, or -1 when the shape is refused (rank > 4096, or a tile of
// rows that does not fit shared memory).
MSTAR_API int mstar_latent_attention(const float* q_abs, const void* q_rot, int ldq, int q_head,
                                     float* out, const void* cache, const int* block_table,
                                     int bt_stride, const int* token_req, const int* cache_pos,
                                     int num_tokens, int heads, int rank, int rot, int page_size,
                                     int window, float scale, int act_dtype, void* stream) {
    if (num_tokens <= 0) return 0;
    if (heads <= 0 || rank <= 0 || rot < 0 || rank > LAT_MAX_ACC * LAT_THREADS) return -1;
    int group = (LAT_MAX_ACC * LAT_THREADS) / rank;
    if (group > heads) group = heads;
    if (group > 16) group = 16;
    const int D = rank + rot;
    const size_t smem = sizeof(float) * ((size_t)group * D + (size_t)LAT_TILE * (D + 1) +
                                         (size_t)group * LAT_TILE + 3 * (size_t)group);
    if (smem > 200 * 1024) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    LatentArgs a{heads, group, rank, rot, page_size, bt_stride, window, ldq, q_head, scale};
    dim3 grid(num_tokens, (heads + group - 1) / group);
    static size_t configured_f32 = 0, configured_bf16 = 0;
    if (act_dtype == MSTAR_F32) {
        if (smem > 48 * 1024 && smem > configured_f32) {
            cudaFuncSetAttribute(latent_attention_kernel<float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            configured_f32 = smem;
        }
        mstar_launch((latent_attention_kernel<float>), grid, dim3(LAT_THREADS), smem, s, q_abs,
                     (const float*)q_rot, out, (const float*)cache, block_table, token_req, cache_pos, a);
    } else {
        if (smem > 48 * 1024 && smem > configured_bf16) {
            cudaFuncSetAttribute(latent_attention_kernel<bf16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            configured_bf16 = smem;
        }
        mstar_launch((latent_attention_kernel<bf16>), grid, dim3(LAT_THREADS), smem, s, q_abs,
                     (const bf16*)q_rot, out, (const bf16*)cache, block_table, token_req, cache_pos, a);
    }
    return launch_status();
}

// ---------------------------------------------------------------- cache fill + rotation
struct LatentFillArgs {
    int heads, qk_dim, rot, rot_dims, rank, page_size, bt_stride;
    int ld;        // elements between tokens of the fused product
    int dkv_off;   // column of the first down-projected feature
    float eps;
};

__device__ __forceinline__ void rotate_pair(float u, float v, int position, double freq, float& x,
                                            float& y) {
    double sn, cs;
    sincos((double)position * freq, &sn, &cs);
    const float c = (float)cs, s = (float)sn;
    x = u * c - v * s;
    y = v * c + u * s;
}

template <typename A>
__global__ void latent_fill_kernel(A* __restrict__ proj, const float* __restrict__ norm_w,
                                   const double* __restrict__ freq, const int* __restrict__ positions,
                                   const int* __restrict__ cache_pos, const int* __restrict__ token_req,
                                   const int* __restrict__ block_table, A* __restrict__ cache,
                                   LatentFillArgs a) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, tid = threadIdx.x;
    proj = pdl_after(proj, pdl_wait());
    A* row = proj + (size_t)t * a.ld;
    const A* dkv = row + a.dkv_off;
    const int pos = positions[t], cp = cache_pos[t];
    const int page = block_table[(size_t)token_req[t] * a.bt_stride + cp / a.page_size];
    A* dst = cache + ((size_t)page * a.page_size + cp % a.page_size) * (a.rank + a.rot);

    float ss = 0.f;
    for (int i = tid; i < a.rank; i += blockDim.x) {
        const float v = to_float(dkv[i]);
        ss = fmaf(v, v, ss);
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)a.rank + a.eps);
    for (int i = tid; i < a.rank; i += blockDim.x)
        dst[i] = from_float<A>(to_float(dkv[i]) * inv * norm_w[i]);
    // the shared key part: rotated pairs, then what lies beyond the rotated dimensions
    const int half = a.rot_dims / 2;
    for (int i = tid; i < half; i += blockDim.x) {
        float x, y;
        rotate_pair(to_float(dkv[a.rank + 2 * i]), to_float(dkv[a.rank + 2 * i + 1]), pos, freq[i], x, y);
        dst[a.rank + 2 * i] = from_float<A>(x);
        dst[a.rank + 2 * i + 1] = from_float<A>(y);
    }
    for (int i = a.rot_dims + tid; i < a.rot; i += blockDim.x) dst[a.rank + i] = dkv[a.rank + i];
    // the rotated part of every query head, in place
    for (int idx = tid; idx < a.heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        A* q = row + (size_t)h * (a.qk_dim + a.rot) + a.qk_dim;
        float x, y;
        rotate_pair(to_float(q[2 * i]), to_float(q[2 * i + 1]), pos, freq[i], x, y);
        q[2 * i] = from_float<A>(x);
        q[2 * i + 1] = from_float<A>(y);
    }
}

MSTAR_API int mstar_latent_fill(void* proj, int act_dtype, int ld, int dkv_off, const float* norm_w,
                                const double* freq, const int* positions, const int* cache_pos,
                                const int* token_req, const int* block_table, int bt_stride,
                                void* cache, int num_tokens, int heads, int qk_dim, int rot,
                                int rot_dims, int rank, int page_size, float eps, void* stream) {
    if (num_tokens <= 0) return 0;
    if (rot_dims % 2 != 0 || rot_dims > rot) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    LatentFillArgs a{heads, qk_dim, rot, rot_dims, rank, page_size, bt_stride, ld, dkv_off, eps};
    const int threads = rank >= 512 ? 256 : 128;
    if (act_dtype == MSTAR_F32)
        mstar_launch((latent_fill_kernel<float>), dim3(num_tokens), dim3(threads), 0, s, (float*)proj,
                     norm_w, freq, positions, cache_pos, token_req, block_table, (float*)cache, a);
    else
        mstar_launch((latent_fill_kernel<bf16>), dim3(num_tokens), dim3(threads), 0, s, (bf16*)proj,
                     norm_w, freq, positions, cache_pos, token_req, block_table, (bf16*)cache, a);
    return launch_status();
}
