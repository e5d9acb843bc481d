// Causal softmax attention whose weights are mixed across heads after the softmax ("talking heads"), with a
// learned temperature per head, over the paged cache.
//
//   s_g(i, j) = q_g(i) . k_kv(g)(j) * scale * temp[g]            j <= i
//   p_g(i, :) = softmax_j s_g(i, :)
//   w_h(i, j) = sum_g talk[h][g] p_g(i, j)
//   o_h(i)    = sum_j w_h(i, j) v_kv(h)(j)
//
// The mix needs every head's *normalised* weight of a key, so a query is worked in two walks over its keys: the
// first finds every head's maximum and sum, the second forms p_g for 32 keys at a time in shared memory, mixes
// them and adds the values.  One block per query token, one warp per head (beyond 32 heads a warp works several); a lane owns a key in the scores and a
// set of value channels in the weighted sum (value pages are [kv_head][dv][token], so 32 keys of a channel are
// contiguous).  Scores, weights and sums are fp32; q, the cache and the output have the storage type.  Key size d
// and value size dv are independent.
#include "common.cuh"

constexpr int kTalkMaxHeads = 128;
constexpr int kTalkMaxVPerLane = 8;      // dv <= 256

template <typename T>
__device__ __forceinline__ float key_dot(const T* __restrict__ krow, const float* __restrict__ qs, int d) {
    float dot = 0.f;
    for (int c = 0; c < d; ++c) dot = fmaf(qs[c], to_f32(krow[c]), dot);
    return dot;
}

template <>
__device__ __forceinline__ float key_dot<bf16>(const bf16* __restrict__ krow, const float* __restrict__ qs, int d) {
    float dot = 0.f;
    if ((d & 7) == 0 && (((uintptr_t)krow) & 15) == 0) {
        for (int c = 0; c < d; c += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(krow + c);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(h2[i]);
                dot = fmaf(qs[c + 2 * i], f.x, dot);
                dot = fmaf(qs[c + 2 * i + 1], f.y, dot);
            }
        }
        return dot;
    }
    for (int c = 0; c < d; ++c) dot = fmaf(qs[c], __bfloat162float(krow[c]), dot);
    return dot;
}

// HPW: heads a warp works: 1 up to 32 heads (a warp each); more heads go round 16 warps.
template <typename T, int HPW>
__global__ void __launch_bounds__(HPW == 1 ? 1024 : 512) talking_attention_kernel(const T* __restrict__ q,            // [tokens, heads, d]
                                         const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                         T* __restrict__ out,                // [tokens, heads, dv]
                                         const int* __restrict__ positions, const int* __restrict__ token_seq,
                                         const int* __restrict__ slots, const int* __restrict__ page_table, int max_pages,
                                         const float* __restrict__ temp, const float* __restrict__ talk,
                                         int n_heads, int n_kv, int d, int dv, float scale) {
    extern __shared__ float smem[];
    float* qs = smem;                               // [heads][d]
    float* P = qs + n_heads * d;                    // [heads][32]
    float* tk = P + n_heads * 32;                   // [heads][heads]
    pdl_launch_dependents();
    for (int i = threadIdx.x; i < n_heads * n_heads; i += blockDim.x) tk[i] = talk[i];
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const int t = blockIdx.x;
    const int p = positions[t];
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    const int rep = n_heads / n_kv;
    for (int i = threadIdx.x; i < n_heads * d; i += blockDim.x) qs[i] = to_f32(q[(int64_t)t * n_heads * d + i]);
    __syncthreads();

    // first walk: every head's maximum and sum
    float M[HPW], inv_L[HPW], s_scale[HPW];
#pragma unroll
    for (int hi = 0; hi < HPW; ++hi) {
        const int g = warp + hi * n_warps;
        M[hi] = 0.f;
        inv_L[hi] = 0.f;
        s_scale[hi] = 0.f;
        if (g >= n_heads) continue;
        const int kvh = g / rep;
        const float* qg = qs + g * d;
        s_scale[hi] = scale * temp[g];
        float m = -INFINITY, l = 0.f;
        for (int j0 = 0; j0 <= p; j0 += 32) {
            const int j = j0 + lane;
            if (j <= p) {
                const int page = CPM_PAGE(pages, j / kPageTokens, max_pages);
                const float s = key_dot(k_cache + page_row_offset(page, kvh, j % kPageTokens, n_kv, d), qg, d) * s_scale[hi];
                const float m_new = fmaxf(m, s);
                l = l * expf(m - m_new) + expf(s - m_new);       // expf(-inf) = 0 at the first key
                m = m_new;
            }
        }
        M[hi] = warp_max(m);
        inv_L[hi] = 1.0f / warp_sum(m == -INFINITY ? 0.f : l * expf(m - M[hi]));
    }

    // second walk: normalised weights of 32 keys, mixed across heads, times the values
    float acc[HPW][kTalkMaxVPerLane];
#pragma unroll
    for (int hi = 0; hi < HPW; ++hi)
#pragma unroll
        for (int i = 0; i < kTalkMaxVPerLane; ++i) acc[hi][i] = 0.f;
    for (int j0 = 0; j0 <= p; j0 += 32) {
        const int j = j0 + lane;
        const int page0 = CPM_PAGE(pages, j0 / kPageTokens, max_pages);      // 32 keys from a multiple of 32 lie in one page
#pragma unroll
        for (int hi = 0; hi < HPW; ++hi) {
            const int g = warp + hi * n_warps;
            if (g >= n_heads) continue;
            float pr = 0.f;
            if (j <= p) {
                const float s = key_dot(k_cache + page_row_offset(page0, g / rep, j % kPageTokens, n_kv, d), qs + g * d, d) * s_scale[hi];
                pr = expf(s - M[hi]) * inv_L[hi];
            }
            P[g * 32 + lane] = pr;
        }
        __syncthreads();
        const int n_here = min(32, p + 1 - j0);
#pragma unroll
        for (int hi = 0; hi < HPW; ++hi) {
            const int h = warp + hi * n_warps;
            if (h >= n_heads) continue;
            float w = 0.f;
            for (int gg = 0; gg < n_heads; ++gg) w = fmaf(tk[h * n_heads + gg], P[gg * 32 + lane], w);
            const T* vbase = v_cache + value_offset(page0, h / rep, 0, j0 % kPageTokens, n_kv, dv);
            for (int jj = 0; jj < n_here; ++jj) {
                const float wj = __shfl_sync(0xffffffffu, w, jj);
#pragma unroll
                for (int i = 0; i < kTalkMaxVPerLane; ++i) {
                    const int c = lane + 32 * i;
                    if (c < dv) acc[hi][i] = fmaf(wj, to_f32(vbase[(int64_t)c * kPageTokens + jj]), acc[hi][i]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int hi = 0; hi < HPW; ++hi) {
        const int h = warp + hi * n_warps;
        if (h >= n_heads) continue;
        T* orow = out + ((int64_t)t * n_heads + h) * dv;
#pragma unroll
        for (int i = 0; i < kTalkMaxVPerLane; ++i) {
            const int c = lane + 32 * i;
            if (c < dv) orow[c] = from_f32<T>(acc[hi][i]);
        }
    }
}

template <typename T, int HPW>
static int launch_talking(const void* q, const void* k_cache, const void* v_cache, void* out, const int* positions,
                          const int* token_seq, const int* slots, const int* page_table, int max_pages, const float* temp,
                          const float* talk, int n_tokens, int n_heads, int n_kv, int d, int dv, float scale, size_t smem,
                          cudaStream_t stream) {
    static bool configured[kMaxDevices] = {};            // per kernel and per device
    if (smem > 48 * 1024) {
        const int e = ensure_dynamic_smem(talking_attention_kernel<T, HPW>, 200 * 1024, configured);
        if (e != CPM_OK) return e;
    }
    const int warps = HPW == 1 ? n_heads : 16;
    cpm_launch(kLaunchAttention, talking_attention_kernel<T, HPW>, dim3(n_tokens), dim3(32 * warps), smem, stream, (const T*)q,
               (const T*)k_cache, (const T*)v_cache, (T*)out, positions, token_seq, slots, page_table, max_pages, temp, talk, n_heads,
               n_kv, d, dv, scale);
    return launch_status();
}

CPM_API int cpm_talking_attention(const void* q, const void* k_cache, const void* v_cache, void* out, const int* positions,
                                  const int* token_seq, const int* slots, const int* page_table, int max_pages,
                                  const float* temp, const float* talk, int n_tokens, int n_heads, int n_kv, int d, int dv,
                                  float scale, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (n_heads < 1 || n_heads > kTalkMaxHeads || n_kv < 1 || n_heads % n_kv || d < 1 || dv < 1 || dv > 32 * kTalkMaxVPerLane)
        return CPM_BAD_ARGUMENT;
    const size_t smem = (size_t)(n_heads * d + n_heads * 32 + n_heads * n_heads) * sizeof(float);
    if (smem > 200 * 1024) return CPM_BAD_ARGUMENT;
#define CPM_TALK(TT, HPW) launch_talking<TT, HPW>(q, k_cache, v_cache, out, positions, token_seq, slots, page_table, max_pages, temp, \
                                                  talk, n_tokens, n_heads, n_kv, d, dv, scale, smem, stream)
    if (dtype == CPM_BF16) return n_heads <= 32 ? CPM_TALK(bf16, 1) : n_heads <= 64 ? CPM_TALK(bf16, 4) : CPM_TALK(bf16, 8);
    return n_heads <= 32 ? CPM_TALK(float, 1) : n_heads <= 64 ? CPM_TALK(float, 4) : CPM_TALK(float, 8);
#undef CPM_TALK
}

// ---------------------------------------------------------------------------
// The same attention from the tensor-core kernels of plain softmax attention.  The mix is linear in the weights, so
//   o_h = sum_g talk[h][g] * A[g][kv(h)],     A[g][c] = sum_j p_g(j) v_c(j)
// and A[.][(kv(g) + s) mod n_kv] for all g is what one run of a plain attention kernel gives whose values come from
// the key-value head s places after the keys' (its ``v_shift``).  n_kv runs, s = 0 .. n_kv - 1, then this mix.  The
// temperature goes into the queries beforehand (scale_heads).
// ---------------------------------------------------------------------------
__global__ void scale_heads_kernel(const bf16* __restrict__ q, const float* __restrict__ temp, bf16* __restrict__ out, int n_heads,
                                   int d) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    for (int i = threadIdx.x; i < n_heads * d; i += blockDim.x)
        out[t * n_heads * d + i] = __float2bfloat16_rn(__bfloat162float(q[t * n_heads * d + i]) * temp[i / d]);
}

// parts [n_kv][tokens][heads][d] (run s at parts[s]) -> out [tokens][heads][d]
__global__ void talk_mix_kernel(const bf16* __restrict__ parts, const float* __restrict__ talk, bf16* __restrict__ out,
                                int64_t n_tokens, int n_heads, int n_kv, int d) {
    extern __shared__ float mix_smem[];          // [n_kv][heads][d] of this token, then talk [heads][heads]
    float* tk = mix_smem + n_kv * n_heads * d;
    pdl_launch_dependents();
    for (int i = threadIdx.x; i < n_heads * n_heads; i += blockDim.x) tk[i] = talk[i];
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int row = n_heads * d;
    for (int i = threadIdx.x; i < n_kv * row; i += blockDim.x)
        mix_smem[i] = __bfloat162float(parts[((int64_t)(i / row) * n_tokens + t) * row + i % row]);
    __syncthreads();
    const int rep = n_heads / n_kv;
    for (int i = threadIdx.x; i < row; i += blockDim.x) {
        const int h = i / d, c = i % d;
        float acc = 0.f;
        for (int g = 0; g < n_heads; ++g) {
            const int s = (h / rep - g / rep + n_kv) % n_kv;          // the run in which head g saw the values of h's head
            acc = fmaf(tk[h * n_heads + g], mix_smem[(s * n_heads + g) * d + c], acc);
        }
        out[t * row + i] = __float2bfloat16_rn(acc);
    }
}

CPM_API int cpm_scale_heads_bf16(const void* q, const float* temp, void* out, int n_tokens, int n_heads, int d, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    cpm_launch(kLaunchRope, scale_heads_kernel, dim3(n_tokens), dim3(n_heads * d >= 1024 ? 256 : 128), 0, stream, (const bf16*)q, temp,
               (bf16*)out, n_heads, d);
    return launch_status();
}

static bool g_mix_smem_done[kMaxDevices];

CPM_API int cpm_talk_mix_bf16(const void* parts, const float* talk, void* out, int n_tokens, int n_heads, int n_kv, int d,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (n_heads < 1 || n_kv < 1 || n_heads % n_kv) return CPM_BAD_ARGUMENT;
    const size_t smem = (size_t)(n_kv * n_heads * d + n_heads * n_heads) * sizeof(float);
    if (smem > 200 * 1024) return CPM_BAD_ARGUMENT;
    if (smem > 48 * 1024) {
        const int e = ensure_dynamic_smem(talk_mix_kernel, 200 * 1024, g_mix_smem_done);
        if (e != CPM_OK) return e;
    }
    cpm_launch(kLaunchCombine, talk_mix_kernel, dim3(n_tokens), dim3(256), smem, stream, (const bf16*)parts, talk, (bf16*)out,
               (int64_t)n_tokens, n_heads, n_kv, d);
    return launch_status();
}

CPM_BOUNDS_TU(talking_attention)
