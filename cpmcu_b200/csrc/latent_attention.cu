// Attention over a cached latent: every token leaves one vector c of ``rank`` values in the cache, and the keys
// and values of all heads are linear maps of it, k_h = Uk_h c and v_h = Uv_h c.  With the key map moved to the query
// side and the value map behind the weighted sum,
//
//   score_h(i, j) = scale * (Uk_h^T q_h(i)) . c_j          o_h(i) = Uv_h (sum_j p_h(i, j) c_j)
//
// the attention runs on the cached latents themselves: one shared "key = value" row per token for all heads.
// A query at position p sees the keys j with 0 <= p - j < window (window 0: every j <= p).
//
//   latent_norm_store   RMS-norms the two parts of the fused down projection [tokens, q_rank + rank] (fp32):
//                       the query latent goes on as an activation, the key-value latent into the cache pages
//   head_project        out[t, h, :] = in[t, h, :] @ w[h]   (w [heads][k][n]; fp32 accumulation), the per-head
//                       maps Uk^T (queries into the latent space) and Uv (weighted latents into values)
//   latent_attention    softmax attention of [tokens, heads, rank] fp32 queries over the latent pages; scores,
//                       softmax and the weighted sum are fp32; a block is one token and up to 16 heads, which share
//                       every tile of 32 latent rows through shared memory
//
// A latent page is [token_in_page][rank] (the key page layout with one key-value head).
#include "common.cuh"

// ---------------------------------------------------------------------------
template <typename T>
__global__ void latent_norm_store_kernel(const float* __restrict__ proj, const float* __restrict__ wq, const float* __restrict__ wkv,
                                         T* __restrict__ cq, T* __restrict__ cache, const int* __restrict__ positions,
                                         const int* __restrict__ token_seq, const int* __restrict__ slots,
                                         const int* __restrict__ page_table, int max_pages, int q_rank, int rank, float eps) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const float* row = proj + (int64_t)t * (q_rank + rank);
    float s = 0.f;
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) s = fmaf(row[c], row[c], s);
    float r = 1.0f / sqrtf(block_sum(s, scratch) / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) cq[(int64_t)t * q_rank + c] = from_f32<T>(row[c] * r * wq[c]);
    row += q_rank;
    s = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) s = fmaf(row[c], row[c], s);
    r = 1.0f / sqrtf(block_sum(s, scratch) / (float)rank + eps);
    if (cache == nullptr) return;
    const int p = positions[t];
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    const int page = CPM_PAGE(pages, p / kPageTokens, max_pages);
    T* dst = cache + page_row_offset(page, 0, p % kPageTokens, 1, rank);
    for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = from_f32<T>(row[c] * r * wkv[c]);
}

CPM_API int cpm_latent_norm_store(const float* proj, const float* wq, const float* wkv, void* cq, void* cache,
                                  const int* positions, const int* token_seq, const int* slots, const int* page_table,
                                  int max_pages, int n_tokens, int q_rank, int rank, float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (q_rank <= 0 || rank <= 0) return CPM_BAD_ARGUMENT;
    const int threads = (q_rank + rank) >= 1024 ? 256 : 128;
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchRope, latent_norm_store_kernel<bf16>, n_tokens, threads, 0, stream, proj, wq, wkv, (bf16*)cq, (bf16*)cache,
                   positions, token_seq, slots, page_table, max_pages, q_rank, rank, eps);
    else
        cpm_launch(kLaunchRope, latent_norm_store_kernel<float>, n_tokens, threads, 0, stream, proj, wq, wkv, (float*)cq,
                   (float*)cache, positions, token_seq, slots, page_table, max_pages, q_rank, rank, eps);
    return launch_status();
}

// ---------------------------------------------------------------------------
constexpr int kProjectTokens = 8;      // tokens of one head that share a pass over the head's matrix

template <typename In, typename Wt, typename Out>
__global__ void head_project_kernel(const In* __restrict__ in, const Wt* __restrict__ w, Out* __restrict__ out,
                                    int n_tokens, int n_heads, int K, int N) {
    extern __shared__ float hp_smem[];      // [kProjectTokens][K]
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y;
    const int t0 = blockIdx.x * kProjectTokens;
    const int nt = min(kProjectTokens, n_tokens - t0);
    for (int i = threadIdx.x; i < nt * K; i += blockDim.x) {
        const int tt = i / K, k = i % K;
        hp_smem[tt * K + k] = to_f32(in[((int64_t)(t0 + tt) * n_heads + h) * K + k]);
    }
    __syncthreads();
    const Wt* wh = w + (int64_t)h * K * N;
    for (int n = threadIdx.x; n < N; n += blockDim.x) {
        float acc[kProjectTokens];
#pragma unroll
        for (int tt = 0; tt < kProjectTokens; ++tt) acc[tt] = 0.f;
        for (int k = 0; k < K; ++k) {
            const float wv = to_f32(wh[(int64_t)k * N + n]);
#pragma unroll
            for (int tt = 0; tt < kProjectTokens; ++tt) acc[tt] = fmaf(hp_smem[tt * K + k], wv, acc[tt]);
        }
        for (int tt = 0; tt < nt; ++tt) out[((int64_t)(t0 + tt) * n_heads + h) * N + n] = from_f32<Out>(acc[tt]);
    }
}

template <typename In, typename Wt, typename Out>
static int launch_head_project(const void* in, const void* w, void* out, int n_tokens, int n_heads, int K, int N,
                               cudaStream_t stream) {
    const size_t smem = (size_t)kProjectTokens * K * sizeof(float);
    auto kern = head_project_kernel<In, Wt, Out>;
    if (smem > 227 * 1024) return CPM_BAD_ARGUMENT;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid((n_tokens + kProjectTokens - 1) / kProjectTokens, n_heads);
    const int threads = N >= 256 ? 256 : (N >= 128 ? 128 : 64);
    cpm_launch(kLaunchProduct, kern, grid, threads, smem, stream, (const In*)in, (const Wt*)w, (Out*)out, n_tokens, n_heads, K, N);
    return launch_status();
}

// in_f32 / out_f32: whether the activations on that side are fp32 (else the storage type ``dtype``); the matrix
// always has the storage type.
CPM_API int cpm_head_project(const void* in, const void* w, void* out, int n_tokens, int n_heads, int K, int N, int in_f32,
                             int out_f32, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (n_heads <= 0 || n_heads > 65535 || K <= 0 || N <= 0) return CPM_BAD_ARGUMENT;
    if (dtype == CPM_F32) return launch_head_project<float, float, float>(in, w, out, n_tokens, n_heads, K, N, stream);
    if (in_f32 && out_f32) return launch_head_project<float, bf16, float>(in, w, out, n_tokens, n_heads, K, N, stream);
    if (in_f32) return launch_head_project<float, bf16, bf16>(in, w, out, n_tokens, n_heads, K, N, stream);
    if (out_f32) return launch_head_project<bf16, bf16, float>(in, w, out, n_tokens, n_heads, K, N, stream);
    return launch_head_project<bf16, bf16, bf16>(in, w, out, n_tokens, n_heads, K, N, stream);
}

// ---------------------------------------------------------------------------
constexpr int kLatentTile = 32;        // latent rows per shared-memory tile (one per lane in the scores)
constexpr int kLatentMaxWarps = 16;    // heads per block

// RL = ceil(rank / 32): what a lane keeps of a head's weighted sum.
template <typename T, int RL>
__global__ void latent_attention_kernel(const float* __restrict__ q /* [tokens, heads, rank] */, const T* __restrict__ cache,
                                        float* __restrict__ out /* [tokens, heads, rank] */, const int* __restrict__ positions,
                                        const int* __restrict__ token_seq, const int* __restrict__ slots,
                                        const int* __restrict__ page_table, int max_pages, int window, int n_heads, int rank,
                                        float scale) {
    extern __shared__ float la_smem[];
    const int n_warps = blockDim.x >> 5;
    const int pitch = rank + 1;                       // odd pitch: lane j reads row j without bank conflicts
    float* qs = la_smem;                              // [warps][rank]
    float* tile = la_smem + n_warps * rank;           // [kLatentTile][pitch]
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * n_warps + warp;
    const bool live = h < n_heads;
    const int p = positions[t];
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    if (live) {
        const float* qrow = q + ((int64_t)t * n_heads + h) * rank;
        for (int c = lane; c < rank; c += 32) qs[warp * rank + c] = qrow[c] * scale;
    }
    float m = -INFINITY, l = 0.f;
    float acc[RL];
#pragma unroll
    for (int i = 0; i < RL; ++i) acc[i] = 0.f;

    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    for (int j0 = lo; j0 <= p; j0 += kLatentTile) {
        const int n_here = min(kLatentTile, p + 1 - j0);
        __syncthreads();                              // the tile of the previous iteration is no longer read
        for (int r = warp; r < n_here; r += n_warps) {
            const int j = j0 + r;
            const int page = CPM_PAGE(pages, j / kPageTokens, max_pages);
            const T* src = cache + page_row_offset(page, 0, j % kPageTokens, 1, rank);
            for (int c = lane; c < rank; c += 32) tile[r * pitch + c] = to_f32(src[c]);
        }
        __syncthreads();
        if (!live) continue;
        float s = -INFINITY;
        if (lane < n_here) {
            const float* row = tile + lane * pitch;
            const float* qh = qs + warp * rank;
            float dot = 0.f;
            for (int c = 0; c < rank; ++c) dot = fmaf(qh[c], row[c], dot);
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float pr = lane < n_here ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(pr);
#pragma unroll
        for (int i = 0; i < RL; ++i) acc[i] *= corr;
        m = m_new;
        for (int jj = 0; jj < n_here; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, pr, jj);
            const float* row = tile + jj * pitch;
#pragma unroll
            for (int i = 0; i < RL; ++i) {
                const int c = lane + 32 * i;
                if (c < rank) acc[i] = fmaf(pj, row[c], acc[i]);
            }
        }
    }
    if (!live) return;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    float* orow = out + ((int64_t)t * n_heads + h) * rank;
#pragma unroll
    for (int i = 0; i < RL; ++i) {
        const int c = lane + 32 * i;
        if (c < rank) orow[c] = acc[i] * inv;
    }
}

template <typename T, int RL>
static int launch_latent_attention(const float* q, const void* cache, float* out, const int* positions, const int* token_seq,
                                   const int* slots, const int* page_table, int max_pages, int window, int n_tokens,
                                   int n_heads, int rank, float scale, cudaStream_t stream) {
    const int warps = n_heads < kLatentMaxWarps ? n_heads : kLatentMaxWarps;
    const size_t smem = ((size_t)warps * rank + (size_t)kLatentTile * (rank + 1)) * sizeof(float);
    auto kern = latent_attention_kernel<T, RL>;
    if (smem > 227 * 1024) return CPM_BAD_ARGUMENT;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(n_tokens, (n_heads + warps - 1) / warps);
    cpm_launch(kLaunchOther, kern, grid, warps * 32, smem, stream, q, (const T*)cache, out, positions, token_seq, slots, page_table,
               max_pages, window, n_heads, rank, scale);
    return launch_status();
}

CPM_API int cpm_latent_attention(const float* q, const void* cache, float* out, const int* positions, const int* token_seq,
                                 const int* slots, const int* page_table, int max_pages, int window, int n_tokens, int n_heads,
                                 int rank, float scale, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (n_heads <= 0 || rank <= 0 || rank > 512 || window < 0) return CPM_BAD_ARGUMENT;
#define CPM_LATENT(RL)                                                                                                        \
    return dtype == CPM_BF16                                                                                                  \
        ? launch_latent_attention<bf16, RL>(q, cache, out, positions, token_seq, slots, page_table, max_pages, window,       \
                                            n_tokens, n_heads, rank, scale, stream)                                           \
        : launch_latent_attention<float, RL>(q, cache, out, positions, token_seq, slots, page_table, max_pages, window,      \
                                             n_tokens, n_heads, rank, scale, stream)
    if (rank <= 64) { CPM_LATENT(2); }
    if (rank <= 128) { CPM_LATENT(4); }
    if (rank <= 256) { CPM_LATENT(8); }
    CPM_LATENT(16);
#undef CPM_LATENT
}

CPM_BOUNDS_TU(latent_attention)
