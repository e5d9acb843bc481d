// Several residual streams per token ("hyper-connections").
//
// Instead of one residual vector a token carries S of them, X[t][s][:] (fp32).  A sublayer reads one blend of
// them and writes back into all:
//
//   read:   u = sum_s in[s] X_s                      h = u / sqrt(mean(u^2) + eps) * gain     (gain: one number)
//   write:  X_r <- sum_s mix[s][r] X_s + out[r] * y  for all r at once from the old X_s       (y: the sublayer's output)
//
// One kernel does a write (when y is given), then a read (when ``in`` is given), then the plain sum of the
// streams (when ``total`` is given), so the write of one sublayer and the read and norm of the next are one pass
// over X.  Everything is fp32; only y and h have the storage type.
#include "common.cuh"

constexpr int kMaxStreams = 16;

template <typename T, int NS>      // NS: a compile-time bound on the streams (the loops are unrolled to it)
__global__ void hyper_step_kernel(float* __restrict__ X, const T* __restrict__ y, const float* __restrict__ mix,
                                  const float* __restrict__ out_w, const float* __restrict__ in_w,
                                  const float* __restrict__ gain, float eps, T* __restrict__ h,
                                  float* __restrict__ total, int S, int W) {
    __shared__ float s_mix[NS * NS], s_out[NS], s_in[NS], scratch[33];
    pdl_launch_dependents();
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[i] = y ? mix[i] : 0.f;
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        s_out[i] = y ? out_w[i] : 0.f;
        s_in[i] = in_w ? in_w[i] : 0.f;
    }
    pdl_wait();
    __syncthreads();
    const int64_t t = blockIdx.x;
    float* xt = X + t * S * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float old[NS];
#pragma unroll
        for (int s = 0; s < NS; ++s) old[s] = s < S ? xt[(int64_t)s * W + c] : 0.f;
        float u = 0.f, sum = 0.f;
        if (y) {
            const float yc = to_f32(y[t * W + c]);
#pragma unroll
            for (int r = 0; r < NS; ++r) {
                if (r < S) {
                    float v = 0.f;
#pragma unroll
                    for (int s = 0; s < NS; ++s)
                        if (s < S) v = fmaf(s_mix[s * S + r], old[s], v);
                    v = fmaf(s_out[r], yc, v);
                    xt[(int64_t)r * W + c] = v;
                    u = fmaf(s_in[r], v, u);
                    sum += v;
                }
            }
        } else {
#pragma unroll
            for (int r = 0; r < NS; ++r)
                if (r < S) {
                    u = fmaf(s_in[r], old[r], u);
                    sum += old[r];
                }
        }
        if (total) total[t * W + c] = sum;
        ss = fmaf(u, u, ss);
    }
    if (!in_w) return;
    ss = block_sum(ss, scratch);
    const float f = rsqrtf(ss / (float)W + eps) * gain[0];
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float u = 0.f;
        for (int r = 0; r < S; ++r) u = fmaf(s_in[r], xt[(int64_t)r * W + c], u);      // this thread's own writes
        h[t * W + c] = from_f32<T>(u * f);
    }
}

__global__ void hyper_fan_out_kernel(const float* __restrict__ x, float* __restrict__ X, int S, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = x[t * W + c];
        for (int s = 0; s < S; ++s) X[(t * S + s) * W + c] = v;
    }
}

// X [tokens, S, W] fp32 in place.  y (nullable) with mix [S, S] (indexed [from][to]) and out_w [S]: the write.
// in_w (nullable) with gain (one float on the device) and eps: the read, h [tokens, W].  total (nullable): the
// sum of the streams after the write, [tokens, W] fp32.
CPM_API int cpm_hyper_step(float* X, const void* y, const float* mix, const float* out_w, const float* in_w,
                           const float* gain, float eps, void* h, float* total, int n_tokens, int S, int W, int dtype,
                           cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (S < 1 || S > kMaxStreams || W < 1) return CPM_BAD_ARGUMENT;
    if (y && (!mix || !out_w)) return CPM_BAD_ARGUMENT;
    if (in_w && (!gain || !h)) return CPM_BAD_ARGUMENT;
    const int threads = W >= 1024 ? 256 : 128;
#define CPM_HYPER(NS)                                                                                                              \
    do {                                                                                                                           \
        if (dtype == CPM_BF16)                                                                                                     \
            cpm_launch(kLaunchNorm, hyper_step_kernel<bf16, NS>, dim3(n_tokens), dim3(threads), 0, stream, X, (const bf16*)y, mix,  \
                       out_w, in_w, gain, eps, (bf16*)h, total, S, W);                                                             \
        else                                                                                                                       \
            cpm_launch(kLaunchNorm, hyper_step_kernel<float, NS>, dim3(n_tokens), dim3(threads), 0, stream, X, (const float*)y,     \
                       mix, out_w, in_w, gain, eps, (float*)h, total, S, W);                                                       \
    } while (0)
    if (S <= 2) CPM_HYPER(2);
    else if (S <= 4) CPM_HYPER(4);
    else if (S <= 8) CPM_HYPER(8);
    else CPM_HYPER(16);
#undef CPM_HYPER
    return launch_status();
}

// X[t][s][:] = x[t][:] for every s.
CPM_API int cpm_hyper_fan_out(const float* x, float* X, int n_tokens, int S, int W, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (S < 1 || W < 1) return CPM_BAD_ARGUMENT;
    cpm_launch(kLaunchNorm, hyper_fan_out_kernel, dim3(n_tokens), dim3(W >= 1024 ? 256 : 128), 0, stream, x, X, S, W);
    return launch_status();
}
