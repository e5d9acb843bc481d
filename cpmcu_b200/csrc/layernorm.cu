// Layer norm with weight and bias on the fp32 residual stream, and the kernels that join it to its
// neighbours in a layer with a norm before and after each sublayer:
//
//   layernorm_rows          y = LN(x)                       (optionally of listed rows only)
//   layernorm_shift         h = LN(x);  y_t = h_t + (h_{t-1} - h_t) * mu    (token shift; h_{-1} = 0)
//   post_norm_add           x += LN(a);  optionally y = LN'(x) in the same pass
//   stream_inject           x += e + v  (a saved stream and a vector per column, either may be absent)
//
// LN(v) = (v - mean) / sqrt(var + eps) * w + b with var the mean of the squared deviations.  Everything is
// computed in fp32 (two passes over a row held in shared memory: the mean first, then the deviations); only
// the loads of ``a`` and the stores of ``y`` touch the storage type.  Weights, biases and mu are fp32.
#include "common.cuh"

// Four consecutive elements as floats (16-byte or 8-byte aligned loads).
__device__ __forceinline__ float4 ln_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ln_load4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

__device__ __forceinline__ void ln_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void ln_store4(bf16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// Copies a normed row from shared memory to its place in the storage type.
template <typename T>
__device__ __forceinline__ void ln_write_row(T* __restrict__ dst, const float* buf, int hidden) {
    if ((hidden & 3) == 0) {
        for (int c = 4 * threadIdx.x; c < hidden; c += 4 * blockDim.x) ln_store4(dst + c, *reinterpret_cast<const float4*>(buf + c));
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = from_f32<T>(buf[c]);
    }
}

// Loads one row into ``buf`` (fp32, 16-byte aligned; it may be the row itself) and leaves there its normed values.
template <typename In>
__device__ __forceinline__ void norm_row_into(const In* src, float* buf, const float* __restrict__ w,
                                              const float* __restrict__ b, int hidden, float eps, float* scratch) {
    const bool wide = (hidden & 3) == 0;
    float s = 0.f;
    if (wide) {
        for (int c = 4 * threadIdx.x; c < hidden; c += 4 * blockDim.x) {
            const float4 v = ln_load4(src + c);
            *reinterpret_cast<float4*>(buf + c) = v;
            s += (v.x + v.y) + (v.z + v.w);
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float v = to_f32(src[c]);
            buf[c] = v;
            s += v;
        }
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    float q = 0.f;
    if (wide) {
        for (int c = 4 * threadIdx.x; c < hidden; c += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(buf + c);
            const float d0 = v.x - mean, d1 = v.y - mean, d2 = v.z - mean, d3 = v.w - mean;
            q = fmaf(d0, d0, fmaf(d1, d1, fmaf(d2, d2, fmaf(d3, d3, q))));
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float d = buf[c] - mean;
            q = fmaf(d, d, q);
        }
    }
    const float var = block_sum(q, scratch) / (float)hidden;
    const float r = 1.0f / sqrtf(var + eps);
    if (wide) {
        for (int c = 4 * threadIdx.x; c < hidden; c += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(buf + c);
            const float4 w4 = *reinterpret_cast<const float4*>(w + c), b4 = *reinterpret_cast<const float4*>(b + c);
            *reinterpret_cast<float4*>(buf + c) = make_float4((v.x - mean) * r * w4.x + b4.x, (v.y - mean) * r * w4.y + b4.y,
                                                              (v.z - mean) * r * w4.z + b4.z, (v.w - mean) * r * w4.w + b4.w);
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) buf[c] = (buf[c] - mean) * r * w[c] + b[c];
    }
}

template <typename T>
__global__ void layernorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                      T* __restrict__ y, const int* __restrict__ rows, int hidden, float eps) {
    extern __shared__ float ln_smem[];
    float* buf = ln_smem;
    float* scratch = ln_smem + hidden;
    pdl_launch_dependents();
    pdl_wait();
    const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
    norm_row_into(x + src * hidden, buf, w, b, hidden, eps, scratch);
    __syncthreads();
    ln_write_row(y + (int64_t)blockIdx.x * hidden, buf, hidden);
}

// One block per token.  The block of a sequence's first token of the step takes h_{t-1} from the sequence's
// state (zeros at position 0) and afterwards leaves the h of the sequence's last token of the step there; no
// other block touches the state, so the read and the write are ordered.  Every other block norms row t-1 itself.
template <typename T>
__global__ void layernorm_shift_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                       const float* __restrict__ mu, float* __restrict__ state,
                                       const int* __restrict__ positions, const int* __restrict__ token_seq,
                                       const int* __restrict__ cu_q, const int* __restrict__ slots,
                                       T* __restrict__ y, int hidden, float eps) {
    extern __shared__ float ln_smem[];
    float* cur = ln_smem;
    float* prev = ln_smem + hidden;
    float* scratch = ln_smem + 2 * hidden;
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int seq = token_seq[t];
    const bool first = t == cu_q[seq];
    norm_row_into(x + (int64_t)t * hidden, cur, w, b, hidden, eps, scratch);
    float* st = nullptr;
    if (first) {
        st = state + (int64_t)slots[seq] * hidden;
        const bool start = positions[t] == 0;
        __syncthreads();                      // the state is read before this block writes it below
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) prev[c] = start ? 0.f : st[c];
    } else {
        norm_row_into(x + (int64_t)(t - 1) * hidden, prev, w, b, hidden, eps, scratch);
    }
    __syncthreads();
    T* yr = y + (int64_t)t * hidden;
    if ((hidden & 3) == 0) {
        for (int c = 4 * threadIdx.x; c < hidden; c += 4 * blockDim.x) {
            const float4 h = *reinterpret_cast<const float4*>(cur + c), pv = *reinterpret_cast<const float4*>(prev + c);
            const float4 m4 = *reinterpret_cast<const float4*>(mu + c);
            ln_store4(yr + c, make_float4(h.x + (pv.x - h.x) * m4.x, h.y + (pv.y - h.y) * m4.y, h.z + (pv.z - h.z) * m4.z,
                                          h.w + (pv.w - h.w) * m4.w));
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float h = cur[c];
            yr[c] = from_f32<T>(h + (prev[c] - h) * mu[c]);
        }
    }
    if (first) {
        const int last = cu_q[seq + 1] - 1;
        if (last == t) {
            for (int c = threadIdx.x; c < hidden; c += blockDim.x) st[c] = cur[c];
        } else {
            __syncthreads();
            norm_row_into(x + (int64_t)last * hidden, prev, w, b, hidden, eps, scratch);
            __syncthreads();
            for (int c = threadIdx.x; c < hidden; c += blockDim.x) st[c] = prev[c];
        }
    }
}

template <typename T>
__global__ void post_norm_add_kernel(float* __restrict__ x, const T* __restrict__ a, const float* __restrict__ w,
                                     const float* __restrict__ b, const float* __restrict__ w2,
                                     const float* __restrict__ b2, T* __restrict__ y, int hidden, float eps) {
    extern __shared__ float ln_smem[];
    float* buf = ln_smem;
    float* scratch = ln_smem + hidden;
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    norm_row_into(a + t * hidden, buf, w, b, hidden, eps, scratch);
    float* xr = x + t * hidden;
    __syncthreads();
    // the new stream goes to its place and stays in shared memory for the norm that follows
    if ((hidden & 3) == 0) {
        for (int c = 4 * threadIdx.x; c < hidden; c += 4 * blockDim.x) {
            const float4 n = *reinterpret_cast<const float4*>(buf + c), old = *reinterpret_cast<const float4*>(xr + c);
            const float4 v = make_float4(old.x + n.x, old.y + n.y, old.z + n.z, old.w + n.w);
            *reinterpret_cast<float4*>(xr + c) = v;
            *reinterpret_cast<float4*>(buf + c) = v;
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float v = xr[c] + buf[c];
            xr[c] = v;
            buf[c] = v;
        }
    }
    if (w2 == nullptr) return;
    __syncthreads();
    norm_row_into(buf, buf, w2, b2, hidden, eps, scratch);
    __syncthreads();
    ln_write_row(y + t * hidden, buf, hidden);
}

__global__ void stream_inject_kernel(float* __restrict__ x, const float* __restrict__ saved, const float* __restrict__ vec,
                                     int hidden, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = x[i];
    if (saved) v += saved[i];
    if (vec) v += vec[i % hidden];
    x[i] = v;
}

static inline int ln_threads(int hidden) { return hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128); }

template <typename Kernel>
static int ln_smem_ok(Kernel kern, size_t smem) {
    if (smem > 227 * 1024) return CPM_BAD_ARGUMENT;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return CPM_OK;
}

CPM_API int cpm_layernorm_rows(const float* x, const float* w, const float* b, void* y, const int* rows, int n_rows,
                               int hidden, float eps, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return CPM_OK;
    const size_t smem = (size_t)(hidden + 33) * sizeof(float);
    if (dtype == CPM_BF16) {
        auto kern = layernorm_rows_kernel<bf16>;
        if (int e = ln_smem_ok(kern, smem)) return e;
        cpm_launch(kLaunchNorm, kern, n_rows, ln_threads(hidden), smem, stream, x, w, b, (bf16*)y, rows, hidden, eps);
    } else {
        auto kern = layernorm_rows_kernel<float>;
        if (int e = ln_smem_ok(kern, smem)) return e;
        cpm_launch(kLaunchNorm, kern, n_rows, ln_threads(hidden), smem, stream, x, w, b, (float*)y, rows, hidden, eps);
    }
    return launch_status();
}

CPM_API int cpm_layernorm_shift(const float* x, const float* w, const float* b, const float* mu, float* state,
                                const int* positions, const int* token_seq, const int* cu_q, const int* slots, void* y,
                                int n_tokens, int hidden, float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    const size_t smem = (size_t)(2 * hidden + 33) * sizeof(float);
    if (dtype == CPM_BF16) {
        auto kern = layernorm_shift_kernel<bf16>;
        if (int e = ln_smem_ok(kern, smem)) return e;
        cpm_launch(kLaunchNorm, kern, n_tokens, ln_threads(hidden), smem, stream, x, w, b, mu, state, positions, token_seq,
                   cu_q, slots, (bf16*)y, hidden, eps);
    } else {
        auto kern = layernorm_shift_kernel<float>;
        if (int e = ln_smem_ok(kern, smem)) return e;
        cpm_launch(kLaunchNorm, kern, n_tokens, ln_threads(hidden), smem, stream, x, w, b, mu, state, positions, token_seq,
                   cu_q, slots, (float*)y, hidden, eps);
    }
    return launch_status();
}

CPM_API int cpm_post_norm_add(float* x, const void* a, const float* w, const float* b, const float* w2, const float* b2,
                              void* y, int n_tokens, int hidden, float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if ((w2 == nullptr) != (y == nullptr) || (w2 == nullptr) != (b2 == nullptr)) return CPM_BAD_ARGUMENT;
    const size_t smem = (size_t)(hidden + 33) * sizeof(float);
    if (dtype == CPM_BF16) {
        auto kern = post_norm_add_kernel<bf16>;
        if (int e = ln_smem_ok(kern, smem)) return e;
        cpm_launch(kLaunchNorm, kern, n_tokens, ln_threads(hidden), smem, stream, x, (const bf16*)a, w, b, w2, b2, (bf16*)y,
                   hidden, eps);
    } else {
        auto kern = post_norm_add_kernel<float>;
        if (int e = ln_smem_ok(kern, smem)) return e;
        cpm_launch(kLaunchNorm, kern, n_tokens, ln_threads(hidden), smem, stream, x, (const float*)a, w, b, w2, b2, (float*)y,
                   hidden, eps);
    }
    return launch_status();
}

CPM_API int cpm_stream_inject(float* x, const float* saved, const float* vec, int n_tokens, int hidden, cudaStream_t stream) {
    const int64_t n = (int64_t)n_tokens * hidden;
    if (n <= 0) return CPM_OK;
    const int threads = 256;
    stream_inject_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, stream>>>(x, saved, vec, hidden, n);
    return launch_status();
}
