// Embedding rows times a scale plus a sinusoidal position vector, into the fp32 residual stream:
//   out[t, 2i] = table[id_t, 2i] * scale + sin(p_t * f_i),   out[t, 2i+1] = table[id_t, 2i+1] * scale + cos(p_t * f_i)
// with f the table of hidden/2 frequencies that the host made in fp32.  Angles, sines and cosines are fp32
// (accurate sinf / cosf: an angle reaches thousands of radians).
#include "common.cuh"

template <typename T>
__global__ void embed_sinusoid_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                      const T* __restrict__ table, const float* __restrict__ freq,
                                      float* __restrict__ out, int hidden, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t row = ids[blockIdx.x];
    const float p = (float)positions[blockIdx.x];
    const T* src = table + row * hidden;
    float* dst = out + (int64_t)blockIdx.x * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float angle = p * freq[c >> 1];
        dst[c] = to_f32(src[c]) * scale + ((c & 1) ? cosf(angle) : sinf(angle));
    }
}

CPM_API int cpm_embed_sinusoid(const int* ids, const int* positions, const void* table, const float* freq, float* out,
                               int n_tokens, int hidden, float scale, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (hidden % 2) return CPM_BAD_ARGUMENT;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchOther, embed_sinusoid_kernel<bf16>, n_tokens, threads, 0, stream, ids, positions, (const bf16*)table,
                   freq, out, hidden, scale);
    else
        cpm_launch(kLaunchOther, embed_sinusoid_kernel<float>, n_tokens, threads, 0, stream, ids, positions, (const float*)table,
                   freq, out, hidden, scale);
    return launch_status();
}
