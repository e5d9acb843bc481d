// h = act(gate) * up for a row of [gate | up] values, with the activation chosen by a code: SiLU, or the
// tanh form of GELU, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).  Arithmetic in fp32.
// interleave == 0: a row is [gate(inter) | up(inter)]; interleave == n: blocks of n gate values followed by
// the n up values of the same features.
#include "common.cuh"

enum : int { CPM_ACT_SILU = 0, CPM_ACT_GELU_TANH = 1 };

__device__ __forceinline__ float act_apply(float z, int act) {
    if (act == CPM_ACT_GELU_TANH) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return z / (1.0f + expf(-z));
}

template <typename T>
__global__ void act_mul_kernel(const T* __restrict__ gu, T* __restrict__ h, int inter, int interleave, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int f = blockIdx.y * blockDim.x + threadIdx.x;
    if (f >= inter) return;
    const T* row = gu + (int64_t)blockIdx.x * 2 * inter;
    const int gi = interleave ? (f / interleave) * 2 * interleave + f % interleave : f;
    const int ui = interleave ? gi + interleave : inter + f;
    h[(int64_t)blockIdx.x * inter + f] = from_f32<T>(act_apply(to_f32(row[gi]), act) * to_f32(row[ui]));
}

CPM_API int cpm_act_mul(const void* gu, void* h, int n_tokens, int inter, int interleave, int act, int dtype,
                        cudaStream_t stream) {
    if (n_tokens <= 0 || inter <= 0) return CPM_OK;
    if (act != CPM_ACT_SILU && act != CPM_ACT_GELU_TANH) return CPM_BAD_ARGUMENT;
    if (interleave < 0 || (interleave && inter % interleave)) return CPM_BAD_ARGUMENT;
    const int threads = 256;
    dim3 grid(n_tokens, (inter + threads - 1) / threads);
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchOther, act_mul_kernel<bf16>, grid, threads, 0, stream, (const bf16*)gu, (bf16*)h, inter, interleave, act);
    else
        cpm_launch(kLaunchOther, act_mul_kernel<float>, grid, threads, 0, stream, (const float*)gu, (float*)h, inter, interleave, act);
    return launch_status();
}
