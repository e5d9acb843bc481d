// A gated recurrence whose gates read only the current token (minGRU), one state value per channel:
//
//   z_t = sigmoid(zr_t + bz)          g(u) = u + 1/2 where u >= 0, sigmoid(u) where u < 0
//   S_t = (1 - z_t) S_{t-1} + z_t g(ur_t + bx)
//   out_t = S_t * silu(gr_t)
//
// zr, ur, gr are the three thirds of a row of the fused projection [tokens, 3 * width] (fp32); the biases, the
// gates, the state and the recurrence are fp32; only ``out`` has the storage type.  The state of a sequence lives
// in a per-sequence tensor [slots, width] and is carried from step to step (zeros at position 0).
//
// Two forms.  mingru_scan_seq: one thread per (sequence, channel) walks the sequence's tokens of the step; it is
// the form of decode steps and of short pieces.  mingru_tile_summary + mingru_tile_apply: the recurrence is
// linear, S_out = A S_in + B over any run of tokens, so every tile of consecutive tokens first reduces to its
// (A, B); a sequence's first tile also notes the carried state there, so that nothing reads the state after the
// first kernel.  The second kernel starts from that note, composes the tiles before its own, walks its tokens
// and, in the sequence's last tile, leaves the new state.  Tiles of one sequence are listed consecutively in
// rising order, ``tile_tokens`` apart.
#include "common.cuh"

__device__ __forceinline__ float sigmoid_f32(float v) { return 1.0f / (1.0f + expf(-v)); }

constexpr int kGruBatch = 16;     // tokens whose projections are loaded before the first is used

struct GruStep { float a, b; };      // S <- a * S + b

__device__ __forceinline__ GruStep mingru_gates(float zr, float ur) {
    const float z = sigmoid_f32(zr);
    const float cand = ur >= 0.f ? ur + 0.5f : sigmoid_f32(ur);
    return GruStep{1.0f - z, z * cand};
}

template <typename T>
__global__ void mingru_scan_seq_kernel(const float* __restrict__ proj, const float* __restrict__ bz, const float* __restrict__ bx,
                                       float* __restrict__ state, const int* __restrict__ positions,
                                       const int* __restrict__ cu_q, const int* __restrict__ slots, T* __restrict__ out,
                                       int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int seq = blockIdx.y;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    if (t1 <= t0) return;
    float* st = state + (int64_t)slots[seq] * width + c;
    float S = positions[t0] == 0 ? 0.f : *st;
    const float bzc = bz[c], bxc = bx[c];
    for (int tb = t0; tb < t1; tb += kGruBatch) {
        float zr[kGruBatch], ur[kGruBatch], gr[kGruBatch];
#pragma unroll
        for (int u = 0; u < kGruBatch; ++u) {
            const float* row = proj + (int64_t)min(tb + u, t1 - 1) * 3 * width + c;
            zr[u] = row[0];
            ur[u] = row[width];
            gr[u] = row[2 * width];
        }
#pragma unroll
        for (int u = 0; u < kGruBatch; ++u) {
            if (tb + u < t1) {
                const GruStep g = mingru_gates(zr[u] + bzc, ur[u] + bxc);
                S = fmaf(g.a, S, g.b);
                out[(int64_t)(tb + u) * width + c] = from_f32<T>(S * (gr[u] * sigmoid_f32(gr[u])));
            }
        }
    }
    *st = S;
}

__global__ void mingru_tile_summary_kernel(const float* __restrict__ proj, const float* __restrict__ bz,
                                           const float* __restrict__ bx, const float* __restrict__ state,
                                           const int* __restrict__ positions, const int* __restrict__ cu_q,
                                           const int* __restrict__ slots, const int* __restrict__ tile_seq,
                                           const int* __restrict__ tile_row, float* __restrict__ summary /* [tiles][3][width] */,
                                           int width, int tile_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int tile = blockIdx.y;
    const int seq = tile_seq[tile], row0 = tile_row[tile];
    const int t0 = cu_q[seq] + row0, t1 = min(t0 + tile_tokens, cu_q[seq + 1]);
    float A = 1.f, B = 0.f, carried = 0.f;
    if (t1 > t0) {
        if (row0 == 0 && positions[t0] != 0) carried = state[(int64_t)slots[seq] * width + c];
        const float bzc = bz[c], bxc = bx[c];
        for (int tb = t0; tb < t1; tb += kGruBatch) {
            float zr[kGruBatch], ur[kGruBatch];
#pragma unroll
            for (int u = 0; u < kGruBatch; ++u) {
                const float* row = proj + (int64_t)min(tb + u, t1 - 1) * 3 * width + c;
                zr[u] = row[0];
                ur[u] = row[width];
            }
#pragma unroll
            for (int u = 0; u < kGruBatch; ++u) {
                if (tb + u < t1) {
                    const GruStep g = mingru_gates(zr[u] + bzc, ur[u] + bxc);
                    B = fmaf(g.a, B, g.b);
                    A *= g.a;
                }
            }
        }
    }
    float* s = summary + (int64_t)tile * 3 * width + c;
    s[0] = A;
    s[width] = B;
    s[2 * width] = carried;
}

template <typename T>
__global__ void mingru_tile_apply_kernel(const float* __restrict__ proj, const float* __restrict__ bz, const float* __restrict__ bx,
                                         float* __restrict__ state, const int* __restrict__ cu_q, const int* __restrict__ slots,
                                         const int* __restrict__ tile_seq, const int* __restrict__ tile_row,
                                         const float* __restrict__ summary, T* __restrict__ out, int width, int tile_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int tile = blockIdx.y;
    const int seq = tile_seq[tile], row0 = tile_row[tile];
    const int t0 = cu_q[seq] + row0, end = cu_q[seq + 1], t1 = min(t0 + tile_tokens, end);
    if (t1 <= t0) return;
    const int first = tile - row0 / tile_tokens;
    float S = summary[((int64_t)first * 3 + 2) * width + c];
    for (int j = first; j < tile; ++j) {
        const float* s = summary + (int64_t)j * 3 * width + c;
        S = fmaf(s[0], S, s[width]);
    }
    const float bzc = bz[c], bxc = bx[c];
    for (int tb = t0; tb < t1; tb += kGruBatch) {
        float zr[kGruBatch], ur[kGruBatch], gr[kGruBatch];
#pragma unroll
        for (int u = 0; u < kGruBatch; ++u) {
            const float* row = proj + (int64_t)min(tb + u, t1 - 1) * 3 * width + c;
            zr[u] = row[0];
            ur[u] = row[width];
            gr[u] = row[2 * width];
        }
#pragma unroll
        for (int u = 0; u < kGruBatch; ++u) {
            if (tb + u < t1) {
                const GruStep g = mingru_gates(zr[u] + bzc, ur[u] + bxc);
                S = fmaf(g.a, S, g.b);
                out[(int64_t)(tb + u) * width + c] = from_f32<T>(S * (gr[u] * sigmoid_f32(gr[u])));
            }
        }
    }
    if (t1 == end) state[(int64_t)slots[seq] * width + c] = S;
}

CPM_API int64_t cpm_mingru_summary_floats(int n_tiles, int width) { return (int64_t)n_tiles * 3 * width; }

// tile_seq == nullptr: one thread per (sequence, channel) walks the sequence's tokens.  Otherwise the two-kernel
// form over ``n_tiles`` tiles of ``tile_tokens`` tokens, with ``summary`` of cpm_mingru_summary_floats floats.
CPM_API int cpm_mingru_scan(const float* proj, const float* bz, const float* bx, float* state, const int* positions,
                            const int* cu_q, const int* slots, const int* tile_seq, const int* tile_row, int n_tiles,
                            int tile_tokens, float* summary, void* out, int n_seqs, int width, int dtype,
                            cudaStream_t stream) {
    if (n_seqs <= 0 || width <= 0) return CPM_OK;
    const int threads = 128;
    const unsigned bx_ = (unsigned)((width + threads - 1) / threads);
    if (tile_seq == nullptr) {
        if (n_seqs > 65535) return CPM_BAD_ARGUMENT;
        dim3 grid(bx_, n_seqs);
        if (dtype == CPM_BF16)
            cpm_launch(kLaunchNorm, mingru_scan_seq_kernel<bf16>, grid, threads, 0, stream, proj, bz, bx, state, positions, cu_q,
                       slots, (bf16*)out, width);
        else
            cpm_launch(kLaunchNorm, mingru_scan_seq_kernel<float>, grid, threads, 0, stream, proj, bz, bx, state, positions, cu_q,
                       slots, (float*)out, width);
        return launch_status();
    }
    if (n_tiles <= 0) return CPM_OK;
    if (n_tiles > 65535 || tile_tokens <= 0 || summary == nullptr) return CPM_BAD_ARGUMENT;
    dim3 grid(bx_, n_tiles);
    cpm_launch(kLaunchNorm, mingru_tile_summary_kernel, grid, threads, 0, stream, proj, bz, bx, (const float*)state, positions,
               cu_q, slots, tile_seq, tile_row, summary, width, tile_tokens);
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchNorm, mingru_tile_apply_kernel<bf16>, grid, threads, 0, stream, proj, bz, bx, state, cu_q, slots,
                   tile_seq, tile_row, (const float*)summary, (bf16*)out, width, tile_tokens);
    else
        cpm_launch(kLaunchNorm, mingru_tile_apply_kernel<float>, grid, threads, 0, stream, proj, bz, bx, state, cu_q, slots,
                   tile_seq, tile_row, (const float*)summary, (float*)out, width, tile_tokens);
    return launch_status();
}
