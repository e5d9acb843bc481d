// Routed experts: choice of experts per token, and the experts' products over the tokens that chose them.
//
// Routing (fp32): scores s = softmax(z) over all experts; choice scores c = s + correction; experts form
// ``n_groups`` equal groups of neighbours, a group's score is its largest choice score, and only experts of the
// ``keep`` best groups can be chosen (the others count as minus infinity); the ``top`` largest choice scores are
// chosen, and their weights are the plain scores s, not renormalised.  Ties go to the lower index.
//
// Products: the (token, choice) pairs are grouped by expert (counts, offsets, a list of pairs in expert order),
// and tiles of 32 pairs of one expert times 64 output features run as blocks of one launch, whose grid is an upper
// bound on the tile count (blocks beyond the last tile leave at once), so nothing is read back on the host:
//   gated:  H[r] = silu(x[token(r)] Wg_e^T) * (x[token(r)] Wu_e^T)     r: place in expert order
//   down:   Y[pair(r)] = H[r] Wd_e^T
// and a last kernel adds up a token's pairs with their weights and the shared expert's output times its gate.
// Accumulation is fp32 on the CUDA cores for both storage types.
#include "common.cuh"

constexpr int kRouteMaxPerLane = 16;      // experts <= 512

__device__ __forceinline__ ArgMax warp_argmax(ArgMax a) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = better(a, b);
    }
    return a;
}

// One warp per token.  logits rows of ``ld`` floats: the first E are the router's, column ``gate_col`` (if >= 0) is the
// shared expert's raw gate.
__global__ void moe_route_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ correction,
                                 int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ shared_gate,
                                 int gate_col, int n_tokens, int E, int top, int n_groups, int keep) {
    extern __shared__ float route_smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= n_tokens) return;
    float* s = route_smem + (size_t)warp * (2 * E + n_groups);      // scores
    float* c = s + E;                                                 // choice scores
    float* gs = c + E;                                                // group scores
    const float* z = logits + (int64_t)t * ld;
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float ex = expf(z[e] - m);
        s[e] = ex;
        sum += ex;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) {
        const float v = s[e] * inv;
        s[e] = v;
        c[e] = v + correction[e];
    }
    __syncwarp();
    const int per = E / n_groups;
    if (n_groups > 1 && keep < n_groups) {
        for (int g = lane; g < n_groups; g += 32) {
            float best = -INFINITY;
            for (int i = 0; i < per; ++i) best = fmaxf(best, c[g * per + i]);
            gs[g] = best;
        }
        __syncwarp();
        // the groups that are not kept: all but the ``keep`` best; a kept group is marked by a score of +inf
        for (int r = 0; r < keep; ++r) {
            ArgMax a{-INFINITY, 0x7fffffff};
            for (int g = lane; g < n_groups; g += 32) {
                const float v = gs[g];
                if (v != INFINITY) a = better(a, ArgMax{v, g});
            }
            a = warp_argmax(a);
            if (lane == 0 && a.i < n_groups) gs[a.i] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) c[e] = -INFINITY;
        __syncwarp();
    }
    for (int r = 0; r < top; ++r) {
        ArgMax a{-INFINITY, 0x7fffffff};
        for (int e = lane; e < E; e += 32) {
            const float v = c[e];
            if (!isnan(v)) a = better(a, ArgMax{v, e});
        }
        a = warp_argmax(a);
        const int e = a.i < E ? a.i : 0;
        if (lane == 0) {
            chosen[(int64_t)t * top + r] = e;
            weights[(int64_t)t * top + r] = s[e];
            c[e] = NAN;                                   // taken
        }
        __syncwarp();
    }
    if (gate_col >= 0 && lane == 0) shared_gate[t] = 1.0f / (1.0f + expf(-z[gate_col]));
}

// One block: pairs per expert, offsets, and the pairs listed in expert order.
__global__ void moe_group_kernel(const int* __restrict__ chosen, int n_pairs, int E, int* __restrict__ offsets /* [E+1] */,
                                 int* __restrict__ order /* [pairs] */) {
    extern __shared__ int group_smem[];      // counts [E], cursor [E]
    int* counts = group_smem;
    int* cursor = counts + E;
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&counts[chosen[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = at;
            cursor[e] = at;
            at += counts[e];
        }
        offsets[E] = at;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) order[atomicAdd(&cursor[chosen[i]], 1)] = i;
}

constexpr int kTileM = 32, kTileN = 64, kTileK = 32;

// C[row_out(r)][n] = sum_k A[row_in(r)][k] * B_e[n][k] for the places r of expert e, tile by tile.
// GATED: A rows are tokens (pair / top), two weight stacks (gate, up) and the result is silu(gate) * up, written at
// row r.  Otherwise A rows are the places r themselves and the result goes to row pair(r).
template <typename T, bool GATED>
__global__ void __launch_bounds__(256)
moe_tile_kernel(const T* __restrict__ A, const T* __restrict__ B0, const T* __restrict__ B1, T* __restrict__ C,
                const int* __restrict__ offsets, const int* __restrict__ order, int E, int top, int N, int K) {
    __shared__ float As[kTileM][kTileK + 1], Bs0[kTileN][kTileK + 1], Bs1[GATED ? kTileN : 1][kTileK + 1];
    __shared__ int s_tile[3];
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        int tile = blockIdx.x, e = 0, found = -1, first = 0;
        for (; e < E; ++e) {
            const int n = offsets[e + 1] - offsets[e];
            const int tiles = (n + kTileM - 1) / kTileM;
            if (tile < tiles) { found = e; first = offsets[e] + tile * kTileM; break; }
            tile -= tiles;
        }
        s_tile[0] = found;
        s_tile[1] = first;
        s_tile[2] = found >= 0 ? min(kTileM, offsets[found + 1] - first) : 0;
    }
    __syncthreads();
    const int e = s_tile[0], r0 = s_tile[1], rows = s_tile[2];
    if (e < 0) return;
    const int n0 = blockIdx.y * kTileN;
    const T* W0 = B0 + (int64_t)e * N * K;
    const T* W1 = GATED ? B1 + (int64_t)e * N * K : nullptr;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // 4 columns, 2 rows a thread
    float acc0[2][4] = {}, acc1[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += kTileK) {
        for (int i = threadIdx.x; i < kTileM * kTileK; i += 256) {
            const int r = i / kTileK, kk = i % kTileK;
            float v = 0.f;
            if (r < rows && k0 + kk < K) {
                const int64_t src = GATED ? (int64_t)(order[r0 + r] / top) : (int64_t)(r0 + r);
                v = to_f32(A[src * K + k0 + kk]);
            }
            As[r][kk] = v;
        }
        for (int i = threadIdx.x; i < kTileN * kTileK; i += 256) {
            const int n = i / kTileK, kk = i % kTileK;
            const bool ok = n0 + n < N && k0 + kk < K;
            Bs0[n][kk] = ok ? to_f32(W0[(int64_t)(n0 + n) * K + k0 + kk]) : 0.f;
            if (GATED) Bs1[n][kk] = ok ? to_f32(W1[(int64_t)(n0 + n) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < kTileK; ++kk) {
            const float a0 = As[ty * 2][kk], a1 = As[ty * 2 + 1][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = Bs0[tx * 4 + j][kk];
                acc0[0][j] = fmaf(a0, b, acc0[0][j]);
                acc0[1][j] = fmaf(a1, b, acc0[1][j]);
                if (GATED) {
                    const float b1 = Bs1[tx * 4 + j][kk];
                    acc1[0][j] = fmaf(a0, b1, acc1[0][j]);
                    acc1[1][j] = fmaf(a1, b1, acc1[1][j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty * 2 + i;
        if (r >= rows) continue;
        const int64_t dst = GATED ? (int64_t)(r0 + r) : (int64_t)order[r0 + r];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc0[i][j];
            if (GATED) v = v / (1.0f + expf(-v)) * acc1[i][j];
            C[dst * N + n] = from_f32<T>(v);
        }
    }
}


// The same products for bf16 on the tensor cores (mma.sync m16n8k16, fp32 accumulation): tiles of 64 places of one
// expert times 64 output features, four warps of 16 rows each, K in steps of 32 through shared memory (rows padded to
// 40 elements: the fragments' 32-bit loads then hit 32 different banks), the next step's global loads issued before
// the current step's products.  K must be a multiple of 8 (16-byte loads).
constexpr int kMmaM = 64, kMmaN = 64, kMmaK = 32, kMmaPad = 40;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool GATED>
__global__ void __launch_bounds__(128)
moe_tile_mma_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B0, const bf16* __restrict__ B1, bf16* __restrict__ C,
                    const int* __restrict__ offsets, const int* __restrict__ order, int E, int top, int N, int K) {
    __shared__ __align__(16) bf16 As[kMmaM][kMmaPad], Bs0[kMmaN][kMmaPad], Bs1[GATED ? kMmaN : 1][kMmaPad];
    __shared__ int s_tile[3];
    __shared__ int s_rows[kMmaM];
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        int tile = blockIdx.x, e = 0, found = -1, first = 0;
        for (; e < E; ++e) {
            const int n = offsets[e + 1] - offsets[e];
            const int tiles = (n + kMmaM - 1) / kMmaM;
            if (tile < tiles) { found = e; first = offsets[e] + tile * kMmaM; break; }
            tile -= tiles;
        }
        s_tile[0] = found;
        s_tile[1] = first;
        s_tile[2] = found >= 0 ? min(kMmaM, offsets[found + 1] - first) : 0;
    }
    __syncthreads();
    const int e = s_tile[0], r0 = s_tile[1], rows = s_tile[2];
    if (e < 0) return;
    if (threadIdx.x < kMmaM) {
        const int r = threadIdx.x;
        s_rows[r] = r < rows ? order[r0 + r] : -1;          // the pair at this place
    }
    __syncthreads();
    const int n0 = blockIdx.y * kMmaN;
    const bf16* W0 = B0 + (int64_t)e * N * K;
    const bf16* W1 = GATED ? B1 + (int64_t)e * N * K : nullptr;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, j = lane & 3;
    // a thread's two 16-byte pieces of each tile: piece p covers row (p >> 2), elements 8 * (p & 3) ..
    uint4 ra[2], rb0[2], rb1[2];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int p = threadIdx.x + 128 * i, r = p >> 2, kk = k0 + 8 * (p & 3);
            ra[i] = rb0[i] = rb1[i] = make_uint4(0, 0, 0, 0);
            if (kk < K) {
                const int pair = s_rows[r];
                if (pair >= 0) ra[i] = *reinterpret_cast<const uint4*>(A + (int64_t)(GATED ? pair / top : r0 + r) * K + kk);
                if (n0 + r < N) {
                    rb0[i] = *reinterpret_cast<const uint4*>(W0 + (int64_t)(n0 + r) * K + kk);
                    if (GATED) rb1[i] = *reinterpret_cast<const uint4*>(W1 + (int64_t)(n0 + r) * K + kk);
                }
            }
        }
    };
    float acc0[8][4] = {}, acc1[GATED ? 8 : 1][4] = {};
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += kMmaK) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int p = threadIdx.x + 128 * i, r = p >> 2, c = 8 * (p & 3);
            *reinterpret_cast<uint4*>(&As[r][c]) = ra[i];
            *reinterpret_cast<uint4*>(&Bs0[r][c]) = rb0[i];
            if (GATED) *reinterpret_cast<uint4*>(&Bs1[r][c]) = rb1[i];
        }
        __syncthreads();
        if (k0 + kMmaK < K) fetch(k0 + kMmaK);
#pragma unroll
        for (int ks = 0; ks < kMmaK; ks += 16) {
            uint32_t a[4];
            a[0] = *reinterpret_cast<const uint32_t*>(&As[warp * 16 + g][ks + 2 * j]);
            a[1] = *reinterpret_cast<const uint32_t*>(&As[warp * 16 + g + 8][ks + 2 * j]);
            a[2] = *reinterpret_cast<const uint32_t*>(&As[warp * 16 + g][ks + 2 * j + 8]);
            a[3] = *reinterpret_cast<const uint32_t*>(&As[warp * 16 + g + 8][ks + 2 * j + 8]);
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&Bs0[nt * 8 + g][ks + 2 * j]);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&Bs0[nt * 8 + g][ks + 2 * j + 8]);
                mma_bf16_16816(acc0[nt], a, b0, b1);
                if (GATED) {
                    const uint32_t u0 = *reinterpret_cast<const uint32_t*>(&Bs1[nt * 8 + g][ks + 2 * j]);
                    const uint32_t u1 = *reinterpret_cast<const uint32_t*>(&Bs1[nt * 8 + g][ks + 2 * j + 8]);
                    mma_bf16_16816(acc1[nt], a, u0, u1);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + g + 8 * half;
        if (r >= rows) continue;
        const int64_t dst = GATED ? (int64_t)(r0 + r) : (int64_t)s_rows[r];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int n = n0 + nt * 8 + 2 * j + q;
                if (n >= N) continue;
                float v = acc0[nt][2 * half + q];
                if (GATED) v = v / (1.0f + expf(-v)) * acc1[nt][2 * half + q];
                C[dst * N + n] = __float2bfloat16_rn(v);
            }
        }
    }
}

// out[t] = sum_k weights[t][k] * Y[t * top + k] + gate[t] * shared[t]
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ Y, const float* __restrict__ weights, const T* __restrict__ shared,
                                   const float* __restrict__ gate, T* __restrict__ out, int top, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v = 0.f;
        for (int k = 0; k < top; ++k) v = fmaf(weights[t * top + k], to_f32(Y[(t * top + k) * W + c]), v);
        if (shared) v = fmaf(gate ? gate[t] : 1.f, to_f32(shared[t * W + c]), v);
        out[t * W + c] = from_f32<T>(v);
    }
}

static int g_moe_tensor_cores = 1;
// 0: the bf16 products stay on the CUDA cores too (for comparisons and tests)
CPM_API int cpm_set_moe_tensor_cores(int on) {
    g_moe_tensor_cores = on;
    return CPM_OK;
}

CPM_API int cpm_moe_route(const float* logits, int ld, const float* correction, int* chosen, float* weights, float* shared_gate,
                          int gate_col, int n_tokens, int E, int top, int n_groups, int keep, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (E < 1 || E > 32 * kRouteMaxPerLane || top < 1 || top > E || n_groups < 1 || E % n_groups || keep < 1 || keep > n_groups ||
        top > keep * (E / n_groups))
        return CPM_BAD_ARGUMENT;
    const int warps = 4;
    const size_t smem = (size_t)warps * (2 * E + n_groups) * sizeof(float);
    cpm_launch(kLaunchOther, moe_route_kernel, dim3((n_tokens + warps - 1) / warps), dim3(warps * 32), smem, stream, logits, ld,
               correction, chosen, weights, shared_gate, gate_col, n_tokens, E, top, n_groups, keep);
    return launch_status();
}

CPM_API int cpm_moe_group(const int* chosen, int n_pairs, int E, int* offsets, int* order, cudaStream_t stream) {
    if (n_pairs <= 0) return CPM_OK;
    if (E < 1 || E > 4096) return CPM_BAD_ARGUMENT;
    cpm_launch(kLaunchOther, moe_group_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), stream, chosen, n_pairs, E, offsets,
               order);
    return launch_status();
}

// gated != 0: A = x [tokens, K], B0 = gate stack [E, N, K], B1 = up stack, C = H [pairs, N] in expert order.
// gated == 0: A = H [pairs, K] in expert order, B0 = down stack [E, N, K], C = Y [pairs, N] by pair.
CPM_API int cpm_moe_expert_product(const void* A, const void* B0, const void* B1, void* C, const int* offsets, const int* order,
                                   int n_pairs, int E, int top, int N, int K, int gated, int dtype, cudaStream_t stream) {
    if (n_pairs <= 0) return CPM_OK;
    if (E < 1 || top < 1 || N < 1 || K < 1) return CPM_BAD_ARGUMENT;
    if (dtype == CPM_BF16 && K % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)B0 & 15) == 0 && ((uintptr_t)B1 & 15) == 0 &&
        g_moe_tensor_cores) {
        const dim3 mgrid((n_pairs + kMmaM - 1) / kMmaM + E, (N + kMmaN - 1) / kMmaN);
        if (mgrid.y > 65535) return CPM_BAD_ARGUMENT;
        if (gated)
            cpm_launch(kLaunchProduct, moe_tile_mma_kernel<true>, mgrid, dim3(128), 0, stream, (const bf16*)A, (const bf16*)B0,
                       (const bf16*)B1, (bf16*)C, offsets, order, E, top, N, K);
        else
            cpm_launch(kLaunchProduct, moe_tile_mma_kernel<false>, mgrid, dim3(128), 0, stream, (const bf16*)A, (const bf16*)B0,
                       (const bf16*)B1, (bf16*)C, offsets, order, E, top, N, K);
        return launch_status();
    }
    const dim3 grid((n_pairs + kTileM - 1) / kTileM + E, (N + kTileN - 1) / kTileN);
    if (grid.y > 65535) return CPM_BAD_ARGUMENT;
#define CPM_MOE(TT, G) cpm_launch(kLaunchProduct, moe_tile_kernel<TT, G>, grid, dim3(256), 0, stream, (const TT*)A, (const TT*)B0, \
                                  (const TT*)B1, (TT*)C, offsets, order, E, top, N, K)
    if (dtype == CPM_BF16) { if (gated) CPM_MOE(bf16, true); else CPM_MOE(bf16, false); }
    else { if (gated) CPM_MOE(float, true); else CPM_MOE(float, false); }
#undef CPM_MOE
    return launch_status();
}

CPM_API int cpm_moe_combine(const void* Y, const float* weights, const void* shared, const float* gate, void* out, int n_tokens,
                            int top, int W, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    const dim3 block(W >= 1024 ? 256 : 128);
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchNorm, moe_combine_kernel<bf16>, dim3(n_tokens), block, 0, stream, (const bf16*)Y, weights, (const bf16*)shared,
                   gate, (bf16*)out, top, W);
    else
        cpm_launch(kLaunchNorm, moe_combine_kernel<float>, dim3(n_tokens), block, 0, stream, (const float*)Y, weights,
                   (const float*)shared, gate, (float*)out, top, W);
    return launch_status();
}
