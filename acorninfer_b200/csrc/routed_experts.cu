// A routed mixture of experts: the router's choice, the grouping of tokens by expert, a matrix
// product per expert over its tokens, and the weighted sum.
//
//   moe_route     per token: s = softmax(z) over all N router outputs; the choice score is s + correction;
//                 the outputs form `groups` equal groups of neighbours, a group's score is its largest choice
//                 score, and only outputs of the `keep` best groups can be chosen; the `top` largest choice
//                 scores win; their weights are s itself (not renormalized).  float32 throughout.
//   moe_plan      counts per expert, offsets (exclusive sums) and a slot for every (token, choice) pair,
//                 so that the pairs of an expert are neighbours: slot_token[slot], slot_of[pair].
//   grouped_gemm  C[slot, :] = A[row(slot), :] W_e^T for the slots of every expert e < E
//   moe_combine   out[t] = sum_k weight_k * (chosen_k >= E ? x[t] : y[slot_of(t, k)])
//                 (router outputs from E on are identity experts: they return their input)
#include "common.cuh"

// One warp per token.  Ties go to the lower index.
__global__ void moe_route_kernel(const float* __restrict__ z, const float* __restrict__ correction,
                                 int* __restrict__ idx, float* __restrict__ wts, int tokens, int N, int top, int groups,
                                 int keep) {
    extern __shared__ float sm[];                       // per warp: s[N], choice[N]
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= tokens) return;
    float* s = sm + (size_t)warp * 2 * N;
    float* choice = s + N;
    const float* zr = z + (int64_t)t * N;
    float m = -INFINITY;
    for (int i = lane; i < N; i += 32) m = fmaxf(m, zr[i]);
    m = warp_max(m);
    float sum = 0.f;
    for (int i = lane; i < N; i += 32) {
        const float e = expf(zr[i] - m);
        s[i] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    for (int i = lane; i < N; i += 32) {
        s[i] = s[i] / sum;
        choice[i] = s[i] + correction[i];
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        // the `keep` groups with the largest best choice score, found one by one; a bit per kept group
        const int per = N / groups;
        unsigned long long kept_lo = 0ull;              // groups <= 64: bit per kept group
        for (int round = 0; round < keep; ++round) {
            float best = -INFINITY;
            int best_g = groups;
            for (int gi = lane; gi < groups; gi += 32) {
                if ((kept_lo >> gi) & 1ull) continue;
                float gm = -INFINITY;
                for (int i = gi * per; i < (gi + 1) * per; ++i) gm = fmaxf(gm, choice[i]);
                if (gm > best || (gm == best && gi < best_g)) {
                    best = gm;
                    best_g = gi;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
                if (ob > best || (ob == best && og < best_g)) {
                    best = ob;
                    best_g = og;
                }
            }
            if (best_g < groups) kept_lo |= 1ull << best_g;
        }
        for (int i = lane; i < N; i += 32)
            if (!((kept_lo >> (i / per)) & 1ull)) choice[i] = -INFINITY;
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_i = N;
        for (int i = lane; i < N; i += 32) {
            const float c = choice[i];
            if (c > best || (c == best && i < best_i && c > -INFINITY)) {
                best = c;
                best_i = i;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ob > best || (ob == best && oi < best_i)) {
                best = ob;
                best_i = oi;
            }
        }
        if (best_i >= N) best_i = 0;                    // nothing left to choose (top > allowed outputs): weight 0
        if (lane == 0) {
            idx[(int64_t)t * top + k] = best_i;
            wts[(int64_t)t * top + k] = best > -INFINITY ? s[best_i] : 0.f;
            choice[best_i] = -INFINITY;
        }
        __syncwarp();
    }
}

extern "C" int acorn_moe_route(const float* z, const float* correction, int* idx, float* wts, int tokens, int N, int top,
                               int groups, int keep, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (N < 1 || top < 1 || top > N || groups < 1 || groups > 64 || N % groups || keep < 1 || keep > groups || N > 2048)
        return ACORN_ERR_UNSUPPORTED;
    const int warps = 4;
    const size_t smem = (size_t)warps * 2 * N * sizeof(float);
    static AcornPerDevice configured;
    if (smem > 48 * 1024 && !configured.seen()) {
        cudaError_t e = cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 2 * 2048 * 4);
        if (e != cudaSuccess) return (int)e;
        configured.mark();
    }
    return acorn_launch(moe_route_kernel, dim3((tokens + warps - 1) / warps), dim3(32 * warps), smem, stream, z, correction,
                        idx, wts, tokens, N, top, groups, keep);
}

// One block: histogram of the chosen outputs, exclusive sums, then a slot for every pair.  Within an
// expert the slots are handed out in whatever order the threads arrive: a row's result does not
// depend on its slot.
__global__ void moe_plan_kernel(const int* __restrict__ idx, int* __restrict__ offsets, int* __restrict__ slot_of,
                                int* __restrict__ slot_token, int pairs, int N, int top) {
    extern __shared__ int cnt[];                        // [N] counts, then [N] cursors
    pdl_wait();
    pdl_trigger();
    int* cursor = cnt + N;
    for (int i = threadIdx.x; i < N; i += blockDim.x) cnt[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&cnt[idx[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < N; ++i) {
            offsets[i] = run;
            cursor[i] = run;
            run += cnt[i];
        }
        offsets[N] = run;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int slot = atomicAdd(&cursor[idx[i]], 1);
        slot_of[i] = slot;
        slot_token[slot] = i / top;
    }
}

extern "C" int acorn_moe_plan(const int* idx, int* offsets, int* slot_of, int* slot_token, int pairs, int N, int top,
                              cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (N > 4096) return ACORN_ERR_UNSUPPORTED;
    return acorn_launch(moe_plan_kernel, dim3(1), dim3(1024), (size_t)2 * N * sizeof(int), stream, idx, offsets, slot_of,
                        slot_token, pairs, N, top);
}

// ---------------------------------------------------------------- a product per expert
// Slots offsets[e] .. offsets[e+1]-1 belong to expert e.  Row `slot` of A is a_rows ? A[a_rows[slot]] : A[slot].
// A block finds its (expert, tile of GG_BM slots) by walking the offsets; blocks beyond the last tile
// leave.  float32 accumulation, one chain over k = 0, 1, ... per output.
#define GG_BM 32
#define GG_BN 64
#define GG_BK 32

template <typename T>
__global__ void __launch_bounds__(256) grouped_gemm_kernel(const T* __restrict__ A, int64_t lda, const int* __restrict__ a_rows,
                                                           const T* __restrict__ W, T* __restrict__ C, int64_t ldc,
                                                           const int* __restrict__ offsets, int E, int N, int K) {
    __shared__ float as[GG_BM][GG_BK + 1];
    __shared__ float ws[GG_BN][GG_BK + 1];
    __shared__ int s_e, s_first, s_end;
    pdl_wait();
    pdl_trigger();
    if (threadIdx.x == 0) {
        int tile = blockIdx.y, e = 0, found = -1;
        for (; e < E; ++e) {
            const int n = offsets[e + 1] - offsets[e];
            const int tiles = (n + GG_BM - 1) / GG_BM;
            if (tile < tiles) {
                found = e;
                break;
            }
            tile -= tiles;
        }
        s_e = found;
        if (found >= 0) {
            s_first = offsets[found] + tile * GG_BM;
            s_end = offsets[found + 1];
        }
    }
    __syncthreads();
    const int e = s_e;
    if (e < 0) return;
    const int first = s_first, end = s_end;
    const int n0 = blockIdx.x * GG_BN;
    const T* We = W + (int64_t)e * N * K;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 16 column groups of 4, 16 row pairs
    float acc[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += GG_BK) {
        for (int i = threadIdx.x; i < GG_BM * GG_BK; i += 256) {
            const int rr = i / GG_BK, kk = i % GG_BK;
            const int slot = first + rr, k = k0 + kk;
            float v = 0.f;
            if (slot < end && k < K) {
                const int64_t row = a_rows ? a_rows[slot] : slot;
                v = to_float(A[row * lda + k]);
            }
            as[rr][kk] = v;
        }
        for (int i = threadIdx.x; i < GG_BN * GG_BK; i += 256) {
            const int nn = i / GG_BK, kk = i % GG_BK;
            const int n = n0 + nn, k = k0 + kk;
            ws[nn][kk] = (n < N && k < K) ? to_float(We[(int64_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GG_BK; ++kk) {
            const float a0 = as[ty][kk], a1 = as[ty + 16][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float w = ws[tx + 16 * j][kk];
                acc[0][j] = fmaf(a0, w, acc[0][j]);
                acc[1][j] = fmaf(a1, w, acc[1][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int slot = first + ty + 16 * i;
        if (slot >= end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n < N) C[(int64_t)slot * ldc + n] = from_float<T>(acc[i][j]);
        }
    }
}

extern "C" int acorn_grouped_gemm(const void* A, int64_t lda, const int* a_rows, const void* W, void* C, int64_t ldc,
                                  const int* offsets, int slots, int E, int N, int K, int dtype, cudaStream_t stream) {
    if (slots <= 0 || E <= 0 || N <= 0) return 0;
    const int64_t tiles = (slots + GG_BM - 1) / GG_BM + E;       // every expert may end in a partly filled tile
    if (tiles > 65535) return ACORN_ERR_UNSUPPORTED;
    dim3 grid((N + GG_BN - 1) / GG_BN, (unsigned)tiles);
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(grouped_gemm_kernel<T>, grid, dim3(256), 0, stream, (const T*)A, lda,
                                                       a_rows, (const T*)W, (T*)C, ldc, offsets, E, N, K));
    return ACORN_ERR_UNSUPPORTED;
}

// out[t, :] = sum over the token's choices, in their order
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const T* __restrict__ x, const int* __restrict__ slot_of,
                                   const int* __restrict__ idx, const float* __restrict__ wts, T* __restrict__ out, int H,
                                   int top, int E) {
    pdl_wait();
    pdl_trigger();
    const int64_t t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int64_t p = t * top + k;
            const float v = idx[p] >= E ? to_float(x[t * H + i]) : to_float(y[(int64_t)slot_of[p] * H + i]);
            acc = fmaf(wts[p], v, acc);
        }
        out[t * H + i] = from_float<T>(acc);
    }
}

extern "C" int acorn_moe_combine(const void* y, const void* x, const int* slot_of, const int* idx, const float* wts, void* out,
                                 int tokens, int H, int top, int E, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(moe_combine_kernel<T>, dim3(tokens), dim3(256), 0, stream, (const T*)y,
                                                       (const T*)x, slot_of, idx, wts, (T*)out, H, top, E));
    return ACORN_ERR_UNSUPPORTED;
}
