// Attention through a shared low-rank latent: what happens between the projections and the
// attention kernel, and the per-head matrix products around it.
//
// A token's projection row holds, head by head, [dim unrotated | rot rotated] query entries and, if
// the layer keeps its own cache, rank latent entries followed by rot entries of one rotated key part
// that all heads share.  The cache keeps one row of rank + rot per token: the latent after an RMS
// norm, and the key part after rotation.  With
//     key_h   = [ U_h c | kr ]          (U_h: the head's key up-projection [dim, rank])
//     score_h = (qu_h . U_h c + qr_h . kr) * scale  =  ([U_h^T qu_h | qr_h] . [c | kr]) * scale
// every head attends over the same cached rows with a query of rank + rot entries, and its values are
// V_h (sum_j p_j c_j): one key/value "head" of size rank + rot whose values are the first rank entries
// of the keys.  latent_prep writes the cache row and the rotated query parts; head_linear does the two
// per-head products (U_h^T qu_h before, V_h o_h after the attention).
#include "common.cuh"

// ---------------------------------------------------------------- prep
// Rotation: pairs (2i, 2i+1), i < rot_dims / 2, by the angle position * inv_freq[i] (float32); cos and
// sin are multiplied by `mag`.  Entries from rot_dims on pass unchanged.
template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ proj, int64_t ld, T* __restrict__ qcat,
                                   const float* __restrict__ c_weight, const float* __restrict__ inv_freq, float mag,
                                   const int* __restrict__ positions, const int* __restrict__ token_row,
                                   const int* __restrict__ block_table, const int* __restrict__ page_base,
                                   int table_stride, T* __restrict__ pages, int H, int dim, int rot, int rank,
                                   int rot_dims, int P, float eps, int write_kv) {
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const T* row = proj + (int64_t)t * ld;
    // the rotated query parts, into the tail of every head's query row
    for (int i = threadIdx.x; i < H * rot; i += blockDim.x) {
        const int h = i / rot, e = i % rot;
        const T* src = row + (int64_t)h * (dim + rot) + dim;
        float v;
        if (e < rot_dims) {
            const int pair = e >> 1;
            float s, c;
            sincosf((float)pos * inv_freq[pair], &s, &c);
            s *= mag;
            c *= mag;
            const float a = to_float(src[2 * pair]), b = to_float(src[2 * pair + 1]);
            v = (e & 1) ? (b * c + a * s) : (a * c - b * s);
        } else {
            v = to_float(src[e]);
        }
        qcat[((int64_t)t * H + h) * (rank + rot) + rank + e] = from_float<T>(v);
    }
    if (!write_kv) return;
    const T* kv = row + (int64_t)H * (dim + rot);
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_float(kv[i]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)rank + eps);
    const int r = token_row[t];
    const int page = block_table[(int64_t)r * table_stride + pos / P - page_base[r]];
    T* dst = pages + ((int64_t)page * P + pos % P) * (rank + rot);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<T>(to_float(kv[i]) * inv * c_weight[i]);
    for (int e = threadIdx.x; e < rot; e += blockDim.x) {
        float v;
        if (e < rot_dims) {
            const int pair = e >> 1;
            float s, c;
            sincosf((float)pos * inv_freq[pair], &s, &c);
            s *= mag;
            c *= mag;
            const float a = to_float(kv[rank + 2 * pair]), b = to_float(kv[rank + 2 * pair + 1]);
            v = (e & 1) ? (b * c + a * s) : (a * c - b * s);
        } else {
            v = to_float(kv[rank + e]);
        }
        dst[rank + e] = from_float<T>(v);
    }
}

extern "C" int acorn_latent_prep(const void* proj, int64_t ld, void* qcat, const float* c_weight, const float* inv_freq,
                                 float mag, const int* positions, const int* token_row, const int* block_table,
                                 const int* page_base, int table_stride, void* pages, int tokens, int H, int dim,
                                 int rot, int rank, int rot_dims, int P, float eps, int write_kv, int dtype,
                                 cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rot_dims % 2 || rot_dims > rot || rot < 0 || rank < 1 || P < 1) return ACORN_ERR_UNSUPPORTED;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(latent_prep_kernel<T>, dim3(tokens), dim3(128), 0, stream,
                                                       (const T*)proj, ld, (T*)qcat, c_weight, inv_freq, mag, positions,
                                                       token_row, block_table, page_base, table_stride, (T*)pages, H,
                                                       dim, rot, rank, rot_dims, P, eps, write_kv));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- per-head matrix products
// y[t, h, o] = sum_i w[h, o, i] * x[t, h, i]: x and y with a token stride and a head stride each (in
// elements; the innermost dimension contiguous), w [H, O, I] contiguous.  float32 accumulation, one
// chain over i = 0, 1, ... per output, so a token's result does not depend on the other tokens.
#define HL_TM 16
#define HL_TN 64
#define HL_TK 32

template <typename T>
__global__ void __launch_bounds__(256) head_linear_kernel(const T* __restrict__ x, int64_t xs_t, int64_t xs_h,
                                                          const T* __restrict__ w, T* __restrict__ y, int64_t ys_t,
                                                          int64_t ys_h, int tokens, int O, int I) {
    __shared__ float xs[HL_TM][HL_TK + 1];
    __shared__ float ws[HL_TN][HL_TK + 1];
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.z;
    const int t0 = blockIdx.x * HL_TM, o0 = blockIdx.y * HL_TN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 16 output groups of 4, 16 tokens
    const T* wh = w + (int64_t)h * O * I;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < I; k0 += HL_TK) {
        for (int e = threadIdx.x; e < HL_TM * HL_TK; e += 256) {
            const int tt = e / HL_TK, kk = e % HL_TK;
            const int t = t0 + tt, k = k0 + kk;
            xs[tt][kk] = (t < tokens && k < I) ? to_float(x[(int64_t)t * xs_t + (int64_t)h * xs_h + k]) : 0.f;
        }
        for (int e = threadIdx.x; e < HL_TN * HL_TK; e += 256) {
            const int oo = e / HL_TK, kk = e % HL_TK;
            const int o = o0 + oo, k = k0 + kk;
            ws[oo][kk] = (o < O && k < I) ? to_float(wh[(int64_t)o * I + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HL_TK; ++kk) {
            const float a = xs[ty][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = fmaf(a, ws[tx + 16 * j][kk], acc[j]);
        }
        __syncthreads();
    }
    const int t = t0 + ty;
    if (t < tokens) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int o = o0 + tx + 16 * j;
            if (o < O) y[(int64_t)t * ys_t + (int64_t)h * ys_h + o] = from_float<T>(acc[j]);
        }
    }
}

extern "C" int acorn_head_linear(const void* x, int64_t xs_t, int64_t xs_h, const void* w, void* y, int64_t ys_t,
                                 int64_t ys_h, int tokens, int H, int O, int I, int dtype, cudaStream_t stream) {
    if (tokens <= 0 || H <= 0 || O <= 0) return 0;
    if (H > 65535 || (O + HL_TN - 1) / HL_TN > 65535) return ACORN_ERR_UNSUPPORTED;
    dim3 grid((tokens + HL_TM - 1) / HL_TM, (O + HL_TN - 1) / HL_TN, H);
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(head_linear_kernel<T>, grid, dim3(256), 0, stream, (const T*)x, xs_t,
                                                       xs_h, (const T*)w, (T*)y, ys_t, ys_h, tokens, O, I));
    return ACORN_ERR_UNSUPPORTED;
}
