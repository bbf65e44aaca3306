// Linear recurrences with a matrix state per head, as the kernels of recurrent mixers.
//
// Per head a state S [N, V] in float32, zero when a request starts, kept in the request's state slot
// between steps.  For every token, with a decay a, a step size w, an input row x [V], a write key
// b [N] and a read key c [N], all float32:
//     S <- a S + b (w x)^T;      y = S^T c (+ skip * x).
// The decay is a number per token and head, or one per head for all tokens; w and skip are optional;
// head h takes the keys of group h / (H / G).  Two mixers are instances:
//   a selective state space layer (state-space duality form): a = exp(-exp(A_log) dt), w = dt, b = B, c = C,
//       skip = D, groups of heads sharing B and C;
//   linear attention with a fixed decay per head: a = decay_h, w = 1, b = k, c = q, x = v, no skip.
//
//   ssm_prep        per token: the short causal convolution over time of the x, B, C channels (inputs
//                   before the step's first token come from the request's state) with bias, silu;
//                   dt = softplus(. + dt_bias) and a = exp(-exp(A_log) dt); float32 outputs
//   silu_rows       out32 = silu(in) (the q, k, v of the linear attention)
//   linear_scan     the recurrence over a row's tokens, state in registers
//   gated_norm      per token: RMS norm in equal groups of the row with a weight, and a gate either
//                   before the norm (y silu(z)) or after it (sigmoid(z)); one rounding
//
// The columns of S (one per element of x) never mix, so a block of linear_scan takes a row, a head and
// a tile of columns; a column's N state entries are spread over LN lanes (N <= 16 LN), entry n with
// lane n % LN, and y's sum over n ends with shuffles among those lanes.  The tokens' a, w, b, c, x come
// through shared memory eight tokens at a time.  In the state slot S lies as [H, V, N].
#include "common.cuh"

#define SCAN_THREADS 128
#define SCAN_STRIP 16                   // state entries of a column a thread holds
#define SCAN_TOKENS 8                   // tokens staged at a time
#define SSM_MAX_TAPS 16

__device__ __forceinline__ float lr_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float lr_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// in [T, ld]: the convolution's C channels start at column c0, the H step-size pre-activations at column dt0.
template <typename T>
__global__ void ssm_prep_kernel(const T* __restrict__ in, int64_t ld, int c0, int dt0, const float* __restrict__ conv_w,
                                const float* __restrict__ conv_b, const float* __restrict__ state, int64_t slot_stride,
                                int64_t conv_off, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                const int* __restrict__ token_row, const int* __restrict__ row_start,
                                const int* __restrict__ row_slot, float* __restrict__ act, float* __restrict__ dt,
                                float* __restrict__ decay, int C, int H, int taps) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int r = token_row[t];
    const int i0 = t - row_start[r];                    // index of the token within its row
    const float* cstate = state + (int64_t)row_slot[r] * slot_stride + conv_off;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = conv_b ? conv_b[c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int idx = i0 - (taps - 1) + j;        // input index within the row; negative: before the step
            const float v = idx >= 0 ? to_float(in[(int64_t)(t - i0 + idx) * ld + c0 + c])
                                     : cstate[(int64_t)(taps - 1 + idx) * C + c];
            acc = fmaf(conv_w[(int64_t)c * taps + j], v, acc);
        }
        act[(int64_t)t * C + c] = acc * lr_sigmoid(acc);
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float step = lr_softplus(to_float(in[(int64_t)t * ld + dt0 + h]) + dt_bias[h]);
        dt[(int64_t)t * H + h] = step;
        decay[(int64_t)t * H + h] = expf(-expf(A_log[h]) * step);
    }
}

extern "C" int acorn_ssm_prep(const void* in, int64_t ld, int c0, int dt0, const float* conv_w, const float* conv_b,
                              const float* state, int64_t slot_stride, int64_t conv_off, const float* A_log,
                              const float* dt_bias, const int* token_row, const int* row_start, const int* row_slot,
                              float* act, float* dt, float* decay, int tokens, int C, int H, int taps, int dtype,
                              cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (taps < 1 || taps > SSM_MAX_TAPS || C < 1 || H < 0) return ACORN_ERR_UNSUPPORTED;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(ssm_prep_kernel<T>, dim3(tokens), dim3(256), 0, stream,
                                                       (const T*)in, ld, c0, dt0, conv_w, conv_b, state, slot_stride,
                                                       conv_off, A_log, dt_bias, token_row, row_start, row_slot, act, dt,
                                                       decay, C, H, taps));
    return ACORN_ERR_UNSUPPORTED;
}

template <typename T>
__global__ void silu_rows_kernel(const T* __restrict__ in, int64_t ld, float* __restrict__ out, int W, int64_t total) {
    pdl_wait();
    pdl_trigger();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / W;
        const float z = to_float(in[t * ld + (i - t * W)]);
        out[i] = z * lr_sigmoid(z);
    }
}

extern "C" int acorn_silu_rows(const void* in, int64_t ld, float* out, int tokens, int W, int dtype, cudaStream_t stream) {
    const int64_t total = (int64_t)tokens * W;
    if (total <= 0) return 0;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(silu_rows_kernel<T>, dim3((int)blocks), dim3(256), 0, stream,
                                                       (const T*)in, ld, out, W, total));
    return ACORN_ERR_UNSUPPORTED;
}

struct ScanParams {
    const float* b;  int64_t ldb;       // write keys [T, ldb], group g at column g * N
    const float* c;  int64_t ldc;       // read keys
    const float* x;  int64_t ldx;       // inputs [T, ldx], head h at column h * V
    const float* decay; int64_t lda;    // [T, lda] at column h, or lda = 0: one number per head
    const float* w;  int64_t ldw;       // step sizes [T, ldw] at column h, or null
    const float* skip;                  // [H] or null
    float* state; int64_t slot_stride, state_off;
    float* y;                           // [T, H * V]
    const int* row_start;
    const int* row_slot;
    int H, G, N, V, LN;
};

__global__ void __launch_bounds__(SCAN_THREADS) linear_scan_kernel(const ScanParams p) {
    extern __shared__ float sm[];
    const int cpb = SCAN_THREADS / p.LN;                // columns a block takes
    float* sB = sm;                                     // [SCAN_TOKENS][N]
    float* sC = sB + SCAN_TOKENS * p.N;
    float* sX = sC + SCAN_TOKENS * p.N;                 // [SCAN_TOKENS][cpb]
    float* sA = sX + SCAN_TOKENS * cpb;                 // [SCAN_TOKENS]
    float* sW = sA + SCAN_TOKENS;
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.y, r = blockIdx.z;
    const int g = h / (p.H / p.G);
    const int col = threadIdx.x / p.LN, l = threadIdx.x % p.LN;
    const int v0 = blockIdx.x * cpb, v = v0 + col;
    const bool live = v < p.V;
    const int first = p.row_start[r], L = p.row_start[r + 1] - first;
    float* S = p.state + (int64_t)p.row_slot[r] * p.slot_stride + p.state_off + ((int64_t)h * p.V + (live ? v : 0)) * p.N;
    float s[SCAN_STRIP];
#pragma unroll
    for (int i = 0; i < SCAN_STRIP; ++i) {
        const int n = l + p.LN * i;
        s[i] = (live && n < p.N) ? S[n] : 0.f;
    }
    const float skip = p.skip ? p.skip[h] : 0.f;
    for (int t0 = 0; t0 < L; t0 += SCAN_TOKENS) {
        const int nt = min(SCAN_TOKENS, L - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * p.N; i += SCAN_THREADS) {
            const int tt = i / p.N, n = i - tt * p.N;
            const int64_t tok = first + t0 + tt;
            sB[tt * p.N + n] = p.b[tok * p.ldb + (int64_t)g * p.N + n];
            sC[tt * p.N + n] = p.c[tok * p.ldc + (int64_t)g * p.N + n];
        }
        for (int i = threadIdx.x; i < nt * cpb; i += SCAN_THREADS) {
            const int tt = i / cpb, cc = i - tt * cpb;
            sX[i] = v0 + cc < p.V ? p.x[(int64_t)(first + t0 + tt) * p.ldx + (int64_t)h * p.V + v0 + cc] : 0.f;
        }
        if (threadIdx.x < nt) {
            const int64_t tok = first + t0 + threadIdx.x;
            sA[threadIdx.x] = p.lda ? p.decay[tok * p.lda + h] : p.decay[h];
            sW[threadIdx.x] = p.w ? p.w[tok * p.ldw + h] : 1.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float a = sA[tt], xv = sX[tt * cpb + col];
            const float u = sW[tt] * xv;
            const float* bb = sB + tt * p.N;
            const float* cc = sC + tt * p.N;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < SCAN_STRIP; ++i) {
                const int n = l + p.LN * i;
                if (n < p.N) {
                    s[i] = fmaf(a, s[i], bb[n] * u);
                    acc = fmaf(s[i], cc[n], acc);
                }
            }
            for (int o = p.LN >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && l == 0) p.y[(int64_t)(first + t0 + tt) * p.H * p.V + (int64_t)h * p.V + v] = acc + skip * xv;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < SCAN_STRIP; ++i) {
            const int n = l + p.LN * i;
            if (n < p.N) S[n] = s[i];
        }
    }
}

extern "C" int acorn_linear_scan(const float* b, int64_t ldb, const float* c, int64_t ldc, const float* x, int64_t ldx,
                                 const float* decay, int64_t lda, const float* w, int64_t ldw, const float* skip,
                                 float* state, int64_t slot_stride, int64_t state_off, float* y, const int* row_start,
                                 const int* row_slot, int rows, int H, int G, int N, int V, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H < 1 || G < 1 || H % G || N < 1 || N > 32 * SCAN_STRIP || V < 1 || rows > 65535 || H > 65535)
        return ACORN_ERR_UNSUPPORTED;
    int LN = 1;
    while (LN * SCAN_STRIP < N) LN *= 2;
    const int cpb = SCAN_THREADS / LN;
    ScanParams p = {b, ldb, c, ldc, x, ldx, decay, lda, w, ldw, skip, state, slot_stride, state_off, y, row_start, row_slot,
                    H, G, N, V, LN};
    const size_t smem = (size_t)SCAN_TOKENS * (2 * N + cpb + 2) * sizeof(float);
    return acorn_launch(linear_scan_kernel, dim3((V + cpb - 1) / cpb, H, rows), dim3(SCAN_THREADS), smem, stream, p);
}

// y32 [T, W] in `groups` equal parts.  mode 0: u = y silu(z), out = u / rms_part(u) * weight;
// mode 1: out = y / rms_part(y) * weight * sigmoid(z).  z = gate[t * ldg + i]; out[t * ldo + i], times out_scale.
template <typename T>
__global__ void gated_norm_kernel(const float* __restrict__ y, const T* __restrict__ gate, int64_t ldg,
                                  const float* __restrict__ weight, T* __restrict__ out, int64_t ldo, int W, int groups,
                                  float eps, int mode, float out_scale) {
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int64_t t = blockIdx.x;
    const int part = W / groups, i0 = blockIdx.y * part;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        float u = y[t * W + i0 + i];
        if (mode == 0) {
            const float z = to_float(gate[t * ldg + i0 + i]);
            u *= z * lr_sigmoid(z);
        }
        ss += u * u;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)part + eps);
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        const float z = to_float(gate[t * ldg + i0 + i]);
        float u = y[t * W + i0 + i];
        u = mode == 0 ? u * (z * lr_sigmoid(z)) * inv * weight[i0 + i] : u * inv * weight[i0 + i] * lr_sigmoid(z);
        out[t * ldo + i0 + i] = from_float<T>(u * out_scale);
    }
}

extern "C" int acorn_gated_norm(const float* y, const void* gate, int64_t ldg, const float* weight, void* out, int64_t ldo,
                                int tokens, int W, int groups, float eps, int mode, float out_scale, int dtype,
                                cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (groups < 1 || W % groups || groups > 65535 || mode < 0 || mode > 1) return ACORN_ERR_UNSUPPORTED;
    const int part = W / groups;
    const int threads = part >= 1024 ? 256 : 128;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(gated_norm_kernel<T>, dim3(tokens, groups), dim3(threads), 0, stream,
                                                       y, (const T*)gate, ldg, weight, (T*)out, ldo, W, groups, eps, mode,
                                                       out_scale));
    return ACORN_ERR_UNSUPPORTED;
}
