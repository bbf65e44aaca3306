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
//                   dt = softplus(. + dt_bias) and a = exp(-exp(A_log) dt); float32 outputs; on request it
//                   also shifts the convolution's memory of rows of one token
//   silu_rows       out32 = silu(in) (the q, k, v of the linear attention)
//   linear_scan     the recurrence over a row's tokens, state in registers
//   gated_norm      per token: RMS norm in equal groups of the row with a weight, and a gate either
//                   before the norm (y silu(z)) or after it (sigmoid(z)); one rounding
//
// The columns of S (one per element of x) never mix, so a block of linear_scan takes a row, a head and
// a tile of columns; a column's N state entries are spread over LN lanes (N <= 16 LN) in runs of four
// (entry n with lane (n / 4) % LN, so that a lane reads its keys 16 bytes at a time; a token's keys are
// padded with zeros to 16 LN in shared memory), and y's sum over n ends with shuffles among those lanes.  The tokens' a, w, b, c, x come
// through shared memory eight tokens at a time.  In the state slot S lies as [H, V, N].
#include "common.cuh"

#define SCAN_THREADS 128
#define SCAN_STRIP 16                   // state entries of a column a thread holds
#define SCAN_TOKENS 8                   // tokens staged at a time
#define SSM_MAX_TAPS 16
#define SSM_PREP_CHANNELS 512

__device__ __forceinline__ float lr_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float lr_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// in [T, ld]: the convolution's C channels start at column c0, the H step-size pre-activations at column dt0.
template <typename T>
__global__ void ssm_prep_kernel(const T* __restrict__ in, int64_t ld, int c0, int dt0, const float* __restrict__ conv_w,
                                const float* __restrict__ conv_b, float* __restrict__ state, int64_t slot_stride,
                                int64_t conv_off, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                const int* __restrict__ token_row, const int* __restrict__ row_start,
                                const int* __restrict__ row_slot, float* __restrict__ act, float* __restrict__ dt,
                                float* __restrict__ decay, int C, int H, int taps, int update_single, int per_block) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int r = token_row[t];
    const int i0 = t - row_start[r];                    // index of the token within its row
    float* cstate = state + (int64_t)row_slot[r] * slot_stride + conv_off;
    // A row of one token (a decoded token): its thread is the only one that reads the channel's memory in this
    // step, so it also shifts the memory by the token's input (no kernel of its own for that in a decode step).
    const bool shift = update_single && row_start[r + 1] - row_start[r] == 1;
    // a block takes per_block channels of a token (blockIdx.y)
    const int c_end = min(C, (int)(blockIdx.y + 1) * per_block);
    for (int c = blockIdx.y * per_block + threadIdx.x; c < c_end; c += blockDim.x) {
        float acc = conv_b ? conv_b[c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int idx = i0 - (taps - 1) + j;        // input index within the row; negative: before the step
            const float v = idx >= 0 ? to_float(in[(int64_t)(t - i0 + idx) * ld + c0 + c])
                                     : cstate[(int64_t)(taps - 1 + idx) * C + c];
            acc = fmaf(conv_w[(int64_t)c * taps + j], v, acc);
        }
        act[(int64_t)t * C + c] = acc * lr_sigmoid(acc);
        if (shift) {
            for (int j = 0; j + 1 < taps - 1; ++j) cstate[(int64_t)j * C + c] = cstate[(int64_t)(j + 1) * C + c];
            if (taps > 1) cstate[(int64_t)(taps - 2) * C + c] = to_float(in[(int64_t)t * ld + c0 + c]);
        }
    }
    if (blockIdx.y != 0) return;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float step = lr_softplus(to_float(in[(int64_t)t * ld + dt0 + h]) + dt_bias[h]);
        dt[(int64_t)t * H + h] = step;
        decay[(int64_t)t * H + h] = expf(-expf(A_log[h]) * step);
    }
}

extern "C" int acorn_ssm_prep(const void* in, int64_t ld, int c0, int dt0, const float* conv_w, const float* conv_b,
                              float* state, int64_t slot_stride, int64_t conv_off, const float* A_log,
                              const float* dt_bias, const int* token_row, const int* row_start, const int* row_slot,
                              float* act, float* dt, float* decay, int tokens, int C, int H, int taps, int dtype,
                              int update_single, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (taps < 1 || taps > SSM_MAX_TAPS || C < 1 || H < 0) return ACORN_ERR_UNSUPPORTED;
    // few tokens (a decode step): many short blocks hide the loads' latency (batch 8 at 6,144 channels: 38 -> 13 us);
    // many tokens: a block a token (2,048 tokens: 85 us against 120 us in short blocks)
    const int per_block = tokens >= 512 ? C : SSM_PREP_CHANNELS;
    const int chunks = (C + per_block - 1) / per_block;
    if (chunks > 65535) return ACORN_ERR_UNSUPPORTED;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(ssm_prep_kernel<T>, dim3(tokens, chunks), dim3(256), 0, stream,
                                                       (const T*)in, ld, c0, dt0, conv_w, conv_b, state, slot_stride,
                                                       conv_off, A_log, dt_bias, token_row, row_start, row_slot, act, dt,
                                                       decay, C, H, taps, update_single, per_block));
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
    // long rows in segments of `seg` tokens (SCAN_SEGMENTS / SCAN_FINISH): per row nseg + 1 states
    // [H, V, N] (the row's state before the step, then the state each segment but the last ends with when it
    // starts from nothing; segment 0 starts from the row's state) and the segments' products of decays [nseg, H]
    float* seg_state;
    float* seg_decay;
    int seg, nseg;
};

#define SCAN_WHOLE 0        // a row from its slot's state to the end, the state back into the slot
#define SCAN_SEGMENTS 1     // every segment but a row's last: its end state and the product of its decays
#define SCAN_FINISH 2       // every segment from the state it really starts with: y, and the row's last state

// Two float32 numbers in a 64-bit register and the packed instructions on them (each half as the scalar
// instruction rounds it): half the issue slots for the scan's multiply-adds.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ void scan_cp4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void scan_cp16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}

// A recurrence runs over a row's tokens one after the other; what runs side by side is heads, columns
// and rows.  A prompt of thousands of tokens alone in its step would leave most of the device idle, so
// long rows are cut into segments that run side by side in two passes: SCAN_SEGMENTS takes every segment
// from a zero state (the first from the row's state) to the state it ends with; SCAN_FINISH puts the
// states before its segment together (S <- P_j S + E_j over the earlier segments: the recurrence is
// linear in S), runs the segment again from there and writes y.  Twice the arithmetic, nseg times the
// blocks.  The tokens' a, w, b, c, x are staged by cp.async, one stage ahead of the arithmetic.
template <int MODE, int CPT>
__global__ void __launch_bounds__(SCAN_THREADS, CPT == 4 ? 3 : 4) linear_scan_kernel(const ScanParams p) {
    extern __shared__ __align__(16) float sm[];
    const int cpl = SCAN_THREADS / p.LN;                // columns side by side in a block; a thread holds CPT of them,
    const int cpb = cpl * CPT;                          // cpl apart, so a block takes cpb columns
    const int NS = SCAN_STRIP * p.LN;                   // a token's keys in shared memory: N of them, then zeros
    const int stage_floats = SCAN_TOKENS * (2 * NS + cpb + 2);
    for (int i = threadIdx.x; i < 2 * stage_floats; i += SCAN_THREADS) sm[i] = 0.f;
    __syncthreads();
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.y;
    const int r = MODE == SCAN_WHOLE ? blockIdx.z : blockIdx.z / p.nseg;
    const int sg = MODE == SCAN_WHOLE ? 0 : blockIdx.z % p.nseg;
    const int g = h / (p.H / p.G);
    const int col = threadIdx.x / p.LN, l = threadIdx.x % p.LN;
    const int v0 = blockIdx.x * cpb;
    int first = p.row_start[r], L = p.row_start[r + 1] - first;
    int nseg_r = 1;
    if (MODE != SCAN_WHOLE) {
        nseg_r = (L + p.seg - 1) / p.seg;
        if (sg >= nseg_r || (MODE == SCAN_SEGMENTS && sg == nseg_r - 1 && sg > 0)) return;
        first += sg * p.seg;
        L = min(p.seg, L - sg * p.seg);
    }
    const int64_t HVN = (int64_t)p.H * p.V * p.N;
    float* slot = p.state + (int64_t)p.row_slot[r] * p.slot_stride + p.state_off;
    float* seg_states = MODE == SCAN_WHOLE ? nullptr : p.seg_state + (int64_t)r * (p.nseg + 1) * HVN;
    // column j of the thread is v0 + col + j * cpl; its state entries start at strip0 + j * strip_step within [H, V, N]
    const int64_t strip0 = ((int64_t)h * p.V + v0 + col) * p.N, strip_step = (int64_t)cpl * p.N;
    f32x2 s[CPT][SCAN_STRIP / 2];                       // entries 2k and 2k + 1 of the thread's strip in s[j][k]
#define SCAN_LIVE(j) (v0 + col + (j) * cpl < p.V)
#define SCAN_AT(j) (strip0 + (j) * strip_step)
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
        float e[SCAN_STRIP];
#pragma unroll
        for (int i = 0; i < SCAN_STRIP; ++i) {
            const int n = (i >> 2) * 4 * p.LN + 4 * l + (i & 3);
            const bool ok = SCAN_LIVE(j) && n < p.N;
            if (MODE == SCAN_WHOLE) {
                e[i] = ok ? slot[SCAN_AT(j) + n] : 0.f;
            } else if (MODE == SCAN_SEGMENTS) {
                e[i] = (ok && sg == 0) ? slot[SCAN_AT(j) + n] : 0.f;
                if (ok && sg == 0) seg_states[SCAN_AT(j) + n] = e[i];             // the row's state before the step
            } else {
                e[i] = ok ? seg_states[(sg == 0 ? 0 : HVN) + SCAN_AT(j) + n] : 0.f;
            }
        }
#pragma unroll
        for (int k = 0; k < SCAN_STRIP / 2; ++k) s[j][k] = pack2(e[2 * k], e[2 * k + 1]);
    }
    if (MODE == SCAN_SEGMENTS && sg == nseg_r - 1) return;      // a row of one segment: only its state was copied
    if (MODE == SCAN_FINISH) {
        for (int k = 1; k < sg; ++k) {                          // the states the earlier segments end with, folded
            const float pk = p.seg_decay[((int64_t)r * p.nseg + k) * p.H + h];
#pragma unroll
            for (int j = 0; j < CPT; ++j)
#pragma unroll
                for (int i = 0; i < SCAN_STRIP; i += 2) {
                    float e[2];
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const int n = ((i + q) >> 2) * 4 * p.LN + 4 * l + ((i + q) & 3);
                        e[q] = (SCAN_LIVE(j) && n < p.N) ? seg_states[(int64_t)(k + 1) * HVN + SCAN_AT(j) + n] : 0.f;
                    }
                    s[j][i / 2] = fma2(pack2(pk, pk), s[j][i / 2], pack2(e[0], e[1]));
                }
        }
    }
    const float skip = p.skip ? p.skip[h] : 0.f;
    float prod = 1.f;
    // keys whose rows start on 16-byte boundaries are copied 16 bytes at a time
    const bool keys16 = (p.N & 3) == 0 && (p.ldb & 3) == 0 && (p.ldc & 3) == 0 &&
                        ((reinterpret_cast<uintptr_t>(p.b) | reinterpret_cast<uintptr_t>(p.c)) & 15) == 0;
    auto stage_in = [&](int t0, int stage) {
        float* sB = sm + stage * stage_floats;                  // [SCAN_TOKENS][NS]
        float* sC = sB + SCAN_TOKENS * NS;
        float* sX = sC + SCAN_TOKENS * NS;                      // [SCAN_TOKENS][cpb]
        float* sA = sX + SCAN_TOKENS * cpb;                     // [SCAN_TOKENS]
        float* sW = sA + SCAN_TOKENS;
        const int nt = min(SCAN_TOKENS, L - t0);
        if (nt > 0) {
            if (keys16) {                                       // 16 bytes a copy: a token's keys in N / 4 pieces
                const int per = p.N >> 2;
                for (int i = threadIdx.x; i < nt * per; i += SCAN_THREADS) {
                    const int tt = i / per, n = (i - tt * per) << 2;
                    const int64_t tok = first + t0 + tt;
                    scan_cp16(sB + tt * NS + n, p.b + tok * p.ldb + (int64_t)g * p.N + n);
                    if (MODE != SCAN_SEGMENTS) scan_cp16(sC + tt * NS + n, p.c + tok * p.ldc + (int64_t)g * p.N + n);
                }
            }
            for (int tt = 0; tt < nt; ++tt) {
                const int64_t tok = first + t0 + tt;
                if (!keys16) {
                    for (int n = threadIdx.x; n < p.N; n += SCAN_THREADS) {
                        scan_cp4(sB + tt * NS + n, p.b + tok * p.ldb + (int64_t)g * p.N + n);
                        if (MODE != SCAN_SEGMENTS) scan_cp4(sC + tt * NS + n, p.c + tok * p.ldc + (int64_t)g * p.N + n);
                    }
                }
                for (int cc = threadIdx.x; cc < cpb; cc += SCAN_THREADS) {
                    if (v0 + cc < p.V) scan_cp4(sX + tt * cpb + cc, p.x + tok * p.ldx + (int64_t)h * p.V + v0 + cc);
                    else sX[tt * cpb + cc] = 0.f;
                }
            }
            if (threadIdx.x < nt) {
                const int64_t tok = first + t0 + threadIdx.x;
                scan_cp4(sA + threadIdx.x, p.lda ? p.decay + tok * p.lda + h : p.decay + h);
                if (p.w) scan_cp4(sW + threadIdx.x, p.w + tok * p.ldw + h);
                else sW[threadIdx.x] = 1.f;
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    stage_in(0, 0);
    for (int t0 = 0, it = 0; t0 < L; t0 += SCAN_TOKENS, ++it) {
        const int stage = it & 1;
        stage_in(t0 + SCAN_TOKENS, stage ^ 1);                  // the stage the step before finished with
        asm volatile("cp.async.wait_group 1;\n" ::);
        __syncthreads();
        const float* sB = sm + stage * stage_floats;
        const float* sC = sB + SCAN_TOKENS * NS;
        const float* sX = sC + SCAN_TOKENS * NS;
        const float* sA = sX + SCAN_TOKENS * cpb;
        const float* sW = sA + SCAN_TOKENS;
        const int nt = min(SCAN_TOKENS, L - t0);
        for (int tt = 0; tt < nt; ++tt) {
            const float a = sA[tt], wt = sW[tt];
            float xv[CPT];
            f32x2 uu[CPT], acc2[CPT];
            const f32x2 aa = pack2(a, a);
#pragma unroll
            for (int j = 0; j < CPT; ++j) {
                xv[j] = sX[tt * cpb + col + j * cpl];
                uu[j] = pack2(wt * xv[j], wt * xv[j]);
                acc2[j] = 0ull;
            }
            const ulonglong2* bb = reinterpret_cast<const ulonglong2*>(sB + tt * NS) + l;
            const ulonglong2* cc = reinterpret_cast<const ulonglong2*>(sC + tt * NS) + l;
            // entries beyond N hold zeros and stay zero (their keys are zeros); a key is read once for the
            // thread's CPT columns; the arithmetic is on pairs of entries (packed float32x2)
#pragma unroll
            for (int i4 = 0; i4 < SCAN_STRIP / 4; ++i4) {
                const ulonglong2 b4 = bb[i4 * p.LN];
                ulonglong2 c4 = make_ulonglong2(0ull, 0ull);
                if (MODE != SCAN_SEGMENTS) c4 = cc[i4 * p.LN];
#pragma unroll
                for (int j = 0; j < CPT; ++j) {
                    s[j][2 * i4] = fma2(aa, s[j][2 * i4], mul2(b4.x, uu[j]));
                    s[j][2 * i4 + 1] = fma2(aa, s[j][2 * i4 + 1], mul2(b4.y, uu[j]));
                    if (MODE != SCAN_SEGMENTS) {
                        acc2[j] = fma2(s[j][2 * i4], c4.x, acc2[j]);
                        acc2[j] = fma2(s[j][2 * i4 + 1], c4.y, acc2[j]);
                    }
                }
            }
            float acc[CPT];
#pragma unroll
            for (int j = 0; j < CPT; ++j) {
                float lo, hi;
                unpack2(acc2[j], lo, hi);
                acc[j] = lo + hi;
            }
            if (MODE == SCAN_SEGMENTS) {
                prod *= a;
            } else {
                for (int o = p.LN >> 1; o > 0; o >>= 1) {
#pragma unroll
                    for (int j = 0; j < CPT; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
                }
                float* yrow = p.y + (int64_t)(first + t0 + tt) * p.H * p.V + (int64_t)h * p.V + v0 + col;
#pragma unroll
                for (int j = 0; j < CPT; ++j)
                    if (SCAN_LIVE(j) && l == 0) yrow[j * cpl] = acc[j] + skip * xv[j];
            }
        }
        __syncthreads();                                        // the stage may be filled again
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    if (MODE == SCAN_FINISH && sg != nseg_r - 1) return;        // only a row's last segment ends with the row's state
    float* dst = MODE == SCAN_SEGMENTS ? seg_states + (int64_t)(sg + 1) * HVN : slot;
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
        if (!SCAN_LIVE(j)) continue;
#pragma unroll
        for (int i = 0; i < SCAN_STRIP; i += 2) {
            float e[2];
            unpack2(s[j][i / 2], e[0], e[1]);
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int n = ((i + q) >> 2) * 4 * p.LN + 4 * l + ((i + q) & 3);
                if (n < p.N) dst[SCAN_AT(j) + n] = e[q];
            }
        }
    }
    if (MODE == SCAN_SEGMENTS && blockIdx.x == 0 && threadIdx.x == 0)
        p.seg_decay[((int64_t)r * p.nseg + sg) * p.H + h] = prod;
#undef SCAN_LIVE
#undef SCAN_AT
}

template <int CPT>
static int launch_scan(const ScanParams& p, int rows, bool cut, cudaStream_t stream) {
    const int cpb = SCAN_THREADS / p.LN * CPT;
    const size_t smem = (size_t)2 * SCAN_TOKENS * (2 * SCAN_STRIP * p.LN + cpb + 2) * sizeof(float);
    if (smem > 48 * 1024) {
        static AcornPerDevice configured;
        if (!configured.seen()) {
            const int most = (int)((size_t)2 * SCAN_TOKENS * (2 * 32 * SCAN_STRIP + SCAN_THREADS * CPT + 2) * sizeof(float));
            cudaError_t e = cudaFuncSetAttribute(linear_scan_kernel<SCAN_WHOLE, CPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_scan_kernel<SCAN_SEGMENTS, CPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_scan_kernel<SCAN_FINISH, CPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
            if (e != cudaSuccess) return (int)e;
            configured.mark();
        }
    }
    const dim3 grid((p.V + cpb - 1) / cpb, p.H, rows * (cut ? p.nseg : 1));
    if (!cut) return acorn_launch(linear_scan_kernel<SCAN_WHOLE, CPT>, grid, dim3(SCAN_THREADS), smem, stream, p);
    const int rc = acorn_launch(linear_scan_kernel<SCAN_SEGMENTS, CPT>, grid, dim3(SCAN_THREADS), smem, stream, p);
    if (rc != 0) return rc;
    return acorn_launch(linear_scan_kernel<SCAN_FINISH, CPT>, grid, dim3(SCAN_THREADS), smem, stream, p);
}

// How many columns a thread of the scan holds for these sizes: a key read from shared memory serves all of
// them, so more is less traffic, as long as the blocks still cover the columns without much waste.
extern "C" int acorn_linear_scan_columns(int N, int V) {
    int LN = 1;
    while (LN * SCAN_STRIP < N) LN *= 2;
    const int cpl = SCAN_THREADS / LN;
    // two measured as fast as four with segments (2,048 tokens: 505 / 277 us against 492 / 313 us for the two mixers
    // at width 2,048) and a third faster on a row in one piece (849 against 1,232 us)
    int most = 2;
    if (const char* e = std::getenv("ACORN_SCAN_COLUMNS")) most = e[0] == '1' ? 1 : (e[0] == '2' ? 2 : 4);   // for experiments
    return (most >= 4 && V >= 4 * cpl) ? 4 : ((most >= 2 && V >= 2 * cpl) ? 2 : 1);
}

// seg_tokens = 0: every row in one piece (seg_state, seg_decay unused).  Otherwise rows are cut into segments of
// seg_tokens tokens, at most nseg a row (the caller sees to nseg * seg_tokens >= the longest row); seg_state holds
// rows * (nseg + 1) * H * V * N floats, seg_decay rows * nseg * H.
extern "C" int acorn_linear_scan(const float* b, int64_t ldb, const float* c, int64_t ldc, const float* x, int64_t ldx,
                                 const float* decay, int64_t lda, const float* w, int64_t ldw, const float* skip,
                                 float* state, int64_t slot_stride, int64_t state_off, float* y, const int* row_start,
                                 const int* row_slot, int rows, int H, int G, int N, int V, int seg_tokens, int nseg,
                                 float* seg_state, float* seg_decay, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H < 1 || G < 1 || H % G || N < 1 || N > 32 * SCAN_STRIP || V < 1 || H > 65535) return ACORN_ERR_UNSUPPORTED;
    const bool cut = seg_tokens > 0;
    if (cut && (nseg < 2 || seg_state == nullptr || seg_decay == nullptr)) return ACORN_ERR_UNSUPPORTED;
    if ((int64_t)rows * (cut ? nseg : 1) > 65535) return ACORN_ERR_UNSUPPORTED;
    int LN = 1;
    while (LN * SCAN_STRIP < N) LN *= 2;
    ScanParams p = {b, ldb, c, ldc, x, ldx, decay, lda, w, ldw, skip, state, slot_stride, state_off, y, row_start, row_slot,
                    H, G, N, V, LN, seg_state, seg_decay, seg_tokens, cut ? nseg : 1};
    switch (acorn_linear_scan_columns(N, V)) {
        case 4: return launch_scan<4>(p, rows, cut, stream);
        case 2: return launch_scan<2>(p, rows, cut, stream);
        default: return launch_scan<1>(p, rows, cut, stream);
    }
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
    // a part of at most GN_KEEP elements a thread stays in registers between the two passes
    constexpr int GN_KEEP = 8;
    const bool keep = part <= GN_KEEP * (int)blockDim.x;
    float uu[GN_KEEP], zz[GN_KEEP];
    float ss = 0.f;
    if (keep) {
#pragma unroll
        for (int k = 0; k < GN_KEEP; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            uu[k] = zz[k] = 0.f;
            if (i < part) {
                zz[k] = to_float(gate[t * ldg + i0 + i]);
                uu[k] = y[t * W + i0 + i];
                if (mode == 0) uu[k] *= zz[k] * lr_sigmoid(zz[k]);
                ss += uu[k] * uu[k];
            }
        }
    } else {
        for (int i = threadIdx.x; i < part; i += blockDim.x) {
            float u = y[t * W + i0 + i];
            if (mode == 0) {
                const float z = to_float(gate[t * ldg + i0 + i]);
                u *= z * lr_sigmoid(z);
            }
            ss += u * u;
        }
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)part + eps);
    if (keep) {
#pragma unroll
        for (int k = 0; k < GN_KEEP; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < part) {
                const float u = mode == 0 ? uu[k] * inv * weight[i0 + i] : uu[k] * inv * weight[i0 + i] * lr_sigmoid(zz[k]);
                out[t * ldo + i0 + i] = from_float<T>(u * out_scale);
            }
        }
        return;
    }
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
