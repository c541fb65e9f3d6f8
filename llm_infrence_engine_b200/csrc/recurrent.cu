// Mixers that carry a state of fixed size from token to token: the short causal convolution, the gated delta rule with a
// decay per key channel, and the state-space recurrence with a decay per head. T is the storage type of the projections
// (float or bfloat16); decays, step sizes, gates, unit norms and the states themselves are 32-bit.
//
// A step's batch is ragged: request r owns the rows seq_starts[r] .. seq_starts[r + 1] - 1, and its state lives in row
// seq_slots[r] of the state tensor (zeroed by the step when the request's first token is among the rows). The same kernels
// run a prompt portion of any length and a single decoded token: the recurrences walk their rows in order, so a position's
// result does not depend on how the request was cut into steps.
#include <math.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_CHUNK = 32;   // tokens of one request that a block walks; at least CONV_MAX_TAPS - 1

// y[t, c] = act(bias[c] + sum_j w[c, j] * u[t - taps + 1 + j, c]) over the rows of each request, where u before the step's
// first row comes from state[slot][taps - 1 + t][c] (t < 0: the request's last taps - 1 inputs of earlier steps) and the
// state is then moved on by the step's rows. A thread owns a channel; only the block of a request's first chunk reads the
// old state and writes the new one, each thread its own channel, so nothing races.
template <typename T>
__global__ void __launch_bounds__(128) causal_conv_kernel(const T* __restrict__ z, int z_stride, int C, const float* __restrict__ w,
                                                          const float* __restrict__ bias, float* __restrict__ state,
                                                          const int* __restrict__ seq_starts, const int* __restrict__ seq_slots,
                                                          T* __restrict__ out, int out_stride, int taps, int act) {
    pdl_trigger();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    float wt[CONV_MAX_TAPS];
    float b = 0.f;
    if (c < C) {
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) wt[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
        if (bias) b = bias[c];
    }
    pdl_wait();
    if (c >= C) return;
    const int r = blockIdx.z;
    const int s0 = seq_starts[r], L = seq_starts[r + 1] - s0;
    const int t0 = blockIdx.y * CONV_CHUNK;
    if (t0 >= L) return;
    float* st = state + (size_t)seq_slots[r] * (taps - 1) * C + c;
    float old[CONV_MAX_TAPS - 1];
    if (t0 == 0) {
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) old[j] = j < taps - 1 ? st[(size_t)j * C] : 0.f;
    }
    // win[j] = input at t - (taps - 1) + j for the token t being computed; shifted by one per token
    float win[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) win[j] = 0.f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
        if (j < taps - 1) {
            const int t = t0 - (taps - 1) + j;   // the inputs before the chunk's first token
            win[j + 1] = t >= 0 ? to_f32(z[(size_t)(s0 + t) * z_stride + c]) : old[taps - 1 + t];
        }
    }
    const int t1 = min(L, t0 + CONV_CHUNK);
    for (int t = t0; t < t1; ++t) {
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) win[j] = win[j + 1];
        const float u = to_f32(z[(size_t)(s0 + t) * z_stride + c]);
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)
            if (j == taps - 1) win[j] = u;
        float y = b;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)
            if (j < taps) y = fmaf(wt[j], win[j], y);
        if (act == 1) y = silu_f(y);
        out[(size_t)(s0 + t) * out_stride + c] = from_f32<T>(y);
    }
    if (t0 == 0) {
        for (int i = 0; i < taps - 1; ++i) {
            const int t = L - (taps - 1) + i;
            st[(size_t)i * C] = t >= 0 ? to_f32(z[(size_t)(s0 + t) * z_stride + c]) : old[taps - 1 + t];
        }
    }
}

// ------------------------------------------------------------------------------------------------
// What the delta rule's recurrence reads, made from the projections in one parallel pass. One warp per (token, head):
//   decay[n, h, d] = exp(-exp(A_log[h]) * softplus(a[n, h, d] + dt_bias[h, d]))
//   beta[n, h]     = sigmoid(b[n, h])
// and, by the first head of every key group g, the unit vectors
//   qn[n, g, :] = q / sqrt(sum q^2 + unit_eps) * q_scale,   kn[n, g, :] = k / sqrt(sum k^2 + unit_eps),   kq[n, g] = kn . qn
template <typename T>
__global__ void __launch_bounds__(128) delta_prepare_kernel(const T* __restrict__ qkv, int qkv_stride, int q_col, int k_col,
                                                            const T* __restrict__ a, int a_stride, const T* __restrict__ bsrc,
                                                            int b_stride, const float* __restrict__ A_log,
                                                            const float* __restrict__ dt_bias, float* __restrict__ qn,
                                                            float* __restrict__ kn, float* __restrict__ kq, float* __restrict__ decay,
                                                            float* __restrict__ beta, int N, int H, int G, int D, float q_scale,
                                                            float unit_eps) {
    pdl_trigger();
    pdl_wait();
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (item >= N * H) return;
    const int n = item / H, h = item % H;
    const float rate = expf(A_log[h]);
    for (int d = lane; d < D; d += 32) {
        const float x = to_f32(a[(size_t)n * a_stride + h * D + d]) + dt_bias[h * D + d];
        decay[((size_t)n * H + h) * D + d] = expf(-rate * softplus_f(x));
    }
    if (lane == 0) beta[(size_t)n * H + h] = sigmoid_f(to_f32(bsrc[(size_t)n * b_stride + h]));
    const int per = H / G;
    if (h % per == 0) {
        const int g = h / per;
        const T* qr = qkv + (size_t)n * qkv_stride + q_col + g * D;
        const T* kr = qkv + (size_t)n * qkv_stride + k_col + g * D;
        float sq = 0.f, sk = 0.f, dot = 0.f;
        for (int d = lane; d < D; d += 32) {
            const float qv = to_f32(qr[d]), kv = to_f32(kr[d]);
            sq = fmaf(qv, qv, sq); sk = fmaf(kv, kv, sk); dot = fmaf(qv, kv, dot);
        }
        sq = warp_sum(sq); sk = warp_sum(sk); dot = warp_sum(dot);
        const float fq = q_scale / sqrtf(sq + unit_eps), fk = 1.0f / sqrtf(sk + unit_eps);
        for (int d = lane; d < D; d += 32) {
            qn[((size_t)n * G + g) * D + d] = to_f32(qr[d]) * fq;
            kn[((size_t)n * G + g) * D + d] = to_f32(kr[d]) * fk;
        }
        if (lane == 0) kq[(size_t)n * G + g] = dot * fq * fk;
    }
}

// ------------------------------------------------------------------------------------------------
// The gated delta rule. Per head, S is [D, DV]; for every token, in order:
//   S <- decay (.) S (row d by decay[d]);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// The columns of S are independent of one another: a warp owns 32 of them, a lane one column, all D entries in registers.
// With S' = decay (.) S both products of a token are taken from S' in one pass over the registers: r = S'^T k and
// S'^T q, and then o = S'^T q + u (k . q), the last factor coming with the token. Tokens arrive in tiles through shared memory.
constexpr int SCAN_TILE = 8;

template <typename T, int DMAX>
__global__ void __launch_bounds__(32) delta_scan_kernel(const T* __restrict__ v, int v_stride, int v_col, const float* __restrict__ qn,
                                                        const float* __restrict__ kn, const float* __restrict__ kq,
                                                        const float* __restrict__ decay, const float* __restrict__ beta,
                                                        float* __restrict__ state, const int* __restrict__ seq_starts,
                                                        const int* __restrict__ seq_slots, float* __restrict__ out, int H, int G, int D,
                                                        int DV) {
    __shared__ __align__(16) float k_s[SCAN_TILE][DMAX], q_s[SCAN_TILE][DMAX], g_s[SCAN_TILE][DMAX];
    __shared__ float beta_s[SCAN_TILE], kq_s[SCAN_TILE];
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x;
    const int col = blockIdx.x * 32 + lane;
    const int h = blockIdx.y, r = blockIdx.z;
    const int g = h / (H / G);
    const bool live = col < DV;
    const int s0 = seq_starts[r], s1 = seq_starts[r + 1];
    float* st = state + (((size_t)seq_slots[r] * H + h) * D) * DV + col;
    float S[DMAX];
#pragma unroll
    for (int d = 0; d < DMAX; ++d) S[d] = (live && d < D) ? st[(size_t)d * DV] : 0.f;
    for (int base = s0; base < s1; base += SCAN_TILE) {
        const int count = min(SCAN_TILE, s1 - base);
        __syncwarp();
        for (int i = lane; i < count * DMAX; i += 32) {
            const int t = i / DMAX, d = i % DMAX;
            const int n = base + t;
            const bool in = d < D;
            k_s[t][d] = in ? kn[((size_t)n * G + g) * D + d] : 0.f;
            q_s[t][d] = in ? qn[((size_t)n * G + g) * D + d] : 0.f;
            g_s[t][d] = in ? decay[((size_t)n * H + h) * D + d] : 0.f;
        }
        if (lane < count) {
            beta_s[lane] = beta[(size_t)(base + lane) * H + h];
            kq_s[lane] = kq[(size_t)(base + lane) * G + g];
        }
        __syncwarp();
        for (int t = 0; t < count; ++t) {
            const int n = base + t;
            const float vv = live ? to_f32(v[(size_t)n * v_stride + v_col + h * DV + col]) : 0.f;
            float rk = 0.f, rq = 0.f;
#pragma unroll
            for (int d = 0; d < DMAX; d += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(&k_s[t][d]);
                const float4 q4 = *reinterpret_cast<const float4*>(&q_s[t][d]);
                const float4 g4 = *reinterpret_cast<const float4*>(&g_s[t][d]);
                S[d] *= g4.x; S[d + 1] *= g4.y; S[d + 2] *= g4.z; S[d + 3] *= g4.w;
                rk = fmaf(S[d], k4.x, rk); rk = fmaf(S[d + 1], k4.y, rk); rk = fmaf(S[d + 2], k4.z, rk); rk = fmaf(S[d + 3], k4.w, rk);
                rq = fmaf(S[d], q4.x, rq); rq = fmaf(S[d + 1], q4.y, rq); rq = fmaf(S[d + 2], q4.z, rq); rq = fmaf(S[d + 3], q4.w, rq);
            }
            const float u = beta_s[t] * (vv - rk);
#pragma unroll
            for (int d = 0; d < DMAX; d += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(&k_s[t][d]);
                S[d] = fmaf(k4.x, u, S[d]); S[d + 1] = fmaf(k4.y, u, S[d + 1]); S[d + 2] = fmaf(k4.z, u, S[d + 2]); S[d + 3] = fmaf(k4.w, u, S[d + 3]);
            }
            if (live) out[(size_t)n * H * DV + h * DV + col] = fmaf(u, kq_s[t], rq);
        }
    }
    if (live) {
#pragma unroll
        for (int d = 0; d < DMAX; ++d)
            if (d < D) st[(size_t)d * DV] = S[d];
    }
}

// ------------------------------------------------------------------------------------------------
// The state-space recurrence with one decay per head. Per head, S is [NS, DV]; for every token, in order:
//   dt = softplus(dt_raw + dt_bias[h]);  S <- exp(-exp(A_log[h]) dt) S + dt B x^T;  y = S^T C + D[h] x
// B and C belong to the head's group. A lane owns a column of S (NS entries in registers), as above.
template <typename T, int NMAX>
__global__ void __launch_bounds__(32) ssm_scan_kernel(const T* __restrict__ xbc, int x_stride, int x_col, int b_col, int c_col,
                                                      const T* __restrict__ dt_raw, int dt_stride, const float* __restrict__ A_log,
                                                      const float* __restrict__ dt_bias, const float* __restrict__ Dskip,
                                                      float* __restrict__ state, const int* __restrict__ seq_starts,
                                                      const int* __restrict__ seq_slots, float* __restrict__ out, int H, int G, int NS,
                                                      int DV) {
    __shared__ __align__(16) float b_s[SCAN_TILE][NMAX], c_s[SCAN_TILE][NMAX];
    __shared__ float a_s[SCAN_TILE], dt_s[SCAN_TILE];
    pdl_trigger();
    const int lane = threadIdx.x;
    const int col = blockIdx.x * 32 + lane;
    const int h = blockIdx.y, r = blockIdx.z;
    const int g = h / (H / G);
    const bool live = col < DV;
    const float rate = expf(A_log[h]), bias = dt_bias[h], skip = Dskip[h];
    pdl_wait();
    const int s0 = seq_starts[r], s1 = seq_starts[r + 1];
    float* st = state + (((size_t)seq_slots[r] * H + h) * NS) * DV + col;
    float S[NMAX];
#pragma unroll
    for (int d = 0; d < NMAX; ++d) S[d] = (live && d < NS) ? st[(size_t)d * DV] : 0.f;
    for (int base = s0; base < s1; base += SCAN_TILE) {
        const int count = min(SCAN_TILE, s1 - base);
        __syncwarp();
        for (int i = lane; i < count * NMAX; i += 32) {
            const int t = i / NMAX, d = i % NMAX;
            const size_t row = (size_t)(base + t) * x_stride;
            const bool in = d < NS;
            b_s[t][d] = in ? to_f32(xbc[row + b_col + g * NS + d]) : 0.f;
            c_s[t][d] = in ? to_f32(xbc[row + c_col + g * NS + d]) : 0.f;
        }
        if (lane < count) {
            const float dt = softplus_f(to_f32(dt_raw[(size_t)(base + lane) * dt_stride + h]) + bias);
            dt_s[lane] = dt;
            a_s[lane] = expf(-rate * dt);
        }
        __syncwarp();
        for (int t = 0; t < count; ++t) {
            const int n = base + t;
            const float x = live ? to_f32(xbc[(size_t)n * x_stride + x_col + h * DV + col]) : 0.f;
            const float a = a_s[t], u = dt_s[t] * x;
            float y = 0.f;
#pragma unroll
            for (int d = 0; d < NMAX; d += 4) {
                const float4 b4 = *reinterpret_cast<const float4*>(&b_s[t][d]);
                const float4 c4 = *reinterpret_cast<const float4*>(&c_s[t][d]);
                S[d] = fmaf(a, S[d], b4.x * u); S[d + 1] = fmaf(a, S[d + 1], b4.y * u);
                S[d + 2] = fmaf(a, S[d + 2], b4.z * u); S[d + 3] = fmaf(a, S[d + 3], b4.w * u);
                y = fmaf(S[d], c4.x, y); y = fmaf(S[d + 1], c4.y, y); y = fmaf(S[d + 2], c4.z, y); y = fmaf(S[d + 3], c4.w, y);
            }
            if (live) out[(size_t)n * H * DV + h * DV + col] = fmaf(skip, x, y);
        }
    }
    if (live) {
#pragma unroll
        for (int d = 0; d < NMAX; ++d)
            if (d < NS) st[(size_t)d * DV] = S[d];
    }
}

template <typename T>
int launch_conv(const T* z, int z_stride, int C, const float* w, const float* bias, float* state, const int* seq_starts,
                const int* seq_slots, T* out, int out_stride, int taps, int act, int R, int max_rows, cudaStream_t s) {
    const dim3 grid((C + 127) / 128, (max_rows + CONV_CHUNK - 1) / CONV_CHUNK, R);
    return launch_kernel(causal_conv_kernel<T>, grid, dim3(128), 0, s, z, z_stride, C, w, bias, state, seq_starts, seq_slots, out,
                         out_stride, taps, act);
}

template <typename T>
int launch_delta_scan(const T* v, int v_stride, int v_col, const float* qn, const float* kn, const float* kq, const float* decay,
                      const float* beta, float* state, const int* seq_starts, const int* seq_slots, float* out, int H, int G, int D,
                      int DV, int R, cudaStream_t s) {
    const dim3 grid((DV + 31) / 32, H, R);
#define LLMIE_DELTA(DM) return launch_kernel(delta_scan_kernel<T, DM>, grid, dim3(32), 0, s, v, v_stride, v_col, qn, kn, kq, decay, beta, state, \
                                             seq_starts, seq_slots, out, H, G, D, DV)
    if (D <= 16) LLMIE_DELTA(16);
    if (D <= 32) LLMIE_DELTA(32);
    if (D <= 64) LLMIE_DELTA(64);
    if (D <= 128) LLMIE_DELTA(128);
    LLMIE_DELTA(256);
#undef LLMIE_DELTA
}

template <typename T>
int launch_ssm_scan(const T* xbc, int x_stride, int x_col, int b_col, int c_col, const T* dt_raw, int dt_stride, const float* A_log,
                    const float* dt_bias, const float* Dskip, float* state, const int* seq_starts, const int* seq_slots, float* out,
                    int H, int G, int NS, int DV, int R, cudaStream_t s) {
    const dim3 grid((DV + 31) / 32, H, R);
#define LLMIE_SSM(NM) return launch_kernel(ssm_scan_kernel<T, NM>, grid, dim3(32), 0, s, xbc, x_stride, x_col, b_col, c_col, dt_raw, dt_stride, \
                                           A_log, dt_bias, Dskip, state, seq_starts, seq_slots, out, H, G, NS, DV)
    if (NS <= 16) LLMIE_SSM(16);
    if (NS <= 32) LLMIE_SSM(32);
    if (NS <= 64) LLMIE_SSM(64);
    if (NS <= 128) LLMIE_SSM(128);
    LLMIE_SSM(256);
#undef LLMIE_SSM
}

}  // namespace

// z: columns 0 .. C - 1 of rows of z_stride elements (the caller offsets the pointer); state [slots][taps - 1][C] float.
LLMIE_API int llmie_causal_conv(const void* z, int z_stride, int C, const float* w, const float* bias, float* state,
                                const int* seq_starts, const int* seq_slots, void* out, int out_stride, int taps, int act, int R,
                                int max_rows, int dtype, cudaStream_t s) {
    if (R <= 0 || max_rows <= 0 || C <= 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS || R > 65535 || (max_rows + CONV_CHUNK - 1) / CONV_CHUNK > 65535 || act < 0 || act > 1)
        return LLMIE_ERR_BAD_ARGUMENT;
    if (dtype == DT_F32)
        return launch_conv<float>((const float*)z, z_stride, C, w, bias, state, seq_starts, seq_slots, (float*)out, out_stride, taps, act, R, max_rows, s);
    return launch_conv<bf16>((const bf16*)z, z_stride, C, w, bias, state, seq_starts, seq_slots, (bf16*)out, out_stride, taps, act, R, max_rows, s);
}

LLMIE_API int llmie_delta_prepare(const void* qkv, int qkv_stride, int q_col, int k_col, const void* a, int a_stride, const void* b,
                                  int b_stride, const float* A_log, const float* dt_bias, float* qn, float* kn, float* kq, float* decay,
                                  float* beta, int N, int H, int G, int D, float q_scale, float unit_eps, int dtype, cudaStream_t s) {
    if (N <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0) return LLMIE_ERR_BAD_ARGUMENT;
    const dim3 grid(((size_t)N * H + 3) / 4);
    if (dtype == DT_F32)
        return launch_kernel(delta_prepare_kernel<float>, grid, dim3(128), 0, s, (const float*)qkv, qkv_stride, q_col, k_col, (const float*)a,
                             a_stride, (const float*)b, b_stride, A_log, dt_bias, qn, kn, kq, decay, beta, N, H, G, D, q_scale, unit_eps);
    return launch_kernel(delta_prepare_kernel<bf16>, grid, dim3(128), 0, s, (const bf16*)qkv, qkv_stride, q_col, k_col, (const bf16*)a, a_stride,
                         (const bf16*)b, b_stride, A_log, dt_bias, qn, kn, kq, decay, beta, N, H, G, D, q_scale, unit_eps);
}

// state [slots][H][D][DV] float; out [N][H * DV] float
LLMIE_API int llmie_delta_scan(const void* v, int v_stride, int v_col, const float* qn, const float* kn, const float* kq,
                               const float* decay, const float* beta, float* state, const int* seq_starts, const int* seq_slots,
                               float* out, int H, int G, int D, int DV, int R, int dtype, cudaStream_t s) {
    if (R <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || D > 256 || DV <= 0 || H > 65535 || R > 65535) return LLMIE_ERR_BAD_ARGUMENT;
    if (dtype == DT_F32)
        return launch_delta_scan<float>((const float*)v, v_stride, v_col, qn, kn, kq, decay, beta, state, seq_starts, seq_slots, out, H, G, D, DV, R, s);
    return launch_delta_scan<bf16>((const bf16*)v, v_stride, v_col, qn, kn, kq, decay, beta, state, seq_starts, seq_slots, out, H, G, D, DV, R, s);
}

// state [slots][H][NS][DV] float; out [N][H * DV] float
LLMIE_API int llmie_ssm_scan(const void* xbc, int x_stride, int x_col, int b_col, int c_col, const void* dt_raw, int dt_stride,
                             const float* A_log, const float* dt_bias, const float* Dskip, float* state, const int* seq_starts,
                             const int* seq_slots, float* out, int H, int G, int NS, int DV, int R, int dtype, cudaStream_t s) {
    if (R <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || NS <= 0 || NS > 256 || DV <= 0 || H > 65535 || R > 65535) return LLMIE_ERR_BAD_ARGUMENT;
    if (dtype == DT_F32)
        return launch_ssm_scan<float>((const float*)xbc, x_stride, x_col, b_col, c_col, (const float*)dt_raw, dt_stride, A_log, dt_bias, Dskip,
                                      state, seq_starts, seq_slots, out, H, G, NS, DV, R, s);
    return launch_ssm_scan<bf16>((const bf16*)xbc, x_stride, x_col, b_col, c_col, (const bf16*)dt_raw, dt_stride, A_log, dt_bias, Dskip, state,
                                 seq_starts, seq_slots, out, H, G, NS, DV, R, s);
}
