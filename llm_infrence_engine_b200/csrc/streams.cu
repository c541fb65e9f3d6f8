// Several residual streams per token (hyper-connections). The streams are one float32 tensor xs[N][S][H].
//
//   expand:  xs[n][s][:] = x[n][:] for every s
//   update:  xs[n][t][:] <- sum_s mix[s][t] xs[n][s][:] + out[t] y[n][:]      (all t from the old streams)
//   norm:    u = sum_s in[s] xs[n][s][:];  h[n][:] = T(u / sqrt(mean(u^2) + eps) * weight)
//
// The norm kernel can carry out an update on its way (`y` given): it reads the old streams once, writes the new ones and
// normalises their weighted sum, so a sublayer's update and the next sublayer's norm are one pass over the streams. With
// `rows` it serves chosen tokens only and stores nothing (the model's last norm, at the rows whose logits are wanted).
// Everything is 32-bit arithmetic in one fixed order per element; y is float32 or the compute dtype.
#include "common.cuh"

namespace {

template <int MAXS, typename TY>
__device__ __forceinline__ void mix_one(float* x, float y, const float* mix_s, const float* out_s, int S) {
    float nw[MAXS];
#pragma unroll
    for (int t = 0; t < MAXS; ++t) {
        if (t < S) {
            float a = 0.f;
#pragma unroll
            for (int s = 0; s < MAXS; ++s)
                if (s < S) a = fmaf(mix_s[s * S + t], x[s], a);
            nw[t] = fmaf(out_s[t], y, a);
        }
    }
#pragma unroll
    for (int t = 0; t < MAXS; ++t)
        if (t < S) x[t] = nw[t];
}

template <int MAXS, typename TY, typename TO>
__global__ void streams_norm_kernel(float* __restrict__ xs, TY* __restrict__ y, int clear_y, const float* __restrict__ mix,
                                    const float* __restrict__ coef_out, const float* __restrict__ coef_in,
                                    const float* __restrict__ weight, TO* __restrict__ out, const int* __restrict__ rows, int S, int H,
                                    float eps) {
    extern __shared__ __align__(16) float sm[];
    float* u_buf = sm;               // H
    float* scratch = u_buf + H;      // 36
    float* mix_s = scratch + 36;     // S * S
    float* out_s = mix_s + S * S;    // S
    float* in_s = out_s + S;         // S
    pdl_trigger();
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) mix_s[i] = mix ? mix[i] : 0.f;
    for (int i = threadIdx.x; i < S; i += blockDim.x) { out_s[i] = coef_out ? coef_out[i] : 0.f; in_s[i] = coef_in[i]; }
    pdl_wait();
    __syncthreads();
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    float* base = xs + (size_t)r * S * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float x[MAXS];
#pragma unroll
        for (int s = 0; s < MAXS; ++s)
            if (s < S) x[s] = base[(size_t)s * H + c];
        if (y) {
            mix_one<MAXS, TY>(x, to_f32(y[(size_t)r * H + c]), mix_s, out_s, S);
            if (clear_y) y[(size_t)r * H + c] = from_f32<TY>(0.f);
            if (!rows) {
#pragma unroll
                for (int s = 0; s < MAXS; ++s)
                    if (s < S) base[(size_t)s * H + c] = x[s];
            }
        }
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < MAXS; ++s)
            if (s < S) u = fmaf(in_s[s], x[s], u);
        u_buf[c] = u;
        ss = fmaf(u, u, ss);
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)blockIdx.x * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = from_f32<TO>(u_buf[c] * rstd * weight[c]);
}

template <int MAXS, typename TY>
__global__ void streams_update_kernel(float* __restrict__ xs, TY* __restrict__ y, int clear_y, const float* __restrict__ mix,
                                      const float* __restrict__ coef_out, int S, int H, long long total) {
    __shared__ float mix_s[MAXS * MAXS], out_s[MAXS];
    pdl_trigger();
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) mix_s[i] = mix[i];
    for (int i = threadIdx.x; i < S; i += blockDim.x) out_s[i] = coef_out[i];
    pdl_wait();
    __syncthreads();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long n = i / H;
    const int c = (int)(i % H);
    float* base = xs + (size_t)n * S * H + c;
    float x[MAXS];
#pragma unroll
    for (int s = 0; s < MAXS; ++s)
        if (s < S) x[s] = base[(size_t)s * H];
    mix_one<MAXS, TY>(x, to_f32(y[i]), mix_s, out_s, S);
    if (clear_y) y[i] = from_f32<TY>(0.f);
#pragma unroll
    for (int s = 0; s < MAXS; ++s)
        if (s < S) base[(size_t)s * H] = x[s];
}

__global__ void streams_expand_kernel(const float* __restrict__ x, float* __restrict__ xs, int S, int H, long long total) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long n = i / H;
    const int c = (int)(i % H);
    const float v = x[i];
    for (int s = 0; s < S; ++s) xs[((size_t)n * S + s) * H + c] = v;
}

template <int MAXS, typename TY, typename TO>
int launch_norm(float* xs, TY* y, int clear_y, const float* mix, const float* coef_out, const float* coef_in, const float* weight, TO* out,
                const int* rows, int n_out, int S, int H, float eps, cudaStream_t s) {
    const size_t smem = sizeof(float) * ((size_t)H + 36 + S * S + 2 * S);
    if (smem > 200 * 1024) return LLMIE_ERR_BAD_ARGUMENT;
    if (smem > 48 * 1024) cudaFuncSetAttribute(streams_norm_kernel<MAXS, TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    int threads = 64;
    while (threads < 512 && threads * 2 <= H) threads *= 2;
    return launch_kernel(streams_norm_kernel<MAXS, TY, TO>, dim3(n_out), dim3(threads), smem, s, xs, y, clear_y, mix, coef_out, coef_in, weight, out,
                         rows, S, H, eps);
}

template <typename TY, typename TO>
int norm_by_streams(float* xs, TY* y, int clear_y, const float* mix, const float* coef_out, const float* coef_in, const float* weight, TO* out,
                    const int* rows, int n_out, int S, int H, float eps, cudaStream_t s) {
    if (S <= 4) return launch_norm<4, TY, TO>(xs, y, clear_y, mix, coef_out, coef_in, weight, out, rows, n_out, S, H, eps, s);
    if (S <= 8) return launch_norm<8, TY, TO>(xs, y, clear_y, mix, coef_out, coef_in, weight, out, rows, n_out, S, H, eps, s);
    return launch_norm<16, TY, TO>(xs, y, clear_y, mix, coef_out, coef_in, weight, out, rows, n_out, S, H, eps, s);
}

template <typename TY>
int update_by_streams(float* xs, TY* y, int clear_y, const float* mix, const float* coef_out, int N, int S, int H, cudaStream_t s) {
    const long long total = (long long)N * H;
    const dim3 grid((unsigned)((total + 255) / 256));
    if (S <= 4) return launch_kernel(streams_update_kernel<4, TY>, grid, dim3(256), 0, s, xs, y, clear_y, mix, coef_out, S, H, total);
    if (S <= 8) return launch_kernel(streams_update_kernel<8, TY>, grid, dim3(256), 0, s, xs, y, clear_y, mix, coef_out, S, H, total);
    return launch_kernel(streams_update_kernel<16, TY>, grid, dim3(256), 0, s, xs, y, clear_y, mix, coef_out, S, H, total);
}

}  // namespace

LLMIE_API int llmie_streams_expand(const float* x, float* xs, int N, int S, int H, cudaStream_t s) {
    if (N <= 0) return 0;
    if (S < 1 || H < 1) return LLMIE_ERR_BAD_ARGUMENT;
    const long long total = (long long)N * H;
    return launch_kernel(streams_expand_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, x, xs, S, H, total);
}

// y_dtype: DT_F32 or DT_BF16. clear_y: y is set to zero after it was read (a buffer that the next sublayer adds into again).
LLMIE_API int llmie_streams_update(float* xs, void* y, int y_dtype, int clear_y, const float* mix, const float* coef_out, int N, int S, int H,
                                   cudaStream_t s) {
    if (N <= 0) return 0;
    if (S < 1 || S > 16 || H < 1 || !y || !mix || !coef_out) return LLMIE_ERR_BAD_ARGUMENT;
    if (y_dtype == DT_F32) return update_by_streams<float>(xs, (float*)y, clear_y, mix, coef_out, N, S, H, s);
    return update_by_streams<bf16>(xs, (bf16*)y, clear_y, mix, coef_out, N, S, H, s);
}

// y == nullptr: no update, only the norm of the weighted sum. rows != nullptr: chosen tokens, nothing stored back.
// With rows and clear_y only the chosen rows of y are cleared.
LLMIE_API int llmie_streams_norm(float* xs, void* y, int y_dtype, int clear_y, const float* mix, const float* coef_out, const float* coef_in,
                                 const float* weight, void* out, int out_dtype, const int* rows, int n_out, int S, int H, float eps,
                                 cudaStream_t s) {
    if (n_out <= 0) return 0;
    if (S < 1 || S > 16 || H < 1 || !coef_in || !weight || (y && (!mix || !coef_out))) return LLMIE_ERR_BAD_ARGUMENT;
    if (out_dtype == DT_F32) {
        if (y_dtype == DT_F32 || !y) return norm_by_streams<float, float>(xs, (float*)y, clear_y, mix, coef_out, coef_in, weight, (float*)out, rows, n_out, S, H, eps, s);
        return norm_by_streams<bf16, float>(xs, (bf16*)y, clear_y, mix, coef_out, coef_in, weight, (float*)out, rows, n_out, S, H, eps, s);
    }
    if (y_dtype == DT_F32 || !y) return norm_by_streams<float, bf16>(xs, (float*)y, clear_y, mix, coef_out, coef_in, weight, (bf16*)out, rows, n_out, S, H, eps, s);
    return norm_by_streams<bf16, bf16>(xs, (bf16*)y, clear_y, mix, coef_out, coef_in, weight, (bf16*)out, rows, n_out, S, H, eps, s);
}
