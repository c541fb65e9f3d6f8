// Between the q/k/v projection and the attention, for mixers whose heads are normed and only partly rotated: per head an
// optional root-mean-square norm with a weight, the rotation of the head's first `rot_dims` entries (pairs (i, i + rot_dims / 2)
// or neighbours (2 i, 2 i + 1)), then the query heads to a row of their own and the key and value heads into the token's
// cache slot. Keys and values may differ in size. Norm and rotation are 32-bit; one warp per (token, head).
#include <math.h>

#include "common.cuh"

namespace {

// z row: [nq heads of dk | nkv heads of dk | nkv heads of dv] from column 0. cos_t / sin_t: [N, rot_dims / 2] (already
// multiplied by whatever factor the encoding puts on them), null when nothing turns.
template <typename T>
__global__ void __launch_bounds__(128) qk_norm_rope_store_kernel(const T* __restrict__ z, int z_stride, T* __restrict__ q_out,
                                                                 const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                                                 const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                                 int rot_dims, int interleaved, const int* __restrict__ slots,
                                                                 T* __restrict__ k_pool, T* __restrict__ v_pool, int N, int nq, int nkv,
                                                                 int dk, int dv, int page_size, int write_kv) {
    pdl_trigger();
    pdl_wait();
    const int heads = nq + 2 * nkv;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (item >= N * heads) return;
    const int n = item / heads, j = item % heads;
    if (j >= nq && !write_kv) return;
    size_t dst_row = 0;
    if (j >= nq) {
        const int slot = slots[n];
        const int page = slot / page_size, off = slot % page_size;
        dst_row = ((size_t)page * nkv + (j - nq) % nkv) * page_size + off;
    }
    if (j >= nq + nkv) {   // a value head: copied as it is
        const T* src = z + (size_t)n * z_stride + (size_t)(nq + nkv) * dk + (size_t)(j - nq - nkv) * dv;
        T* dst = v_pool + dst_row * dv;
        for (int i = lane; i < dv; i += 32) dst[i] = src[i];
        return;
    }
    const T* src = z + (size_t)n * z_stride + (size_t)j * dk;
    T* dst = j < nq ? q_out + ((size_t)n * nq + j) * dk : k_pool + dst_row * dk;
    const float* w = j < nq ? q_w : k_w;
    float f = 1.f;
    if (w) {
        float sq = 0.f;
        for (int i = lane; i < dk; i += 32) { const float v = to_f32(src[i]); sq = fmaf(v, v, sq); }
        f = 1.0f / sqrtf(warp_sum(sq) / (float)dk + eps);
    }
    const int half = rot_dims / 2;
    for (int i = lane; i < half; i += 32) {
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
        float a = to_f32(src[ia]) * f, b = to_f32(src[ib]) * f;
        if (w) { a *= w[ia]; b *= w[ib]; }
        const float c = cos_t[(size_t)n * half + i], sn = sin_t[(size_t)n * half + i];
        dst[ia] = from_f32<T>(a * c - b * sn);
        dst[ib] = from_f32<T>(b * c + a * sn);
    }
    for (int i = rot_dims + lane; i < dk; i += 32) {
        float a = to_f32(src[i]) * f;
        if (w) a *= w[i];
        dst[i] = from_f32<T>(a);
    }
}

}  // namespace

LLMIE_API int llmie_qk_norm_rope_store(const void* z, int z_stride, void* q_out, const float* q_w, const float* k_w, float eps,
                                       const float* cos_t, const float* sin_t, int rot_dims, int interleaved, const int* slots,
                                       void* k_pool, void* v_pool, int N, int nq, int nkv, int dk, int dv, int page_size, int write_kv,
                                       int dtype, cudaStream_t s) {
    if (N <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || dk <= 0 || dv <= 0 || rot_dims < 0 || rot_dims % 2 || rot_dims > dk || page_size <= 0 ||
        (rot_dims && (!cos_t || !sin_t)) || (write_kv && (!slots || !k_pool || !v_pool)) || ((q_w == nullptr) != (k_w == nullptr)))
        return LLMIE_ERR_BAD_ARGUMENT;
    const long long items = (long long)N * (nq + 2 * nkv);
    const dim3 grid((unsigned)((items + 3) / 4));
    if (dtype == DT_F32)
        return launch_kernel(qk_norm_rope_store_kernel<float>, grid, dim3(128), 0, s, (const float*)z, z_stride, (float*)q_out, q_w, k_w, eps, cos_t,
                             sin_t, rot_dims, interleaved, slots, (float*)k_pool, (float*)v_pool, N, nq, nkv, dk, dv, page_size, write_kv);
    return launch_kernel(qk_norm_rope_store_kernel<bf16>, grid, dim3(128), 0, s, (const bf16*)z, z_stride, (bf16*)q_out, q_w, k_w, eps, cos_t, sin_t,
                         rot_dims, interleaved, slots, (bf16*)k_pool, (bf16*)v_pool, N, nq, nkv, dk, dv, page_size, write_kv);
}
