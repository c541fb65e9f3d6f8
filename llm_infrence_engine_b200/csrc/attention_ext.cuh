// Paged attention of single tokens with the extras that some mixers ask for, in float32 or bfloat16 storage with all
// arithmetic in 32-bit. It is the generic kernel's scheme (one block per token, key/value head, chunk of the group's query
// heads and slice of the keys; four warps of 32 keys each; online softmax; slices merged by a second kernel) with
//
//   * keys and values of different sizes (dk, dv), and values that may lie INSIDE the key rows (their first dv entries,
//     `v_pool == nullptr`): a latent cache row serves as key and as value;
//   * a query temperature: the scores of the token at position p are multiplied by 1 + coef * ln(floor((p + 1) / every) + 1);
//   * a bias by distance: rel[row(p - j), head] is added to the scaled score, row(n) = rows_of[n] for n < n_rows_of and the
//     table's last row beyond;
//   * a sink: exp(sink[head]) joins the softmax's denominator once (it has no key and no value, and is not scaled);
//   * an output gate: the result is multiplied by sigmoid(gate[n, head]) or sigmoid(gate[n, head * dv + i]);
//   * a sliding window, as in the generic kernel; with `keep_first` the first tokens of the request stay visible after the
//     window has passed them (at their true positions);
//   * chunks: with `chunk` > 0 a position sees only keys of its own run of `chunk` positions, counted from the request's start;
//   * a soft cap: score <- cap * tanh(score / cap), applied to the scaled score.
//
// Each extra is off when its pointer is null (or `temp_every` is 0). Sink and gate are applied where a (token, head) is
// finished: in the block when there is one slice, in the merge kernel otherwise. With `slice_keys` > 0 the slices lie at
// fixed places of the request, so every bit of a token's result depends on its own position alone.
#pragma once
#include <math.h>

#include "common.cuh"

namespace attn_ext {

constexpr int WARPS = 4;

struct Extras {
    float temp_coef;          // query temperature (see above); temp_every == 0: none
    int temp_every;
    const float* rel;         // [rel_rows, nq] or null
    const int* rows_of;       // [n_rows_of]: distance -> row of rel
    int n_rows_of, rel_rows;
    const float* sink;        // [nq] or null
    const void* gate;         // storage type of q; row n starts at gate + n * gate_stride
    int gate_stride, gate_mode;  // 0: none, 1: one number per head, 2: one per output element
    int keep_first = 0;       // keys below this position are seen even when the window has passed them
    int chunk = 0;            // > 0: only keys with floor(key / chunk) == floor(position / chunk) are seen
    float softcap = 0.f;      // > 0: the scaled score s becomes softcap * tanh(s / softcap)
};

// First key that position p may see apart from the kept first tokens (window and chunk together).
__device__ __forceinline__ int first_visible(int p, int window, const Extras& ex) {
    int lo = window > 0 ? max(0, p - window + 1) : 0;
    if (ex.chunk > 0) lo = max(lo, (p / ex.chunk) * ex.chunk);
    return lo;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// What the sums of one (token, head) are multiplied by at the end: the sink joins the denominator, then the division and the
// gate per head. The same arithmetic wherever a (token, head) is finished, so that a result does not depend on whether its
// keys were cut into slices.
template <typename T>
__device__ __forceinline__ float finish_scale(float M, float L, const Extras& ex, int head, const T* gate_row) {
    float f = 1.f;
    if (ex.sink) {
        const float sk = ex.sink[head];
        const float M2 = fmaxf(M, sk);
        f = expf(M - M2);   // M = -inf (no visible key) gives 0
        L = L * f + expf(sk - M2);
    }
    float g = f / L;
    if (ex.gate_mode == 1) g *= sigmoidf_(to_f32(gate_row[head]));
    return g;
}

template <typename T>
__device__ __forceinline__ float finish(float A, float M, float L, const Extras& ex, int head, int dim, int dv, const T* gate_row) {
    float o = A * finish_scale<T>(M, L, ex, head, gate_row);
    if (ex.gate_mode == 2) o *= sigmoidf_(to_f32(gate_row[(size_t)head * dv + dim]));
    return o;
}

template <typename T, int DPL, int GC>
__global__ void __launch_bounds__(WARPS * 32) paged_attn_ext_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
    const int* __restrict__ block_table, int max_blocks, const int* __restrict__ token_seq, const int* __restrict__ positions,
    T* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml, int nq, int nkv, int dk, int dv, int page_size,
    float scale, int window, int num_splits, int slice_keys, int vec_ok, Extras ex) {
    constexpr int DMAX = DPL * 32;
    extern __shared__ __align__(16) float smem[];
    const int dkp = (dk + 3) & ~3;
    float* qs = smem;                                  // [GC][dkp]
    float* ps = qs + GC * dkp;                         // [WARPS][GC][32]
    float* acc_s = ps + WARPS * GC * 32;               // [WARPS][GC][DMAX]
    float* m_s = acc_s + WARPS * GC * DMAX;            // [WARPS][GC]
    float* l_s = m_s + WARPS * GC;                     // [WARPS][GC]

    const int n = blockIdx.x;
    const int G = nq / nkv;
    const int chunks = (G + GC - 1) / GC;
    const int kvh = blockIdx.y / chunks;
    const int g0 = (blockIdx.y % chunks) * GC;
    const int ng = min(GC, G - g0);
    const int split = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    const int p = positions[n];
    const int lo = first_visible(p, window, ex);
    const int kept = min(ex.keep_first, lo);   // keys [0, kept) are seen besides [lo, p]
    const int hi = p + 1;
    int start, end;
    if (slice_keys > 0) {
        start = split * slice_keys;
        end = min(hi, start + slice_keys);
    } else {
        const int from = kept > 0 ? 0 : lo;
        int per = (hi - from + num_splits - 1) / num_splits;
        per = (per + 31) & ~31;
        start = from + split * per;
        end = min(hi, start + per);
    }
    const int* table = block_table + (size_t)token_seq[n] * max_blocks;

    float factor = scale;
    if (ex.temp_every > 0) factor = scale * (1.0f + ex.temp_coef * logf((float)((p + 1) / ex.temp_every + 1)));
    for (int i = threadIdx.x; i < GC * dkp; i += blockDim.x) {
        const int g = i / dkp, c = i % dkp;
        float v = 0.f;
        if (g < ng && c < dk) v = to_f32(q[(size_t)n * q_stride + (size_t)(kvh * G + g0 + g) * dk + c]) * factor;
        qs[i] = v;
    }
    __syncthreads();

    float m[GC], l[GC], acc[GC][DPL];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] = 0.f;
    }

    // values: a pool of their own, or the first dv entries of the key rows
    const T* v_base = v_pool ? v_pool : k_pool;
    const int v_row = v_pool ? dv : dk;

    constexpr int VN = Vec16<T>::N;
    for (int base = start + warp * 32; base < end; base += WARPS * 32) {
        if (base + 32 <= lo && base >= kept) continue;  // every key of the chunk lies before the window and behind the kept ones
        const int key = base + lane;
        const bool valid = key < end && (key >= lo || key < kept);
        int row = 0;
        float s[GC];
#pragma unroll
        for (int g = 0; g < GC; ++g) s[g] = 0.f;
        if (valid) {
            const int blk = table[key / page_size];
            row = (blk * nkv + kvh) * page_size + key % page_size;
            const T* kr = k_pool + (size_t)row * dk;
            if (vec_ok) {
                for (int c = 0; c < dk; c += VN) {
                    float kf[VN];
                    Vec16<T>::load(kr + c, kf);
#pragma unroll
                    for (int g = 0; g < GC; ++g)
#pragma unroll
                        for (int i = 0; i < VN; ++i) s[g] = fmaf(qs[g * dkp + c + i], kf[i], s[g]);
                }
            } else {
                for (int c = 0; c < dk; ++c) {
                    const float kf = to_f32(kr[c]);
#pragma unroll
                    for (int g = 0; g < GC; ++g) s[g] = fmaf(qs[g * dkp + c], kf, s[g]);
                }
            }
            if (ex.softcap > 0.f) {
#pragma unroll
                for (int g = 0; g < GC; ++g) s[g] = ex.softcap * tanhf(s[g] / ex.softcap);
            }
            if (ex.rel) {
                const int dist = p - key;
                const int r = dist < ex.n_rows_of ? ex.rows_of[dist] : ex.rel_rows - 1;
#pragma unroll
                for (int g = 0; g < GC; ++g)
                    if (g < ng) s[g] += ex.rel[(size_t)r * nq + kvh * G + g0 + g];
            }
        }
        float corr[GC];
#pragma unroll
        for (int g = 0; g < GC; ++g) {
            const float sv = valid ? s[g] : -INFINITY;
            const float m_new = fmaxf(m[g], warp_max(sv));
            const float pv = valid ? expf(sv - m_new) : 0.f;
            corr[g] = expf(m[g] - m_new);
            l[g] = l[g] * corr[g] + warp_sum(pv);
            m[g] = m_new;
            ps[(warp * GC + g) * 32 + lane] = pv;
        }
        __syncwarp();
#pragma unroll
        for (int g = 0; g < GC; ++g)
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[g][i] *= corr[g];
        const int count = min(32, end - base);
        for (int j = 0; j < count; ++j) {
            if (base + j < lo && base + j >= kept) continue;
            const int rj = __shfl_sync(0xffffffffu, row, j);
            const T* vr = v_base + (size_t)rj * v_row;
            float vv[DPL];
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int dim = lane + 32 * i;
                vv[i] = dim < dv ? to_f32(vr[dim]) : 0.f;
            }
#pragma unroll
            for (int g = 0; g < GC; ++g) {
                const float pj = ps[(warp * GC + g) * 32 + j];
#pragma unroll
                for (int i = 0; i < DPL; ++i) acc[g][i] = fmaf(pj, vv[i], acc[g][i]);
            }
        }
        __syncwarp();
    }

#pragma unroll
    for (int g = 0; g < GC; ++g) {
        if (lane == 0) { m_s[warp * GC + g] = m[g]; l_s[warp * GC + g] = l[g]; }
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc_s[(warp * GC + g) * DMAX + lane + 32 * i] = acc[g][i];
    }
    __syncthreads();

    const T* gate_row = ex.gate_mode ? reinterpret_cast<const T*>(ex.gate) + (size_t)n * ex.gate_stride : nullptr;
    for (int i = threadIdx.x; i < ng * dv; i += blockDim.x) {
        const int g = i / dv, dim = i % dv;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, m_s[w * GC + g]);
        float L = 0.f, A = 0.f;
        if (M > -INFINITY) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float f = expf(m_s[w * GC + g] - M);
                L = fmaf(l_s[w * GC + g], f, L);
                A = fmaf(acc_s[(w * GC + g) * DMAX + dim], f, A);
            }
        }
        const int head = kvh * G + g0 + g;
        if (num_splits == 1) {
            out[((size_t)n * nq + head) * dv + dim] = from_f32<T>(finish<T>(A, M, L, ex, head, dim, dv, gate_row));
        } else {
            const size_t slot = ((size_t)n * nq + head) * num_splits + split;
            part_acc[slot * dv + dim] = A;
            if (dim == 0) { part_ml[slot * 2] = M; part_ml[slot * 2 + 1] = L; }
        }
    }
}

// The slices of one (token, head) merged, then finished (sink, division, gate). A slice's weight e^(m_s - M) is computed once
// (the first warp, a slice per lane) and kept in shared memory; every sum runs in one fixed order.
template <typename T>
__global__ void attn_ext_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, T* __restrict__ out,
                                        int nq, int dv, int num_splits, Extras ex) {
    constexpr int KEPT = 128;
    __shared__ float w_s[KEPT];
    __shared__ float scale_s, max_s;
    const size_t th = blockIdx.x;  // token * nq + head
    const int n = (int)(th / nq), head = (int)(th % nq);
    const float* ml = part_ml + th * num_splits * 2;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float M = -INFINITY;
        for (int s = lane; s < num_splits; s += 32) M = fmaxf(M, ml[2 * s]);
        M = warp_max(M);
        float L = 0.f;
        for (int s = lane; s < num_splits; s += 32) {
            const float w = ml[2 * s] > -INFINITY ? expf(ml[2 * s] - M) : 0.f;
            if (s < KEPT) w_s[s] = w;
            L = fmaf(ml[2 * s + 1], w, L);
        }
        L = warp_sum(L);
        if (lane == 0) {
            scale_s = finish_scale<T>(M, L, ex, head, ex.gate_mode ? reinterpret_cast<const T*>(ex.gate) + (size_t)n * ex.gate_stride : nullptr);
            max_s = M;
        }
    }
    __syncthreads();
    const float g = scale_s, M = max_s;
    const T* gate_row = ex.gate_mode == 2 ? reinterpret_cast<const T*>(ex.gate) + (size_t)n * ex.gate_stride + (size_t)head * dv : nullptr;
    const float* acc = part_acc + th * num_splits * dv;
    for (int dim = threadIdx.x; dim < dv; dim += blockDim.x) {
        float A = 0.f;
#pragma unroll 4
        for (int s = 0; s < num_splits; ++s) {   // (unrolled: four slices' loads are in flight; the order of the additions stays)
            const float w = s < KEPT ? w_s[s] : (ml[2 * s] > -INFINITY ? expf(ml[2 * s] - M) : 0.f);
            A = fmaf(acc[(size_t)s * dv + dim], w, A);
        }
        float o = A * g;
        if (gate_row) o *= sigmoidf_(to_f32(gate_row[dim]));
        out[th * dv + dim] = from_f32<T>(o);
    }
}

inline size_t smem_bytes(int GC, int DPL, int dk) {
    const int dkp = (dk + 3) & ~3;
    return sizeof(float) * ((size_t)GC * dkp + WARPS * GC * 32 + (size_t)WARPS * GC * DPL * 32 + 2 * WARPS * GC);
}

template <typename T, int DPL, int GC>
int launch_one(dim3 grid, cudaStream_t s, const T* q, int q_stride, const T* k_pool, const T* v_pool, const int* block_table,
               int max_blocks, const int* token_seq, const int* positions, T* out, float* part_acc, float* part_ml, int nq, int nkv,
               int dk, int dv, int page_size, float scale, int window, int num_splits, int slice_keys, int vec_ok, const Extras& ex) {
    const size_t smem = smem_bytes(GC, DPL, dk);
    if (smem > 200 * 1024) return LLMIE_ERR_BAD_ARGUMENT;
    if (smem > 48 * 1024) cudaFuncSetAttribute(paged_attn_ext_kernel<T, DPL, GC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    paged_attn_ext_kernel<T, DPL, GC><<<grid, WARPS * 32, smem, s>>>(q, q_stride, k_pool, v_pool, block_table, max_blocks, token_seq,
                                                                     positions, out, part_acc, part_ml, nq, nkv, dk, dv, page_size,
                                                                     scale, window, num_splits, slice_keys, vec_ok, ex);
    return launch_status();
}

// Scratch needed for `num_splits` > 1, in floats: N * nq * num_splits * (dv + 2).
template <typename T>
int paged_attention_ext(const T* q, int q_stride, const T* k_pool, const T* v_pool, const int* block_table, int max_blocks,
                        const int* token_seq, const int* positions, T* out, float* scratch, int N, int nq, int nkv, int dk, int dv,
                        int page_size, float scale, int window, int num_splits, int slice_keys, const Extras& ex, cudaStream_t s) {
    if (N <= 0) return 0;
    if (nkv <= 0 || nq % nkv || dk <= 0 || dv <= 0 || dv > 512 || dk > 4096 || page_size <= 0 || num_splits < 1 || slice_keys < 0 ||
        slice_keys % 32 || (num_splits > 1 && !scratch) || (!v_pool && dv > dk) || (ex.rel && (!ex.rows_of || ex.rel_rows < 1)) ||
        (ex.gate_mode && !ex.gate))
        return LLMIE_ERR_BAD_ARGUMENT;
    constexpr int VN = Vec16<T>::N;
    const int vec_ok = dk % VN == 0 && ((uintptr_t)k_pool % 16 == 0);
    const int G = nq / nkv;
    // heads of a group that a block serves together: fewer for long value rows (the accumulators live in registers)
    int GC = G >= 5 ? 8 : (G >= 3 ? 4 : G);
    if (dv > 128 && GC > 4) GC = 4;
    if (dv > 256 && GC > 2) GC = 2;
    const int chunks = (G + GC - 1) / GC;
    if ((long long)nkv * chunks > 65535 || num_splits > 65535) return LLMIE_ERR_BAD_ARGUMENT;
    const dim3 grid(N, nkv * chunks, num_splits);
    float* part_acc = scratch;
    float* part_ml = scratch ? scratch + (size_t)N * nq * num_splits * dv : nullptr;
    int rc;
#define LLMIE_EXT(DPLV, GCV) rc = launch_one<T, DPLV, GCV>(grid, s, q, q_stride, k_pool, v_pool, block_table, max_blocks, token_seq, positions, out, \
                                                          part_acc, part_ml, nq, nkv, dk, dv, page_size, scale, window, num_splits, slice_keys, vec_ok, ex)
#define LLMIE_EXT_GC(DPLV)                                     \
    switch (GC) {                                              \
        case 1: LLMIE_EXT(DPLV, 1); break;                     \
        case 2: LLMIE_EXT(DPLV, 2); break;                     \
        case 4: LLMIE_EXT(DPLV, 4); break;                     \
        default: LLMIE_EXT(DPLV, 8); break;                    \
    }
    if (dv <= 32) { LLMIE_EXT_GC(1) }
    else if (dv <= 64) { LLMIE_EXT_GC(2) }
    else if (dv <= 128) { LLMIE_EXT_GC(4) }
    else if (dv <= 256) {
        switch (GC) {
            case 1: LLMIE_EXT(8, 1); break;
            case 2: LLMIE_EXT(8, 2); break;
            default: LLMIE_EXT(8, 4); break;
        }
    } else {
        switch (GC) {
            case 1: LLMIE_EXT(16, 1); break;
            default: LLMIE_EXT(16, 2); break;
        }
    }
#undef LLMIE_EXT_GC
#undef LLMIE_EXT
    if (rc) return rc;
    if (num_splits > 1) {
        attn_ext_combine_kernel<T><<<N * nq, 128, 0, s>>>(part_acc, part_ml, out, nq, dv, num_splits, ex);
        rc = launch_status();
    }
    return rc;
}

}  // namespace attn_ext
