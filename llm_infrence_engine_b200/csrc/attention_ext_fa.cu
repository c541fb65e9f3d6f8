// Paged attention with extras (see attention_ext.cuh) for PROMPT PORTIONS with keys and values of up to 128 entries, bfloat16:
// the shape in which a warp needs no other warp. A block of four warps works on a tile of 64 rows, row = (token of the tile,
// query head of the group); a warp owns 16 rows and, per chunk of 64 keys, computes all their scores (mma.sync m16n8k16, its
// queries held in registers for the whole tile, keys by ldmatrix from shared memory), scales, biases and masks them, takes
// maxima and sums inside its quads (four lanes share a row), and feeds the rounded weights straight from the score registers
// into the P V products. The only barriers are the two per chunk around the cp.async ring of keys and values (two stages).
// Key slices (grid.z) and the finishing of rows (sink, division, gate) are those of attention_ext_mma.cu.
#include "attention_ext.cuh"

namespace {

using attn_ext::Extras;

constexpr int WARPS = 4, ROWS = 16 * WARPS, KEYS = 64, THREADS = 32 * WARPS;

struct Params {
    const bf16* q; int q_stride;
    const bf16* k_pool; const bf16* v_pool;
    const int* block_table; int max_blocks;
    const int* token_seq; const int* positions; const int* tile_info;
    bf16* out; float* part_acc; float* part_ml;
    int nq, nkv, dk, dv, page_size; float scale; int window, num_splits, gh, head_chunks;
    int bias_in_smem;
    Extras ex;
};

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// KD: steps of 16 over the key entries (dk = 16 KD); NV: pairs of n8 tiles over the value entries (dv = 16 NV)
// MASKS: kept first tokens, chunks and the soft cap are compiled in (else they are not looked at, and cost nothing)
template <int KD, int NV, bool MASKS>
__global__ void __launch_bounds__(THREADS) attn_ext_fa_kernel(const Params P) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int dk = 16 * KD, dv = 16 * NV, ks = dk + 8, vs = dv + 8;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);            // [ROWS][ks]: only until the queries are in registers
    bf16* Ks = Qs + ROWS * ks;                               // [2][KEYS][ks]
    bf16* Vs = Ks + 2 * KEYS * ks;                           // [2][KEYS][vs]
    float* bias_val = reinterpret_cast<float*>(Vs + 2 * KEYS * vs);   // [rel_rows][gh]
    unsigned short* bias_row = reinterpret_cast<unsigned short*>(bias_val + (P.bias_in_smem ? P.ex.rel_rows * P.gh : 0));

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
    const int G = P.nq / P.nkv;
    const int kvh = blockIdx.y / P.head_chunks, hc = blockIdx.y % P.head_chunks;
    const int gh = P.gh;
    const int tokens_per_tile = ROWS / gh;
    const int split = blockIdx.z;

    pdl_trigger();
    if (P.bias_in_smem) {
        for (int i = tid; i < P.ex.rel_rows * gh; i += THREADS) {
            const int g = hc * gh + i % gh;
            bias_val[i] = g < G ? P.ex.rel[(size_t)(i / gh) * P.nq + kvh * G + g] : 0.f;
        }
        for (int i = tid; i < P.ex.n_rows_of; i += THREADS) bias_row[i] = (unsigned short)P.ex.rows_of[i];
    }
    pdl_wait();
    int n0 = P.tile_info[2 * blockIdx.x], ntok = min(P.tile_info[2 * blockIdx.x + 1], tokens_per_tile);
    const int p_first = P.positions[n0], p_last = P.positions[n0 + ntok - 1];
    int lo = P.window > 0 ? max(0, p_first - P.window + 1) : 0;
    if (MASKS && P.ex.chunk > 0) lo = max(lo, (p_first / P.ex.chunk) * P.ex.chunk);
    const int kept = MASKS ? min(P.ex.keep_first, lo) : 0;                   // keys [0, kept) are seen besides [lo, hi)
    const int npre = (MASKS && split == 0 && kept > 0) ? (kept + KEYS - 1) / KEYS : 0;   // their chunks come first, in the first slice
    const int hi = p_last + 1;
    int per = (hi - lo + P.num_splits - 1) / P.num_splits;
    per = (per + KEYS - 1) / KEYS * KEYS;
    const int start = lo + split * per;
    const int end = min(hi, start + per);
    const int* table = P.block_table + (size_t)P.token_seq[n0] * P.max_blocks;

    int row_pos[2], row_head[2], row_tok[2], row_g[2], row_lo[2];   // row_lo: the first key the row sees apart from the kept ones
    float row_factor[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = warp * 16 + gid + 8 * i;
        const int t = row / gh, g = hc * gh + row % gh;
        const bool ok = t < ntok && g < G;
        row_tok[i] = ok ? n0 + t : -1;
        row_head[i] = ok ? kvh * G + g : 0;
        row_g[i] = ok ? row % gh : 0;
        row_pos[i] = ok ? P.positions[n0 + t] : -1;
        row_lo[i] = ok ? (MASKS ? attn_ext::first_visible(row_pos[i], P.window, P.ex) : (P.window > 0 ? max(0, row_pos[i] - P.window + 1) : 0)) : 0;
        float f = P.scale;
        if (P.ex.temp_every > 0 && ok) f = P.scale * (1.0f + P.ex.temp_coef * logf((float)((row_pos[i] + 1) / P.ex.temp_every + 1)));
        row_factor[i] = f;
    }
    const bool warp_live = warp * 16 < ntok * gh;   // a warp without rows only fetches
    // the span of my warp's positions: a chunk that all its rows see in full needs no mask arithmetic
    int w_min = row_pos[0] < 0 || row_pos[1] < 0 ? -1 : min(row_pos[0], row_pos[1]), w_lo = max(row_lo[0], row_lo[1]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        w_min = min(w_min, __shfl_xor_sync(0xffffffffu, w_min, o));   // -1 if any row of the warp is not a row of the tile
        w_lo = max(w_lo, __shfl_xor_sync(0xffffffffu, w_lo, o));      // from this key on, every row of the warp sees what is causal
    }

    constexpr int segs = dk / 8, vsegs = dv / 8;
    for (int i = tid; i < ROWS * segs; i += THREADS) {
        const int row = i / segs, sgm = i % segs;
        const int t = row / gh, g = hc * gh + row % gh;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < ntok && g < G)
            v = *reinterpret_cast<const uint4*>(P.q + (size_t)(n0 + t) * P.q_stride + (size_t)(kvh * G + g) * dk + sgm * 8);
        *reinterpret_cast<uint4*>(Qs + row * ks + sgm * 8) = v;
    }

    // two threads to a key: one look at the block table per thread and chunk, then every second 16-byte piece of the row
    const int my_key = tid >> 1, odd = tid & 1;
    auto load_chunk = [&](int c, int stage) {
        const int key = (c < npre ? c * KEYS : start + (c - npre) * KEYS) + my_key;
        const bool ok = c < npre ? key < kept : (key < end && key >= lo);
        size_t row = 0;
        if (ok) row = ((size_t)table[key / P.page_size] * P.nkv + kvh) * P.page_size + key % P.page_size;
        const int bytes = ok ? 16 : 0;
        bf16* kd = Ks + (stage * KEYS + my_key) * ks;
        const bf16* ksrc = P.k_pool + row * dk;
#pragma unroll
        for (int sgm = odd; sgm < segs; sgm += 2) cp_async16(kd + sgm * 8, ksrc + sgm * 8, bytes);
        bf16* vd = Vs + (stage * KEYS + my_key) * vs;
        const bf16* vsrc = P.v_pool + row * dv;
#pragma unroll
        for (int sgm = odd; sgm < vsegs; sgm += 2) cp_async16(vd + sgm * 8, vsrc + sgm * 8, bytes);
    };

    const int nchunks = npre + (end > start ? (end - start + KEYS - 1) / KEYS : 0);
    if (nchunks > 0) load_chunk(0, 0);
    cp_commit();
    __syncthreads();
    // my 16 rows of Q as A operands, kept for the whole tile
    uint32_t qf[KD][4];
#pragma unroll
    for (int k = 0; k < KD; ++k) ldsm_x4(qf[k][0], qf[k][1], qf[k][2], qf[k][3], Qs + (warp * 16 + (lane & 15)) * ks + k * 16 + (lane >> 4) * 8);

    float acc[2 * NV][4];
#pragma unroll
    for (int t = 0; t < 2 * NV; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    for (int c = 0; c < nchunks; ++c) {
        const int stage = c & 1;
        const int base = c < npre ? c * KEYS : start + (c - npre) * KEYS;
        const int range_lo = c < npre ? 0 : lo, range_hi = c < npre ? kept : end;
        __syncthreads();                      // everyone is done with the stage that is filled next
        if (c + 1 < nchunks) load_chunk(c + 1, stage ^ 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();                      // chunk c is in shared memory
        if (!warp_live) continue;

        // ---- S: 16 rows x 64 keys = 8 tiles of 8 keys
        float s[8][4];
#pragma unroll
        for (int t = 0; t < 8; ++t) s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
        {
            const bf16* kb = Ks + stage * KEYS * ks + ((lane & 7) + ((lane >> 4) << 3)) * ks + ((lane >> 3) & 1) * 8;
#pragma unroll
            for (int k = 0; k < KD; ++k) {
#pragma unroll
                for (int t = 0; t < 8; t += 2) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(b0, b1, b2, b3, kb + (t * 8) * ks + k * 16);
                    mma_bf16(s[t], qf[k][0], qf[k][1], qf[k][2], qf[k][3], b0, b1);
                    mma_bf16(s[t + 1], qf[k][0], qf[k][1], qf[k][2], qf[k][3], b2, b3);
                }
            }
        }
        // scale, bias, mask; element (tile t, e): row gid + 8 * (e >> 1), key base + t * 8 + 2 * tig + (e & 1)
        float mx[2] = {-INFINITY, -INFINITY};
        const bool interior = c >= npre && w_min >= 0 && base + KEYS - 1 <= w_min && base + KEYS <= end && base >= lo && base >= w_lo;
        if (interior) {
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    float v = s[t][e] * row_factor[i];
                    if (MASKS && P.ex.softcap > 0.f) v = P.ex.softcap * tanhf(v / P.ex.softcap);
                    if (P.ex.rel) {
                        const int dist = row_pos[i] - (base + t * 8 + 2 * tig + (e & 1));
                        if (P.bias_in_smem) {
                            const int br = dist < P.ex.n_rows_of ? bias_row[dist] : P.ex.rel_rows - 1;
                            v += bias_val[br * gh + row_g[i]];
                        } else {
                            const int br = dist < P.ex.n_rows_of ? P.ex.rows_of[dist] : P.ex.rel_rows - 1;
                            v += P.ex.rel[(size_t)br * P.nq + row_head[i]];
                        }
                    }
                    s[t][e] = v;
                    mx[i] = fmaxf(mx[i], v);
                }
        } else {
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    const int key = base + t * 8 + 2 * tig + (e & 1);
                    const int p = row_pos[i];
                    const bool seen = key <= p && key < range_hi && key >= range_lo && (key >= row_lo[i] || (MASKS && key < P.ex.keep_first));
                    float v = -INFINITY;
                    if (seen) {
                        v = s[t][e] * row_factor[i];
                        if (MASKS && P.ex.softcap > 0.f) v = P.ex.softcap * tanhf(v / P.ex.softcap);
                        if (P.ex.rel) {
                            const int dist = p - key;
                            if (P.bias_in_smem) {
                                const int br = dist < P.ex.n_rows_of ? bias_row[dist] : P.ex.rel_rows - 1;
                                v += bias_val[br * gh + row_g[i]];
                            } else {
                                const int br = dist < P.ex.n_rows_of ? P.ex.rows_of[dist] : P.ex.rel_rows - 1;
                                v += P.ex.rel[(size_t)br * P.nq + row_head[i]];
                            }
                        }
                    }
                    s[t][e] = v;
                    mx[i] = fmaxf(mx[i], v);
                }
        }
        float corr[2], m_use[2], sum[2] = {0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            const float m_new = fmaxf(m_run[i], mx[i]);
            m_use[i] = m_new == -INFINITY ? 0.f : m_new;
            corr[i] = expf(m_run[i] - m_use[i]);
            m_run[i] = m_new;
        }
        // the weights, rounded to bfloat16 as the products use them (the sums are taken over the rounded weights), as A operands
        uint32_t pf[4][4];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                // (the weights are rounded to 8 bits: the fast exponential's 1e-7 does not show)
                const uint32_t pb = pack2(__expf(s[t][2 * i] - m_use[i]), __expf(s[t][2 * i + 1] - m_use[i]));
                const __nv_bfloat162 back = *reinterpret_cast<const __nv_bfloat162*>(&pb);
                sum[i] += __low2float(back) + __high2float(back);
                pf[t >> 1][(t & 1) * 2 + i] = pb;   // step t / 2: a0, a1 from tile 2 kk (rows gid, gid + 8), a2, a3 from tile 2 kk + 1
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
            sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
            l_run[i] = l_run[i] * corr[i] + sum[i];
        }
#pragma unroll
        for (int t = 0; t < 2 * NV; ++t) { acc[t][0] *= corr[0]; acc[t][1] *= corr[0]; acc[t][2] *= corr[1]; acc[t][3] *= corr[1]; }
        // ---- O += P V
        {
            const bf16* vb = Vs + stage * KEYS * vs + (lane & 15) * vs + (lane >> 4) * 8;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                for (int t = 0; t < NV; ++t) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_t(b0, b1, b2, b3, vb + (kk * 16) * vs + t * 16);
                    mma_bf16(acc[2 * t], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b0, b1);
                    mma_bf16(acc[2 * t + 1], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b2, b3);
                }
            }
        }
    }
    cp_wait<0>();

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (row_tok[i] < 0) continue;
        const int n = row_tok[i], head = row_head[i];
        if (P.num_splits == 1) {
            float M = m_run[i], L = l_run[i], f = 1.f;
            if (P.ex.sink) {
                const float sk = P.ex.sink[head];
                const float M2 = fmaxf(M, sk);
                f = expf(M - M2);
                L = L * f + expf(sk - M2);
            }
            const float inv = f / L;
            const bf16* gate_row = P.ex.gate_mode ? reinterpret_cast<const bf16*>(P.ex.gate) + (size_t)n * P.ex.gate_stride : nullptr;
            float gh1 = 1.f;
            if (P.ex.gate_mode == 1) gh1 = attn_ext::sigmoidf_(to_f32(gate_row[head]));
            bf16* o = P.out + ((size_t)n * P.nq + head) * dv;
#pragma unroll
            for (int t = 0; t < 2 * NV; ++t) {
                const int col = t * 8 + 2 * tig;
                float y0 = acc[t][2 * i] * inv * gh1, y1 = acc[t][2 * i + 1] * inv * gh1;
                if (P.ex.gate_mode == 2) {
                    const bf16* gp = gate_row + (size_t)head * dv + col;
                    y0 *= attn_ext::sigmoidf_(to_f32(gp[0]));
                    y1 *= attn_ext::sigmoidf_(to_f32(gp[1]));
                }
                *reinterpret_cast<__nv_bfloat162*>(o + col) = __floats2bfloat162_rn(y0, y1);
            }
        } else {
            const size_t slot = ((size_t)n * P.nq + head) * P.num_splits + split;
            float* pa = P.part_acc + slot * dv;
#pragma unroll
            for (int t = 0; t < 2 * NV; ++t) *reinterpret_cast<float2*>(pa + t * 8 + 2 * tig) = make_float2(acc[t][2 * i], acc[t][2 * i + 1]);
            if (tig == 0) { P.part_ml[slot * 2] = m_run[i]; P.part_ml[slot * 2 + 1] = l_run[i]; }
        }
    }
}

size_t smem_bytes(int dk, int dv) { return 2 * ((size_t)ROWS * (dk + 8) + 2 * KEYS * (dk + 8) + 2 * KEYS * (dv + 8)); }
size_t bias_bytes(int rel_rows, int gh, int n_rows_of) { return sizeof(float) * (size_t)rel_rows * gh + 2 * (size_t)((n_rows_of + 1) & ~1); }

template <int KD, int NV, bool MASKS>
int launch_as(const Params& P, dim3 grid, size_t smem, cudaStream_t s) {
    static bool set = false;
    if (!set) {
        cudaFuncSetAttribute(attn_ext_fa_kernel<KD, NV, MASKS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        set = true;
    }
    return launch_kernel(attn_ext_fa_kernel<KD, NV, MASKS>, grid, dim3(THREADS), smem, s, P);
}

template <int KD, int NV>
int launch(const Params& P, dim3 grid, size_t smem, cudaStream_t s) {
    if (P.ex.keep_first > 0 || P.ex.chunk > 0 || P.ex.softcap > 0.f) return launch_as<KD, NV, true>(P, grid, smem, s);
    return launch_as<KD, NV, false>(P, grid, smem, s);
}

}  // namespace

// 64 (the rows of a tile) if the kernel takes these sizes: bfloat16, a value pool of its own, heads of 64 or 128 entries for keys
// and for values (either combination), groups of up to 64 heads; else 0.
LLMIE_API int llmie_attention_ext_fa_fits(int dk, int dv, int own_values, int group) {
    return (own_values && (dk == 64 || dk == 128) && (dv == 64 || dv == 128) && group >= 1) ? ROWS : 0;
}

// tile_info: [tiles][2] = (first token, tokens) with at most 64 / min(group, 64) tokens of one request per tile.
LLMIE_API int llmie_paged_attention_ext_fa(const bf16* q, int q_stride, const bf16* k_pool, const bf16* v_pool, const int* block_table,
                                           int max_blocks, const int* token_seq, const int* positions, const int* tile_info, int tiles,
                                           bf16* out, float* scratch, int N, int nq, int nkv, int dk, int dv, int page_size, float scale,
                                           int window, int num_splits, float temp_coef, int temp_every, const float* rel, const int* rows_of,
                                           int n_rows_of, int rel_rows, const float* sink, const bf16* gate, int gate_stride, int gate_mode,
                                           int keep_first, int chunk, float softcap, cudaStream_t s) {
    if (N <= 0 || tiles <= 0) return 0;
    if (nkv <= 0 || nq % nkv || !llmie_attention_ext_fa_fits(dk, dv, v_pool != nullptr, nq / nkv) || !tile_info || page_size <= 0 ||
        num_splits < 1 || (num_splits > 1 && !scratch) || q_stride % 8 || ((uintptr_t)q % 16) || ((uintptr_t)k_pool % 16) ||
        ((uintptr_t)v_pool % 16) || (rel && (!rows_of || rel_rows < 1)) || (gate_mode && !gate))
        return LLMIE_ERR_BAD_ARGUMENT;
    Params P;
    P.q = q; P.q_stride = q_stride; P.k_pool = k_pool; P.v_pool = v_pool; P.block_table = block_table; P.max_blocks = max_blocks;
    P.token_seq = token_seq; P.positions = positions; P.tile_info = tile_info; P.out = out;
    P.part_acc = scratch; P.part_ml = scratch ? scratch + (size_t)N * nq * num_splits * dv : nullptr;
    P.nq = nq; P.nkv = nkv; P.dk = dk; P.dv = dv; P.page_size = page_size; P.scale = scale; P.window = window; P.num_splits = num_splits;
    const int G = nq / nkv;
    P.gh = G < ROWS ? G : ROWS;
    P.head_chunks = (G + P.gh - 1) / P.gh;
    P.ex.temp_coef = temp_coef; P.ex.temp_every = temp_every; P.ex.rel = rel; P.ex.rows_of = rows_of; P.ex.n_rows_of = n_rows_of;
    P.ex.rel_rows = rel_rows; P.ex.sink = sink; P.ex.gate = gate; P.ex.gate_stride = gate_stride; P.ex.gate_mode = gate_mode;
    P.ex.keep_first = keep_first; P.ex.chunk = chunk; P.ex.softcap = softcap;
    if ((long long)nkv * P.head_chunks > 65535 || num_splits > 65535) return LLMIE_ERR_BAD_ARGUMENT;
    size_t smem = smem_bytes(dk, dv);
    P.bias_in_smem = 0;
    if (rel && rel_rows <= 65535 && bias_bytes(rel_rows, P.gh, n_rows_of) <= 24 * 1024) {
        P.bias_in_smem = 1;
        smem += bias_bytes(rel_rows, P.gh, n_rows_of);
    }
    const dim3 grid(tiles, nkv * P.head_chunks, num_splits);
    int rc;
    if (dk == 64 && dv == 64) rc = launch<4, 4>(P, grid, smem, s);
    else if (dk == 64) rc = launch<4, 8>(P, grid, smem, s);
    else if (dv == 64) rc = launch<8, 4>(P, grid, smem, s);
    else rc = launch<8, 8>(P, grid, smem, s);
    if (rc) return rc;
    if (num_splits > 1) {
        attn_ext::attn_ext_combine_kernel<bf16><<<N * nq, 128, 0, s>>>(P.part_acc, P.part_ml, out, nq, dv, num_splits, P.ex);
        rc = launch_status();
    }
    return rc;
}
