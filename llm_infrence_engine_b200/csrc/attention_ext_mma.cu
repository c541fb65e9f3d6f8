// Paged attention with extras (see attention_ext.cuh) on the tensor cores, bfloat16, for prompt portions and decoded tokens
// alike: keys and values of different sizes up to a latent cache row that is key and value at once (dk = 576, dv = 512),
// query temperature, bias by distance, sink, gate, window.
//
// A block works on a tile of 32, 64 or 128 rows: row = (token of the tile, query head of the group), tokens being neighbours
// of one request, so a chunk of 64 keys is fetched once (cp.async through the block table, two stages) for all of them. Eight
// warps = 2 sets of row blocks of 16 rows x 4 parts. For S = Q K^T (mma.sync m16n8k16, Q and K by ldmatrix from shared memory) a
// part takes 16 of the chunk's 64 keys; the row's maximum and sum over the chunk meet through shared memory (two barriers of
// the row block's 128 threads); P goes to shared memory as bfloat16 and every part multiplies the whole P by ITS quarter of
// the value dimensions (dv / 4 columns, accumulators in registers: 64 floats per thread at dv = 512), so no product is done
// twice. Scores, softmax and accumulators are 32-bit. Key slices (grid.z) leave partial results that the merge kernel of
// attention_ext.cuh finishes; with one slice the block finishes its rows itself.
#include "attention_ext.cuh"

namespace {

using attn_ext::Extras;

constexpr int ROWS = 32, KEYS = 64, THREADS = 256;

struct Params {
    const bf16* q; int q_stride;
    const bf16* k_pool; const bf16* v_pool;
    const int* block_table; int max_blocks;
    const int* token_seq; const int* positions; const int* tile_info;
    bf16* out; float* part_acc; float* part_ml;
    int nq, nkv, dk, dv, page_size; float scale; int window, num_splits, gh, head_chunks;
    int bias_in_smem;   // the distance table's rows (as 16-bit numbers) and this block's heads' columns of it are copied to shared memory
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
__device__ __forceinline__ void ldsm_x2_t(uint32_t& r0, uint32_t& r1, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(a));
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
__device__ __forceinline__ void bar_rows(int id) { asm volatile("bar.sync %0, 128;\n" ::"r"(id)); }

// NT: n8 tiles of a part's value columns (dv = 32 * NT). R: row blocks of 16 rows per warp: a tile has 32 * R rows, and a warp
// (rb, part) works on the row blocks rb * R .. rb * R + R - 1, so a chunk's keys and values are fetched and read from shared
// memory once for R times the rows (prompt portions; decoded tokens take R = 1).
// MASKS: kept first tokens, chunks and the soft cap are compiled in (else they are not looked at, and cost nothing)
template <int NT, int R, int ST, bool MASKS>
__global__ void __launch_bounds__(THREADS) attn_ext_mma_kernel(const Params P) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int ROWS_T = ROWS * R;
    const int dk = P.dk, dv = P.dv;
    const int ks = dk + 8, vs = P.v_pool ? dv + 8 : ks;        // row strides in elements: + 16 bytes keeps ldmatrix off bank conflicts
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);               // [ROWS_T][ks]
    bf16* Ks = Qs + ROWS_T * ks;                                // [ST][KEYS][ks]
    bf16* Vs = P.v_pool ? Ks + ST * KEYS * ks : Ks;             // [ST][KEYS][vs], or the key rows themselves
    bf16* Ps = (P.v_pool ? Vs + ST * KEYS * vs : Ks + ST * KEYS * ks);   // [ROWS_T][KEYS + 8]
    float* red_max = reinterpret_cast<float*>(Ps + ROWS_T * (KEYS + 8));  // [2 R][4][16]
    float* red_sum = red_max + 2 * R * 4 * 16;                  // [2 R][4][16]
    float* bias_val = red_sum + 2 * R * 4 * 16;                 // [rel_rows][gh]: the distance table's columns of this block's heads
    unsigned short* bias_row = reinterpret_cast<unsigned short*>(bias_val + (P.bias_in_smem ? P.ex.rel_rows * P.gh : 0));   // [n_rows_of]
    constexpr int PS = KEYS + 8;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rb = warp >> 2, part = warp & 3, gid = lane >> 2, tig = lane & 3;
    const int G = P.nq / P.nkv;
    const int kvh = blockIdx.y / P.head_chunks, hc = blockIdx.y % P.head_chunks;
    const int gh = P.gh;                       // heads of the group in this chunk's rows
    const int tokens_per_tile = ROWS_T / gh;
    const int split = blockIdx.z;

    pdl_trigger();
    if (P.bias_in_smem) {   // weights of the model: fetched before the wait for the kernel before
        for (int i = tid; i < P.ex.rel_rows * gh; i += THREADS) {
            const int g = hc * gh + i % gh;
            bias_val[i] = g < G ? P.ex.rel[(size_t)(i / gh) * P.nq + kvh * G + g] : 0.f;
        }
        for (int i = tid; i < P.ex.n_rows_of; i += THREADS) bias_row[i] = (unsigned short)P.ex.rows_of[i];
    }
    pdl_wait();
    int n0, ntok;
    if (P.tile_info) { n0 = P.tile_info[2 * blockIdx.x]; ntok = P.tile_info[2 * blockIdx.x + 1]; }
    else { n0 = blockIdx.x; ntok = 1; }
    ntok = min(ntok, tokens_per_tile);
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

    // my rows (gid and gid + 8 of each of my row blocks): token, head, position
    int row_pos[R][2], row_head[R][2], row_tok[R][2], row_g[R][2], row_lo[R][2];   // row_lo: the first key the row sees apart from the kept ones
    float row_factor[R][2];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int row = (rb * R + r) * 16 + gid + 8 * i;
            const int t = row / gh, g = hc * gh + row % gh;
            const bool ok = t < ntok && g < G;
            row_tok[r][i] = ok ? n0 + t : -1;
            row_head[r][i] = ok ? kvh * G + g : 0;
            row_g[r][i] = ok ? row % gh : 0;
            row_pos[r][i] = ok ? P.positions[n0 + t] : -1;
            row_lo[r][i] = ok ? (MASKS ? attn_ext::first_visible(row_pos[r][i], P.window, P.ex) : (P.window > 0 ? max(0, row_pos[r][i] - P.window + 1) : 0)) : 0;
            float f = P.scale;
            if (P.ex.temp_every > 0 && ok) f = P.scale * (1.0f + P.ex.temp_coef * logf((float)((row_pos[r][i] + 1) / P.ex.temp_every + 1)));
            row_factor[r][i] = f;
        }

    // the queries of the tile's rows
    const int segs = dk >> 3;
    for (int i = tid; i < ROWS_T * segs; i += THREADS) {
        const int row = i / segs, sgm = i % segs;
        const int t = row / gh, g = hc * gh + row % gh;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < ntok && g < G)
            v = *reinterpret_cast<const uint4*>(P.q + (size_t)(n0 + t) * P.q_stride + (size_t)(kvh * G + g) * dk + sgm * 8);
        *reinterpret_cast<uint4*>(Qs + row * ks + sgm * 8) = v;
    }

    // A chunk's rows come by cp.async, four threads to a key: one look at the block table per thread and chunk, then the
    // thread's share of the row's 16-byte pieces (pieces quarter, quarter + 4, ...). Keys outside the slice are filled with zeros.
    const int vsegs = dv >> 3;
    const int my_key = tid >> 2, quarter = tid & 3;
    auto load_chunk = [&](int c, int stage) {
        const int key = (c < npre ? c * KEYS : start + (c - npre) * KEYS) + my_key;
        const bool ok = c < npre ? key < kept : (key < end && key >= lo);
        size_t row = 0;
        if (ok) row = ((size_t)table[key / P.page_size] * P.nkv + kvh) * P.page_size + key % P.page_size;
        const int bytes = ok ? 16 : 0;
        bf16* kd = Ks + (stage * KEYS + my_key) * ks;
        const bf16* ksrc = P.k_pool + row * dk;
        for (int sgm = quarter; sgm < segs; sgm += 4) cp_async16(kd + sgm * 8, ksrc + sgm * 8, bytes);
        if (P.v_pool) {
            bf16* vd = Vs + (stage * KEYS + my_key) * vs;
            const bf16* vsrc = P.v_pool + row * dv;
            for (int sgm = quarter; sgm < vsegs; sgm += 4) cp_async16(vd + sgm * 8, vsrc + sgm * 8, bytes);
        }
    };

    // row blocks without a single row of the tile (a decoded token brings only its group's heads) keep out of the arithmetic;
    // a warp none of whose row blocks has one also keeps out of the row blocks' barriers. It still fetches its share of every chunk.
    const int live_rows = ntok * gh;
    int r_live = 0;   // my row blocks 0 .. r_live - 1 hold rows
#pragma unroll
    for (int r = 0; r < R; ++r)
        if ((rb * R + r) * 16 < live_rows) r_live = r + 1;

    float acc[R][NT][4];
    float m_run[R][2], l_run[R][2];
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[r][t][0] = acc[r][t][1] = acc[r][t][2] = acc[r][t][3] = 0.f;
        m_run[r][0] = m_run[r][1] = -INFINITY;
        l_run[r][0] = l_run[r][1] = 0.f;
    }

    // A ring of ST stages: the chunks c + 1 .. c + ST - 1 are on their way while chunk c is worked on (ST = 2 for prompt
    // portions, whose keys come from L2; more for decoded tokens, whose keys come from memory). One group of copies per chunk,
    // also an empty one, so that the count of groups in flight says which chunk has landed.
    const int nchunks = npre + (end > start ? (end - start + KEYS - 1) / KEYS : 0);
#pragma unroll
    for (int i = 0; i < ST - 1; ++i) {
        if (i < nchunks) load_chunk(i, i);
        cp_commit();
    }

    for (int c = 0; c < nchunks; ++c) {
        const int stage = c % ST;
        const int base = c < npre ? c * KEYS : start + (c - npre) * KEYS;
        const int range_lo = c < npre ? 0 : lo, range_hi = c < npre ? kept : end;
        __syncthreads();                      // everyone is done with the stage that is filled next, with P and with the sums
        if (c + ST - 1 < nchunks) load_chunk(c + ST - 1, (c + ST - 1) % ST);
        cp_commit();
        cp_wait<ST - 1>();
        __syncthreads();                      // chunk c (and, the first time, the queries) are in shared memory
        if (r_live == 0) continue;

        // ---- S: my 16 keys of the chunk against my row blocks' rows; two sets of sums (even and odd steps over the inner
        // dimension) keep more products in flight
        float s[R][2][4], s2[R][2][4];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[r][t][e] = s2[r][t][e] = 0.f;
        {
            const bf16* qa = Qs + (rb * R * 16 + (lane & 15)) * ks + (lane >> 4) * 8;
            const bf16* kb = Ks + stage * KEYS * ks + (part * 16 + (lane & 7) + ((lane >> 4) << 3)) * ks + ((lane >> 3) & 1) * 8;
            int k0 = 0;
            for (; k0 + 32 <= dk; k0 += 32) {
                uint32_t b0, b1, b2, b3, d0, d1, d2, d3;
                ldsm_x4(b0, b1, b2, b3, kb + k0);
                ldsm_x4(d0, d1, d2, d3, kb + k0 + 16);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (r >= r_live) break;
                    uint32_t a0, a1, a2, a3, c0, c1, c2, c3;
                    ldsm_x4(a0, a1, a2, a3, qa + r * 16 * ks + k0);
                    ldsm_x4(c0, c1, c2, c3, qa + r * 16 * ks + k0 + 16);
                    mma_bf16(s[r][0], a0, a1, a2, a3, b0, b1);
                    mma_bf16(s[r][1], a0, a1, a2, a3, b2, b3);
                    mma_bf16(s2[r][0], c0, c1, c2, c3, d0, d1);
                    mma_bf16(s2[r][1], c0, c1, c2, c3, d2, d3);
                }
            }
            if (k0 < dk) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(b0, b1, b2, b3, kb + k0);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (r >= r_live) break;
                    uint32_t a0, a1, a2, a3;
                    ldsm_x4(a0, a1, a2, a3, qa + r * 16 * ks + k0);
                    mma_bf16(s[r][0], a0, a1, a2, a3, b0, b1);
                    mma_bf16(s[r][1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        // scale, bias, mask; element (tile t, e): row gid + 8 * (e >> 1), key base + part * 16 + t * 8 + 2 * tig + (e & 1)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (r >= r_live) break;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    const int key = base + part * 16 + t * 8 + 2 * tig + (e & 1);
                    const int p = row_pos[r][i];
                    const bool seen = key <= p && key < range_hi && key >= range_lo && (key >= row_lo[r][i] || (MASKS && key < P.ex.keep_first));
                    float v = -INFINITY;
                    if (seen) {
                        v = (s[r][t][e] + s2[r][t][e]) * row_factor[r][i];
                        if (MASKS && P.ex.softcap > 0.f) v = P.ex.softcap * tanhf(v / P.ex.softcap);
                        if (P.ex.rel) {
                            const int dist = p - key;
                            if (P.bias_in_smem) {
                                const int br = dist < P.ex.n_rows_of ? bias_row[dist] : P.ex.rel_rows - 1;
                                v += bias_val[br * gh + row_g[r][i]];
                            } else {
                                const int br = dist < P.ex.n_rows_of ? P.ex.rows_of[dist] : P.ex.rel_rows - 1;
                                v += P.ex.rel[(size_t)br * P.nq + row_head[r][i]];
                            }
                        }
                    }
                    s[r][t][e] = v;
                    mx[i] = fmaxf(mx[i], v);
                }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                if (tig == 0) red_max[((rb * R + r) * 4 + part) * 16 + gid + 8 * i] = mx[i];
            }
        }
        bar_rows(1 + rb);
        float corr[R][2];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (r >= r_live) break;
            float m_use[2], sum[2] = {0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float m_new = m_run[r][i];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) m_new = fmaxf(m_new, red_max[((rb * R + r) * 4 + q4) * 16 + gid + 8 * i]);
                m_use[i] = m_new == -INFINITY ? 0.f : m_new;
                corr[r][i] = expf(m_run[r][i] - m_use[i]);     // -inf before the first seen key: 0
                m_run[r][i] = m_new;
            }
#pragma unroll
            for (int t = 0; t < 2; ++t) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    // (rounded to 8 bits below: the fast exponential's 1e-7 does not show)
                    const float p0 = __expf(s[r][t][2 * i] - m_use[i]), p1 = __expf(s[r][t][2 * i + 1] - m_use[i]);
                    const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
                    // the sum is taken over the rounded weights: what the product with the values uses
                    sum[i] += __low2float(pb) + __high2float(pb);
                    *reinterpret_cast<__nv_bfloat162*>(Ps + ((rb * R + r) * 16 + gid + 8 * i) * PS + part * 16 + t * 8 + 2 * tig) = pb;
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
                sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
                if (tig == 0) red_sum[((rb * R + r) * 4 + part) * 16 + gid + 8 * i] = sum[i];
            }
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                acc[r][t][0] *= corr[r][0]; acc[r][t][1] *= corr[r][0]; acc[r][t][2] *= corr[r][1]; acc[r][t][3] *= corr[r][1];
            }
        }
        bar_rows(1 + rb);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (r >= r_live) break;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float add = 0.f;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) add += red_sum[((rb * R + r) * 4 + q4) * 16 + gid + 8 * i];
                l_run[r][i] = l_run[r][i] * corr[r][i] + add;
            }
        }
        // ---- O += P V over my quarter of the value columns: a step's values are read once for all my row blocks
        {
            const bf16* pa = Ps + (rb * R * 16 + (lane & 15)) * PS + (lane >> 4) * 8;
            const bf16* vb = Vs + stage * KEYS * vs + part * (NT * 8);
#pragma unroll
            for (int k0 = 0; k0 < KEYS; k0 += 16) {
                uint32_t a[R][4];
#pragma unroll
                for (int r = 0; r < R; ++r)
                    if (r < r_live) ldsm_x4(a[r][0], a[r][1], a[r][2], a[r][3], pa + r * 16 * PS + k0);
#pragma unroll
                for (int t = 0; t + 1 < NT; t += 2) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_t(b0, b1, b2, b3, vb + (k0 + (lane & 15)) * vs + t * 8 + (lane >> 4) * 8);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        if (r >= r_live) break;
                        mma_bf16(acc[r][t], a[r][0], a[r][1], a[r][2], a[r][3], b0, b1);
                        mma_bf16(acc[r][t + 1], a[r][0], a[r][1], a[r][2], a[r][3], b2, b3);
                    }
                }
                if constexpr (NT & 1) {
                    uint32_t b0, b1;
                    ldsm_x2_t(b0, b1, vb + (k0 + (lane & 15)) * vs + (NT - 1) * 8);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        if (r >= r_live) break;
                        mma_bf16(acc[r][NT - 1], a[r][0], a[r][1], a[r][2], a[r][3], b0, b1);
                    }
                }
            }
        }
    }
    cp_wait<0>();

    // ---- finish my rows' quarter of the value columns
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (row_tok[r][i] < 0) continue;
            const int n = row_tok[r][i], head = row_head[r][i];
            if (P.num_splits == 1) {
                float M = m_run[r][i], L = l_run[r][i], f = 1.f;
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
                bf16* o = P.out + ((size_t)n * P.nq + head) * dv + part * (NT * 8);
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const int col = t * 8 + 2 * tig;
                    float y0 = acc[r][t][2 * i] * inv * gh1, y1 = acc[r][t][2 * i + 1] * inv * gh1;
                    if (P.ex.gate_mode == 2) {
                        const bf16* gp = gate_row + (size_t)head * dv + part * (NT * 8) + col;
                        y0 *= attn_ext::sigmoidf_(to_f32(gp[0]));
                        y1 *= attn_ext::sigmoidf_(to_f32(gp[1]));
                    }
                    *reinterpret_cast<__nv_bfloat162*>(o + col) = __floats2bfloat162_rn(y0, y1);
                }
            } else {
                const size_t slot = ((size_t)n * P.nq + head) * P.num_splits + split;
                float* pa = P.part_acc + slot * dv + part * (NT * 8);
#pragma unroll
                for (int t = 0; t < NT; ++t) *reinterpret_cast<float2*>(pa + t * 8 + 2 * tig) = make_float2(acc[r][t][2 * i], acc[r][t][2 * i + 1]);
                if (part == 0 && tig == 0) { P.part_ml[slot * 2] = m_run[r][i]; P.part_ml[slot * 2 + 1] = l_run[r][i]; }
            }
        }
}

size_t smem_bytes(int dk, int dv, bool own_values, int R, int stages = 2) {
    const size_t ks = dk + 8, vs = dv + 8, rows = (size_t)ROWS * R;
    return 2 * (rows * ks + stages * KEYS * ks + (own_values ? stages * KEYS * vs : 0) + rows * (KEYS + 8)) + sizeof(float) * 2 * 2 * R * 4 * 16;
}

// what a copy of the distance table in shared memory takes (see Params::bias_in_smem)
size_t bias_bytes(int rel_rows, int gh, int n_rows_of) { return sizeof(float) * (size_t)rel_rows * gh + 2 * (size_t)((n_rows_of + 1) & ~1); }

constexpr int DEEP = 4;   // stages of the ring for decoded tokens, where shared memory has room for them

template <int NT, int R, int ST, bool MASKS>
int launch_st_as(const Params& P, dim3 grid, size_t smem, cudaStream_t s) {
    static bool set = false;
    if (!set) {
        cudaFuncSetAttribute(attn_ext_mma_kernel<NT, R, ST, MASKS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        set = true;
    }
    return launch_kernel(attn_ext_mma_kernel<NT, R, ST, MASKS>, grid, dim3(THREADS), smem, s, P);
}

template <int NT, int R, int ST>
int launch_st(const Params& P, dim3 grid, size_t smem, cudaStream_t s) {
    if (P.ex.keep_first > 0 || P.ex.chunk > 0 || P.ex.softcap > 0.f) return launch_st_as<NT, R, ST, true>(P, grid, smem, s);
    return launch_st_as<NT, R, ST, false>(P, grid, smem, s);
}

template <int NT, int R>
int launch(const Params& P, dim3 grid, size_t smem, cudaStream_t s, bool deep) {
    if constexpr (R == 1) {
        if (deep) return launch_st<NT, 1, DEEP>(P, grid, smem, s);
    }
    return launch_st<NT, R, 2>(P, grid, smem, s);
}

// the most row blocks per warp that registers allow for value rows of 32 * nt entries
int max_r(int nt) { return nt <= 2 ? 4 : (nt <= 8 ? 2 : 1); }

}  // namespace

// 0 if the kernel does not take these sizes (bfloat16 only): dk a multiple of 16, dv one of 32 * {1, 2, 3, 4, 6, 8, 12, 16}, and
// shared memory for two stages of keys. Otherwise the most rows a tile may have: 32, 64 or 128.
LLMIE_API int llmie_attention_ext_mma_fits(int dk, int dv, int own_values) {
    const int nt = dv / 32;
    const bool nt_ok = dv % 32 == 0 && (nt == 1 || nt == 2 || nt == 3 || nt == 4 || nt == 6 || nt == 8 || nt == 12 || nt == 16);
    if (!(dk % 16 == 0 && dk >= 16 && nt_ok && (own_values || dv <= dk))) return 0;
    for (int r = max_r(nt); r >= 1; r >>= 1)
        if (smem_bytes(dk, dv, own_values != 0, r) <= 227 * 1024) return ROWS * r;
    return 0;
}

// tile_info: [tiles][2] = (first token, tokens) with at most tile_rows / gh tokens of one request per tile, or null: one token per
// tile. tile_rows: 32, 64 or 128 (at most what llmie_attention_ext_mma_fits says); gh = min(group, 32) heads per token in a tile;
// scratch (num_splits > 1): N * nq * num_splits * (dv + 2) floats.
LLMIE_API int llmie_paged_attention_ext_mma(const bf16* q, int q_stride, const bf16* k_pool, const bf16* v_pool, const int* block_table,
                                            int max_blocks, const int* token_seq, const int* positions, const int* tile_info, int tiles,
                                            int tile_rows, bf16* out, float* scratch, int N, int nq, int nkv, int dk, int dv, int page_size,
                                            float scale, int window, int num_splits, float temp_coef, int temp_every, const float* rel,
                                            const int* rows_of, int n_rows_of, int rel_rows, const float* sink, const bf16* gate,
                                            int gate_stride, int gate_mode, int keep_first, int chunk, float softcap, cudaStream_t s) {
    if (N <= 0 || tiles <= 0) return 0;
    const int fits = llmie_attention_ext_mma_fits(dk, dv, v_pool != nullptr);
    if (nkv <= 0 || nq % nkv || !fits || tile_rows > fits || (tile_rows != 32 && tile_rows != 64 && tile_rows != 128) || page_size <= 0 ||
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
    const dim3 grid(tiles, nkv * P.head_chunks, num_splits);
    const int R = tile_rows / ROWS;
    // decoded tokens alone (no tiles of several tokens): a deeper ring where two blocks still fit on a multiprocessor with it
    // (measured at heads of 128, where it costs the second block: batch 64 at 4,096 keys 162 -> 225 us; heads of 64 gain 2 %)
    const size_t table_bytes = rel ? bias_bytes(rel_rows, G < ROWS ? G : ROWS, n_rows_of) : 0;
    const bool deep = !tile_info && R == 1 &&
                      2 * (smem_bytes(dk, dv, v_pool != nullptr, 1, DEEP) + (table_bytes <= 32 * 1024 ? table_bytes : 0) + 1024) <= 227 * 1024;
    size_t smem = smem_bytes(dk, dv, v_pool != nullptr, R, deep ? DEEP : 2);
    P.bias_in_smem = 0;
    if (rel && rel_rows <= 65535 && bias_bytes(rel_rows, P.gh, n_rows_of) <= 32 * 1024 && smem + bias_bytes(rel_rows, P.gh, n_rows_of) <= 227 * 1024) {
        P.bias_in_smem = 1;
        smem += bias_bytes(rel_rows, P.gh, n_rows_of);
    }
    int rc = LLMIE_ERR_BAD_ARGUMENT;
#define LLMIE_MMA(NTV)                                                         \
    if (R == 1) rc = launch<NTV, 1>(P, grid, smem, s, deep);                         \
    else if (R == 2 && NTV <= 8) rc = launch<NTV, (NTV <= 8 ? 2 : 1)>(P, grid, smem, s, false); \
    else if (R == 4 && NTV <= 2) rc = launch<NTV, (NTV <= 2 ? 4 : 1)>(P, grid, smem, s, false);
    switch (dv / 32) {
        case 1: LLMIE_MMA(1) break;
        case 2: LLMIE_MMA(2) break;
        case 3: LLMIE_MMA(3) break;
        case 4: LLMIE_MMA(4) break;
        case 6: LLMIE_MMA(6) break;
        case 8: LLMIE_MMA(8) break;
        case 12: LLMIE_MMA(12) break;
        default: LLMIE_MMA(16) break;
    }
#undef LLMIE_MMA
    if (rc) return rc;
    if (num_splits > 1) {
        attn_ext::attn_ext_combine_kernel<bf16><<<N * nq, 128, 0, s>>>(P.part_acc, P.part_ml, out, nq, dv, num_splits, P.ex);
        rc = launch_status();
    }
    return rc;
}
