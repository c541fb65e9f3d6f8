// bfloat16 instantiation of the paged attention with extras (temperature, distance bias, sink, gate, values inside the keys).
#include "attention_ext.cuh"

LLMIE_API int llmie_paged_attention_ext_bf16(const bf16* q, int q_stride, const bf16* k_pool, const bf16* v_pool, const int* block_table,
                                           int max_blocks, const int* token_seq, const int* positions, bf16* out, float* scratch, int N,
                                           int nq, int nkv, int dk, int dv, int page_size, float scale, int window, int num_splits,
                                           int slice_keys, float temp_coef, int temp_every, const float* rel, const int* rows_of,
                                           int n_rows_of, int rel_rows, const float* sink, const bf16* gate, int gate_stride, int gate_mode,
                                           int keep_first, int chunk, float softcap, cudaStream_t s) {
    attn_ext::Extras ex;
    ex.temp_coef = temp_coef; ex.temp_every = temp_every;
    ex.rel = rel; ex.rows_of = rows_of; ex.n_rows_of = n_rows_of; ex.rel_rows = rel_rows;
    ex.sink = sink; ex.gate = gate; ex.gate_stride = gate_stride; ex.gate_mode = gate_mode;
    ex.keep_first = keep_first; ex.chunk = chunk; ex.softcap = softcap;
    return attn_ext::paged_attention_ext<bf16>(q, q_stride, k_pool, v_pool, block_table, max_blocks, token_seq, positions, out, scratch, N,
                                            nq, nkv, dk, dv, page_size, scale, window, num_splits, slice_keys, ex, s);
}
