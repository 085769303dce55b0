// Exported launchers of attention_bf16.cu, declared once for every file that calls them
// (attention_decode_noalloc.cu does): a change of a signature then fails to compile instead of
// linking and passing garbage.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Floats of scratch the decode path needs: partial outputs and (max, sum) pairs of every split.
long long ts_attention_bf16_scratch_floats(int num_seqs, int nh, int hd, int max_ctx_len);

// 1 where the tensor-core kernels take these sizes (head 64 or 128, pages of a multiple of 64 tokens).
int ts_attention_bf16_supported(int hd, int page_tokens, int nh, int nkv);

// max_q_len / min_q_len: longest and shortest number of tokens a request feeds in this step (which
// kernels run); max_ctx_len: an upper bound of the lengths of the requests that feed one token (the
// decode grid and scratch).  prefill_seqs (optional, device): the requests that feed more than one
// token, so that the prefill grid has no CTAs for the others.
int ts_paged_attention_bf16(const void* qkv, void* out, const void* k_pool, const void* v_pool, long long page_stride,
                            long long entry_offset, int page_tokens, int num_pages, const int* block_table,
                            int table_width, const int* cu_q, const int* ctx_lens, int num_seqs, int max_q_len,
                            int min_q_len, int max_ctx_len, int nh, int nkv, int hd, float scale, int window,
                            float* scratch, long long scratch_floats, const int* prefill_seqs, int num_prefill_seqs,
                            cudaStream_t stream);

// The same kernels with sigmoid weights: a visible key's weight is sigmoid(score * scale - slopes[h] (i - j) +
// head_bias[h]), nothing is normalised over the keys, and head h's output is multiplied by sigmoid(gate[t, h])
// (null pointers: the term is absent).  Queries in a matrix of their own, q_stride elements a row.
int ts_paged_attention_bf16_sigmoid(const void* q, long long q_stride, void* out, const void* k_pool, const void* v_pool,
                                    long long page_stride, long long entry_offset, int page_tokens, int num_pages,
                                    const int* block_table, int table_width, const int* cu_q, const int* ctx_lens,
                                    int num_seqs, int max_q_len, int min_q_len, int max_ctx_len, int nh, int nkv, int hd,
                                    float scale, int window, float* scratch, long long scratch_floats,
                                    const int* prefill_seqs, int num_prefill_seqs, const float* slopes,
                                    const float* head_bias, const void* gate, long long gate_stride, cudaStream_t stream);

// Softmax attention with options of the mask and of the score: `chunk` n > 0 hides every key before
// floor(i / n) * n from query i, `softcap` c > 0 turns the scaled product into c tanh(. / c), `value_heads` g > 0
// says that the value pool holds g heads (key head j reads value head j / (nkv / g)); the value pool has a geometry
// of its own.  Queries in a matrix of their own, q_stride elements a row.
int ts_paged_attention_bf16_masked(const void* q, long long q_stride, void* out, const void* k_pool, const void* v_pool,
                                   long long page_stride, long long entry_offset, long long v_page_stride,
                                   long long v_entry_offset, int page_tokens, int num_pages, const int* block_table,
                                   int table_width, const int* cu_q, const int* ctx_lens, int num_seqs, int max_q_len,
                                   int min_q_len, int max_ctx_len, int nh, int nkv, int hd, float scale, int window,
                                   int chunk, float softcap, int value_heads, float* scratch, long long scratch_floats,
                                   const int* prefill_seqs, int num_prefill_seqs, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
