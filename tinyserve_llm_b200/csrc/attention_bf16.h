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

#ifdef __cplusplus
}
#endif
