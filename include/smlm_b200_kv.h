/* smlm_b200_kv - C ABI of the paged key-value cache next to the SMLM path on B200 (sm_100a): the
 * attention step between the q/k/v projections and the o projection of a decode batch.
 *
 * Conventions are those of smlm_b200.h: raw device pointers, sizes, a cudaStream_t passed as
 * void*, int status (SMLM_OK == 0, codes of smlm_b200.h), nothing synchronises, nothing allocates.
 *
 * The cache layout is the reference's and is shared with its other kernels: a pool of pages, each
 * one tensor [num_layers, 2, num_kv_heads, page_size, head_dim] of the 16-bit storage type
 * (kernel_src/src/loquetier/utils/kvcache.py:40-60), described per batch by
 *   kv_ptrs[total_pages]        device addresses of the pages of all requests, request by request
 *   kv_indptr[batch + 1]        first page of every request in kv_ptrs (int32)
 *   last_page_offset[batch]     valid entries of every request's last page, 1 .. page_size (int32)
 * (BatchedKvCache, kvcache.py:143-165).  A request's sequence length is
 * (pages - 1) * page_size + last_page_offset.  Keys are stored as projected, not rotated.
 *
 * Shapes served: head_dim 128; page_size 8, 16, 32 or 64; num_qo_heads / num_kv_heads in
 * {1, 2, 4, 8}; fp16 and bf16.  Anything else is SMLM_ERR_NO_KERNEL, the reference's
 * "No suitable kernel." (kernel_src/csrc/loquetier_ops.cc:157-159).
 *
 * `status_word` (may be NULL) is a device int that the kernels OR fault bits into instead of
 * touching a bad address: bit 1 an index pointer that is negative, decreasing or reaches past
 * total_pages (or more new tokens than the pages hold), bit 2 a page address that is null or not
 * 16-byte aligned.  Clear it before the call, read it after the stream has caught up.
 */
#ifndef SMLM_B200_KV_H_
#define SMLM_B200_KV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Bytes of the workspace of smlm_b200_batch_decode for this batch shape.  The reference asks its
 * caller for a fixed 64 MiB `tmpbuf` (loquetier_ops.cc:152-153); here the size follows the batch.  The
 * head of the workspace - smlm_b200_batch_decode_ticket_bytes(...) bytes - must be zero when a launch starts;
 * every launch leaves it zeroed again.  So: zero-fill once after allocation, and zero the head again whenever
 * batch_size * num_kv_heads differs from the previous call's on the same workspace (a different shape moves the
 * boundary between the tickets and the parked softmax states).  Launches that may overlap in time must not share
 * a workspace. */
size_t smlm_b200_batch_decode_workspace_bytes(int batch_size, int num_qo_heads, int num_kv_heads);
size_t smlm_b200_batch_decode_ticket_bytes(int batch_size, int num_kv_heads);

/* Decode attention of a batch of one-token requests over their paged caches:
 *   o[b, h] = softmax( rope(q[b, h], L_b - 1) . rope(K_b[:, h / group], 0..L_b-1)^T / sqrt(head_dim) ) . V_b
 * with Llama rotary embedding of base `rope_theta` and scale 1 applied to q and to the keys as they
 * are read.  Replaces batch_decode (kernel_src/csrc/loquetier_ops.cc:138-180; FlashInferBatchDecodeKernel,
 * kernel_src/csrc/flashinfer_adapter/flashinfer_all.cu:85-108; BatchDecodeWithPagedKVCacheKernel,
 * kernel_src/third_party/flashinfer/include/flashinfer/decode.cuh:451-620).  q, o: [batch, num_qo_heads,
 * head_dim], 16-byte aligned.  Every K and V page is read once per kv head; small batches are cut into
 * page ranges whose partial results are merged in a fixed order (deterministic).  A request with no
 * pages yields zeros. */
int smlm_b200_batch_decode(void* o, const void* q, const void* const* kv_ptrs, const int32_t* kv_indptr,
                           const int32_t* last_page_offset, void* workspace, size_t workspace_bytes, int* status_word,
                           int batch_size, int total_pages, int num_qo_heads, int num_kv_heads, int head_dim,
                           int num_layers, int layer_idx, int page_size, float rope_theta, int dtype, void* stream);

/* Bytes of the workspace of smlm_b200_batch_prefill: one dense copy of the batch's keys (rotated) and values,
 * total_pages * page_size * 2 * num_kv_heads * head_dim elements of the storage type.  Its contents need not
 * survive between calls. */
size_t smlm_b200_batch_prefill_workspace_bytes(int total_pages, int page_size, int num_kv_heads);

/* Causal self-attention of a ragged batch of prompts over their paged caches.  Request b owns the rows
 * qo_indptr[b] .. qo_indptr[b + 1] of q and o ([total_q, num_qo_heads, head_dim], 16-byte aligned); its cache
 * already holds all L_b >= n_b keys (init_kv ran before).  Query i of the request stands at position
 * L_b - n_b + i and attends to the keys 0 .. its own position:
 *   o[i, h] = softmax( rope(q[i, h], pos_i) . rope(K_b[0..pos_i, h / group])^T / sqrt(head_dim) ) . V_b[0..pos_i]
 * Replaces batch_prefill (kernel_src/csrc/loquetier_ops.cc:90-136; FlashInferBatchPrefillKernel,
 * kernel_src/csrc/flashinfer_adapter/flashinfer_all.cu:48-83; BatchPrefillWithPagedKVCacheKernel,
 * kernel_src/third_party/flashinfer/include/flashinfer/prefill.cuh:904-1060), without its copy of qo_indptr
 * to the host and its synchronisation.  Two launches: the pages are gathered once into the workspace (128-byte
 * aligned, sized by the function above; the reference asks for a 64 MiB `tmpbuf` instead) with the keys rotated
 * for their positions, then the attention kernel streams tiles of it with TMA.  A request with more queries
 * than keys sets bit 1 of the status word; its rows that see no key are zeros.  Status value 8: a bounded wait
 * inside the kernel gave up (the output is then not valid). */
int smlm_b200_batch_prefill(void* o, const void* q, const int32_t* qo_indptr, const void* const* kv_ptrs,
                            const int32_t* kv_indptr, const int32_t* last_page_offset, void* workspace,
                            size_t workspace_bytes, int* status_word, int batch_size, int total_q, int total_pages, int num_qo_heads, int num_kv_heads,
                            int head_dim, int num_layers, int layer_idx, int page_size, float rope_theta, int dtype,
                            void* stream);

/* Writes the key and value of ONE new token per request into the last valid entry of its cache
 * (the pages must already account for the token).  k, v: [batch, num_kv_heads, head_dim].  Replaces
 * append_kv (loquetier_ops.cc:230-273; AppendPagedKVCacheDecodeKernel, page.cuh:368-396), without its
 * stream synchronisation. */
int smlm_b200_append_kv(const void* const* kv_ptrs, const int32_t* kv_indptr, const int32_t* last_page_offset,
                        const void* k, const void* v, int* status_word, int batch_size, int total_pages,
                        int num_layers, int layer_idx, int num_kv_heads, int head_dim, int page_size, int dtype,
                        void* stream);

/* Writes a run of new tokens per request - tokens seqlen_indptr[b] .. seqlen_indptr[b + 1] of k and v,
 * [total_tokens, num_kv_heads, head_dim] - into the LAST entries of its cache, i.e. behind whatever the
 * cache held before.  Replaces init_kv (loquetier_ops.cc:182-228; AppendPagedKVCachePrefillKernel,
 * page.cuh:411-444), without its stream synchronisation. */
int smlm_b200_init_kv(const void* const* kv_ptrs, const int32_t* kv_indptr, const int32_t* last_page_offset,
                      const void* k, const void* v, const int32_t* seqlen_indptr, int* status_word, int batch_size,
                      int total_pages, int total_tokens, int num_layers, int layer_idx, int num_kv_heads, int head_dim,
                      int page_size, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SMLM_B200_KV_H_ */
