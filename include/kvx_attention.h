/*
 * Decode attention that reads the paged cache in place: the consumer of the gather, fused with
 * it.  One query token per sequence attends over that sequence's cached tokens, found through
 * the block table exactly as kvx_launch_gather_kv finds them, so the contiguous K/V copy the
 * gather would write (and attention would read back) never exists.
 *
 * No reference counterpart: the reference stops at the gather (kernels/kvx_paged_kv.h:19-21)
 * and names this fusion as future work.  The cache side keeps the reference's descriptors
 * (kvx_abi.h:73-128: cache tensors with their layout and strides, PACKED block table, sequence
 * lengths) and the gather's conventions for bad data.
 *
 *   out[s][q][:] = sum_t softmax_t(scale * <query[s][q][:], K[s][t][kv(q)][:]>) * V[s][t][kv(q)][:]
 *
 * over the cached tokens t < min(seq_lens[s], max_seq_len) of sequence s that the table
 * resolves (a token whose logical block is >= max_blocks_per_seq, or whose page id is negative
 * or >= num_blocks, takes no part, as in the gather), with kv(q) = q / (num_q_heads /
 * num_kv_heads) (grouped-query attention; num_q_heads a multiple of num_kv_heads).  A sequence
 * with no token that takes part gets out = 0.  Scores, softmax and the weighted sum are
 * accumulated in f32; the result is rounded once to the query's type.
 */
#ifndef KVX_ATTENTION_H
#define KVX_ATTENTION_H

#include "kvx_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct kvx_attention_desc {
  uint32_t size;
  uint32_t num_q_heads;   /* a multiple of cache->num_kv_heads */
  uint32_t max_seq_len;   /* tokens beyond it are ignored; bounds the work split */
  float scale;            /* multiplies the scores before the softmax, e.g. 1/sqrt(head_dim) */
  kvx_tensor_desc_t query; /* [seq_count, num_q_heads, head_dim], F16 / BF16 / F32, dense */
  kvx_tensor_desc_t out;   /* same shape and type as query, dense */
  kvx_block_table_t block_table; /* PACKED */
  kvx_seq_lens_t seq_lens;       /* same index type as the table */
} kvx_attention_desc_t;

#if defined(__cplusplus)
static_assert(sizeof(kvx_attention_desc_t) == 328, "kvx_attention_desc_t layout");
#elif defined(__STDC_VERSION__) && __STDC_VERSION__ >= 201112L
_Static_assert(sizeof(kvx_attention_desc_t) == 328, "kvx_attention_desc_t layout");
#endif

/* Bytes of caller-owned DEVICE scratch kvx_launch_paged_attention_decode needs for this
 * problem size: a work counter and, when contexts are split in chunks, the chunks' partial
 * results.  The library allocates nothing itself; the scratch needs no initialisation and may
 * be reused by the next call on the same stream. */
KVX_API size_t kvx_paged_attention_workspace_bytes(uint32_t seq_count, uint32_t num_q_heads,
                                                   uint32_t num_kv_heads, uint32_t head_dim,
                                                   uint32_t max_seq_len);

/* Enqueues the attention on `stream` (1 to 3 kernels) and returns without synchronising.
 *
 * Cache: F16 / BF16 / F32 (query and out of the same type), or F8_E4M3 with 16/32-bit query
 * and F32 scales in k_scale / v_scale (PER_TENSOR or PER_HEAD, as for the fp8 gather; NULL
 * otherwise): K and V are dequantised on the fly as value * scale.
 *
 * Status: INVALID_ARGUMENT for NULL / undersized descriptors, shapes that disagree, a query
 * head count that is not a multiple of the KV heads, scratch smaller than
 * kvx_paged_attention_workspace_bytes() or misaligned (16 bytes); UNSUPPORTED for a table that
 * is not PACKED, mismatched types and non-dense query / out; OK without a launch when there is
 * no sequence.  Bad DATA is skipped as described above. */
KVX_API kvx_status_t kvx_launch_paged_attention_decode(const kvx_cache_desc_t *cache,
                                                       const kvx_attention_desc_t *attn,
                                                       const kvx_scale_desc_t *k_scale,
                                                       const kvx_scale_desc_t *v_scale,
                                                       void *workspace, size_t workspace_bytes,
                                                       void *stream);

#ifdef __cplusplus
}
#endif
#endif /* KVX_ATTENTION_H */
