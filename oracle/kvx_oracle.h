/*
 * CPU ORACLE -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.  See kvx_oracle.c.
 * Every pointer inside the descriptors addresses HOST memory.
 */
#ifndef KVX_ORACLE_H
#define KVX_ORACLE_H

#include "kvx_abi.h"
#include "kvx_attention.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Element-by-element write; fp8-e4m3 cache + 16/32-bit IO quantises with the write
 * descriptor's scales. */
kvx_status_t kvx_oracle_write_kv(const kvx_cache_desc_t *cache, const kvx_write_desc_t *write);

/* Element-by-element gather; k_scale / v_scale are consulted only for an fp8-e4m3 cache. */
kvx_status_t kvx_oracle_gather_kv(const kvx_cache_desc_t *cache, const kvx_gather_desc_t *gather,
                                  const kvx_scale_desc_t *k_scale, const kvx_scale_desc_t *v_scale);

/* The same gather into un-padded [rows, heads, dim] outputs: token tok of sequence s goes to
 * row out_indptr[s] + tok while below out_indptr[s + 1] and below rows = io.num_tokens.
 * out_indptr == NULL is the padded form. */
kvx_status_t kvx_oracle_gather_kv_varlen(const kvx_cache_desc_t *cache, const kvx_gather_desc_t *gather,
                                         const void *out_indptr, kvx_dtype_t out_indptr_dtype,
                                         const kvx_scale_desc_t *k_scale, const kvx_scale_desc_t *v_scale);

/* Decode attention over the paged cache in double precision (include/kvx_attention.h). */
kvx_status_t kvx_oracle_paged_attention_decode(const kvx_cache_desc_t *cache, const kvx_attention_desc_t *attn,
                                               const kvx_scale_desc_t *k_scale, const kvx_scale_desc_t *v_scale);

/* scale = absmax / 448 per head or per tensor; outputs are host float arrays. */
kvx_status_t kvx_oracle_kv_scales(const kvx_kv_io_desc_t *io, kvx_scale_granularity_t granularity,
                                  float *k_scale_out, float *v_scale_out);

uint8_t kvx_oracle_e4m3_from_f32(float y);
float kvx_oracle_e4m3_to_f32(uint8_t q);

/* Threaded row/page-chunk memcpy form of the same write and gather, used only to time a
 * CPU baseline; NHD canonical pages, equal IO and cache dtype.  Returns UNSUPPORTED
 * otherwise.  Defined in kvx_cpu_baseline.c and checked against the functions above. */
kvx_status_t kvx_cpu_baseline_write_kv(const kvx_cache_desc_t *cache, const kvx_write_desc_t *write,
                                       int threads);
kvx_status_t kvx_cpu_baseline_gather_kv(const kvx_cache_desc_t *cache,
                                        const kvx_gather_desc_t *gather, int threads);

#ifdef __cplusplus
}
#endif
#endif
