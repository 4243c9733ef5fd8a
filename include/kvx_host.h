/*
 * Host-buffer front end of the paged KV write / gather: K/V batches, slot mappings, block
 * tables and gathered outputs live in HOST memory (ideally page-locked), the page pools
 * live on the device.  A pipe owns the device staging buffers, streams and events needed
 * to overlap host<->device copies with the kernels; nothing is allocated per call.
 *
 * The reference's kvx_write_kv / kvx_gather_kv (kvx_abi.h:194-199, kvx_abi.c:354-466)
 * accept descriptors whose buffers are KVX_MEMORY_HOST -- its ABI test calls them on stack
 * arrays (tests/kvx_abi_test.c:257-261, :284-295) -- but only validate them.  These entry
 * points take the same descriptors and move the data.
 */
#ifndef KVX_HOST_H
#define KVX_HOST_H

#include "kvx_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct kvx_host_pipe kvx_host_pipe_t;

/* Creates a pipe on the current device.  `chunk_bytes` bounds one staged K (or V) chunk;
 * two rings of three chunk sets are allocated, one for writes and one for gathers (about
 * 12 * chunk_bytes of device memory plus slots).
 * `max_seqs * max_blocks_per_seq` bounds the block tables it can stage.
 * OUT_OF_RANGE when device memory cannot be had. */
KVX_API kvx_status_t kvx_host_pipe_create(size_t chunk_bytes, uint32_t max_seqs,
                                          uint32_t max_blocks_per_seq, kvx_host_pipe_t **out_pipe);

KVX_API void kvx_host_pipe_destroy(kvx_host_pipe_t *pipe);

/* write->io.key/value.data and write->slots.slots are HOST pointers; cache->k/v.data are
 * DEVICE pointers.  Tokens are staged chunk by chunk (host->device copy of chunk i+1
 * overlaps the kernel of chunk i).  Asynchronous: returns once everything is enqueued; the
 * host buffers must stay valid until kvx_host_pipe_sync.  Semantics and status codes are
 * those of kvx_launch_write_kv, including key / value whose token rows are further apart than
 * num_kv_heads * head_dim elements (stride[0] larger than dense; the rows are then copied with a
 * pitched copy and staged densely); elements inside a token row must be dense (UNSUPPORTED
 * otherwise), and K and V must have one dtype. */
KVX_API kvx_status_t kvx_host_write_kv(kvx_host_pipe_t *pipe, const kvx_cache_desc_t *cache,
                                       const kvx_write_desc_t *write);

/* gather->io.key/value.data, block_table.indices and seq_lens.lengths are HOST pointers.
 * Sequences are gathered into device staging a group at a time and only the bytes the
 * gather defines (positions below the sequence length whose page id is valid) are copied
 * back, so every other byte of the host outputs stays untouched, as with
 * kvx_launch_gather_kv.  Ordered after earlier kvx_host_write_kv calls on the same pipe.
 * Where the value output lies behind the key output at a distance of less than 2 GB (one
 * allocation for both: out[2][seq_count][max_seq_len][heads][dim], say), a sequence's K run
 * and V run return as the two rows of one 2-D copy, which costs one copy's set-up instead of
 * two (measured: 8 % more end-to-end rate with runs of 4-5 MB).
 * k_scale / v_scale (host descriptors with DEVICE data) are needed for an fp8 cache only. */
KVX_API kvx_status_t kvx_host_gather_kv(kvx_host_pipe_t *pipe, const kvx_cache_desc_t *cache,
                                        const kvx_gather_desc_t *gather,
                                        const kvx_scale_desc_t *k_scale,
                                        const kvx_scale_desc_t *v_scale);

/* Blocks until every copy and kernel enqueued through the pipe has finished.
 * INTERNAL_ERROR if any of them failed, or if a gather kernel abandoned a bounded wait
 * (kvx_b200_device_error in kvx_paged_kv.h; the word is cleared). */
KVX_API kvx_status_t kvx_host_pipe_sync(kvx_host_pipe_t *pipe);

/* Bytes moved host->device and device->host through the pipe since creation. */
KVX_API void kvx_host_pipe_traffic(const kvx_host_pipe_t *pipe, uint64_t *h2d_bytes,
                                   uint64_t *d2h_bytes);

#ifdef __cplusplus
}
#endif
#endif /* KVX_HOST_H */
