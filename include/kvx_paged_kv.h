/*
 * Launch layer of the paged KV-cache hot path: the entry points that move K/V bytes on
 * the GPU.  Same names and signatures as the reference launch header
 * (reference: kernels/kvx_paged_kv.h:11-57), implemented by hand-written sm_100a kernels.
 *
 * Every launcher:
 *   - takes host-resident descriptors whose data / slots / indices / lengths / scale
 *     pointers address memory of the CURRENT device;
 *   - enqueues its kernel on `stream` (an opaque cudaStream_t; NULL = the legacy default
 *     stream) and returns without synchronising;
 *   - allocates nothing and keeps no pointer after returning;
 *   - returns KVX_STATUS_OK without launching when there is nothing to move;
 *   - reports a failed launch as KVX_STATUS_INTERNAL_ERROR;
 *   - treats bad DATA as "skip": a token whose slot is negative or addresses a block
 *     >= num_blocks is not written; a sequence position >= seq_lens[s], a logical block
 *     >= max_blocks_per_seq, or a block id that is negative (or >= num_blocks) is not
 *     gathered and the corresponding output bytes stay untouched.
 *
 * Descriptor checks and their status codes follow the reference launchers in evaluation
 * order (reference: kernels/kvx_paged_kv.cu:315-376, :493-559, :763-829).
 */
#ifndef KVX_PAGED_KV_H
#define KVX_PAGED_KV_H

#include "kvx_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ write ------------
 * cache[slot / block_size][slot % block_size][h][d] = key[t][h][d] (and value), for every
 * token t with a valid slot, honouring the cache tensors' own strides and layout
 * (NHD, HND, HND_PACKED).  Bits are copied unchanged.
 *
 * kvx_launch_write_kv dispatches on cache->k.dtype: F16 / BF16 / F32 need IO tensors of
 * the same type; F8_E4M3 (ABI 1.2) quantises 16/32-bit IO on the fly, see below.
 *
 * key / value are [num_tokens, heads, dim] with dense heads and dims (stride[2] = 1,
 * stride[1] = dim).  Their token stride may exceed heads * dim -- slices of a fused projection
 * output are written as they are; the reference's launchers answer UNSUPPORTED for anything
 * but stride[0] = heads * dim (kernels/kvx_paged_kv.cu:269-313), which still applies to the
 * validate-only kvx_write_kv and to a token stride below heads * dim.
 * reference: kernels/kvx_paged_kv.h:11-13, kernels/kvx_paged_kv.cu:472-491 */
KVX_API kvx_status_t kvx_launch_write_kv(const kvx_cache_desc_t *cache,
                                         const kvx_write_desc_t *write, void *stream);

/* Same result as kvx_launch_write_kv.  `tokens_per_seq` must be > 0 and divide
 * io.num_tokens; it is validated, never used for scheduling.
 * reference: kernels/kvx_paged_kv.h:15-17, kernels/kvx_paged_kv.cu:739-761 */
KVX_API kvx_status_t kvx_launch_write_kv_prefill(const kvx_cache_desc_t *cache,
                                                 const kvx_write_desc_t *write,
                                                 int32_t tokens_per_seq, void *stream);

/* Type-pinned variants: UNSUPPORTED unless cache AND io tensors have exactly this dtype.
 * reference: kernels/kvx_paged_kv.h:23-45, kernels/kvx_paged_kv.cu:453-470, :718-737 */
KVX_API kvx_status_t kvx_launch_write_kv_f32(const kvx_cache_desc_t *cache,
                                             const kvx_write_desc_t *write, void *stream);
KVX_API kvx_status_t kvx_launch_write_kv_f16(const kvx_cache_desc_t *cache,
                                             const kvx_write_desc_t *write, void *stream);
KVX_API kvx_status_t kvx_launch_write_kv_bf16(const kvx_cache_desc_t *cache,
                                              const kvx_write_desc_t *write, void *stream);
KVX_API kvx_status_t kvx_launch_write_kv_prefill_f32(const kvx_cache_desc_t *cache,
                                                     const kvx_write_desc_t *write,
                                                     int32_t tokens_per_seq, void *stream);
KVX_API kvx_status_t kvx_launch_write_kv_prefill_f16(const kvx_cache_desc_t *cache,
                                                     const kvx_write_desc_t *write,
                                                     int32_t tokens_per_seq, void *stream);
KVX_API kvx_status_t kvx_launch_write_kv_prefill_bf16(const kvx_cache_desc_t *cache,
                                                      const kvx_write_desc_t *write,
                                                      int32_t tokens_per_seq, void *stream);

/* ------------------------------------------------------------------ gather -----------
 * out[s][tok][h][d] = cache[table[s][tok / block_size]][tok % block_size][h][d] for
 * tok < seq_lens[s]; table and seq_lens share one index type.
 * reference: kernels/kvx_paged_kv.h:19-21, kernels/kvx_paged_kv.cu:891-910
 *
 * Block-table formats: PACKED as in the reference.  RAGGED (ABI 1.2; the reference validates
 * it, kvx_abi.c:142-160, but its launcher answers UNSUPPORTED, kernels/kvx_paged_kv.cu:788-790)
 * follows KVX_SPEC.md:108-114: `indices` holds ONE PAGE ID PER CACHED TOKEN, `indptr`
 * (seq_count + 1 entries, S32 or S64) the prefix sums of the per-sequence token counts; token
 * tok of sequence s lives in page indices[indptr[s] + tok] at offset tok % block_size, and
 * the gather stops at min(seq_lens[s], indptr[s + 1] - indptr[s], max_seq_len).  Outputs keep
 * the padded [seq_count, max_seq_len, heads, dim] form.
 *
 * KV_OFFSETS (ABI 1.2; validated by the reference, kvx_abi.c:161-189, never executed) follows
 * KVX_SPEC.md:116-122 and KV_CACHE_LAYOUTS.md:89-96: `indices` is an S32 table
 * [seq_count, beam_width, 2, max_blocks_per_seq] of pool offsets, [s][0][0][lb] naming the K
 * page and [s][0][1][lb] the V page of logical block lb.  Bit 31 of an entry selects
 * cache->pool.secondary, otherwise cache->pool.primary; the low 31 bits count blocks:
 *     page = pool + offset * cache->pool.bytes_per_block.
 * Inside a page cache->k / cache->v give layout, dtype and the strides of the token, head and
 * dim axes; their data pointers and block strides are not used.  Skipped without error: an
 * entry for the secondary pool when there is none, and an offset that is not below
 * cache->num_blocks (which therefore counts the blocks of one pool).  The validate-only
 * rules apply (S32, KVCACHEINDEX flag, power-of-two block_size, indices_count, no indptr,
 * pool with bytes_per_block and primary); beam_width must be 1 (UNSUPPORTED otherwise: the
 * output has one row per sequence). */
KVX_API kvx_status_t kvx_launch_gather_kv(const kvx_cache_desc_t *cache,
                                          const kvx_gather_desc_t *gather, void *stream);

/* reference: kernels/kvx_paged_kv.h:47-57, kernels/kvx_paged_kv.cu:872-889 */
KVX_API kvx_status_t kvx_launch_gather_kv_f32(const kvx_cache_desc_t *cache,
                                              const kvx_gather_desc_t *gather, void *stream);
KVX_API kvx_status_t kvx_launch_gather_kv_f16(const kvx_cache_desc_t *cache,
                                              const kvx_gather_desc_t *gather, void *stream);
KVX_API kvx_status_t kvx_launch_gather_kv_bf16(const kvx_cache_desc_t *cache,
                                               const kvx_gather_desc_t *gather, void *stream);

/* ------------------------------------------------------------------ fp8-e4m3 ---------
 * The reference declares the fp8 dtype and the scale descriptors (kvx_abi.h:47,154-180)
 * but its launchers answer UNSUPPORTED for them (kernels/kvx_paged_kv.cu:488,907); the
 * entry points below have no data-moving counterpart there.
 *
 * Cache tensors are KVX_DTYPE_F8_E4M3 (1 byte per element, any of the three layouts); IO
 * tensors are F16, BF16 or F32 (K and V alike).
 *   write : q = e4m3_rn_satfinite((float)x / scale)      one IEEE f32 division, one
 *           rounding to E4M3 (ties to even), |y| > 448 and +-inf -> +-448, NaN -> 0x7F.
 *   gather: out = io_type_rn((float)e4m3(q) * scale)     one f32 multiply, then round to
 *           the IO type (ties to even); NaN comes out as the canonical quiet NaN.
 * Scale selection, separately for K and V:
 *   *_scale_desc.data != NULL : dtype F32, granularity PER_TENSOR (one value) or PER_HEAD
 *                               (ndim 1, shape[0] = num_kv_heads, stride[0] in elements);
 *   otherwise                 : the device scalar k_scale / v_scale (per tensor);
 *   neither                   : KVX_STATUS_UNSUPPORTED.
 * kvx_launch_write_kv / kvx_launch_gather_kv route here when cache->k.dtype is F8_E4M3.
 * A gather descriptor has no scale fields, so the dequantising gather takes them as
 * arguments. */
KVX_API kvx_status_t kvx_launch_write_kv_f8e4m3(const kvx_cache_desc_t *cache,
                                                const kvx_write_desc_t *write, void *stream);

KVX_API kvx_status_t kvx_launch_gather_kv_f8e4m3(const kvx_cache_desc_t *cache,
                                                 const kvx_gather_desc_t *gather,
                                                 const kvx_scale_desc_t *k_scale,
                                                 const kvx_scale_desc_t *v_scale, void *stream);

/* Un-padded gather (no reference counterpart; the reference's gather only writes the padded
 * [seq_count, max_seq_len, heads, dim] rectangle).  gather->io.key / value are dense 3-D
 * [rows, heads, dim] tensors with rows = gather->io.num_tokens; `out_indptr` is a DEVICE array
 * of seq_count + 1 row numbers (S32 or S64, `out_indptr_dtype`), normally the prefix sums of
 * the sequence lengths.  Token tok of sequence s is written to row out_indptr[s] + tok for
 *     tok < min(seq_lens[s], max_seq_len, out_indptr[s + 1] - out_indptr[s]),
 * and never at or beyond `rows`; a sequence with a negative out_indptr is skipped.  All block
 * table formats and the fp8 cache are accepted; k_scale / v_scale are read only for an fp8
 * cache (NULL otherwise).  Every other check and status is that of kvx_launch_gather_kv. */
KVX_API kvx_status_t kvx_launch_gather_kv_varlen(const kvx_cache_desc_t *cache,
                                                 const kvx_gather_desc_t *gather, const void *out_indptr,
                                                 kvx_dtype_t out_indptr_dtype,
                                                 const kvx_scale_desc_t *k_scale,
                                                 const kvx_scale_desc_t *v_scale, void *stream);

/* Per-head (or per-tensor) scales of one write batch: scale = absmax / 448, absmax taken
 * over every token and dim of the head (PER_HEAD) or of the tensor (PER_TENSOR), K and V
 * separately; an absmax of zero (or NaN) yields 1.0f.  Outputs are F32 device arrays of
 * num_kv_heads (PER_HEAD) or 1 (PER_TENSOR) elements.
 * `workspace` is device scratch of at least kvx_kv_scales_workspace_bytes(num_kv_heads)
 * bytes, 256-byte aligned, that MUST be zero before the first call; each call leaves it
 * zeroed again.  Calls sharing one workspace must not overlap on the GPU.
 * No counterpart in the reference. */
KVX_API size_t kvx_kv_scales_workspace_bytes(uint32_t num_kv_heads);

KVX_API kvx_status_t kvx_launch_kv_scales(const kvx_kv_io_desc_t *io,
                                          kvx_scale_granularity_t granularity, float *k_scale_out,
                                          float *v_scale_out, void *workspace,
                                          size_t workspace_bytes, void *stream);

/* The same reduction for callers that cannot hand over device scratch.  Serving engines that
 * give every free byte of HBM to their page pool at start-up, or that forbid driver
 * allocations on the request path because cudaMalloc / cudaFree synchronise the whole device,
 * have nowhere to take a workspace from; for them the scratch lives inside the library, in a
 * fixed device array sized for KVX_KV_SCALES_STATIC_MAX_HEADS heads (8 448 bytes held by every
 * GPU that loads the library, until the process exits).
 *   - io->num_kv_heads above the maximum returns KVX_STATUS_OUT_OF_RANGE and does nothing.
 *   - No allocation of any kind happens here, on the device or through a library.
 *   - The first call on each device looks up the array's device address (one runtime query,
 *     cached per device); make that first call before any stream capture starts.
 *   - All calls on one device share the one array.  It is cleared on `stream` before every
 *     reduction, so calls issued one after the other are independent, but two calls whose
 *     kernels overlap on the GPU (different streams, no ordering) race on it and produce
 *     wrong scales: order them.
 * Results are identical to kvx_launch_kv_scales.  No counterpart in the reference. */
#define KVX_KV_SCALES_STATIC_MAX_HEADS 1024

KVX_API kvx_status_t kvx_launch_kv_scales_static(const kvx_kv_io_desc_t *io,
                                                 kvx_scale_granularity_t granularity,
                                                 float *k_scale_out, float *v_scale_out, void *stream);

/* ------------------------------------------------------------------ introspection ----
 * Number of kernels this library has launched in this process since load (or since the
 * last reset).  Lets a benchmark state how many of its timed launches were these kernels.
 * No counterpart in the reference. */
KVX_API uint64_t kvx_b200_launch_count(void);
KVX_API void kvx_b200_reset_launch_count(void);

/* Device-side give-up word.  The only kernels of this library that wait on anything are those
 * of the bulk-async gather path ("gather_path" = 1, off by default): a wait on a staged copy is
 * abandoned after one second ("bulk_wait_us"), the waiting thread sets a word in device memory,
 * lets its copies in flight finish and returns; rows it had not reached stay unwritten, and the
 * launcher has long since returned KVX_STATUS_OK.  This call returns that word for the current
 * device (0 = no wait ever gave up, 1 = one did, -1 = the word could not be read) and, when
 * `reset` is non-zero, clears it.  It copies from the device synchronously: call it after the
 * streams in question have been synchronised.  kvx_host_pipe_sync consults it for its own
 * launches.  No counterpart in the reference. */
KVX_API int kvx_b200_device_error(int reset);

/* Tuning knobs for experiments: name = "write_vecs_per_cta", "gather_path" (0 = registers,
 * 1 = bulk-async staging), ...; returns 0 when the name is known.  Defaults are the
 * measured-best values; production callers never need this.  Each knob is an atomic word: it
 * may be set from any host thread at any time, and a launch that is being prepared meanwhile
 * uses the old or the new value.  No counterpart in the reference. */
KVX_API int kvx_b200_set_option(const char *name, int64_t value);
KVX_API int64_t kvx_b200_get_option(const char *name);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* KVX_PAGED_KV_H */
