/*
 * Descriptor validation for the KVX C ABI -- CUDA-free C11, host only.
 *
 * The four exported functions never touch K/V bytes and ignore `stream`: they answer
 * "is this descriptor set well-formed?" with the same status, for the same input, as the
 * reference validators (reference: kvx_abi.c:313-466).  The order of the checks is part
 * of that contract, because the first failing check decides between INVALID_ARGUMENT and
 * UNSUPPORTED; each function below lists its order and the reference lines it mirrors.
 *
 * Structure: every layout is reduced to a "canonical geometry" (rank, extents and the
 * contiguous row-major strides of those extents), and one comparison routine checks a
 * tensor descriptor against it.  IO tensors reuse the same routine with a dense 3-D or
 * 4-D geometry.
 */
#include "kvx_abi.h"

#define KVX_FAIL_IF(cond, status) \
  do {                            \
    if (cond) return (status);    \
  } while (0)

/* Extents and dense row-major strides a tensor is expected to have. */
typedef struct kvx_geometry {
  uint32_t ndim;
  int64_t shape[KVX_MAX_TENSOR_DIMS];
  int64_t stride[KVX_MAX_TENSOR_DIMS];
} kvx_geometry_t;

static void kvx_geometry_dense(kvx_geometry_t *g, uint32_t ndim, const int64_t *shape) {
  int64_t run = 1;
  g->ndim = ndim;
  for (uint32_t i = 0; i < KVX_MAX_TENSOR_DIMS; ++i) {
    g->shape[i] = 0;
    g->stride[i] = 0;
  }
  for (uint32_t k = ndim; k-- > 0;) {
    g->shape[k] = shape[k];
    g->stride[k] = run;
    run *= shape[k];
  }
}

/* reference: kvx_abi.c:5-16 */
static int kvx_dtype_is_float(kvx_dtype_t t) {
  return t == KVX_DTYPE_F16 || t == KVX_DTYPE_BF16 || t == KVX_DTYPE_F32 ||
         t == KVX_DTYPE_F8_E4M3 || t == KVX_DTYPE_F8_E5M2;
}

/* reference: kvx_abi.c:18-20 */
static int kvx_dtype_is_index(kvx_dtype_t t) { return t == KVX_DTYPE_S32 || t == KVX_DTYPE_S64; }

/*
 * IO element type against cache element type.  The reference demands equality
 * (kvx_abi.c:377-380, :426-429).  ABI 1.2 adds one more legal pairing: an fp8-e4m3 cache
 * fed from / read into 16- or 32-bit float tensors (quantise-on-write, dequantise-on-
 * gather); K and V IO tensors must then share one type.
 */
static int kvx_io_dtypes_ok(const kvx_kv_io_desc_t *io, const kvx_cache_desc_t *c) {
  if (io->key.dtype == c->k.dtype && io->value.dtype == c->v.dtype) return 1;
  if (c->k.dtype == KVX_DTYPE_F8_E4M3 && c->v.dtype == KVX_DTYPE_F8_E4M3 &&
      io->key.dtype == io->value.dtype &&
      (io->key.dtype == KVX_DTYPE_F16 || io->key.dtype == KVX_DTYPE_BF16 ||
       io->key.dtype == KVX_DTYPE_F32))
    return 1;
  return 0;
}

static int kvx_shape_differs(const kvx_tensor_desc_t *t, const kvx_geometry_t *g) {
  for (uint32_t i = 0; i < g->ndim; ++i)
    if (t->shape[i] != g->shape[i]) return 1;
  return 0;
}

static int kvx_stride_differs(const kvx_tensor_desc_t *t, const kvx_geometry_t *g) {
  for (uint32_t i = 0; i < g->ndim; ++i)
    if (t->stride[i] != g->stride[i]) return 1;
  return 0;
}

/*
 * Dense IO tensor, rank 3 (write) or 4 (gather).  Order: NULL, size, float dtype, rank,
 * extents -> INVALID_ARGUMENT; strides -> UNSUPPORTED; NULL data of a non-empty tensor ->
 * INVALID_ARGUMENT.  reference: kvx_abi.c:26-55 (3-D), :57-88 (4-D).
 * `nonempty` is the reference's emptiness rule: num_tokens > 0 for 3-D,
 * seq_count > 0 && max_seq_len > 0 for 4-D (heads and dim are not consulted).
 */
static kvx_status_t kvx_check_io_tensor(const kvx_tensor_desc_t *t, const kvx_geometry_t *g,
                                        int nonempty) {
  KVX_FAIL_IF(t == NULL, KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(t->size < sizeof(kvx_tensor_desc_t), KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(!kvx_dtype_is_float(t->dtype), KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(t->ndim != g->ndim, KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(kvx_shape_differs(t, g), KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(kvx_stride_differs(t, g), KVX_STATUS_UNSUPPORTED);
  KVX_FAIL_IF(nonempty && t->data == NULL, KVX_STATUS_INVALID_ARGUMENT);
  return KVX_STATUS_OK;
}

/*
 * One page tensor of the cache.  Order: NULL, size, float dtype, NULL data, layout field,
 * rank in 1..5, then per layout: rank, (packed: pack > 0, head_dim % pack == 0), extents
 * -> INVALID_ARGUMENT; canonical strides -> UNSUPPORTED.  CUSTOM or unknown layouts are
 * UNSUPPORTED.  reference: kvx_abi.c:216-311.
 */
static kvx_status_t kvx_check_cache_tensor(const kvx_cache_desc_t *c, const kvx_tensor_desc_t *t,
                                           kvx_layout_t layout) {
  kvx_geometry_t g;
  int64_t dims[KVX_MAX_TENSOR_DIMS];

  KVX_FAIL_IF(t == NULL || c == NULL, KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(t->size < sizeof(kvx_tensor_desc_t), KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(!kvx_dtype_is_float(t->dtype), KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(t->data == NULL, KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(t->layout != layout, KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(t->ndim == 0 || t->ndim > KVX_MAX_TENSOR_DIMS, KVX_STATUS_INVALID_ARGUMENT);

  if (layout == KVX_LAYOUT_BLOCK_NHD || layout == KVX_LAYOUT_BLOCK_HND) {
    const int nhd = (layout == KVX_LAYOUT_BLOCK_NHD);
    KVX_FAIL_IF(t->ndim != 4, KVX_STATUS_INVALID_ARGUMENT);
    dims[0] = c->num_blocks;
    dims[1] = nhd ? c->block_size : c->num_kv_heads;
    dims[2] = nhd ? c->num_kv_heads : c->block_size;
    dims[3] = c->head_dim;
    kvx_geometry_dense(&g, 4, dims);
  } else if (layout == KVX_LAYOUT_BLOCK_HND_PACKED) {
    const int64_t pack = t->shape[4];
    KVX_FAIL_IF(t->ndim != 5, KVX_STATUS_INVALID_ARGUMENT);
    KVX_FAIL_IF(pack <= 0, KVX_STATUS_INVALID_ARGUMENT);
    KVX_FAIL_IF(((int64_t)c->head_dim % pack) != 0, KVX_STATUS_INVALID_ARGUMENT);
    dims[0] = c->num_blocks;
    dims[1] = c->num_kv_heads;
    dims[2] = (int64_t)c->head_dim / pack;
    dims[3] = c->block_size;
    dims[4] = pack;
    kvx_geometry_dense(&g, 5, dims);
  } else {
    return KVX_STATUS_UNSUPPORTED;
  }
  KVX_FAIL_IF(kvx_shape_differs(t, &g), KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(kvx_stride_differs(t, &g), KVX_STATUS_UNSUPPORTED);
  return KVX_STATUS_OK;
}

/* reference: kvx_abi.c:90-108 */
static kvx_status_t kvx_check_slots(const kvx_slot_mapping_t *s, uint32_t num_tokens) {
  KVX_FAIL_IF(s == NULL, KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(s->size < sizeof(kvx_slot_mapping_t), KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(!kvx_dtype_is_index(s->dtype), KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(s->token_count != num_tokens, KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(num_tokens > 0 && s->slots == NULL, KVX_STATUS_INVALID_ARGUMENT);
  return KVX_STATUS_OK;
}

/* reference: kvx_abi.c:196-214 */
static kvx_status_t kvx_check_seq_lens(const kvx_seq_lens_t *l, uint32_t seq_count) {
  KVX_FAIL_IF(l == NULL, KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(l->size < sizeof(kvx_seq_lens_t), KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(!kvx_dtype_is_index(l->dtype), KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(l->seq_count != seq_count, KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(seq_count > 0 && l->lengths == NULL, KVX_STATUS_INVALID_ARGUMENT);
  return KVX_STATUS_OK;
}

/*
 * Block table, every format.  All failures are INVALID_ARGUMENT.  The element-count
 * products are formed in 32 bits, as the reference does (kvx_abi.c:124,163).
 * reference: kvx_abi.c:110-194.
 */
static kvx_status_t kvx_check_block_table(const kvx_cache_desc_t *c, const kvx_block_table_t *b) {
  const kvx_status_t bad = KVX_STATUS_INVALID_ARGUMENT;
  KVX_FAIL_IF(b == NULL || c == NULL, bad);
  KVX_FAIL_IF(b->size < sizeof(kvx_block_table_t), bad);
  KVX_FAIL_IF(b->seq_count == 0 || b->max_blocks_per_seq == 0, bad);

  if (b->format == KVX_BLOCK_TABLE_PACKED) {
    const uint32_t want = b->seq_count * b->max_blocks_per_seq;
    KVX_FAIL_IF(!kvx_dtype_is_index(b->index_dtype), bad);
    KVX_FAIL_IF(b->beam_width != 1, bad);
    KVX_FAIL_IF(b->indices_count != want, bad);
    KVX_FAIL_IF(b->indptr != NULL || b->indptr_count != 0, bad);
    KVX_FAIL_IF(b->indices_count > 0 && b->indices == NULL, bad);
    return KVX_STATUS_OK;
  }
  if (b->format == KVX_BLOCK_TABLE_RAGGED) {
    KVX_FAIL_IF(!kvx_dtype_is_index(b->index_dtype) || !kvx_dtype_is_index(b->indptr_dtype), bad);
    KVX_FAIL_IF(b->beam_width != 1, bad);
    KVX_FAIL_IF(b->indptr == NULL, bad);
    KVX_FAIL_IF(b->indptr_count != b->seq_count + 1, bad);
    KVX_FAIL_IF(b->indices_count > 0 && b->indices == NULL, bad);
    return KVX_STATUS_OK;
  }
  if (b->format == KVX_BLOCK_TABLE_KV_OFFSETS) {
    const uint32_t want = b->seq_count * b->beam_width * 2u * b->max_blocks_per_seq;
    const uint32_t bs = c->block_size;
    KVX_FAIL_IF(b->index_dtype != KVX_DTYPE_S32, bad);
    KVX_FAIL_IF((b->flags & KVX_BLOCK_TABLE_FLAG_KVCACHEINDEX) == 0, bad);
    KVX_FAIL_IF(b->beam_width == 0, bad);
    KVX_FAIL_IF(bs == 0 || (bs & (bs - 1u)) != 0, bad); /* power-of-two pages only */
    KVX_FAIL_IF(b->indices_count != want, bad);
    KVX_FAIL_IF(b->indptr != NULL || b->indptr_count != 0, bad);
    KVX_FAIL_IF(b->indices_count > 0 && b->indices == NULL, bad);
    KVX_FAIL_IF(c->pool.bytes_per_block == 0 || c->pool.primary == NULL, bad);
    return KVX_STATUS_OK;
  }
  return bad;
}

KVX_API kvx_status_t kvx_get_version(kvx_version_t *out_version) {
  KVX_FAIL_IF(out_version == NULL, KVX_STATUS_INVALID_ARGUMENT);
  out_version->size = (uint32_t)sizeof(kvx_version_t);
  out_version->abi_major = KVX_ABI_VERSION_MAJOR;
  out_version->abi_minor = KVX_ABI_VERSION_MINOR;
  out_version->abi_patch = 0;
  return KVX_STATUS_OK;
}

KVX_API kvx_status_t kvx_validate_cache_desc(const kvx_cache_desc_t *cache) {
  kvx_status_t st;
  KVX_FAIL_IF(cache == NULL, KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(cache->size < sizeof(kvx_cache_desc_t), KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(cache->num_blocks == 0 || cache->block_size == 0 || cache->num_kv_heads == 0 ||
                  cache->head_dim == 0,
              KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(cache->k.layout != cache->v.layout, KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(cache->k.dtype != cache->v.dtype, KVX_STATUS_INVALID_ARGUMENT);
  st = kvx_check_cache_tensor(cache, &cache->k, cache->k.layout);
  KVX_FAIL_IF(st != KVX_STATUS_OK, st);
  return kvx_check_cache_tensor(cache, &cache->v, cache->v.layout);
}

/*
 * Order: NULLs; write/io/slots size guards; cache; io heads/dim non-zero and equal to the
 * cache's; io dtype == cache dtype; K tensor; V tensor; slot mapping.
 * reference: kvx_abi.c:354-398.
 */
KVX_API kvx_status_t kvx_write_kv(const kvx_cache_desc_t *cache, const kvx_write_desc_t *write,
                                  void *stream) {
  kvx_status_t st;
  kvx_geometry_t g;
  int64_t dims[3];
  (void)stream;
  KVX_FAIL_IF(cache == NULL || write == NULL, KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(write->size < sizeof(kvx_write_desc_t) ||
                  write->io.size < sizeof(kvx_kv_io_desc_t) ||
                  write->slots.size < sizeof(kvx_slot_mapping_t),
              KVX_STATUS_INVALID_ARGUMENT);
  st = kvx_validate_cache_desc(cache);
  KVX_FAIL_IF(st != KVX_STATUS_OK, st);
  KVX_FAIL_IF(write->io.num_kv_heads == 0 || write->io.head_dim == 0,
              KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(write->io.num_kv_heads != cache->num_kv_heads ||
                  write->io.head_dim != cache->head_dim,
              KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(!kvx_io_dtypes_ok(&write->io, cache), KVX_STATUS_INVALID_ARGUMENT);
  dims[0] = write->io.num_tokens;
  dims[1] = write->io.num_kv_heads;
  dims[2] = write->io.head_dim;
  kvx_geometry_dense(&g, 3, dims);
  st = kvx_check_io_tensor(&write->io.key, &g, write->io.num_tokens > 0);
  KVX_FAIL_IF(st != KVX_STATUS_OK, st);
  st = kvx_check_io_tensor(&write->io.value, &g, write->io.num_tokens > 0);
  KVX_FAIL_IF(st != KVX_STATUS_OK, st);
  return kvx_check_slots(&write->slots, write->io.num_tokens);
}

/*
 * Order: NULLs; gather/io/table/lens size guards; cache; io heads/dim/max_seq_len
 * non-zero; heads/dim equal to the cache's; io dtype == cache dtype; block table;
 * seq_lens; index dtype == lens dtype; io.num_tokens == seq_count * max_seq_len (32-bit
 * product); K out tensor; V out tensor; finally any format other than PACKED is
 * UNSUPPORTED.  reference: kvx_abi.c:400-466.
 */
KVX_API kvx_status_t kvx_gather_kv(const kvx_cache_desc_t *cache, const kvx_gather_desc_t *gather,
                                   void *stream) {
  kvx_status_t st;
  kvx_geometry_t g;
  int64_t dims[4];
  uint32_t seqs;
  (void)stream;
  KVX_FAIL_IF(cache == NULL || gather == NULL, KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(gather->size < sizeof(kvx_gather_desc_t) ||
                  gather->io.size < sizeof(kvx_kv_io_desc_t) ||
                  gather->block_table.size < sizeof(kvx_block_table_t) ||
                  gather->seq_lens.size < sizeof(kvx_seq_lens_t),
              KVX_STATUS_INVALID_ARGUMENT);
  st = kvx_validate_cache_desc(cache);
  KVX_FAIL_IF(st != KVX_STATUS_OK, st);
  KVX_FAIL_IF(gather->io.num_kv_heads == 0 || gather->io.head_dim == 0 ||
                  gather->max_seq_len == 0,
              KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(gather->io.num_kv_heads != cache->num_kv_heads ||
                  gather->io.head_dim != cache->head_dim,
              KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(!kvx_io_dtypes_ok(&gather->io, cache), KVX_STATUS_INVALID_ARGUMENT);
  st = kvx_check_block_table(cache, &gather->block_table);
  KVX_FAIL_IF(st != KVX_STATUS_OK, st);
  seqs = gather->block_table.seq_count;
  st = kvx_check_seq_lens(&gather->seq_lens, seqs);
  KVX_FAIL_IF(st != KVX_STATUS_OK, st);
  KVX_FAIL_IF(gather->block_table.index_dtype != gather->seq_lens.dtype,
              KVX_STATUS_INVALID_ARGUMENT);
  KVX_FAIL_IF(gather->io.num_tokens != seqs * gather->max_seq_len, KVX_STATUS_INVALID_ARGUMENT);
  dims[0] = seqs;
  dims[1] = gather->max_seq_len;
  dims[2] = gather->io.num_kv_heads;
  dims[3] = gather->io.head_dim;
  kvx_geometry_dense(&g, 4, dims);
  st = kvx_check_io_tensor(&gather->io.key, &g, seqs > 0 && gather->max_seq_len > 0);
  KVX_FAIL_IF(st != KVX_STATUS_OK, st);
  st = kvx_check_io_tensor(&gather->io.value, &g, seqs > 0 && gather->max_seq_len > 0);
  KVX_FAIL_IF(st != KVX_STATUS_OK, st);
  KVX_FAIL_IF(gather->block_table.format != KVX_BLOCK_TABLE_PACKED, KVX_STATUS_UNSUPPORTED);
  return KVX_STATUS_OK;
}
