/*
 * KVX C ABI, version 1.2 -- descriptors, enumerations and the four validate-only entry
 * points of the paged KV-cache interface.
 *
 * This header is the drop-in boundary.  Every public name, enumerator value, field order
 * and field type is the one published by the KVX project (reference: kvx_abi.h:11-199), so
 * code written against that header (its vLLM patch, its TGI / TensorRT-LLM adapter stubs,
 * its own tests) compiles against this one without edits and produces structs with the
 * same bytes (x86-64 sizes are frozen by the static assertions at the end of this file).
 *
 * What differs from the reference header:
 *   - KVX_ABI_VERSION_MINOR is 2: the launch layer additionally accepts an fp8-e4m3 cache
 *     with 16/32-bit IO tensors when a scale is supplied (see kvx_paged_kv.h).  Nothing
 *     was removed, so a consumer built for 1.1 keeps working (same major).
 *   - the declarations are documented.
 *
 * Conventions shared by every struct:
 *   - the first field is `size`; the caller stores sizeof(struct) there and a callee
 *     accepts any value >= its own sizeof (reference: KVX_SPEC.md:29-34).
 *   - strides are counted in elements, never bytes (reference: KVX_SPEC.md:47-49).
 *   - descriptors live in host memory; `data`, `slots`, `indices`, `lengths` and scale
 *     `data` point at device memory when handed to the launch layer.
 *   - the callee keeps no pointer after it returns.
 */
#ifndef KVX_ABI_H
#define KVX_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KVX_ABI_VERSION_MAJOR 1
#define KVX_ABI_VERSION_MINOR 2

/* Symbol export decoration (reference: kvx_abi.h:14-24). */
#if defined(_WIN32) && defined(KVX_BUILD_DLL)
#define KVX_API __declspec(dllexport)
#elif defined(_WIN32) && defined(KVX_USE_DLL)
#define KVX_API __declspec(dllimport)
#else
#define KVX_API
#endif

/* Largest tensor rank a descriptor can carry (HND_PACKED uses all five). */
enum { KVX_MAX_TENSOR_DIMS = 5 };

/* ---------------------------------------------------------------- enumerations ------- */

/* Result of every entry point (reference: kvx_abi.h:26-33).  Bad *data* -- a negative or
 * out-of-range slot, a negative block id, a short sequence -- is never an error: such
 * entries are skipped and the call still reports OK. */
typedef enum kvx_status {
  KVX_STATUS_OK = 0,
  KVX_STATUS_INVALID_ARGUMENT = 1, /* malformed descriptor */
  KVX_STATUS_UNSUPPORTED = 2,      /* well-formed, but not implemented here */
  KVX_STATUS_OUT_OF_RANGE = 3,
  KVX_STATUS_INCOMPATIBLE = 4, /* ABI major mismatch */
  KVX_STATUS_INTERNAL_ERROR = 5 /* the CUDA launch itself failed */
} kvx_status_t;

/* Element types (reference: kvx_abi.h:42-54).  F16/BF16/F32/F8_* are "float" types for
 * cache and IO tensors; S32/S64 are the only legal index types. */
typedef enum kvx_dtype {
  KVX_DTYPE_INVALID = 0,
  KVX_DTYPE_F16 = 1,
  KVX_DTYPE_BF16 = 2,
  KVX_DTYPE_F32 = 3,
  KVX_DTYPE_F8_E4M3 = 4,
  KVX_DTYPE_F8_E5M2 = 5,
  KVX_DTYPE_S32 = 6,
  KVX_DTYPE_S64 = 7,
  KVX_DTYPE_U32 = 8,
  KVX_DTYPE_U64 = 9,
  KVX_DTYPE_U8 = 10
} kvx_dtype_t;

/* Where a buffer lives (reference: kvx_abi.h:56-61).  Informational for the launch layer. */
typedef enum kvx_memory_type {
  KVX_MEMORY_UNKNOWN = 0,
  KVX_MEMORY_HOST = 1,
  KVX_MEMORY_DEVICE = 2,
  KVX_MEMORY_UNIFIED = 3
} kvx_memory_type_t;

/* Page layouts (reference: kvx_abi.h:63-69, KVX_SPEC.md:51-58).
 *   NHD         [num_blocks, block_size, num_kv_heads, head_dim]
 *   HND         [num_blocks, num_kv_heads, block_size, head_dim]
 *   HND_PACKED  [num_blocks, num_kv_heads, head_dim/pack, block_size, pack], pack = shape[4]
 */
typedef enum kvx_layout {
  KVX_LAYOUT_INVALID = 0,
  KVX_LAYOUT_BLOCK_NHD = 1,
  KVX_LAYOUT_BLOCK_HND = 2,
  KVX_LAYOUT_BLOCK_HND_PACKED = 3,
  KVX_LAYOUT_BLOCK_CUSTOM = 15
} kvx_layout_t;

/* Block-table encodings (reference: kvx_abi.h:103-108).  Only PACKED,
 * a dense [seq_count, max_blocks_per_seq] matrix, is executed by the launch layer. */
typedef enum kvx_block_table_format {
  KVX_BLOCK_TABLE_INVALID = 0,
  KVX_BLOCK_TABLE_PACKED = 1,
  KVX_BLOCK_TABLE_RAGGED = 2,
  KVX_BLOCK_TABLE_KV_OFFSETS = 3
} kvx_block_table_format_t;

typedef enum kvx_block_table_flags {
  KVX_BLOCK_TABLE_FLAG_NONE = 0,
  KVX_BLOCK_TABLE_FLAG_KVCACHEINDEX = 1 << 0
} kvx_block_table_flags_t;

/* How many scale values accompany a quantised cache (reference: kvx_abi.h:154-160). */
typedef enum kvx_scale_granularity {
  KVX_SCALE_NONE = 0,
  KVX_SCALE_PER_TENSOR = 1,
  KVX_SCALE_PER_BLOCK = 2,
  KVX_SCALE_PER_HEAD = 3,
  KVX_SCALE_PER_BLOCK_HEAD = 4
} kvx_scale_granularity_t;

/* ---------------------------------------------------------------- descriptors -------- */

/* Filled by kvx_get_version (reference: kvx_abi.h:35-40). */
typedef struct kvx_version {
  uint32_t size;
  uint32_t abi_major;
  uint32_t abi_minor;
  uint32_t abi_patch;
} kvx_version_t;

/* One strided tensor: a K or V page pool, or a dense IO tensor
 * (reference: kvx_abi.h:73-82). */
typedef struct kvx_tensor_desc {
  uint32_t size;
  kvx_dtype_t dtype;
  kvx_layout_t layout; /* meaningful for cache tensors; ignored for IO tensors */
  kvx_memory_type_t memory;
  uint32_t ndim;
  int64_t shape[KVX_MAX_TENSOR_DIMS];
  int64_t stride[KVX_MAX_TENSOR_DIMS]; /* elements */
  void *data;
} kvx_tensor_desc_t;

/* Raw block pools for offset-style tables (reference: kvx_abi.h:84-90).  Carried and
 * validated, not consumed by the kernels. */
typedef struct kvx_pool_desc {
  uint32_t size;
  kvx_memory_type_t memory;
  uint32_t bytes_per_block;
  void *primary;
  void *secondary;
} kvx_pool_desc_t;

/* The paged cache of one layer: geometry plus its K and V page tensors
 * (reference: kvx_abi.h:92-101). */
typedef struct kvx_cache_desc {
  uint32_t size;
  uint32_t num_blocks;
  uint32_t block_size; /* tokens per page */
  uint32_t num_kv_heads;
  uint32_t head_dim;
  kvx_tensor_desc_t k;
  kvx_tensor_desc_t v;
  kvx_pool_desc_t pool;
} kvx_cache_desc_t;

/* Logical-to-physical page map of a batch of sequences (reference: kvx_abi.h:115-128).
 * PACKED: indices[seq * max_blocks_per_seq + logical_block]; a negative id = no page. */
typedef struct kvx_block_table {
  uint32_t size;
  kvx_block_table_format_t format;
  kvx_dtype_t index_dtype;
  kvx_dtype_t indptr_dtype;
  uint32_t seq_count;
  uint32_t beam_width;
  uint32_t max_blocks_per_seq;
  const void *indices;
  const void *indptr;
  uint32_t indices_count;
  uint32_t indptr_count;
  uint32_t flags; /* kvx_block_table_flags_t bits */
} kvx_block_table_t;

/* Destination slot of every token of a write batch, slot = block * block_size + offset
 * (reference: kvx_abi.h:130-136).  A negative slot marks padding and is skipped;
 * `invalid_slot` documents the caller's marker, the kernels test `slot < 0`. */
typedef struct kvx_slot_mapping {
  uint32_t size;
  kvx_dtype_t dtype; /* S32 or S64 */
  uint32_t token_count;
  int64_t invalid_slot;
  const void *slots;
} kvx_slot_mapping_t;

/* Valid token count of every sequence of a gather (reference: kvx_abi.h:138-143). */
typedef struct kvx_seq_lens {
  uint32_t size;
  kvx_dtype_t dtype; /* must equal the block table's index_dtype */
  uint32_t seq_count;
  const void *lengths;
} kvx_seq_lens_t;

/* The dense K and V tensors moved in or out (reference: kvx_abi.h:145-152):
 * write  [num_tokens, num_kv_heads, head_dim];
 * gather [seq_count, max_seq_len, num_kv_heads, head_dim], num_tokens = their product. */
typedef struct kvx_kv_io_desc {
  uint32_t size;
  kvx_tensor_desc_t key;
  kvx_tensor_desc_t value;
  uint32_t num_tokens;
  uint32_t num_kv_heads;
  uint32_t head_dim;
} kvx_kv_io_desc_t;

/* Quantisation scales of a cache tensor (reference: kvx_abi.h:162-170).  The fp8 path
 * consumes PER_TENSOR ([1]) and PER_HEAD ([num_kv_heads]) F32 scales. */
typedef struct kvx_scale_desc {
  uint32_t size;
  kvx_dtype_t dtype;
  kvx_scale_granularity_t granularity;
  uint32_t ndim;
  int64_t shape[KVX_MAX_TENSOR_DIMS];
  int64_t stride[KVX_MAX_TENSOR_DIMS];
  const void *data;
} kvx_scale_desc_t;

/* One write call = one layer's new tokens (reference: kvx_abi.h:172-180).
 * k_scale / v_scale are per-tensor F32 device scalars used when the matching
 * *_scale_desc carries no data pointer. */
typedef struct kvx_write_desc {
  uint32_t size;
  kvx_kv_io_desc_t io;
  kvx_slot_mapping_t slots;
  const void *k_scale;
  const void *v_scale;
  kvx_scale_desc_t k_scale_desc;
  kvx_scale_desc_t v_scale_desc;
} kvx_write_desc_t;

/* One gather call = one layer's pages of a batch of sequences, materialised contiguously
 * (reference: kvx_abi.h:182-188). */
typedef struct kvx_gather_desc {
  uint32_t size;
  kvx_kv_io_desc_t io;
  kvx_block_table_t block_table;
  kvx_seq_lens_t seq_lens;
  uint32_t max_seq_len;
} kvx_gather_desc_t;

/* ---------------------------------------------------------------- entry points ------- */
/* These four live in a CUDA-free C11 translation unit and only inspect descriptors; they
 * never dereference a data pointer and ignore `stream`.  The data-moving entry points are
 * declared in kvx_paged_kv.h. */

/* reference: kvx_abi.h:190, kvx_abi.c:313-322 */
KVX_API kvx_status_t kvx_get_version(kvx_version_t *out_version);

/* Geometry non-zero, K and V agree on layout and dtype, both tensors have the shape of
 * their layout (INVALID_ARGUMENT otherwise) and its canonical contiguous strides
 * (UNSUPPORTED otherwise).  reference: kvx_abi.h:192, kvx_abi.c:324-352 */
KVX_API kvx_status_t kvx_validate_cache_desc(const kvx_cache_desc_t *cache);

/* Full descriptor check of a write batch.  reference: kvx_abi.h:194-195, kvx_abi.c:354-398 */
KVX_API kvx_status_t kvx_write_kv(const kvx_cache_desc_t *cache,
                                  const kvx_write_desc_t *write, void *stream);

/* Full descriptor check of a gather.  reference: kvx_abi.h:197-199, kvx_abi.c:400-466 */
KVX_API kvx_status_t kvx_gather_kv(const kvx_cache_desc_t *cache,
                                   const kvx_gather_desc_t *gather, void *stream);

#ifdef __cplusplus
} /* extern "C" */
#endif

/* Struct layout freeze for LP64 targets: the byte sizes the reference header produces with
 * gcc on x86-64.  A mismatch means a field was reordered or retyped. */
#if defined(__LP64__) && (defined(__cplusplus) || (defined(__STDC_VERSION__) && __STDC_VERSION__ >= 201112L))
#ifdef __cplusplus
#define KVX_ABI_SIZE_CHECK(type, bytes) static_assert(sizeof(type) == (bytes), #type " size changed")
#else
#define KVX_ABI_SIZE_CHECK(type, bytes) _Static_assert(sizeof(type) == (bytes), #type " size changed")
#endif
KVX_ABI_SIZE_CHECK(kvx_version_t, 16);
KVX_ABI_SIZE_CHECK(kvx_tensor_desc_t, 112);
KVX_ABI_SIZE_CHECK(kvx_pool_desc_t, 32);
KVX_ABI_SIZE_CHECK(kvx_cache_desc_t, 280);
KVX_ABI_SIZE_CHECK(kvx_block_table_t, 64);
KVX_ABI_SIZE_CHECK(kvx_slot_mapping_t, 32);
KVX_ABI_SIZE_CHECK(kvx_seq_lens_t, 24);
KVX_ABI_SIZE_CHECK(kvx_kv_io_desc_t, 248);
KVX_ABI_SIZE_CHECK(kvx_scale_desc_t, 104);
KVX_ABI_SIZE_CHECK(kvx_write_desc_t, 512);
KVX_ABI_SIZE_CHECK(kvx_gather_desc_t, 352);
#undef KVX_ABI_SIZE_CHECK
#endif

#endif /* KVX_ABI_H */
