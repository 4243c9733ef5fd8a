/*
 * torch operators over the C-ABI library, registered as torch.ops.kvx_b200.*:
 *
 *   reshape_and_cache_flash_kvx(key, value, key_cache!, value_cache!, slot_mapping,
 *                               kv_cache_dtype, k_scale, v_scale) -> ()
 *   gather_kv(key_cache, value_cache, block_table, seq_lens, key_out!, value_out!,
 *             kv_cache_dtype, k_scale, v_scale) -> ()
 *
 * The first has the schema, the checks and the descriptor filling of the operator the
 * reference's vLLM patch adds to vLLM's _C extension (reference: patches/vllm/kvx.patch:176-275,
 * schema :288-296): tensors are described as they are (sizes and strides, no copies), the cache
 * layout is inferred from sizes and strides (cache_form below), the batch is sized by
 * slot_mapping, the launch goes to the current CUDA stream, and a status other than OK
 * raises.  Going through the dispatcher instead of ctypes keeps the host cost of a decode-size
 * call at a few microseconds.  This file only marshals arguments; all data movement is in
 * kvx_paged_kv.cu.
 */
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

#include <cstring>
#include <string>

#include "kvx_attention.h"
#include "kvx_paged_kv.h"

namespace {

kvx_dtype_t float_code(at::ScalarType t) {
  switch (t) {
    case at::ScalarType::Float:
      return KVX_DTYPE_F32;
    case at::ScalarType::Half:
      return KVX_DTYPE_F16;
    case at::ScalarType::BFloat16:
      return KVX_DTYPE_BF16;
    default:
      return KVX_DTYPE_INVALID;
  }
}

kvx_dtype_t index_code(at::ScalarType t) {
  return t == at::ScalarType::Int ? KVX_DTYPE_S32 : t == at::ScalarType::Long ? KVX_DTYPE_S64 : KVX_DTYPE_INVALID;
}

void describe(kvx_tensor_desc_t *d, const torch::Tensor &t, kvx_dtype_t dtype, kvx_layout_t layout) {
  std::memset(d, 0, sizeof(*d));
  d->size = sizeof(*d);
  d->dtype = dtype;
  d->layout = layout;
  d->memory = KVX_MEMORY_DEVICE;
  d->ndim = static_cast<uint32_t>(t.dim());
  for (int64_t i = 0; i < t.dim() && i < KVX_MAX_TENSOR_DIMS; ++i) {
    d->shape[i] = t.size(i);
    d->stride[i] = t.stride(i);
  }
  d->data = t.data_ptr();
}

// Which page layout a 4-D cache tensor has.  The reference's operator decides by one stride
// (NHD when stride(2) == head_dim, reference: kvx.patch:132-135, :222-229), which misreads a
// contiguous [blocks, heads, block_size, dim] tensor; this rule agrees with it wherever it is
// right and also accepts that tensor and vLLM's permuted view of HND memory:
//   stride(1) < stride(2)          a [blocks, block_size, heads, dim] VIEW of HND memory
//   else size(2) == heads only     NHD   [blocks, block_size, heads, dim]
//   else size(1) == heads only     HND   [blocks, heads, block_size, dim]
//   else (block_size == heads)     the reference's stride rule
enum class CacheForm { kNhd, kHnd, kHndView };

CacheForm cache_form(const torch::Tensor &c, int64_t heads, int64_t head_dim) {
  if (c.stride(1) < c.stride(2)) return CacheForm::kHndView;
  const bool nhd = c.size(2) == heads, hnd = c.size(1) == heads;
  if (nhd != hnd) return nhd ? CacheForm::kNhd : CacheForm::kHnd;
  return c.stride(2) == head_dim ? CacheForm::kNhd : CacheForm::kHnd;
}

void describe_pages(kvx_tensor_desc_t *d, const torch::Tensor &t, kvx_dtype_t dtype, CacheForm form) {
  describe(d, t, dtype, form == CacheForm::kNhd ? KVX_LAYOUT_BLOCK_NHD : KVX_LAYOUT_BLOCK_HND);
  if (form == CacheForm::kHndView) {  // describe the memory: axes 1 and 2 swapped back
    d->shape[1] = t.size(2), d->shape[2] = t.size(1);
    d->stride[1] = t.stride(2), d->stride[2] = t.stride(1);
  }
}

// Cache descriptor from a pair of 4-D page tensors (reference: kvx.patch:222-245).
kvx_dtype_t describe_cache(kvx_cache_desc_t *c, const torch::Tensor &key_cache, const torch::Tensor &value_cache,
                           const std::string &kv_cache_dtype, int64_t heads, int64_t head_dim) {
  TORCH_CHECK(key_cache.is_cuda() && value_cache.is_cuda(), "cache tensors must be CUDA tensors");
  TORCH_CHECK(key_cache.dim() == 4 && key_cache.sizes() == value_cache.sizes(), "key/value cache shape mismatch");
  TORCH_CHECK(key_cache.scalar_type() == value_cache.scalar_type(), "cache dtype mismatch");
  kvx_dtype_t code;
  if (kv_cache_dtype == "auto") {
    code = float_code(key_cache.scalar_type());
    TORCH_CHECK(code != KVX_DTYPE_INVALID, "KVX cache: unsupported cache dtype");
  } else {
    TORCH_CHECK(kv_cache_dtype == "fp8" || kv_cache_dtype == "fp8_e4m3", "KVX cache: unsupported kv_cache_dtype ",
                kv_cache_dtype);
    TORCH_CHECK(key_cache.element_size() == 1, "an fp8 cache must have 1-byte elements");
    code = KVX_DTYPE_F8_E4M3;
  }
  const CacheForm form = cache_form(key_cache, heads, head_dim);
  TORCH_CHECK(cache_form(value_cache, heads, head_dim) == form, "key/value cache layout mismatch");
  std::memset(c, 0, sizeof(*c));
  c->size = sizeof(*c);
  c->num_blocks = static_cast<uint32_t>(key_cache.size(0));
  c->block_size = static_cast<uint32_t>(form == CacheForm::kHnd ? key_cache.size(2) : key_cache.size(1));
  c->num_kv_heads = static_cast<uint32_t>(form == CacheForm::kHnd ? key_cache.size(1) : key_cache.size(2));
  c->head_dim = static_cast<uint32_t>(key_cache.size(3));
  describe_pages(&c->k, key_cache, code, form);
  describe_pages(&c->v, value_cache, code, form);
  c->pool.size = sizeof(c->pool);
  return code;
}

void describe_scale(kvx_scale_desc_t *d, const torch::Tensor &scale, int64_t heads) {
  std::memset(d, 0, sizeof(*d));
  d->size = sizeof(*d);
  d->dtype = KVX_DTYPE_F32;
  if (!scale.defined() || scale.numel() == 0) return;
  TORCH_CHECK(scale.is_cuda() && scale.scalar_type() == at::ScalarType::Float, "scales must be float32 CUDA tensors");
  TORCH_CHECK(scale.numel() == 1 || (scale.dim() == 1 && scale.numel() == heads),
              "a scale must have 1 or num_kv_heads elements");
  d->granularity = scale.numel() == 1 ? KVX_SCALE_PER_TENSOR : KVX_SCALE_PER_HEAD;
  d->ndim = 1;
  d->shape[0] = scale.numel();
  d->stride[0] = scale.dim() == 1 ? scale.stride(0) : 1;
  d->data = scale.data_ptr();
}

void reshape_and_cache_flash_kvx(torch::Tensor &key, torch::Tensor &value, torch::Tensor &key_cache,
                                 torch::Tensor &value_cache, torch::Tensor &slot_mapping,
                                 const std::string &kv_cache_dtype, torch::Tensor &k_scale, torch::Tensor &v_scale) {
  TORCH_CHECK(key.is_cuda() && value.is_cuda(), "key/value must be CUDA tensors");
  TORCH_CHECK(key.dim() == 3 && value.dim() == 3, "key/value must be [num_tokens, num_heads, head_dim]");
  TORCH_CHECK(key.scalar_type() == value.scalar_type(), "key/value dtype mismatch");
  const kvx_dtype_t io = float_code(key.scalar_type());
  TORCH_CHECK(io != KVX_DTYPE_INVALID, "KVX cache write unsupported dtype");
  const kvx_dtype_t slot_dtype = index_code(slot_mapping.scalar_type());
  TORCH_CHECK(slot_dtype != KVX_DTYPE_INVALID && slot_mapping.dim() == 1, "slot_mapping must be 1-D int32 or int64");
  TORCH_CHECK(slot_mapping.is_cuda() && slot_mapping.is_contiguous(), "slot_mapping must be a contiguous CUDA tensor");
  const int64_t tokens = slot_mapping.size(0), heads = key.size(1), dim = key.size(2);
  // the batch is sized by slot_mapping (as in the operator this one stands in for), so key and
  // value must hold at least that many token rows
  TORCH_CHECK(key.size(0) >= tokens && value.size(0) >= tokens, "key/value hold fewer tokens than slot_mapping");
  TORCH_CHECK(key_cache.is_cuda() && value_cache.is_cuda(), "cache tensors must be CUDA tensors");
  const at::cuda::OptionalCUDAGuard guard(at::device_of(key_cache));  // launch on the tensors' device and its stream

  kvx_cache_desc_t cache;
  const kvx_dtype_t cache_code = describe_cache(&cache, key_cache, value_cache, kv_cache_dtype, heads, dim);
  TORCH_CHECK(cache_code == io || cache_code == KVX_DTYPE_F8_E4M3, "key/value dtype must match cache dtype");

  kvx_write_desc_t write;
  std::memset(&write, 0, sizeof(write));
  write.size = sizeof(write);
  write.io.size = sizeof(write.io);
  write.io.num_tokens = static_cast<uint32_t>(tokens);
  write.io.num_kv_heads = static_cast<uint32_t>(heads);
  write.io.head_dim = static_cast<uint32_t>(dim);
  describe(&write.io.key, key, io, KVX_LAYOUT_INVALID);
  describe(&write.io.value, value, io, KVX_LAYOUT_INVALID);
  write.io.key.shape[0] = write.io.value.shape[0] = tokens;  // the batch is sized by slot_mapping
  write.slots.size = sizeof(write.slots);
  write.slots.dtype = slot_dtype;
  write.slots.token_count = static_cast<uint32_t>(tokens);
  write.slots.invalid_slot = -1;
  write.slots.slots = slot_mapping.data_ptr();
  describe_scale(&write.k_scale_desc, k_scale, heads);
  describe_scale(&write.v_scale_desc, v_scale, heads);

  void *stream = reinterpret_cast<void *>(at::cuda::getCurrentCUDAStream().stream());
  const kvx_status_t status = kvx_launch_write_kv(&cache, &write, stream);
  TORCH_CHECK(status == KVX_STATUS_OK, "kvx cache write failed with status=", static_cast<int>(status));
}

void gather_kv(torch::Tensor &key_cache, torch::Tensor &value_cache, torch::Tensor &block_table,
               torch::Tensor &seq_lens, torch::Tensor &key_out, torch::Tensor &value_out,
               const std::string &kv_cache_dtype, torch::Tensor &k_scale, torch::Tensor &v_scale) {
  TORCH_CHECK(key_out.is_cuda() && value_out.is_cuda(), "outputs must be CUDA tensors");
  TORCH_CHECK(key_out.dim() == 4 && key_out.sizes() == value_out.sizes(),
              "outputs must be [seq_count, max_seq_len, heads, dim]");
  const kvx_dtype_t io = float_code(key_out.scalar_type());
  TORCH_CHECK(io != KVX_DTYPE_INVALID && value_out.scalar_type() == key_out.scalar_type(), "unsupported output dtype");
  TORCH_CHECK(block_table.dim() == 2 && block_table.is_contiguous(), "block_table must be contiguous and 2-D");
  const kvx_dtype_t idx = index_code(block_table.scalar_type());
  TORCH_CHECK(idx != KVX_DTYPE_INVALID && seq_lens.scalar_type() == block_table.scalar_type(),
              "block_table and seq_lens must share an int32 or int64 dtype");
  const int64_t seqs = key_out.size(0), max_len = key_out.size(1), heads = key_out.size(2), dim = key_out.size(3);
  TORCH_CHECK(block_table.is_cuda() && seq_lens.is_cuda() && seq_lens.is_contiguous(),
              "block_table and seq_lens must be contiguous CUDA tensors");
  TORCH_CHECK(seq_lens.dim() == 1 && seq_lens.numel() == block_table.size(0),
              "seq_lens must have one entry per row of block_table");
  TORCH_CHECK(key_cache.is_cuda() && value_cache.is_cuda(), "cache tensors must be CUDA tensors");
  const at::cuda::OptionalCUDAGuard guard(at::device_of(key_cache));

  kvx_cache_desc_t cache;
  const kvx_dtype_t cache_code = describe_cache(&cache, key_cache, value_cache, kv_cache_dtype, heads, dim);

  kvx_gather_desc_t g;
  std::memset(&g, 0, sizeof(g));
  g.size = sizeof(g);
  g.io.size = sizeof(g.io);
  g.io.num_tokens = static_cast<uint32_t>(seqs * max_len);
  g.io.num_kv_heads = static_cast<uint32_t>(heads);
  g.io.head_dim = static_cast<uint32_t>(dim);
  describe(&g.io.key, key_out, io, KVX_LAYOUT_INVALID);
  describe(&g.io.value, value_out, io, KVX_LAYOUT_INVALID);
  g.block_table.size = sizeof(g.block_table);
  g.block_table.format = KVX_BLOCK_TABLE_PACKED;
  g.block_table.index_dtype = idx;
  g.block_table.seq_count = static_cast<uint32_t>(block_table.size(0));
  g.block_table.beam_width = 1;
  g.block_table.max_blocks_per_seq = static_cast<uint32_t>(block_table.size(1));
  g.block_table.indices = block_table.data_ptr();
  g.block_table.indices_count = static_cast<uint32_t>(block_table.numel());
  g.seq_lens.size = sizeof(g.seq_lens);
  g.seq_lens.dtype = idx;
  g.seq_lens.seq_count = static_cast<uint32_t>(seq_lens.size(0));
  g.seq_lens.lengths = seq_lens.data_ptr();
  g.max_seq_len = static_cast<uint32_t>(max_len);

  void *stream = reinterpret_cast<void *>(at::cuda::getCurrentCUDAStream().stream());
  kvx_status_t status;
  if (cache_code == KVX_DTYPE_F8_E4M3) {
    kvx_scale_desc_t ks, vs;
    describe_scale(&ks, k_scale, heads);
    describe_scale(&vs, v_scale, heads);
    status = kvx_launch_gather_kv_f8e4m3(&cache, &g, &ks, &vs, stream);
  } else {
    status = kvx_launch_gather_kv(&cache, &g, stream);
  }
  TORCH_CHECK(status == KVX_STATUS_OK, "kvx cache gather failed with status=", static_cast<int>(status));
}

// Decode attention over the paged cache (include/kvx_attention.h).  `workspace` is a uint8 CUDA
// tensor of at least kvx_paged_attention_workspace_bytes() bytes (see attention_workspace_bytes).
void paged_attention_decode(torch::Tensor &out, torch::Tensor &query, torch::Tensor &key_cache,
                            torch::Tensor &value_cache, torch::Tensor &block_table, torch::Tensor &seq_lens,
                            double scale, int64_t max_seq_len, int64_t num_kv_heads, torch::Tensor &workspace,
                            const std::string &kv_cache_dtype, torch::Tensor &k_scale, torch::Tensor &v_scale) {
  TORCH_CHECK(query.is_cuda() && out.is_cuda(), "query/out must be CUDA tensors");
  TORCH_CHECK(query.dim() == 3 && query.sizes() == out.sizes() && query.scalar_type() == out.scalar_type(),
              "query/out must be matching [seq_count, q_heads, head_dim] tensors");
  const kvx_dtype_t io = float_code(query.scalar_type());
  TORCH_CHECK(io != KVX_DTYPE_INVALID, "unsupported query dtype");
  TORCH_CHECK(block_table.dim() == 2 && block_table.is_contiguous(), "block_table must be contiguous and 2-D");
  const kvx_dtype_t idx = index_code(block_table.scalar_type());
  TORCH_CHECK(idx != KVX_DTYPE_INVALID && seq_lens.scalar_type() == block_table.scalar_type(),
              "block_table and seq_lens must share an int32 or int64 dtype");
  const int64_t q_heads = query.size(1), dim = query.size(2);
  TORCH_CHECK(block_table.is_cuda() && seq_lens.is_cuda() && seq_lens.is_contiguous(),
              "block_table and seq_lens must be contiguous CUDA tensors");
  TORCH_CHECK(seq_lens.dim() == 1 && seq_lens.numel() == block_table.size(0),
              "seq_lens must have one entry per row of block_table");
  TORCH_CHECK(key_cache.is_cuda() && value_cache.is_cuda(), "cache tensors must be CUDA tensors");
  const at::cuda::OptionalCUDAGuard guard(at::device_of(key_cache));
  // KV heads: given, or read off the cache with the reference's stride rule (axis 2 when it is
  // contiguous over head_dim or the tensor is a permuted view, else axis 1)
  TORCH_CHECK(key_cache.dim() == 4, "cache tensors must be 4-D");
  const int64_t kv_heads = num_kv_heads > 0 ? num_kv_heads
                           : (key_cache.stride(1) < key_cache.stride(2) || key_cache.stride(2) == dim)
                               ? key_cache.size(2)
                               : key_cache.size(1);
  kvx_cache_desc_t cache;
  describe_cache(&cache, key_cache, value_cache, kv_cache_dtype, kv_heads, dim);

  kvx_attention_desc_t a;
  std::memset(&a, 0, sizeof(a));
  a.size = sizeof(a);
  a.num_q_heads = static_cast<uint32_t>(q_heads);
  a.max_seq_len = static_cast<uint32_t>(max_seq_len);
  a.scale = static_cast<float>(scale);
  describe(&a.query, query, io, KVX_LAYOUT_INVALID);
  describe(&a.out, out, io, KVX_LAYOUT_INVALID);
  a.block_table.size = sizeof(a.block_table);
  a.block_table.format = KVX_BLOCK_TABLE_PACKED;
  a.block_table.index_dtype = idx;
  a.block_table.seq_count = static_cast<uint32_t>(block_table.size(0));
  a.block_table.beam_width = 1;
  a.block_table.max_blocks_per_seq = static_cast<uint32_t>(block_table.size(1));
  a.block_table.indices = block_table.data_ptr();
  a.block_table.indices_count = static_cast<uint32_t>(block_table.numel());
  a.seq_lens.size = sizeof(a.seq_lens);
  a.seq_lens.dtype = idx;
  a.seq_lens.seq_count = static_cast<uint32_t>(seq_lens.size(0));
  a.seq_lens.lengths = seq_lens.data_ptr();
  kvx_scale_desc_t ks, vs;
  describe_scale(&ks, k_scale, cache.num_kv_heads);
  describe_scale(&vs, v_scale, cache.num_kv_heads);
  TORCH_CHECK(workspace.is_cuda() && workspace.is_contiguous(), "workspace must be a contiguous CUDA tensor");
  void *stream = reinterpret_cast<void *>(at::cuda::getCurrentCUDAStream().stream());
  const kvx_status_t status = kvx_launch_paged_attention_decode(
      &cache, &a, &ks, &vs, workspace.data_ptr(), static_cast<size_t>(workspace.numel() * workspace.element_size()), stream);
  TORCH_CHECK(status == KVX_STATUS_OK, "kvx paged attention failed with status=", static_cast<int>(status));
}

}  // namespace

TORCH_LIBRARY(kvx_b200, m) {
  m.def(
      "reshape_and_cache_flash_kvx(Tensor key, Tensor value, Tensor! key_cache, Tensor! value_cache,"
      " Tensor slot_mapping, str kv_cache_dtype, Tensor k_scale, Tensor v_scale) -> ()");
  m.def(
      "gather_kv(Tensor key_cache, Tensor value_cache, Tensor block_table, Tensor seq_lens, Tensor! key_out,"
      " Tensor! value_out, str kv_cache_dtype, Tensor k_scale, Tensor v_scale) -> ()");
  m.def(
      "paged_attention_decode(Tensor! out, Tensor query, Tensor key_cache, Tensor value_cache, Tensor block_table,"
      " Tensor seq_lens, float scale, int max_seq_len, int num_kv_heads, Tensor! workspace, str kv_cache_dtype,"
      " Tensor k_scale,"
      " Tensor v_scale) -> ()");
}

TORCH_LIBRARY_IMPL(kvx_b200, CUDA, m) {
  m.impl("reshape_and_cache_flash_kvx", &reshape_and_cache_flash_kvx);
  m.impl("gather_kv", &gather_kv);
  m.impl("paged_attention_decode", &paged_attention_decode);
}
