/*
 * Host-buffer pipeline over the launch layer: stages host K/V batches into device memory in
 * chunks (copy of chunk i+1 overlaps the kernel of chunk i) and brings gathered sequences
 * back, copying only the bytes the gather defines.  See include/kvx_host.h.
 */
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <new>

#include "kvx_host.h"
#include "kvx_paged_kv.h"

namespace {

constexpr int kSets = 3;   // staging sets in rotation, per ring
constexpr int kRings = 2;  // ring 0 stages write batches, ring 1 stages gathered sequences
// Longest K (or V) run that returns paired with the other tensor's as one 2-D copy: beyond it
// a copy's set-up no longer shows, and 2-D copies with rows of 64 MB measured erratic.
constexpr int64_t kPairedRunBytes = int64_t{16} << 20;

int64_t elem_bytes(kvx_dtype_t t) {
  switch (t) {
    case KVX_DTYPE_F16:
    case KVX_DTYPE_BF16:
      return 2;
    case KVX_DTYPE_F32:
      return 4;
    case KVX_DTYPE_F8_E4M3:
      return 1;
    default:
      return 0;
  }
}

int64_t index_at(const void *p, kvx_dtype_t t, int64_t i) {
  return t == KVX_DTYPE_S32 ? static_cast<int64_t>(static_cast<const int32_t *>(p)[i])
                            : static_cast<const int64_t *>(p)[i];
}

}  // namespace

struct kvx_host_pipe {
  size_t chunk_bytes = 0;
  size_t table_cap = 0;  // index entries
  uint32_t max_seqs = 0;
  // Writes and gathers use separate rings so that host->device copies of the next write never
  // wait for device->host copies of the previous gather: both PCIe directions stay busy.
  char *k_stage[kRings * kSets] = {};
  char *v_stage[kRings * kSets] = {};
  char *slot_stage[kSets] = {};
  size_t slot_cap = 0;  // bytes per slot staging buffer
  char *table_dev = nullptr;
  char *lens_dev = nullptr;
  cudaStream_t h2d = nullptr, exec = nullptr, d2h = nullptr;
  cudaStream_t d2h_v = nullptr;  // V runs come back on a stream of their own: the gaps between the many
                                 // per-sequence copies of one stream are filled by the other
  cudaEvent_t v_back = nullptr;  // the V copies of a staging set are done
  cudaEvent_t ready[kRings * kSets] = {};  // staging set filled (h2d) / gathered (exec)
  cudaEvent_t freed[kRings * kSets] = {};  // staging set consumed (exec) / copied back (d2h)
  cudaEvent_t meta_done = nullptr;   // kernels of the last gather are done with table_dev / lens_dev
  cudaEvent_t meta_ready = nullptr;  // table_dev / lens_dev hold the current call's metadata
  uint64_t uses[kRings] = {};  // staging sets handed out so far, per ring
  uint64_t h2d_bytes = 0, d2h_bytes = 0;
  bool failed = false;
};

namespace {

bool ok(kvx_host_pipe *p, cudaError_t e) {
  if (e != cudaSuccess) p->failed = true;
  return e == cudaSuccess;
}

// Next staging set; the stream that will fill it first waits until its previous contents
// were consumed.
int acquire_set(kvx_host_pipe *p, int ring, cudaStream_t filler) {
  const int s = ring * kSets + static_cast<int>(p->uses[ring] % kSets);
  if (p->uses[ring] >= kSets) ok(p, cudaStreamWaitEvent(filler, p->freed[s], 0));
  ++p->uses[ring];
  return s;
}

}  // namespace

extern "C" {

KVX_API kvx_status_t kvx_host_pipe_create(size_t chunk_bytes, uint32_t max_seqs, uint32_t max_blocks_per_seq,
                                          kvx_host_pipe_t **out_pipe) {
  if (out_pipe == nullptr || chunk_bytes < 4096 || max_seqs == 0 || max_blocks_per_seq == 0)
    return KVX_STATUS_INVALID_ARGUMENT;
  kvx_host_pipe *p = new (std::nothrow) kvx_host_pipe();
  if (p == nullptr) return KVX_STATUS_INTERNAL_ERROR;
  p->chunk_bytes = chunk_bytes / 256 * 256;
  p->slot_cap = p->chunk_bytes / 16 * 8 + 256;  // a token row is at least 16 bytes here
  p->table_cap = static_cast<size_t>(max_seqs) * max_blocks_per_seq;
  p->max_seqs = max_seqs;
  bool good = true;
  for (int i = 0; i < kRings * kSets && good; ++i) {
    // K and V staging of a set are one allocation, V one chunk behind K: a K run and the V run
    // of the same rows are then the two rows of one 2-D copy
    good = cudaMalloc(&p->k_stage[i], 2 * p->chunk_bytes) == cudaSuccess &&
           (p->v_stage[i] = p->k_stage[i] + p->chunk_bytes) != nullptr &&
           (i >= kSets || cudaMalloc(&p->slot_stage[i], p->slot_cap) == cudaSuccess) &&
           cudaEventCreateWithFlags(&p->ready[i], cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&p->freed[i], cudaEventDisableTiming) == cudaSuccess;
  }
  good = good && cudaMalloc(&p->table_dev, p->table_cap * 8) == cudaSuccess &&
         cudaMalloc(&p->lens_dev, static_cast<size_t>(max_seqs) * 8) == cudaSuccess &&
         cudaStreamCreateWithFlags(&p->h2d, cudaStreamNonBlocking) == cudaSuccess &&
         cudaStreamCreateWithFlags(&p->exec, cudaStreamNonBlocking) == cudaSuccess &&
         cudaStreamCreateWithFlags(&p->d2h, cudaStreamNonBlocking) == cudaSuccess &&
         cudaStreamCreateWithFlags(&p->d2h_v, cudaStreamNonBlocking) == cudaSuccess &&
         cudaEventCreateWithFlags(&p->v_back, cudaEventDisableTiming) == cudaSuccess &&
         cudaEventCreateWithFlags(&p->meta_done, cudaEventDisableTiming) == cudaSuccess &&
         cudaEventCreateWithFlags(&p->meta_ready, cudaEventDisableTiming) == cudaSuccess;
  if (!good) {
    cudaGetLastError();
    kvx_host_pipe_destroy(p);
    return KVX_STATUS_OUT_OF_RANGE;
  }
  *out_pipe = p;
  return KVX_STATUS_OK;
}

KVX_API void kvx_host_pipe_destroy(kvx_host_pipe_t *p) {
  if (p == nullptr) return;
  if (p->h2d) cudaStreamSynchronize(p->h2d);
  if (p->exec) cudaStreamSynchronize(p->exec);
  if (p->d2h) cudaStreamSynchronize(p->d2h);
  if (p->d2h_v) cudaStreamSynchronize(p->d2h_v);
  for (int i = 0; i < kRings * kSets; ++i) {
    cudaFree(p->k_stage[i]);  // (V staging is its second half)
    if (i < kSets) cudaFree(p->slot_stage[i]);
    if (p->ready[i]) cudaEventDestroy(p->ready[i]);
    if (p->freed[i]) cudaEventDestroy(p->freed[i]);
  }
  cudaFree(p->table_dev);
  cudaFree(p->lens_dev);
  if (p->meta_done) cudaEventDestroy(p->meta_done);
  if (p->meta_ready) cudaEventDestroy(p->meta_ready);
  if (p->h2d) cudaStreamDestroy(p->h2d);
  if (p->exec) cudaStreamDestroy(p->exec);
  if (p->d2h) cudaStreamDestroy(p->d2h);
  if (p->d2h_v) cudaStreamDestroy(p->d2h_v);
  if (p->v_back) cudaEventDestroy(p->v_back);
  delete p;
}

KVX_API kvx_status_t kvx_host_write_kv(kvx_host_pipe_t *p, const kvx_cache_desc_t *cache,
                                       const kvx_write_desc_t *write) {
  if (p == nullptr || cache == nullptr || write == nullptr) return KVX_STATUS_INVALID_ARGUMENT;
  if (write->size < sizeof(kvx_write_desc_t)) return KVX_STATUS_INVALID_ARGUMENT;
  const int64_t T = write->io.num_tokens;
  const int64_t row = static_cast<int64_t>(write->io.num_kv_heads) * write->io.head_dim *
                      elem_bytes(write->io.key.dtype);
  const int64_t slot_b = write->slots.dtype == KVX_DTYPE_S32 ? 4 : 8;
  if (T == 0 || row == 0) return kvx_launch_write_kv(cache, write, p->exec);  // validates, launches nothing
  if (write->io.key.data == nullptr || write->io.value.data == nullptr || write->slots.slots == nullptr)
    return KVX_STATUS_INVALID_ARGUMENT;
  if (row < 16 || static_cast<size_t>(row) > p->chunk_bytes) return KVX_STATUS_UNSUPPORTED;
  // Host token rows may lie further apart than heads * dim elements (a view of a fused
  // projection output), as kvx_launch_write_kv allows for device rows; inside a row the
  // elements must be dense.  Rows are staged densely, so the kernels always see dense rows.
  const int64_t e = elem_bytes(write->io.key.dtype);
  const int64_t hd = static_cast<int64_t>(write->io.num_kv_heads) * write->io.head_dim;
  for (const kvx_tensor_desc_t *t : {&write->io.key, &write->io.value}) {
    if (t->ndim != 3) return KVX_STATUS_INVALID_ARGUMENT;
    if (t->shape[0] != T || t->shape[1] != write->io.num_kv_heads || t->shape[2] != write->io.head_dim)
      return KVX_STATUS_INVALID_ARGUMENT;
    if (t->stride[2] != 1 || t->stride[1] != write->io.head_dim || t->stride[0] < hd) return KVX_STATUS_UNSUPPORTED;
  }
  if (write->io.value.dtype != write->io.key.dtype) return KVX_STATUS_UNSUPPORTED;
  const int64_t k_pitch = write->io.key.stride[0] * e, v_pitch = write->io.value.stride[0] * e;
  const int64_t per_chunk = static_cast<int64_t>(p->chunk_bytes) / row;

  for (int64_t t0 = 0; t0 < T; t0 += per_chunk) {
    const int64_t n = std::min(per_chunk, T - t0);
    const int s = acquire_set(p, 0, p->h2d);
    const char *hk = static_cast<const char *>(write->io.key.data) + t0 * k_pitch;
    const char *hv = static_cast<const char *>(write->io.value.data) + t0 * v_pitch;
    const char *hs = static_cast<const char *>(write->slots.slots) + t0 * slot_b;
    if (k_pitch == row)
      ok(p, cudaMemcpyAsync(p->k_stage[s], hk, n * row, cudaMemcpyHostToDevice, p->h2d));
    else
      ok(p, cudaMemcpy2DAsync(p->k_stage[s], row, hk, k_pitch, row, n, cudaMemcpyHostToDevice, p->h2d));
    if (v_pitch == row)
      ok(p, cudaMemcpyAsync(p->v_stage[s], hv, n * row, cudaMemcpyHostToDevice, p->h2d));
    else
      ok(p, cudaMemcpy2DAsync(p->v_stage[s], row, hv, v_pitch, row, n, cudaMemcpyHostToDevice, p->h2d));
    ok(p, cudaMemcpyAsync(p->slot_stage[s], hs, n * slot_b, cudaMemcpyHostToDevice, p->h2d));
    ok(p, cudaEventRecord(p->ready[s], p->h2d));
    ok(p, cudaStreamWaitEvent(p->exec, p->ready[s], 0));
    p->h2d_bytes += static_cast<uint64_t>(n) * (2 * row + slot_b);

    kvx_write_desc_t w = *write;
    w.io.num_tokens = static_cast<uint32_t>(n);
    w.io.key.shape[0] = w.io.value.shape[0] = n;
    w.io.key.stride[0] = w.io.value.stride[0] = hd;  // staged rows are dense
    w.io.key.data = p->k_stage[s];
    w.io.value.data = p->v_stage[s];
    w.io.key.memory = w.io.value.memory = KVX_MEMORY_DEVICE;
    w.slots.token_count = static_cast<uint32_t>(n);
    w.slots.slots = p->slot_stage[s];
    const kvx_status_t st = kvx_launch_write_kv(cache, &w, p->exec);
    ok(p, cudaEventRecord(p->freed[s], p->exec));
    if (st != KVX_STATUS_OK) return st;
  }
  return p->failed ? KVX_STATUS_INTERNAL_ERROR : KVX_STATUS_OK;
}

KVX_API kvx_status_t kvx_host_gather_kv(kvx_host_pipe_t *p, const kvx_cache_desc_t *cache,
                                        const kvx_gather_desc_t *gather, const kvx_scale_desc_t *k_scale,
                                        const kvx_scale_desc_t *v_scale) {
  if (p == nullptr || cache == nullptr || gather == nullptr) return KVX_STATUS_INVALID_ARGUMENT;
  if (gather->size < sizeof(kvx_gather_desc_t)) return KVX_STATUS_INVALID_ARGUMENT;
  const kvx_block_table_t &bt = gather->block_table;
  const int64_t S = bt.seq_count, mb = bt.max_blocks_per_seq, L = gather->max_seq_len;
  const int64_t bs = cache->block_size;
  const int64_t row = static_cast<int64_t>(gather->io.num_kv_heads) * gather->io.head_dim *
                      elem_bytes(gather->io.key.dtype);
  const bool fp8 = cache->k.dtype == KVX_DTYPE_F8_E4M3;
  auto launch = [&](const kvx_gather_desc_t *g, void *stream) {
    return fp8 ? kvx_launch_gather_kv_f8e4m3(cache, g, k_scale, v_scale, stream)
               : kvx_launch_gather_kv(cache, g, stream);
  };
  if (S == 0 || L == 0 || row == 0 || mb == 0) return launch(gather, p->exec);
  if (bt.format != KVX_BLOCK_TABLE_PACKED) return KVX_STATUS_UNSUPPORTED;
  if (bt.index_dtype != gather->seq_lens.dtype ||
      (bt.index_dtype != KVX_DTYPE_S32 && bt.index_dtype != KVX_DTYPE_S64))
    return KVX_STATUS_INVALID_ARGUMENT;
  if (gather->io.key.data == nullptr || gather->io.value.data == nullptr || bt.indices == nullptr ||
      gather->seq_lens.lengths == nullptr || bs == 0)
    return KVX_STATUS_INVALID_ARGUMENT;
  const int64_t idx_b = bt.index_dtype == KVX_DTYPE_S32 ? 4 : 8;
  const int64_t seq_bytes = L * row;
  if (static_cast<size_t>(S * mb) > p->table_cap || S > p->max_seqs ||
      static_cast<size_t>(seq_bytes) > p->chunk_bytes)
    return KVX_STATUS_UNSUPPORTED;

  // Index metadata goes over once per call.
  ok(p, cudaStreamWaitEvent(p->h2d, p->meta_done, 0));  // previous call's kernels are done with it
  ok(p, cudaMemcpyAsync(p->table_dev, bt.indices, S * mb * idx_b, cudaMemcpyHostToDevice, p->h2d));
  ok(p, cudaMemcpyAsync(p->lens_dev, gather->seq_lens.lengths, S * idx_b, cudaMemcpyHostToDevice, p->h2d));
  p->h2d_bytes += static_cast<uint64_t>(S * mb * idx_b + S * idx_b);
  ok(p, cudaEventRecord(p->meta_ready, p->h2d));
  ok(p, cudaStreamWaitEvent(p->exec, p->meta_ready, 0));

  const int64_t per_chunk = std::max<int64_t>(1, static_cast<int64_t>(p->chunk_bytes) / seq_bytes);
  kvx_status_t status = KVX_STATUS_OK;
  for (int64_t s0 = 0; s0 < S && status == KVX_STATUS_OK; s0 += per_chunk) {
    const int64_t n = std::min(per_chunk, S - s0);
    const int set = acquire_set(p, 1, p->exec);
    kvx_gather_desc_t g = *gather;
    g.io.num_tokens = static_cast<uint32_t>(n * L);
    g.io.key.shape[0] = g.io.value.shape[0] = n;
    g.io.key.data = p->k_stage[set];
    g.io.value.data = p->v_stage[set];
    g.io.key.memory = g.io.value.memory = KVX_MEMORY_DEVICE;
    g.block_table.seq_count = static_cast<uint32_t>(n);
    g.block_table.indices = p->table_dev + s0 * mb * idx_b;
    g.block_table.indices_count = static_cast<uint32_t>(n * mb);
    g.seq_lens.seq_count = static_cast<uint32_t>(n);
    g.seq_lens.lengths = p->lens_dev + s0 * idx_b;
    status = launch(&g, p->exec);
    ok(p, cudaEventRecord(p->ready[set], p->exec));
    ok(p, cudaStreamWaitEvent(p->d2h, p->ready[set], 0));
    ok(p, cudaStreamWaitEvent(p->d2h_v, p->ready[set], 0));

    // Copy back runs of consecutive defined pages, never a byte more.  Under load from the other
    // direction a device->host copy costs about 20 us whatever its size, and a sequence's runs are
    // a few MB, so where the caller's K and V outputs lie a fixed distance apart that a 2-D copy
    // can use as its pitch (V behind K, less than 2 GB: one allocation for both, say), the K run
    // and the V run go back as the two rows of ONE copy.
    const int64_t kv_apart = static_cast<char *>(gather->io.value.data) - static_cast<char *>(gather->io.key.data);
    const bool paired = kvx_b200_get_option("host_pair_kv") != 0 && kv_apart >= S * seq_bytes && kv_apart <= INT32_MAX;
    for (int64_t i = 0; i < n && status == KVX_STATUS_OK; ++i) {
      const int64_t s = s0 + i;
      int64_t len = index_at(gather->seq_lens.lengths, bt.index_dtype, s);
      len = std::min(len, std::min(L, mb * bs));
      const int64_t pages = len > 0 ? (len + bs - 1) / bs : 0;
      int64_t run_begin = -1;
      for (int64_t lb = 0; lb <= pages; ++lb) {
        bool valid = false;
        if (lb < pages) {
          const int64_t b = index_at(bt.indices, bt.index_dtype, s * mb + lb);
          valid = b >= 0 && b < static_cast<int64_t>(cache->num_blocks);
        }
        if (valid && run_begin < 0) run_begin = lb;
        if (!valid && run_begin >= 0) {
          const int64_t tok0 = run_begin * bs, tok1 = std::min(lb * bs, len);
          const int64_t off = tok0 * row, bytes = (tok1 - tok0) * row;
          char *hk = static_cast<char *>(gather->io.key.data) + s * seq_bytes + off;
          char *hv = static_cast<char *>(gather->io.value.data) + s * seq_bytes + off;
          if (paired && bytes <= kPairedRunBytes) {
            ok(p, cudaMemcpy2DAsync(hk, static_cast<size_t>(kv_apart), p->k_stage[set] + i * seq_bytes + off, p->chunk_bytes,
                                    static_cast<size_t>(bytes), 2, cudaMemcpyDeviceToHost, p->d2h));
          } else {
            ok(p, cudaMemcpyAsync(hk, p->k_stage[set] + i * seq_bytes + off, bytes, cudaMemcpyDeviceToHost, p->d2h));
            ok(p, cudaMemcpyAsync(hv, p->v_stage[set] + i * seq_bytes + off, bytes, cudaMemcpyDeviceToHost, p->d2h_v));
          }
          p->d2h_bytes += static_cast<uint64_t>(2 * bytes);
          run_begin = -1;
        }
      }
    }
    ok(p, cudaEventRecord(p->v_back, p->d2h_v));
    ok(p, cudaStreamWaitEvent(p->d2h, p->v_back, 0));
    ok(p, cudaEventRecord(p->freed[set], p->d2h));
  }
  ok(p, cudaEventRecord(p->meta_done, p->exec));
  if (status != KVX_STATUS_OK) return status;
  return p->failed ? KVX_STATUS_INTERNAL_ERROR : KVX_STATUS_OK;
}

KVX_API kvx_status_t kvx_host_pipe_sync(kvx_host_pipe_t *p) {
  if (p == nullptr) return KVX_STATUS_INVALID_ARGUMENT;
  bool good = cudaStreamSynchronize(p->h2d) == cudaSuccess;
  good = (cudaStreamSynchronize(p->exec) == cudaSuccess) && good;
  good = (cudaStreamSynchronize(p->d2h) == cudaSuccess) && good;
  good = (cudaStreamSynchronize(p->d2h_v) == cudaSuccess) && good;
  // a gather kernel that abandoned a bounded wait has left rows unwritten
  if (good && kvx_b200_device_error(1) != 0) good = false;
  if (!good || p->failed) {
    p->failed = false;
    return KVX_STATUS_INTERNAL_ERROR;
  }
  return KVX_STATUS_OK;
}

KVX_API void kvx_host_pipe_traffic(const kvx_host_pipe_t *p, uint64_t *h2d_bytes, uint64_t *d2h_bytes) {
  if (p == nullptr) return;
  if (h2d_bytes) *h2d_bytes = p->h2d_bytes;
  if (d2h_bytes) *d2h_bytes = p->d2h_bytes;
}

}  // extern "C"
