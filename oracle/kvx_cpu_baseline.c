/*
 * CPU BASELINE -- TEST / BENCHMARK INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * The fastest straightforward host form of the write and the gather: one memcpy per valid
 * token row (write) and one memcpy per (sequence, page) chunk (gather), split over
 * pthreads.  It exists so the benchmark can print "what the host cores do with the same
 * bytes" beside the GPU number; results are checked against kvx_oracle.c in the tests.
 * Semantics: kernels/kvx_paged_kv.cu:98-123 (write) and :232-266 (gather) of the reference.
 */
#include "kvx_oracle.h"

#include <pthread.h>
#include <string.h>

typedef struct job {
  const kvx_cache_desc_t *cache;
  const kvx_write_desc_t *write;
  const kvx_gather_desc_t *gather;
  int64_t begin, end; /* token range (write) or sequence*block range (gather) */
  size_t row_bytes;
} job_t;

static size_t elem_size(kvx_dtype_t t) {
  return (t == KVX_DTYPE_F32) ? 4 : (t == KVX_DTYPE_F16 || t == KVX_DTYPE_BF16) ? 2 : 0;
}

static int nhd_canonical(const kvx_cache_desc_t *c, const kvx_tensor_desc_t *t) {
  const int64_t H = c->num_kv_heads, D = c->head_dim, bs = c->block_size;
  return t->layout == KVX_LAYOUT_BLOCK_NHD && t->stride[3] == 1 && t->stride[2] == D &&
         t->stride[1] == H * D && t->stride[0] == bs * H * D;
}

static int64_t index_at(const void *p, kvx_dtype_t t, int64_t i) {
  return t == KVX_DTYPE_S32 ? (int64_t)((const int32_t *)p)[i] : ((const int64_t *)p)[i];
}

static void *write_worker(void *arg) {
  const job_t *j = (const job_t *)arg;
  const kvx_cache_desc_t *c = j->cache;
  const kvx_write_desc_t *w = j->write;
  const int64_t bs = c->block_size;
  for (int64_t t = j->begin; t < j->end; ++t) {
    const int64_t slot = index_at(w->slots.slots, w->slots.dtype, t);
    if (slot < 0 || slot / bs >= (int64_t)c->num_blocks) continue;
    memcpy((char *)c->k.data + (size_t)slot * j->row_bytes,
           (const char *)w->io.key.data + (size_t)t * j->row_bytes, j->row_bytes);
    memcpy((char *)c->v.data + (size_t)slot * j->row_bytes,
           (const char *)w->io.value.data + (size_t)t * j->row_bytes, j->row_bytes);
  }
  return NULL;
}

static void *gather_worker(void *arg) {
  const job_t *j = (const job_t *)arg;
  const kvx_cache_desc_t *c = j->cache;
  const kvx_gather_desc_t *g = j->gather;
  const int64_t bs = c->block_size, mb = g->block_table.max_blocks_per_seq;
  const int64_t Lmax = g->max_seq_len;
  for (int64_t item = j->begin; item < j->end; ++item) {
    const int64_t s = item / mb, lb = item - s * mb;
    int64_t len = index_at(g->seq_lens.lengths, g->seq_lens.dtype, s);
    if (len > Lmax) len = Lmax;
    const int64_t first = lb * bs;
    if (first >= len) continue;
    const int64_t n = (len - first < bs) ? len - first : bs;
    const int64_t block = index_at(g->block_table.indices, g->block_table.index_dtype, item);
    if (block < 0 || block >= (int64_t)c->num_blocks) continue;
    const size_t src = (size_t)block * bs * j->row_bytes;
    const size_t dst = (size_t)(s * Lmax + first) * j->row_bytes;
    memcpy((char *)g->io.key.data + dst, (const char *)c->k.data + src, (size_t)n * j->row_bytes);
    memcpy((char *)g->io.value.data + dst, (const char *)c->v.data + src, (size_t)n * j->row_bytes);
  }
  return NULL;
}

static void run_split(void *(*fn)(void *), job_t proto, int64_t total, int threads) {
  enum { MAX_T = 512 };
  pthread_t tid[MAX_T];
  job_t jobs[MAX_T];
  if (threads < 1) threads = 1;
  if (threads > MAX_T) threads = MAX_T;
  if (threads == 1) {
    proto.begin = 0;
    proto.end = total;
    fn(&proto);
    return;
  }
  for (int i = 0; i < threads; ++i) {
    jobs[i] = proto;
    jobs[i].begin = total * i / threads;
    jobs[i].end = total * (i + 1) / threads;
    pthread_create(&tid[i], NULL, fn, &jobs[i]);
  }
  for (int i = 0; i < threads; ++i) pthread_join(tid[i], NULL);
}

kvx_status_t kvx_cpu_baseline_write_kv(const kvx_cache_desc_t *cache, const kvx_write_desc_t *write,
                                       int threads) {
  job_t j;
  if (cache == NULL || write == NULL) return KVX_STATUS_INVALID_ARGUMENT;
  if (!nhd_canonical(cache, &cache->k) || !nhd_canonical(cache, &cache->v) ||
      cache->k.dtype != write->io.key.dtype || cache->v.dtype != write->io.value.dtype ||
      cache->k.dtype != cache->v.dtype || elem_size(cache->k.dtype) == 0)
    return KVX_STATUS_UNSUPPORTED;
  memset(&j, 0, sizeof j);
  j.cache = cache;
  j.write = write;
  j.row_bytes = (size_t)cache->num_kv_heads * cache->head_dim * elem_size(cache->k.dtype);
  run_split(write_worker, j, write->io.num_tokens, threads);
  return KVX_STATUS_OK;
}

kvx_status_t kvx_cpu_baseline_gather_kv(const kvx_cache_desc_t *cache,
                                        const kvx_gather_desc_t *gather, int threads) {
  job_t j;
  if (cache == NULL || gather == NULL) return KVX_STATUS_INVALID_ARGUMENT;
  if (!nhd_canonical(cache, &cache->k) || !nhd_canonical(cache, &cache->v) ||
      cache->k.dtype != gather->io.key.dtype || cache->v.dtype != gather->io.value.dtype ||
      cache->k.dtype != cache->v.dtype || elem_size(cache->k.dtype) == 0 ||
      gather->block_table.format != KVX_BLOCK_TABLE_PACKED ||
      gather->block_table.index_dtype != gather->seq_lens.dtype)
    return KVX_STATUS_UNSUPPORTED;
  memset(&j, 0, sizeof j);
  j.cache = cache;
  j.gather = gather;
  j.row_bytes = (size_t)cache->num_kv_heads * cache->head_dim * elem_size(cache->k.dtype);
  run_split(gather_worker, j,
            (int64_t)gather->block_table.seq_count * gather->block_table.max_blocks_per_seq, threads);
  return KVX_STATUS_OK;
}
