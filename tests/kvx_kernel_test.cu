/*
 * kvx_kernel_test: native consumer of the launch ABI (include/kvx_paged_kv.h), C++ calling the
 * library with no Python in between.  Every case builds its inputs on the host, runs the
 * launchers on the device and compares ALL bytes of the page pool and of the gathered outputs
 * (untouched ones included: pools and outputs start from sentinel patterns) with host loops
 * written here, by memcmp.
 *
 * The nine records of the reference's kernel test (tests/kvx_kernel_test.cu:788-813:
 * write / prefill / gather x f32 / f16 / bf16) keep their names and their toy shapes
 * (:161-193, :456-466, :620-627, :629-655, values 0.1 + 0.01 i) and are extended with what
 * that test never exercises: negative and out-of-range slots, ragged lengths, permuted and
 * damaged block tables, HND and HND_PACKED pages (K and V with different pack factors), table
 * widths and max_seq_len that cut sequences short.  Further records cover what the reference
 * only declares: RAGGED block tables, the un-padded gather and the fp8-e4m3 cache (the e4m3
 * conversion is restated below: one IEEE division, one rounding to nearest even, saturating).
 *
 * Prints "<record>: ok|fail" per record on stderr and "kvx_kernel_test passed" on stdout,
 * exit code 1 on any failure -- the reference test's contract.
 */
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <cmath>
#include <random>
#include <string>
#include <vector>

#include "kvx_paged_kv.h"

namespace {

void cuda_ok(cudaError_t e, const char *what) {
  if (e != cudaSuccess) {
    fprintf(stderr, "%s: %s\n", what, cudaGetErrorString(e));
    exit(1);
  }
}

int64_t elem_bytes(kvx_dtype_t t) { return t == KVX_DTYPE_F32 ? 4 : (t == KVX_DTYPE_F8_E4M3 ? 1 : 2); }

// float -> raw bits of the element type, round to nearest even
uint32_t to_bits(float x, kvx_dtype_t t) {
  if (t == KVX_DTYPE_F32) {
    uint32_t b;
    memcpy(&b, &x, 4);
    return b;
  }
  if (t == KVX_DTYPE_F16) return __half_as_ushort(__float2half_rn(x));
  return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}
float from_bits(uint32_t b, kvx_dtype_t t) {
  if (t == KVX_DTYPE_F32) {
    float x;
    memcpy(&x, &b, 4);
    return x;
  }
  if (t == KVX_DTYPE_F16) return __half2float(__ushort_as_half(static_cast<uint16_t>(b)));
  return __bfloat162float(__ushort_as_bfloat16(static_cast<uint16_t>(b)));
}

// ---- e4m3 (1 sign, 4 exponent bits of bias 7, 3 mantissa bits; 0x7F / 0xFF = NaN, no inf) ----
// Nearest even, saturating to +-448; the write is e4m3(RN(x / scale)).
uint8_t e4m3_from_f32(float x) {
  if (std::isnan(x)) return 0x7F;
  const uint8_t sign = std::signbit(x) ? 0x80 : 0x00;
  const float a = std::fabs(x);
  if (a >= 448.0f) return sign | 0x7E;  // everything that would round above the largest finite value
  if (a == 0.0f) return sign;
  int e;
  std::frexp(a, &e);  // a = m * 2^e, m in [0.5, 1)
  int exp2 = std::max(e - 1, -6);                      // exponent of the leading bit, -6 for subnormals
  const float step = std::ldexp(1.0f, exp2 - 3);       // spacing of e4m3 values at this exponent
  const float q = std::nearbyint(a / step) * step;     // ties to even (default rounding mode); exact
  if (q == 0.0f) return sign;
  std::frexp(q, &e);
  exp2 = e - 1;
  if (exp2 < -6) return sign | static_cast<uint8_t>(std::lround(q / std::ldexp(1.0f, -9)));  // subnormal: 1 .. 7
  const int mant = static_cast<int>(std::lround((q / std::ldexp(1.0f, exp2) - 1.0f) * 8.0f));
  return sign | static_cast<uint8_t>(((exp2 + 7) << 3) | mant);
}
float e4m3_to_f32(uint8_t c) {
  const int exp = (c >> 3) & 0xF, mant = c & 7;
  float v;
  if (exp == 0xF && mant == 7)
    v = NAN;
  else if (exp == 0)
    v = std::ldexp(static_cast<float>(mant), -9);
  else
    v = std::ldexp(1.0f + mant / 8.0f, exp - 7);
  return (c & 0x80) ? -v : v;
}

// ---- a case ---------------------------------------------------------------------------

struct Spec {
  const char *name = "";
  kvx_dtype_t io = KVX_DTYPE_F32;
  bool fp8 = false;                 // cache in e4m3, per-head scales
  int layout = 0;                   // 0 NHD, 1 HND, 2 HND_PACKED
  int pack_k = 1, pack_v = 1;       // HND_PACKED pack factors
  int heads = 2, dim = 4, bs = 4, num_blocks = 2;
  std::vector<int> lens = {4, 4};
  int tokens_per_seq = 0;           // > 0: the reference's toy write (last tokens of every sequence, identity table)
  bool prefill = false;             // through kvx_launch_write_kv_prefill
  double pad = 0.0;                 // fraction of slots replaced by negative values
  int oob_slots = 0, bad_blocks = 0;
  int max_seq_len = 0, max_blocks = 0;  // 0: what the lengths need
  bool ragged = false, varlen = false;
  bool toy_values = true;           // 0.1 + 0.01 i (the reference's values) or seeded random bits
  uint64_t seed = 1;
};

struct Layout {
  int kind;
  int64_t bs, heads, dim, pack;
  int64_t offset(int64_t b, int64_t o, int64_t h, int64_t d) const {
    if (kind == 0) return ((b * bs + o) * heads + h) * dim + d;
    if (kind == 1) return ((b * heads + h) * bs + o) * dim + d;
    return (((b * heads + h) * (dim / pack) + d / pack) * bs + o) * pack + d % pack;
  }
};

void describe_pages(kvx_tensor_desc_t *t, const Layout &l, int64_t nb, kvx_dtype_t dtype, void *data) {
  memset(t, 0, sizeof(*t));
  t->size = sizeof(*t), t->dtype = dtype, t->memory = KVX_MEMORY_DEVICE, t->data = data;
  std::vector<int64_t> shape;
  if (l.kind == 0)
    t->layout = KVX_LAYOUT_BLOCK_NHD, shape = {nb, l.bs, l.heads, l.dim};
  else if (l.kind == 1)
    t->layout = KVX_LAYOUT_BLOCK_HND, shape = {nb, l.heads, l.bs, l.dim};
  else
    t->layout = KVX_LAYOUT_BLOCK_HND_PACKED, shape = {nb, l.heads, l.dim / l.pack, l.bs, l.pack};
  t->ndim = static_cast<uint32_t>(shape.size());
  int64_t run = 1;
  for (int i = static_cast<int>(shape.size()) - 1; i >= 0; --i) t->shape[i] = shape[i], t->stride[i] = run, run *= shape[i];
}
void describe_dense(kvx_tensor_desc_t *t, std::vector<int64_t> shape, kvx_dtype_t dtype, void *data) {
  memset(t, 0, sizeof(*t));
  t->size = sizeof(*t), t->dtype = dtype, t->layout = KVX_LAYOUT_BLOCK_CUSTOM, t->memory = KVX_MEMORY_DEVICE;
  t->data = data, t->ndim = static_cast<uint32_t>(shape.size());
  int64_t run = 1;
  for (int i = static_cast<int>(shape.size()) - 1; i >= 0; --i) t->shape[i] = shape[i], t->stride[i] = run, run *= shape[i];
}

template <typename T>
T *to_device(const std::vector<T> &v) {
  T *d = nullptr;
  cuda_ok(cudaMalloc(&d, std::max<size_t>(v.size(), 1) * sizeof(T)), "cudaMalloc");
  if (!v.empty()) cuda_ok(cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice), "cudaMemcpy");
  return d;
}
template <typename T>
void from_device(std::vector<T> *v, const T *d) {
  if (!v->empty()) cuda_ok(cudaMemcpy(v->data(), d, v->size() * sizeof(T), cudaMemcpyDeviceToHost), "cudaMemcpy");
}

bool same(const std::vector<uint8_t> &a, const std::vector<uint8_t> &b, const char *what, const char *name) {
  if (a.size() == b.size() && (a.empty() || memcmp(a.data(), b.data(), a.size()) == 0)) return true;
  size_t at = 0;
  while (at < a.size() && a[at] == b[at]) ++at;
  fprintf(stderr, "  %s: %s differs at byte %zu of %zu\n", name, what, at, a.size());
  return false;
}

bool run_case(const Spec &c) {
  std::mt19937_64 rng(c.seed);
  std::uniform_real_distribution<double> unit(0.0, 1.0);
  const int64_t H = c.heads, D = c.dim, bs = c.bs, nb = c.num_blocks, S = static_cast<int64_t>(c.lens.size());
  const kvx_dtype_t io = c.io, cd = c.fp8 ? KVX_DTYPE_F8_E4M3 : c.io;
  const int64_t e_io = elem_bytes(io), e_c = elem_bytes(cd);
  const Layout lk{c.layout, bs, H, D, c.pack_k}, lv{c.layout, bs, H, D, c.pack_v};

  // pages of the sequences: the identity table for the toy cases, a seeded permutation otherwise
  std::vector<int64_t> need(S);
  int64_t pages = 0, mb = 1, longest = 1;
  for (int64_t s = 0; s < S; ++s) {
    need[s] = (c.lens[s] + bs - 1) / bs;
    pages += need[s], mb = std::max(mb, need[s]), longest = std::max<int64_t>(longest, c.lens[s]);
  }
  if (c.max_blocks > 0) mb = c.max_blocks;
  const int64_t L = c.max_seq_len > 0 ? c.max_seq_len : longest;
  if (pages > nb) {
    fprintf(stderr, "  %s: pool too small\n", c.name);
    return false;
  }
  std::vector<int32_t> perm(nb);
  for (int64_t i = 0; i < nb; ++i) perm[i] = static_cast<int32_t>(i);
  if (c.tokens_per_seq == 0) std::shuffle(perm.begin(), perm.end(), rng);
  std::vector<int32_t> table(static_cast<size_t>(S * mb), -1);
  std::vector<int64_t> slots;
  int64_t next = 0;
  for (int64_t s = 0; s < S; ++s) {
    for (int64_t b = 0; b < need[s] && b < mb; ++b) table[s * mb + b] = perm[next + b];
    const int64_t first = c.tokens_per_seq > 0 ? c.lens[s] - c.tokens_per_seq : 0;
    for (int64_t p = first; p < c.lens[s]; ++p) slots.push_back(static_cast<int64_t>(perm[next + p / bs]) * bs + p % bs);
    next += need[s];
  }
  const int64_t T = static_cast<int64_t>(slots.size());
  for (int64_t t = 0; t < T; ++t)
    if (c.pad > 0 && unit(rng) < c.pad) slots[t] = (t % 3 == 0) ? -1 : -(1 + static_cast<int64_t>(unit(rng) * 1e9));
  for (int i = 0; i < c.oob_slots && T > 0; ++i) slots[(i * 7919) % T] = nb * bs + i * bs + i % bs;
  for (int i = 0; i < c.bad_blocks; ++i) {
    const int64_t s = i % S;
    if (need[s] > 0) table[s * mb + i % std::min(need[s], mb)] = (i % 2 == 0) ? -1 : static_cast<int32_t>(nb + i);
  }

  // inputs
  std::vector<uint8_t> key(static_cast<size_t>(T * H * D * e_io)), value(key.size());
  for (int64_t i = 0; i < T * H * D; ++i) {
    uint32_t a, b;
    if (c.fp8) {  // ordinary magnitudes with a few large ones, so that saturation and subnormals both occur
      const float x = static_cast<float>((unit(rng) - 0.5) * 4.0) * (unit(rng) < 0.01 ? 400.0f : 1.0f);
      const float y = static_cast<float>((unit(rng) - 0.5) * 0.01);
      a = to_bits(x, io), b = to_bits(y, io);
    } else if (c.toy_values) {
      a = to_bits(0.1f + 0.01f * static_cast<float>(i), io), b = to_bits(0.6f + 0.01f * static_cast<float>(i), io);
    } else {  // arbitrary bit patterns: a copy must keep NaN payloads, -0 and denormals as they are
      a = static_cast<uint32_t>(rng()), b = static_cast<uint32_t>(rng());
    }
    memcpy(&key[i * e_io], &a, e_io), memcpy(&value[i * e_io], &b, e_io);
  }
  std::vector<float> k_scale(H), v_scale(H);
  for (int64_t h = 0; h < H; ++h) k_scale[h] = 0.004f + 0.001f * h, v_scale[h] = 0.00002f * (h + 1);

  const size_t pool_bytes = static_cast<size_t>(nb * bs * H * D * e_c);
  const int64_t out_rows = c.varlen ? [&] { int64_t r = 0; for (int64_t s = 0; s < S; ++s) r += std::min<int64_t>(c.lens[s], L); return r + 2; }() : S * L;
  const size_t out_bytes = static_cast<size_t>(out_rows * H * D * e_io);
  std::vector<uint8_t> pool_k(pool_bytes, 0xA5), pool_v(pool_bytes, 0x5A), out_k(out_bytes, 0xC3), out_v(out_bytes, 0x3C);
  std::vector<int32_t> lens32(c.lens.begin(), c.lens.end());
  // RAGGED: one page id per cached token, indptr = prefix sums
  std::vector<int32_t> ragged, indptr = {0}, out_indptr = {0};
  for (int64_t s = 0; s < S; ++s) {
    const int64_t n = std::min<int64_t>(c.lens[s], mb * bs);
    for (int64_t p = 0; p < n; ++p) ragged.push_back(table[s * mb + p / bs]);
    indptr.push_back(static_cast<int32_t>(ragged.size()));
    out_indptr.push_back(out_indptr.back() + static_cast<int32_t>(std::min<int64_t>(c.lens[s], L)));
  }

  // device buffers and descriptors
  uint8_t *d_key = to_device(key), *d_value = to_device(value), *d_pk = to_device(pool_k), *d_pv = to_device(pool_v);
  uint8_t *d_ok = to_device(out_k), *d_ov = to_device(out_v);
  int64_t *d_slots = to_device(slots);
  int32_t *d_table = to_device(c.ragged ? ragged : table), *d_lens = to_device(lens32);
  int32_t *d_indptr = to_device(indptr), *d_out_indptr = to_device(out_indptr);
  float *d_ks = to_device(k_scale), *d_vs = to_device(v_scale);

  kvx_cache_desc_t cache;
  memset(&cache, 0, sizeof(cache));
  cache.size = sizeof(cache), cache.pool.size = sizeof(cache.pool);
  cache.num_blocks = static_cast<uint32_t>(nb), cache.block_size = static_cast<uint32_t>(bs);
  cache.num_kv_heads = static_cast<uint32_t>(H), cache.head_dim = static_cast<uint32_t>(D);
  describe_pages(&cache.k, lk, nb, cd, d_pk);
  describe_pages(&cache.v, lv, nb, cd, d_pv);
  kvx_scale_desc_t ks, vs;
  memset(&ks, 0, sizeof(ks));
  ks.size = sizeof(ks), ks.dtype = KVX_DTYPE_F32;
  vs = ks;
  if (c.fp8) {
    ks.granularity = vs.granularity = KVX_SCALE_PER_HEAD;
    ks.ndim = vs.ndim = 1, ks.shape[0] = vs.shape[0] = H, ks.stride[0] = vs.stride[0] = 1;
    ks.data = d_ks, vs.data = d_vs;
  }
  kvx_write_desc_t w;
  memset(&w, 0, sizeof(w));
  w.size = sizeof(w), w.io.size = sizeof(w.io);
  w.io.num_tokens = static_cast<uint32_t>(T), w.io.num_kv_heads = static_cast<uint32_t>(H), w.io.head_dim = static_cast<uint32_t>(D);
  describe_dense(&w.io.key, {T, H, D}, io, d_key);
  describe_dense(&w.io.value, {T, H, D}, io, d_value);
  w.slots.size = sizeof(w.slots), w.slots.dtype = KVX_DTYPE_S64, w.slots.token_count = static_cast<uint32_t>(T);
  w.slots.invalid_slot = -1, w.slots.slots = d_slots;
  w.k_scale_desc = ks, w.v_scale_desc = vs;
  kvx_gather_desc_t g;
  memset(&g, 0, sizeof(g));
  g.size = sizeof(g), g.io.size = sizeof(g.io);
  g.io.num_tokens = static_cast<uint32_t>(out_rows), g.io.num_kv_heads = static_cast<uint32_t>(H), g.io.head_dim = static_cast<uint32_t>(D);
  if (c.varlen) {
    describe_dense(&g.io.key, {out_rows, H, D}, io, d_ok);
    describe_dense(&g.io.value, {out_rows, H, D}, io, d_ov);
  } else {
    describe_dense(&g.io.key, {S, L, H, D}, io, d_ok);
    describe_dense(&g.io.value, {S, L, H, D}, io, d_ov);
  }
  kvx_block_table_t &bt = g.block_table;
  bt.size = sizeof(bt), bt.index_dtype = KVX_DTYPE_S32, bt.seq_count = static_cast<uint32_t>(S), bt.beam_width = 1;
  bt.max_blocks_per_seq = static_cast<uint32_t>(mb), bt.indices = d_table;
  if (c.ragged) {
    bt.format = KVX_BLOCK_TABLE_RAGGED, bt.indices_count = static_cast<uint32_t>(ragged.size());
    bt.indptr_dtype = KVX_DTYPE_S32, bt.indptr = d_indptr, bt.indptr_count = static_cast<uint32_t>(S + 1);
  } else {
    bt.format = KVX_BLOCK_TABLE_PACKED, bt.indices_count = static_cast<uint32_t>(S * mb);
  }
  g.seq_lens.size = sizeof(g.seq_lens), g.seq_lens.dtype = KVX_DTYPE_S32, g.seq_lens.seq_count = static_cast<uint32_t>(S);
  g.seq_lens.lengths = d_lens;
  g.max_seq_len = static_cast<uint32_t>(L);

  // ---- run ----
  kvx_status_t st = c.prefill ? kvx_launch_write_kv_prefill(&cache, &w, std::max(c.tokens_per_seq, 1), nullptr)
                              : kvx_launch_write_kv(&cache, &w, nullptr);
  bool good = st == KVX_STATUS_OK;
  if (!good) fprintf(stderr, "  %s: write status %d\n", c.name, st);
  cuda_ok(cudaDeviceSynchronize(), "write");
  std::vector<uint8_t> got_k(pool_bytes), got_v(pool_bytes);
  from_device(&got_k, d_pk), from_device(&got_v, d_pv);

  // ---- expected pages: a negative slot and a slot beyond the pool are skipped ----
  std::vector<uint8_t> exp_k = pool_k, exp_v = pool_v;
  for (int64_t t = 0; t < T; ++t) {
    const int64_t sl = slots[t];
    if (sl < 0 || sl / bs >= nb) continue;
    for (int64_t h = 0; h < H; ++h)
      for (int64_t d = 0; d < D; ++d) {
        const size_t from = static_cast<size_t>(((t * H + h) * D + d) * e_io);
        const size_t tk = static_cast<size_t>(lk.offset(sl / bs, sl % bs, h, d) * e_c);
        const size_t tv = static_cast<size_t>(lv.offset(sl / bs, sl % bs, h, d) * e_c);
        if (c.fp8) {
          uint32_t a = 0, b = 0;
          memcpy(&a, &key[from], e_io), memcpy(&b, &value[from], e_io);
          exp_k[tk] = e4m3_from_f32(from_bits(a, io) / k_scale[h]);
          exp_v[tv] = e4m3_from_f32(from_bits(b, io) / v_scale[h]);
        } else {
          memcpy(&exp_k[tk], &key[from], e_c), memcpy(&exp_v[tv], &value[from], e_c);
        }
      }
  }
  good = same(exp_k, got_k, "K pages", c.name) && good;
  good = same(exp_v, got_v, "V pages", c.name) && good;

  if (c.varlen)
    st = kvx_launch_gather_kv_varlen(&cache, &g, d_out_indptr, KVX_DTYPE_S32, &ks, &vs, nullptr);
  else if (c.fp8)
    st = kvx_launch_gather_kv_f8e4m3(&cache, &g, &ks, &vs, nullptr);
  else
    st = kvx_launch_gather_kv(&cache, &g, nullptr);
  if (st != KVX_STATUS_OK) fprintf(stderr, "  %s: gather status %d\n", c.name, st), good = false;
  cuda_ok(cudaDeviceSynchronize(), "gather");
  std::vector<uint8_t> got_ok(out_bytes), got_ov(out_bytes);
  from_device(&got_ok, d_ok), from_device(&got_ov, d_ov);

  // ---- expected outputs: positions below the length whose page id is valid ----
  std::vector<uint8_t> exp_ok = out_k, exp_ov = out_v;
  for (int64_t s = 0; s < S; ++s) {
    const int64_t row0 = c.varlen ? out_indptr[s] : s * L;
    for (int64_t p = 0; p < std::min<int64_t>(c.lens[s], L); ++p) {
      if (p / bs >= mb) continue;
      const int64_t b = table[s * mb + p / bs];
      if (b < 0 || b >= nb) continue;
      for (int64_t h = 0; h < H; ++h)
        for (int64_t d = 0; d < D; ++d) {
          const size_t to = static_cast<size_t>((((row0 + p) * H + h) * D + d) * e_io);
          const size_t fk = static_cast<size_t>(lk.offset(b, p % bs, h, d) * e_c);
          const size_t fv = static_cast<size_t>(lv.offset(b, p % bs, h, d) * e_c);
          if (c.fp8) {
            const uint32_t a = to_bits(e4m3_to_f32(exp_k[fk]) * k_scale[h], io);
            const uint32_t b2 = to_bits(e4m3_to_f32(exp_v[fv]) * v_scale[h], io);
            memcpy(&exp_ok[to], &a, e_io), memcpy(&exp_ov[to], &b2, e_io);
          } else {
            memcpy(&exp_ok[to], &exp_k[fk], e_io), memcpy(&exp_ov[to], &exp_v[fv], e_io);
          }
        }
    }
  }
  good = same(exp_ok, got_ok, "K out", c.name) && good;
  good = same(exp_ov, got_ov, "V out", c.name) && good;

  cudaFree(d_key), cudaFree(d_value), cudaFree(d_pk), cudaFree(d_pv), cudaFree(d_ok), cudaFree(d_ov), cudaFree(d_slots);
  cudaFree(d_table), cudaFree(d_lens), cudaFree(d_indptr), cudaFree(d_out_indptr), cudaFree(d_ks), cudaFree(d_vs);
  return good;
}

// The reference's toy write: 2 sequences of 4 tokens, pages of 4, the last tokens_per_seq
// tokens of each written (tests/kvx_kernel_test.cu:161-193; HND variant :311-343).
Spec toy(kvx_dtype_t t, int heads, int dim, int tps, int layout, bool prefill) {
  Spec c;
  c.name = "toy", c.io = t, c.layout = layout, c.heads = heads, c.dim = dim, c.tokens_per_seq = tps, c.prefill = prefill;
  return c;
}

// What the reference's cases leave out, for one element type.
std::vector<Spec> extended(kvx_dtype_t t, uint64_t seed) {
  std::vector<Spec> v;
  auto add = [&](const char *name, auto &&fill) {
    Spec c;
    c.name = name, c.io = t, c.toy_values = false, c.seed = seed + v.size();
    fill(c);
    v.push_back(c);
  };
  const int x = static_cast<int>(16 / elem_bytes(t));  // elements of a 16-byte pack group
  add("ragged lengths, padded and out-of-range slots", [&](Spec &c) {
    c.heads = 8, c.dim = 128, c.bs = 16, c.num_blocks = 96, c.lens = {300, 77, 512, 9, 0, 130}, c.pad = 0.1, c.oob_slots = 3;
  });
  add("damaged block table, narrow table, short max_seq_len", [&](Spec &c) {
    c.heads = 2, c.dim = 64, c.bs = 8, c.num_blocks = 64, c.lens = {50, 70, 33}, c.bad_blocks = 3, c.max_seq_len = 40, c.max_blocks = 6;
  });
  add("odd head_dim, nothing a power of two", [&](Spec &c) {
    c.heads = 3, c.dim = 7, c.bs = 5, c.num_blocks = 40, c.lens = {11, 5, 0, 3, 29}, c.pad = 0.2;
  });
  add("HND pages", [&](Spec &c) {
    c.layout = 1, c.heads = 8, c.dim = 128, c.bs = 16, c.num_blocks = 64, c.lens = {100, 17, 256, 1}, c.pad = 0.1, c.bad_blocks = 2;
  });
  add("HND_PACKED pages, 16-byte pack groups", [&](Spec &c) {
    c.layout = 2, c.pack_k = c.pack_v = x, c.heads = 8, c.dim = 128, c.bs = 16, c.num_blocks = 64, c.lens = {100, 17, 256, 1}, c.pad = 0.1;
  });
  add("HND_PACKED pages, K packed and V [blocks, heads, dim, block_size]", [&](Spec &c) {
    c.layout = 2, c.pack_k = x, c.pack_v = 1, c.heads = 4, c.dim = 64, c.bs = 32, c.num_blocks = 24, c.lens = {64, 1, 200}, c.bad_blocks = 2;
  });
  add("HND_PACKED pages, small pack, page size that no vector tier takes", [&](Spec &c) {
    c.layout = 2, c.pack_k = c.pack_v = 2, c.heads = 2, c.dim = 20, c.bs = 5, c.num_blocks = 16, c.lens = {13, 9};
  });
  return v;
}

bool run_all(const std::vector<Spec> &cases) {
  bool ok = true;
  for (const Spec &c : cases) {
    const bool good = run_case(c);
    if (!good) fprintf(stderr, "  case failed: %s\n", c.name);
    ok = ok && good;
  }
  return ok;
}

bool write_record(kvx_dtype_t t, bool prefill) {
  std::vector<Spec> cases;
  if (!prefill) {  // tests/kvx_kernel_test.cu:456-466
    cases = {toy(t, 2, 4, 1, 0, false), toy(t, 1, 7, 1, 0, false), toy(t, 2, 4, 2, 0, false), toy(t, 2, 4, 1, 1, false),
             toy(t, 1, 7, 2, 1, false)};
  } else {  // :620-627
    cases = {toy(t, 2, 4, 2, 0, true), toy(t, 1, 7, 2, 0, true)};
  }
  bool ok = run_all(cases);
  for (Spec c : extended(t, prefill ? 500 : 100)) {
    c.prefill = prefill;
    c.tokens_per_seq = 0;
    ok = run_case(c) && ok;
  }
  if (prefill) {  // tokens_per_seq <= 0 is refused before anything else (:607-618)
    kvx_cache_desc_t cache;
    kvx_write_desc_t w;
    memset(&cache, 0, sizeof(cache)), memset(&w, 0, sizeof(w));
    cache.k.dtype = cache.v.dtype = t;
    ok = kvx_launch_write_kv_prefill(&cache, &w, 0, nullptr) == KVX_STATUS_INVALID_ARGUMENT && ok;
  }
  return ok;
}

bool gather_record(kvx_dtype_t t) {
  // the reference's gather case (:629-655): identity table, two full sequences of one page;
  // nothing is written first (tokens_per_seq keeps the identity table, lens 4 -> the write covers
  // the pages, which the gather then reads back)
  Spec c = toy(t, 2, 4, 4, 0, false);
  bool ok = run_case(c);
  for (const Spec &e : extended(t, 900)) ok = run_case(e) && ok;
  return ok;
}

}  // namespace

int main() {
  int devices = 0;
  cuda_ok(cudaGetDeviceCount(&devices), "cudaGetDeviceCount");
  bool ok = true;
  auto record = [&](const char *name, bool result) {
    fprintf(stderr, "%s: %s\n", name, result ? "ok" : "fail");
    ok &= result;
  };
  record("write_f32", write_record(KVX_DTYPE_F32, false));
  record("write_f16", write_record(KVX_DTYPE_F16, false));
  record("write_bf16", write_record(KVX_DTYPE_BF16, false));
  record("prefill_f32", write_record(KVX_DTYPE_F32, true));
  record("prefill_f16", write_record(KVX_DTYPE_F16, true));
  record("prefill_bf16", write_record(KVX_DTYPE_BF16, true));
  record("gather_f32", gather_record(KVX_DTYPE_F32));
  record("gather_f16", gather_record(KVX_DTYPE_F16));
  record("gather_bf16", gather_record(KVX_DTYPE_BF16));

  // beyond the reference's records
  {
    bool good = true;
    for (kvx_dtype_t t : {KVX_DTYPE_BF16, KVX_DTYPE_F32}) {
      Spec c;
      c.name = "RAGGED table", c.io = t, c.toy_values = false, c.ragged = true, c.seed = 41;
      c.heads = 8, c.dim = 128, c.bs = 16, c.num_blocks = 60, c.lens = {100, 17, 256, 1, 0, 333}, c.bad_blocks = 3;
      good = run_case(c) && good;
      c.name = "un-padded output", c.ragged = false, c.varlen = true, c.seed = 42;
      good = run_case(c) && good;
      c.name = "RAGGED table, un-padded output, odd head_dim", c.ragged = true, c.heads = 1, c.dim = 7, c.bs = 4, c.num_blocks = 200;
      good = run_case(c) && good;
    }
    record("ragged_and_unpadded", good);
  }
  {
    bool good = true;
    for (kvx_dtype_t t : {KVX_DTYPE_BF16, KVX_DTYPE_F16, KVX_DTYPE_F32}) {
      Spec c;
      c.name = "fp8-e4m3 cache", c.io = t, c.fp8 = true, c.seed = 77;
      c.heads = 16, c.dim = 256, c.bs = 64, c.num_blocks = 12, c.lens = {200, 64, 130, 1}, c.pad = 0.05;
      good = run_case(c) && good;
      c.name = "fp8-e4m3 cache, HND, small shapes", c.layout = 1, c.heads = 3, c.dim = 24, c.bs = 8, c.num_blocks = 20;
      c.lens = {50, 70, 9}, c.max_seq_len = 60;
      good = run_case(c) && good;
    }
    record("fp8_e4m3", good);
  }
  if (!ok) {
    fprintf(stderr, "kvx_kernel_test failed\n");
    return 1;
  }
  printf("kvx_kernel_test passed\n");
  return 0;
}
