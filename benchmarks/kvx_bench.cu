/*
 * kvx_bench: micro-benchmark of the paged KV write / gather launchers, a C++ host program
 * over the C ABI (include/kvx_paged_kv.h) and nothing else.
 *
 * It keeps the command line and the CSV lines of the reference's benchmark program
 * (benchmarks/kvx_bench.cu:12-37 defaults, :92-126 flags, :544-558 output; the format is
 * what benchmarks/fair_bench.py:120-146 and benchmarks/tests/kvx_bench_cli_test.py parse):
 *
 *   --seq-count N --seq-len N --tokens-per-seq N --block-size N --num-heads N --head-dim N
 *   --warmup N --iters N --dtype float32|float16|bfloat16        (also as --flag=value)
 *
 * and, without further flags, runs the reference's workload: every sequence owns consecutive
 * pages, the last tokens-per-seq tokens of each are written, the full sequences are gathered.
 * Added here:
 *
 *   --config c1..c5   one of the five benchmark configurations (ragged seeded lengths, pages
 *                     taken from a seeded permutation of the pool, padded slots, fp8 for c5)
 *   --gpus N          the cache sharded by KV head over N devices of this box, one host thread
 *                     per device, a host barrier in front of the timed region, the time of the
 *                     slowest device counted
 *   --layers N        page tensors the launches rotate over (every layer its own pages)
 *   --layout nhd|hnd|packed|paged
 *   --pad-frac F --seed N --pool-blocks N --peak-gbs X --check
 *
 * Output: the reference's two human-readable lines, then its CSV header and its `write,` and
 * `gather,` lines with columns appended (the first 13 keep their meaning: gb_per_s counts
 * 2^30 bytes and four element moves per element, as the reference does):
 *   dtype, layout, gpus, layers, valid_tokens, bytes, gbs, pct_of_8000, pct_of_peak, checked
 * where bytes = algorithmic bytes of one launch on all devices (rows read + rows written +
 * index metadata), gbs = bytes / time in 10^9 bytes per second, pct_of_peak = gbs per device
 * against --peak-gbs (the measured copy bandwidth of the device; empty when not given) and
 * checked = 1 when --check compared every byte of the last layer with host loops.
 */
#include <cuda_runtime.h>
#include <pthread.h>
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

struct Options {
  int32_t seq_count = 8, seq_len = 128, tokens_per_seq = 1, block_size = 16, num_heads = 8, head_dim = 128;
  int32_t warmup = 10, iters = 50;
  kvx_dtype_t dtype = KVX_DTYPE_F32;
  std::string dtype_name = "float32";
  std::string config;           // "" = the reference's workload
  std::string layout = "nhd";
  int32_t gpus = 1, layers = 1;
  double pad_frac = -1.0;       // < 0: the configuration's own
  uint64_t seed = 0x4B5658;
  int64_t pool_blocks = 0;      // 0: the configuration's own
  double peak_gbs = 0.0;
  bool check = false;
  bool fp8 = false;             // cache in e4m3 (c5)
};

[[noreturn]] void die(const char *what) {
  fprintf(stderr, "%s\n", what);
  exit(1);
}

void cuda_ok(cudaError_t e, const char *what) {
  if (e != cudaSuccess) {
    fprintf(stderr, "%s: %s\n", what, cudaGetErrorString(e));
    exit(1);
  }
}

// "--name value" or "--name=value"; returns the value or NULL when `arg` is another flag.
const char *flag_value(const char *name, int argc, char **argv, int *i) {
  const size_t n = strlen(name);
  const char *arg = argv[*i];
  if (strncmp(arg, name, n) != 0) return nullptr;
  if (arg[n] == '=') return arg + n + 1;
  if (arg[n] == '\0' && *i + 1 < argc) return argv[++*i];
  return nullptr;
}

Options parse(int argc, char **argv) {
  Options o;
  struct IntFlag {
    const char *name;
    int32_t *dst;
  } ints[] = {{"--seq-count", &o.seq_count}, {"--seq-len", &o.seq_len}, {"--tokens-per-seq", &o.tokens_per_seq},
              {"--block-size", &o.block_size}, {"--num-heads", &o.num_heads}, {"--head-dim", &o.head_dim},
              {"--warmup", &o.warmup}, {"--iters", &o.iters}, {"--gpus", &o.gpus}, {"--layers", &o.layers}};
  for (int i = 1; i < argc; ++i) {
    bool taken = false;
    for (IntFlag &f : ints) {
      if (const char *v = flag_value(f.name, argc, argv, &i)) {
        *f.dst = atoi(v);
        taken = true;
        break;
      }
    }
    if (taken) continue;
    if (const char *v = flag_value("--dtype", argc, argv, &i)) {
      o.dtype_name = v;
      if (o.dtype_name == "float32")
        o.dtype = KVX_DTYPE_F32;
      else if (o.dtype_name == "float16")
        o.dtype = KVX_DTYPE_F16;
      else if (o.dtype_name == "bfloat16")
        o.dtype = KVX_DTYPE_BF16;
      else {
        fprintf(stderr, "Unsupported --dtype=%s\n", v);
        exit(1);
      }
    } else if (const char *v = flag_value("--config", argc, argv, &i)) {
      o.config = v;
    } else if (const char *v = flag_value("--layout", argc, argv, &i)) {
      o.layout = v;
    } else if (const char *v = flag_value("--pad-frac", argc, argv, &i)) {
      o.pad_frac = atof(v);
    } else if (const char *v = flag_value("--seed", argc, argv, &i)) {
      o.seed = strtoull(v, nullptr, 0);
    } else if (const char *v = flag_value("--pool-blocks", argc, argv, &i)) {
      o.pool_blocks = atoll(v);
    } else if (const char *v = flag_value("--peak-gbs", argc, argv, &i)) {
      o.peak_gbs = atof(v);
    } else if (strcmp(argv[i], "--check") == 0) {
      o.check = true;
    }
  }
  return o;
}

// ---------------------------------------------------------------------- workload ------

struct Workload {
  int32_t seqs = 0, heads = 0, dim = 0, block_size = 0, max_blocks = 0, max_seq_len = 0;
  int64_t num_blocks = 0;
  std::vector<int32_t> lens, table;  // table [seqs, max_blocks], -1 = unused
  std::vector<int64_t> slots;        // [T], -1 = padding
  int64_t valid = 0, gathered = 0, pages = 0;
  int64_t tokens() const { return static_cast<int64_t>(slots.size()); }
};

// The reference's own workload (benchmarks/kvx_bench.cu:214-250): sequence s owns pages
// s * max_blocks .. , the write covers the last tokens_per_seq positions of every sequence.
Workload reference_workload(const Options &o) {
  Workload w;
  w.seqs = o.seq_count, w.heads = o.num_heads, w.dim = o.head_dim, w.block_size = o.block_size;
  w.max_blocks = (o.seq_len + o.block_size - 1) / o.block_size;
  w.max_seq_len = o.seq_len;
  w.num_blocks = static_cast<int64_t>(o.seq_count) * w.max_blocks;
  w.lens.assign(o.seq_count, o.seq_len);
  w.table.resize(static_cast<size_t>(o.seq_count) * w.max_blocks);
  for (size_t i = 0; i < w.table.size(); ++i) w.table[i] = static_cast<int32_t>(i);
  for (int32_t s = 0; s < o.seq_count; ++s)
    for (int32_t t = 0; t < o.tokens_per_seq; ++t) {
      const int32_t pos = o.seq_len - o.tokens_per_seq + t;
      w.slots.push_back((static_cast<int64_t>(s) * w.max_blocks + pos / o.block_size) * o.block_size + pos % o.block_size);
    }
  w.valid = w.tokens();
  w.gathered = static_cast<int64_t>(o.seq_count) * o.seq_len;
  w.pages = w.num_blocks;
  return w;
}

struct Preset {
  const char *name, *dtype;
  int32_t heads, dim, block_size, seqs, len_lo, len_hi;
  bool log_uniform, decode, fp8;
  double pad_frac;
  int64_t pool_blocks;  // 0 = twice the pages the sequences need
};
const Preset kPresets[] = {
    {"c1", "float16", 4, 64, 16, 8, 128, 128, false, false, false, 0.0, 512},
    {"c2", "bfloat16", 8, 128, 16, 64, 512, 4096, false, false, false, 0.10, 71525},
    {"c3", "bfloat16", 8, 128, 32, 512, 1, 32768, true, true, false, 0.0, 0},
    {"c4", "float16", 8, 128, 16, 32, 8192, 8192, false, false, false, 0.0, 0},
    {"c5", "bfloat16", 16, 256, 64, 128, 2048, 2048, false, false, true, 0.0, 0},
};

// One of the five configurations: seeded lengths, pages from a seeded permutation of the
// pool, prefill slots in sequence order (or one new token per sequence for the decode step),
// a fraction of the slots replaced by -1.
Workload preset_workload(Options *o) {
  const Preset *p = nullptr;
  for (const Preset &c : kPresets)
    if (o->config == c.name) p = &c;
  if (p == nullptr) die("unknown --config (c1 .. c5)");
  o->dtype_name = p->dtype;
  o->dtype = strcmp(p->dtype, "float16") == 0 ? KVX_DTYPE_F16 : KVX_DTYPE_BF16;
  o->num_heads = p->heads, o->head_dim = p->dim, o->block_size = p->block_size, o->seq_count = p->seqs;
  o->fp8 = p->fp8;
  const double pad = o->pad_frac >= 0 ? o->pad_frac : p->pad_frac;
  std::mt19937_64 rng(o->seed + static_cast<uint64_t>(p - kPresets));
  Workload w;
  w.seqs = p->seqs, w.heads = p->heads, w.dim = p->dim, w.block_size = p->block_size;
  std::uniform_real_distribution<double> unit(0.0, 1.0);
  for (int32_t s = 0; s < p->seqs; ++s) {
    int64_t len;
    if (p->log_uniform)
      len = std::llround(std::exp(unit(rng) * std::log(static_cast<double>(p->len_hi))));
    else
      len = p->len_lo + static_cast<int64_t>(unit(rng) * (p->len_hi - p->len_lo + 1));
    w.lens.push_back(static_cast<int32_t>(std::min<int64_t>(std::max<int64_t>(len, p->len_lo), p->len_hi)));
  }
  std::vector<int64_t> need(p->seqs);
  for (int32_t s = 0; s < p->seqs; ++s) {
    need[s] = (w.lens[s] + p->block_size - 1) / p->block_size;
    w.pages += need[s];
    w.gathered += w.lens[s];
    w.max_blocks = std::max<int32_t>(w.max_blocks, static_cast<int32_t>(need[s]));
    w.max_seq_len = std::max(w.max_seq_len, w.lens[s]);
  }
  w.num_blocks = o->pool_blocks > 0 ? o->pool_blocks : (p->pool_blocks > 0 ? p->pool_blocks : 2 * w.pages);
  w.num_blocks = std::max(w.num_blocks, w.pages);
  // the first `pages` entries of a random permutation of the pool (partial Fisher-Yates)
  std::vector<int32_t> perm(w.num_blocks);
  for (int64_t i = 0; i < w.num_blocks; ++i) perm[i] = static_cast<int32_t>(i);
  for (int64_t i = 0; i < w.pages; ++i) {
    const int64_t j = i + static_cast<int64_t>(unit(rng) * (w.num_blocks - i));
    std::swap(perm[i], perm[std::min(j, w.num_blocks - 1)]);
  }
  w.table.assign(static_cast<size_t>(p->seqs) * w.max_blocks, -1);
  int64_t next = 0;
  for (int32_t s = 0; s < p->seqs; ++s) {
    for (int64_t b = 0; b < need[s]; ++b) w.table[static_cast<size_t>(s) * w.max_blocks + b] = perm[next + b];
    if (p->decode) {
      const int32_t pos = w.lens[s] - 1;
      w.slots.push_back(static_cast<int64_t>(perm[next + pos / p->block_size]) * p->block_size + pos % p->block_size);
    } else {
      for (int32_t pos = 0; pos < w.lens[s]; ++pos)
        w.slots.push_back(static_cast<int64_t>(perm[next + pos / p->block_size]) * p->block_size + pos % p->block_size);
    }
    next += need[s];
  }
  for (int64_t &sl : w.slots)
    if (pad > 0 && unit(rng) < pad) sl = -1;
  for (int64_t sl : w.slots) w.valid += sl >= 0;
  o->seq_len = w.max_seq_len;
  o->tokens_per_seq = p->decode ? 1 : w.max_seq_len;
  return w;
}

int64_t elem_bytes(kvx_dtype_t t) { return t == KVX_DTYPE_F32 ? 4 : (t == KVX_DTYPE_F8_E4M3 ? 1 : 2); }

// ---------------------------------------------------------------------- page layouts --

// Element offset of (block, token in block, head, dim) in a page tensor of `heads` heads.
struct PageLayout {
  std::string name;
  int64_t bs, heads, dim, pack;  // pack > 0: HND_PACKED with that pack factor
  int64_t offset(int64_t b, int64_t o, int64_t h, int64_t d) const {
    if (name == "nhd") return ((b * bs + o) * heads + h) * dim + d;
    if (pack == 0) return ((b * heads + h) * bs + o) * dim + d;
    return (((b * heads + h) * (dim / pack) + d / pack) * bs + o) * pack + d % pack;
  }
};

void describe_pages(kvx_tensor_desc_t *t, const PageLayout &l, int64_t num_blocks, kvx_dtype_t dtype, void *data) {
  memset(t, 0, sizeof(*t));
  t->size = sizeof(*t);
  t->dtype = dtype;
  t->memory = KVX_MEMORY_DEVICE;
  t->data = data;
  int64_t shape[5];
  if (l.name == "nhd") {
    t->layout = KVX_LAYOUT_BLOCK_NHD, t->ndim = 4;
    shape[0] = num_blocks, shape[1] = l.bs, shape[2] = l.heads, shape[3] = l.dim;
  } else if (l.pack == 0) {
    t->layout = KVX_LAYOUT_BLOCK_HND, t->ndim = 4;
    shape[0] = num_blocks, shape[1] = l.heads, shape[2] = l.bs, shape[3] = l.dim;
  } else {
    t->layout = KVX_LAYOUT_BLOCK_HND_PACKED, t->ndim = 5;
    shape[0] = num_blocks, shape[1] = l.heads, shape[2] = l.dim / l.pack, shape[3] = l.bs, shape[4] = l.pack;
  }
  int64_t run = 1;
  for (int i = static_cast<int>(t->ndim) - 1; i >= 0; --i) {
    t->shape[i] = shape[i];
    t->stride[i] = run;
    run *= shape[i];
  }
}

void describe_dense(kvx_tensor_desc_t *t, std::initializer_list<int64_t> shape, kvx_dtype_t dtype, void *data) {
  memset(t, 0, sizeof(*t));
  t->size = sizeof(*t);
  t->dtype = dtype;
  t->layout = KVX_LAYOUT_BLOCK_CUSTOM;
  t->memory = KVX_MEMORY_DEVICE;
  t->ndim = static_cast<uint32_t>(shape.size());
  t->data = data;
  int i = 0;
  for (int64_t n : shape) t->shape[i++] = n;
  int64_t run = 1;
  for (int k = static_cast<int>(t->ndim) - 1; k >= 0; --k) {
    t->stride[k] = run;
    run *= t->shape[k];
  }
}

// ---------------------------------------------------------------------- one device ----

constexpr uint8_t kPoolFill = 0x5A, kOutFill = 0xC3;

struct Shared {  // what the per-device threads share
  const Options *opt;
  const Workload *wl;
  pthread_barrier_t barrier;
  std::vector<double> write_ms, gather_ms;  // per device, per launch
  std::vector<int> checked;                 // per device: 1 ok, 0 not asked, -1 failed
};

struct Device {
  Shared *sh;
  int rank;
};

// Deterministic element bits: a cheap hash of the global element index, so that every device
// draws its own heads' slice of one global K (or V) tensor.
__host__ __device__ inline uint32_t element_bits(uint64_t index, uint64_t salt) {
  uint64_t z = (index + salt) * 0x9E3779B97F4A7C15ull;
  z ^= z >> 29;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 32;
  return static_cast<uint32_t>(z);
}

// bf16 bits of a roughly normal value (sum of four uniforms), times 50 for one element in a
// thousand: the fp8 configuration's input distribution.
__host__ __device__ inline uint16_t normal_bf16(uint64_t index, uint64_t salt) {
  const uint32_t a = element_bits(index, salt), b = element_bits(index, salt + 0x51ED);
  const float u = ((a & 0xFFFF) + (a >> 16) + (b & 0xFFFF) + (b >> 16)) / 65536.0f - 2.0f;  // var 1/3
  float x = u * 1.7320508f;
  if ((element_bits(index, salt + 0xABCD) % 1000u) == 0u) x *= 50.0f;
  uint32_t bits;
  memcpy(&bits, &x, 4);
  return static_cast<uint16_t>((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
}

// Fills one device's [tokens, heads, dim] slice (heads h0 .. h0 + heads of `heads_global`) of
// the global K (salt 1) or V (salt 2) tensor.  The benchmark's own set-up, not library code.
__global__ void fill_inputs_kernel(uint8_t *out, int64_t elems, int64_t heads, int64_t h0, int64_t heads_global,
                                   int64_t dim, int elem, uint64_t salt, int normal) {
  const int64_t at = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (at >= elems) return;
  const int64_t d = at % dim, h = (at / dim) % heads, t = at / (dim * heads);
  const uint64_t g = (static_cast<uint64_t>(t) * heads_global + (h0 + h)) * dim + d;
  if (normal) {
    reinterpret_cast<uint16_t *>(out)[at] = normal_bf16(g, salt);
  } else if (elem == 4) {
    reinterpret_cast<uint32_t *>(out)[at] = element_bits(g, salt);
  } else {
    reinterpret_cast<uint16_t *>(out)[at] = static_cast<uint16_t>(element_bits(g, salt));
  }
}

void *device_main(void *arg) {
  Device *me = static_cast<Device *>(arg);
  Shared *sh = me->sh;
  const Options &o = *sh->opt;
  const Workload &w = *sh->wl;
  const int rank = me->rank;
  cuda_ok(cudaSetDevice(rank), "cudaSetDevice");
  const int64_t H = w.heads / o.gpus, h0 = rank * H, D = w.dim, bs = w.block_size;
  const kvx_dtype_t io = o.dtype, cd = o.fp8 ? KVX_DTYPE_F8_E4M3 : o.dtype;
  const int64_t e_io = elem_bytes(io), e_c = elem_bytes(cd);
  const int64_t T = w.tokens(), S = w.seqs, L = w.max_seq_len;
  const int64_t row_io = H * D * e_io;
  const int64_t pack16 = 16 / e_c;
  PageLayout lk{o.layout, bs, H, D, 0}, lv = lk;
  if (o.layout == "packed") lk.pack = lv.pack = pack16;
  if (o.layout == "paged") lk.pack = pack16, lv.pack = 1;

  const size_t in_bytes = static_cast<size_t>(T * row_io);
  const size_t tensor_bytes = static_cast<size_t>(w.num_blocks * bs * H * D * e_c);
  const size_t out_bytes = static_cast<size_t>(S * L * row_io);
  char *d_key, *d_value, *d_ok, *d_ov, *d_slots, *d_table, *d_lens;
  std::vector<char *> d_k(o.layers), d_v(o.layers);
  cuda_ok(cudaMalloc(&d_key, in_bytes), "cudaMalloc key");
  cuda_ok(cudaMalloc(&d_value, in_bytes), "cudaMalloc value");
  cuda_ok(cudaMalloc(&d_ok, out_bytes), "cudaMalloc key_out");
  cuda_ok(cudaMalloc(&d_ov, out_bytes), "cudaMalloc value_out");
  cuda_ok(cudaMalloc(&d_slots, T * 8), "cudaMalloc slots");
  cuda_ok(cudaMalloc(&d_table, w.table.size() * 4), "cudaMalloc block_table");
  cuda_ok(cudaMalloc(&d_lens, S * 4), "cudaMalloc seq_lens");
  for (int l = 0; l < o.layers; ++l) {
    cuda_ok(cudaMalloc(&d_k[l], tensor_bytes), "cudaMalloc key_cache");
    cuda_ok(cudaMalloc(&d_v[l], tensor_bytes), "cudaMalloc value_cache");
    cuda_ok(cudaMemset(d_k[l], kPoolFill, tensor_bytes), "cudaMemset");
    cuda_ok(cudaMemset(d_v[l], kPoolFill, tensor_bytes), "cudaMemset");
  }
  cuda_ok(cudaMemset(d_ok, kOutFill, out_bytes), "cudaMemset");
  cuda_ok(cudaMemset(d_ov, kOutFill, out_bytes), "cudaMemset");
  {  // inputs: this device's heads of the global tensors, drawn on the device
    const int64_t elems = T * H * D;
    const unsigned blocks = static_cast<unsigned>((elems + 255) / 256);
    fill_inputs_kernel<<<blocks, 256>>>(reinterpret_cast<uint8_t *>(d_key), elems, H, h0, w.heads, D,
                                        static_cast<int>(e_io), 1, o.fp8 ? 1 : 0);
    fill_inputs_kernel<<<blocks, 256>>>(reinterpret_cast<uint8_t *>(d_value), elems, H, h0, w.heads, D,
                                        static_cast<int>(e_io), 2, o.fp8 ? 1 : 0);
    cuda_ok(cudaDeviceSynchronize(), "input fill");
  }
  cuda_ok(cudaMemcpy(d_slots, w.slots.data(), T * 8, cudaMemcpyHostToDevice), "cudaMemcpy slots");
  cuda_ok(cudaMemcpy(d_table, w.table.data(), w.table.size() * 4, cudaMemcpyHostToDevice), "cudaMemcpy table");
  cuda_ok(cudaMemcpy(d_lens, w.lens.data(), S * 4, cudaMemcpyHostToDevice), "cudaMemcpy lens");

  cudaStream_t stream;
  cuda_ok(cudaStreamCreate(&stream), "cudaStreamCreate");

  std::vector<kvx_cache_desc_t> caches(o.layers);
  for (int l = 0; l < o.layers; ++l) {
    kvx_cache_desc_t &c = caches[l];
    memset(&c, 0, sizeof(c));
    c.size = sizeof(c);
    c.num_blocks = static_cast<uint32_t>(w.num_blocks), c.block_size = static_cast<uint32_t>(bs);
    c.num_kv_heads = static_cast<uint32_t>(H), c.head_dim = static_cast<uint32_t>(D);
    describe_pages(&c.k, lk, w.num_blocks, cd, d_k[l]);
    describe_pages(&c.v, lv, w.num_blocks, cd, d_v[l]);
    c.pool.size = sizeof(c.pool);
  }
  kvx_write_desc_t wd;
  memset(&wd, 0, sizeof(wd));
  wd.size = sizeof(wd), wd.io.size = sizeof(wd.io);
  wd.io.num_tokens = static_cast<uint32_t>(T), wd.io.num_kv_heads = static_cast<uint32_t>(H);
  wd.io.head_dim = static_cast<uint32_t>(D);
  describe_dense(&wd.io.key, {T, H, D}, io, d_key);
  describe_dense(&wd.io.value, {T, H, D}, io, d_value);
  wd.slots.size = sizeof(wd.slots), wd.slots.dtype = KVX_DTYPE_S64;
  wd.slots.token_count = static_cast<uint32_t>(T), wd.slots.invalid_slot = -1, wd.slots.slots = d_slots;
  wd.k_scale_desc.size = wd.v_scale_desc.size = sizeof(kvx_scale_desc_t);
  wd.k_scale_desc.dtype = wd.v_scale_desc.dtype = KVX_DTYPE_F32;
  kvx_gather_desc_t gd;
  memset(&gd, 0, sizeof(gd));
  gd.size = sizeof(gd), gd.io.size = sizeof(gd.io);
  gd.io.num_tokens = static_cast<uint32_t>(S * L), gd.io.num_kv_heads = static_cast<uint32_t>(H);
  gd.io.head_dim = static_cast<uint32_t>(D);
  describe_dense(&gd.io.key, {S, L, H, D}, io, d_ok);
  describe_dense(&gd.io.value, {S, L, H, D}, io, d_ov);
  gd.block_table.size = sizeof(gd.block_table), gd.block_table.format = KVX_BLOCK_TABLE_PACKED;
  gd.block_table.index_dtype = KVX_DTYPE_S32, gd.block_table.seq_count = static_cast<uint32_t>(S);
  gd.block_table.beam_width = 1, gd.block_table.max_blocks_per_seq = static_cast<uint32_t>(w.max_blocks);
  gd.block_table.indices = d_table, gd.block_table.indices_count = static_cast<uint32_t>(w.table.size());
  gd.seq_lens.size = sizeof(gd.seq_lens), gd.seq_lens.dtype = KVX_DTYPE_S32;
  gd.seq_lens.seq_count = static_cast<uint32_t>(S), gd.seq_lens.lengths = d_lens;
  gd.max_seq_len = static_cast<uint32_t>(L);

  // fp8: per-head scales = absmax / 448 of this batch, by the library's reduction
  float *d_scales = nullptr;
  void *d_work = nullptr;
  kvx_scale_desc_t ks, vs;
  memset(&ks, 0, sizeof(ks));
  ks.size = sizeof(ks), ks.dtype = KVX_DTYPE_F32;
  vs = ks;
  if (o.fp8) {
    const size_t need = kvx_kv_scales_workspace_bytes(static_cast<uint32_t>(H));
    cuda_ok(cudaMalloc(&d_scales, 2 * H * sizeof(float)), "cudaMalloc scales");
    cuda_ok(cudaMalloc(&d_work, need), "cudaMalloc workspace");
    cuda_ok(cudaMemset(d_work, 0, need), "cudaMemset");
    if (kvx_launch_kv_scales(&wd.io, KVX_SCALE_PER_HEAD, d_scales, d_scales + H, d_work, need, stream) != KVX_STATUS_OK)
      die("kvx_launch_kv_scales failed");
    for (kvx_scale_desc_t *d : {&ks, &vs}) {
      d->granularity = KVX_SCALE_PER_HEAD, d->ndim = 1, d->shape[0] = H, d->stride[0] = 1;
    }
    ks.data = d_scales, vs.data = d_scales + H;
    wd.k_scale_desc = ks, wd.v_scale_desc = vs;
  }

  auto write_all = [&]() {
    for (int l = 0; l < o.layers; ++l)
      if (kvx_launch_write_kv(&caches[l], &wd, stream) != KVX_STATUS_OK) die("kvx_launch_write_kv failed");
  };
  auto gather_all = [&]() {
    for (int l = 0; l < o.layers; ++l) {
      const kvx_status_t st = o.fp8 ? kvx_launch_gather_kv_f8e4m3(&caches[l], &gd, &ks, &vs, stream)
                                    : kvx_launch_gather_kv(&caches[l], &gd, stream);
      if (st != KVX_STATUS_OK) die("kvx_launch_gather_kv failed");
    }
  };
  auto timed = [&](auto &&run) {
    cudaEvent_t a, b;
    cuda_ok(cudaEventCreate(&a), "cudaEventCreate");
    cuda_ok(cudaEventCreate(&b), "cudaEventCreate");
    for (int i = 0; i < o.warmup; ++i) run();
    cuda_ok(cudaStreamSynchronize(stream), "warm-up");
    pthread_barrier_wait(&sh->barrier);  // every device starts its timed region together
    cuda_ok(cudaEventRecord(a, stream), "cudaEventRecord");
    for (int i = 0; i < o.iters; ++i) run();
    cuda_ok(cudaEventRecord(b, stream), "cudaEventRecord");
    cuda_ok(cudaEventSynchronize(b), "timed region");
    float ms = 0.f;
    cuda_ok(cudaEventElapsedTime(&ms, a, b), "cudaEventElapsedTime");
    cudaEventDestroy(a), cudaEventDestroy(b);
    return static_cast<double>(ms) / (static_cast<double>(o.iters) * o.layers);
  };
  sh->write_ms[rank] = timed(write_all);
  sh->gather_ms[rank] = timed(gather_all);

  // ---- every byte of the last layer against host loops ---------------------------------
  if (o.check && !o.fp8) {
    std::vector<uint8_t> hk(in_bytes), hv(in_bytes);
    cuda_ok(cudaMemcpy(hk.data(), d_key, in_bytes, cudaMemcpyDeviceToHost), "copy back");
    cuda_ok(cudaMemcpy(hv.data(), d_value, in_bytes, cudaMemcpyDeviceToHost), "copy back");
    std::vector<uint8_t> ck(tensor_bytes), cv(tensor_bytes), ok(out_bytes), ov(out_bytes);
    cuda_ok(cudaMemcpy(ck.data(), d_k[o.layers - 1], tensor_bytes, cudaMemcpyDeviceToHost), "copy back");
    cuda_ok(cudaMemcpy(cv.data(), d_v[o.layers - 1], tensor_bytes, cudaMemcpyDeviceToHost), "copy back");
    cuda_ok(cudaMemcpy(ok.data(), d_ok, out_bytes, cudaMemcpyDeviceToHost), "copy back");
    cuda_ok(cudaMemcpy(ov.data(), d_ov, out_bytes, cudaMemcpyDeviceToHost), "copy back");
    std::vector<uint8_t> ek(tensor_bytes, kPoolFill), ev(tensor_bytes, kPoolFill);
    for (int64_t t = 0; t < T; ++t) {
      const int64_t sl = w.slots[t];
      if (sl < 0 || sl / bs >= w.num_blocks) continue;
      for (int64_t h = 0; h < H; ++h)
        for (int64_t d = 0; d < D; ++d) {
          const size_t from = static_cast<size_t>(((t * H + h) * D + d) * e_io);
          memcpy(&ek[lk.offset(sl / bs, sl % bs, h, d) * e_c], &hk[from], e_c);
          memcpy(&ev[lv.offset(sl / bs, sl % bs, h, d) * e_c], &hv[from], e_c);
        }
    }
    bool good = memcmp(ek.data(), ck.data(), tensor_bytes) == 0 && memcmp(ev.data(), cv.data(), tensor_bytes) == 0;
    std::vector<uint8_t> eok(out_bytes, kOutFill), eov(out_bytes, kOutFill);
    for (int64_t s = 0; s < S; ++s)
      for (int64_t p = 0; p < std::min<int64_t>(w.lens[s], L); ++p) {
        const int64_t b = w.table[s * w.max_blocks + p / bs];
        if (b < 0 || b >= w.num_blocks) continue;
        for (int64_t h = 0; h < H; ++h)
          for (int64_t d = 0; d < D; ++d) {
            const size_t to = static_cast<size_t>((((s * L + p) * H + h) * D + d) * e_io);
            memcpy(&eok[to], &ek[lk.offset(b, p % bs, h, d) * e_c], e_c);
            memcpy(&eov[to], &ev[lv.offset(b, p % bs, h, d) * e_c], e_c);
          }
      }
    good = good && memcmp(eok.data(), ok.data(), out_bytes) == 0 && memcmp(eov.data(), ov.data(), out_bytes) == 0;
    sh->checked[rank] = good ? 1 : -1;
  }

  cudaStreamDestroy(stream);
  for (int l = 0; l < o.layers; ++l) cudaFree(d_k[l]), cudaFree(d_v[l]);
  cudaFree(d_key), cudaFree(d_value), cudaFree(d_ok), cudaFree(d_ov), cudaFree(d_slots), cudaFree(d_table);
  cudaFree(d_lens), cudaFree(d_scales), cudaFree(d_work);
  return nullptr;
}

}  // namespace

int main(int argc, char **argv) {
  Options o = parse(argc, argv);
  if (o.seq_count <= 0 || o.seq_len <= 0 || o.tokens_per_seq <= 0 || o.block_size <= 0 || o.num_heads <= 0 ||
      o.head_dim <= 0 || o.iters <= 0 || o.warmup < 0 || o.gpus <= 0 || o.layers <= 0)
    die("Invalid config values.");
  if (o.tokens_per_seq > o.seq_len) die("tokens_per_seq cannot exceed seq_len.");
  if (o.layout != "nhd" && o.layout != "hnd" && o.layout != "packed" && o.layout != "paged") die("unknown --layout");
  Workload w = o.config.empty() ? reference_workload(o) : preset_workload(&o);
  if (w.heads % o.gpus != 0) die("--gpus must divide the number of KV heads");
  int devices = 0;
  cuda_ok(cudaGetDeviceCount(&devices), "cudaGetDeviceCount");
  if (devices < o.gpus) die("fewer CUDA devices than --gpus");

  Shared sh;
  sh.opt = &o, sh.wl = &w;
  sh.write_ms.assign(o.gpus, 0.0), sh.gather_ms.assign(o.gpus, 0.0), sh.checked.assign(o.gpus, 0);
  pthread_barrier_init(&sh.barrier, nullptr, o.gpus);
  std::vector<Device> dev(o.gpus);
  std::vector<pthread_t> threads(o.gpus);
  for (int r = 0; r < o.gpus; ++r) {
    dev[r] = Device{&sh, r};
    if (pthread_create(&threads[r], nullptr, device_main, &dev[r]) != 0) die("pthread_create failed");
  }
  for (int r = 0; r < o.gpus; ++r) pthread_join(threads[r], nullptr);
  pthread_barrier_destroy(&sh.barrier);

  const double write_ms = *std::max_element(sh.write_ms.begin(), sh.write_ms.end());
  const double gather_ms = *std::max_element(sh.gather_ms.begin(), sh.gather_ms.end());
  int checked = 0;
  for (int c : sh.checked) checked = (c < 0 || checked < 0) ? -1 : std::max(checked, c);

  const kvx_dtype_t cd = o.fp8 ? KVX_DTYPE_F8_E4M3 : o.dtype;
  const double row_io = static_cast<double>(w.heads) * w.dim * elem_bytes(o.dtype);
  const double row_c = static_cast<double>(w.heads) * w.dim * elem_bytes(cd);
  const double write_bytes = 2.0 * w.valid * (row_io + row_c) + 8.0 * w.tokens();
  const double gather_bytes = 2.0 * w.gathered * (row_io + row_c) + 4.0 * w.pages + 4.0 * w.seqs;
  const double gib = 1024.0 * 1024.0 * 1024.0;
  const double write_tok_s = w.valid / (write_ms / 1e3), gather_tok_s = w.gathered / (gather_ms / 1e3);
  // the reference's figure: four element moves per element, 2^30 bytes per GB
  const double write_gib_s = 2.0 * w.valid * (row_io + row_c) / (write_ms / 1e3) / gib;
  const double gather_gib_s = 2.0 * w.gathered * (row_io + row_c) / (gather_ms / 1e3) / gib;
  const double write_gbs = write_bytes / (write_ms / 1e3) / 1e9, gather_gbs = gather_bytes / (gather_ms / 1e3) / 1e9;

  printf("write: %.3f ms, %.2f tokens/s, %.2f GB/s\n", write_ms, write_tok_s, write_gib_s);
  printf("gather: %.3f ms, %.2f tokens/s, %.2f GB/s\n", gather_ms, gather_tok_s, gather_gib_s);
  printf("kernel,seq_count,seq_len,block_size,num_heads,head_dim,num_blocks,iters,warmup,ms_per,tokens_per_s,"
         "gb_per_s,tokens_per_seq,dtype,layout,gpus,layers,valid_tokens,bytes,gbs,pct_of_8000,pct_of_peak,checked\n");
  const std::string dtype = o.fp8 ? o.dtype_name + "->f8e4m3" : o.dtype_name;
  auto line = [&](const char *kernel, double ms, double tok_s, double gib_s, int64_t tokens, double bytes, double gbs) {
    char peak[32] = "";
    if (o.peak_gbs > 0) snprintf(peak, sizeof(peak), "%.1f", 100.0 * gbs / o.gpus / o.peak_gbs);
    printf("%s,%d,%d,%d,%d,%d,%lld,%d,%d,%.6f,%.2f,%.2f,%d,%s,%s,%d,%d,%lld,%.0f,%.1f,%.1f,%s,%d\n", kernel, o.seq_count,
           o.seq_len, o.block_size, o.num_heads, o.head_dim, static_cast<long long>(w.num_blocks), o.iters, o.warmup, ms,
           tok_s, gib_s, o.tokens_per_seq, dtype.c_str(), o.layout.c_str(), o.gpus, o.layers,
           static_cast<long long>(tokens), bytes, gbs, 100.0 * gbs / o.gpus / 8000.0, peak, checked);
  };
  line("write", write_ms, write_tok_s, write_gib_s, w.valid, write_bytes, write_gbs);
  line("gather", gather_ms, gather_tok_s, gather_gib_s, w.gathered, gather_bytes, gather_gbs);
  return checked < 0 ? 2 : 0;
}
