/*
 * Decode attention over the paged KV cache (include/kvx_attention.h): the gather's consumer
 * fused with the gather, so K and V pages are read once from where they live and the
 * contiguous copy is never written.  No reference counterpart; the token walk follows the
 * reference's gather (reference: kernels/kvx_paged_kv.cu:232-266) and the page addressing its
 * per-layout offset rule (:54-75).
 *
 * The op is HBM-bound (one query token: every K and V byte is used once, about 4 flop per
 * byte with 4 query heads per KV head), so the design goal is the gather's read stream with
 * the arithmetic hidden under it:
 *
 *   fast tier   16-bit or e4m3 cache, head_dim 64 / 128 / 256, pages of a multiple of 16 tokens, up to 16 query
 *               heads per KV head.  Work items are (sequence, chunk of the context, KV head)
 *               triples of chunks that exist; persistent CTAs claim them from a counter in
 *               caller scratch, and their warps take 16-token steps whose K and V rows are staged
 *               by cp.async into a warp-private ring in shared memory.  All query heads of the
 *               KV head ride in the 8-column operand of mma.sync.m16n8k16 (tokens in its 16
 *               rows), so K / V are read once per group, not once per query head.  Online
 *               softmax in f32 (exp2 domain); per-warp partial results are merged in shared
 *               memory, per-chunk partials in a second small kernel.
 *   generic     any layout (HND_PACKED included), any head_dim up to 1 024, any page size,
 *               f32 and fp8-e4m3 caches: one CTA per (sequence, query head), element loads,
 *               the same online softmax.  Correctness tier.
 *
 * Nothing here allocates; split partials live in caller-provided scratch.
 */
#include "kvx_attention.h"
#include "kvx_paged_kv.h"

#include "kvx_pages.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <algorithm>
#include <atomic>

namespace {

// ------------------------------------------------------------------ page addressing ----

using kvx_detail::PageView;
using kvx_detail::ScaleView;
using kvx_detail::dtype_bytes;
using kvx_detail::make_page_view;

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Rows of head_dim contiguous elements that 16-byte loads can address.
bool view_rows16(const PageView &v, int64_t elem) {
  return v.pack == 1 && v.dhi == elem && aligned16(v.base) && v.blk % 16 == 0 && v.tok % 16 == 0 &&
         v.head % 16 == 0 && v.blk >= 0 && v.tok >= 0 && v.head >= 0;
}

// ------------------------------------------------------------------ parameters ---------

struct AttnParams {
  PageView k, v;
  const void *table, *lens;
  const char *query;
  char *out;
  float *part_o;   // [S, Hq, splits, D] normalised partial outputs
  float *part_ml;  // [S, Hq, splits, 2] running maximum (exp2 domain) and denominator
  unsigned long long *counter;  // next unclaimed work item of the fast kernel (zero at launch)
  ScaleView ks, vs;
  float scale_log2;  // scale * log2(e)
  int32_t seq_count, max_blocks, max_seq_len, num_blocks, block_size;
  int32_t bs_shift;  // log2(block_size) or -1
  int32_t heads_q, heads_kv, group, dim;
  int32_t chunk, splits;
  int32_t use_prefix;  // 1: the fast kernel compacts its work list with a prefix sum in shared memory
  int32_t carry;       // 1: the fast kernel starts an item's first loads ahead of the previous item's epilogue
};

template <typename IdxT>
__device__ __forceinline__ int64_t read_idx(const void *p, int64_t i) {
  return static_cast<int64_t>(static_cast<const IdxT *>(p)[i]);
}

// Work split shared by the launcher, the workspace query and the kernels: contexts are cut in
// chunks of `chunk` tokens (a multiple of 64); long chunks when there are many (sequence, KV
// head) pairs, shorter ones when the batch alone would leave the persistent CTAs with only a
// few work items each (the bound uses max_seq_len; real contexts are shorter).
#ifndef KVX_ATTN_MIN_ITEMS
#define KVX_ATTN_MIN_ITEMS 2048
#endif
inline int32_t choose_chunk(int64_t seq_count, int64_t heads_kv, int64_t max_seq_len) {
  int64_t want = kvx_b200_get_option("attn_min_items");  // tuning knob; 0 = the built-in value
  if (want <= 0) want = KVX_ATTN_MIN_ITEMS;
  int64_t chunk = 2048;
  while (chunk > 256 && seq_count * heads_kv * ((max_seq_len + chunk - 1) / chunk) < want) chunk >>= 1;
  return static_cast<int32_t>(chunk);
}

// Sequences whose chunk counts the fast kernel can prefix-sum in shared memory; with more,
// it walks the padded (sequence, chunk) rectangle instead.
constexpr int kMaxPrefixSeqs = 8192;

// Chunks sequence s really has.
template <typename IdxT>
__device__ __forceinline__ int32_t chunks_of(const AttnParams &p, int32_t s) {
  int64_t len = static_cast<int64_t>(static_cast<const IdxT *>(p.lens)[s]);
  if (len <= 0) return 0;
  if (len > p.max_seq_len) len = p.max_seq_len;
  return static_cast<int32_t>((len + p.chunk - 1) / p.chunk);
}

// ------------------------------------------------------------------ element types ------

struct Bf16 {
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&r);
  }
  static __device__ __forceinline__ uint16_t round1(float z) { return __bfloat16_as_ushort(__float2bfloat16_rn(z)); }
  static __device__ __forceinline__ uint32_t to_f16x2(uint32_t x) {  // two bf16 -> two f16 (nearest)
    const __half2 r = __floats2half2_rn(__uint_as_float(x << 16), __uint_as_float(x & 0xFFFF0000u));
    return *reinterpret_cast<const uint32_t *>(&r);
  }
  static __device__ __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

struct Fp16 {
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __half2 r = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&r);
  }
  static __device__ __forceinline__ uint16_t round1(float z) { return __half_as_ushort(__float2half_rn(z)); }
  static __device__ __forceinline__ uint32_t to_f16x2(uint32_t x) { return x; }
  static __device__ __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

// exp2(a - b) for running maxima, 0 when `a` is -inf (nothing accumulated yet).
__device__ __forceinline__ float exp2_diff(float a, float b) { return a == -INFINITY ? 0.f : exp2f(a - b); }

// Programmatic dependent launch: the kernels are launched with the stream-serialization
// attribute, let the next kernel of the stream schedule its CTAs at once, and read or write
// nothing before everything enqueued ahead of them has completed.
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ------------------------------------------------------------------ work list of the fast tier --

constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;

// Work items are (sequence, chunk, KV head) triples of chunks that exist, ordered longest first:
// all full chunks (sequence-major), then the sequences' last, shorter chunks in kRemClasses
// classes of falling length.  CTAs claim items in that order, so the last round of a launch is
// made of the shortest items and the tail, when some CTAs have run out of work, is short.
// The lengths live on the device, so every CTA builds the same lists in shared memory:
// sm_prefix[0..S] = exclusive prefix sum of full chunks per sequence, sm_rem[] = the sequences
// that have a shorter last chunk, by class (the order inside a class is the sequences' order:
// every CTA must arrive at the same list).  With too many sequences for that the CTAs enumerate
// the padded (sequence, chunk) rectangle in its natural order and meet chunks that do not
// exist.  Returns the item count.
constexpr int kRemClasses = 4;
constexpr int kListCounts = 1 + kRemClasses;

struct WorkList {
  int32_t *prefix;    // [S + 1]
  uint16_t *rem;      // [S]
  int32_t full, rems;  // totals
};

// Full chunks of sequence s and the class of its shorter last chunk (-1 = none).
template <typename IdxT>
__device__ __forceinline__ void chunk_counts(const AttnParams &p, int32_t s, int32_t *full, int32_t *rem_class) {
  int64_t len = read_idx<IdxT>(p.lens, s);
  if (len > p.max_seq_len) len = p.max_seq_len;
  if (len <= 0) {
    *full = 0, *rem_class = -1;
    return;
  }
  const int32_t f = static_cast<int32_t>(len / p.chunk);
  const int32_t r = static_cast<int32_t>(len - static_cast<int64_t>(f) * p.chunk);
  *full = f;
  *rem_class = r == 0 ? -1 : kRemClasses - 1 - (r - 1) * kRemClasses / p.chunk;  // class 0 = the longest
}

// `scratch`: kListCounts * kAttnWarps ints of shared memory, free to overwrite afterwards.
template <typename IdxT>
__device__ int64_t build_work_list(const AttnParams &p, WorkList *wl, int32_t *scratch) {
  wl->full = wl->rems = 0;
  if (!p.use_prefix) return static_cast<int64_t>(p.seq_count) * p.splits * p.heads_kv;
  const int S = p.seq_count;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = (S + kAttnThreads - 1) / kAttnThreads;
  const int begin = min(tid * per, S), end = min(begin + per, S);
  int32_t local[kListCounts];
#pragma unroll
  for (int c = 0; c < kListCounts; ++c) local[c] = 0;
  for (int s = begin; s < end; ++s) {
    int32_t f, rc;
    chunk_counts<IdxT>(p, s, &f, &rc);
    local[0] += f;
#pragma unroll
    for (int c = 0; c < kRemClasses; ++c) local[1 + c] += (rc == c);
  }
  // exclusive scan of every count over the CTA's threads: inside the warps by shuffles, across
  // them through shared memory
  int32_t incl[kListCounts];
#pragma unroll
  for (int c = 0; c < kListCounts; ++c) {
    int32_t v = local[c];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t n = __shfl_up_sync(0xFFFFFFFFu, v, d);
      if (lane >= d) v += n;
    }
    incl[c] = v;
    if (lane == 31) scratch[c * kAttnWarps + warp] = v;
  }
  __syncthreads();
  int32_t start[kListCounts], total[kListCounts];
#pragma unroll
  for (int c = 0; c < kListCounts; ++c) {
    int32_t before = 0, all = 0;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const int32_t t = scratch[c * kAttnWarps + w];
      if (w < warp) before += t;
      all += t;
    }
    start[c] = before + incl[c] - local[c];
    total[c] = all;
  }
  // classes follow one another in the remainder list
  int32_t class_base = 0;
#pragma unroll
  for (int c = 0; c < kRemClasses; ++c) {
    start[1 + c] += class_base;
    class_base += total[1 + c];
  }
  for (int s = begin; s < end; ++s) {
    int32_t f, rc;
    chunk_counts<IdxT>(p, s, &f, &rc);
    wl->prefix[s] = start[0];
    start[0] += f;
#pragma unroll
    for (int c = 0; c < kRemClasses; ++c)
      if (rc == c) wl->rem[start[1 + c]++] = static_cast<uint16_t>(s);
  }
  if (tid == kAttnThreads - 1) wl->prefix[S] = start[0];
  __syncthreads();
  wl->full = total[0];
  wl->rems = class_base;
  return static_cast<int64_t>(total[0] + class_base) * p.heads_kv;
}

struct WorkItem {
  int seq, split, kvh;
  int64_t begin, end;  // token range of the chunk; empty for a chunk the sequence does not have
};

// Claiming the CTA's next item (one thread does it).  With a counter, CTAs claim items as they
// become free; without one (few items: one per CTA) they stride over the list.
__device__ __forceinline__ unsigned long long claim_item(const AttnParams &p, unsigned long long *round) {
  const unsigned long long r = (*round)++;
  return p.counter != nullptr ? atomicAdd(p.counter, 1ull) : blockIdx.x + r * static_cast<unsigned long long>(gridDim.x);
}

// (sequence, chunk, KV head) and token range of item `item` of the work list.
template <typename IdxT>
__device__ __forceinline__ WorkItem locate_item(const AttnParams &p, int64_t item, const WorkList &wl) {
  WorkItem w;
  w.kvh = static_cast<int>(item % p.heads_kv);
  const int64_t ci = item / p.heads_kv;
  int64_t len;
  if (p.use_prefix) {
    if (ci < wl.full) {
      int lo = 0, hi = p.seq_count;  // last s with prefix[s] <= ci
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (wl.prefix[mid] <= ci)
          lo = mid;
        else
          hi = mid;
      }
      w.seq = lo;
      w.split = static_cast<int>(ci - wl.prefix[lo]);
      len = read_idx<IdxT>(p.lens, w.seq);
      if (len > p.max_seq_len) len = p.max_seq_len;
    } else {  // a sequence's shorter last chunk
      w.seq = wl.rem[ci - wl.full];
      len = read_idx<IdxT>(p.lens, w.seq);
      if (len > p.max_seq_len) len = p.max_seq_len;
      w.split = static_cast<int>(len / p.chunk);
    }
  } else {
    w.seq = static_cast<int>(ci / p.splits);
    w.split = static_cast<int>(ci - static_cast<int64_t>(w.seq) * p.splits);
    len = read_idx<IdxT>(p.lens, w.seq);
    if (len > p.max_seq_len) len = p.max_seq_len;
  }
  w.begin = static_cast<int64_t>(w.split) * p.chunk;
  w.end = min(len, w.begin + p.chunk);
  return w;
}

// A sequence without cached tokens has no work item; its output is defined as zero.  With more
// than one chunk per sequence the merge kernel writes it, otherwise the fast kernels call this.
template <typename IdxT>
__device__ void zero_empty_sequences(const AttnParams &p) {
  if (p.splits != 1) return;
  for (int s = blockIdx.x; s < p.seq_count; s += gridDim.x) {
    if (read_idx<IdxT>(p.lens, s) > 0) continue;
    for (int i = threadIdx.x; i < p.heads_q * p.dim; i += kAttnThreads)
      reinterpret_cast<uint16_t *>(p.out)[static_cast<int64_t>(s) * p.heads_q * p.dim + i] = 0;
  }
}

// ------------------------------------------------------------------ fast tier ----------

// ------------------------------------------------------------------ fast tier ----------
//
// Tokens, not query heads, sit in the 16-row dimension of mma.sync.m16n8k16, and 8 query heads in
// its 8 columns:
//   scores^T [16 tokens x 8 heads] = K [16 tokens x dims]  x  Q^T [dims x 8 heads]
//   out^T    [16 dims   x 8 heads] = V^T [16 dims x 16 tokens] x P^T [16 tokens x 8 heads]
// so no MMA row is padding (with heads in the rows 4 of 16 would be used), a step of head_dim 128
// costs 16 MMAs and 32 accumulator registers per 8 heads, and the softmax statistics of a head
// sit in the thread that owns its output columns.  Operand layouts (g = lane / 4, j = lane % 4):
//   A (16 x 16, row): a0 = (row g, k 2j..2j+1)  a1 = (row g+8, same k)  a2 = (row g, k 2j+8..2j+9)  a3 = (row g+8, ..)
//   B (16 x 8, col) : b0 = (k 2j..2j+1, col g)  b1 = (k 2j+8..2j+9, col g)
//   C (16 x 8)      : c0, c1 = (row g, cols 2j, 2j+1)   c2, c3 = (row g+8, cols 2j, 2j+1)
//
// Memory pipeline.  A warp's K and V rows for one 16-token step (8 KB at head_dim 128) are staged
// by cp.async (16 bytes per lane, whole rows per warp instruction, coalesced) into a ring of
// kTStages steps in shared memory that is private to the warp: lanes wait for their own copy
// groups and meet in __syncwarp before reading each other's chunks, no CTA barrier involved.
// Rows are padded by 16 bytes, which makes ldmatrix conflict-free and every staging address a
// per-lane base plus a compile-time constant.  K rows are A operands as they lie (ldmatrix),
// V^T comes from ldmatrix.trans, P^T from the score accumulators through movmatrix.trans.
// 3 CTAs x 4 warps per SM keep 12 steps in flight while 12 are being multiplied.
//
// Work distribution.  Items are (sequence, chunk, KV head) triples of chunks that exist; CTAs
// claim them one at a time from a counter in the caller's scratch (cleared by a one-warp kernel ahead of it), so
// short and long items balance out.
constexpr size_t kCounterBytes = 16;  // head of the scratch: the work counter, padded

__device__ __forceinline__ float fast_exp2(float x) {  // ex2.approx: 2 ulp, -inf -> 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

#ifndef KVX_ATTN_T_STAGES
#define KVX_ATTN_T_STAGES 2
#endif
#ifndef KVX_ATTN_T_CTAS
#define KVX_ATTN_T_CTAS 3
#endif
constexpr int kTStages = KVX_ATTN_T_STAGES;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t a) {  // a: shared-window address
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t a) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void cp_async16_s(uint32_t dst, const void *gmem_src) {  // dst: shared-window address
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void st_shared_zero16(uint32_t dst) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0u) : "memory");
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

// Two e4m3 pairs (the halves of x) -> two f16x2 registers, exact.
__device__ __forceinline__ void e4m3x4_to_f16x4(uint32_t x, uint32_t *lo, uint32_t *hi) {
  asm("{ .reg .b16 a, b;\n\t"
      "mov.b32 {a, b}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, a;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, b; }"
      : "=r"(*lo), "=r"(*hi)
      : "r"(x));
}

// kNt = 8-head column tiles: 1 for up to 8 query heads per KV head, 2 for 9..16 (twice the MMAs and
// accumulators on the same K / V operands).
// kFp8: the pages hold e4m3 bytes.  They are staged as they are (half the bytes per step) and
// converted to f16 between ldmatrix and the MMA, which is exact; QT is the query / output type
// (the query is converted to f16 for the MMA), T is then Fp16.  ldmatrix moves 16-bit units, so
// a lane receives e4m3 pairs: for K four consecutive dims, used as (k 2j..2j+1 | k 2j+8..2j+9)
// of one k-step -- a permutation of the reduction index that Q^T follows; for V^T two tokens x
// two dims, unzipped by one byte permute into the rows of dims 16 c + 2g (rows g) and 16 c + 2g + 1
// (rows g + 8) of the MMA for chunk c.  The K scale multiplies the scores, the V scale the output.
constexpr int attn_ctas_per_sm(int dim, int column_tiles) {  // what registers and the ring allow
  return dim > 128 ? (column_tiles == 1 ? 2 : 1) : (column_tiles == 1 ? KVX_ATTN_T_CTAS : 2);
}

template <typename T, int kD, typename IdxT, int kNt, bool kFp8 = false, typename QT = T>
__global__ void __launch_bounds__(kAttnThreads, attn_ctas_per_sm(kD, kNt))
    kvx_attention_decode_t_kernel(const AttnParams p) {
  constexpr int kKs = kD / 16;          // k-steps of the score MMAs = 16-dim row tiles of the output
  constexpr int kRowBytes = kFp8 ? kD : kD * 2;  // one token row of K or V
  constexpr int kPitch = kRowBytes + 16;  // staged rows are 16 bytes apart from a multiple of 64:
                                          // 8 consecutive rows then start in 8 different bank groups
  constexpr int kChunks = kRowBytes / 16;  // 16-byte chunks per row
  constexpr int kTile = 16 * kPitch;    // one staged 16-token step of K (or of V)
  constexpr int kPerLane = 16 * kChunks / 32;  // chunks of K (and of V) each lane copies per step
  extern __shared__ uint4 sm_dyn[];     // ring [warp][stage][K tile | V tile], then the chunk prefix
  __shared__ float sm_m[kAttnWarps][8 * kNt];
  __shared__ float sm_l[kAttnWarps][8 * kNt];
  __shared__ int32_t sm_page[kAttnWarps][kTStages];
  __shared__ int32_t sm_scan[kListCounts * kAttnWarps];
  __shared__ unsigned long long sm_item[3];  // this item and the next two: items are claimed two ahead
  char *ring = reinterpret_cast<char *>(sm_dyn);
  // Merge buffers of the epilogue, [8 * kNt][kD + 8] floats: they live in the ring, which is
  // idle by then.  Where one fits a stage, every warp uses the last stage of its own ring -- the
  // other stages may already hold the first steps of the next item (see "carried" below).
  // Where it does not (e4m3 pages with 9 to 16 query heads per KV head), the warps add into one
  // buffer at the start of the ring and nothing is carried.
  constexpr bool kCanCarry = 8 * kNt * (kD + 8) * 4 <= 2 * kTile;
  float (*sm_o)[kD + 8] = reinterpret_cast<float (*)[kD + 8]>(ring);
  const bool carry = kCanCarry && p.carry != 0;
  // behind the ring: the work list ([S + 1] prefix of full chunks, [S] sequences with a shorter last chunk)
  WorkList wl;
  wl.prefix = reinterpret_cast<int32_t *>(ring + kAttnWarps * kTStages * 2 * kTile);
  wl.rem = reinterpret_cast<uint16_t *>(wl.prefix + p.seq_count + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, j = lane & 3;
  const int G = p.group;
  // 32-bit shared-window address of this warp's ring: all staging addresses below are this
  // plus small offsets, most of them compile-time
  const uint32_t my_ring = static_cast<uint32_t>(__cvta_generic_to_shared(ring + warp * (kTStages * 2 * kTile)));

  // Programmatic launch: while the kernel ahead (the counter reset, or the caller's previous
  // kernel) drains, the lengths and the block table are asked into the L2; no value is used
  // before the wait.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  {
    const int64_t at = (static_cast<int64_t>(blockIdx.x) * kAttnThreads + threadIdx.x) * 128;
    if (at < static_cast<int64_t>(p.seq_count) * p.max_blocks * static_cast<int64_t>(sizeof(IdxT)))
      asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const char *>(p.table) + at));
    if (at < static_cast<int64_t>(p.seq_count) * static_cast<int64_t>(sizeof(IdxT)))
      asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const char *>(p.lens) + at));
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // The first two items are claimed at once (see below): the atomics travel while the work
  // list is built.
  unsigned long long round = 0;
  if (threadIdx.x == 0) {
    sm_item[0] = claim_item(p, &round);
    sm_item[1] = claim_item(p, &round);
  }
  const int64_t items = build_work_list<IdxT>(p, &wl, sm_scan);

  zero_empty_sequences<IdxT>(p);

  // Fixed per lane: which chunks of a step it copies (row = it * (32 / kChunks) + lane / kChunks,
  // chunk = lane % kChunks: a warp instruction copies whole rows, coalesced), and where its
  // ldmatrix instructions start.
  constexpr int cp_rows_per_it = 32 / kChunks;
  const int cp_row0 = lane / kChunks, cp_chunk = lane % kChunks;
  const uint32_t cp_at0 = cp_row0 * kPitch + cp_chunk * 16;
  const int64_t k_step = cp_rows_per_it * p.k.tok, v_step = cp_rows_per_it * p.v.tok;
  // ldmatrix (K as A operand): matrix i = lane / 8 -> rows 8 (i & 1) + lane % 8, chunk 2 kk + (i >> 1)
  const uint32_t lk_at = ((lane & 7) + 8 * ((lane >> 3) & 1)) * kPitch + (lane >> 4) * 16;
  // ldmatrix.trans (V^T as A operand): matrix i -> tokens 8 (i >> 1) + lane % 8, chunk 2 mt + (i & 1)
  const uint32_t lv_at = kTile + ((lane & 7) + 8 * (lane >> 4)) * kPitch + ((lane >> 3) & 1) * 16;

  // One 16-token step of an item into stage i % kTStages of the warp's ring (an empty copy
  // group beyond the warp's steps, so that the group count stays one per call).
  auto issue = [&](int seq, int64_t cbeg, int64_t cend, int kvh, int mine, int i) {
    if (i < mine) {
      const uint32_t t0 = static_cast<uint32_t>(cbeg) + static_cast<uint32_t>(warp + i * kAttnWarps) * 16u;
      const uint32_t lb = p.bs_shift >= 0 ? (t0 >> p.bs_shift) : (t0 / static_cast<uint32_t>(p.block_size));
      const uint32_t o0 = t0 - lb * static_cast<uint32_t>(p.block_size);  // a step never straddles pages
      int64_t b = -1;
      if (lb < static_cast<uint32_t>(p.max_blocks)) {
        b = read_idx<IdxT>(p.table, static_cast<int64_t>(seq) * p.max_blocks + lb);
        if (b < 0 || b >= p.num_blocks) b = -1;  // as the gather: skipped
      }
      const int stage = i % kTStages;
      sm_page[warp][stage] = static_cast<int32_t>(b);  // every lane writes the same value
      if (b >= 0) {
        const int left = static_cast<int>(min(static_cast<int64_t>(16), cend - t0));  // valid rows
        // this lane's first row of the step; later rows are cp_rows_per_it rows further on
        const char *kp = p.k.base + b * p.k.blk + static_cast<int64_t>(kvh) * p.k.head +
                         (static_cast<int64_t>(o0) + cp_row0) * p.k.tok + 16 * cp_chunk;
        const char *vp = p.v.base + b * p.v.blk + static_cast<int64_t>(kvh) * p.v.head +
                         (static_cast<int64_t>(o0) + cp_row0) * p.v.tok + 16 * cp_chunk;
        const uint32_t kd = my_ring + stage * (2 * kTile) + cp_at0, vd = kd + kTile;
        if (left == 16) {
#pragma unroll
          for (int it = 0; it < kPerLane; ++it) {
            cp_async16_s(kd + it * cp_rows_per_it * kPitch, kp + it * k_step);
            cp_async16_s(vd + it * cp_rows_per_it * kPitch, vp + it * v_step);
          }
        } else {
#pragma unroll
          for (int it = 0; it < kPerLane; ++it) {
            if (it * cp_rows_per_it + cp_row0 < left) {
              cp_async16_s(kd + it * cp_rows_per_it * kPitch, kp + it * k_step);
              cp_async16_s(vd + it * cp_rows_per_it * kPitch, vp + it * v_step);
            } else {  // beyond the chunk: zeros, so that a zero weight never meets what the page holds there
              st_shared_zero16(kd + it * cp_rows_per_it * kPitch);
              st_shared_zero16(vd + it * cp_rows_per_it * kPitch);
            }
          }
        }
      }
    }
    cp_async_commit();
  };
  // This warp's steps of a chunk: every kAttnWarps-th, starting at its own number.
  auto steps_of = [&](int64_t cbeg, int64_t cend) {
    const int nsteps = cend > cbeg ? static_cast<int>((cend - cbeg + 15) >> 4) : 0;
    return nsteps > warp ? (nsteps - warp + kAttnWarps - 1) / kAttnWarps : 0;
  };

  // Q^T as B operands: column g of tile nt = query head 8 nt + g of the group (zero beyond the
  // group), b0 = dims 16 kk + 2j, +1; b1 = dims 16 kk + 8 + 2j, +1.  An item's rows are asked
  // for before the previous item's epilogue, which needs none of these registers.
  uint32_t qb[kNt][kKs][2];
  auto load_query = [&](int seq, int kvh) {
    const int64_t q_row0 = static_cast<int64_t>(seq) * p.heads_q + static_cast<int64_t>(kvh) * G;
#pragma unroll
    for (int nt = 0; nt < kNt; ++nt) {
#pragma unroll
      for (int kk = 0; kk < kKs; ++kk) {
        qb[nt][kk][0] = qb[nt][kk][1] = 0;
        if (8 * nt + g < G) {
          const char *qrow = p.query + (q_row0 + 8 * nt + g) * (kD * 2);
          if (kFp8) {  // dims 16 kk + 4j .. 4j+3, as f16 (see the note on the K operand above)
            const uint2 q4 = *reinterpret_cast<const uint2 *>(qrow + (16 * kk + 4 * j) * 2);
            qb[nt][kk][0] = QT::to_f16x2(q4.x);
            qb[nt][kk][1] = QT::to_f16x2(q4.y);
          } else {
            qb[nt][kk][0] = *reinterpret_cast<const uint32_t *>(qrow + (16 * kk + 2 * j) * 2);
            qb[nt][kk][1] = *reinterpret_cast<const uint32_t *>(qrow + (16 * kk + 8 + 2 * j) * 2);
          }
        }
      }
    }
  };

  // Items are claimed two ahead (by one thread, behind an item's first loads, so that the round
  // trip of the atomic is off the path between two items): the barrier that ends an item makes
  // the number of the item after the next one visible, and every warp knows the next item while
  // it works on this one.  "Carried": after its last step of an item a warp issues its first
  // kTStages - 1 steps of the next item, so that the lookups and the first rows of that item
  // travel while the CTA merges and writes this item's result.
  __syncthreads();
  WorkItem w;
  bool have = static_cast<int64_t>(sm_item[0]) < items;
  if (have) {
    w = locate_item<IdxT>(p, static_cast<int64_t>(sm_item[0]), wl);
    load_query(w.seq, w.kvh);
  }
  bool carried = false;
  for (int n = 0; have; n = n == 2 ? 0 : n + 1) {
    const int n1 = n == 2 ? 0 : n + 1, n2 = n1 == 2 ? 0 : n1 + 1;
    const int seq = w.seq, split = w.split, kvh = w.kvh;
    const int64_t cbeg = w.begin, cend = w.end;
    const int64_t q_row0 = static_cast<int64_t>(seq) * p.heads_q + static_cast<int64_t>(kvh) * G;

    const float score_mul = kFp8 ? p.scale_log2 * p.ks.base[kvh * p.ks.stride] : p.scale_log2;

    // out^T: tile mt = dims 16 mt ..; c0, c1 = (dim g, heads 8 nt + 2j, + 1), c2, c3 = (dim g + 8, ..)
    float o[kNt][kKs][4];
    float m0[kNt], m1[kNt], l0[kNt], l1[kNt];  // running maxima / denominators of heads 8 nt + 2j and + 1
#pragma unroll
    for (int nt = 0; nt < kNt; ++nt) {
#pragma unroll
      for (int mt = 0; mt < kKs; ++mt) o[nt][mt][0] = o[nt][mt][1] = o[nt][mt][2] = o[nt][mt][3] = 0.f;
      m0[nt] = m1[nt] = -INFINITY;
      l0[nt] = l1[nt] = 0.f;
    }

    const int mine = steps_of(cbeg, cend);
    if (!carried) {
#pragma unroll
      for (int i = 0; i < kTStages - 1; ++i) issue(seq, cbeg, cend, kvh, mine, i);
    }
    if (threadIdx.x == 0) sm_item[n2] = claim_item(p, &round);
    for (int i = 0; i < mine; ++i) {
      issue(seq, cbeg, cend, kvh, mine, i + kTStages - 1);
      cp_async_wait<kTStages - 1>();
      __syncwarp();  // every lane's chunks of step i are in place
      const int stage = i % kTStages;
      if (sm_page[warp][stage] < 0) continue;
      const int64_t t0 = cbeg + static_cast<int64_t>(warp + i * kAttnWarps) * 16;
      const uint32_t tile = my_ring + stage * (2 * kTile);

      float s[kNt][4];  // (token g, heads 8 nt + 2j, + 1), (token g + 8, same heads)
#pragma unroll
      for (int nt = 0; nt < kNt; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      if (kFp8) {
#pragma unroll
        for (int cc = 0; cc < kKs / 2; ++cc) {  // one ldmatrix = chunks 2 cc and 2 cc + 1 = two k-steps
          uint32_t r[4], a[4];
          ldmatrix_x4(r, tile + lk_at + 32 * cc);
          e4m3x4_to_f16x4(r[0], &a[0], &a[2]);
          e4m3x4_to_f16x4(r[1], &a[1], &a[3]);
#pragma unroll
          for (int nt = 0; nt < kNt; ++nt) T::mma(s[nt], a[0], a[1], a[2], a[3], qb[nt][2 * cc][0], qb[nt][2 * cc][1]);
          e4m3x4_to_f16x4(r[2], &a[0], &a[2]);
          e4m3x4_to_f16x4(r[3], &a[1], &a[3]);
#pragma unroll
          for (int nt = 0; nt < kNt; ++nt)
            T::mma(s[nt], a[0], a[1], a[2], a[3], qb[nt][2 * cc + 1][0], qb[nt][2 * cc + 1][1]);
        }
      } else {
#pragma unroll
        for (int kk = 0; kk < kKs; ++kk) {
          uint32_t a[4];
          ldmatrix_x4(a, tile + lk_at + 32 * kk);
#pragma unroll
          for (int nt = 0; nt < kNt; ++nt) T::mma(s[nt], a[0], a[1], a[2], a[3], qb[nt][kk][0], qb[nt][kk][1]);
        }
      }
      const int64_t left = cend - t0;
      uint32_t pb[kNt][2];  // P^T as B operand: (tokens 2j, 2j+1 | head g of the tile), (tokens 2j+8, 2j+9 | ..)
#pragma unroll
      for (int nt = 0; nt < kNt; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] *= score_mul;
        if (left < 16) {
          if (g >= left) s[nt][0] = s[nt][1] = -INFINITY;
          if (g + 8 >= left) s[nt][2] = s[nt][3] = -INFINITY;
        }
        // maxima of the two heads over the step's 16 tokens: this lane's two, then over g
        float x0 = fmaxf(s[nt][0], s[nt][2]), x1 = fmaxf(s[nt][1], s[nt][3]);
#pragma unroll
        for (int d = 4; d < 32; d <<= 1) {
          x0 = fmaxf(x0, __shfl_xor_sync(0xFFFFFFFFu, x0, d));
          x1 = fmaxf(x1, __shfl_xor_sync(0xFFFFFFFFu, x1, d));
        }
        const float n0 = fmaxf(m0[nt], x0), n1 = fmaxf(m1[nt], x1);
        // The running maximum rarely moves after the first steps: rescale only when some head's did.
        if (__any_sync(0xFFFFFFFFu, n0 != m0[nt] || n1 != m1[nt])) {
          const float c0 = exp2_diff(m0[nt], n0), c1 = exp2_diff(m1[nt], n1);
          l0[nt] *= c0, l1[nt] *= c1;
#pragma unroll
          for (int mt = 0; mt < kKs; ++mt) {
            o[nt][mt][0] *= c0, o[nt][mt][2] *= c0;
            o[nt][mt][1] *= c1, o[nt][mt][3] *= c1;
          }
          m0[nt] = n0, m1[nt] = n1;
        }
        // exp2(-inf - finite) = 0 for masked tokens; a head whose maximum is still -inf (scores
        // that are -inf in the data) must not compute -inf - -inf: it subtracts 0 instead.
        const float z0 = n0 == -INFINITY ? 0.f : n0, z1 = n1 == -INFINITY ? 0.f : n1;
        const float p0 = fast_exp2(s[nt][0] - z0), p1 = fast_exp2(s[nt][1] - z1);
        const float p2 = fast_exp2(s[nt][2] - z0), p3 = fast_exp2(s[nt][3] - z1);
        l0[nt] += p0 + p2;
        l1[nt] += p1 + p3;
        pb[nt][0] = movmatrix_trans(T::pack2(p0, p1));
        pb[nt][1] = movmatrix_trans(T::pack2(p2, p3));
      }
      if (kFp8) {
#pragma unroll
        for (int cc = 0; cc < kKs / 2; ++cc) {
          // x[0], x[1] = tokens 0-7 of chunks 2 cc, 2 cc + 1; x[2], x[3] = tokens 8-15: each holds
          // bytes (token 2j | dims d, d+1), (token 2j+1 | dims d, d+1) with d = 16 c + 2g
          uint32_t x[4], a[4];
          ldmatrix_x4_trans(x, tile + lv_at + 32 * cc);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            e4m3x4_to_f16x4(__byte_perm(x[half], 0, 0x3120), &a[0], &a[1]);      // (d | tokens), (d + 1 | tokens)
            e4m3x4_to_f16x4(__byte_perm(x[2 + half], 0, 0x3120), &a[2], &a[3]);  // the same for tokens 8-15
#pragma unroll
            for (int nt = 0; nt < kNt; ++nt) T::mma(o[nt][2 * cc + half], a[0], a[1], a[2], a[3], pb[nt][0], pb[nt][1]);
          }
        }
      } else {
#pragma unroll
        for (int mt = 0; mt < kKs; ++mt) {
          uint32_t a[4];
          ldmatrix_x4_trans(a, tile + lv_at + 32 * mt);
#pragma unroll
          for (int nt = 0; nt < kNt; ++nt) T::mma(o[nt][mt], a[0], a[1], a[2], a[3], pb[nt][0], pb[nt][1]);
        }
      }
    }
    cp_async_wait<0>();

    // The next item, and its first steps on their way before this item's epilogue.
    have = static_cast<int64_t>(sm_item[n1]) < items;
    carried = false;
    if (have) {
      w = locate_item<IdxT>(p, static_cast<int64_t>(sm_item[n1]), wl);
      load_query(w.seq, w.kvh);
      if (carry) {
        const int next_mine = steps_of(w.begin, w.end);
#pragma unroll
        for (int i = 0; i < kTStages - 1; ++i) issue(w.seq, w.begin, w.end, w.kvh, next_mine, i);
        carried = true;
      }
    }

    // Denominators were kept per lane (its two tokens per step): complete them over g.
#pragma unroll
    for (int nt = 0; nt < kNt; ++nt) {
#pragma unroll
      for (int d = 4; d < 32; d <<= 1) {
        l0[nt] += __shfl_xor_sync(0xFFFFFFFFu, l0[nt], d);
        l1[nt] += __shfl_xor_sync(0xFFFFFFFFu, l1[nt], d);
      }
      if (g == 0) {
        sm_m[warp][8 * nt + 2 * j] = m0[nt], sm_m[warp][8 * nt + 2 * j + 1] = m1[nt];
        sm_l[warp][8 * nt + 2 * j] = l0[nt], sm_l[warp][8 * nt + 2 * j + 1] = l1[nt];
      }
    }
    if constexpr (kCanCarry) {
      // Every warp lays its own (unscaled) result down in the last stage of its own ring -- no
      // zeroing, no atomics -- and after one barrier the CTA sums the four with their weights.
      constexpr int kWarpRing = kTStages * 2 * kTile;
      float (*my_o)[kD + 8] = reinterpret_cast<float (*)[kD + 8]>(ring + warp * kWarpRing + (kTStages - 1) * 2 * kTile);
#pragma unroll
      for (int nt = 0; nt < kNt; ++nt) {
        const int h0 = 8 * nt + 2 * j;
#pragma unroll
        for (int mt = 0; mt < kKs; ++mt) {
          const int d_lo = kFp8 ? 16 * mt + 2 * g : 16 * mt + g, d_hi = kFp8 ? d_lo + 1 : d_lo + 8;
          my_o[h0][d_lo] = o[nt][mt][0], my_o[h0][d_hi] = o[nt][mt][2];
          my_o[h0 + 1][d_lo] = o[nt][mt][1], my_o[h0 + 1][d_hi] = o[nt][mt][3];
        }
      }
      __syncthreads();
      for (int i = threadIdx.x; i < G * kD; i += kAttnThreads) {
        const int row = i / kD, d = i - row * kD;
        float M = -INFINITY, L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, sm_m[w][row]);
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
          const float f = exp2_diff(sm_m[w][row], M);
          L += sm_l[w][row] * f;
          acc += reinterpret_cast<const float (*)[kD + 8]>(ring + w * kWarpRing + (kTStages - 1) * 2 * kTile)[row][d] * f;
        }
        float val = L > 0.f ? acc / L : 0.f;
        if (kFp8) val *= p.vs.base[kvh * p.vs.stride];
        const int64_t q = q_row0 + row;
        if (p.splits == 1) {
          reinterpret_cast<uint16_t *>(p.out)[q * kD + d] = QT::round1(val);
        } else {
          const int64_t at = q * p.splits + split;
          p.part_o[at * kD + d] = val;
          if (d == 0) {
            p.part_ml[at * 2] = M;
            p.part_ml[at * 2 + 1] = L;
          }
        }
      }
      __syncthreads();  // the number of the item after the next is visible; merge buffers and the ring are free again
      continue;
    }
    __syncthreads();  // every warp is done with its part of the ring
    for (int i = threadIdx.x; i < 8 * kNt * (kD + 8); i += kAttnThreads) (&sm_o[0][0])[i] = 0.f;
    __syncthreads();
#pragma unroll
    for (int nt = 0; nt < kNt; ++nt) {
      const int h0 = 8 * nt + 2 * j;
      float M0 = -INFINITY, M1 = -INFINITY;
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) {
        M0 = fmaxf(M0, sm_m[w][h0]);
        M1 = fmaxf(M1, sm_m[w][h0 + 1]);
      }
      const float f0 = exp2_diff(m0[nt], M0), f1 = exp2_diff(m1[nt], M1);
#pragma unroll
      for (int mt = 0; mt < kKs; ++mt) {
        // rows g and g + 8 of output tile mt: dims 16 mt + g, + 8, or (fp8) 16 mt + 2g, + 1
        const int d_lo = kFp8 ? 16 * mt + 2 * g : 16 * mt + g, d_hi = kFp8 ? d_lo + 1 : d_lo + 8;
        if (h0 < G) {
          atomicAdd(&sm_o[h0][d_lo], o[nt][mt][0] * f0);
          atomicAdd(&sm_o[h0][d_hi], o[nt][mt][2] * f0);
        }
        if (h0 + 1 < G) {
          atomicAdd(&sm_o[h0 + 1][d_lo], o[nt][mt][1] * f1);
          atomicAdd(&sm_o[h0 + 1][d_hi], o[nt][mt][3] * f1);
        }
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * kD; i += kAttnThreads) {
      const int row = i / kD, d = i - row * kD;
      float M = -INFINITY, L = 0.f;
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, sm_m[w][row]);
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) L += sm_l[w][row] * exp2_diff(sm_m[w][row], M);
      float val = L > 0.f ? sm_o[row][d] / L : 0.f;
      if (kFp8) val *= p.vs.base[kvh * p.vs.stride];
      const int64_t q = q_row0 + row;
      if (p.splits == 1) {
        reinterpret_cast<uint16_t *>(p.out)[q * kD + d] = QT::round1(val);
      } else {
        const int64_t at = q * p.splits + split;
        p.part_o[at * kD + d] = val;
        if (d == 0) {
          p.part_ml[at * 2] = M;
          p.part_ml[at * 2 + 1] = L;
        }
      }
    }
    __syncthreads();  // the number of the item after the next is visible; merge buffers and the ring are free again
  }
}

// Clears the work counter ahead of the fast kernel.
__global__ void kvx_attention_reset_kernel(unsigned long long *counter) {
  pdl_prologue();
  if (threadIdx.x == 0) *counter = 0ull;
}

// ------------------------------------------------------------------ merge of chunks ----

// One CTA per (sequence, query head): out = sum_s w_s O_s / sum_s w_s over the chunks the
// sequence really has, w_s = L_s * exp2(M_s - max M).  The loads are laid out so that few of
// them wait for one another: a lane per chunk asks for (M_s, L_s), the weights go through shared
// memory (each warp keeps its own copy: no barrier), and a thread's partial outputs are asked
// for four at a time.
template <typename IdxT>
__global__ void __launch_bounds__(128) kvx_attention_merge_kernel(const AttnParams p, int out_code) {
  pdl_prologue();
  __shared__ float s_w[4][32];
  const int64_t q = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int seq = static_cast<int>(q / p.heads_q);
  int64_t len = read_idx<IdxT>(p.lens, seq);
  if (len > p.max_seq_len) len = p.max_seq_len;
  const int live = len <= 0 ? 0 : static_cast<int>(min(static_cast<int64_t>(p.splits), (len + p.chunk - 1) / p.chunk));
  const float2 *ml = reinterpret_cast<const float2 *>(p.part_ml) + q * p.splits;  // (M_s, L_s)
  const float *po = p.part_o + q * p.splits * p.dim;
  float M = -INFINITY;
  for (int s = lane; s < live; s += 32) M = fmaxf(M, ml[s].x);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, d));
  // a thread owns dims threadIdx.x and threadIdx.x + 128 (the fast tier's head_dim is at most 256)
  const int d0 = threadIdx.x, d1 = threadIdx.x + 128;
  float W = 0.f, acc0 = 0.f, acc1 = 0.f;
  for (int s0 = 0; s0 < live; s0 += 32) {
    float w = 0.f;
    if (s0 + lane < live) {
      const float2 v = ml[s0 + lane];
      w = v.y * exp2_diff(v.x, M);
    }
    W += w;
    __syncwarp();
    s_w[warp][lane] = w;
    __syncwarp();
    const int n = min(32, live - s0);
    const float *from = po + static_cast<int64_t>(s0) * p.dim;
    for (int k0 = 0; k0 < n; k0 += 4) {
      float x0[4], x1[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const bool in = k0 + k < n;
        x0[k] = in && d0 < p.dim ? from[static_cast<int64_t>(k0 + k) * p.dim + d0] : 0.f;
        x1[k] = in && d1 < p.dim ? from[static_cast<int64_t>(k0 + k) * p.dim + d1] : 0.f;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float wk = k0 + k < n ? s_w[warp][k0 + k] : 0.f;
        acc0 += wk * x0[k];
        acc1 += wk * x1[k];
      }
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) W += __shfl_xor_sync(0xFFFFFFFFu, W, d);
  auto put = [&](int d, float acc) {
    if (d >= p.dim) return;
    const float val = W > 0.f ? acc / W : 0.f;
    const int64_t at = q * p.dim + d;
    if (out_code == KVX_DTYPE_BF16)
      reinterpret_cast<uint16_t *>(p.out)[at] = Bf16::round1(val);
    else if (out_code == KVX_DTYPE_F16)
      reinterpret_cast<uint16_t *>(p.out)[at] = Fp16::round1(val);
    else
      reinterpret_cast<float *>(p.out)[at] = val;
  };
  put(d0, acc0);
  put(d1, acc1);
}

// ------------------------------------------------------------------ generic tier -------

__device__ __forceinline__ float load_f32(const char *at, int code) {
  switch (code) {
    case KVX_DTYPE_BF16:
      return __uint_as_float(static_cast<uint32_t>(*reinterpret_cast<const uint16_t *>(at)) << 16);
    case KVX_DTYPE_F16:
      return __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(at)));
    case KVX_DTYPE_F8_E4M3: {
      uint32_t h2;
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(*reinterpret_cast<const uint8_t *>(at))));
      return __half2float(__ushort_as_half(static_cast<uint16_t>(h2 & 0xFFFFu)));
    }
    default:
      return *reinterpret_cast<const float *>(at);
  }
}

__device__ __forceinline__ int64_t elem_offset(const PageView &v, int64_t o, int64_t h, int32_t d) {
  const int32_t hi = d / v.pack;
  return o * v.tok + h * v.head + hi * v.dhi + (d - hi * v.pack) * v.dlo;
}

constexpr int kGenThreads = 128;
constexpr int kGenChunk = 1024;   // tokens whose probabilities are staged in shared memory
constexpr int kGenMaxDim = 1024;  // kGenThreads * 8 accumulators

__device__ float block_reduce(float x, bool take_max, float *scratch) {
  for (int d = 16; d > 0; d >>= 1) {
    const float y = __shfl_xor_sync(0xFFFFFFFFu, x, d);
    x = take_max ? fmaxf(x, y) : x + y;
  }
  __syncthreads();  // scratch may still be read from the previous use
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = x;
  __syncthreads();
  float r = scratch[0];
  for (int w = 1; w < kGenThreads / 32; ++w) r = take_max ? fmaxf(r, scratch[w]) : r + scratch[w];
  return r;
}

// One CTA per (sequence, query head).  Per staged chunk: every thread scores its tokens
// (element loads through the layout's offset rule), the CTA agrees on the new maximum, then
// every thread accumulates the output dims it owns over the chunk's tokens.
template <typename IdxT>
__global__ void __launch_bounds__(kGenThreads)
    kvx_attention_generic_kernel(const AttnParams p, int cache_code, int io_code) {
  extern __shared__ float sm_q[];  // [dim] query, then [kGenChunk] probabilities
  __shared__ int64_t sm_page[kGenChunk];  // byte offset of the token's page + token, -1 = no part
  __shared__ float scratch[kGenThreads / 32];
  float *sm_p = sm_q + p.dim;
  pdl_prologue();
  const int64_t q = blockIdx.x;
  const int seq = static_cast<int>(q / p.heads_q);
  const int head_q = static_cast<int>(q - static_cast<int64_t>(seq) * p.heads_q);
  const int h = head_q / p.group;
  const int elem_io = io_code == KVX_DTYPE_F32 ? 4 : 2;
  const float k_mul = p.ks.base ? p.ks.base[h * p.ks.stride] : 1.f;
  const float v_mul = p.vs.base ? p.vs.base[h * p.vs.stride] : 1.f;
  int64_t len = read_idx<IdxT>(p.lens, seq);
  if (len > p.max_seq_len) len = p.max_seq_len;
  for (int d = threadIdx.x; d < p.dim; d += kGenThreads)
    sm_q[d] = load_f32(p.query + (q * p.dim + d) * elem_io, io_code);
  float acc[kGenMaxDim / kGenThreads];
#pragma unroll
  for (int i = 0; i < kGenMaxDim / kGenThreads; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  __syncthreads();

  for (int64_t c0 = 0; c0 < len; c0 += kGenChunk) {
    const int n = static_cast<int>(min(static_cast<int64_t>(kGenChunk), len - c0));
    float mx = -INFINITY;
    for (int t = threadIdx.x; t < n; t += kGenThreads) {
      const int64_t tok = c0 + t;
      const int64_t lb = tok / p.block_size;
      int64_t at = -1;
      float s = -INFINITY;
      if (lb < p.max_blocks) {
        const int64_t b = read_idx<IdxT>(p.table, static_cast<int64_t>(seq) * p.max_blocks + lb);
        if (b >= 0 && b < p.num_blocks) {
          const int64_t o = tok - lb * p.block_size;
          at = b;  // page id; K and V may have different block strides
          float dot = 0.f;
          const char *kp = p.k.base + b * p.k.blk;
          for (int d = 0; d < p.dim; ++d)
            dot = fmaf(sm_q[d], load_f32(kp + elem_offset(p.k, o, h, d), cache_code) * k_mul, dot);
          s = dot * p.scale_log2;
        }
      }
      sm_page[t] = at;
      sm_p[t] = s;
      mx = fmaxf(mx, s);
    }
    const float m_new = fmaxf(m, block_reduce(mx, true, scratch));
    const float corr = exp2_diff(m, m_new);
    float sum = 0.f;
    for (int t = threadIdx.x; t < n; t += kGenThreads) {
      const float pr = (sm_page[t] < 0 || m_new == -INFINITY) ? 0.f : exp2f(sm_p[t] - m_new);
      sm_p[t] = pr;
      sum += pr;
    }
    l = l * corr + block_reduce(sum, false, scratch);  // ends with a barrier: sm_p is complete
    m = m_new;
#pragma unroll
    for (int i = 0; i < kGenMaxDim / kGenThreads; ++i) {
      const int d = threadIdx.x + i * kGenThreads;
      if (d < p.dim) {
        float a = acc[i] * corr;
        for (int t = 0; t < n; ++t) {
          const int64_t b = sm_page[t];
          if (b < 0) continue;
          const int64_t tok = c0 + t;
          const int64_t o = tok - (tok / p.block_size) * p.block_size;
          a = fmaf(sm_p[t], load_f32(p.v.base + b * p.v.blk + elem_offset(p.v, o, h, d), cache_code) * v_mul, a);
        }
        acc[i] = a;
      }
    }
    __syncthreads();  // the next chunk overwrites sm_p / sm_page
  }
#pragma unroll
  for (int i = 0; i < kGenMaxDim / kGenThreads; ++i) {
    const int d = threadIdx.x + i * kGenThreads;
    if (d < p.dim) {
      const float val = l > 0.f ? acc[i] / l : 0.f;
      const int64_t at = q * p.dim + d;
      if (io_code == KVX_DTYPE_BF16)
        reinterpret_cast<uint16_t *>(p.out)[at] = Bf16::round1(val);
      else if (io_code == KVX_DTYPE_F16)
        reinterpret_cast<uint16_t *>(p.out)[at] = Fp16::round1(val);
      else
        reinterpret_cast<float *>(p.out)[at] = val;
    }
  }
}

// ------------------------------------------------------------------ host ---------------

bool dense3(const kvx_tensor_desc_t *t, int64_t a, int64_t b, int64_t c, kvx_status_t *why) {
  if (t->ndim != 3 || t->shape[0] != a || t->shape[1] != b || t->shape[2] != c) {
    *why = KVX_STATUS_INVALID_ARGUMENT;
    return false;
  }
  if (t->stride[2] != 1 || t->stride[1] != c || t->stride[0] != b * c) {
    *why = KVX_STATUS_UNSUPPORTED;
    return false;
  }
  return true;
}

// Launch with the programmatic-stream-serialization attribute (see pdl_prologue).
template <typename... Args>
void launch_pdl(void (*kernel)(Args...), unsigned grid, unsigned block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <typename T, int kD, typename IdxT, bool kFp8, typename QT>
void launch_t(const AttnParams &p, unsigned grid, size_t smem, cudaStream_t st) {
  // (the attribute is per device and cheap to set, so it is set on every launch)
  if (p.group <= 8) {
    cudaFuncSetAttribute(kvx_attention_decode_t_kernel<T, kD, IdxT, 1, kFp8, QT>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_pdl(kvx_attention_decode_t_kernel<T, kD, IdxT, 1, kFp8, QT>, grid, kAttnThreads, smem, st, p);
  } else {
    cudaFuncSetAttribute(kvx_attention_decode_t_kernel<T, kD, IdxT, 2, kFp8, QT>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_pdl(kvx_attention_decode_t_kernel<T, kD, IdxT, 2, kFp8, QT>, grid, kAttnThreads, smem, st, p);
  }
}

// T = MMA operand type, QT = query / output type (they differ only for an fp8 cache).
template <typename T, typename IdxT, bool kFp8, typename QT>
void launch_t_dim(const AttnParams &p, unsigned grid, size_t smem, cudaStream_t st) {
  if (p.dim == 256)
    launch_t<T, 256, IdxT, kFp8, QT>(p, grid, smem, st);
  else if (p.dim == 128)
    launch_t<T, 128, IdxT, kFp8, QT>(p, grid, smem, st);
  else
    launch_t<T, 64, IdxT, kFp8, QT>(p, grid, smem, st);
}

template <typename IdxT>
void launch_t_types(const AttnParams &p, kvx_dtype_t cache, kvx_dtype_t io, unsigned grid, size_t smem,
                    cudaStream_t st) {
  if (cache == KVX_DTYPE_F8_E4M3) {
    if (io == KVX_DTYPE_BF16)
      launch_t_dim<Fp16, IdxT, true, Bf16>(p, grid, smem, st);
    else
      launch_t_dim<Fp16, IdxT, true, Fp16>(p, grid, smem, st);
  } else if (cache == KVX_DTYPE_BF16) {
    launch_t_dim<Bf16, IdxT, false, Bf16>(p, grid, smem, st);
  } else {
    launch_t_dim<Fp16, IdxT, false, Fp16>(p, grid, smem, st);
  }
}

// SM count of the current device, looked up once per device.
int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

}  // namespace

extern "C" {

KVX_API size_t kvx_paged_attention_workspace_bytes(uint32_t seq_count, uint32_t num_q_heads,
                                                   uint32_t num_kv_heads, uint32_t head_dim,
                                                   uint32_t max_seq_len) {
  if (seq_count == 0 || num_q_heads == 0 || num_kv_heads == 0 || head_dim == 0 || max_seq_len == 0) return 0;
  const int64_t chunk = choose_chunk(seq_count, num_kv_heads, max_seq_len);
  const int64_t splits = (static_cast<int64_t>(max_seq_len) + chunk - 1) / chunk;
  size_t bytes = kCounterBytes;  // the work counter
  if (splits > 1)
    bytes += static_cast<size_t>(seq_count) * num_q_heads * splits * (static_cast<size_t>(head_dim) + 2) * sizeof(float);
  return bytes;
}

KVX_API kvx_status_t kvx_launch_paged_attention_decode(const kvx_cache_desc_t *cache,
                                                       const kvx_attention_desc_t *attn,
                                                       const kvx_scale_desc_t *k_scale,
                                                       const kvx_scale_desc_t *v_scale, void *workspace,
                                                       size_t workspace_bytes, void *stream) {
  if (cache == nullptr || attn == nullptr) return KVX_STATUS_INVALID_ARGUMENT;
  if (cache->size < sizeof(kvx_cache_desc_t) || attn->size < sizeof(kvx_attention_desc_t) ||
      attn->block_table.size < sizeof(kvx_block_table_t) || attn->seq_lens.size < sizeof(kvx_seq_lens_t))
    return KVX_STATUS_INVALID_ARGUMENT;
  const int64_t H = cache->num_kv_heads, D = cache->head_dim, Hq = attn->num_q_heads;
  if (H == 0 || D == 0 || Hq == 0 || Hq % H != 0 || cache->block_size == 0 || attn->max_seq_len == 0)
    return KVX_STATUS_INVALID_ARGUMENT;
  if (cache->k.dtype != cache->v.dtype) return KVX_STATUS_INVALID_ARGUMENT;
  if (attn->block_table.format != KVX_BLOCK_TABLE_PACKED) return KVX_STATUS_UNSUPPORTED;
  const kvx_dtype_t io = attn->query.dtype, cd = cache->k.dtype;
  if ((io != KVX_DTYPE_F16 && io != KVX_DTYPE_BF16 && io != KVX_DTYPE_F32) || attn->out.dtype != io)
    return KVX_STATUS_UNSUPPORTED;
  AttnParams p;
  p.ks = ScaleView{nullptr, 0};
  p.vs = ScaleView{nullptr, 0};
  if (cd == KVX_DTYPE_F8_E4M3) {
    if (!kvx_detail::resolve_scale(k_scale, nullptr, cache->num_kv_heads, &p.ks) ||
        !kvx_detail::resolve_scale(v_scale, nullptr, cache->num_kv_heads, &p.vs))
      return KVX_STATUS_UNSUPPORTED;
  } else if (cd != io) {
    return KVX_STATUS_UNSUPPORTED;
  }
  const int64_t S = attn->block_table.seq_count;
  if (attn->seq_lens.seq_count != S) return KVX_STATUS_INVALID_ARGUMENT;
  kvx_status_t why = KVX_STATUS_OK;
  if (!dense3(&attn->query, S, Hq, D, &why) || !dense3(&attn->out, S, Hq, D, &why)) return why;
  const bool s32 = attn->block_table.index_dtype == KVX_DTYPE_S32 && attn->seq_lens.dtype == KVX_DTYPE_S32;
  const bool s64 = attn->block_table.index_dtype == KVX_DTYPE_S64 && attn->seq_lens.dtype == KVX_DTYPE_S64;
  if (!s32 && !s64) return KVX_STATUS_INVALID_ARGUMENT;
  if (S == 0) return KVX_STATUS_OK;
  const int64_t elem = dtype_bytes(cd);
  kvx_status_t st = make_page_view(cache, &cache->k, elem, &p.k);
  if (st != KVX_STATUS_OK) return st;
  st = make_page_view(cache, &cache->v, elem, &p.v);
  if (st != KVX_STATUS_OK) return st;
  if (attn->query.data == nullptr || attn->out.data == nullptr || attn->block_table.indices == nullptr ||
      attn->seq_lens.lengths == nullptr || cache->k.data == nullptr || cache->v.data == nullptr ||
      attn->block_table.max_blocks_per_seq == 0 || cache->num_blocks > static_cast<uint32_t>(INT32_MAX) ||
      S > INT32_MAX || attn->max_seq_len > static_cast<uint32_t>(INT32_MAX) ||
      attn->block_table.max_blocks_per_seq > static_cast<uint32_t>(INT32_MAX) || Hq > INT32_MAX || D > INT32_MAX)
    return KVX_STATUS_INVALID_ARGUMENT;

  p.table = attn->block_table.indices;
  p.lens = attn->seq_lens.lengths;
  p.query = static_cast<const char *>(attn->query.data);
  p.out = static_cast<char *>(attn->out.data);
  p.part_o = nullptr;
  p.part_ml = nullptr;
  p.counter = nullptr;
  p.carry = 0;
  p.scale_log2 = attn->scale * 1.4426950408889634f;
  p.seq_count = static_cast<int32_t>(S);
  p.max_blocks = static_cast<int32_t>(attn->block_table.max_blocks_per_seq);
  p.max_seq_len = static_cast<int32_t>(attn->max_seq_len);
  p.num_blocks = static_cast<int32_t>(cache->num_blocks);
  p.block_size = static_cast<int32_t>(cache->block_size);
  p.bs_shift = -1;
  for (int sh = 0; sh < 31; ++sh)
    if ((1u << sh) == cache->block_size) p.bs_shift = sh;
  p.heads_q = static_cast<int32_t>(Hq);
  p.heads_kv = static_cast<int32_t>(H);
  p.group = static_cast<int32_t>(Hq / H);
  p.dim = static_cast<int32_t>(D);
  p.chunk = choose_chunk(S, H, attn->max_seq_len);
  p.splits = static_cast<int32_t>((static_cast<int64_t>(attn->max_seq_len) + p.chunk - 1) / p.chunk);
  const cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);

  const bool fp8 = cd == KVX_DTYPE_F8_E4M3;
  const bool fast = (cd == KVX_DTYPE_BF16 || cd == KVX_DTYPE_F16 || (fp8 && io != KVX_DTYPE_F32)) &&
                    (D == 64 || D == 128 || D == 256) && cache->block_size % 16 == 0 && p.group <= 16 && view_rows16(p.k, elem) &&
                    view_rows16(p.v, elem) && aligned16(p.query) && H <= 65535 && S <= 65535;
  if (fast) {
    const size_t need = kvx_paged_attention_workspace_bytes(static_cast<uint32_t>(S), static_cast<uint32_t>(Hq),
                                                            static_cast<uint32_t>(H), static_cast<uint32_t>(D),
                                                            attn->max_seq_len);
    if (workspace == nullptr || workspace_bytes < need || !aligned16(workspace)) return KVX_STATUS_INVALID_ARGUMENT;
    p.counter = static_cast<unsigned long long *>(workspace);
    if (p.splits > 1) {
      p.part_o = reinterpret_cast<float *>(static_cast<char *>(workspace) + kCounterBytes);
      p.part_ml = p.part_o + S * Hq * p.splits * D;
    }
    p.use_prefix = S <= kMaxPrefixSeqs ? 1 : 0;
    p.carry = kvx_b200_get_option("attn_carry") != 0 ? 1 : 0;  // tuning knob; on unless set to 0
    const int per_sm = attn_ctas_per_sm(static_cast<int>(D), p.group <= 8 ? 1 : 2);  // the kernels' launch bounds
    // K and V steps of 16 rows, each row padded by 16 bytes
    const size_t ring = static_cast<size_t>(kAttnWarps) * kTStages * 2 * 16 * (D * elem + 16);
    // behind the ring: the prefix of full chunks and the list of sequences with a shorter last chunk
    const size_t smem = ring + (p.use_prefix ? static_cast<size_t>(S + 1) * sizeof(int32_t) + (static_cast<size_t>(S) * 2 + 15) / 16 * 16 : 0);
    const int64_t most = S * p.splits * H;  // work items if every context had max_seq_len tokens
    const int64_t grid = std::max<int64_t>(1, std::min<int64_t>(most, static_cast<int64_t>(sm_count()) * per_sm));
    if (most <= grid)
      p.counter = nullptr;  // every possible item has its own CTA: nothing to balance, no counter to clear
    else  // a kernel, not a memset: it keeps the chain of programmatic launches unbroken
      launch_pdl(kvx_attention_reset_kernel, 1u, 32u, size_t{0}, cs, p.counter);
    if (s32)
      launch_t_types<int32_t>(p, cd, io, static_cast<unsigned>(grid), smem, cs);
    else
      launch_t_types<int64_t>(p, cd, io, static_cast<unsigned>(grid), smem, cs);
    if (p.splits > 1) {
      if (s32)
        launch_pdl(kvx_attention_merge_kernel<int32_t>, static_cast<unsigned>(S * Hq), 128u, size_t{0}, cs, p, static_cast<int>(io));
      else
        launch_pdl(kvx_attention_merge_kernel<int64_t>, static_cast<unsigned>(S * Hq), 128u, size_t{0}, cs, p, static_cast<int>(io));
    }
    return cudaGetLastError() == cudaSuccess ? KVX_STATUS_OK : KVX_STATUS_INTERNAL_ERROR;
  }

  if (D > kGenMaxDim || S * Hq > INT32_MAX) return KVX_STATUS_UNSUPPORTED;
  p.splits = 1;
  const size_t smem = (static_cast<size_t>(D) + kGenChunk) * sizeof(float);
  if (s32)
    launch_pdl(kvx_attention_generic_kernel<int32_t>, static_cast<unsigned>(S * Hq), static_cast<unsigned>(kGenThreads), smem, cs, p,
               static_cast<int>(cd), static_cast<int>(io));
  else
    launch_pdl(kvx_attention_generic_kernel<int64_t>, static_cast<unsigned>(S * Hq), static_cast<unsigned>(kGenThreads), smem, cs, p,
               static_cast<int>(cd), static_cast<int>(io));
  return cudaGetLastError() == cudaSuccess ? KVX_STATUS_OK : KVX_STATUS_INTERNAL_ERROR;
}

}  // extern "C"
