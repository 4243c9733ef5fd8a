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
 *   fast tier   16-bit cache, head_dim 64 / 128, pages of a multiple of 16 tokens.
 *               One CTA per (sequence, KV head, chunk of the context); its warps take
 *               16-token steps.  K and V rows go from global memory straight into
 *               mma.sync.m16n8k16 operand registers with 16-byte loads (no shared-memory
 *               staging, no ldmatrix): the reduction index of an MMA can be permuted freely
 *               as long as both operands agree, so each lane's 16 contiguous bytes of a K row
 *               feed two k-steps, and V's token pairs are zipped with one byte-permute per
 *               operand register.  All query heads of the KV head ride in the 16 rows of the
 *               A operand, so K / V are read once per group, not once per query head.
 *               Online softmax in f32 (exp2 domain); per-warp partial results are merged in
 *               shared memory, per-chunk partials in a second small kernel.
 *   generic     any layout (HND_PACKED included), any head_dim up to 1 024, any page size,
 *               f32 and fp8-e4m3 caches: one CTA per (sequence, query head), element loads,
 *               the same online softmax.  Correctness tier.
 *
 * Nothing here allocates; split partials live in caller-provided scratch.
 */
#include "kvx_attention.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <algorithm>

namespace {

// ------------------------------------------------------------------ page addressing ----

// A page tensor with its axes renamed (block, token-in-block, head, dim), strides in BYTES:
// element (b, o, h, d) sits at b*blk + o*tok + h*head + (d / pack)*dhi + (d % pack)*dlo.
struct PageView {
  const char *base;
  int64_t blk, tok, head, dhi, dlo;
  int32_t pack;
};

int64_t dtype_bytes(kvx_dtype_t t) {
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

kvx_status_t make_page_view(const kvx_cache_desc_t *c, const kvx_tensor_desc_t *t, int64_t elem, PageView *out) {
  const int64_t *s = t->stride;
  out->base = static_cast<const char *>(t->data);
  out->pack = 1;
  out->dlo = 0;
  switch (t->layout) {
    case KVX_LAYOUT_BLOCK_NHD:
      out->blk = s[0] * elem, out->tok = s[1] * elem, out->head = s[2] * elem, out->dhi = s[3] * elem;
      return KVX_STATUS_OK;
    case KVX_LAYOUT_BLOCK_HND:
      out->blk = s[0] * elem, out->head = s[1] * elem, out->tok = s[2] * elem, out->dhi = s[3] * elem;
      return KVX_STATUS_OK;
    case KVX_LAYOUT_BLOCK_HND_PACKED: {
      const int64_t pack = t->shape[4];
      if (pack <= 0 || (static_cast<int64_t>(c->head_dim) % pack) != 0 || pack > INT32_MAX)
        return KVX_STATUS_INVALID_ARGUMENT;
      out->blk = s[0] * elem, out->head = s[1] * elem, out->dhi = s[2] * elem, out->tok = s[3] * elem;
      out->dlo = s[4] * elem;
      out->pack = static_cast<int32_t>(pack);
      return KVX_STATUS_OK;
    }
    default:
      return KVX_STATUS_UNSUPPORTED;
  }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Rows of head_dim contiguous elements that 16-byte loads can address.
bool view_rows16(const PageView &v, int64_t elem) {
  return v.pack == 1 && v.dhi == elem && aligned16(v.base) && v.blk % 16 == 0 && v.tok % 16 == 0 &&
         v.head % 16 == 0 && v.blk >= 0 && v.tok >= 0 && v.head >= 0;
}

struct ScaleView {
  const float *base;  // NULL = no scale (not an fp8 cache)
  int64_t stride;     // elements between heads (0 = one scale for all)
};

bool resolve_scale(const kvx_scale_desc_t *d, uint32_t heads, ScaleView *out) {
  if (d == nullptr || d->size < sizeof(kvx_scale_desc_t) || d->data == nullptr || d->dtype != KVX_DTYPE_F32)
    return false;
  if (d->granularity == KVX_SCALE_PER_TENSOR) {
    *out = ScaleView{static_cast<const float *>(d->data), 0};
    return true;
  }
  if (d->granularity == KVX_SCALE_PER_HEAD && d->ndim == 1 && d->shape[0] == static_cast<int64_t>(heads)) {
    *out = ScaleView{static_cast<const float *>(d->data), d->stride[0]};
    return true;
  }
  return false;
}

// ------------------------------------------------------------------ parameters ---------

struct AttnParams {
  PageView k, v;
  const void *table, *lens;
  const char *query;
  char *out;
  float *part_o;   // [S, Hq, splits, D] normalised partial outputs
  float *part_ml;  // [S, Hq, splits, 2] running maximum (exp2 domain) and denominator
  ScaleView ks, vs;
  float scale_log2;  // scale * log2(e)
  int32_t seq_count, max_blocks, max_seq_len, num_blocks, block_size;
  int32_t heads_q, heads_kv, group, dim;
  int32_t chunk, splits;
};

template <typename IdxT>
__device__ __forceinline__ int64_t read_idx(const void *p, int64_t i) {
  return static_cast<int64_t>(static_cast<const IdxT *>(p)[i]);
}

// Work split shared by the launcher, the workspace query and the kernels: contexts are cut in
// chunks of `chunk` tokens (a multiple of 64); fewer, longer chunks when there are many
// (sequence, KV head) pairs, shorter ones when the batch alone cannot fill the machine.
__host__ __device__ inline int32_t choose_chunk(int64_t seq_count, int64_t heads_kv, int64_t max_seq_len) {
  int64_t chunk = 2048;
  while (chunk > 256 && seq_count * heads_kv * ((max_seq_len + chunk - 1) / chunk) < 1024) chunk >>= 1;
  return static_cast<int32_t>(chunk);
}

// ------------------------------------------------------------------ element types ------

struct Bf16 {
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&r);
  }
  static __device__ __forceinline__ uint16_t round1(float z) { return __bfloat16_as_ushort(__float2bfloat16_rn(z)); }
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
  static __device__ __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

__device__ __forceinline__ uint4 load_stream(const void *p) {  // read-once data: no L1 allocation
  uint4 r;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) {
  return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// exp2(a - b) for running maxima, 0 when `a` is -inf (nothing accumulated yet).
__device__ __forceinline__ float exp2_diff(float a, float b) { return a == -INFINITY ? 0.f : exp2f(a - b); }

// ------------------------------------------------------------------ fast tier ----------

constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;

// MMA operand layouts used below (m16n8k16, g = lane / 4, j = lane % 4):
//   A (16 x 16, row): a0 = (row g, k 2j..2j+1)  a1 = (row g+8, same k)  a2 = (row g, k 2j+8..2j+9)  a3 = (row g+8, ..)
//   B (16 x 8, col) : b0 = (k 2j..2j+1, col g)  b1 = (k 2j+8..2j+9, col g)
//   C (16 x 8)      : c0, c1 = (row g, cols 2j, 2j+1)   c2, c3 = (row g+8, cols 2j, 2j+1)
// Scores: rows = query heads of the group, k = head dims, cols = tokens.  A lane's 16 bytes at
// dims 32c + 8j .. 8j+7 of a Q row and of a K row are used as (k 2j..2j+1 | k 2j+8..2j+9) of
// k-step 2c and of k-step 2c+1: a permutation of the dims, the same on both operands.
// Output: rows = query heads, k = tokens, cols = head dims.  P comes straight from the score
// accumulators (C of two 8-token tiles is A of one 16-token step).  For V a lane loads the
// rows of tokens 2j, 2j+1, 2j+8, 2j+9 at dims 64*hd + 8g .. 8g+7 and zips element i of two
// rows into one register for MMA i, whose column g is therefore head dim 64*hd + 8g + i.
template <typename T, int kD, typename IdxT, bool kUpper>
__global__ void __launch_bounds__(kAttnThreads, 2) kvx_attention_decode_kernel(const AttnParams p) {
  constexpr int kC = kD / 32;   // 16-byte loads per K row and lane
  constexpr int kHd = kD / 64;  // 64-dim halves of a V row
  constexpr int kNt = kD / 8;   // output column tiles
  __shared__ float sm_m[kAttnWarps][16];
  __shared__ float sm_l[kAttnWarps][16];
  __shared__ float sm_o[16][kD];

  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, j = lane & 3;
  const int G = p.group;
  int64_t len = read_idx<IdxT>(p.lens, seq);
  if (len > p.max_seq_len) len = p.max_seq_len;
  const int64_t cbeg = static_cast<int64_t>(split) * p.chunk;
  const int64_t cend = min(len, cbeg + p.chunk);
  const int64_t q_row0 = static_cast<int64_t>(seq) * p.heads_q + static_cast<int64_t>(kvh) * G;
  if (cbeg >= cend) {
    if (p.splits == 1) {  // empty context: the output is defined as zero
      for (int i = threadIdx.x; i < G * kD; i += kAttnThreads)
        reinterpret_cast<uint16_t *>(p.out)[q_row0 * kD + i] = 0;
    }
    return;
  }

  // Query rows of this KV head as A operands, kept for the whole kernel.
  uint4 qa[kC], qb[kC];
#pragma unroll
  for (int c = 0; c < kC; ++c) {
    qa[c] = make_uint4(0, 0, 0, 0);
    qb[c] = make_uint4(0, 0, 0, 0);
    if (g < G) qa[c] = *reinterpret_cast<const uint4 *>(p.query + ((q_row0 + g) * kD + 32 * c + 8 * j) * 2);
    if (kUpper && g + 8 < G)
      qb[c] = *reinterpret_cast<const uint4 *>(p.query + ((q_row0 + g + 8) * kD + 32 * c + 8 * j) * 2);
  }

  float o[kNt][4];
#pragma unroll
  for (int nt = 0; nt < kNt; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;  // rows g and g + 8

  const int nsteps = static_cast<int>((cend - cbeg + 15) >> 4);
  const int64_t head_k = static_cast<int64_t>(kvh) * p.k.head, head_v = static_cast<int64_t>(kvh) * p.v.head;
  for (int st = warp; st < nsteps; st += kAttnWarps) {
    const int64_t t0 = cbeg + static_cast<int64_t>(st) * 16;
    const int64_t lb = t0 / p.block_size;
    if (lb >= p.max_blocks) break;  // beyond the table: these tokens take no part
    const int64_t b = read_idx<IdxT>(p.table, static_cast<int64_t>(seq) * p.max_blocks + lb);
    if (b < 0 || b >= p.num_blocks) continue;  // as the gather: skipped
    const int64_t o0 = t0 - lb * p.block_size;  // a 16-token step never straddles pages
    const char *kp = p.k.base + b * p.k.blk + head_k + o0 * p.k.tok + 16 * j;
    const char *vp = p.v.base + b * p.v.blk + head_v + o0 * p.v.tok + 16 * g;

    uint4 k0[kC], k1[kC], vv[kHd][4];
#pragma unroll
    for (int c = 0; c < kC; ++c) {
      k0[c] = load_stream(kp + g * p.k.tok + 64 * c);
      k1[c] = load_stream(kp + (g + 8) * p.k.tok + 64 * c);
    }
#pragma unroll
    for (int hd = 0; hd < kHd; ++hd) {
      vv[hd][0] = load_stream(vp + (2 * j) * p.v.tok + 128 * hd);
      vv[hd][1] = load_stream(vp + (2 * j + 1) * p.v.tok + 128 * hd);
      vv[hd][2] = load_stream(vp + (2 * j + 8) * p.v.tok + 128 * hd);
      vv[hd][3] = load_stream(vp + (2 * j + 9) * p.v.tok + 128 * hd);
    }

    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < kC; ++c) {
      T::mma(s0, qa[c].x, qb[c].x, qa[c].y, qb[c].y, k0[c].x, k0[c].y);
      T::mma(s0, qa[c].z, qb[c].z, qa[c].w, qb[c].w, k0[c].z, k0[c].w);
      T::mma(s1, qa[c].x, qb[c].x, qa[c].y, qb[c].y, k1[c].x, k1[c].y);
      T::mma(s1, qa[c].z, qb[c].z, qa[c].w, qb[c].w, k1[c].z, k1[c].w);
    }

    // Scale into the exp2 domain; tokens at or beyond the end of the chunk take no part, and
    // their V rows (whatever the page holds there) are cleared so that 0 * garbage stays 0.
    const int64_t left = cend - t0;  // valid tokens in this step, >= 1
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int tok0 = 2 * j + (e & 1), tok1 = tok0 + 8;
      s0[e] = tok0 < left ? s0[e] * p.scale_log2 : -INFINITY;
      s1[e] = tok1 < left ? s1[e] * p.scale_log2 : -INFINITY;
    }
    if (left < 16) {
#pragma unroll
      for (int hd = 0; hd < kHd; ++hd) {
        if (2 * j >= left) vv[hd][0] = make_uint4(0, 0, 0, 0);
        if (2 * j + 1 >= left) vv[hd][1] = make_uint4(0, 0, 0, 0);
        if (2 * j + 8 >= left) vv[hd][2] = make_uint4(0, 0, 0, 0);
        if (2 * j + 9 >= left) vv[hd][3] = make_uint4(0, 0, 0, 0);
      }
    }

    float mx_lo = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
    float mx_hi = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xFFFFFFFFu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xFFFFFFFFu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xFFFFFFFFu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xFFFFFFFFu, mx_hi, 2));
    const float n_lo = fmaxf(m_lo, mx_lo), n_hi = fmaxf(m_hi, mx_hi);
    const float c_lo = exp2_diff(m_lo, n_lo), c_hi = exp2_diff(m_hi, n_hi);
    m_lo = n_lo, m_hi = n_hi;
    // exp2(-inf - finite) = 0 for masked tokens; a row whose maximum is still -inf (scores
    // that are -inf or NaN in the data) keeps p = 0 through the guard.
    float pr[8];
    pr[0] = n_lo == -INFINITY ? 0.f : exp2f(s0[0] - n_lo);
    pr[1] = n_lo == -INFINITY ? 0.f : exp2f(s0[1] - n_lo);
    pr[2] = n_hi == -INFINITY ? 0.f : exp2f(s0[2] - n_hi);
    pr[3] = n_hi == -INFINITY ? 0.f : exp2f(s0[3] - n_hi);
    pr[4] = n_lo == -INFINITY ? 0.f : exp2f(s1[0] - n_lo);
    pr[5] = n_lo == -INFINITY ? 0.f : exp2f(s1[1] - n_lo);
    pr[6] = n_hi == -INFINITY ? 0.f : exp2f(s1[2] - n_hi);
    pr[7] = n_hi == -INFINITY ? 0.f : exp2f(s1[3] - n_hi);
    l_lo = l_lo * c_lo + (pr[0] + pr[1] + pr[4] + pr[5]);
    l_hi = l_hi * c_hi + (pr[2] + pr[3] + pr[6] + pr[7]);
#pragma unroll
    for (int nt = 0; nt < kNt; ++nt) {
      o[nt][0] *= c_lo, o[nt][1] *= c_lo;
      o[nt][2] *= c_hi, o[nt][3] *= c_hi;
    }
    const uint32_t pa0 = T::pack2(pr[0], pr[1]), pa1 = T::pack2(pr[2], pr[3]);
    const uint32_t pa2 = T::pack2(pr[4], pr[5]), pa3 = T::pack2(pr[6], pr[7]);
#pragma unroll
    for (int hd = 0; hd < kHd; ++hd) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;  // high or low halves of both words
        const uint32_t b0 = __byte_perm(word_of(vv[hd][0], i >> 1), word_of(vv[hd][1], i >> 1), sel);
        const uint32_t b1 = __byte_perm(word_of(vv[hd][2], i >> 1), word_of(vv[hd][3], i >> 1), sel);
        T::mma(o[hd * 8 + i], pa0, pa1, pa2, pa3, b0, b1);
      }
    }
  }

  // Denominators were kept per lane; complete them over the 4 lanes that share a row.
  l_lo += __shfl_xor_sync(0xFFFFFFFFu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xFFFFFFFFu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xFFFFFFFFu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xFFFFFFFFu, l_hi, 2);

  // Merge the warps' partial results: common maximum, rescaled sums.
  if (j == 0) {
    sm_m[warp][g] = m_lo, sm_m[warp][g + 8] = m_hi;
    sm_l[warp][g] = l_lo, sm_l[warp][g + 8] = l_hi;
  }
  for (int i = threadIdx.x; i < 16 * kD; i += kAttnThreads) (&sm_o[0][0])[i] = 0.f;
  __syncthreads();
  float M_lo = -INFINITY, M_hi = -INFINITY;
#pragma unroll
  for (int w = 0; w < kAttnWarps; ++w) {
    M_lo = fmaxf(M_lo, sm_m[w][g]);
    M_hi = fmaxf(M_hi, sm_m[w][g + 8]);
  }
  const float f_lo = exp2_diff(m_lo, M_lo), f_hi = exp2_diff(m_hi, M_hi);
#pragma unroll
  for (int nt = 0; nt < kNt; ++nt) {
    const int d0 = 64 * (nt >> 3) + 16 * j + (nt & 7);  // column 2j -> head dim 64 hd + 8 (2j) + i
    if (g < G) {
      atomicAdd(&sm_o[g][d0], o[nt][0] * f_lo);
      atomicAdd(&sm_o[g][d0 + 8], o[nt][1] * f_lo);
    }
    if (kUpper && g + 8 < G) {
      atomicAdd(&sm_o[g + 8][d0], o[nt][2] * f_hi);
      atomicAdd(&sm_o[g + 8][d0 + 8], o[nt][3] * f_hi);
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
    const float val = L > 0.f ? sm_o[row][d] / L : 0.f;
    const int64_t q = q_row0 + row;
    if (p.splits == 1) {
      reinterpret_cast<uint16_t *>(p.out)[q * kD + d] = T::round1(val);
    } else {
      const int64_t at = q * p.splits + split;
      p.part_o[at * kD + d] = val;
      if (d == 0) {
        p.part_ml[at * 2] = M;
        p.part_ml[at * 2 + 1] = L;
      }
    }
  }
}

// ------------------------------------------------------------------ merge of chunks ----

// One CTA per (sequence, query head): out = sum_s w_s O_s / sum_s w_s over the chunks the
// sequence really has, w_s = L_s * exp2(M_s - max M).
template <typename IdxT>
__global__ void __launch_bounds__(128) kvx_attention_merge_kernel(const AttnParams p, int out_code) {
  const int64_t q = blockIdx.x;
  const int seq = static_cast<int>(q / p.heads_q);
  int64_t len = read_idx<IdxT>(p.lens, seq);
  if (len > p.max_seq_len) len = p.max_seq_len;
  const int live = len <= 0 ? 0 : static_cast<int>(min(static_cast<int64_t>(p.splits), (len + p.chunk - 1) / p.chunk));
  float M = -INFINITY, W = 0.f;
  for (int s = 0; s < live; ++s) M = fmaxf(M, p.part_ml[(q * p.splits + s) * 2]);
  for (int s = 0; s < live; ++s)
    W += p.part_ml[(q * p.splits + s) * 2 + 1] * exp2_diff(p.part_ml[(q * p.splits + s) * 2], M);
  for (int d = threadIdx.x; d < p.dim; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < live; ++s) {
      const float w = p.part_ml[(q * p.splits + s) * 2 + 1] * exp2_diff(p.part_ml[(q * p.splits + s) * 2], M);
      acc += w * p.part_o[(q * p.splits + s) * p.dim + d];
    }
    const float val = W > 0.f ? acc / W : 0.f;
    const int64_t at = q * p.dim + d;
    if (out_code == KVX_DTYPE_BF16)
      reinterpret_cast<uint16_t *>(p.out)[at] = Bf16::round1(val);
    else if (out_code == KVX_DTYPE_F16)
      reinterpret_cast<uint16_t *>(p.out)[at] = Fp16::round1(val);
    else
      reinterpret_cast<float *>(p.out)[at] = val;
  }
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

template <typename T, int kD, typename IdxT>
void launch_fast(const AttnParams &p, dim3 grid, cudaStream_t st) {
  if (p.group > 8)
    kvx_attention_decode_kernel<T, kD, IdxT, true><<<grid, kAttnThreads, 0, st>>>(p);
  else
    kvx_attention_decode_kernel<T, kD, IdxT, false><<<grid, kAttnThreads, 0, st>>>(p);
}

template <typename T, typename IdxT>
void launch_fast_dim(const AttnParams &p, dim3 grid, cudaStream_t st) {
  if (p.dim == 128)
    launch_fast<T, 128, IdxT>(p, grid, st);
  else
    launch_fast<T, 64, IdxT>(p, grid, st);
}

}  // namespace

extern "C" {

KVX_API size_t kvx_paged_attention_workspace_bytes(uint32_t seq_count, uint32_t num_q_heads,
                                                   uint32_t num_kv_heads, uint32_t head_dim,
                                                   uint32_t max_seq_len) {
  if (seq_count == 0 || num_q_heads == 0 || num_kv_heads == 0 || head_dim == 0 || max_seq_len == 0) return 0;
  const int64_t chunk = choose_chunk(seq_count, num_kv_heads, max_seq_len);
  const int64_t splits = (static_cast<int64_t>(max_seq_len) + chunk - 1) / chunk;
  if (splits <= 1) return 0;
  return static_cast<size_t>(seq_count) * num_q_heads * splits * (static_cast<size_t>(head_dim) + 2) * sizeof(float);
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
    if (!resolve_scale(k_scale, cache->num_kv_heads, &p.ks) || !resolve_scale(v_scale, cache->num_kv_heads, &p.vs))
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
  p.scale_log2 = attn->scale * 1.4426950408889634f;
  p.seq_count = static_cast<int32_t>(S);
  p.max_blocks = static_cast<int32_t>(attn->block_table.max_blocks_per_seq);
  p.max_seq_len = static_cast<int32_t>(attn->max_seq_len);
  p.num_blocks = static_cast<int32_t>(cache->num_blocks);
  p.block_size = static_cast<int32_t>(cache->block_size);
  p.heads_q = static_cast<int32_t>(Hq);
  p.heads_kv = static_cast<int32_t>(H);
  p.group = static_cast<int32_t>(Hq / H);
  p.dim = static_cast<int32_t>(D);
  p.chunk = choose_chunk(S, H, attn->max_seq_len);
  p.splits = static_cast<int32_t>((static_cast<int64_t>(attn->max_seq_len) + p.chunk - 1) / p.chunk);
  const cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);

  const bool fast = (cd == KVX_DTYPE_BF16 || cd == KVX_DTYPE_F16) && (D == 64 || D == 128) &&
                    cache->block_size % 16 == 0 && p.group <= 16 && view_rows16(p.k, elem) && view_rows16(p.v, elem) &&
                    aligned16(p.query) && H <= 65535 && S <= 65535;
  if (fast) {
    if (p.splits > 1) {
      const size_t need = kvx_paged_attention_workspace_bytes(static_cast<uint32_t>(S), static_cast<uint32_t>(Hq),
                                                              static_cast<uint32_t>(H), static_cast<uint32_t>(D),
                                                              attn->max_seq_len);
      if (workspace == nullptr || workspace_bytes < need || !aligned16(workspace)) return KVX_STATUS_INVALID_ARGUMENT;
      p.part_o = static_cast<float *>(workspace);
      p.part_ml = p.part_o + S * Hq * p.splits * D;
    }
    const dim3 grid(static_cast<unsigned>(p.splits), static_cast<unsigned>(H), static_cast<unsigned>(S));
    if (cd == KVX_DTYPE_BF16) {
      if (s32)
        launch_fast_dim<Bf16, int32_t>(p, grid, cs);
      else
        launch_fast_dim<Bf16, int64_t>(p, grid, cs);
    } else {
      if (s32)
        launch_fast_dim<Fp16, int32_t>(p, grid, cs);
      else
        launch_fast_dim<Fp16, int64_t>(p, grid, cs);
    }
    if (p.splits > 1) {
      if (s32)
        kvx_attention_merge_kernel<int32_t><<<static_cast<unsigned>(S * Hq), 128, 0, cs>>>(p, io);
      else
        kvx_attention_merge_kernel<int64_t><<<static_cast<unsigned>(S * Hq), 128, 0, cs>>>(p, io);
    }
    return cudaGetLastError() == cudaSuccess ? KVX_STATUS_OK : KVX_STATUS_INTERNAL_ERROR;
  }

  if (D > kGenMaxDim || S * Hq > INT32_MAX) return KVX_STATUS_UNSUPPORTED;
  p.splits = 1;
  const size_t smem = (static_cast<size_t>(D) + kGenChunk) * sizeof(float);
  if (s32)
    kvx_attention_generic_kernel<int32_t><<<static_cast<unsigned>(S * Hq), kGenThreads, smem, cs>>>(p, cd, io);
  else
    kvx_attention_generic_kernel<int64_t><<<static_cast<unsigned>(S * Hq), kGenThreads, smem, cs>>>(p, cd, io);
  return cudaGetLastError() == cudaSuccess ? KVX_STATUS_OK : KVX_STATUS_INTERNAL_ERROR;
}

}  // extern "C"
