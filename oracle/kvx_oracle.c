/*
 * CPU ORACLE -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of what the reference's CUDA kernels compute for the paged
 * KV-cache write and gather, one element at a time, on HOST memory.  Only the test-suite,
 * the smoke check and the CPU-baseline leg of the benchmark may build, load or call this
 * file; the library that ships never does.
 *
 * The reference has no CPU data path (its kvx_write_kv / kvx_gather_kv only validate,
 * kvx_abi.c:354-466), so this follows the kernels themselves:
 *   offset arithmetic per layout .......... kernels/kvx_paged_kv.cu:54-75
 *   write semantics and its two skips ..... kernels/kvx_paged_kv.cu:98-123
 *   gather semantics and its three skips .. kernels/kvx_paged_kv.cu:232-266
 *   the independent expected-value loops .. tests/kvx_kernel_test.cu:264-301, :415-446, :749-777
 *
 * Parity pin: checked against (a) the closed-form toy cases of the reference's kernel
 * test, (b) byte dumps produced by the reference's own kernels (compiled unmodified for
 * sm_100a and run on a B200) stored under tests/golden/, (c) for fp8, the e4m3 conversion
 * of ml_dtypes / torch on the finite range.  The fp8 variant itself has no reference
 * implementation -- its parity is pinned by (c) only.
 *
 * Descriptors are the public ABI structs with every pointer addressing host memory.
 */
#include "kvx_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ helpers ---------- */

static size_t elem_bytes(kvx_dtype_t t) {
  switch (t) {
    case KVX_DTYPE_F16:
    case KVX_DTYPE_BF16:
      return 2;
    case KVX_DTYPE_F32:
      return 4;
    case KVX_DTYPE_F8_E4M3:
    case KVX_DTYPE_F8_E5M2:
      return 1;
    default:
      return 0;
  }
}

static int64_t read_index(const void *base, kvx_dtype_t t, int64_t i) {
  return t == KVX_DTYPE_S32 ? (int64_t)((const int32_t *)base)[i] : ((const int64_t *)base)[i];
}

/* Element offset of (block, offset-in-block, head, dim) inside a page tensor, using the
 * descriptor's own strides.  kernels/kvx_paged_kv.cu:54-75 */
static int64_t page_offset(const kvx_tensor_desc_t *t, int64_t block, int64_t off, int64_t head,
                           int64_t dim) {
  const int64_t *s = t->stride;
  switch (t->layout) {
    case KVX_LAYOUT_BLOCK_NHD:
      return block * s[0] + off * s[1] + head * s[2] + dim * s[3];
    case KVX_LAYOUT_BLOCK_HND:
      return block * s[0] + head * s[1] + off * s[2] + dim * s[3];
    case KVX_LAYOUT_BLOCK_HND_PACKED: {
      const int64_t pack = t->shape[4];
      const int64_t hi = dim / pack;
      return block * s[0] + head * s[1] + hi * s[2] + off * s[3] + (dim - hi * pack) * s[4];
    }
    default:
      return 0;
  }
}

static int layout_known(kvx_layout_t l) {
  return l == KVX_LAYOUT_BLOCK_NHD || l == KVX_LAYOUT_BLOCK_HND || l == KVX_LAYOUT_BLOCK_HND_PACKED;
}

/* ------------------------------------------------------------------ fp8 e4m3 --------- */

static uint32_t f32_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
static float bits_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* One rounding f32 -> E4M3 (bias 7, 3 mantissa bits, subnormals down to 2^-9, largest
 * finite 448 = 0x7E, no infinities), ties to even, saturating: |y| >= 448 and +-inf give
 * +-448; NaN gives 0x7F with the sign dropped.  This is what cvt.rn.satfinite.e4m3x2.f32
 * computes. */
uint8_t kvx_oracle_e4m3_from_f32(float y) {
  const uint32_t u = f32_bits(y);
  const uint32_t a = u & 0x7FFFFFFFu;
  const uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  if (a > 0x7F800000u) return 0x7F;              /* NaN */
  if (a >= 0x43E00000u) return sign | 0x7E;      /* |y| >= 448 (incl. inf) */
  if (a < 0x3C800000u) {                         /* |y| < 2^-6: subnormal grid of 2^-9 */
    /* |y| * 512 is exact in f32; nearbyintf rounds ties to even in the default mode.  The
     * result 0..8 is the code itself (8 = smallest normal, 2^-6). */
    const float q = nearbyintf(bits_f32(a) * 512.0f);
    return sign | (uint8_t)q;
  }
  /* normal: keep 3 mantissa bits; adding the half-ulp minus one plus the kept lsb rounds
   * to nearest-even and lets a mantissa carry ripple into the exponent. */
  {
    const uint32_t r = (a + 0x7FFFFu + ((a >> 20) & 1u)) >> 20; /* (exp8 << 3) | mant3 */
    const uint32_t code = r - ((127u - 7u) << 3);
    return sign | (uint8_t)(code > 0x7Eu ? 0x7Eu : code);
  }
}

/* Exact E4M3 -> f32.  0x7F / 0xFF are NaN. */
float kvx_oracle_e4m3_to_f32(uint8_t q) {
  const uint32_t sign = (uint32_t)(q & 0x80u) << 24;
  const int e = (q >> 3) & 0xF;
  const int m = q & 7;
  float mag;
  if (e == 15 && m == 7) return bits_f32(0x7FFFFFFFu);
  if (e == 0)
    mag = (float)m * (1.0f / 512.0f);
  else
    mag = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  return bits_f32(f32_bits(mag) | sign);
}

static float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t e = (h >> 10) & 0x1Fu;
  const uint32_t m = h & 0x3FFu;
  if (e == 0x1F) return bits_f32(sign | 0x7F800000u | (m << 13));
  if (e == 0) {
    const float mag = (float)m * (1.0f / 16777216.0f); /* m * 2^-24, exact */
    return bits_f32(f32_bits(mag) | sign);
  }
  return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}

/* f32 -> bf16, ties to even; NaN -> 0x7FFF (what __float2bfloat16_rn returns). */
static uint16_t f32_to_bf16(float f) {
  const uint32_t u = f32_bits(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF;
  return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

/* f32 -> f16, ties to even, overflow to infinity; NaN -> 0x7FFF (cvt.rn.f16.f32). */
static uint16_t f32_to_f16(float f) {
  const uint32_t u = f32_bits(f);
  const uint32_t a = u & 0x7FFFFFFFu;
  const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  if (a > 0x7F800000u) return 0x7FFF;
  if (a >= 0x47800000u) return sign | 0x7C00;      /* >= 65536 (incl. inf) */
  if (a < 0x38800000u) {                           /* < 2^-14: subnormal grid of 2^-24 */
    const float q = nearbyintf(bits_f32(a) * 16777216.0f); /* 0..1024 */
    return sign | (uint16_t)q;
  }
  {
    const uint32_t r = (a + 0xFFFu + ((a >> 13) & 1u)) >> 13; /* (exp8 << 10) | mant10 */
    const uint32_t code = r - (112u << 10);
    return sign | (uint16_t)(code > 0x7C00u ? 0x7C00u : code); /* 65520.. rounds to inf */
  }
}

static float load_as_f32(const void *p, kvx_dtype_t t, int64_t i) {
  switch (t) {
    case KVX_DTYPE_BF16:
      return bits_f32((uint32_t)((const uint16_t *)p)[i] << 16);
    case KVX_DTYPE_F16:
      return f16_to_f32(((const uint16_t *)p)[i]);
    default:
      return ((const float *)p)[i];
  }
}

static void store_from_f32(void *p, kvx_dtype_t t, int64_t i, float z) {
  switch (t) {
    case KVX_DTYPE_BF16:
      ((uint16_t *)p)[i] = f32_to_bf16(z);
      break;
    case KVX_DTYPE_F16:
      ((uint16_t *)p)[i] = f32_to_f16(z);
      break;
    default:
      ((float *)p)[i] = (z != z) ? bits_f32(0x7FFFFFFFu) : z;
      break;
  }
}

/* Scale applying to head h.  desc->data wins over the per-tensor scalar. */
static int resolve_scale(const kvx_scale_desc_t *d, const void *scalar, uint32_t heads,
                         const float **base, int64_t *stride) {
  if (d != NULL && d->data != NULL) {
    if (d->dtype != KVX_DTYPE_F32) return 0;
    if (d->granularity == KVX_SCALE_PER_TENSOR) {
      *base = (const float *)d->data;
      *stride = 0;
      return 1;
    }
    if (d->granularity == KVX_SCALE_PER_HEAD && d->ndim == 1 && d->shape[0] == (int64_t)heads) {
      *base = (const float *)d->data;
      *stride = d->stride[0];
      return 1;
    }
    return 0;
  }
  if (scalar != NULL) {
    *base = (const float *)scalar;
    *stride = 0;
    return 1;
  }
  return 0;
}

static int io_dtype_quantisable(kvx_dtype_t t) {
  return t == KVX_DTYPE_F16 || t == KVX_DTYPE_BF16 || t == KVX_DTYPE_F32;
}

/* ------------------------------------------------------------------ write ------------ */

/* One tensor (K or V) of a write.  kernels/kvx_paged_kv.cu:98-123 */
static void write_one(const kvx_cache_desc_t *c, const kvx_tensor_desc_t *pages,
                      const kvx_tensor_desc_t *src, const kvx_slot_mapping_t *slots,
                      uint32_t tokens, const float *scale, int64_t scale_stride) {
  const int64_t H = c->num_kv_heads, D = c->head_dim, bs = c->block_size;
  const size_t E = elem_bytes(pages->dtype);
  const int quant = (pages->dtype == KVX_DTYPE_F8_E4M3 && src->dtype != KVX_DTYPE_F8_E4M3);
  for (int64_t t = 0; t < (int64_t)tokens; ++t) {
    const int64_t slot = read_index(slots->slots, slots->dtype, t);
    if (slot < 0) continue; /* padding */
    const int64_t block = slot / bs;
    const int64_t off = slot - block * bs;
    if (block >= (int64_t)c->num_blocks) continue; /* silently skipped */
    for (int64_t h = 0; h < H; ++h) {
      for (int64_t d = 0; d < D; ++d) {
        const int64_t si = t * src->stride[0] + h * D + d; /* token rows may be pitched; dense: stride[0] = H * D */
        const int64_t di = page_offset(pages, block, off, h, d);
        if (quant) {
          const float x = load_as_f32(src->data, src->dtype, si);
          const float y = x / scale[h * scale_stride]; /* one IEEE division */
          ((uint8_t *)pages->data)[di] = kvx_oracle_e4m3_from_f32(y);
        } else {
          memcpy((char *)pages->data + (size_t)di * E, (const char *)src->data + (size_t)si * E, E);
        }
      }
    }
  }
}

kvx_status_t kvx_oracle_write_kv(const kvx_cache_desc_t *cache, const kvx_write_desc_t *write) {
  const float *ks = NULL, *vs = NULL;
  int64_t kss = 0, vss = 0;
  if (cache == NULL || write == NULL) return KVX_STATUS_INVALID_ARGUMENT;
  if (!layout_known(cache->k.layout) || !layout_known(cache->v.layout)) return KVX_STATUS_UNSUPPORTED;
  if (cache->k.dtype != cache->v.dtype) return KVX_STATUS_INVALID_ARGUMENT;
  if (write->slots.dtype != KVX_DTYPE_S32 && write->slots.dtype != KVX_DTYPE_S64)
    return KVX_STATUS_INVALID_ARGUMENT;
  if (cache->k.dtype == KVX_DTYPE_F8_E4M3) {
    if (!io_dtype_quantisable(write->io.key.dtype) || write->io.key.dtype != write->io.value.dtype)
      return KVX_STATUS_UNSUPPORTED;
    if (!resolve_scale(&write->k_scale_desc, write->k_scale, cache->num_kv_heads, &ks, &kss) ||
        !resolve_scale(&write->v_scale_desc, write->v_scale, cache->num_kv_heads, &vs, &vss))
      return KVX_STATUS_UNSUPPORTED;
  } else if (write->io.key.dtype != cache->k.dtype || write->io.value.dtype != cache->v.dtype) {
    return KVX_STATUS_UNSUPPORTED;
  }
  write_one(cache, &cache->k, &write->io.key, &write->slots, write->io.num_tokens, ks, kss);
  write_one(cache, &cache->v, &write->io.value, &write->slots, write->io.num_tokens, vs, vss);
  return KVX_STATUS_OK;
}

/* ------------------------------------------------------------------ gather ----------- */

/* One tensor of a gather.  kernels/kvx_paged_kv.cu:232-266; additionally a block id
 * >= num_blocks is skipped (the reference reads out of bounds there). */
static void gather_one(const kvx_cache_desc_t *c, const kvx_tensor_desc_t *pages, int kv,
                       const kvx_tensor_desc_t *dst, const kvx_gather_desc_t *g, const float *scale,
                       int64_t scale_stride, const void *out_indptr, kvx_dtype_t out_indptr_dtype) {
  const int64_t H = c->num_kv_heads, D = c->head_dim, bs = c->block_size;
  const int64_t S = g->block_table.seq_count, Lmax = g->max_seq_len;
  const int64_t mb = g->block_table.max_blocks_per_seq;
  const size_t E = elem_bytes(pages->dtype);
  const int dequant = (pages->dtype == KVX_DTYPE_F8_E4M3 && dst->dtype != KVX_DTYPE_F8_E4M3);
  for (int64_t s = 0; s < S; ++s) {
    const int64_t len = read_index(g->seq_lens.lengths, g->seq_lens.dtype, s);
    /* Un-padded output: row out_indptr[s] + tok, inside the rows set aside for the sequence
     * and inside the tensor (no reference counterpart). */
    int64_t row0 = s * Lmax, room = Lmax;
    if (out_indptr != NULL) {
      row0 = read_index(out_indptr, out_indptr_dtype, s);
      room = read_index(out_indptr, out_indptr_dtype, s + 1);
      if (room > (int64_t)g->io.num_tokens) room = (int64_t)g->io.num_tokens;
      room -= row0;
      if (row0 < 0) room = 0;
    }
    for (int64_t tok = 0; tok < Lmax; ++tok) {
      if (tok >= len || tok >= room) continue;
      const int64_t lb = tok / bs;
      int64_t block;
      const char *page_base = (const char *)pages->data; /* block 0 of the tensor */
      if (g->block_table.format == KVX_BLOCK_TABLE_KV_OFFSETS) {
        /* TensorRT-LLM form (KVX_SPEC.md:116-122, KV_CACHE_LAYOUTS.md:89-96): int32 table
         * [S, beam_width, 2, max_blocks]; [s][0][0][lb] names the K page, [s][0][1][lb] the V
         * page.  Bit 31 selects the secondary pool, the low 31 bits count pool blocks:
         * page = pool + offset * bytes_per_block; inside the page the tensor's own strides
         * apply.  Skipped: a secondary entry without a secondary pool, an offset that is not
         * below num_blocks.  The reference does not execute this format. */
        uint32_t e;
        const char *pool;
        if (lb >= mb) continue;
        e = ((const uint32_t *)g->block_table.indices)[((s * g->block_table.beam_width) * 2 + kv) * mb + lb];
        pool = (const char *)((e >> 31) ? c->pool.secondary : c->pool.primary);
        if (pool == NULL || (e & 0x7FFFFFFFu) >= c->num_blocks) continue;
        page_base = pool + (size_t)(e & 0x7FFFFFFFu) * c->pool.bytes_per_block;
        block = 0;
      } else if (g->block_table.format == KVX_BLOCK_TABLE_RAGGED) {
        /* One page id per cached token: indices[indptr[s] + tok] for tok below
         * indptr[s + 1] - indptr[s]; offset in the page is tok % block_size
         * (KVX_SPEC.md:108-114).  The reference does not execute this format. */
        const int64_t first = read_index(g->block_table.indptr, g->block_table.indptr_dtype, s);
        const int64_t count = read_index(g->block_table.indptr, g->block_table.indptr_dtype, s + 1) - first;
        if (tok >= count) continue;
        /* a damaged indptr must not lead outside the index array: such tokens are skipped */
        if (first < 0 || first + tok >= (int64_t)g->block_table.indices_count) continue;
        block = read_index(g->block_table.indices, g->block_table.index_dtype, first + tok);
      } else {
        if (lb >= mb) continue;
        block = read_index(g->block_table.indices, g->block_table.index_dtype, s * mb + lb);
      }
      if (block < 0 || block >= (int64_t)c->num_blocks) continue;
      const int64_t off = tok - lb * bs;
      for (int64_t h = 0; h < H; ++h) {
        for (int64_t d = 0; d < D; ++d) {
          const int64_t oi = ((row0 + tok) * H + h) * D + d;
          const int64_t ci = page_offset(pages, block, off, h, d);
          if (dequant) {
            const float f = kvx_oracle_e4m3_to_f32(((const uint8_t *)page_base)[ci]);
            store_from_f32(dst->data, dst->dtype, oi, f * scale[h * scale_stride]);
          } else {
            memcpy((char *)dst->data + (size_t)oi * E, page_base + (size_t)ci * E, E);
          }
        }
      }
    }
  }
}

kvx_status_t kvx_oracle_gather_kv(const kvx_cache_desc_t *cache, const kvx_gather_desc_t *gather,
                                  const kvx_scale_desc_t *k_scale, const kvx_scale_desc_t *v_scale) {
  return kvx_oracle_gather_kv_varlen(cache, gather, NULL, KVX_DTYPE_INVALID, k_scale, v_scale);
}

kvx_status_t kvx_oracle_gather_kv_varlen(const kvx_cache_desc_t *cache, const kvx_gather_desc_t *gather,
                                         const void *out_indptr, kvx_dtype_t out_indptr_dtype,
                                         const kvx_scale_desc_t *k_scale, const kvx_scale_desc_t *v_scale) {
  const float *ks = NULL, *vs = NULL;
  int64_t kss = 0, vss = 0;
  if (cache == NULL || gather == NULL) return KVX_STATUS_INVALID_ARGUMENT;
  if (!layout_known(cache->k.layout) || !layout_known(cache->v.layout)) return KVX_STATUS_UNSUPPORTED;
  if (gather->block_table.format != KVX_BLOCK_TABLE_PACKED && gather->block_table.format != KVX_BLOCK_TABLE_RAGGED &&
      gather->block_table.format != KVX_BLOCK_TABLE_KV_OFFSETS)
    return KVX_STATUS_UNSUPPORTED;
  if (gather->block_table.format == KVX_BLOCK_TABLE_KV_OFFSETS &&
      (gather->block_table.beam_width != 1 || gather->block_table.index_dtype != KVX_DTYPE_S32 ||
       cache->pool.primary == NULL || cache->pool.bytes_per_block == 0))
    return gather->block_table.beam_width > 1 ? KVX_STATUS_UNSUPPORTED : KVX_STATUS_INVALID_ARGUMENT;
  if (gather->block_table.index_dtype != gather->seq_lens.dtype) return KVX_STATUS_INVALID_ARGUMENT;
  if (gather->seq_lens.dtype != KVX_DTYPE_S32 && gather->seq_lens.dtype != KVX_DTYPE_S64)
    return KVX_STATUS_INVALID_ARGUMENT;
  if (cache->k.dtype == KVX_DTYPE_F8_E4M3) {
    if (!io_dtype_quantisable(gather->io.key.dtype) || gather->io.key.dtype != gather->io.value.dtype)
      return KVX_STATUS_UNSUPPORTED;
    if (!resolve_scale(k_scale, NULL, cache->num_kv_heads, &ks, &kss) ||
        !resolve_scale(v_scale, NULL, cache->num_kv_heads, &vs, &vss))
      return KVX_STATUS_UNSUPPORTED;
  } else if (gather->io.key.dtype != cache->k.dtype || gather->io.value.dtype != cache->v.dtype) {
    return KVX_STATUS_UNSUPPORTED;
  }
  gather_one(cache, &cache->k, 0, &gather->io.key, gather, ks, kss, out_indptr, out_indptr_dtype);
  gather_one(cache, &cache->v, 1, &gather->io.value, gather, vs, vss, out_indptr, out_indptr_dtype);
  return KVX_STATUS_OK;
}

/* ------------------------------------------------------------------ scales ----------- */

/* absmax over (token, dim) per head (or over everything for PER_TENSOR), taken on the
 * magnitude bits -- exact and order-independent; a NaN input therefore wins the maximum.
 * scale = absmax / 448 as one f32 division; anything that is not > 0 (zero, NaN)
 * becomes 1.0f. */
static void scales_one(const kvx_tensor_desc_t *src, uint32_t tokens, uint32_t H, uint32_t D,
                       kvx_scale_granularity_t gran, float *out) {
  const uint32_t n = (gran == KVX_SCALE_PER_HEAD) ? H : 1;
  for (uint32_t i = 0; i < n; ++i) {
    uint32_t best = 0;
    for (int64_t t = 0; t < (int64_t)tokens; ++t) {
      const uint32_t h0 = (gran == KVX_SCALE_PER_HEAD) ? i : 0;
      const uint32_t h1 = (gran == KVX_SCALE_PER_HEAD) ? i + 1 : H;
      for (uint32_t h = h0; h < h1; ++h)
        for (uint32_t d = 0; d < D; ++d) {
          const uint32_t a = f32_bits(load_as_f32(src->data, src->dtype, (t * H + h) * (int64_t)D + d)) & 0x7FFFFFFFu;
          if (a > best) best = a;
        }
    }
    {
      const float s = bits_f32(best) / 448.0f;
      out[i] = (s > 0.0f) ? s : 1.0f;
    }
  }
}

kvx_status_t kvx_oracle_kv_scales(const kvx_kv_io_desc_t *io, kvx_scale_granularity_t granularity,
                                  float *k_scale_out, float *v_scale_out) {
  if (io == NULL || k_scale_out == NULL || v_scale_out == NULL) return KVX_STATUS_INVALID_ARGUMENT;
  if (granularity != KVX_SCALE_PER_HEAD && granularity != KVX_SCALE_PER_TENSOR)
    return KVX_STATUS_UNSUPPORTED;
  if (!io_dtype_quantisable(io->key.dtype) || io->key.dtype != io->value.dtype)
    return KVX_STATUS_UNSUPPORTED;
  scales_one(&io->key, io->num_tokens, io->num_kv_heads, io->head_dim, granularity, k_scale_out);
  scales_one(&io->value, io->num_tokens, io->num_kv_heads, io->head_dim, granularity, v_scale_out);
  return KVX_STATUS_OK;
}

/* ------------------------------------------------------------------ attention -------- */

/* Decode attention over the paged cache, one (sequence, query head) at a time, in double
 * precision: scores, a two-pass softmax (maximum first) and the weighted sum of V rows.  No
 * reference counterpart (the reference stops at the gather); the token walk is the gather's
 * (kernels/kvx_paged_kv.cu:232-266 plus the >= num_blocks skip), the arithmetic is the
 * definition in include/kvx_attention.h.  An fp8 cache is dequantised as value * scale in f32
 * first, exactly as the dequantising gather does. */
static float cache_elem_f32(const kvx_tensor_desc_t *pages, int64_t at, const float *scale, int64_t scale_stride,
                            int64_t h) {
  if (pages->dtype == KVX_DTYPE_F8_E4M3)
    return kvx_oracle_e4m3_to_f32(((const uint8_t *)pages->data)[at]) * scale[h * scale_stride];
  return load_as_f32(pages->data, pages->dtype, at);
}

kvx_status_t kvx_oracle_paged_attention_decode(const kvx_cache_desc_t *cache, const kvx_attention_desc_t *attn,
                                               const kvx_scale_desc_t *k_scale, const kvx_scale_desc_t *v_scale) {
  const float *ks = NULL, *vs = NULL;
  int64_t kss = 0, vss = 0;
  int64_t S, Hq, H, D, G, bs, mb, Lmax;
  double *score, *acc;
  if (cache == NULL || attn == NULL) return KVX_STATUS_INVALID_ARGUMENT;
  if (!layout_known(cache->k.layout) || !layout_known(cache->v.layout)) return KVX_STATUS_UNSUPPORTED;
  if (attn->block_table.format != KVX_BLOCK_TABLE_PACKED) return KVX_STATUS_UNSUPPORTED;
  if (attn->block_table.index_dtype != attn->seq_lens.dtype) return KVX_STATUS_INVALID_ARGUMENT;
  if (cache->num_kv_heads == 0 || attn->num_q_heads == 0 || attn->num_q_heads % cache->num_kv_heads != 0)
    return KVX_STATUS_INVALID_ARGUMENT;
  if (!io_dtype_quantisable(attn->query.dtype) || attn->out.dtype != attn->query.dtype) return KVX_STATUS_UNSUPPORTED;
  if (cache->k.dtype == KVX_DTYPE_F8_E4M3) {
    if (!resolve_scale(k_scale, NULL, cache->num_kv_heads, &ks, &kss) ||
        !resolve_scale(v_scale, NULL, cache->num_kv_heads, &vs, &vss))
      return KVX_STATUS_UNSUPPORTED;
  } else if (cache->k.dtype != attn->query.dtype) {
    return KVX_STATUS_UNSUPPORTED;
  }
  S = attn->block_table.seq_count, Hq = attn->num_q_heads, H = cache->num_kv_heads, D = cache->head_dim;
  G = Hq / H, bs = cache->block_size, mb = attn->block_table.max_blocks_per_seq, Lmax = attn->max_seq_len;
  if (Lmax == 0 || bs == 0) return KVX_STATUS_INVALID_ARGUMENT;
  score = (double *)malloc(sizeof(double) * (size_t)Lmax);
  acc = (double *)malloc(sizeof(double) * (size_t)D);
  if (score == NULL || acc == NULL) {
    free(score);
    free(acc);
    return KVX_STATUS_INTERNAL_ERROR;
  }
  for (int64_t s = 0; s < S; ++s) {
    int64_t len = read_index(attn->seq_lens.lengths, attn->seq_lens.dtype, s);
    if (len > Lmax) len = Lmax;
    for (int64_t q = 0; q < Hq; ++q) {
      const int64_t h = q / G;
      double best = -INFINITY, denom = 0.0;
      for (int64_t d = 0; d < D; ++d) acc[d] = 0.0;
      for (int64_t tok = 0; tok < len; ++tok) {
        const int64_t lb = tok / bs;
        int64_t block;
        score[tok] = -INFINITY; /* takes no part */
        if (lb >= mb) continue;
        block = read_index(attn->block_table.indices, attn->block_table.index_dtype, s * mb + lb);
        if (block < 0 || block >= (int64_t)cache->num_blocks) continue;
        {
          double dot = 0.0;
          for (int64_t d = 0; d < D; ++d) {
            const float kq = cache_elem_f32(&cache->k, page_offset(&cache->k, block, tok - lb * bs, h, d), ks, kss, h);
            dot += (double)load_as_f32(attn->query.data, attn->query.dtype, (s * Hq + q) * D + d) * (double)kq;
          }
          score[tok] = dot * (double)attn->scale;
          if (score[tok] > best) best = score[tok];
        }
      }
      for (int64_t tok = 0; tok < len; ++tok) {
        const int64_t lb = tok / bs;
        double p;
        int64_t block;
        if (score[tok] == -INFINITY) continue;
        p = exp(score[tok] - best);
        denom += p;
        block = read_index(attn->block_table.indices, attn->block_table.index_dtype, s * mb + lb);
        for (int64_t d = 0; d < D; ++d)
          acc[d] += p * (double)cache_elem_f32(&cache->v, page_offset(&cache->v, block, tok - lb * bs, h, d), vs, vss, h);
      }
      for (int64_t d = 0; d < D; ++d)
        store_from_f32(attn->out.data, attn->out.dtype, (s * Hq + q) * D + d,
                       denom > 0.0 ? (float)(acc[d] / denom) : 0.0f);
    }
  }
  free(score);
  free(acc);
  return KVX_STATUS_OK;
}
