/*
 * Internal to the library: how both CUDA translation units (kvx_paged_kv.cu, kvx_attention.cu)
 * see a page tensor and a scale descriptor.  Not part of the C ABI; included by quote from the
 * directory of the sources, so the single-source build of kvx_paged_kv.cu keeps working.
 */
#ifndef KVX_B200_PAGES_H
#define KVX_B200_PAGES_H

#include <stdint.h>

#include "kvx_abi.h"

namespace kvx_detail {

// A page tensor with its axes renamed (block, token-in-block, head, dim) whatever the
// layout, strides in BYTES.  The offset of element (b, o, h, d) is
//   b*blk + o*tok + h*head + (d / pack)*dhi + (d % pack)*dlo
// which restates the reference's per-layout switch (kernels/kvx_paged_kv.cu:54-75):
//   NHD        strides (s0,s1,s2,s3)     -> blk=s0 tok=s1 head=s2 dhi=s3 pack=1
//   HND        strides (s0,s1,s2,s3)     -> blk=s0 head=s1 tok=s2 dhi=s3 pack=1
//   HND_PACKED strides (s0,s1,s2,s3,s4)  -> blk=s0 head=s1 dhi=s2 tok=s3 dlo=s4 pack=shape[4]
struct PageView {
  char *base;
  int64_t blk, tok, head, dhi, dlo;
  int32_t pack;
};

inline kvx_status_t make_page_view(const kvx_cache_desc_t *c, const kvx_tensor_desc_t *t, int64_t elem,
                                   PageView *out) {
  const int64_t *s = t->stride;
  out->base = static_cast<char *>(t->data);
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

inline int64_t dtype_bytes(kvx_dtype_t t) {
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

// F32 scales of an fp8 cache, on the device.
struct ScaleView {
  const float *base;  // NULL = none
  int64_t stride;     // elements between heads; 0 = one scale per tensor
};

// PER_TENSOR ([1]) or PER_HEAD ([heads]) F32 scales from a descriptor; when the descriptor
// carries no data pointer, `scalar` (a per-tensor device scalar, may be NULL) stands in.
inline bool resolve_scale(const kvx_scale_desc_t *d, const void *scalar, uint32_t heads, ScaleView *out) {
  if (d != nullptr && d->size >= sizeof(kvx_scale_desc_t) && d->data != nullptr) {
    if (d->dtype != KVX_DTYPE_F32) return false;
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
  if (scalar != nullptr) {
    *out = ScaleView{static_cast<const float *>(scalar), 0};
    return true;
  }
  return false;
}

}  // namespace kvx_detail

#endif  // KVX_B200_PAGES_H
