"""TGI (text-generation-inference) -> KVX descriptors.

The view has the fields of the reference's stub (reference: adapters/tgi_adapter.py:5-18,
which raises NotImplementedError at :21-23); the mapping follows adapters/README.md:10-24 and
KV_CACHE_LAYOUTS.md:52-80:

    layout "flashinfer" / "flashdecoding"   K, V [num_blocks, BLOCK_SIZE, heads, head_size]     -> NHD
    layout "ipex"                           K, V [num_blocks, heads, BLOCK_SIZE, head_size]     -> HND
    layout "paged"   K [num_blocks, heads, head_size / x, BLOCK_SIZE, x],
                     V [num_blocks, heads, head_size, BLOCK_SIZE]       -> HND_PACKED (V: pack 1)

    block_tables_tensor  [num_reqs, max_blocks] int32 -> PACKED
    block_tables_ragged  one block id per cached token -> RAGGED (indptr = prefix sums of the
                         sequence lengths, filled in by adapters.gather)
    slots                [num_tokens] -> kvx_slot_mapping_t
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any, Optional

from .. import abi

_LAYOUTS = {"flashinfer": abi.LAYOUT_NHD, "flashdecoding": abi.LAYOUT_NHD, "nhd": abi.LAYOUT_NHD,
            "ipex": abi.LAYOUT_HND, "hnd": abi.LAYOUT_HND, "paged": abi.LAYOUT_HND_PACKED}


@dataclass
class TgiCacheView:
    """Normalised view of one layer of a TGI paged cache and of a batch's metadata."""

    k_cache: Any
    v_cache: Any
    block_tables_tensor: Any
    block_tables_ragged: Optional[Any]
    slots: Any
    block_size: int
    num_kv_heads: int
    head_dim: int
    kv_cache_dtype: str
    layout: str


def _cache_dtype(tensor, kv_cache_dtype: str) -> int:
    import torch
    from ..ops import _FLOAT_CODES
    if kv_cache_dtype.startswith("fp8"):
        if kv_cache_dtype not in ("fp8", "fp8_e4m3", "fp8_e4m3fn"):
            raise ValueError(f"unsupported kv_cache_dtype {kv_cache_dtype!r} (e4m3 only)")
        if tensor.element_size() != 1:
            raise TypeError("an fp8 cache must have 1-byte elements")
        return abi.DTYPE_F8_E4M3
    if tensor.dtype not in _FLOAT_CODES:
        raise TypeError(f"unsupported cache dtype {tensor.dtype}")
    return _FLOAT_CODES[tensor.dtype]


def _pages(tensor, code: int, layout: int) -> abi.TensorDesc:
    shape, stride = list(tensor.shape), list(tensor.stride())
    if layout == abi.LAYOUT_HND_PACKED and tensor.dim() == 4:  # [blocks, heads, dim, BLOCK_SIZE]: pack 1
        shape.append(1)
        stride.append(1)
    return abi.tensor_desc(tensor.data_ptr(), code, shape, stride, layout)


def build_kvx_descriptors(view: TgiCacheView, ragged: bool = False) -> dict:
    """``{"cache": kvx_cache_desc_t, "block_table": kvx_block_table_t, "slot_mapping":
    kvx_slot_mapping_t}`` over the view's tensors (no copies; the view must outlive them).
    ``ragged`` selects ``block_tables_ragged`` instead of ``block_tables_tensor``."""
    from ..ops import _INDEX_CODES
    layout = _LAYOUTS.get(view.layout.lower())
    if layout is None:
        raise ValueError(f"unknown TGI cache layout {view.layout!r}")
    k, v = view.k_cache, view.v_cache
    code = _cache_dtype(k, view.kv_cache_dtype)
    cache = abi.CacheDesc()
    cache.size = C.sizeof(abi.CacheDesc)
    cache.num_blocks, cache.block_size = k.shape[0], view.block_size
    cache.num_kv_heads, cache.head_dim = view.num_kv_heads, view.head_dim
    cache.k, cache.v = _pages(k, code, layout), _pages(v, code, layout)
    cache.pool.size = C.sizeof(abi.PoolDesc)
    want = abi.page_shape(layout, k.shape[0], view.block_size, view.num_kv_heads, view.head_dim,
                          k.shape[4] if layout == abi.LAYOUT_HND_PACKED else 1)
    if tuple(k.shape) != tuple(want):
        raise ValueError(f"k_cache has shape {tuple(k.shape)}, layout {view.layout!r} wants {tuple(want)}")

    table = abi.BlockTable()
    table.size = C.sizeof(abi.BlockTable)
    table.beam_width = 1
    if ragged:
        ids = view.block_tables_ragged
        if ids is None:
            raise ValueError("the view has no block_tables_ragged")
        table.format, table.index_dtype = abi.TABLE_RAGGED, _INDEX_CODES[ids.dtype]
        table.seq_count = view.block_tables_tensor.shape[0]
        table.max_blocks_per_seq = view.block_tables_tensor.shape[1]
        table.indices, table.indices_count = ids.data_ptr(), ids.numel()
    else:
        t = view.block_tables_tensor
        if t.dim() != 2 or not t.is_contiguous():
            raise ValueError("block_tables_tensor must be a contiguous [num_reqs, max_blocks] tensor")
        table.format, table.index_dtype = abi.TABLE_PACKED, _INDEX_CODES[t.dtype]
        table.seq_count, table.max_blocks_per_seq = t.shape[0], t.shape[1]
        table.indices, table.indices_count = t.data_ptr(), t.numel()

    slots = abi.SlotMapping()
    slots.size = C.sizeof(abi.SlotMapping)
    slots.dtype, slots.token_count = _INDEX_CODES[view.slots.dtype], view.slots.shape[0]
    slots.invalid_slot = -1
    slots.slots = view.slots.data_ptr()
    return {"cache": cache, "block_table": table, "slot_mapping": slots, "keepalive": [view]}
