"""TensorRT-LLM -> KVX descriptors.

The view has the fields of the reference's stub (reference: adapters/trt_llm_adapter.py:5-17,
which raises NotImplementedError at :20-22) plus an optional block bound; the mapping follows
adapters/README.md:26-39 and KV_CACHE_LAYOUTS.md:78-100:

    pages            [heads, tokens_per_block, head_dim] each, K and V pages in the same pools
    kv_block_offsets [B, W, 2, M] int32 KVCacheIndex values (bit 31 = secondary pool)
                     -> KVX_BLOCK_TABLE_KV_OFFSETS with the KVCACHEINDEX flag
    page address     pool + offset * bytes_per_block  -> kvx_pool_desc_t
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any, Optional

from .. import abi

_DTYPES = {"fp16": abi.DTYPE_F16, "float16": abi.DTYPE_F16, "half": abi.DTYPE_F16,
           "bf16": abi.DTYPE_BF16, "bfloat16": abi.DTYPE_BF16,
           "fp32": abi.DTYPE_F32, "float32": abi.DTYPE_F32,
           "fp8": abi.DTYPE_F8_E4M3, "fp8_e4m3": abi.DTYPE_F8_E4M3}
_BYTES = {abi.DTYPE_F16: 2, abi.DTYPE_BF16: 2, abi.DTYPE_F32: 4, abi.DTYPE_F8_E4M3: 1}


@dataclass
class TrtLlmCacheView:
    """Normalised view of a TensorRT-LLM block-pool cache (one layer's pools)."""

    kv_block_offsets: Any
    pool_primary: Any            # tensor or device address
    pool_secondary: Any          # tensor, device address or None
    bytes_per_block: int
    tokens_per_block: int
    num_kv_heads: int
    head_dim: int
    kv_cache_dtype: str
    num_blocks: Optional[int] = None   # blocks addressable in EACH pool; default: the smaller tensor's capacity


def _address(pool) -> int:
    if pool is None:
        return 0
    return int(pool) if isinstance(pool, int) else pool.data_ptr()


def _capacity(pool, bytes_per_block: int) -> Optional[int]:
    if pool is None or isinstance(pool, int):
        return None
    return pool.numel() * pool.element_size() // bytes_per_block


def build_kvx_descriptors(view: TrtLlmCacheView) -> dict:
    """``{"cache": kvx_cache_desc_t (with its pool), "block_table": kvx_block_table_t}`` over
    the view's memory (no copies; the view must outlive them)."""
    import torch
    code = _DTYPES.get(view.kv_cache_dtype.lower())
    if code is None:
        raise ValueError(f"unsupported kv_cache_dtype {view.kv_cache_dtype!r}")
    bs, heads, dim = view.tokens_per_block, view.num_kv_heads, view.head_dim
    if bs <= 0 or bs & (bs - 1):
        raise ValueError("tokens_per_block must be a power of two")
    if view.bytes_per_block < bs * heads * dim * _BYTES[code]:
        raise ValueError("bytes_per_block is smaller than one [heads, tokens_per_block, head_dim] page")
    offsets = view.kv_block_offsets
    if offsets.dtype != torch.int32 or offsets.dim() != 4 or offsets.shape[2] != 2 or not offsets.is_contiguous():
        raise ValueError("kv_block_offsets must be a contiguous int32 [B, W, 2, M] tensor")
    blocks = view.num_blocks
    if blocks is None:
        caps = [c for c in (_capacity(view.pool_primary, view.bytes_per_block),
                            _capacity(view.pool_secondary, view.bytes_per_block)) if c is not None]
        if not caps:
            raise ValueError("num_blocks is required when the pools are given as addresses")
        blocks = min(caps)
    primary = _address(view.pool_primary)
    cache = abi.cache_desc(abi.CacheGeometry(blocks, bs, heads, dim, abi.LAYOUT_HND), code, primary, primary)
    cache.pool.memory = abi.MEMORY_DEVICE
    cache.pool.bytes_per_block = view.bytes_per_block
    cache.pool.primary = primary
    cache.pool.secondary = _address(view.pool_secondary) or None

    table = abi.BlockTable()
    table.size = C.sizeof(abi.BlockTable)
    table.format, table.index_dtype = abi.TABLE_KV_OFFSETS, abi.DTYPE_S32
    table.flags = abi.TABLE_FLAG_KVCACHEINDEX
    table.seq_count, table.beam_width, table.max_blocks_per_seq = offsets.shape[0], offsets.shape[1], offsets.shape[3]
    table.indices, table.indices_count = offsets.data_ptr(), offsets.numel()
    return {"cache": cache, "block_table": table, "keepalive": [view]}
