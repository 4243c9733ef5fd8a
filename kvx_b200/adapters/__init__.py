"""Engine adapters: normalised views of other engines' paged caches -> KVX descriptors.

The reference ships these two modules as stubs that raise NotImplementedError
(reference: adapters/tgi_adapter.py, adapters/trt_llm_adapter.py, contract in
adapters/README.md).  Here they build real descriptors, and :func:`write` / :func:`gather`
run them through the C-ABI launchers.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import abi
from .._lib import lib
from ..ops import KvxError, _FLOAT_CODES, _INDEX_CODES, _scale_desc, _stream


def io_desc(key: torch.Tensor, value: torch.Tensor, rows: int) -> abi.KvIoDesc:
    """Dense ``[..., heads, dim]`` K / V tensors with ``rows`` leading rows in total."""
    if key.dtype != value.dtype or key.dtype not in _FLOAT_CODES or key.shape != value.shape:
        raise TypeError("key/value must be matching float16 / bfloat16 / float32 tensors")
    io = abi.KvIoDesc()
    io.size = C.sizeof(abi.KvIoDesc)
    io.num_tokens, io.num_kv_heads, io.head_dim = rows, key.shape[-2], key.shape[-1]
    code = _FLOAT_CODES[key.dtype]
    io.key = abi.tensor_desc(key.data_ptr(), code, key.shape, key.stride(), abi.LAYOUT_INVALID)
    io.value = abi.tensor_desc(value.data_ptr(), code, value.shape, value.stride(), abi.LAYOUT_INVALID)
    return io


def write(descs: dict, key: torch.Tensor, value: torch.Tensor, k_scale: Optional[torch.Tensor] = None,
          v_scale: Optional[torch.Tensor] = None) -> None:
    """Scatter ``key`` / ``value`` ``[num_tokens, heads, dim]`` through ``descs["slot_mapping"]``."""
    slots = descs["slot_mapping"]
    w = abi.WriteDesc()
    w.size = C.sizeof(abi.WriteDesc)
    w.io = io_desc(key, value, slots.token_count)
    w.io.key.shape[0] = w.io.value.shape[0] = slots.token_count
    w.slots = slots
    w.k_scale_desc = _scale_desc(k_scale, key.shape[1])
    w.v_scale_desc = _scale_desc(v_scale, key.shape[1])
    status = lib().kvx_launch_write_kv(C.byref(descs["cache"]), C.byref(w), _stream())
    if status != abi.STATUS_OK:
        raise KvxError("kvx cache write", status)


def gather(descs: dict, seq_lens: torch.Tensor, key_out: torch.Tensor, value_out: torch.Tensor,
           k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None) -> None:
    """Materialise the cached tokens of every sequence into ``key_out`` / ``value_out``
    ``[seq_count, max_seq_len, heads, dim]`` through ``descs["block_table"]`` (any format).

    ``seq_lens`` must have the table's index dtype.  A RAGGED table built without ``indptr``
    gets the prefix sums of ``seq_lens`` (computed on the device, kept alive in ``descs``)."""
    table = descs["block_table"]
    if seq_lens.dtype not in _INDEX_CODES or _INDEX_CODES[seq_lens.dtype] != table.index_dtype:
        raise TypeError("seq_lens must have the block table's index dtype")
    seqs, max_len = key_out.shape[0], key_out.shape[1]
    g = abi.GatherDesc()
    g.size = C.sizeof(abi.GatherDesc)
    g.io = io_desc(key_out, value_out, seqs * max_len)
    g.block_table = table
    if table.format == abi.TABLE_RAGGED and not table.indptr:
        zero = torch.zeros(1, dtype=seq_lens.dtype, device=seq_lens.device)
        indptr = torch.cat([zero, torch.cumsum(seq_lens, 0).to(seq_lens.dtype)])
        descs.setdefault("keepalive", []).append(indptr)
        g.block_table.indptr_dtype = table.index_dtype
        g.block_table.indptr, g.block_table.indptr_count = indptr.data_ptr(), indptr.numel()
    g.seq_lens.size = C.sizeof(abi.SeqLens)
    g.seq_lens.dtype, g.seq_lens.seq_count = table.index_dtype, seq_lens.shape[0]
    g.seq_lens.lengths = seq_lens.data_ptr()
    g.max_seq_len = max_len
    cache = descs["cache"]
    if cache.k.dtype == abi.DTYPE_F8_E4M3:
        ks, vs = _scale_desc(k_scale, key_out.shape[2]), _scale_desc(v_scale, key_out.shape[2])
        status = lib().kvx_launch_gather_kv_f8e4m3(C.byref(cache), C.byref(g), C.byref(ks), C.byref(vs), _stream())
    else:
        status = lib().kvx_launch_gather_kv(C.byref(cache), C.byref(g), _stream())
    if status != abi.STATUS_OK:
        raise KvxError("kvx cache gather", status)
