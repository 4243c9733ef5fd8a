"""Torch-tensor front end of the C-ABI library.

The write operator keeps the name, argument order and checks of the operator the
reference's vLLM patch registers (``reshape_and_cache_flash_kvx``, reference:
patches/vllm/kvx.patch:176-275): it fills the ABI descriptors from tensor sizes and strides
without canonicalising them, passes torch's current CUDA stream and raises when the status
is not OK.  Torch is used for device memory and streams only; all data movement happens in
``libkvx_b200.so``.  Nothing here falls back to PyTorch indexing.

When ``lib/libkvx_b200_torch.so`` is built, calls on 4-D caches go through the operators it
registers with torch's dispatcher (``torch.ops.kvx_b200.*``), which do the same descriptor
filling in C++ and cost a few microseconds of host time per call; otherwise, and for 5-D
packed caches and the prefill entry point, the descriptors are filled here through ctypes.
"""
from __future__ import annotations

import ctypes as C
import os
import re
from typing import Optional

import torch

from . import abi
from ._lib import lib

_FLOAT_CODES = {torch.float16: abi.DTYPE_F16, torch.bfloat16: abi.DTYPE_BF16,
                torch.float32: abi.DTYPE_F32}
_INDEX_CODES = {torch.int32: abi.DTYPE_S32, torch.int64: abi.DTYPE_S64}
_FP8_TORCH = (torch.float8_e4m3fn, torch.uint8)


class KvxError(RuntimeError):
    """A launcher returned a status other than ``KVX_STATUS_OK``."""

    def __init__(self, what: str, status: int):
        super().__init__(f"{what} failed with status={status} ({abi.STATUS_NAMES.get(status, '?')})")
        self.status = status


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_NATIVE = None          # torch.ops.kvx_b200 once libkvx_b200_torch.so is loaded; False if it is not built
_NO_SCALE: dict = {}    # one empty float32 tensor per device, standing for "no scale"
_STATUS_RE = re.compile(r"(kvx [\w ]+?) failed with status=(\d+)")


def native_ops():
    """``torch.ops.kvx_b200`` (the dispatcher-registered operators of ``csrc/kvx_torch_ops.cpp``),
    or None when that library has not been built; the ctypes route below is then used."""
    global _NATIVE
    if _NATIVE is None:
        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libkvx_b200_torch.so")
        if os.path.exists(path):
            lib()  # libkvx_b200.so first, so that the operator library binds to the same copy
            torch.ops.load_library(path)
            _NATIVE = torch.ops.kvx_b200
        else:
            _NATIVE = False
    return _NATIVE or None


def _scale_arg(scale: Optional[torch.Tensor], device: torch.device) -> torch.Tensor:
    if scale is not None:
        return scale
    t = _NO_SCALE.get(device)
    if t is None:
        t = _NO_SCALE[device] = torch.empty(0, dtype=torch.float32, device=device)
    return t


def _call_native(op, *args) -> None:
    try:
        op(*args)
    except RuntimeError as exc:
        m = _STATUS_RE.search(str(exc))
        if m is None:
            raise
        raise KvxError(m.group(1), int(m.group(2))) from None


def _cache_code(t: torch.Tensor, kv_cache_dtype: str) -> int:
    if kv_cache_dtype in ("fp8", "fp8_e4m3"):
        if t.dtype not in _FP8_TORCH:
            raise TypeError("an fp8 cache must be a float8_e4m3fn or uint8 tensor")
        return abi.DTYPE_F8_E4M3
    if kv_cache_dtype != "auto":
        raise ValueError(f"unsupported kv_cache_dtype {kv_cache_dtype!r}")
    if t.dtype not in _FLOAT_CODES:
        raise TypeError(f"unsupported cache dtype {t.dtype}")
    return _FLOAT_CODES[t.dtype]


def cache_desc_from_tensors(key_cache: torch.Tensor, value_cache: torch.Tensor,
                            kv_cache_dtype: str = "auto", heads: Optional[int] = None,
                            layout: Optional[int] = None) -> abi.CacheDesc:
    """Describe a pair of 4-D (NHD / HND) or 5-D (HND_PACKED) page tensors.

    For 4-D tensors the layout is inferred unless given.  The reference's operator decides
    by one stride (NHD when stride(2) == head_dim, reference: patches/vllm/kvx.patch:132-135,
    :222-229), which misreads a contiguous ``[blocks, heads, block_size, dim]`` tensor; the
    rule here agrees with it wherever it is right and also accepts that tensor and vLLM's
    permuted view of HND memory: ``stride(1) < stride(2)`` is a ``[blocks, block_size, heads,
    dim]`` view of HND memory; otherwise the axis whose size equals ``heads`` names the
    layout; when ``block_size == heads`` (or ``heads`` is not given) the reference's stride
    rule decides.
    """
    if key_cache.shape != value_cache.shape:
        raise ValueError("key/value cache shape mismatch")
    code = _cache_code(key_cache, kv_cache_dtype)
    k_shape, k_stride = list(key_cache.shape), list(key_cache.stride())
    v_shape, v_stride = list(value_cache.shape), list(value_cache.stride())
    if key_cache.dim() == 5:
        layout = abi.LAYOUT_HND_PACKED
        nb, heads, dhi, bs, pack = key_cache.shape
        dim = dhi * pack
    else:
        dim = key_cache.shape[3]
        if layout is None and k_stride[1] < k_stride[2]:
            layout = abi.LAYOUT_HND  # a logical-NHD view of HND memory: describe the memory
            for shape, stride in ((k_shape, k_stride), (v_shape, v_stride)):
                shape[1], shape[2] = shape[2], shape[1]
                stride[1], stride[2] = stride[2], stride[1]
        elif layout is None:
            nhd, hnd = k_shape[2] == heads, k_shape[1] == heads
            if heads is not None and nhd != hnd:
                layout = abi.LAYOUT_NHD if nhd else abi.LAYOUT_HND
            else:
                layout = abi.LAYOUT_NHD if k_stride[2] == dim else abi.LAYOUT_HND
        if layout == abi.LAYOUT_NHD:
            nb, bs, heads, _ = k_shape
        else:
            nb, heads, bs, _ = k_shape
    c = abi.CacheDesc()
    c.size = C.sizeof(abi.CacheDesc)
    c.num_blocks, c.block_size, c.num_kv_heads, c.head_dim = nb, bs, heads, dim
    c.k = abi.tensor_desc(key_cache.data_ptr(), code, k_shape, k_stride, layout)
    c.v = abi.tensor_desc(value_cache.data_ptr(), code, v_shape, v_stride, layout)
    c.pool.size = C.sizeof(abi.PoolDesc)
    return c


def _scale_desc(scale: Optional[torch.Tensor], heads: int) -> abi.ScaleDesc:
    if scale is None:
        return abi.scale_desc(None, abi.SCALE_NONE, heads)
    if scale.dtype != torch.float32 or not scale.is_cuda:
        raise TypeError("scales must be float32 CUDA tensors")
    if scale.numel() == 1:
        return abi.scale_desc(scale.data_ptr(), abi.SCALE_PER_TENSOR, heads)
    if scale.dim() == 1 and scale.numel() == heads:
        return abi.scale_desc(scale.data_ptr(), abi.SCALE_PER_HEAD, heads, scale.stride(0))
    raise ValueError("a scale must have 1 or num_kv_heads elements")


def reshape_and_cache_flash_kvx(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor,
                                value_cache: torch.Tensor, slot_mapping: torch.Tensor,
                                kv_cache_dtype: str = "auto", k_scale: Optional[torch.Tensor] = None,
                                v_scale: Optional[torch.Tensor] = None,
                                tokens_per_seq: Optional[int] = None) -> None:
    """Scatter ``key`` / ``value`` ``[num_tokens, heads, dim]`` into the paged caches.

    ``slot_mapping[t] = block * block_size + offset``; negative slots are padding and are
    skipped.  ``kv_cache_dtype="auto"`` copies bits; ``"fp8"`` quantises to e4m3 with
    ``k_scale`` / ``v_scale`` (1 or ``heads`` float32 values).  ``tokens_per_seq`` selects
    the prefill entry point, whose result is identical.
    """
    native = native_ops() if tokens_per_seq is None and key_cache.dim() == 4 else None
    if native is not None:
        dev = key.device
        _call_native(native.reshape_and_cache_flash_kvx, key, value, key_cache, value_cache, slot_mapping,
                     kv_cache_dtype, _scale_arg(k_scale, dev), _scale_arg(v_scale, dev))
        return
    if not (key.is_cuda and value.is_cuda and key_cache.is_cuda and value_cache.is_cuda):
        raise ValueError("key/value and cache tensors must be CUDA tensors")
    if key.dtype != value.dtype or key.dtype not in _FLOAT_CODES:
        raise TypeError("key/value dtype mismatch or unsupported")
    if key.dim() != 3 or value.shape != key.shape:
        raise ValueError("key/value must be [num_tokens, num_heads, head_dim]")
    if slot_mapping.dtype not in _INDEX_CODES or slot_mapping.dim() != 1:
        raise TypeError("slot_mapping must be a 1-D int32 or int64 tensor")
    num_tokens = slot_mapping.shape[0]
    heads, dim = key.shape[1], key.shape[2]
    cache = cache_desc_from_tensors(key_cache, value_cache, kv_cache_dtype, heads)
    w = abi.WriteDesc()
    w.size = C.sizeof(abi.WriteDesc)
    w.io.size = C.sizeof(abi.KvIoDesc)
    w.io.num_tokens, w.io.num_kv_heads, w.io.head_dim = num_tokens, heads, dim
    code = _FLOAT_CODES[key.dtype]
    shape = (num_tokens, heads, dim)  # the patch sizes the batch by slot_mapping (kvx.patch:208)
    w.io.key = abi.tensor_desc(key.data_ptr(), code, shape, key.stride(), abi.LAYOUT_INVALID)
    w.io.value = abi.tensor_desc(value.data_ptr(), code, shape, value.stride(), abi.LAYOUT_INVALID)
    w.slots.size = C.sizeof(abi.SlotMapping)
    w.slots.dtype, w.slots.token_count = _INDEX_CODES[slot_mapping.dtype], num_tokens
    w.slots.invalid_slot = -1
    w.slots.slots = slot_mapping.data_ptr()
    w.k_scale_desc = _scale_desc(k_scale, heads)
    w.v_scale_desc = _scale_desc(v_scale, heads)
    if tokens_per_seq is None:
        status = lib().kvx_launch_write_kv(C.byref(cache), C.byref(w), _stream())
    else:
        status = lib().kvx_launch_write_kv_prefill(C.byref(cache), C.byref(w), int(tokens_per_seq), _stream())
    if status != abi.STATUS_OK:
        raise KvxError("kvx cache write", status)


def gather_kv(key_cache: torch.Tensor, value_cache: torch.Tensor, block_table: torch.Tensor,
              seq_lens: torch.Tensor, key_out: torch.Tensor, value_out: torch.Tensor,
              kv_cache_dtype: str = "auto", k_scale: Optional[torch.Tensor] = None,
              v_scale: Optional[torch.Tensor] = None) -> None:
    """Materialise ``out[s, tok] = cache[block_table[s, tok // bs], tok % bs]`` for
    ``tok < seq_lens[s]``; other positions of ``key_out`` / ``value_out`` stay untouched.

    ``block_table`` is ``[seq_count, max_blocks_per_seq]`` (int32 or int64, same dtype as
    ``seq_lens``); outputs are dense ``[seq_count, max_seq_len, heads, dim]``.
    """
    native = native_ops() if key_cache.dim() == 4 else None
    if native is not None:
        dev = key_out.device
        _call_native(native.gather_kv, key_cache, value_cache, block_table, seq_lens, key_out, value_out,
                     kv_cache_dtype, _scale_arg(k_scale, dev), _scale_arg(v_scale, dev))
        return
    if block_table.dim() != 2 or not block_table.is_contiguous():
        raise ValueError("block_table must be a contiguous [seq_count, max_blocks_per_seq] tensor")
    if block_table.dtype not in _INDEX_CODES or seq_lens.dtype != block_table.dtype:
        raise TypeError("block_table and seq_lens must share an int32 or int64 dtype")
    if key_out.dim() != 4 or key_out.shape != value_out.shape or key_out.dtype not in _FLOAT_CODES:
        raise ValueError("outputs must be [seq_count, max_seq_len, heads, dim] float tensors")
    seqs, max_len, heads, dim = key_out.shape
    cache = cache_desc_from_tensors(key_cache, value_cache, kv_cache_dtype, heads)
    g = abi.gather_desc(seqs, max_len, heads, dim, _FLOAT_CODES[key_out.dtype], key_out.data_ptr(),
                        value_out.data_ptr(), _INDEX_CODES[block_table.dtype], block_table.data_ptr(),
                        block_table.shape[1], seq_lens.data_ptr())
    for t, src in ((g.io.key, key_out), (g.io.value, value_out)):
        for i, s in enumerate(src.stride()):
            t.stride[i] = s
    g.block_table.seq_count = block_table.shape[0]
    g.seq_lens.seq_count = seq_lens.shape[0]
    if cache.k.dtype == abi.DTYPE_F8_E4M3:
        ks, vs = _scale_desc(k_scale, heads), _scale_desc(v_scale, heads)
        status = lib().kvx_launch_gather_kv_f8e4m3(C.byref(cache), C.byref(g), C.byref(ks), C.byref(vs), _stream())
    else:
        status = lib().kvx_launch_gather_kv(C.byref(cache), C.byref(g), _stream())
    if status != abi.STATUS_OK:
        raise KvxError("kvx cache gather", status)


def gather_kv_varlen(key_cache: torch.Tensor, value_cache: torch.Tensor, block_table: torch.Tensor,
                     seq_lens: torch.Tensor, out_indptr: torch.Tensor, key_out: torch.Tensor,
                     value_out: torch.Tensor, max_seq_len: int, kv_cache_dtype: str = "auto",
                     k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None) -> None:
    """The gather into un-padded ``[rows, heads, dim]`` outputs (the form variable-length
    attention kernels take, with ``out_indptr`` as their cumulative sequence lengths): token
    ``tok`` of sequence ``s`` goes to row ``out_indptr[s] + tok`` for ``tok < min(seq_lens[s],
    max_seq_len, out_indptr[s + 1] - out_indptr[s])``; other rows stay untouched."""
    if block_table.dim() != 2 or not block_table.is_contiguous():
        raise ValueError("block_table must be a contiguous [seq_count, max_blocks_per_seq] tensor")
    if block_table.dtype not in _INDEX_CODES or seq_lens.dtype != block_table.dtype:
        raise TypeError("block_table and seq_lens must share an int32 or int64 dtype")
    if out_indptr.dtype not in _INDEX_CODES or out_indptr.numel() != block_table.shape[0] + 1:
        raise ValueError("out_indptr must hold seq_count + 1 int32 or int64 row numbers")
    if key_out.dim() != 3 or key_out.shape != value_out.shape or key_out.dtype not in _FLOAT_CODES:
        raise ValueError("outputs must be [rows, heads, dim] float tensors")
    rows, heads, dim = key_out.shape
    seqs = block_table.shape[0]
    cache = cache_desc_from_tensors(key_cache, value_cache, kv_cache_dtype, heads)
    g = abi.gather_desc(seqs, max_seq_len, heads, dim, _FLOAT_CODES[key_out.dtype], key_out.data_ptr(),
                        value_out.data_ptr(), _INDEX_CODES[block_table.dtype], block_table.data_ptr(),
                        block_table.shape[1], seq_lens.data_ptr())
    code = _FLOAT_CODES[key_out.dtype]
    g.io.num_tokens = rows
    g.io.key = abi.tensor_desc(key_out.data_ptr(), code, key_out.shape, key_out.stride(), abi.LAYOUT_INVALID)
    g.io.value = abi.tensor_desc(value_out.data_ptr(), code, value_out.shape, value_out.stride(), abi.LAYOUT_INVALID)
    g.seq_lens.seq_count = seq_lens.shape[0]
    ks, vs = _scale_desc(k_scale, heads), _scale_desc(v_scale, heads)
    status = lib().kvx_launch_gather_kv_varlen(C.byref(cache), C.byref(g), out_indptr.data_ptr(),
                                               _INDEX_CODES[out_indptr.dtype], C.byref(ks), C.byref(vs), _stream())
    if status != abi.STATUS_OK:
        raise KvxError("kvx cache gather", status)


def paged_attention_decode(query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                           block_table: torch.Tensor, seq_lens: torch.Tensor, scale: float,
                           max_seq_len: Optional[int] = None, out: Optional[torch.Tensor] = None,
                           workspace: Optional[torch.Tensor] = None, kv_cache_dtype: str = "auto",
                           k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None,
                           num_kv_heads: Optional[int] = None) -> torch.Tensor:
    """Decode attention that reads the paged cache in place (``include/kvx_attention.h``):
    ``query`` ``[seq_count, q_heads, dim]`` attends over each sequence's cached tokens, found
    through ``block_table`` / ``seq_lens`` as the gather finds them; returns ``out`` (same shape
    and dtype).  ``max_seq_len`` bounds the context (default: all the table can address).
    ``workspace`` is reusable uint8 scratch of :func:`attention_workspace_bytes` bytes; it is
    allocated per call when not given.  ``num_kv_heads`` names the cache's head axis when the
    layout cannot be read off the strides (a contiguous ``[blocks, heads, block_size, dim]``
    tensor)."""
    if query.dim() != 3 or query.dtype not in _FLOAT_CODES or not query.is_contiguous():
        raise ValueError("query must be a contiguous [seq_count, q_heads, dim] float tensor")
    if block_table.dim() != 2 or not block_table.is_contiguous():
        raise ValueError("block_table must be a contiguous [seq_count, max_blocks_per_seq] tensor")
    if block_table.dtype not in _INDEX_CODES or seq_lens.dtype != block_table.dtype:
        raise TypeError("block_table and seq_lens must share an int32 or int64 dtype")
    seqs, q_heads, dim = query.shape
    if out is None:
        out = torch.empty_like(query)
    cache = cache_desc_from_tensors(key_cache, value_cache, kv_cache_dtype, num_kv_heads)
    if max_seq_len is None:
        max_seq_len = block_table.shape[1] * cache.block_size
    need = lib().kvx_paged_attention_workspace_bytes(seqs, q_heads, cache.num_kv_heads, dim, max_seq_len)
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=query.device)
    native = native_ops() if key_cache.dim() == 4 else None
    if native is not None:
        dev = query.device
        _call_native(native.paged_attention_decode, out, query, key_cache, value_cache, block_table, seq_lens,
                     float(scale), int(max_seq_len), int(cache.num_kv_heads), workspace, kv_cache_dtype,
                     _scale_arg(k_scale, dev), _scale_arg(v_scale, dev))
        return out
    a = abi.attention_desc(seqs, q_heads, dim, _FLOAT_CODES[query.dtype], query.data_ptr(), out.data_ptr(),
                           float(scale), int(max_seq_len), _INDEX_CODES[block_table.dtype], block_table.data_ptr(),
                           block_table.shape[1], seq_lens.data_ptr())
    a.seq_lens.seq_count = seq_lens.shape[0]
    ks, vs = _scale_desc(k_scale, cache.num_kv_heads), _scale_desc(v_scale, cache.num_kv_heads)
    status = lib().kvx_launch_paged_attention_decode(
        C.byref(cache), C.byref(a), C.byref(ks), C.byref(vs), workspace.data_ptr(),
        workspace.numel() * workspace.element_size(), _stream())
    if status != abi.STATUS_OK:
        raise KvxError("kvx paged attention", status)
    return out


def attention_workspace_bytes(seq_count: int, q_heads: int, kv_heads: int, dim: int, max_seq_len: int) -> int:
    return lib().kvx_paged_attention_workspace_bytes(seq_count, q_heads, kv_heads, dim, max_seq_len)


def scales_workspace(heads: int, device: torch.device) -> torch.Tensor:
    """Zeroed scratch for :func:`compute_kv_scales`; reusable across calls on one stream."""
    n = lib().kvx_kv_scales_workspace_bytes(heads)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def compute_kv_scales(key: torch.Tensor, value: torch.Tensor, per_head: bool = True,
                      workspace: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """``absmax / 448`` of K and of V per head (or per tensor), as float32 CUDA tensors."""
    if key.dim() != 3 or key.shape != value.shape or key.dtype != value.dtype:
        raise ValueError("key/value must be matching [num_tokens, heads, dim] tensors")
    tokens, heads, dim = key.shape
    n = heads if per_head else 1
    k_out = torch.empty(n, dtype=torch.float32, device=key.device)
    v_out = torch.empty(n, dtype=torch.float32, device=key.device)
    if workspace is None:
        workspace = scales_workspace(heads, key.device)
    io = abi.KvIoDesc()
    io.size = C.sizeof(abi.KvIoDesc)
    io.num_tokens, io.num_kv_heads, io.head_dim = tokens, heads, dim
    code = _FLOAT_CODES[key.dtype]
    io.key = abi.tensor_desc(key.data_ptr(), code, key.shape, key.stride(), abi.LAYOUT_INVALID)
    io.value = abi.tensor_desc(value.data_ptr(), code, value.shape, value.stride(), abi.LAYOUT_INVALID)
    status = lib().kvx_launch_kv_scales(C.byref(io), abi.SCALE_PER_HEAD if per_head else abi.SCALE_PER_TENSOR,
                                        k_out.data_ptr(), v_out.data_ptr(), workspace.data_ptr(),
                                        workspace.numel(), _stream())
    if status != abi.STATUS_OK:
        raise KvxError("kvx scale reduction", status)
    return k_out, v_out
