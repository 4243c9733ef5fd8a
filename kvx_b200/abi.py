"""ctypes mirror of the KVX C ABI (``include/kvx_abi.h``) and descriptor builders.

The structures reproduce the C structs field for field (reference: kvx_abi.h:35-188); the
sizes asserted at import time are the ones the C header freezes.  Builders accept a raw
address plus geometry, so the same code describes host memory (for the CPU checker in the
tests) and device memory (for the CUDA launch layer).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

KVX_MAX_TENSOR_DIMS = 5

# kvx_status_t (reference: kvx_abi.h:26-33)
STATUS_OK, STATUS_INVALID_ARGUMENT, STATUS_UNSUPPORTED = 0, 1, 2
STATUS_OUT_OF_RANGE, STATUS_INCOMPATIBLE, STATUS_INTERNAL_ERROR = 3, 4, 5
STATUS_NAMES = {0: "OK", 1: "INVALID_ARGUMENT", 2: "UNSUPPORTED", 3: "OUT_OF_RANGE",
                4: "INCOMPATIBLE", 5: "INTERNAL_ERROR"}

# kvx_dtype_t (reference: kvx_abi.h:42-54)
DTYPE_INVALID, DTYPE_F16, DTYPE_BF16, DTYPE_F32, DTYPE_F8_E4M3, DTYPE_F8_E5M2 = 0, 1, 2, 3, 4, 5
DTYPE_S32, DTYPE_S64, DTYPE_U32, DTYPE_U64, DTYPE_U8 = 6, 7, 8, 9, 10
DTYPE_BYTES = {DTYPE_F16: 2, DTYPE_BF16: 2, DTYPE_F32: 4, DTYPE_F8_E4M3: 1, DTYPE_F8_E5M2: 1,
               DTYPE_S32: 4, DTYPE_S64: 8}

# kvx_memory_type_t (reference: kvx_abi.h:56-61)
MEMORY_UNKNOWN, MEMORY_HOST, MEMORY_DEVICE, MEMORY_UNIFIED = 0, 1, 2, 3

# kvx_layout_t (reference: kvx_abi.h:63-69)
LAYOUT_INVALID, LAYOUT_NHD, LAYOUT_HND, LAYOUT_HND_PACKED, LAYOUT_CUSTOM = 0, 1, 2, 3, 15

# kvx_block_table_format_t / flags (reference: kvx_abi.h:103-113)
TABLE_INVALID, TABLE_PACKED, TABLE_RAGGED, TABLE_KV_OFFSETS = 0, 1, 2, 3
TABLE_FLAG_NONE, TABLE_FLAG_KVCACHEINDEX = 0, 1

# kvx_scale_granularity_t (reference: kvx_abi.h:154-160)
SCALE_NONE, SCALE_PER_TENSOR, SCALE_PER_BLOCK, SCALE_PER_HEAD, SCALE_PER_BLOCK_HEAD = 0, 1, 2, 3, 4

_Dims = C.c_int64 * KVX_MAX_TENSOR_DIMS


class Version(C.Structure):
    _fields_ = [("size", C.c_uint32), ("abi_major", C.c_uint32), ("abi_minor", C.c_uint32),
                ("abi_patch", C.c_uint32)]


class TensorDesc(C.Structure):
    _fields_ = [("size", C.c_uint32), ("dtype", C.c_int), ("layout", C.c_int), ("memory", C.c_int),
                ("ndim", C.c_uint32), ("shape", _Dims), ("stride", _Dims), ("data", C.c_void_p)]


class PoolDesc(C.Structure):
    _fields_ = [("size", C.c_uint32), ("memory", C.c_int), ("bytes_per_block", C.c_uint32),
                ("primary", C.c_void_p), ("secondary", C.c_void_p)]


class CacheDesc(C.Structure):
    _fields_ = [("size", C.c_uint32), ("num_blocks", C.c_uint32), ("block_size", C.c_uint32),
                ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("k", TensorDesc),
                ("v", TensorDesc), ("pool", PoolDesc)]


class BlockTable(C.Structure):
    _fields_ = [("size", C.c_uint32), ("format", C.c_int), ("index_dtype", C.c_int),
                ("indptr_dtype", C.c_int), ("seq_count", C.c_uint32), ("beam_width", C.c_uint32),
                ("max_blocks_per_seq", C.c_uint32), ("indices", C.c_void_p), ("indptr", C.c_void_p),
                ("indices_count", C.c_uint32), ("indptr_count", C.c_uint32), ("flags", C.c_uint32)]


class SlotMapping(C.Structure):
    _fields_ = [("size", C.c_uint32), ("dtype", C.c_int), ("token_count", C.c_uint32),
                ("invalid_slot", C.c_int64), ("slots", C.c_void_p)]


class SeqLens(C.Structure):
    _fields_ = [("size", C.c_uint32), ("dtype", C.c_int), ("seq_count", C.c_uint32),
                ("lengths", C.c_void_p)]


class KvIoDesc(C.Structure):
    _fields_ = [("size", C.c_uint32), ("key", TensorDesc), ("value", TensorDesc),
                ("num_tokens", C.c_uint32), ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32)]


class ScaleDesc(C.Structure):
    _fields_ = [("size", C.c_uint32), ("dtype", C.c_int), ("granularity", C.c_int),
                ("ndim", C.c_uint32), ("shape", _Dims), ("stride", _Dims), ("data", C.c_void_p)]


class WriteDesc(C.Structure):
    _fields_ = [("size", C.c_uint32), ("io", KvIoDesc), ("slots", SlotMapping),
                ("k_scale", C.c_void_p), ("v_scale", C.c_void_p), ("k_scale_desc", ScaleDesc),
                ("v_scale_desc", ScaleDesc)]


class GatherDesc(C.Structure):
    _fields_ = [("size", C.c_uint32), ("io", KvIoDesc), ("block_table", BlockTable),
                ("seq_lens", SeqLens), ("max_seq_len", C.c_uint32)]


class AttentionDesc(C.Structure):
    """``kvx_attention_desc_t`` (include/kvx_attention.h)."""
    _fields_ = [("size", C.c_uint32), ("num_q_heads", C.c_uint32), ("max_seq_len", C.c_uint32),
                ("scale", C.c_float), ("query", TensorDesc), ("out", TensorDesc),
                ("block_table", BlockTable), ("seq_lens", SeqLens)]


# x86-64 sizes frozen by the C header's static assertions.
ABI_SIZES = {Version: 16, TensorDesc: 112, PoolDesc: 32, CacheDesc: 280, BlockTable: 64,
             SlotMapping: 32, SeqLens: 24, KvIoDesc: 248, ScaleDesc: 104, WriteDesc: 512,
             GatherDesc: 352, AttentionDesc: 328}
for _cls, _bytes in ABI_SIZES.items():
    assert C.sizeof(_cls) == _bytes, (_cls.__name__, C.sizeof(_cls), _bytes)


def dense_strides(shape: Sequence[int]) -> list[int]:
    """Row-major element strides of ``shape``."""
    out, run = [0] * len(shape), 1
    for i in range(len(shape) - 1, -1, -1):
        out[i] = run
        run *= int(shape[i])
    return out


def tensor_desc(addr: int, dtype: int, shape: Sequence[int], stride: Optional[Sequence[int]] = None,
                layout: int = LAYOUT_CUSTOM, memory: int = MEMORY_DEVICE) -> TensorDesc:
    """A ``kvx_tensor_desc_t`` for memory at ``addr``; dense strides unless given."""
    t = TensorDesc()
    t.size = C.sizeof(TensorDesc)
    t.dtype, t.layout, t.memory, t.ndim = dtype, layout, memory, len(shape)
    stride = dense_strides(shape) if stride is None else stride
    for i, (n, s) in enumerate(zip(shape, stride)):
        t.shape[i], t.stride[i] = int(n), int(s)
    t.data = addr
    return t


def page_shape(layout: int, num_blocks: int, block_size: int, heads: int, dim: int,
               pack: int = 1) -> tuple[int, ...]:
    """Extents of a page tensor in the given layout (reference: KVX_SPEC.md:51-58)."""
    if layout == LAYOUT_NHD:
        return (num_blocks, block_size, heads, dim)
    if layout == LAYOUT_HND:
        return (num_blocks, heads, block_size, dim)
    if layout == LAYOUT_HND_PACKED:
        return (num_blocks, heads, dim // pack, block_size, pack)
    raise ValueError(f"no page shape for layout {layout}")


@dataclass
class CacheGeometry:
    """Geometry of one layer's paged cache."""
    num_blocks: int
    block_size: int
    num_kv_heads: int
    head_dim: int
    layout: int = LAYOUT_NHD
    pack: int = 1

    @property
    def shape(self) -> tuple[int, ...]:
        return page_shape(self.layout, self.num_blocks, self.block_size, self.num_kv_heads,
                          self.head_dim, self.pack)

    @property
    def elems(self) -> int:
        return self.num_blocks * self.block_size * self.num_kv_heads * self.head_dim


def cache_desc(geom: CacheGeometry, dtype: int, k_addr: int, v_addr: int,
               memory: int = MEMORY_DEVICE, k_stride: Optional[Sequence[int]] = None,
               v_stride: Optional[Sequence[int]] = None) -> CacheDesc:
    """A ``kvx_cache_desc_t``; canonical contiguous strides unless given."""
    c = CacheDesc()
    c.size = C.sizeof(CacheDesc)
    c.num_blocks, c.block_size = geom.num_blocks, geom.block_size
    c.num_kv_heads, c.head_dim = geom.num_kv_heads, geom.head_dim
    c.k = tensor_desc(k_addr, dtype, geom.shape, k_stride, geom.layout, memory)
    c.v = tensor_desc(v_addr, dtype, geom.shape, v_stride, geom.layout, memory)
    c.pool.size = C.sizeof(PoolDesc)
    return c


def scale_desc(addr: Optional[int], granularity: int, heads: int, stride: int = 1) -> ScaleDesc:
    """A ``kvx_scale_desc_t`` for F32 scales: PER_HEAD ``[heads]`` or PER_TENSOR ``[1]``."""
    s = ScaleDesc()
    s.size = C.sizeof(ScaleDesc)
    s.dtype, s.granularity = DTYPE_F32, granularity
    if addr:
        s.ndim = 1
        s.shape[0] = heads if granularity == SCALE_PER_HEAD else 1
        s.stride[0] = stride
        s.data = addr
    return s


def kv_io_desc(num_tokens: int, heads: int, dim: int, io_dtype: int, key_addr: int, value_addr: int,
               memory: int = MEMORY_DEVICE) -> KvIoDesc:
    """A ``kvx_kv_io_desc_t`` for dense ``[num_tokens, heads, dim]`` K and V."""
    io = KvIoDesc()
    io.size = C.sizeof(KvIoDesc)
    io.num_tokens, io.num_kv_heads, io.head_dim = num_tokens, heads, dim
    io.key = tensor_desc(key_addr, io_dtype, (num_tokens, heads, dim), memory=memory)
    io.value = tensor_desc(value_addr, io_dtype, (num_tokens, heads, dim), memory=memory)
    return io


def write_desc(num_tokens: int, heads: int, dim: int, io_dtype: int, key_addr: int, value_addr: int,
               slot_dtype: int, slots_addr: int, memory: int = MEMORY_DEVICE,
               k_scale: Optional[ScaleDesc] = None, v_scale: Optional[ScaleDesc] = None) -> WriteDesc:
    """A ``kvx_write_desc_t`` for dense ``[num_tokens, heads, dim]`` K and V."""
    w = WriteDesc()
    w.size = C.sizeof(WriteDesc)
    w.io.size = C.sizeof(KvIoDesc)
    w.io.num_tokens, w.io.num_kv_heads, w.io.head_dim = num_tokens, heads, dim
    w.io.key = tensor_desc(key_addr, io_dtype, (num_tokens, heads, dim), memory=memory)
    w.io.value = tensor_desc(value_addr, io_dtype, (num_tokens, heads, dim), memory=memory)
    w.slots.size = C.sizeof(SlotMapping)
    w.slots.dtype, w.slots.token_count, w.slots.invalid_slot = slot_dtype, num_tokens, -1
    w.slots.slots = slots_addr
    w.k_scale_desc = k_scale if k_scale is not None else scale_desc(None, SCALE_NONE, heads)
    w.v_scale_desc = v_scale if v_scale is not None else scale_desc(None, SCALE_NONE, heads)
    return w


def gather_desc(seq_count: int, max_seq_len: int, heads: int, dim: int, io_dtype: int,
                key_addr: int, value_addr: int, index_dtype: int, table_addr: int,
                max_blocks_per_seq: int, lens_addr: int,
                memory: int = MEMORY_DEVICE) -> GatherDesc:
    """A ``kvx_gather_desc_t`` with a PACKED block table and dense 4-D outputs."""
    g = GatherDesc()
    g.size = C.sizeof(GatherDesc)
    g.io.size = C.sizeof(KvIoDesc)
    g.io.num_tokens = (seq_count * max_seq_len) & 0xFFFFFFFF
    g.io.num_kv_heads, g.io.head_dim = heads, dim
    shape = (seq_count, max_seq_len, heads, dim)
    g.io.key = tensor_desc(key_addr, io_dtype, shape, memory=memory)
    g.io.value = tensor_desc(value_addr, io_dtype, shape, memory=memory)
    b = g.block_table
    b.size = C.sizeof(BlockTable)
    b.format, b.index_dtype, b.seq_count, b.beam_width = TABLE_PACKED, index_dtype, seq_count, 1
    b.max_blocks_per_seq = max_blocks_per_seq
    b.indices = table_addr
    b.indices_count = (seq_count * max_blocks_per_seq) & 0xFFFFFFFF
    g.seq_lens.size = C.sizeof(SeqLens)
    g.seq_lens.dtype, g.seq_lens.seq_count, g.seq_lens.lengths = index_dtype, seq_count, lens_addr
    g.max_seq_len = max_seq_len
    return g


def attention_desc(seq_count: int, q_heads: int, dim: int, io_dtype: int, query_addr: int, out_addr: int,
                   scale: float, max_seq_len: int, index_dtype: int, table_addr: int, max_blocks_per_seq: int,
                   lens_addr: int, memory: int = MEMORY_DEVICE) -> AttentionDesc:
    """A ``kvx_attention_desc_t`` with dense ``[seq_count, q_heads, dim]`` query / out and a
    PACKED block table."""
    a = AttentionDesc()
    a.size = C.sizeof(AttentionDesc)
    a.num_q_heads, a.max_seq_len, a.scale = q_heads, max_seq_len, scale
    a.query = tensor_desc(query_addr, io_dtype, (seq_count, q_heads, dim), memory=memory)
    a.out = tensor_desc(out_addr, io_dtype, (seq_count, q_heads, dim), memory=memory)
    b = a.block_table
    b.size = C.sizeof(BlockTable)
    b.format, b.index_dtype, b.seq_count, b.beam_width = TABLE_PACKED, index_dtype, seq_count, 1
    b.max_blocks_per_seq = max_blocks_per_seq
    b.indices = table_addr
    b.indices_count = (seq_count * max_blocks_per_seq) & 0xFFFFFFFF
    a.seq_lens.size = C.sizeof(SeqLens)
    a.seq_lens.dtype, a.seq_lens.seq_count, a.seq_lens.lengths = index_dtype, seq_count, lens_addr
    return a
