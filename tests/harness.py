"""Shared machinery of the parity tests: build one write/gather case as raw bit patterns in
numpy, run it through the CPU checker (host descriptors), through the CUDA library (device
descriptors, via the C ABI) or through the reference project's own kernels, and hand back
the resulting bytes for comparison.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from kvx_b200 import abi

NP_OF = {abi.DTYPE_F16: np.uint16, abi.DTYPE_BF16: np.uint16, abi.DTYPE_F32: np.uint32,
         abi.DTYPE_F8_E4M3: np.uint8, abi.DTYPE_S32: np.int32, abi.DTYPE_S64: np.int64}


def f32_to_bits(x: np.ndarray, code: int) -> np.ndarray:
    """float32 values -> raw bit patterns of the element type (round to nearest even)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if code == abi.DTYPE_F32:
        return x.view(np.uint32).copy()
    if code == abi.DTYPE_F16:
        return x.astype(np.float16).view(np.uint16).copy()
    if code == abi.DTYPE_BF16:
        u = x.view(np.uint32).astype(np.uint64)
        return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    raise ValueError(code)


def bits_to_f32(b: np.ndarray, code: int) -> np.ndarray:
    if code == abi.DTYPE_F32:
        return b.view(np.float32)
    if code == abi.DTYPE_F16:
        return b.view(np.float16).astype(np.float32)
    if code == abi.DTYPE_BF16:
        return (b.astype(np.uint32) << 16).view(np.float32)
    raise ValueError(code)


def random_bits(rng: np.random.Generator, shape, code: int) -> np.ndarray:
    """Arbitrary bit patterns (NaN payloads, -0, denormals included): a copy must keep them."""
    dt = NP_OF[code]
    return rng.integers(0, np.iinfo(dt).max, size=shape, dtype=dt, endpoint=True)


def canonical_strides(geom: abi.CacheGeometry) -> list[int]:
    return abi.dense_strides(geom.shape)


def extent(shape, stride) -> int:
    """Elements a strided tensor spans."""
    return 1 + sum((int(n) - 1) * int(s) for n, s in zip(shape, stride)) if all(shape) else 0


@dataclass
class Case:
    geom: abi.CacheGeometry
    cache_dtype: int
    io_dtype: int
    key: np.ndarray            # [T, H, D] raw bits
    value: np.ndarray
    slots: np.ndarray          # [T] int32 / int64
    cache_k: np.ndarray        # 1-D raw bits, the page pool before the call
    cache_v: np.ndarray
    k_stride: Optional[list[int]] = None
    v_stride: Optional[list[int]] = None
    k_scale: Optional[np.ndarray] = None   # float32 [H] or [1]
    v_scale: Optional[np.ndarray] = None
    scale_gran: int = abi.SCALE_NONE
    # gather side
    table: Optional[np.ndarray] = None     # [S, max_blocks] int32 / int64
    lens: Optional[np.ndarray] = None      # [S]
    max_seq_len: int = 0
    out_k: Optional[np.ndarray] = None     # [S, Lmax, H, D] raw bits before the call
    out_v: Optional[np.ndarray] = None
    # RAGGED form of the block table (one page id per cached token); used instead of `table`
    ragged: Optional[np.ndarray] = None    # [sum(counts)] int32 / int64
    indptr: Optional[np.ndarray] = None    # [S + 1] int32 / int64
    # KV_OFFSETS form (TensorRT-LLM): K and V pages live in block pools; used instead of `table`
    # for the lookup and instead of cache_k / cache_v for the data
    kv_offsets: Optional[np.ndarray] = None      # [S, beam_width, 2, max_blocks] int32 (bit 31 = secondary)
    pool_primary: Optional[np.ndarray] = None    # 1-D raw bits
    pool_secondary: Optional[np.ndarray] = None  # 1-D raw bits or None
    pool_block_bytes: int = 0
    # un-padded output (kvx_launch_gather_kv_varlen): out_k / out_v are [rows, H, D] and
    # sequence s starts at row out_indptr[s]
    out_indptr: Optional[np.ndarray] = None      # [S + 1] int32 / int64
    # token rows of key / value further apart than heads * dim: key / value are then [T, pitch]
    # arrays whose first heads * dim columns are the row (elements; 0 = dense [T, H, D])
    key_pitch: int = 0
    value_pitch: int = 0
    # HND_PACKED pools whose V tensor has a pack factor of its own (vLLM / TGI "paged" caches: K in
    # 16-byte pack groups, V [blocks, heads, dim, block_size] = pack 1); 0 = the geometry's pack
    v_pack: int = 0
    note: str = ""
    keep: list = field(default_factory=list)

    @property
    def T(self) -> int:
        return int(self.slots.shape[0])


def index_code(a: np.ndarray) -> int:
    return abi.DTYPE_S32 if a.dtype == np.int32 else abi.DTYPE_S64


def _addr(a) -> int:
    """Address of a numpy array or a torch tensor."""
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    return a.data_ptr()


def _scale(case: Case, arr, which: str) -> abi.ScaleDesc:
    if arr is None:
        return abi.scale_desc(None, abi.SCALE_NONE, case.geom.num_kv_heads)
    return abi.scale_desc(_addr(arr), case.scale_gran, case.geom.num_kv_heads)


def descriptors(case: Case, bufs: dict, memory: int):
    """(cache, write, gather, k_scale, v_scale) descriptors over the buffers in ``bufs``
    (numpy arrays for the host, torch tensors for the device)."""
    g = case.geom
    if case.kv_offsets is not None:
        base = _addr(bufs["pool_primary"])
        cache = abi.cache_desc(g, case.cache_dtype, base, base, memory, case.k_stride, case.v_stride)
        cache.pool.memory = memory
        cache.pool.bytes_per_block = case.pool_block_bytes
        cache.pool.primary = base
        cache.pool.secondary = _addr(bufs["pool_secondary"]) if "pool_secondary" in bufs else None
    else:
        cache = abi.cache_desc(g, case.cache_dtype, _addr(bufs["cache_k"]), _addr(bufs["cache_v"]), memory,
                               case.k_stride, case.v_stride)
        if case.v_pack:
            import dataclasses
            gv = dataclasses.replace(g, pack=case.v_pack)
            cache.v = abi.tensor_desc(_addr(bufs["cache_v"]), case.cache_dtype, gv.shape, case.v_stride, g.layout, memory)
    ks, vs = _scale(case, bufs.get("k_scale"), "k"), _scale(case, bufs.get("v_scale"), "v")
    write = abi.write_desc(case.T, g.num_kv_heads, g.head_dim, case.io_dtype, _addr(bufs["key"]),
                           _addr(bufs["value"]), index_code(case.slots), _addr(bufs["slots"]), memory, ks, vs)
    if case.key_pitch:
        write.io.key.stride[0] = case.key_pitch
    if case.value_pitch:
        write.io.value.stride[0] = case.value_pitch
    gather = None
    if case.table is not None:
        S, mb = case.table.shape
        gather = abi.gather_desc(S, case.max_seq_len, g.num_kv_heads, g.head_dim, case.io_dtype,
                                 _addr(bufs["out_k"]), _addr(bufs["out_v"]), index_code(case.table),
                                 _addr(bufs["table"]), mb, _addr(bufs["lens"]), memory)
        if case.ragged is not None:
            b = gather.block_table
            b.format = abi.TABLE_RAGGED
            b.indptr_dtype = index_code(case.indptr)
            b.indices, b.indices_count = _addr(bufs["ragged"]), int(case.ragged.shape[0])
            b.indptr, b.indptr_count = _addr(bufs["indptr"]), int(case.indptr.shape[0])
        if case.out_indptr is not None:
            rows = int(case.out_k.shape[0])
            gather.io.num_tokens = rows
            for t, buf in ((gather.io.key, "out_k"), (gather.io.value, "out_v")):
                new = abi.tensor_desc(_addr(bufs[buf]), case.io_dtype, (rows, g.num_kv_heads, g.head_dim), memory=memory)
                C.memmove(C.byref(t), C.byref(new), C.sizeof(new))
        if case.kv_offsets is not None:
            b = gather.block_table
            b.format, b.flags = abi.TABLE_KV_OFFSETS, abi.TABLE_FLAG_KVCACHEINDEX
            b.beam_width, b.max_blocks_per_seq = int(case.kv_offsets.shape[1]), int(case.kv_offsets.shape[3])
            b.indices, b.indices_count = _addr(bufs["kv_offsets"]), int(case.kv_offsets.size)
    return cache, write, gather, ks, vs


_FIELDS = ("key", "value", "slots", "cache_k", "cache_v", "k_scale", "v_scale", "table", "lens", "out_k", "out_v",
           "ragged", "indptr", "kv_offsets", "pool_primary", "pool_secondary", "out_indptr")


def host_buffers(case: Case) -> dict:
    return {f: getattr(case, f).copy() for f in _FIELDS if getattr(case, f) is not None}


def device_buffers(case: Case, device="cuda") -> dict:
    import torch
    out = {}
    for f in _FIELDS:
        a = getattr(case, f)
        if a is None:
            continue
        if a.size == 0:
            # keep a real (non-NULL) allocation behind empty tensors
            out[f] = torch.zeros(16, dtype=torch.uint8, device=device)
            continue
        out[f] = torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1).copy()).to(device)
    return out


def back(t, like: np.ndarray) -> np.ndarray:
    """Device bytes -> numpy array shaped and typed like ``like``."""
    if like.size == 0:
        return like.copy()
    return t.cpu().numpy().view(like.dtype).reshape(like.shape)


# ---------------------------------------------------------------------------- runners ----

def oracle_write(case: Case):
    from oracle.kvx_oracle import oracle
    b = host_buffers(case)
    cache, write, _, _, _ = descriptors(case, b, abi.MEMORY_HOST)
    st = oracle().kvx_oracle_write_kv(C.byref(cache), C.byref(write))
    return st, b["cache_k"], b["cache_v"]


def oracle_gather(case: Case, cache_k=None, cache_v=None):
    from oracle.kvx_oracle import oracle
    b = host_buffers(case)
    if cache_k is not None:
        b["cache_k"], b["cache_v"] = cache_k.copy(), cache_v.copy()
    cache, _, gather, ks, vs = descriptors(case, b, abi.MEMORY_HOST)
    if case.out_indptr is not None:
        st = oracle().kvx_oracle_gather_kv_varlen(C.byref(cache), C.byref(gather), _addr(b["out_indptr"]),
                                                  index_code(case.out_indptr), C.byref(ks), C.byref(vs))
    else:
        st = oracle().kvx_oracle_gather_kv(C.byref(cache), C.byref(gather), C.byref(ks), C.byref(vs))
    return st, b["out_k"], b["out_v"]


WRITE_ENTRIES = {abi.DTYPE_F32: "f32", abi.DTYPE_F16: "f16", abi.DTYPE_BF16: "bf16"}


def _call_write(L, case: Case, cache, write, entry: str, tokens_per_seq: int, stream):
    suffix = WRITE_ENTRIES.get(case.cache_dtype, "")
    if entry == "dispatch":
        return L.kvx_launch_write_kv(C.byref(cache), C.byref(write), stream)
    if entry == "typed":
        fn = L.kvx_launch_write_kv_f8e4m3 if case.cache_dtype == abi.DTYPE_F8_E4M3 else getattr(L, "kvx_launch_write_kv_" + suffix)
        return fn(C.byref(cache), C.byref(write), stream)
    if entry == "prefill":
        return L.kvx_launch_write_kv_prefill(C.byref(cache), C.byref(write), tokens_per_seq, stream)
    if entry == "prefill_typed":
        return getattr(L, "kvx_launch_write_kv_prefill_" + suffix)(C.byref(cache), C.byref(write), tokens_per_seq, stream)
    raise ValueError(entry)


def gpu_write(case: Case, entry: str = "dispatch", tokens_per_seq: int = 1, L=None, stream=None):
    """Run the write through a C-ABI library on the current CUDA device."""
    import torch
    import kvx_b200
    L = L or kvx_b200.lib()
    b = device_buffers(case)
    cache, write, _, _, _ = descriptors(case, b, abi.MEMORY_DEVICE)
    st = _call_write(L, case, cache, write, entry, tokens_per_seq, stream)
    torch.cuda.synchronize()
    return st, back(b["cache_k"], case.cache_k), back(b["cache_v"], case.cache_v)


def gpu_gather(case: Case, cache_k=None, cache_v=None, entry: str = "dispatch", L=None, stream=None):
    import torch
    import kvx_b200
    L = L or kvx_b200.lib()
    src = case
    if cache_k is not None:
        import dataclasses
        src = dataclasses.replace(case, cache_k=cache_k, cache_v=cache_v)
    b = device_buffers(src)
    cache, _, gather, ks, vs = descriptors(src, b, abi.MEMORY_DEVICE)
    if case.out_indptr is not None:
        st = L.kvx_launch_gather_kv_varlen(C.byref(cache), C.byref(gather), _addr(b["out_indptr"]),
                                           index_code(case.out_indptr), C.byref(ks), C.byref(vs), stream)
    elif case.cache_dtype == abi.DTYPE_F8_E4M3:
        st = L.kvx_launch_gather_kv_f8e4m3(C.byref(cache), C.byref(gather), C.byref(ks), C.byref(vs), stream)
    elif entry == "dispatch":
        st = L.kvx_launch_gather_kv(C.byref(cache), C.byref(gather), stream)
    else:
        st = getattr(L, "kvx_launch_gather_kv_" + WRITE_ENTRIES[case.cache_dtype])(C.byref(cache), C.byref(gather), stream)
    torch.cuda.synchronize()
    return st, back(b["out_k"], case.out_k), back(b["out_v"], case.out_v)
