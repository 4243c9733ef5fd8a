"""Loads ``libkvx_b200.so`` and declares its C signatures.  There is no fallback: if the
library is missing, :func:`lib` raises."""
from __future__ import annotations

import ctypes as C
import os

from . import abi

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libkvx_b200.so")
_lib = None

# Every symbol include/kvx_abi.h, include/kvx_paged_kv.h and include/kvx_host.h declare.
EXPORTS = [
    "kvx_get_version", "kvx_validate_cache_desc", "kvx_write_kv", "kvx_gather_kv",
    "kvx_launch_write_kv", "kvx_launch_write_kv_prefill", "kvx_launch_gather_kv",
    "kvx_launch_write_kv_f32", "kvx_launch_write_kv_f16", "kvx_launch_write_kv_bf16",
    "kvx_launch_write_kv_prefill_f32", "kvx_launch_write_kv_prefill_f16",
    "kvx_launch_write_kv_prefill_bf16", "kvx_launch_gather_kv_f32", "kvx_launch_gather_kv_f16",
    "kvx_launch_gather_kv_bf16", "kvx_launch_write_kv_f8e4m3", "kvx_launch_gather_kv_f8e4m3",
    "kvx_launch_gather_kv_varlen", "kvx_kv_scales_workspace_bytes", "kvx_launch_kv_scales", "kvx_launch_kv_scales_static",
    "kvx_b200_launch_count", "kvx_b200_device_error",
    "kvx_b200_reset_launch_count", "kvx_b200_set_option", "kvx_b200_get_option",
    "kvx_host_pipe_create", "kvx_host_pipe_destroy", "kvx_host_write_kv", "kvx_host_gather_kv",
    "kvx_host_pipe_sync", "kvx_host_pipe_traffic",
    "kvx_paged_attention_workspace_bytes", "kvx_launch_paged_attention_decode",
]


def lib_path() -> str:
    return _LIB_PATH


def lib() -> C.CDLL:
    """The loaded C-ABI library.  Raises ``RuntimeError`` when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(f"{_LIB_PATH} is missing: build it with `python -m kvx_b200.build` "
                           "(there is no CPU or PyTorch fallback for the KV write/gather path)")
    L = C.CDLL(_LIB_PATH)
    P = C.POINTER
    st = C.c_int
    L.kvx_get_version.argtypes, L.kvx_get_version.restype = [P(abi.Version)], st
    L.kvx_validate_cache_desc.argtypes, L.kvx_validate_cache_desc.restype = [P(abi.CacheDesc)], st
    for name in ("kvx_write_kv", "kvx_launch_write_kv", "kvx_launch_write_kv_f32",
                 "kvx_launch_write_kv_f16", "kvx_launch_write_kv_bf16", "kvx_launch_write_kv_f8e4m3"):
        f = getattr(L, name)
        f.argtypes, f.restype = [P(abi.CacheDesc), P(abi.WriteDesc), C.c_void_p], st
    for name in ("kvx_launch_write_kv_prefill", "kvx_launch_write_kv_prefill_f32",
                 "kvx_launch_write_kv_prefill_f16", "kvx_launch_write_kv_prefill_bf16"):
        f = getattr(L, name)
        f.argtypes, f.restype = [P(abi.CacheDesc), P(abi.WriteDesc), C.c_int32, C.c_void_p], st
    for name in ("kvx_gather_kv", "kvx_launch_gather_kv", "kvx_launch_gather_kv_f32",
                 "kvx_launch_gather_kv_f16", "kvx_launch_gather_kv_bf16"):
        f = getattr(L, name)
        f.argtypes, f.restype = [P(abi.CacheDesc), P(abi.GatherDesc), C.c_void_p], st
    L.kvx_launch_gather_kv_f8e4m3.argtypes = [P(abi.CacheDesc), P(abi.GatherDesc), P(abi.ScaleDesc),
                                              P(abi.ScaleDesc), C.c_void_p]
    L.kvx_launch_gather_kv_f8e4m3.restype = st
    L.kvx_launch_gather_kv_varlen.argtypes = [P(abi.CacheDesc), P(abi.GatherDesc), C.c_void_p, C.c_int,
                                              P(abi.ScaleDesc), P(abi.ScaleDesc), C.c_void_p]
    L.kvx_launch_gather_kv_varlen.restype = st
    L.kvx_paged_attention_workspace_bytes.argtypes = [C.c_uint32] * 5
    L.kvx_paged_attention_workspace_bytes.restype = C.c_size_t
    L.kvx_launch_paged_attention_decode.argtypes = [P(abi.CacheDesc), P(abi.AttentionDesc), P(abi.ScaleDesc),
                                                    P(abi.ScaleDesc), C.c_void_p, C.c_size_t, C.c_void_p]
    L.kvx_launch_paged_attention_decode.restype = st
    L.kvx_kv_scales_workspace_bytes.argtypes, L.kvx_kv_scales_workspace_bytes.restype = [C.c_uint32], C.c_size_t
    L.kvx_launch_kv_scales.argtypes = [P(abi.KvIoDesc), C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_size_t, C.c_void_p]
    L.kvx_launch_kv_scales.restype = st
    L.kvx_launch_kv_scales_static.argtypes = [P(abi.KvIoDesc), C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    L.kvx_launch_kv_scales_static.restype = st
    L.kvx_b200_launch_count.argtypes, L.kvx_b200_launch_count.restype = [], C.c_uint64
    L.kvx_b200_device_error.argtypes, L.kvx_b200_device_error.restype = [C.c_int], C.c_int
    L.kvx_b200_reset_launch_count.argtypes, L.kvx_b200_reset_launch_count.restype = [], None
    L.kvx_b200_set_option.argtypes, L.kvx_b200_set_option.restype = [C.c_char_p, C.c_int64], C.c_int
    L.kvx_b200_get_option.argtypes, L.kvx_b200_get_option.restype = [C.c_char_p], C.c_int64
    L.kvx_host_pipe_create.argtypes = [C.c_size_t, C.c_uint32, C.c_uint32, P(C.c_void_p)]
    L.kvx_host_pipe_create.restype = st
    L.kvx_host_pipe_destroy.argtypes, L.kvx_host_pipe_destroy.restype = [C.c_void_p], None
    L.kvx_host_write_kv.argtypes, L.kvx_host_write_kv.restype = [C.c_void_p, P(abi.CacheDesc), P(abi.WriteDesc)], st
    L.kvx_host_gather_kv.argtypes = [C.c_void_p, P(abi.CacheDesc), P(abi.GatherDesc), P(abi.ScaleDesc), P(abi.ScaleDesc)]
    L.kvx_host_gather_kv.restype = st
    L.kvx_host_pipe_sync.argtypes, L.kvx_host_pipe_sync.restype = [C.c_void_p], st
    L.kvx_host_pipe_traffic.argtypes = [C.c_void_p, P(C.c_uint64), P(C.c_uint64)]
    L.kvx_host_pipe_traffic.restype = None
    _lib = L
    return L


def set_option(name: str, value: int) -> None:
    if lib().kvx_b200_set_option(name.encode(), int(value)) != 0:
        raise KeyError(name)


def get_option(name: str) -> int:
    return int(lib().kvx_b200_get_option(name.encode()))
