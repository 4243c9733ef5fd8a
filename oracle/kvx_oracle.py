"""ctypes access to the CPU checker -- TEST INFRASTRUCTURE, NOT PRODUCT CODE."""
from __future__ import annotations

import ctypes as C
import os

from kvx_b200 import abi

from . import build as _build

_oracle = None
_ref = None


def oracle() -> C.CDLL:
    """The C restatement (``kvx_oracle.c`` + ``kvx_cpu_baseline.c``), built on demand."""
    global _oracle
    if _oracle is None:
        L = C.CDLL(_build.build_oracle())
        P = C.POINTER
        L.kvx_oracle_write_kv.argtypes = [P(abi.CacheDesc), P(abi.WriteDesc)]
        L.kvx_oracle_gather_kv.argtypes = [P(abi.CacheDesc), P(abi.GatherDesc), P(abi.ScaleDesc), P(abi.ScaleDesc)]
        L.kvx_oracle_gather_kv_varlen.argtypes = [P(abi.CacheDesc), P(abi.GatherDesc), C.c_void_p, C.c_int,
                                                  P(abi.ScaleDesc), P(abi.ScaleDesc)]
        L.kvx_oracle_gather_kv_varlen.restype = C.c_int
        L.kvx_oracle_paged_attention_decode.argtypes = [P(abi.CacheDesc), P(abi.AttentionDesc), P(abi.ScaleDesc),
                                                        P(abi.ScaleDesc)]
        L.kvx_oracle_paged_attention_decode.restype = C.c_int
        L.kvx_oracle_kv_scales.argtypes = [P(abi.KvIoDesc), C.c_int, C.c_void_p, C.c_void_p]
        L.kvx_oracle_e4m3_from_f32.argtypes, L.kvx_oracle_e4m3_from_f32.restype = [C.c_float], C.c_uint8
        L.kvx_oracle_e4m3_to_f32.argtypes, L.kvx_oracle_e4m3_to_f32.restype = [C.c_uint8], C.c_float
        L.kvx_cpu_baseline_write_kv.argtypes = [P(abi.CacheDesc), P(abi.WriteDesc), C.c_int]
        L.kvx_cpu_baseline_gather_kv.argtypes = [P(abi.CacheDesc), P(abi.GatherDesc), C.c_int]
        _oracle = L
    return _oracle


def reference() -> C.CDLL | None:
    """The reference project's own validators + CUDA launch layer, compiled unmodified
    (``_ref/libkvx_ref.so``); ``None`` where it could not be built and is not present."""
    global _ref
    if _ref is None:
        path = _build.build_reference()
        if path is None or not os.path.exists(path):
            return None
        L = C.CDLL(path)
        P = C.POINTER
        L.kvx_validate_cache_desc.argtypes = [P(abi.CacheDesc)]
        for name in ("kvx_write_kv", "kvx_launch_write_kv", "kvx_launch_write_kv_f32",
                     "kvx_launch_write_kv_f16", "kvx_launch_write_kv_bf16"):
            getattr(L, name).argtypes = [P(abi.CacheDesc), P(abi.WriteDesc), C.c_void_p]
        for name in ("kvx_launch_write_kv_prefill", "kvx_launch_write_kv_prefill_f32",
                     "kvx_launch_write_kv_prefill_f16", "kvx_launch_write_kv_prefill_bf16"):
            getattr(L, name).argtypes = [P(abi.CacheDesc), P(abi.WriteDesc), C.c_int32, C.c_void_p]
        for name in ("kvx_gather_kv", "kvx_launch_gather_kv", "kvx_launch_gather_kv_f32",
                     "kvx_launch_gather_kv_f16", "kvx_launch_gather_kv_bf16"):
            getattr(L, name).argtypes = [P(abi.CacheDesc), P(abi.GatherDesc), C.c_void_p]
        _ref = L
    return _ref
