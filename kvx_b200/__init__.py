"""kvx_b200 -- B200-native paged KV-cache write / gather behind the KVX C ABI.

``abi``   ctypes mirror of ``include/kvx_abi.h`` and descriptor builders
``ops``   torch-tensor front end (the vLLM-patch operator signature and a gather)
``build`` compiles ``lib/libkvx_b200.so`` for sm_100a
"""
from . import abi  # noqa: F401
from ._lib import get_option, lib, lib_path, set_option  # noqa: F401

__all__ = ["abi", "lib", "lib_path", "set_option", "get_option"]
