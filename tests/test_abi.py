"""Boundary tests that need no GPU: the validate-only entry points, the exported symbol
list, struct sizes, and a differential run against the reference project's validators."""
import ctypes as C
import os
import random
import subprocess

import numpy as np
import pytest

from kvx_b200 import abi
from kvx_b200._lib import EXPORTS
from oracle.build import REFERENCE_ROOT  # the KVX_REFERENCE_ROOT environment variable, or the usual place

OK, INVALID, UNSUPPORTED = abi.STATUS_OK, abi.STATUS_INVALID_ARGUMENT, abi.STATUS_UNSUPPORTED
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Toy:
    """Host buffers + descriptors of the reference ABI test's toy shapes
    (tests/kvx_abi_test.c:94-188: 2 blocks of 4 tokens, 2 heads of 8, F32, host memory)."""

    def __init__(self, dtype=abi.DTYPE_F32):
        self.geom = abi.CacheGeometry(2, 4, 2, 8)
        self.k = np.zeros(128, np.float32)
        self.v = np.zeros(128, np.float32)
        self.key = np.zeros(64, np.float32)
        self.value = np.zeros(64, np.float32)
        self.slots = np.array([0, 1, 2, 3], np.int64)
        self.table = np.array([0, 1], np.int32)
        self.lens = np.array([4, 4], np.int32)
        self.gk = np.zeros(2 * 4 * 2 * 8, np.float32)
        self.gv = np.zeros(2 * 4 * 2 * 8, np.float32)
        self.dtype = dtype

    def cache(self):
        return abi.cache_desc(self.geom, self.dtype, self.k.ctypes.data, self.v.ctypes.data, abi.MEMORY_HOST)

    def write(self, slots_addr="default", slot_dtype=abi.DTYPE_S64):
        addr = self.slots.ctypes.data if slot_dtype and slots_addr == "default" else slots_addr
        return abi.write_desc(4, 2, 8, self.dtype, self.key.ctypes.data, self.value.ctypes.data, slot_dtype,
                              addr, abi.MEMORY_HOST)

    def gather(self):
        return abi.gather_desc(2, 4, 2, 8, self.dtype, self.gk.ctypes.data, self.gv.ctypes.data, abi.DTYPE_S32,
                               self.table.ctypes.data, 1, self.lens.ctypes.data, abi.MEMORY_HOST)


def test_struct_sizes_match_c_header():
    for cls, n in abi.ABI_SIZES.items():
        assert C.sizeof(cls) == n
    assert abi.TensorDesc.shape.offset == 24 and abi.TensorDesc.stride.offset == 64
    assert abi.TensorDesc.data.offset == 104
    assert abi.CacheDesc.k.offset == 24 and abi.CacheDesc.v.offset == 136 and abi.CacheDesc.pool.offset == 248
    assert abi.WriteDesc.slots.offset == 256 and abi.WriteDesc.k_scale.offset == 288
    assert abi.WriteDesc.k_scale_desc.offset == 304 and abi.WriteDesc.v_scale_desc.offset == 408
    assert abi.GatherDesc.block_table.offset == 256 and abi.GatherDesc.seq_lens.offset == 320
    assert abi.GatherDesc.max_seq_len.offset == 344


def test_library_exports_every_declared_symbol(built_lib):
    for name in EXPORTS:
        assert hasattr(built_lib, name), name
    # every KVX_API prototype in include/*.h must be in EXPORTS (and therefore exported)
    import re
    declared = set()
    for hdr in os.listdir(os.path.join(ROOT, "include")):
        text = open(os.path.join(ROOT, "include", hdr)).read()
        declared |= set(re.findall(r"KVX_API\s+[\w\s\*]+?\b(kvx_\w+)\s*\(", text))
    assert declared, "no prototypes found"
    missing = declared - set(EXPORTS)
    assert not missing, missing


def test_version(built_lib):
    v = abi.Version()
    assert built_lib.kvx_get_version(C.byref(v)) == OK
    assert (v.abi_major, v.abi_minor) == (1, 2) and v.size >= C.sizeof(abi.Version)
    assert built_lib.kvx_get_version(None) == INVALID


def test_cache_desc_validation(built_lib):
    """tests/kvx_abi_test.c:217-251 restated."""
    L, t = built_lib, Toy()
    c = t.cache()
    assert L.kvx_validate_cache_desc(C.byref(c)) == OK
    c.block_size = 0
    assert L.kvx_validate_cache_desc(C.byref(c)) == INVALID
    c = t.cache(); c.size = C.sizeof(c) - 4
    assert L.kvx_validate_cache_desc(C.byref(c)) == INVALID
    c = t.cache(); c.k.stride[0] += 1
    assert L.kvx_validate_cache_desc(C.byref(c)) == UNSUPPORTED
    c = t.cache(); c.v.layout = abi.LAYOUT_HND
    assert L.kvx_validate_cache_desc(C.byref(c)) == INVALID
    # HND_PACKED with pack=3 and head_dim=8 (not divisible) -> INVALID
    g = abi.CacheGeometry(1, 4, 2, 8, abi.LAYOUT_HND_PACKED, 3)
    shape = (1, 2, 8 // 3, 4, 3)
    p = abi.cache_desc(abi.CacheGeometry(1, 4, 2, 8), abi.DTYPE_F16, t.k.ctypes.data, t.v.ctypes.data, abi.MEMORY_HOST)
    for d in (p.k, p.v):
        nd = abi.tensor_desc(d.data, abi.DTYPE_F16, shape, None, abi.LAYOUT_HND_PACKED, abi.MEMORY_HOST)
        C.memmove(C.byref(d), C.byref(nd), C.sizeof(nd))
    assert L.kvx_validate_cache_desc(C.byref(p)) == INVALID
    assert g.pack == 3
    # well-formed HND and HND_PACKED pools
    for layout, pack in ((abi.LAYOUT_HND, 1), (abi.LAYOUT_HND_PACKED, 4)):
        geom = abi.CacheGeometry(2, 4, 2, 8, layout, pack)
        c = abi.cache_desc(geom, abi.DTYPE_BF16, t.k.ctypes.data, t.v.ctypes.data, abi.MEMORY_HOST)
        assert L.kvx_validate_cache_desc(C.byref(c)) == OK
    c = t.cache(); c.k.layout = c.v.layout = abi.LAYOUT_CUSTOM
    assert L.kvx_validate_cache_desc(C.byref(c)) == UNSUPPORTED


def test_write_desc_validation(built_lib):
    """tests/kvx_abi_test.c:253-282 restated."""
    L, t = built_lib, Toy()
    c, w = t.cache(), t.write()
    assert L.kvx_write_kv(C.byref(c), C.byref(w), None) == OK
    w.slots.dtype = abi.DTYPE_U32
    assert L.kvx_write_kv(C.byref(c), C.byref(w), None) == INVALID
    w = t.write(); w.slots.token_count = 3
    assert L.kvx_write_kv(C.byref(c), C.byref(w), None) == INVALID
    w = t.write(slots_addr=None)
    assert L.kvx_write_kv(C.byref(c), C.byref(w), None) == INVALID
    w = t.write(); w.io.key.size = C.sizeof(abi.TensorDesc) - 4
    assert L.kvx_write_kv(C.byref(c), C.byref(w), None) == INVALID
    w = t.write(); w.io.value.stride[0] += 1
    assert L.kvx_write_kv(C.byref(c), C.byref(w), None) == UNSUPPORTED
    w = t.write(); w.io.key.dtype = abi.DTYPE_F16
    assert L.kvx_write_kv(C.byref(c), C.byref(w), None) == INVALID
    assert L.kvx_write_kv(None, C.byref(w), None) == INVALID


def test_gather_desc_validation(built_lib):
    """tests/kvx_abi_test.c:284-313 restated."""
    L, t = built_lib, Toy()
    c, g = t.cache(), t.gather()
    assert L.kvx_gather_kv(C.byref(c), C.byref(g), None) == OK
    g.block_table.indices_count = 1
    assert L.kvx_gather_kv(C.byref(c), C.byref(g), None) == INVALID
    g = t.gather(); g.seq_lens.seq_count = 1
    assert L.kvx_gather_kv(C.byref(c), C.byref(g), None) == INVALID
    g = t.gather(); g.block_table.index_dtype = abi.DTYPE_U32
    assert L.kvx_gather_kv(C.byref(c), C.byref(g), None) == INVALID
    g = t.gather(); g.seq_lens.dtype = abi.DTYPE_S64
    assert L.kvx_gather_kv(C.byref(c), C.byref(g), None) == INVALID
    g = t.gather(); g.io.num_tokens = 7
    assert L.kvx_gather_kv(C.byref(c), C.byref(g), None) == INVALID
    g = t.gather(); g.max_seq_len = 0
    assert L.kvx_gather_kv(C.byref(c), C.byref(g), None) == INVALID
    # RAGGED tables validate but are not executed
    g = t.gather()
    indptr = np.array([0, 1, 2], np.int32)
    g.block_table.format = abi.TABLE_RAGGED
    g.block_table.indptr_dtype = abi.DTYPE_S32
    g.block_table.indptr, g.block_table.indptr_count = indptr.ctypes.data, 3
    assert L.kvx_gather_kv(C.byref(c), C.byref(g), None) == UNSUPPORTED


def test_fp8_pairing_is_accepted_by_validators(built_lib):
    """ABI 1.2: fp8-e4m3 pool with 16/32-bit IO tensors is a legal descriptor set."""
    L, t = built_lib, Toy(abi.DTYPE_F8_E4M3)
    c = t.cache()
    for io in (abi.DTYPE_BF16, abi.DTYPE_F16, abi.DTYPE_F32):
        w = t.write(); w.io.key.dtype = w.io.value.dtype = io
        assert L.kvx_write_kv(C.byref(c), C.byref(w), None) == OK
    w = t.write(); w.io.key.dtype, w.io.value.dtype = abi.DTYPE_BF16, abi.DTYPE_F16
    assert L.kvx_write_kv(C.byref(c), C.byref(w), None) == INVALID


# ------------------------------------------------------------------ differential ---------

def _mutate(rng: random.Random, obj, depth=0):
    """Randomly perturb one scalar field somewhere inside a descriptor."""
    fields = obj._fields_
    name, typ = rng.choice(fields)
    val = getattr(obj, name)
    if isinstance(val, C.Structure):
        return _mutate(rng, val, depth + 1)
    if isinstance(val, C.Array):
        i = rng.randrange(len(val))
        val[i] = rng.choice([0, 1, -1, val[i] + 1, val[i] * 2, 3])
        return f"{name}[{i}]"
    if typ is C.c_void_p:
        if rng.random() < 0.5:
            setattr(obj, name, None)
        return name
    setattr(obj, name, rng.choice([0, 1, 2, 3, 4, 5, 6, 7, 8, 15, (val or 0) + 1, max((val or 0) - 4, 0)]))
    return name


@pytest.mark.skipif(not os.path.exists(os.path.join(REFERENCE_ROOT, "kvx_abi.c")),
                    reason="reference checkout not present")
def test_validators_agree_with_reference_on_mutated_descriptors(built_lib):
    """Same status as the reference's own validators on thousands of randomly corrupted
    descriptor sets (one or two mutated fields each)."""
    from oracle.kvx_oracle import reference
    R = reference()
    assert R is not None
    rng = random.Random(20240607)
    t = Toy()
    checked = 0
    for it in range(6000):
        layout, pack = rng.choice([(abi.LAYOUT_NHD, 1), (abi.LAYOUT_HND, 1), (abi.LAYOUT_HND_PACKED, 4)])
        t.geom = abi.CacheGeometry(2, 4, 2, 8, layout, pack)
        c, w, g = t.cache(), t.write(), t.gather()
        which = rng.choice("cwg")
        target = {"c": c, "w": w, "g": g}[which]
        for _ in range(rng.choice([0, 1, 1, 2])):
            _mutate(rng, target)
        # the fp8 pairing is this ABI's extension; the reference rejects it by design
        if c.k.dtype == abi.DTYPE_F8_E4M3 and c.v.dtype == abi.DTYPE_F8_E4M3:
            continue
        mine = (built_lib.kvx_validate_cache_desc(C.byref(c)), built_lib.kvx_write_kv(C.byref(c), C.byref(w), None),
                built_lib.kvx_gather_kv(C.byref(c), C.byref(g), None))
        ref = (R.kvx_validate_cache_desc(C.byref(c)), R.kvx_write_kv(C.byref(c), C.byref(w), None),
               R.kvx_gather_kv(C.byref(c), C.byref(g), None))
        assert mine == ref, (it, which, mine, ref)
        checked += 1
    assert checked > 4000


@pytest.mark.skipif(not os.path.exists(os.path.join(REFERENCE_ROOT, "tests", "kvx_abi_test.c")),
                    reason="reference checkout not present")
def test_reference_abi_test_program_passes_against_this_header(tmp_path):
    """The reference's own assert-based ABI test, compiled unmodified against this header and
    these validators, exits 0."""
    exe = tmp_path / "kvx_abi_test"
    subprocess.run(["gcc", "-std=c11", "-I" + os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "kvx_b200", "csrc", "kvx_abi.c"),
                    os.path.join(REFERENCE_ROOT, "tests", "kvx_abi_test.c"), "-o", str(exe)], check=True)
    assert subprocess.run([str(exe)]).returncode == 0


def test_torch_operator_library_registers_its_operators(built_lib):
    """libkvx_b200_torch.so builds against the installed torch, loads without a GPU and
    registers the write operator under the name and schema of the reference's vLLM patch
    (reference: patches/vllm/kvx.patch:288-296) plus the gather operator."""
    from kvx_b200 import build, ops
    build.build_torch_ops()
    native = ops.native_ops()
    assert native is not None
    write = native.reshape_and_cache_flash_kvx.default._schema
    names = [a.name for a in write.arguments]
    assert names == ["key", "value", "key_cache", "value_cache", "slot_mapping", "kv_cache_dtype", "k_scale", "v_scale"]
    assert [a.name for a in write.arguments if a.alias_info is not None and a.alias_info.is_write] == \
        ["key_cache", "value_cache"]
    gather = native.gather_kv.default._schema
    assert [a.name for a in gather.arguments][:6] == ["key_cache", "value_cache", "block_table", "seq_lens",
                                                       "key_out", "value_out"]


def test_single_source_build_as_in_the_vllm_patch(tmp_path):
    """The reference's vLLM patch compiles <root>/kernels/kvx_paged_kv.cu as ONE source file with
    <root> and <root>/kernels on the include path and nothing else from this project
    (patches/vllm/kvx.patch:25-32, :43, :53).  The forwarding files must keep that working."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    out = tmp_path / "kvx_paged_kv.o"
    cmd = [nvcc, "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", "-I" + ROOT,
           "-I" + os.path.join(ROOT, "kernels"), "-c", os.path.join(ROOT, "kernels", "kvx_paged_kv.cu"), "-o", str(out)]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert out.stat().st_size > 0
