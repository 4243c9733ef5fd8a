"""Status codes of the launch layer for malformed descriptors.  Every case here is rejected
(or found empty) on the host before any kernel launch, so no GPU is needed.  The matrix
follows the reference launchers' evaluation order (kernels/kvx_paged_kv.cu:320-376,
:497-559, :768-863)."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

from kvx_b200 import abi
from oracle.build import REFERENCE_ROOT

OK, INVALID, UNSUPPORTED = abi.STATUS_OK, abi.STATUS_INVALID_ARGUMENT, abi.STATUS_UNSUPPORTED
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FAKE = 0x10000  # a non-NULL "device" address that is never dereferenced on these paths


def cache(dtype=abi.DTYPE_BF16, layout=abi.LAYOUT_NHD, pack=1):
    return abi.cache_desc(abi.CacheGeometry(4, 4, 2, 8, layout, pack), dtype, FAKE, FAKE)


def write(dtype=abi.DTYPE_BF16, tokens=4, slot_dtype=abi.DTYPE_S64):
    return abi.write_desc(tokens, 2, 8, dtype, FAKE, FAKE, slot_dtype, FAKE)


def gather(dtype=abi.DTYPE_BF16, index=abi.DTYPE_S32):
    return abi.gather_desc(2, 4, 2, 8, dtype, FAKE, FAKE, index, FAKE, 1, FAKE)


def W(L, c, w, name="kvx_launch_write_kv"):
    return getattr(L, name)(C.byref(c) if c is not None else None, C.byref(w) if w is not None else None, None)


def P(L, c, w, tps, name="kvx_launch_write_kv_prefill"):
    return getattr(L, name)(C.byref(c), C.byref(w), tps, None)


def G(L, c, g, name="kvx_launch_gather_kv"):
    return getattr(L, name)(C.byref(c) if c is not None else None, C.byref(g) if g is not None else None, None)


def test_write_launcher_statuses(built_lib):
    L = built_lib
    assert W(L, None, write()) == INVALID and W(L, cache(), None) == INVALID
    c = cache(); c.v.dtype = abi.DTYPE_F16
    assert W(L, c, write()) == INVALID                      # K/V cache dtype differ (dispatcher)
    for bad in (abi.DTYPE_F8_E5M2, abi.DTYPE_S32, abi.DTYPE_INVALID):
        assert W(L, cache(bad), write()) == UNSUPPORTED     # dtype the dispatcher does not know
    for field in ("size",):
        w = write(); w.size -= 4
        assert W(L, cache(), w) == INVALID
        w = write(); w.io.size -= 4
        assert W(L, cache(), w) == INVALID
        w = write(); w.slots.size -= 4
        assert W(L, cache(), w) == INVALID
    assert W(L, cache(), write(), "kvx_launch_write_kv_f16") == UNSUPPORTED   # pinned to another dtype
    assert W(L, cache(), write(abi.DTYPE_F16)) == UNSUPPORTED                 # io dtype != cache dtype
    w = write(); w.io.head_dim = 16
    assert W(L, cache(), w) == INVALID
    w = write(); w.io.key.ndim = 4
    assert W(L, cache(), w) == INVALID
    w = write(); w.io.value.shape[0] = 5
    assert W(L, cache(), w) == INVALID
    w = write(); w.io.key.stride[0] = 8                       # rows overlap
    assert W(L, cache(), w) == UNSUPPORTED
    w = write(); w.io.value.stride[1] = 9                     # heads not dense
    assert W(L, cache(), w) == UNSUPPORTED
    # (a token pitch ABOVE heads * dim is accepted here, unlike in the reference: GPU tests)
    w = write(); w.slots.token_count = 3
    assert W(L, cache(), w) == INVALID
    c = cache(); c.k.layout = c.v.layout = abi.LAYOUT_CUSTOM
    assert W(L, c, write()) == UNSUPPORTED
    c = cache(layout=abi.LAYOUT_HND_PACKED, pack=4); c.k.shape[4] = 3
    assert W(L, c, write()) == INVALID
    c = cache(layout=abi.LAYOUT_HND_PACKED, pack=4); c.v.shape[4] = 0
    assert W(L, c, write()) == INVALID
    # nothing to move: OK without a launch, even with an unknown slot dtype
    w = write(tokens=0, slot_dtype=abi.DTYPE_U32)
    assert W(L, cache(), w) == OK
    assert W(L, cache(), write(slot_dtype=abi.DTYPE_U32)) == INVALID
    # stricter than the reference: NULL buffers are refused instead of faulting on the device
    w = write(); w.io.key.data = None
    assert W(L, cache(), w) == INVALID
    w = write(); w.slots.slots = None
    assert W(L, cache(), w) == INVALID


def test_prefill_launcher_statuses(built_lib):
    L = built_lib
    # tests/kvx_kernel_test.cu:607-618: zeroed descriptors, tokens_per_seq = 0 -> INVALID
    c, w = abi.CacheDesc(), abi.WriteDesc()
    for code in (abi.DTYPE_F32, abi.DTYPE_F16, abi.DTYPE_BF16):
        c.k.dtype = c.v.dtype = code
        assert P(L, c, w, 0) == INVALID
    assert P(L, cache(), write(), -1) == INVALID
    assert P(L, cache(), write(), 3) == INVALID             # 4 tokens not divisible by 3
    assert P(L, cache(), write(abi.DTYPE_F16), 2) == UNSUPPORTED
    assert P(L, cache(), write(), 2, "kvx_launch_write_kv_prefill_f32") == UNSUPPORTED
    w = write(); w.size -= 4
    assert P(L, cache(), w, 2) == INVALID
    assert P(L, cache(), write(tokens=0), 2) == OK


def test_gather_launcher_statuses(built_lib):
    L = built_lib
    assert G(L, None, gather()) == INVALID and G(L, cache(), None) == INVALID
    c = cache(); c.v.dtype = abi.DTYPE_F32
    assert G(L, c, gather()) == INVALID
    assert G(L, cache(abi.DTYPE_F8_E4M3), gather()) == UNSUPPORTED  # fp8 needs the scale-taking entry
    for attr in ("size", "io.size", "block_table.size", "seq_lens.size"):
        g = gather()
        obj = g
        *path, last = attr.split(".")
        for p in path:
            obj = getattr(obj, p)
        setattr(obj, last, getattr(obj, last) - 4)
        assert G(L, cache(), g) == INVALID, attr
    assert G(L, cache(), gather(), "kvx_launch_gather_kv_f32") == UNSUPPORTED
    assert G(L, cache(), gather(abi.DTYPE_F32)) == UNSUPPORTED
    g = gather(); g.block_table.format = abi.TABLE_RAGGED      # RAGGED is executed here; without indptr it is malformed
    assert G(L, cache(), g) == INVALID
    # KV_OFFSETS is executed here too: the validate-only entry point's rules (reference:
    # kvx_abi.c:161-189), then UNSUPPORTED for more than one beam
    def offsets(beams=1):
        g = gather()
        b = g.block_table
        b.format, b.flags, b.beam_width = abi.TABLE_KV_OFFSETS, abi.TABLE_FLAG_KVCACHEINDEX, beams
        b.indices_count = b.seq_count * beams * 2 * b.max_blocks_per_seq
        c = cache()
        c.pool.bytes_per_block, c.pool.primary = 64, FAKE
        return c, g
    c, g = offsets(); g.block_table.flags = 0
    assert G(L, c, g) == INVALID
    c, g = offsets(); c.pool.primary = None
    assert G(L, c, g) == INVALID
    c, g = offsets(); c.pool.bytes_per_block = 0
    assert G(L, c, g) == INVALID
    c, g = offsets(); g.block_table.indices_count -= 1
    assert G(L, c, g) == INVALID
    c, g = offsets(); c.block_size = 3; c.k.shape[1] = c.v.shape[1] = 3
    assert G(L, c, g) == INVALID                            # block_size must be a power of two
    c, g = offsets(2)
    assert G(L, c, g) == UNSUPPORTED
    g = gather(); g.io.num_kv_heads = 3
    assert G(L, cache(), g) == INVALID
    g = gather(); g.seq_lens.seq_count = 1
    assert G(L, cache(), g) == INVALID
    g = gather(); g.io.key.shape[1] = 5
    assert G(L, cache(), g) == INVALID
    g = gather(); g.io.value.stride[1] = 17
    assert G(L, cache(), g) == UNSUPPORTED
    g = gather(); g.seq_lens.dtype = abi.DTYPE_S64          # table S32 + lens S64
    assert G(L, cache(), g) == INVALID
    g = gather(index=abi.DTYPE_U32)
    assert G(L, cache(), g) == INVALID
    g = gather(); g.block_table.indices = None
    assert G(L, cache(), g) == INVALID


def test_fp8_launcher_statuses(built_lib):
    L = built_lib
    c = cache(abi.DTYPE_F8_E4M3)
    w = write(abi.DTYPE_BF16)
    assert W(L, c, w) == UNSUPPORTED                        # no scale supplied
    assert W(L, c, write(abi.DTYPE_F8_E4M3)) == UNSUPPORTED
    w = write(abi.DTYPE_BF16)
    w.k_scale_desc = abi.scale_desc(FAKE, abi.SCALE_PER_BLOCK, 2)
    w.v_scale_desc = abi.scale_desc(FAKE, abi.SCALE_PER_HEAD, 2)
    assert W(L, c, w) == UNSUPPORTED                        # granularity not implemented
    w.k_scale_desc = abi.scale_desc(FAKE, abi.SCALE_PER_HEAD, 3)
    assert W(L, c, w) == UNSUPPORTED                        # wrong number of heads
    w = write(abi.DTYPE_BF16, tokens=0)
    w.k_scale = w.v_scale = FAKE
    assert W(L, c, w) == OK                                 # per-tensor scalars accepted; empty batch
    g = gather(abi.DTYPE_BF16)
    ks = abi.scale_desc(FAKE, abi.SCALE_PER_HEAD, 2)
    none = abi.scale_desc(None, abi.SCALE_NONE, 2)
    assert L.kvx_launch_gather_kv_f8e4m3(C.byref(c), C.byref(g), C.byref(ks), C.byref(none), None) == UNSUPPORTED
    assert L.kvx_launch_gather_kv_f8e4m3(C.byref(cache()), C.byref(g), C.byref(ks), C.byref(ks), None) == UNSUPPORTED
    assert L.kvx_launch_kv_scales(None, abi.SCALE_PER_HEAD, FAKE, FAKE, FAKE, 4096, None) == INVALID
    w = write(abi.DTYPE_BF16)
    assert L.kvx_launch_kv_scales(C.byref(w.io), abi.SCALE_PER_BLOCK, FAKE, FAKE, 0x10000, 4096, None) == UNSUPPORTED
    assert L.kvx_launch_kv_scales(C.byref(w.io), abi.SCALE_PER_HEAD, FAKE, FAKE, 0x10000, 8, None) == INVALID


def test_attention_launcher_statuses_before_any_launch(built_lib):
    """kvx_launch_paged_attention_decode: every verdict that is reached without touching a device."""
    L = built_lib

    def attn(**kw):
        a = abi.attention_desc(2, 4, 8, abi.DTYPE_BF16, FAKE, FAKE, 0.5, 16, abi.DTYPE_S32, FAKE, 1, FAKE)
        for k, v in kw.items():
            setattr(a, k, v)
        return a

    none = abi.scale_desc(None, abi.SCALE_NONE, 2)

    def A(c, a):
        return L.kvx_launch_paged_attention_decode(C.byref(c) if c is not None else None,
                                                   C.byref(a) if a is not None else None, C.byref(none), C.byref(none),
                                                   None, 0, None)

    assert A(None, attn()) == INVALID and A(cache(), None) == INVALID
    a = attn(); a.size -= 4
    assert A(cache(), a) == INVALID
    assert A(cache(), attn(num_q_heads=3)) == INVALID            # not a multiple of the 2 KV heads
    assert A(cache(), attn(num_q_heads=0)) == INVALID
    assert A(cache(), attn(max_seq_len=0)) == INVALID
    a = attn(); a.block_table.format = abi.TABLE_RAGGED
    assert A(cache(), a) == UNSUPPORTED
    a = attn(); a.out.dtype = abi.DTYPE_F16
    assert A(cache(), a) == UNSUPPORTED
    assert A(cache(abi.DTYPE_F16), attn()) == UNSUPPORTED          # cache and query types differ
    assert A(cache(abi.DTYPE_F8_E4M3), attn()) == UNSUPPORTED      # fp8 cache without scales
    a = attn(); a.query.shape[2] = 16
    assert A(cache(), a) == INVALID
    a = attn(); a.out.stride[1] = 9
    assert A(cache(), a) == UNSUPPORTED
    a = attn(); a.seq_lens.dtype = abi.DTYPE_S64
    assert A(cache(), a) == INVALID
    a = attn(); a.block_table.seq_count = a.seq_lens.seq_count = 0
    a.query.shape[0] = a.out.shape[0] = 0
    a.query.stride[0] = a.out.stride[0] = 32
    assert A(cache(), a) == OK                                   # no sequence: nothing to do
    assert L.kvx_paged_attention_workspace_bytes(0, 4, 2, 8, 16) == 0
    small = L.kvx_paged_attention_workspace_bytes(2, 4, 2, 8, 16)
    big = L.kvx_paged_attention_workspace_bytes(2, 4, 2, 8, 100000)
    assert 0 < small < big


def test_options_and_counter(built_lib):
    import kvx_b200
    assert kvx_b200.get_option("gather_path") in (0, 1, 2)
    old = kvx_b200.get_option("write_unroll")
    kvx_b200.set_option("write_unroll", 2)
    assert kvx_b200.get_option("write_unroll") == 2
    kvx_b200.set_option("write_unroll", old)
    with pytest.raises(KeyError):
        kvx_b200.set_option("no_such_option", 1)
    # the knobs the GPU tests and the benchmark switch, with their built-in values
    for name, value in (("attn_carry", 1), ("attn_min_items", 0), ("packed_fill_halves", 1), ("packed_lines_variant", 0),
                        ("packed_tiles", 1), ("packed_tile_tokens", 32), ("host_pair_kv", 1), ("gather_rect_items", 40000),
                        ("gather_ctas_per_sm", 256), ("bulk_test_stall", 0)):
        assert kvx_b200.get_option(name) == value, name
    built_lib.kvx_b200_reset_launch_count()
    assert built_lib.kvx_b200_launch_count() == 0


DIFFERENTIAL = r"""
import ctypes as C, random, sys
sys.path.insert(0, %(root)r); sys.path.insert(0, %(tests)r)
import kvx_b200
from kvx_b200 import abi
from oracle.kvx_oracle import reference
from test_abi import _mutate
from test_launch_status import cache, write, gather
L, R = kvx_b200.lib(), reference()
assert R is not None
rng = random.Random(99)
n = 0
for it in range(8000):
    layout, pack = rng.choice([(abi.LAYOUT_NHD, 1), (abi.LAYOUT_HND, 1), (abi.LAYOUT_HND_PACKED, 4)])
    dt = rng.choice([abi.DTYPE_F32, abi.DTYPE_F16, abi.DTYPE_BF16])
    c, w, g = cache(dt, layout, pack), write(dt), gather(dt)
    for _ in range(rng.choice([1, 1, 2])):
        _mutate(rng, rng.choice([c, w, g]))
    if abi.DTYPE_F8_E4M3 in (c.k.dtype, c.v.dtype) or g.block_table.format in (abi.TABLE_RAGGED, abi.TABLE_KV_OFFSETS):
        continue  # this ABI's extensions
    if w.io.key.stride[0] > 16 or w.io.value.stride[0] > 16:
        continue  # token rows further apart than heads * dim: accepted by this library's write launchers
    tps = rng.choice([0, 1, 2, 3, 4])
    for name, args in (("kvx_launch_write_kv", (C.byref(c), C.byref(w), None)),
                       ("kvx_launch_write_kv_bf16", (C.byref(c), C.byref(w), None)),
                       ("kvx_launch_write_kv_prefill", (C.byref(c), C.byref(w), tps, None)),
                       ("kvx_launch_gather_kv", (C.byref(c), C.byref(g), None)),
                       ("kvx_launch_gather_kv_f16", (C.byref(c), C.byref(g), None))):
        mine, ref = getattr(L, name)(*args), getattr(R, name)(*args)
        # 5 = a launch was attempted (there is no device in this process).  Where the
        # reference would launch, this library launches too or refuses a NULL / oversized
        # argument; every host-side verdict must be identical.
        ok = (mine == ref) or (ref == 5 and mine == 1)
        assert ok, (it, name, mine, ref)
        n += 1
print("compared", n)
"""


@pytest.mark.skipif(not os.path.exists(os.path.join(REFERENCE_ROOT, "kernels", "kvx_paged_kv.cu")),
                    reason="reference checkout not present")
def test_launcher_statuses_agree_with_reference(built_lib):
    """Thousands of randomly corrupted descriptor sets through this launch layer and through
    the reference's own (compiled unmodified): same host-side verdicts.  Runs in a child
    process with all CUDA devices hidden, so a descriptor that survives validation can only
    produce a failed launch, never touch a GPU."""
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    code = DIFFERENTIAL % {"root": ROOT, "tests": os.path.join(ROOT, "tests")}
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "compared" in r.stdout
