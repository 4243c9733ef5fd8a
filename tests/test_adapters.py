"""Engine adapters on CPU tensors: the descriptors they build pass the ABI validators, carry
the right format / layout / counts, and malformed views are refused (reference contract:
adapters/README.md; the reference's own adapters are stubs that raise NotImplementedError)."""
import ctypes as C

import pytest
import torch

from kvx_b200 import abi
from kvx_b200.adapters import tgi_adapter, trt_llm_adapter


def _tgi(layout="flashinfer", dtype=torch.float16, ragged=None, **kw):
    nb, bs, H, D = 8, 16, 4, 64
    if layout in ("flashinfer", "flashdecoding"):
        k = torch.zeros(nb, bs, H, D, dtype=dtype); v = k.clone()
    elif layout == "ipex":
        k = torch.zeros(nb, H, bs, D, dtype=dtype); v = k.clone()
    else:
        x = 16 // k_elem(dtype)
        k = torch.zeros(nb, H, D // x, bs, x, dtype=dtype); v = torch.zeros(nb, H, D, bs, dtype=dtype)
    fields = dict(k_cache=k, v_cache=v, block_tables_tensor=torch.zeros(2, 3, dtype=torch.int32),
                  block_tables_ragged=ragged, slots=torch.arange(20), block_size=bs, num_kv_heads=H, head_dim=D,
                  kv_cache_dtype="auto", layout=layout)
    fields.update(kw)
    return tgi_adapter.TgiCacheView(**fields)


def k_elem(dtype):
    return torch.empty(0, dtype=dtype).element_size()


@pytest.mark.parametrize("layout,code", [("flashinfer", abi.LAYOUT_NHD), ("flashdecoding", abi.LAYOUT_NHD),
                                         ("ipex", abi.LAYOUT_HND), ("paged", abi.LAYOUT_HND_PACKED)])
def test_tgi_descriptors_validate(built_lib, layout, code):
    d = tgi_adapter.build_kvx_descriptors(_tgi(layout))
    c = d["cache"]
    assert built_lib.kvx_validate_cache_desc(C.byref(c)) == abi.STATUS_OK
    assert c.k.layout == code and (c.num_blocks, c.block_size, c.num_kv_heads, c.head_dim) == (8, 16, 4, 64)
    if layout == "paged":
        assert c.k.shape[4] == 8 and c.v.ndim == 5 and c.v.shape[4] == 1
    t, s = d["block_table"], d["slot_mapping"]
    assert (t.format, t.index_dtype, t.seq_count, t.max_blocks_per_seq, t.indices_count) == \
        (abi.TABLE_PACKED, abi.DTYPE_S32, 2, 3, 6)
    assert (s.dtype, s.token_count, s.invalid_slot) == (abi.DTYPE_S64, 20, -1)
    # the validate-only write entry point accepts the cache + slot mapping with a matching batch
    key = torch.zeros(20, 4, 64, dtype=torch.float16)
    w = abi.write_desc(20, 4, 64, abi.DTYPE_F16, key.data_ptr(), key.data_ptr(), s.dtype, s.slots, abi.MEMORY_HOST)
    assert built_lib.kvx_write_kv(C.byref(c), C.byref(w), None) == abi.STATUS_OK


def test_tgi_ragged_table_and_refusals():
    ids = torch.zeros(37, dtype=torch.int32)
    d = tgi_adapter.build_kvx_descriptors(_tgi(ragged=ids), ragged=True)
    t = d["block_table"]
    assert (t.format, t.indices_count, t.seq_count, t.beam_width) == (abi.TABLE_RAGGED, 37, 2, 1)
    assert not t.indptr                                   # filled in by adapters.gather from seq_lens
    with pytest.raises(ValueError):
        tgi_adapter.build_kvx_descriptors(_tgi(), ragged=True)          # no ragged table in the view
    with pytest.raises(ValueError):
        tgi_adapter.build_kvx_descriptors(_tgi(layout="triton"))
    with pytest.raises(ValueError):
        tgi_adapter.build_kvx_descriptors(_tgi(block_size=32))          # shape disagrees with the layout
    with pytest.raises(TypeError):
        tgi_adapter.build_kvx_descriptors(_tgi(kv_cache_dtype="fp8"))   # 2-byte tensor as an fp8 cache
    fp8 = _tgi(dtype=torch.uint8, kv_cache_dtype="fp8_e4m3fn")
    assert tgi_adapter.build_kvx_descriptors(fp8)["cache"].k.dtype == abi.DTYPE_F8_E4M3


def _trt(**kw):
    H, bs, D = 4, 16, 64
    page = H * bs * D * 2
    fields = dict(kv_block_offsets=torch.zeros(3, 1, 2, 5, dtype=torch.int32),
                  pool_primary=torch.zeros(12 * page // 2, dtype=torch.float16),
                  pool_secondary=torch.zeros(7 * page // 2, dtype=torch.float16), bytes_per_block=page,
                  tokens_per_block=bs, num_kv_heads=H, head_dim=D, kv_cache_dtype="fp16")
    fields.update(kw)
    return trt_llm_adapter.TrtLlmCacheView(**fields)


def test_trt_llm_descriptors_validate(built_lib):
    d = trt_llm_adapter.build_kvx_descriptors(_trt())
    c, t = d["cache"], d["block_table"]
    assert built_lib.kvx_validate_cache_desc(C.byref(c)) == abi.STATUS_OK
    assert c.k.layout == abi.LAYOUT_HND and c.num_blocks == 7          # the smaller pool bounds the offsets
    assert c.pool.bytes_per_block == 4 * 16 * 64 * 2 and c.pool.primary and c.pool.secondary
    assert (t.format, t.index_dtype, t.flags, t.seq_count, t.beam_width, t.max_blocks_per_seq, t.indices_count) == \
        (abi.TABLE_KV_OFFSETS, abi.DTYPE_S32, abi.TABLE_FLAG_KVCACHEINDEX, 3, 1, 5, 30)
    # the validate-only gather entry point reaches its last check (the format), as in the reference
    out = torch.zeros(3, 8, 4, 64, dtype=torch.float16)
    lens = torch.zeros(3, dtype=torch.int32)
    g = abi.gather_desc(3, 8, 4, 64, abi.DTYPE_F16, out.data_ptr(), out.data_ptr(), abi.DTYPE_S32, 0, 5,
                        lens.data_ptr(), abi.MEMORY_HOST)
    g.block_table = t
    assert built_lib.kvx_gather_kv(C.byref(c), C.byref(g), None) == abi.STATUS_UNSUPPORTED
    d = trt_llm_adapter.build_kvx_descriptors(_trt(pool_secondary=None, num_blocks=12))
    assert d["cache"].num_blocks == 12 and not d["cache"].pool.secondary


def test_trt_llm_refusals():
    with pytest.raises(ValueError):
        trt_llm_adapter.build_kvx_descriptors(_trt(tokens_per_block=24))
    with pytest.raises(ValueError):
        trt_llm_adapter.build_kvx_descriptors(_trt(bytes_per_block=100))
    with pytest.raises(ValueError):
        trt_llm_adapter.build_kvx_descriptors(_trt(kv_block_offsets=torch.zeros(3, 1, 2, 5, dtype=torch.int64)))
    with pytest.raises(ValueError):
        trt_llm_adapter.build_kvx_descriptors(_trt(kv_cache_dtype="int8"))
    with pytest.raises(ValueError):
        trt_llm_adapter.build_kvx_descriptors(_trt(pool_primary=0x10000, pool_secondary=None))  # no bound given
