"""Engine adapters end to end on the device: a TGI-style cache written through `slots` and read
back through the padded and the ragged block tables, TGI's "paged" layout, and a TensorRT-LLM
style block pool read through a KV_OFFSETS table -- all checked against the CPU checker."""
import dataclasses

import numpy as np
import pytest

from kvx_b200 import abi

import cases
from harness import oracle_gather, oracle_write

pytestmark = pytest.mark.gpu


def _dev(torch, arr, dtype):
    return torch.from_numpy(np.ascontiguousarray(arr).view(np.uint8).reshape(-1)).cuda().view(dtype)


def _bits(t, like):
    import torch
    return t.contiguous().view(torch.uint8).cpu().numpy().view(like.dtype).reshape(like.shape)


@pytest.mark.parametrize("layout,name", [(abi.LAYOUT_NHD, "flashinfer"), (abi.LAYOUT_HND, "ipex")])
def test_tgi_view_write_then_gather_packed_and_ragged(layout, name):
    import torch

    from kvx_b200 import adapters
    from kvx_b200.adapters import tgi_adapter

    case = cases.make_case(61, layout=layout, dtype=abi.DTYPE_BF16, num_blocks=48, block_size=16, heads=4, dim=64,
                           lens=[70, 5, 0, 130, 33], pad_frac=0.1, slot_dtype=np.int64, index_dtype=np.int32)
    _, ek, ev = oracle_write(case)
    _, eok, eov = oracle_gather(case, ek, ev)
    rag = cases.to_ragged(case)
    bf = torch.bfloat16
    k_cache = _dev(torch, case.cache_k, bf).view(case.geom.shape)
    v_cache = _dev(torch, case.cache_v, bf).view(case.geom.shape)
    view = tgi_adapter.TgiCacheView(
        k_cache=k_cache, v_cache=v_cache, block_tables_tensor=torch.from_numpy(case.table).cuda(),
        block_tables_ragged=torch.from_numpy(rag.ragged).cuda(), slots=torch.from_numpy(case.slots).cuda(),
        block_size=16, num_kv_heads=4, head_dim=64, kv_cache_dtype="auto", layout=name)
    d = tgi_adapter.build_kvx_descriptors(view)
    adapters.write(d, _dev(torch, case.key, bf).view(case.key.shape), _dev(torch, case.value, bf).view(case.value.shape))
    torch.cuda.synchronize()
    assert np.array_equal(_bits(k_cache, ek), ek) and np.array_equal(_bits(v_cache, ev), ev)
    lens = torch.from_numpy(case.lens).cuda()
    for ragged in (False, True):
        d = tgi_adapter.build_kvx_descriptors(view, ragged=ragged)
        ok = _dev(torch, case.out_k, bf).view(case.out_k.shape)
        ov = _dev(torch, case.out_v, bf).view(case.out_v.shape)
        adapters.gather(d, lens, ok, ov)
        torch.cuda.synchronize()
        assert np.array_equal(_bits(ok, eok), eok) and np.array_equal(_bits(ov, eov), eov), ragged


def test_tgi_paged_layout_round_trip():
    """K [blocks, heads, dim / x, BLOCK_SIZE, x] with x = 16 / element size, V [blocks, heads,
    dim, BLOCK_SIZE]: write, compare with a direct numpy statement of both layouts, gather back."""
    import torch

    from kvx_b200 import adapters
    from kvx_b200.adapters import tgi_adapter

    nb, bs, H, D, x = 12, 16, 2, 64, 8
    case = cases.make_case(62, dtype=abi.DTYPE_F16, num_blocks=nb, block_size=bs, heads=H, dim=D, lens=[40, 90, 17],
                           slot_dtype=np.int64, index_dtype=np.int32)
    k_cache = torch.zeros((nb, H, D // x, bs, x), dtype=torch.float16, device="cuda")
    v_cache = torch.zeros((nb, H, D, bs), dtype=torch.float16, device="cuda")
    view = tgi_adapter.TgiCacheView(k_cache, v_cache, torch.from_numpy(case.table).cuda(), None,
                                    torch.from_numpy(case.slots).cuda(), bs, H, D, "auto", "paged")
    d = tgi_adapter.build_kvx_descriptors(view)
    f16 = torch.float16
    adapters.write(d, _dev(torch, case.key, f16).view(case.key.shape), _dev(torch, case.value, f16).view(case.value.shape))
    torch.cuda.synchronize()
    ek = np.zeros((nb, H, D // x, bs, x), np.uint16)
    ev = np.zeros((nb, H, D, bs), np.uint16)
    for t, slot in enumerate(case.slots.tolist()):
        b, o = divmod(slot, bs)
        ek[b, :, :, o, :] = case.key[t].reshape(H, D // x, x)
        ev[b, :, :, o] = case.value[t]
    assert np.array_equal(_bits(k_cache, ek), ek) and np.array_equal(_bits(v_cache, ev), ev)
    ok = torch.zeros(case.out_k.shape, dtype=f16, device="cuda")
    ov = torch.zeros(case.out_v.shape, dtype=f16, device="cuda")
    adapters.gather(d, torch.from_numpy(case.lens).cuda(), ok, ov)
    torch.cuda.synchronize()
    gk, gv = _bits(ok, case.out_k), _bits(ov, case.out_v)
    first = 0
    for s, n in enumerate(case.lens.tolist()):
        assert np.array_equal(gk[s, :n], case.key[first:first + n]) and np.array_equal(gv[s, :n], case.value[first:first + n])
        assert not gk[s, n:].any() and not gv[s, n:].any()
        first += n


@pytest.mark.parametrize("fp8", [False, True])
def test_trt_llm_view_gather(fp8):
    import torch

    from kvx_b200 import adapters
    from kvx_b200.adapters import trt_llm_adapter

    kw = dict(cache_dtype=abi.DTYPE_F8_E4M3, scale_gran=abi.SCALE_PER_HEAD, real_values=True) if fp8 else {}
    packed = cases.make_case(63, layout=abi.LAYOUT_HND, dtype=abi.DTYPE_BF16, num_blocks=40, block_size=32, heads=4,
                             dim=128, lens=[100, 1, 333, 64], index_dtype=np.int32, **kw)
    _, k, v = oracle_write(packed)
    _, eok, eov = oracle_gather(packed, k, v)
    off = cases.to_kv_offsets(packed, k, v, seed=3)
    pool_dtype = torch.uint8 if fp8 else torch.bfloat16
    view = trt_llm_adapter.TrtLlmCacheView(
        kv_block_offsets=torch.from_numpy(off.kv_offsets).cuda(), pool_primary=_dev(torch, off.pool_primary, pool_dtype),
        pool_secondary=_dev(torch, off.pool_secondary, pool_dtype), bytes_per_block=off.pool_block_bytes,
        tokens_per_block=32, num_kv_heads=4, head_dim=128, kv_cache_dtype="fp8" if fp8 else "bf16")
    d = trt_llm_adapter.build_kvx_descriptors(view)
    assert d["cache"].num_blocks == 80
    ok = _dev(torch, packed.out_k, torch.bfloat16).view(packed.out_k.shape)
    ov = _dev(torch, packed.out_v, torch.bfloat16).view(packed.out_v.shape)
    scales = (torch.from_numpy(packed.k_scale).cuda(), torch.from_numpy(packed.v_scale).cuda()) if fp8 else (None, None)
    adapters.gather(d, torch.from_numpy(packed.lens).cuda(), ok, ov, *scales)
    torch.cuda.synchronize()
    assert np.array_equal(_bits(ok, eok), eok) and np.array_equal(_bits(ov, eov), eov)
