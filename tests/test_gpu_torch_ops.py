"""The torch front end (kvx_b200.ops) on real tensors: the dispatcher-registered operators
(torch.ops.kvx_b200.*) and the ctypes route must both equal the CPU checker byte for byte,
on the layouts and dtypes the vLLM patch's operator accepts (reference:
patches/vllm/kvx.patch:176-275 for the operator, :328-398 for its test)."""
import numpy as np
import pytest

from kvx_b200 import abi

import cases
from harness import NP_OF, oracle_gather, oracle_write

pytestmark = pytest.mark.gpu

TORCH_OF = {abi.DTYPE_F16: "float16", abi.DTYPE_BF16: "bfloat16", abi.DTYPE_F32: "float32"}


def _to_dev(torch, arr, code):
    """numpy bit patterns -> CUDA tensor of the float type they encode."""
    t = torch.from_numpy(np.ascontiguousarray(arr).view(np.uint8).reshape(-1)).cuda()
    if code == abi.DTYPE_F8_E4M3:
        return t
    return t.view(getattr(torch, TORCH_OF[code]))


def _bits(t, code):
    return t.contiguous().view(__import__("torch").uint8).cpu().numpy().view(NP_OF[code]).reshape(-1)


def _run(case, route):
    """Write then gather through kvx_b200.ops; ``route`` is "native" (dispatcher operators) or
    "ctypes" (descriptors filled in Python)."""
    import torch

    from kvx_b200 import ops

    native = ops.native_ops()
    assert native is not None, "libkvx_b200_torch.so is not built"
    g = case.geom
    fp8 = case.cache_dtype == abi.DTYPE_F8_E4M3
    ck = _to_dev(torch, case.cache_k, case.cache_dtype).view(g.shape)
    cv = _to_dev(torch, case.cache_v, case.cache_dtype).view(g.shape)
    key = _to_dev(torch, case.key, case.io_dtype).view(case.key.shape)
    value = _to_dev(torch, case.value, case.io_dtype).view(case.value.shape)
    slots = torch.from_numpy(case.slots).cuda()
    table = torch.from_numpy(case.table).cuda()
    lens = torch.from_numpy(case.lens).cuda()
    ok = _to_dev(torch, case.out_k, case.io_dtype).view(case.out_k.shape)
    ov = _to_dev(torch, case.out_v, case.io_dtype).view(case.out_v.shape)
    kind = "fp8" if fp8 else "auto"
    ks = torch.from_numpy(case.k_scale).cuda() if fp8 else None
    vs = torch.from_numpy(case.v_scale).cuda() if fp8 else None
    if route == "native":
        ops.reshape_and_cache_flash_kvx(key, value, ck, cv, slots, kind, ks, vs)
        ops.gather_kv(ck, cv, table, lens, ok, ov, kind, ks, vs)
    else:
        saved, ops._NATIVE = ops._NATIVE, False
        try:
            ops.reshape_and_cache_flash_kvx(key, value, ck, cv, slots, kind, ks, vs)
            ops.gather_kv(ck, cv, table, lens, ok, ov, kind, ks, vs)
        finally:
            ops._NATIVE = saved
    torch.cuda.synchronize()
    return _bits(ck, case.cache_dtype), _bits(cv, case.cache_dtype), _bits(ok, case.io_dtype), _bits(ov, case.io_dtype)


@pytest.mark.parametrize("route", ["native", "ctypes"])
@pytest.mark.parametrize("layout", [abi.LAYOUT_NHD, abi.LAYOUT_HND])
@pytest.mark.parametrize("dtype", [abi.DTYPE_F16, abi.DTYPE_BF16, abi.DTYPE_F32])
def test_ops_equal_checker(route, layout, dtype):
    case = cases.make_case(31 + dtype, layout=layout, dtype=dtype, num_blocks=40, block_size=16, heads=4, dim=64,
                           lens=[70, 0, 16, 129, 5], pad_frac=0.1, slot_dtype=np.int64, index_dtype=np.int32)
    st, ek, ev = oracle_write(case)
    assert st == abi.STATUS_OK
    st, eok, eov = oracle_gather(case, ek, ev)
    assert st == abi.STATUS_OK
    k, v, ok, ov = _run(case, route)
    assert np.array_equal(k, ek.reshape(-1)) and np.array_equal(v, ev.reshape(-1))
    assert np.array_equal(ok, eok.reshape(-1)) and np.array_equal(ov, eov.reshape(-1))


@pytest.mark.parametrize("route", ["native", "ctypes"])
@pytest.mark.parametrize("gran", [abi.SCALE_PER_TENSOR, abi.SCALE_PER_HEAD])
def test_ops_fp8_equal_checker(route, gran):
    case = cases.make_case(77, dtype=abi.DTYPE_BF16, cache_dtype=abi.DTYPE_F8_E4M3, scale_gran=gran, num_blocks=24,
                           block_size=16, heads=8, dim=128, lens=[100, 33, 64], real_values=True, pad_frac=0.05,
                           index_dtype=np.int64)
    st, ek, ev = oracle_write(case)
    assert st == abi.STATUS_OK
    st, eok, eov = oracle_gather(case, ek, ev)
    k, v, ok, ov = _run(case, route)
    assert np.array_equal(k, ek.reshape(-1)) and np.array_equal(v, ev.reshape(-1))
    assert np.array_equal(ok, eok.reshape(-1)) and np.array_equal(ov, eov.reshape(-1))


def test_ops_slice_of_a_larger_batch_and_int32_slots():
    """The batch is sized by slot_mapping, so key/value may hold more rows than are written
    (reference: kvx.patch:208).  Views of a fused projection output, whose token rows are not
    dense, are written as they are (the reference's operator refuses them, kvx.patch:213-218;
    vLLM's own operator takes them); a view with strided heads is still UNSUPPORTED."""
    import torch

    from kvx_b200 import ops

    case = cases.make_case(5, dtype=abi.DTYPE_F16, num_blocks=16, block_size=16, heads=4, dim=64, lens=[48, 20],
                           slot_dtype=np.int32)
    T = case.key.shape[0]
    st, ek, ev = oracle_write(case)
    slots = torch.from_numpy(case.slots).cuda()
    kv = torch.zeros((2, T + 3, 4, 64), dtype=torch.float16, device="cuda")
    kv[0, :T] = _to_dev(torch, case.key, case.io_dtype).view(case.key.shape)
    kv[1, :T] = _to_dev(torch, case.value, case.io_dtype).view(case.value.shape)
    qkv = torch.randn((T, 3, 4, 64), device="cuda").to(torch.float16)       # [token, q|k|v, head, dim]
    qkv[:, 1] = kv[0, :T]
    qkv[:, 2] = kv[1, :T]
    for key, value in ((kv[0], kv[1]), (qkv[:, 1], qkv[:, 2])):
        for native in (True, False):
            ck = _to_dev(torch, case.cache_k, case.cache_dtype).view(case.geom.shape)
            cv = _to_dev(torch, case.cache_v, case.cache_dtype).view(case.geom.shape)
            saved = ops._NATIVE
            if not native:
                ops._NATIVE = False
            try:
                ops.reshape_and_cache_flash_kvx(key, value, ck, cv, slots)
            finally:
                ops._NATIVE = saved
            torch.cuda.synchronize()
            assert np.array_equal(_bits(ck, case.cache_dtype), ek.reshape(-1))
            assert np.array_equal(_bits(cv, case.cache_dtype), ev.reshape(-1))
    hqkv = torch.zeros((T, 4, 3, 64), dtype=torch.float16, device="cuda")   # heads not dense in the view
    with pytest.raises(ops.KvxError) as e:
        ops.reshape_and_cache_flash_kvx(hqkv[:, :, 1], hqkv[:, :, 2], ck.clone(), cv.clone(), slots)
    assert e.value.status == abi.STATUS_UNSUPPORTED


def test_ops_varlen_gather_matches_padded_gather():
    import torch

    from kvx_b200 import ops

    case = cases.make_case(15, dtype=abi.DTYPE_BF16, num_blocks=40, block_size=16, heads=8, dim=128,
                           lens=[70, 0, 16, 129, 5], index_dtype=np.int32)
    _, ek, ev = oracle_write(case)
    ck = _to_dev(torch, ek, case.cache_dtype).view(case.geom.shape)
    cv = _to_dev(torch, ev, case.cache_dtype).view(case.geom.shape)
    table, lens = torch.from_numpy(case.table).cuda(), torch.from_numpy(case.lens).cuda()
    pk = torch.zeros(case.out_k.shape, dtype=torch.bfloat16, device="cuda"); pv = pk.clone()
    ops.gather_kv(ck, cv, table, lens, pk, pv)
    indptr = torch.cat([torch.zeros(1, dtype=torch.int32, device="cuda"), torch.cumsum(lens, 0).to(torch.int32)])
    rows = int(indptr[-1])
    vk = torch.full((rows, 8, 128), 3.0, dtype=torch.bfloat16, device="cuda"); vv = vk.clone()
    ops.gather_kv_varlen(ck, cv, table, lens, indptr, vk, vv, case.max_seq_len)
    torch.cuda.synchronize()
    for s, n in enumerate(case.lens.tolist()):
        a = int(indptr[s])
        i16 = torch.int16  # compare bit patterns: the random payload contains NaNs
        assert torch.equal(vk[a:a + n].view(i16), pk[s, :n].view(i16))
        assert torch.equal(vv[a:a + n].view(i16), pv[s, :n].view(i16))


def test_ops_report_the_status():
    """A launcher status other than OK surfaces as KvxError carrying it, on both routes."""
    import torch

    from kvx_b200 import ops

    key = torch.zeros((4, 2, 8), dtype=torch.float16, device="cuda")
    cache = torch.zeros((2, 4, 2, 16), dtype=torch.float16, device="cuda")  # head_dim 16 != 8
    slots = torch.arange(4, device="cuda")
    with pytest.raises(ops.KvxError) as e:
        ops.reshape_and_cache_flash_kvx(key, key, cache, cache.clone(), slots)
    assert e.value.status == abi.STATUS_INVALID_ARGUMENT
    saved, ops._NATIVE = ops._NATIVE, False
    try:
        with pytest.raises(ops.KvxError) as e2:
            ops.reshape_and_cache_flash_kvx(key, key, cache, cache.clone(), slots)
    finally:
        ops._NATIVE = saved
    assert e2.value.status == e.value.status
