"""Decode attention over the paged cache (kvx_launch_paged_attention_decode) against the CPU
checker's double-precision statement, which tests/test_oracle.py pins to an independent numpy
formulation.  Floating point, so a tolerance applies -- the only one in this suite:

    |out - expected| <= atol + rtol * |expected|, with (atol, rtol) = (1.5e-2, 1.6e-2) for
    bfloat16, (2e-3, 2e-3) for float16 and (2e-5, 2e-5) for float32 data.

The bf16 / f16 figures are two units in the last place of the type plus the rounding of the
softmax weights to that type inside the tensor-core path; scores and sums are f32."""
import ctypes as C
import dataclasses

import numpy as np
import pytest

import kvx_b200
from kvx_b200 import abi

import cases
from harness import NP_OF, bits_to_f32, device_buffers, descriptors, f32_to_bits, host_buffers, oracle_write

pytestmark = pytest.mark.gpu
TOL = {abi.DTYPE_BF16: (1.5e-2, 1.6e-2), abi.DTYPE_F16: (2e-3, 2e-3), abi.DTYPE_F32: (2e-5, 2e-5)}


@pytest.fixture(autouse=True, params=["carried_first_loads", "no_carry"])
def item_hand_over(request):
    """Every test runs with the fast kernel's two ways of going from one work item to the next:
    the next item's first loads issued ahead of the epilogue (the default), or after it."""
    saved = kvx_b200.get_option("attn_carry")
    kvx_b200.set_option("attn_carry", 1 if request.param == "carried_first_loads" else 0)
    yield request.param
    kvx_b200.set_option("attn_carry", saved)


def _query(case, group, seed):
    rng = np.random.default_rng(seed)
    S, Hq, D = case.table.shape[0], case.geom.num_kv_heads * group, case.geom.head_dim
    return f32_to_bits(rng.standard_normal((S, Hq, D)).astype(np.float32), case.io_dtype)


def _attn_desc(case, q_addr, out_addr, bufs, Hq, scale, max_seq_len, memory):
    a = abi.attention_desc(case.table.shape[0], Hq, case.geom.head_dim, case.io_dtype, q_addr, out_addr, scale,
                           max_seq_len, abi.DTYPE_S32 if case.table.dtype == np.int32 else abi.DTYPE_S64,
                           bufs["table"].ctypes.data if memory == abi.MEMORY_HOST else bufs["table"].data_ptr(),
                           case.table.shape[1],
                           bufs["lens"].ctypes.data if memory == abi.MEMORY_HOST else bufs["lens"].data_ptr(), memory)
    return a


def run_both(case, k, v, group, seed=0, max_seq_len=None, scale=None):
    """(expected f32, got f32) for one case whose pages hold k / v."""
    import torch
    from oracle.kvx_oracle import oracle
    D = case.geom.head_dim
    Hq = case.geom.num_kv_heads * group
    scale = float(1.0 / np.sqrt(D)) if scale is None else scale
    max_seq_len = case.max_seq_len if max_seq_len is None else max_seq_len
    q = _query(case, group, seed)
    src = dataclasses.replace(case, cache_k=k, cache_v=v)
    # checker
    hb = host_buffers(src)
    cache, _, _, ks, vs = descriptors(src, hb, abi.MEMORY_HOST)
    exp = np.zeros_like(q)
    a = _attn_desc(case, q.ctypes.data, exp.ctypes.data, hb, Hq, scale, max_seq_len, abi.MEMORY_HOST)
    assert oracle().kvx_oracle_paged_attention_decode(C.byref(cache), C.byref(a), C.byref(ks), C.byref(vs)) == 0
    # device
    db = device_buffers(src)
    cache, _, _, ks, vs = descriptors(src, db, abi.MEMORY_DEVICE)
    dq = torch.from_numpy(q.view(np.uint8).reshape(-1).copy()).cuda()
    dout = torch.full((q.nbytes,), 0x5A, dtype=torch.uint8, device="cuda")
    a = _attn_desc(case, dq.data_ptr(), dout.data_ptr(), db, Hq, scale, max_seq_len, abi.MEMORY_DEVICE)
    L = kvx_b200.lib()
    need = L.kvx_paged_attention_workspace_bytes(case.table.shape[0], Hq, case.geom.num_kv_heads, D, max_seq_len)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    st = L.kvx_launch_paged_attention_decode(C.byref(cache), C.byref(a), C.byref(ks), C.byref(vs), ws.data_ptr(),
                                             need, None)
    torch.cuda.synchronize()
    assert st == abi.STATUS_OK, st
    got = dout.cpu().numpy().view(NP_OF[case.io_dtype]).reshape(q.shape)
    return bits_to_f32(exp, case.io_dtype), bits_to_f32(got, case.io_dtype)


def check(case, k, v, group, **kw):
    exp, got = run_both(case, k, v, group, **kw)
    atol, rtol = TOL[case.io_dtype]
    err = np.abs(got - exp)
    bad = err > atol + rtol * np.abs(exp)
    assert not bad.any(), (case.note, float(err.max()), np.argwhere(bad)[:5].tolist())


@pytest.mark.parametrize("dtype", [abi.DTYPE_BF16, abi.DTYPE_F16])
@pytest.mark.parametrize("layout", [abi.LAYOUT_NHD, abi.LAYOUT_HND])
def test_fast_tier_shapes(layout, dtype):
    """Tensor-core tier: head_dim 64 / 128 / 256, pages of 16 / 32 / 64 tokens, 1..16 query heads per KV
    head, empty / one-token / page-edge / long contexts, invalid page ids, both index widths."""
    for i, kw in enumerate([
        dict(heads=2, dim=128, block_size=16, num_blocks=80, lens=[100, 17, 256, 1, 0, 333, 16, 15], group=4),
        dict(heads=4, dim=64, block_size=32, num_blocks=40, lens=[31, 33, 160, 64], group=1, index_dtype=np.int64),
        dict(heads=1, dim=128, block_size=16, num_blocks=64, lens=[500, 3], group=8, bad_blocks=3),
        dict(heads=2, dim=64, block_size=16, num_blocks=32, lens=[47, 200], group=16),
        dict(heads=1, dim=128, block_size=64, num_blocks=12, lens=[130, 400], group=12),
        dict(heads=2, dim=256, block_size=16, num_blocks=60, lens=[130, 400, 1], group=4),
        dict(heads=1, dim=256, block_size=32, num_blocks=20, lens=[99, 300], group=9),
    ]):
        group = kw.pop("group")
        case = cases.make_case(2000 + i, layout=layout, dtype=dtype, real_values=True, **kw)
        case.note = f"fast {i}"
        _, k, v = oracle_write(case)
        check(case, k, v, group, seed=i)


def test_split_contexts_and_merge():
    """Contexts longer than one chunk: partial results per chunk merged by the second kernel;
    max_seq_len below the longest context truncates it."""
    case = cases.make_case(2100, dtype=abi.DTYPE_BF16, real_values=True, heads=2, dim=128, block_size=16,
                           num_blocks=700, lens=[5000, 700, 0, 2049, 256, 1])
    _, k, v = oracle_write(case)
    assert kvx_b200.lib().kvx_paged_attention_workspace_bytes(6, 8, 2, 128, 5000) > 0
    check(case, k, v, 4)
    check(case, k, v, 4, max_seq_len=3000)
    check(case, k, v, 4, max_seq_len=100)


def test_many_items_per_cta_from_the_compacted_list():
    """Thousands of work items for a few hundred persistent CTAs: every CTA takes many items in a
    row (claimed two ahead, the next item's first rows issued before an item's epilogue), full
    chunks first, then last chunks of every length class; sequences without tokens in between."""
    rng = np.random.default_rng(79)
    lens = [int(x) for x in rng.choice([0, 1, 15, 16, 17, 40, 63, 64, 65, 130, 255, 256, 257, 300, 511, 520, 700],
                                       size=500)]
    lens[7], lens[250], lens[499] = 2049, 4100, 5000  # contexts of several chunks: partial results and the merge
    for i, (dtype, group, dim) in enumerate(((abi.DTYPE_BF16, 4, 128), (abi.DTYPE_F16, 12, 64))):
        case = cases.make_case(2170 + i, dtype=dtype, real_values=True, heads=8, dim=dim, block_size=16,
                               num_blocks=sum(-(-n // 16) for n in lens) + 8, lens=lens)
        case.note = f"many items, group {group}"
        _, k, v = oracle_write(case)
        check(case, k, v, group, seed=i)


def test_more_sequences_than_the_shared_memory_prefix_holds():
    """Beyond 8 192 sequences the tensor-core kernels enumerate the padded (sequence, chunk)
    rectangle instead of a compacted list; both forms (heads in columns / in rows)."""
    rng = np.random.default_rng(78)
    lens = [int(x) for x in rng.integers(0, 40, size=8300)]
    for i, group in enumerate((2, 12)):
        case = cases.make_case(2150 + i, dtype=abi.DTYPE_F16, real_values=True, heads=1, dim=64, block_size=16,
                               num_blocks=25000, lens=lens)
        case.note = f"many sequences, group {group}"
        _, k, v = oracle_write(case)
        check(case, k, v, group)


@pytest.mark.parametrize("dtype", [abi.DTYPE_BF16, abi.DTYPE_F16])
@pytest.mark.parametrize("layout", [abi.LAYOUT_NHD, abi.LAYOUT_HND])
def test_fp8_cache_fast_tier(layout, dtype):
    """e4m3 pages under the tensor-core tier: bytes are staged as they are and converted to f16
    between ldmatrix and the MMA; K scale on the scores, V scale on the output; per-head and
    per-tensor scales, one and two column tiles of query heads, split contexts."""
    for i, (kw, group, gran) in enumerate([
        (dict(heads=2, dim=128, block_size=16, num_blocks=80, lens=[100, 17, 256, 1, 0, 333, 16, 15]), 4, abi.SCALE_PER_HEAD),
        (dict(heads=4, dim=64, block_size=32, num_blocks=40, lens=[31, 33, 160, 64], index_dtype=np.int64), 1,
         abi.SCALE_PER_TENSOR),
        (dict(heads=1, dim=128, block_size=64, num_blocks=12, lens=[130, 400], bad_blocks=1), 12, abi.SCALE_PER_HEAD),
        (dict(heads=2, dim=128, block_size=16, num_blocks=400, lens=[3000, 700, 2049]), 8, abi.SCALE_PER_HEAD),
        (dict(heads=2, dim=256, block_size=64, num_blocks=24, lens=[300, 5, 640]), 4, abi.SCALE_PER_HEAD),
        (dict(heads=1, dim=256, block_size=16, num_blocks=40, lens=[200, 77]), 16, abi.SCALE_PER_TENSOR),
    ]):
        case = cases.make_case(2500 + i, layout=layout, dtype=dtype, cache_dtype=abi.DTYPE_F8_E4M3, scale_gran=gran,
                               real_values=True, **kw)
        case.note = f"fp8 fast {i}"
        _, k, v = oracle_write(case)
        check(case, k, v, group, seed=i)


def test_generic_tier_shapes():
    """Everything the tensor-core tier does not take: f32 data, odd head_dim, small pages,
    HND_PACKED pages, an fp8-e4m3 cache with per-head scales."""
    for i, (dtype, kw, group) in enumerate([
        (abi.DTYPE_F32, dict(heads=2, dim=64, block_size=16, num_blocks=40, lens=[100, 17, 0, 333]), 2),
        (abi.DTYPE_BF16, dict(heads=3, dim=40, block_size=6, num_blocks=50, lens=[7, 100, 13]), 2),
        (abi.DTYPE_F16, dict(heads=2, dim=64, block_size=8, num_blocks=200, lens=[50, 70, 1200]), 4),
        (abi.DTYPE_BF16, dict(heads=2, dim=64, block_size=16, num_blocks=24, lens=[50, 70], layout=abi.LAYOUT_HND_PACKED,
                              pack=8), 1),
        (abi.DTYPE_BF16, dict(heads=4, dim=80, block_size=16, num_blocks=24, lens=[100, 40, 7],
                              cache_dtype=abi.DTYPE_F8_E4M3, scale_gran=abi.SCALE_PER_HEAD), 2),
    ]):
        case = cases.make_case(2200 + i, dtype=dtype, real_values=True, **kw)
        case.note = f"generic {i}"
        _, k, v = oracle_write(case)
        check(case, k, v, group, seed=i)


def test_statuses():
    import torch
    case = cases.make_case(2400, dtype=abi.DTYPE_BF16, real_values=True, heads=2, dim=128, block_size=16,
                           num_blocks=400, lens=[3000, 5])
    db = device_buffers(case)
    cache, _, _, ks, vs = descriptors(case, db, abi.MEMORY_DEVICE)
    q = torch.zeros((2, 8, 128), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros_like(q)
    L = kvx_b200.lib()

    def call(a, ws=None, nbytes=0):
        return L.kvx_launch_paged_attention_decode(C.byref(cache), C.byref(a), C.byref(ks), C.byref(vs), ws, nbytes, None)

    def desc(**kw):
        a = _attn_desc(case, q.data_ptr(), out.data_ptr(), db, 8, 0.1, 3000, abi.MEMORY_DEVICE)
        for key, val in kw.items():
            setattr(a, key, val)
        return a

    need = L.kvx_paged_attention_workspace_bytes(2, 8, 2, 128, 3000)
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    assert call(desc(), ws.data_ptr(), need) == abi.STATUS_OK
    assert call(desc(), None, 0) == abi.STATUS_INVALID_ARGUMENT             # scratch missing
    assert call(desc(), ws.data_ptr(), need - 1) == abi.STATUS_INVALID_ARGUMENT
    assert call(desc(num_q_heads=7), ws.data_ptr(), need) == abi.STATUS_INVALID_ARGUMENT  # not a multiple of 2
    assert call(desc(max_seq_len=0), ws.data_ptr(), need) == abi.STATUS_INVALID_ARGUMENT
    a = desc(); a.block_table.format = abi.TABLE_RAGGED
    assert call(a, ws.data_ptr(), need) == abi.STATUS_UNSUPPORTED
    a = desc(); a.out.dtype = abi.DTYPE_F16
    assert call(a, ws.data_ptr(), need) == abi.STATUS_UNSUPPORTED
    a = desc(); a.query.stride[0] = 8 * 128 + 8
    assert call(a, ws.data_ptr(), need) == abi.STATUS_UNSUPPORTED
    a = desc(); a.size -= 4
    assert call(a, ws.data_ptr(), need) == abi.STATUS_INVALID_ARGUMENT
    torch.cuda.synchronize()


def test_python_front_end_matches_dense_attention():
    """ops.paged_attention_decode against gather + a dense f32 softmax in torch."""
    import torch
    from kvx_b200 import ops
    torch.manual_seed(5)
    S, Hkv, G, D, bs, nb = 6, 2, 4, 128, 16, 200
    kc = torch.randn((nb, bs, Hkv, D), device="cuda").to(torch.bfloat16)
    vc = torch.randn((nb, bs, Hkv, D), device="cuda").to(torch.bfloat16)
    lens = torch.tensor([1, 16, 100, 257, 0, 411], dtype=torch.int32, device="cuda")
    perm = torch.randperm(nb, device="cuda").to(torch.int32)
    mb = 32
    table = perm[: S * mb].reshape(S, mb).contiguous()
    q = torch.randn((S, Hkv * G, D), device="cuda").to(torch.bfloat16)
    scale = D ** -0.5
    out = ops.paged_attention_decode(q, kc, vc, table, lens, scale)
    Lmax = int(lens.max())
    gk = torch.zeros((S, Lmax, Hkv, D), dtype=torch.bfloat16, device="cuda"); gv = torch.zeros_like(gk)
    ops.gather_kv(kc, vc, table, lens, gk, gv)
    torch.cuda.synchronize()
    for s in range(S):
        n = int(lens[s])
        if n == 0:
            assert not out[s].float().abs().any()
            continue
        kk = gk[s, :n].float().repeat_interleave(G, dim=1)      # [n, Hq, D]
        vv = gv[s, :n].float().repeat_interleave(G, dim=1)
        sc = torch.einsum("hd,nhd->hn", q[s].float(), kk) * scale
        ref = torch.einsum("hn,nhd->hd", torch.softmax(sc, dim=-1), vv)
        assert torch.allclose(out[s].float(), ref, atol=1.5e-2, rtol=1.6e-2), s
