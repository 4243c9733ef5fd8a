"""Pins the CPU checker (no GPU needed): against an independent numpy statement of the
reference kernel test's expected-value loops, against the reference test's closed-form toy
cases, against ml_dtypes / torch for the e4m3 conversion, and against the byte dumps the
reference's own kernels produced on a B200 (tests/golden)."""
import ctypes as C
import glob
import os

import numpy as np
import pytest

from kvx_b200 import abi

import cases
from harness import (Case, bits_to_f32, descriptors, f32_to_bits, host_buffers, oracle_gather,
                     oracle_write)

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
LAYOUTS = [(abi.LAYOUT_NHD, 1), (abi.LAYOUT_HND, 1), (abi.LAYOUT_HND_PACKED, 4), (abi.LAYOUT_HND_PACKED, 8)]
DTYPES = [abi.DTYPE_F32, abi.DTYPE_F16, abi.DTYPE_BF16]


@pytest.mark.parametrize("layout,pack", LAYOUTS)
@pytest.mark.parametrize("dtype", DTYPES)
def test_write_and_gather_match_numpy_statement(layout, pack, dtype):
    for seed, kw in enumerate([
        dict(), dict(pad_frac=0.3, slot_dtype=np.int32), dict(oob_slots=3, bad_blocks=3, index_dtype=np.int64),
        dict(lens=[0, 9, 4, 1], num_blocks=16), dict(lens=[5, 12], max_seq_len=7, max_blocks=2),
    ]):
        case = cases.make_case(100 + seed, layout=layout, pack=pack, dtype=dtype, **kw)
        st, k, v = oracle_write(case)
        assert st == abi.STATUS_OK
        ek, ev = cases.expected_write_numpy(case)
        assert np.array_equal(k, ek) and np.array_equal(v, ev)
        st, ok_, ov_ = oracle_gather(case, k, v)
        assert st == abi.STATUS_OK
        gk, gv = cases.expected_gather_numpy(case, k, v)
        assert np.array_equal(ok_, gk) and np.array_equal(ov_, gv)


def _reference_toy(dtype, heads, dim, tokens_per_seq, layout):
    """The write cases of tests/kvx_kernel_test.cu:161-193 / :312-344: 2 sequences of 4
    tokens, block_size 4, identity pages, the LAST tokens_per_seq positions are written,
    K = 0.1 + 0.01 i, V = K + 0.5, S64 slots."""
    geom = abi.CacheGeometry(2, 4, heads, dim, layout)
    n = 2 * tokens_per_seq * heads * dim
    val = (np.float32(0.1) + np.float32(0.01) * np.arange(n, dtype=np.float32)).astype(np.float32)
    key = f32_to_bits(val, dtype).reshape(-1, heads, dim)
    value = f32_to_bits(val + np.float32(0.5), dtype).reshape(-1, heads, dim)
    slots = np.array([s * 4 + (4 - tokens_per_seq) + t for s in range(2) for t in range(tokens_per_seq)], np.int64)
    zeros = np.zeros(geom.elems, dtype=key.dtype)
    return Case(geom=geom, cache_dtype=dtype, io_dtype=dtype, key=key, value=value, slots=slots,
                cache_k=zeros.copy(), cache_v=zeros.copy())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,tps,layout", [
    (2, 4, 1, abi.LAYOUT_NHD), (1, 7, 1, abi.LAYOUT_NHD), (2, 4, 2, abi.LAYOUT_NHD),
    (2, 4, 1, abi.LAYOUT_HND), (1, 7, 2, abi.LAYOUT_HND)])
def test_reference_kernel_test_write_cases(dtype, heads, dim, tps, layout):
    """tests/kvx_kernel_test.cu:456-466 with its own expected-offset arithmetic (:264-301,
    :415-446), compared exactly instead of within the reference's tolerance."""
    case = _reference_toy(dtype, heads, dim, tps, layout)
    st, k, v = oracle_write(case)
    assert st == abi.STATUS_OK
    for t in range(case.T):
        b, o = divmod(int(case.slots[t]), 4)
        for h in range(heads):
            for d in range(dim):
                off = (b * 4 * heads * dim + o * heads * dim + h * dim + d if layout == abi.LAYOUT_NHD
                       else b * heads * 4 * dim + h * 4 * dim + o * dim + d)
                assert k[off] == case.key[t, h, d] and v[off] == case.value[t, h, d]
    assert np.count_nonzero(k) == case.key.size  # nothing else was touched


@pytest.mark.parametrize("dtype", DTYPES)
def test_reference_kernel_test_gather_case(dtype):
    """tests/kvx_kernel_test.cu:629-786: 2 sequences x 4 tokens, H=2, D=4, identity S32 table,
    cache = 0.05 + 0.01 i (V + 0.5)."""
    geom = abi.CacheGeometry(2, 4, 2, 4)
    val = np.float32(0.05) + np.float32(0.01) * np.arange(geom.elems, dtype=np.float32)
    ck, cv = f32_to_bits(val, dtype), f32_to_bits(val + np.float32(0.5), dtype)
    empty = np.zeros((0, 2, 4), ck.dtype)
    out = np.zeros((2, 4, 2, 4), ck.dtype)
    case = Case(geom=geom, cache_dtype=dtype, io_dtype=dtype, key=empty, value=empty,
                slots=np.zeros(0, np.int64), cache_k=ck, cache_v=cv,
                table=np.array([[0], [1]], np.int32), lens=np.array([4, 4], np.int32), max_seq_len=4,
                out_k=out.copy(), out_v=out.copy())
    st, ok_, ov_ = oracle_gather(case)
    assert st == abi.STATUS_OK
    assert np.array_equal(ok_.reshape(-1), ck) and np.array_equal(ov_.reshape(-1), cv)


@pytest.mark.parametrize("layout", [abi.LAYOUT_NHD, abi.LAYOUT_HND])
def test_ragged_table_gather_matches_numpy_statement(layout):
    """RAGGED tables: one page id per cached token (KVX_SPEC.md:108-114).  Same result as the
    PACKED form of the same pages; a token list shorter than seq_lens stops the gather."""
    for seed, kw in enumerate([dict(lens=[9, 4, 0, 13], num_blocks=16), dict(lens=[5, 12], max_seq_len=7, bad_blocks=2),
                               dict(lens=[20, 3], index_dtype=np.int64, block_size=5, num_blocks=8)]):
        packed = cases.make_case(400 + seed, layout=layout, dtype=abi.DTYPE_BF16, **kw)
        _, k, v = oracle_write(packed)
        _, pk, pv = oracle_gather(packed, k, v)
        for indptr_dtype, trunc in ((np.int32, ()), (np.int64, (0,))):
            rag = cases.to_ragged(packed, indptr_dtype, truncate=trunc)
            st, rk, rv = oracle_gather(rag, k, v)
            assert st == abi.STATUS_OK
            ek, ev = cases.expected_gather_ragged_numpy(rag, k, v)
            assert np.array_equal(rk, ek) and np.array_equal(rv, ev)
            if not trunc and packed.table.shape[1] * packed.geom.block_size >= packed.max_seq_len:
                assert np.array_equal(rk, pk) and np.array_equal(rv, pv)
            bad = cases.damage_indptr(rag, seed)
            st, rk, rv = oracle_gather(bad, k, v)
            assert st == abi.STATUS_OK
            ek, ev = cases.expected_gather_ragged_numpy(bad, k, v)
            assert np.array_equal(rk, ek) and np.array_equal(rv, ev)


@pytest.mark.parametrize("layout", [abi.LAYOUT_NHD, abi.LAYOUT_HND])
def test_kv_offsets_table_gather_equals_packed(layout):
    """KV_OFFSETS tables (KVX_SPEC.md:116-122): K and V pages scattered over a primary and a
    secondary pool give the PACKED result of the same pages; without the secondary pool its
    pages are skipped; more than one beam is UNSUPPORTED."""
    for seed, kw in enumerate([dict(lens=[9, 4, 0, 13], num_blocks=16), dict(lens=[5, 12], max_seq_len=7, bad_blocks=2),
                               dict(lens=[20, 3], block_size=8, num_blocks=8, max_blocks=2)]):
        packed = cases.make_case(450 + seed, layout=layout, dtype=abi.DTYPE_BF16, **kw)
        _, k, v = oracle_write(packed)
        _, pk, pv = oracle_gather(packed, k, v)
        off = cases.to_kv_offsets(packed, k, v, seed=seed)
        st, ok_, ov_ = oracle_gather(off)
        assert st == abi.STATUS_OK
        assert np.array_equal(ok_, pk) and np.array_equal(ov_, pv)
        bare = cases.to_kv_offsets(packed, k, v, seed=seed, with_secondary=False)
        st, ok_, ov_ = oracle_gather(bare)
        assert st == abi.STATUS_OK
        ek, ev = cases.expected_without_secondary(packed, bare, pk, pv)
        assert np.array_equal(ok_, ek) and np.array_equal(ov_, ev)
        if seed == 0:
            assert not np.array_equal(ek, pk), "the case should have pages in the secondary pool"
    import dataclasses
    beams = dataclasses.replace(off, kv_offsets=np.repeat(off.kv_offsets, 2, axis=1))
    assert oracle_gather(beams)[0] == abi.STATUS_UNSUPPORTED


def test_varlen_output_gather_equals_padded_rows():
    """Un-padded outputs: row out_indptr[s] + tok holds what the padded gather puts at [s, tok];
    rows between sequences, beyond a short allotment and beyond the tensor stay untouched."""
    for seed, kw in enumerate([dict(lens=[9, 4, 0, 13], num_blocks=16), dict(lens=[5, 12], max_seq_len=7, bad_blocks=2),
                               dict(lens=[20, 3], index_dtype=np.int64, block_size=5, num_blocks=8)]):
        packed = cases.make_case(470 + seed, dtype=abi.DTYPE_F16, **kw)
        _, k, v = oracle_write(packed)
        _, pk, pv = oracle_gather(packed, k, v)
        for vkw in (dict(), dict(indptr_dtype=np.int64, gap=2), dict(short=(0,)), dict(rows_cut=3)):
            var = cases.to_varlen(packed, **vkw)
            st, ok_, ov_ = oracle_gather(var, k, v)
            assert st == abi.STATUS_OK
            ek, ev = cases.expected_varlen_from_padded(var, pk, pv)
            assert np.array_equal(ok_, ek) and np.array_equal(ov_, ev), (seed, vkw)
        rag = cases.to_varlen(cases.to_ragged(packed))
        st, ok_, ov_ = oracle_gather(rag, k, v)
        ek, ev = cases.expected_varlen_from_padded(rag, pk, pv)
        if packed.table.shape[1] * packed.geom.block_size >= packed.max_seq_len:
            assert np.array_equal(ok_, ek) and np.array_equal(ov_, ev)


@pytest.mark.parametrize("layout", [abi.LAYOUT_NHD, abi.LAYOUT_HND, abi.LAYOUT_HND_PACKED])
def test_attention_checker_matches_numpy_statement(layout):
    """The checker's decode attention against an independent numpy formulation: gather the
    sequence's K / V rows through the numpy statement of the gather, then a float64 softmax."""
    import ctypes as C
    from harness import bits_to_f32, descriptors, f32_to_bits, host_buffers
    from oracle.kvx_oracle import oracle
    pack = 4 if layout == abi.LAYOUT_HND_PACKED else 1
    case = cases.make_case(480, layout=layout, pack=pack, dtype=abi.DTYPE_F32, real_values=True, heads=2, dim=8,
                           block_size=4, num_blocks=16, lens=[9, 4, 0, 13], bad_blocks=1)
    _, k, v = oracle_write(case)
    G, S, H, D = 3, 4, 2, 8
    rng = np.random.default_rng(1)
    q = rng.standard_normal((S, H * G, D)).astype(np.float32)
    out = np.zeros_like(q)
    import dataclasses
    hb = host_buffers(dataclasses.replace(case, cache_k=k, cache_v=v))
    cache, _, _, ks, vs = descriptors(case, hb, abi.MEMORY_HOST)
    a = abi.attention_desc(S, H * G, D, abi.DTYPE_F32, q.ctypes.data, out.ctypes.data, 0.3, case.max_seq_len,
                           abi.DTYPE_S32, hb["table"].ctypes.data, case.table.shape[1], hb["lens"].ctypes.data,
                           abi.MEMORY_HOST)
    assert oracle().kvx_oracle_paged_attention_decode(C.byref(cache), C.byref(a), C.byref(ks), C.byref(vs)) == 0
    # numpy: the gather statement leaves skipped tokens at the sentinel; find them with a marker
    marked = dataclasses.replace(case, out_k=np.full_like(case.out_k, 0x7FC00001), out_v=np.full_like(case.out_v, 0x7FC00001))
    gk, gv = cases.expected_gather_numpy(marked, k, v)
    gk, gv = gk.view(np.float32), gv.view(np.float32)
    for s in range(S):
        n = min(int(case.lens[s]), case.max_seq_len)
        for hq in range(H * G):
            h = hq // G
            live = [t for t in range(n) if not np.isnan(gk[s, t, h, 0])]
            if not live:
                assert not out[s, hq].any()
                continue
            sc = np.array([np.dot(q[s, hq].astype(np.float64), gk[s, t, h].astype(np.float64)) * np.float64(np.float32(0.3)) for t in live])
            w = np.exp(sc - sc.max()); w /= w.sum()
            ref = sum(w[i] * gv[s, t, h].astype(np.float64) for i, t in enumerate(live))
            assert np.allclose(out[s, hq], ref, rtol=1e-6, atol=1e-7), (s, hq)


def test_noncanonical_strides_and_untouched_bytes():
    for layout in (abi.LAYOUT_NHD, abi.LAYOUT_HND):
        case = cases.make_case(7, layout=layout, stride_pad=(16, 8, 8), pad_frac=0.2, lens=[6, 3])
        st, k, v = oracle_write(case)
        assert st == abi.STATUS_OK
        valid = int(np.count_nonzero((case.slots >= 0)))
        g = case.geom
        touched_k = int(np.count_nonzero(k != case.cache_k))
        # random payloads may collide with the sentinel, never exceed the written span
        assert touched_k <= valid * g.num_kv_heads * g.head_dim
        assert touched_k >= valid * g.num_kv_heads * g.head_dim - 4
        st, ok_, _ = oracle_gather(case, k, v)
        assert st == abi.STATUS_OK
        t = 0
        for s, n in enumerate(case.lens.tolist()):
            for tok in range(n):
                if case.slots[t] >= 0:
                    assert np.array_equal(ok_[s, tok], case.key[t])
                t += 1


def test_write_then_gather_round_trip_tinyllama_shape():
    """TinyLlama KV shape: fp16, 4 heads of 64, block 16, 8 sequences x 128 tokens, pages from
    a seeded permutation of a 512-block pool; gather(write(x)) == x."""
    case = cases.make_case(1, dtype=abi.DTYPE_F16, num_blocks=512, block_size=16, heads=4, dim=64,
                           lens=[128] * 8, real_values=True)
    st, k, v = oracle_write(case)
    assert st == abi.STATUS_OK
    st, ok_, ov_ = oracle_gather(case, k, v)
    assert st == abi.STATUS_OK
    assert np.array_equal(ok_.reshape(case.key.shape), case.key)
    assert np.array_equal(ov_.reshape(case.value.shape), case.value)


def test_cpu_baseline_matches_oracle():
    from oracle.kvx_oracle import oracle
    case = cases.make_case(5, dtype=abi.DTYPE_BF16, num_blocks=64, block_size=8, heads=4, dim=32,
                           lens=[40, 3, 0, 17, 64], pad_frac=0.15, oob_slots=2, bad_blocks=2)
    st, k, v = oracle_write(case)
    for threads in (1, 3):
        b = host_buffers(case)
        cache, write, gather, _, _ = descriptors(case, b, abi.MEMORY_HOST)
        assert oracle().kvx_cpu_baseline_write_kv(C.byref(cache), C.byref(write), threads) == abi.STATUS_OK
        assert np.array_equal(b["cache_k"], k) and np.array_equal(b["cache_v"], v)
        assert oracle().kvx_cpu_baseline_gather_kv(C.byref(cache), C.byref(gather), threads) == abi.STATUS_OK
        _, ok_, ov_ = oracle_gather(case, k, v)
        assert np.array_equal(b["out_k"], ok_) and np.array_equal(b["out_v"], ov_)


# ------------------------------------------------------------------ fp8 e4m3 -------------

def _oracle_encode(x: np.ndarray) -> np.ndarray:
    from oracle.kvx_oracle import oracle
    f = oracle().kvx_oracle_e4m3_from_f32
    return np.array([f(float(v)) for v in x], dtype=np.uint8)


def test_e4m3_decode_table_matches_ml_dtypes():
    import ml_dtypes
    from oracle.kvx_oracle import oracle
    codes = np.arange(256, dtype=np.uint8)
    want = codes.view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    got = np.array([oracle().kvx_oracle_e4m3_to_f32(int(c)) for c in codes], dtype=np.float32)
    finite = ~np.isnan(want)
    assert np.array_equal(got[finite].view(np.uint32), want[finite].view(np.uint32))
    assert np.isnan(got[~finite]).all() and set(codes[~finite].tolist()) == {0x7F, 0xFF}


def test_e4m3_encode_matches_ml_dtypes_on_finite_range_and_saturates():
    """Every bf16 value times a few scales + random f32 patterns.  ml_dtypes / torch round to
    nearest even but overflow to NaN above 464, so inputs are clamped to +-448 for them; the
    checker itself must saturate."""
    import ml_dtypes
    rng = np.random.default_rng(3)
    bf = (np.arange(1 << 16, dtype=np.uint32) << 16).view(np.float32)
    xs = [bf, bf * np.float32(0.37), bf * np.float32(3.3), rng.integers(0, 2 ** 32, 200000, dtype=np.uint64).astype(np.uint32).view(np.float32),
          np.array([448.0, 449.0, 463.9, 464.0, 1e9, np.inf, -np.inf, 17.0, 19.0, 2 ** -10, 3 * 2 ** -11, 2 ** -9, 0.0, -0.0], np.float32)]
    x = np.concatenate(xs)
    x = x[~np.isnan(x)]
    got = _oracle_encode(x)
    want = np.clip(x, -448.0, 448.0).astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    assert np.array_equal(got, want)
    assert _oracle_encode(np.array([np.nan], np.float32))[0] == 0x7F
    neg_nan = np.array([0xFFC00001], np.uint32).view(np.float32)
    assert _oracle_encode(neg_nan)[0] == 0x7F
    assert _oracle_encode(np.array([-0.0], np.float32))[0] == 0x80


def test_e4m3_encode_matches_torch():
    import torch
    x = torch.randn(100000, dtype=torch.float32) * 60
    want = x.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(_oracle_encode(x.numpy()), want)


@pytest.mark.parametrize("io", DTYPES)
@pytest.mark.parametrize("gran", [abi.SCALE_PER_HEAD, abi.SCALE_PER_TENSOR])
def test_fp8_write_gather_semantics(io, gran):
    """quantise = one f32 division + one rounding; dequantise = one f32 multiply + rounding
    to the IO type.  Recomputed with numpy / ml_dtypes."""
    import ml_dtypes
    case = cases.make_case(11, dtype=io, cache_dtype=abi.DTYPE_F8_E4M3, real_values=True, heads=3, dim=16,
                           lens=[9, 5], num_blocks=8, pad_frac=0.2, scale_gran=gran)
    st, k, v = oracle_write(case)
    assert st == abi.STATUS_OK
    g = case.geom
    kk = k.reshape(g.shape)
    x = bits_to_f32(case.key, io)
    scale = case.k_scale if gran == abi.SCALE_PER_HEAD else np.repeat(case.k_scale, g.num_kv_heads)
    for t, slot in enumerate(case.slots.tolist()):
        if slot < 0:
            continue
        b, o = divmod(slot, g.block_size)
        y = (x[t] / scale[:, None].astype(np.float32)).astype(np.float32)
        want = np.clip(y, -448, 448).astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
        assert np.array_equal(kk[b, o], want)
    st, ok_, _ = oracle_gather(case, k, v)
    assert st == abi.STATUS_OK
    t = 0
    for s, n in enumerate(case.lens.tolist()):
        for tok in range(n):
            if case.slots[t] >= 0:
                b, o = divmod(int(case.slots[t]), g.block_size)
                f = kk[b, o].view(ml_dtypes.float8_e4m3fn).astype(np.float32)
                z = (f * scale[:, None].astype(np.float32)).astype(np.float32)
                assert np.array_equal(ok_[s, tok], f32_to_bits(z, io))
            t += 1


def test_scales_from_absmax():
    from oracle.kvx_oracle import oracle
    rng = np.random.default_rng(9)
    for io in DTYPES:
        x = rng.standard_normal((37, 4, 16)).astype(np.float32)
        x[5, 2, 3] = -77.0
        key, value = f32_to_bits(x, io), f32_to_bits(x * 0, io)
        kio = abi.write_desc(37, 4, 16, io, key.ctypes.data, value.ctypes.data, abi.DTYPE_S64, 0, abi.MEMORY_HOST).io
        ks, vs = np.zeros(4, np.float32), np.zeros(4, np.float32)
        assert oracle().kvx_oracle_kv_scales(C.byref(kio), abi.SCALE_PER_HEAD, ks.ctypes.data, vs.ctypes.data) == 0
        want = (np.abs(bits_to_f32(key, io)).max(axis=(0, 2)) / np.float32(448.0)).astype(np.float32)
        assert np.array_equal(ks, want) and np.array_equal(vs, np.ones(4, np.float32))
        assert oracle().kvx_oracle_kv_scales(C.byref(kio), abi.SCALE_PER_TENSOR, ks.ctypes.data, vs.ctypes.data) == 0
        assert ks[0] == want.max()


# ------------------------------------------------------------------ golden fixtures ------

def test_oracle_matches_reference_kernel_dumps():
    """tests/golden/ref_*.npz hold inputs and the bytes the reference's own CUDA kernels
    (compiled unmodified for sm_100a) produced on a B200 for them."""
    files = sorted(glob.glob(os.path.join(GOLDEN, "ref_*.npz")))
    if not files:
        pytest.skip("no reference dumps committed yet")
    from golden.make_golden_from_ref import case_from_npz
    for path in files:
        z = np.load(path)
        case = case_from_npz(z)
        st, k, v = oracle_write(case)
        assert st == abi.STATUS_OK
        assert np.array_equal(k, z["ref_cache_k"]) and np.array_equal(v, z["ref_cache_v"]), path
        st, ok_, ov_ = oracle_gather(case, k, v)
        assert st == abi.STATUS_OK
        assert np.array_equal(ok_, z["ref_out_k"]) and np.array_equal(ov_, z["ref_out_v"]), path
