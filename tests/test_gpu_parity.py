"""Parity tests proper: the CUDA library, called through its C ABI on a B200, against the
CPU checker on the same seeded inputs -- byte for byte, untouched bytes included."""
import ctypes as C
import dataclasses

import numpy as np
import pytest

import kvx_b200
from kvx_b200 import abi

import cases
from harness import (Case, device_buffers, descriptors, f32_to_bits, gpu_gather, gpu_write, oracle_gather,
                     oracle_write)

pytestmark = pytest.mark.gpu

OK = abi.STATUS_OK
DTYPES = [abi.DTYPE_F32, abi.DTYPE_F16, abi.DTYPE_BF16]
LAYOUTS = [(abi.LAYOUT_NHD, 1), (abi.LAYOUT_HND, 1), (abi.LAYOUT_HND_PACKED, 4)]


@pytest.fixture(autouse=True)
def _defaults():
    """Every test starts from the library's default tuning."""
    saved = {n: kvx_b200.get_option(n) for n in ("gather_path", "force_generic", "write_unroll",
                                                  "write_vecs_per_cta", "gather_part_bytes", "gather_tile_bytes", "wide", "pdl",
                                                  "write_prefetch_waves", "gather_rect_items")}
    yield
    for n, v in saved.items():
        kvx_b200.set_option(n, v)


def check_write(case: Case, entry="dispatch", tps=1):
    st, ek, ev = oracle_write(case)
    assert st == OK
    st, k, v = gpu_write(case, entry, tps)
    assert st == OK, (entry, st)
    assert np.array_equal(k, ek), f"K cache differs ({case.note}, {entry})"
    assert np.array_equal(v, ev), f"V cache differs ({case.note}, {entry})"
    return ek, ev


def check_gather(case: Case, k, v, entry="dispatch"):
    """Every case runs twice: with the (sequence, page) rectangle compacted in the kernel, and
    walked as it is (what the library picks for small rectangles like the ones tested here)."""
    st, ek, ev = oracle_gather(case, k, v)
    assert st == OK
    saved = kvx_b200.get_option("gather_rect_items")
    try:
        for rect in (0, 1 << 40):
            kvx_b200.set_option("gather_rect_items", rect)
            st, gk, gv = gpu_gather(case, k, v, entry)
            assert st == OK, (entry, st)
            assert np.array_equal(gk, ek), f"K out differs ({case.note}, {entry}, rect {rect})"
            assert np.array_equal(gv, ev), f"V out differs ({case.note}, {entry}, rect {rect})"
    finally:
        kvx_b200.set_option("gather_rect_items", saved)


# ------------------------------------------------------------------ reference's own cases -

def _toy(dtype, heads, dim, tps, layout):
    geom = abi.CacheGeometry(2, 4, heads, dim, layout)
    n = 2 * tps * heads * dim
    val = np.float32(0.1) + np.float32(0.01) * np.arange(n, dtype=np.float32)
    key = f32_to_bits(val, dtype).reshape(-1, heads, dim)
    value = f32_to_bits(val + np.float32(0.5), dtype).reshape(-1, heads, dim)
    slots = np.array([s * 4 + (4 - tps) + t for s in range(2) for t in range(tps)], np.int64)
    zeros = np.zeros(geom.elems, dtype=key.dtype)
    return Case(geom=geom, cache_dtype=dtype, io_dtype=dtype, key=key, value=value, slots=slots,
                cache_k=zeros.copy(), cache_v=zeros.copy(), note=f"toy h{heads} d{dim} tps{tps}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,tps,layout", [
    (2, 4, 1, abi.LAYOUT_NHD), (1, 7, 1, abi.LAYOUT_NHD), (2, 4, 2, abi.LAYOUT_NHD),
    (2, 4, 1, abi.LAYOUT_HND), (1, 7, 2, abi.LAYOUT_HND)])
def test_reference_write_cases(dtype, heads, dim, tps, layout):
    """tests/kvx_kernel_test.cu:456-466 and :621-627, every entry point, exact."""
    case = _toy(dtype, heads, dim, tps, layout)
    for entry in ("dispatch", "typed", "prefill", "prefill_typed"):
        check_write(case, entry, tps)


@pytest.mark.parametrize("dtype", DTYPES)
def test_reference_gather_case(dtype):
    """tests/kvx_kernel_test.cu:629-786."""
    geom = abi.CacheGeometry(2, 4, 2, 4)
    val = np.float32(0.05) + np.float32(0.01) * np.arange(geom.elems, dtype=np.float32)
    ck, cv = f32_to_bits(val, dtype), f32_to_bits(val + np.float32(0.5), dtype)
    empty = np.zeros((0, 2, 4), ck.dtype)
    out = np.zeros((2, 4, 2, 4), ck.dtype)
    case = Case(geom=geom, cache_dtype=dtype, io_dtype=dtype, key=empty, value=empty,
                slots=np.zeros(0, np.int64), cache_k=ck, cache_v=cv, table=np.array([[0], [1]], np.int32),
                lens=np.array([4, 4], np.int32), max_seq_len=4, out_k=out.copy(), out_v=out.copy())
    for entry in ("dispatch", "typed"):
        check_gather(case, ck, cv, entry)


# ------------------------------------------------------------------ the matrix ------------

VARIANTS = [
    dict(),
    dict(pad_frac=0.3, slot_dtype=np.int32),
    dict(oob_slots=3, bad_blocks=3, index_dtype=np.int64),
    dict(lens=[0, 9, 4, 1], num_blocks=16),
    dict(lens=[5, 12], max_seq_len=7, max_blocks=2),
    dict(heads=1, dim=7, lens=[9, 2]),                       # odd head_dim -> generic tier
    dict(heads=3, dim=24, block_size=5, lens=[11, 5, 0, 3], num_blocks=9),  # nothing is a power of two
]


@pytest.mark.parametrize("layout,pack", LAYOUTS)
@pytest.mark.parametrize("dtype", DTYPES)
def test_matrix_small(layout, pack, dtype):
    for i, kw in enumerate(VARIANTS):
        if layout == abi.LAYOUT_HND_PACKED and kw.get("dim", 8) % pack:
            continue
        case = cases.make_case(200 + i, layout=layout, pack=pack, dtype=dtype, **kw)
        case.note = f"variant {i}"
        k, v = check_write(case)
        check_write(case, "prefill", 1)
        check_gather(case, k, v)


@pytest.mark.parametrize("layout", [abi.LAYOUT_NHD, abi.LAYOUT_HND])
@pytest.mark.parametrize("dtype", DTYPES)
def test_vector_tier_shapes(layout, dtype):
    """Shapes whose rows are whole 16-byte vectors: the vector tiers, ragged lengths,
    padding, out-of-range ids, both index widths."""
    for i, kw in enumerate([
        dict(heads=8, dim=128, block_size=16, num_blocks=40, lens=[100, 17, 256, 1, 0, 33], pad_frac=0.1),
        dict(heads=1, dim=128, block_size=16, num_blocks=40, lens=[64, 200], slot_dtype=np.int32, index_dtype=np.int64,
             oob_slots=5, bad_blocks=4),
        dict(heads=4, dim=64, block_size=32, num_blocks=20, lens=[31, 33, 160], pad_frac=0.5),
        dict(heads=3, dim=40, block_size=6, num_blocks=50, lens=[7, 100, 13], pad_frac=0.05),
        dict(heads=2, dim=8, block_size=4, num_blocks=64, lens=[50, 70], max_seq_len=40, max_blocks=9),
    ]):
        case = cases.make_case(300 + i, layout=layout, dtype=dtype, **kw)
        case.note = f"vec {i}"
        k, v = check_write(case)
        check_gather(case, k, v)
        kvx_b200.set_option("force_generic", 1)
        check_write(case)
        check_gather(case, k, v)
        kvx_b200.set_option("force_generic", 0)


@pytest.mark.parametrize("layout", [abi.LAYOUT_NHD, abi.LAYOUT_HND])
def test_noncanonical_strides(layout):
    """Padded block / token / head pitches (what views of a fused [blocks, 2, ...] allocation
    look like): still the vector tier, K and V with different strides."""
    # (32, 16, 16): every pitch a multiple of 32 bytes -> the 256-bit segmented gather;
    # (3, 1, 1) is misaligned -> generic
    for pad in ((16, 8, 8), (32, 16, 16), (4096, 0, 0), (0, 8, 0), (3, 1, 1)):
        case = cases.make_case(41, layout=layout, dtype=abi.DTYPE_BF16, heads=4, dim=64, block_size=8,
                               num_blocks=12, lens=[20, 8, 31], pad_frac=0.1, stride_pad=pad)
        case.note = f"pad {pad}"
        k, v = check_write(case)
        check_gather(case, k, v)


def test_tuning_knobs_do_not_change_results():
    case = cases.make_case(77, dtype=abi.DTYPE_BF16, heads=8, dim=128, block_size=16, num_blocks=80,
                           lens=[300, 77, 512, 9], pad_frac=0.1)
    _, ek, ev = oracle_write(case)
    for unroll in (1, 2, 4):
        for vecs in (128, 1024, 8192):
            kvx_b200.set_option("write_unroll", unroll)
            kvx_b200.set_option("write_vecs_per_cta", vecs)
            check_write(case)
    kvx_b200.set_option("gather_path", 0)  # CTA-granular items
    for tile in (4096, 16384, 65536):
        kvx_b200.set_option("gather_tile_bytes", tile)
        check_gather(case, ek, ev)
    kvx_b200.set_option("gather_path", 2)  # warp-granular items
    for wide in (0, 1):                    # 128-bit and 256-bit accesses
        for pdl in (0, 1):                 # with and without programmatic dependent launch
            kvx_b200.set_option("wide", wide)
            kvx_b200.set_option("pdl", pdl)
            for part in (512, 4096, 65536):
                kvx_b200.set_option("gather_part_bytes", part)
                check_gather(case, ek, ev)
            for waves in (0, 1, 2):        # leading write CTAs that prefetch their rows
                kvx_b200.set_option("write_prefetch_waves", waves)
                check_write(case)


def test_bulk_gather_path_matches():
    """cp.async.bulk staging tier of the gather."""
    kvx_b200.set_option("gather_path", 1)
    for i, kw in enumerate([
        dict(heads=8, dim=128, block_size=16, num_blocks=60, lens=[100, 17, 256, 1, 0, 333], bad_blocks=3),
        dict(heads=2, dim=64, block_size=32, num_blocks=30, lens=[31, 33, 160], index_dtype=np.int64),
        dict(heads=8, dim=128, block_size=32, num_blocks=12, lens=[300, 5]),  # chunk larger than a stage
        dict(heads=1, dim=8, block_size=4, num_blocks=64, lens=[50, 70], max_seq_len=40, max_blocks=9),
    ]):
        case = cases.make_case(500 + i, dtype=abi.DTYPE_BF16, **kw)
        _, k, v = oracle_write(case)
        check_gather(case, k, v)


@pytest.mark.parametrize("dtype", [abi.DTYPE_BF16, abi.DTYPE_F32])
@pytest.mark.parametrize("layout", [abi.LAYOUT_NHD, abi.LAYOUT_HND])
def test_ragged_block_table_gather(layout, dtype):
    """RAGGED tables (one page id per cached token), which the reference validates but answers
    UNSUPPORTED for: vector tier, generic tier (odd head_dim), both index widths, truncated
    token lists, invalid ids."""
    for i, kw in enumerate([
        dict(heads=8, dim=128, block_size=16, num_blocks=60, lens=[100, 17, 256, 1, 0, 333], bad_blocks=3),
        dict(heads=2, dim=64, block_size=32, num_blocks=30, lens=[31, 33, 160], index_dtype=np.int64),
        dict(heads=1, dim=7, block_size=4, num_blocks=16, lens=[9, 4, 0, 6]),
        dict(heads=3, dim=24, block_size=5, num_blocks=40, lens=[50, 70], max_seq_len=40),
    ]):
        packed = cases.make_case(800 + i, layout=layout, dtype=dtype, **kw)
        _, k, v = oracle_write(packed)
        for indptr_dtype, trunc in ((np.int32, ()), (np.int64, (0, 1))):
            rag = cases.to_ragged(packed, indptr_dtype, truncate=trunc)
            rag.note = f"ragged {i}"
            check_gather(rag, k, v)
            check_gather(rag, k, v, "typed")
            bad = cases.damage_indptr(rag, i)   # entries outside the index array are skipped, never read
            bad.note = f"ragged {i}, damaged indptr"
            check_gather(bad, k, v)


def test_ragged_block_table_gather_fp8():
    packed = cases.make_case(850, dtype=abi.DTYPE_BF16, cache_dtype=abi.DTYPE_F8_E4M3, real_values=True, heads=4,
                             dim=64, block_size=16, num_blocks=24, lens=[100, 40, 7], scale_gran=abi.SCALE_PER_HEAD)
    _, k, v = oracle_write(packed)
    check_gather(cases.to_ragged(packed), k, v)


@pytest.mark.parametrize("dtype", [abi.DTYPE_BF16, abi.DTYPE_F32])
@pytest.mark.parametrize("layout", [abi.LAYOUT_NHD, abi.LAYOUT_HND])
def test_kv_offsets_block_table_gather(layout, dtype):
    """KV_OFFSETS tables (TensorRT-LLM form: separate K and V page offsets into a primary and a
    secondary pool, bit 31 selecting the pool), which the reference validates but answers
    UNSUPPORTED for: vector tier and generic tier (odd head_dim), entries beyond the pool,
    a withheld secondary pool; the result must also equal the PACKED gather of the same pages."""
    for i, kw in enumerate([
        dict(heads=8, dim=128, block_size=16, num_blocks=60, lens=[100, 17, 256, 1, 0, 333], bad_blocks=3),
        dict(heads=2, dim=64, block_size=32, num_blocks=30, lens=[31, 33, 160]),
        dict(heads=1, dim=7, block_size=4, num_blocks=16, lens=[9, 4, 0, 6]),
        dict(heads=3, dim=24, block_size=8, num_blocks=40, lens=[50, 70], max_seq_len=40),
    ]):
        packed = cases.make_case(900 + i, layout=layout, dtype=dtype, **kw)
        _, k, v = oracle_write(packed)
        _, pk, pv = oracle_gather(packed, k, v)
        off = cases.to_kv_offsets(packed, k, v, seed=i)
        off.note = f"kv_offsets {i}"
        check_gather(off, k, v)
        check_gather(off, k, v, "typed")
        st, gk, gv = gpu_gather(off, k, v)
        assert np.array_equal(gk, pk) and np.array_equal(gv, pv)
        bare = cases.to_kv_offsets(packed, k, v, seed=i, with_secondary=False)
        check_gather(bare, k, v)
        ek, ev = cases.expected_without_secondary(packed, bare, pk, pv)
        st, gk, gv = gpu_gather(bare, k, v)
        assert np.array_equal(gk, ek) and np.array_equal(gv, ev)


def test_kv_offsets_block_table_gather_fp8():
    packed = cases.make_case(950, dtype=abi.DTYPE_BF16, cache_dtype=abi.DTYPE_F8_E4M3, real_values=True, heads=4,
                             dim=64, block_size=16, num_blocks=24, lens=[100, 40, 7], scale_gran=abi.SCALE_PER_HEAD,
                             layout=abi.LAYOUT_HND)
    _, k, v = oracle_write(packed)
    _, pk, pv = oracle_gather(packed, k, v)
    off = cases.to_kv_offsets(packed, k, v, seed=5)
    check_gather(off, k, v)
    st, gk, gv = gpu_gather(off, k, v)
    assert np.array_equal(gk, pk) and np.array_equal(gv, pv)


@pytest.mark.parametrize("layout", [abi.LAYOUT_NHD, abi.LAYOUT_HND])
def test_varlen_output_gather(layout):
    """kvx_launch_gather_kv_varlen: un-padded [rows, H, D] outputs addressed through out_indptr,
    with every table format, both index widths, gaps, short allotments and truncated tensors;
    the vector tiers (wide and 16-byte) and the generic tier (odd head_dim)."""
    for i, kw in enumerate([
        dict(heads=8, dim=128, block_size=16, num_blocks=60, lens=[100, 17, 256, 1, 0, 333], bad_blocks=3),
        dict(heads=2, dim=64, block_size=32, num_blocks=30, lens=[31, 33, 160], index_dtype=np.int64),
        dict(heads=1, dim=7, block_size=4, num_blocks=16, lens=[9, 4, 0, 6]),
        dict(heads=3, dim=24, block_size=8, num_blocks=40, lens=[50, 70], max_seq_len=40),
    ]):
        packed = cases.make_case(1000 + i, layout=layout, dtype=abi.DTYPE_BF16, **kw)
        _, k, v = oracle_write(packed)
        _, pk, pv = oracle_gather(packed, k, v)
        for vkw in (dict(), dict(indptr_dtype=np.int64, gap=3), dict(short=(0, 1)), dict(rows_cut=5)):
            var = cases.to_varlen(packed, **vkw)
            var.note = f"varlen {i} {vkw}"
            check_gather(var, k, v)
            ek, ev = cases.expected_varlen_from_padded(var, pk, pv)
            st, gk, gv = gpu_gather(var, k, v)
            assert np.array_equal(gk, ek) and np.array_equal(gv, ev), var.note
        check_gather(cases.to_varlen(cases.to_ragged(packed)), k, v)
        if packed.table.dtype == np.int32:
            check_gather(cases.to_varlen(cases.to_kv_offsets(packed, k, v, seed=i)), k, v)


def test_varlen_output_gather_fp8_and_statuses():
    packed = cases.make_case(1050, dtype=abi.DTYPE_BF16, cache_dtype=abi.DTYPE_F8_E4M3, real_values=True, heads=4,
                             dim=64, block_size=16, num_blocks=24, lens=[100, 40, 7], scale_gran=abi.SCALE_PER_HEAD)
    _, k, v = oracle_write(packed)
    var = cases.to_varlen(packed, gap=1)
    check_gather(var, k, v)
    # a 4-D output, a missing or mistyped out_indptr are refused before any launch
    import ctypes as C
    import kvx_b200
    from harness import descriptors, device_buffers
    L = kvx_b200.lib()
    b = device_buffers(var)
    cache, _, g, ks, vs = descriptors(var, b, abi.MEMORY_DEVICE)
    ptr = b["out_indptr"].data_ptr()
    assert L.kvx_launch_gather_kv_varlen(C.byref(cache), C.byref(g), None, abi.DTYPE_S32, C.byref(ks), C.byref(vs), None) \
        == abi.STATUS_INVALID_ARGUMENT
    assert L.kvx_launch_gather_kv_varlen(C.byref(cache), C.byref(g), ptr, abi.DTYPE_F32, C.byref(ks), C.byref(vs), None) \
        == abi.STATUS_INVALID_ARGUMENT
    b2 = device_buffers(packed)
    cache2, _, g2, ks2, vs2 = descriptors(packed, b2, abi.MEMORY_DEVICE)
    assert L.kvx_launch_gather_kv_varlen(C.byref(cache2), C.byref(g2), ptr, abi.DTYPE_S32, C.byref(ks2), C.byref(vs2), None) \
        == abi.STATUS_INVALID_ARGUMENT


@pytest.mark.parametrize("dtype", [abi.DTYPE_BF16, abi.DTYPE_F16, abi.DTYPE_F32])
def test_hnd_packed_with_16_byte_pack_groups(dtype):
    """HND_PACKED pages [blocks, heads, dim / x, block_size, x] with x = 16 bytes / element size
    (the packing of vLLM's and TGI's non-flash paged attention) take the vector tier: one
    16-byte vector per pack group.  Other packings stay on the generic tier; both must equal
    the checker."""
    x = 16 // (4 if dtype == abi.DTYPE_F32 else 2)
    for i, kw in enumerate([
        dict(heads=4, dim=64, block_size=16, num_blocks=40, lens=[100, 17, 256, 1, 0, 33], pad_frac=0.1, bad_blocks=2),
        dict(heads=8, dim=128, block_size=32, num_blocks=20, lens=[300, 5, 64], index_dtype=np.int64,
             slot_dtype=np.int32),
        dict(heads=1, dim=x, block_size=4, num_blocks=16, lens=[9, 4, 0, 6]),
        dict(heads=2, dim=4 * x, block_size=8, num_blocks=12, lens=[50, 20], max_seq_len=40, oob_slots=2),
    ]):
        case = cases.make_case(1100 + i, layout=abi.LAYOUT_HND_PACKED, pack=x, dtype=dtype, **kw)
        case.note = f"packed16 {i}"
        k, v = check_write(case)
        check_write(case, "prefill", 1)
        check_gather(case, k, v)
        check_gather(case, k, v, "typed")
        check_gather(cases.to_varlen(case, gap=1), k, v)
        wide = cases.make_case(1150 + i, layout=abi.LAYOUT_HND_PACKED, pack=2 * x, dtype=dtype,
                               **{**kw, "dim": max(kw["dim"], 2 * x)})
        k, v = check_write(wide)
        check_gather(wide, k, v)


def test_more_sequences_than_the_shared_memory_prefix_holds():
    """Beyond 10 240 sequences the gather kernels cannot keep the page-count prefix in shared
    memory and walk the padded (sequence, page) rectangle instead; same result."""
    rng = np.random.default_rng(77)
    lens = [int(x) for x in rng.integers(0, 10, size=10500)]
    for dim in (16, 8):  # 256-bit and 128-bit vector kernels
        case = cases.make_case(1200 + dim, dtype=abi.DTYPE_BF16, heads=1, dim=dim, block_size=4, num_blocks=27000,
                               lens=lens, bad_blocks=5)
        case.note = f"many sequences, dim {dim}"
        _, k, v = oracle_write(case)
        check_gather(case, k, v)
        check_gather(cases.to_varlen(case), k, v)


@pytest.mark.parametrize("layout", [abi.LAYOUT_NHD, abi.LAYOUT_HND])
def test_key_value_rows_with_a_token_pitch(layout):
    """key / value whose token rows are further apart than heads * dim (slices of a fused
    projection output, which vLLM passes to its own operator): accepted by the write launchers
    here (the reference answers UNSUPPORTED), vector tier for 16-byte pitches, generic tier
    otherwise, fp8 cache included; what lies between the rows must not reach the cache."""
    for i, (kw, extras) in enumerate([
        (dict(heads=8, dim=128, block_size=16, num_blocks=40, lens=[100, 17, 256, 1, 0, 33], pad_frac=0.1), (2048, 1024)),
        (dict(heads=2, dim=64, block_size=32, num_blocks=20, lens=[31, 33, 160], slot_dtype=np.int32), (8, 0)),
        (dict(heads=2, dim=64, block_size=16, num_blocks=20, lens=[50, 70]), (3, 5)),           # misaligned pitch
        (dict(heads=3, dim=40, block_size=6, num_blocks=50, lens=[7, 100, 13], oob_slots=2), (40, 40)),
    ]):
        case = cases.to_pitched(cases.make_case(1300 + i, layout=layout, dtype=abi.DTYPE_BF16, **kw), *extras, seed=i)
        case.note = f"pitched {i}"
        check_write(case)
        check_write(case, "typed")
        check_write(case, "prefill", 1)
    f8 = cases.make_case(1350, layout=layout, dtype=abi.DTYPE_BF16, cache_dtype=abi.DTYPE_F8_E4M3, real_values=True,
                         heads=4, dim=64, block_size=16, num_blocks=24, lens=[100, 40, 7], scale_gran=abi.SCALE_PER_HEAD)
    check_write(cases.to_pitched(f8, 256, 64))
    check_write(cases.to_pitched(f8, 1, 0))


def test_empty_and_degenerate_batches():
    case = cases.make_case(3, dtype=abi.DTYPE_F16, heads=2, dim=64, lens=[0, 0], num_blocks=4)
    assert case.T == 0
    st, k, v = gpu_write(case)
    assert st == OK and np.array_equal(k, case.cache_k) and np.array_equal(v, case.cache_v)
    st, gk, gv = gpu_gather(case, k, v)
    assert st == OK and np.array_equal(gk, case.out_k) and np.array_equal(gv, case.out_v)
    # every slot padded
    case = cases.make_case(4, dtype=abi.DTYPE_F16, heads=2, dim=64, lens=[9, 3], num_blocks=4, pad_frac=1.1)
    st, k, v = gpu_write(case)
    assert st == OK and np.array_equal(k, case.cache_k)


def test_non_default_stream():
    import torch
    case = cases.make_case(8, dtype=abi.DTYPE_BF16, heads=4, dim=64, block_size=16, num_blocks=16, lens=[100, 50])
    _, ek, ev = oracle_write(case)
    s = torch.cuda.Stream()
    st, k, v = gpu_write(case, stream=s.cuda_stream)
    assert st == OK and np.array_equal(k, ek) and np.array_equal(v, ev)
    _, eok, _ = oracle_gather(case, ek, ev)
    st, gk, _ = gpu_gather(case, ek, ev, stream=s.cuda_stream)
    assert st == OK and np.array_equal(gk, eok)
