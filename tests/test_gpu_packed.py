"""HND_PACKED pages ([blocks, heads, dim / pack, block_size, pack]) through the transposing
kernels: every pack size whose group is 2, 4, 8 or 16 bytes, K and V with different packs (the
"paged" caches of vLLM and TGI: K in 16-byte groups, V [blocks, heads, dim, block_size]), page
sizes and strides that do and do not qualify, padding, out-of-range slots and page ids, partial
last pages, pitched key / value rows -- byte for byte against the CPU checker, and against the
one-element-per-thread tier of the library itself."""
import numpy as np
import pytest

import kvx_b200
from kvx_b200 import abi

import cases
from harness import gpu_gather, gpu_write, oracle_gather, oracle_write

pytestmark = pytest.mark.gpu
OK = abi.STATUS_OK
PACKED = abi.LAYOUT_HND_PACKED


@pytest.fixture(autouse=True)
def _defaults():
    saved = {n: kvx_b200.get_option(n) for n in ("packed_tiles", "force_generic", "gather_rect_items",
                                                 "packed_lines_variant", "packed_fill_halves")}
    yield
    for n, v in saved.items():
        kvx_b200.set_option(n, v)


def _check(case, knobs=(1,)):
    """knobs: values of the packed_tiles tuning knob to run with: 1 = the library's choice, 2 = the
    fragment write kernel also where K and V are both in 16-byte groups, 3 = the gather without its
    whole-line lane order, 0 = the older tiers (row kernel for 16-byte groups, one element per thread
    otherwise)."""
    st, ek, ev = oracle_write(case)
    assert st == OK
    st, eok, eov = oracle_gather(case, ek, ev)
    assert st == OK
    for knob in knobs:
        kvx_b200.set_option("packed_tiles", knob)
        st, k, v = gpu_write(case)
        assert st == OK
        assert np.array_equal(k, ek), f"K pages differ ({case.note}, packed_tiles {knob})"
        assert np.array_equal(v, ev), f"V pages differ ({case.note}, packed_tiles {knob})"
        for rect in (0, 1 << 40):
            kvx_b200.set_option("gather_rect_items", rect)
            st, gk, gv = gpu_gather(case, ek, ev)
            assert st == OK
            assert np.array_equal(gk, eok), f"K out differs ({case.note}, packed_tiles {knob}, rect {rect})"
            assert np.array_equal(gv, eov), f"V out differs ({case.note}, packed_tiles {knob}, rect {rect})"


@pytest.mark.parametrize("dtype,packs", [(abi.DTYPE_BF16, (1, 2, 4, 8, 16, 32)), (abi.DTYPE_F16, (8,)),
                                         (abi.DTYPE_F32, (1, 2, 4, 8, 16))])
def test_every_pack_size(dtype, packs):
    """Units of 2 / 4 / 8 / 16 bytes (the transposing kernels) and of 32 / 64 bytes (the vector tier
    with group-wise addressing); lengths that leave partial pages; slots with holes."""
    for i, pack in enumerate(packs):
        for j, kw in enumerate([
            dict(heads=8, dim=128, block_size=16, num_blocks=64, lens=[100, 17, 256, 1, 0, 333], pad_frac=0.1, bad_blocks=3),
            dict(heads=2, dim=64, block_size=32, num_blocks=24, lens=[31, 33, 160], oob_slots=3, index_dtype=np.int64),
            dict(heads=3, dim=48, block_size=16, num_blocks=20, lens=[50, 70, 9], max_seq_len=60, slot_dtype=np.int32),
        ]):
            if kw["dim"] % pack:
                continue
            case = cases.make_case(2000 + 10 * i + j, layout=PACKED, pack=pack, dtype=dtype, **kw)
            case.note = f"pack {pack} case {j}"
            _check(case, knobs=(1, 2, 3, 0))


@pytest.mark.parametrize("dtype", [abi.DTYPE_BF16, abi.DTYPE_F16])
def test_paged_attention_cache_k_packed_v_transposed(dtype):
    """K [blocks, heads, dim / 8, block_size, 8], V [blocks, heads, dim, block_size] (pack 1)."""
    for j, kw in enumerate([
        dict(heads=8, dim=128, block_size=16, num_blocks=80, lens=[300, 77, 512, 9, 130], pad_frac=0.1),
        dict(heads=4, dim=64, block_size=32, num_blocks=20, lens=[64, 1, 200], bad_blocks=2),
        dict(heads=1, dim=256, block_size=16, num_blocks=12, lens=[16, 16, 47]),
    ]):
        case = cases.make_case(2100 + j, layout=PACKED, pack=8, v_pack=1, dtype=dtype, **kw)
        case.note = f"paged {j}"
        _check(case, knobs=(1, 0))


def test_decode_sized_batches_and_scattered_slots():
    """One token per sequence (every fragment a single slot), slots in reverse order, repeated
    windows met from two sides."""
    case = cases.make_case(2200, layout=PACKED, pack=1, dtype=abi.DTYPE_BF16, heads=4, dim=64, block_size=16,
                           num_blocks=64, lens=[33] * 20)
    rng = np.random.default_rng(5)
    order = rng.permutation(case.T)
    shuffled = cases.reorder_tokens(case, order)
    shuffled.note = "shuffled tokens"
    _check(shuffled)
    backwards = cases.reorder_tokens(case, np.arange(case.T)[::-1])
    backwards.note = "tokens backwards"
    _check(backwards)
    one = cases.reorder_tokens(case, np.array([t for t in range(case.T) if t % 33 == 32]))
    one.note = "last token of every sequence"
    _check(one)


@pytest.mark.parametrize("pad", [0.0, 0.02, 0.3])
def test_batches_large_enough_for_full_token_tiles(pad):
    """Tens of thousands of tokens, so that a CTA takes a full tile of tokens: tiles without a hole
    and tiles with holes then lie next to each other and take different routes through the write
    kernel; every token must be written by exactly one of them.  16-byte groups (both routes), the
    paged pairing and 4-byte groups (fragments that continue across tile borders)."""
    for j, kw in enumerate([dict(pack=8), dict(pack=8, v_pack=1), dict(pack=2)]):
        case = cases.make_case(2500 + j, layout=PACKED, dtype=abi.DTYPE_BF16, heads=2, dim=64, block_size=16,
                               num_blocks=1400, lens=[2000, 1999, 2001, 2500, 1500, 2000, 2040, 1960, 2000, 2000, 1000],
                               pad_frac=pad, **kw)
        case.note = f"large batch {j}, pad {pad}"
        assert case.T > 148 * 4 * 32   # CTAs take full 32-token tiles
        _check(case)
        if j == 0:  # the whole-line kernel's other shape, and without the sector prefetch of lone halves
            kvx_b200.set_option("packed_lines_variant", 1)
            kvx_b200.set_option("packed_fill_halves", 0)
            _check(case)
            kvx_b200.set_option("packed_lines_variant", 0)
            kvx_b200.set_option("packed_fill_halves", 1)


@pytest.mark.parametrize("heads", [1, 2, 4])
def test_a_shard_of_the_heads(heads):
    """One, two or four KV heads (what a rank of a head-sharded cache holds): a gather item then
    spans two, four or eight octets of a page's tokens instead of one.  Pages of 16 to 128 tokens,
    last pages that end inside an octet, inside a span and on its border; batches past the size up
    to which the gather takes another route."""
    lens = [1, 7, 8, 9, 15, 16, 17, 31, 33, 63, 64, 65, 100, 127, 128, 129, 200, 255, 300, 0, 5]
    for j, bs in enumerate([16, 32, 64, 128]):
        for dim in (64, 128):
            case = cases.make_case(2700 + 10 * j + dim // 64, layout=PACKED, pack=8, dtype=abi.DTYPE_BF16, heads=heads,
                                   dim=dim, block_size=bs, num_blocks=sum(-(-n // bs) for n in lens) + 4, lens=lens,
                                   pad_frac=0.05 + 0.1 * (j % 2), bad_blocks=2, oob_slots=j,
                                   slot_dtype=np.int32 if j % 2 else np.int64)
            case.note = f"{heads} heads, pages of {bs}, dim {dim}"
            _check(case, knobs=(1, 3))


def test_unpadded_output_from_packed_pages():
    """kvx_launch_gather_kv_varlen over packed pages: rows of a sequence start at out_indptr[s];
    sequences given fewer rows than they have tokens stop there, rows cut off the end stay unwritten."""
    for j, kw in enumerate([dict(pack=8), dict(pack=8, v_pack=1), dict(pack=1), dict(pack=4)]):
        base = cases.make_case(2600 + j, layout=PACKED, dtype=abi.DTYPE_BF16, heads=4, dim=64, block_size=16,
                               num_blocks=48, lens=[100, 17, 256, 1, 0, 90], bad_blocks=2, **kw)
        _, k, v = oracle_write(base)
        for variant in (dict(), dict(indptr_dtype=np.int64, gap=3, short=(0, 2)), dict(rows_cut=37)):
            case = cases.to_varlen(base, **variant)
            st, ek, ev = oracle_gather(case, k, v)
            assert st == OK
            for rect in (0, 1 << 40):
                kvx_b200.set_option("gather_rect_items", rect)
                st, gk, gv = gpu_gather(case, k, v)
                assert st == OK
                assert np.array_equal(gk, ek) and np.array_equal(gv, ev), (j, variant, rect)


def test_shapes_that_do_not_qualify_fall_back():
    """Group rows that are not whole 32-byte units, padded group rows, a head_dim whose rows are not
    whole vectors: still exact (other tiers)."""
    for j, kw in enumerate([
        dict(pack=1, heads=2, dim=64, block_size=8, num_blocks=16, lens=[20, 9]),        # 8 tokens x 2 bytes = 16-byte rows
        dict(pack=2, heads=2, dim=20, block_size=16, num_blocks=16, lens=[40, 9]),       # 40-byte heads
        dict(pack=4, heads=2, dim=64, block_size=5, num_blocks=16, lens=[13, 9]),
    ]):
        case = cases.make_case(2300 + j, layout=PACKED, dtype=abi.DTYPE_BF16, **kw)
        case.note = f"fallback {j}"
        _check(case)


def test_padded_strides_and_pitched_rows():
    """Group rows, heads and blocks further apart than dense (multiples of 32 bytes: the tile
    kernels; other multiples: the other tiers), and key / value rows with a token pitch."""
    for j, (pad, pack, vp) in enumerate([((32, 16, 48), 8, 0), ((16, 32, 0), 1, 0), ((64, 16, 16), 8, 1), ((3, 5, 7), 2, 0)]):
        case = cases.make_case(2400 + j, layout=PACKED, pack=pack, v_pack=vp, dtype=abi.DTYPE_BF16, heads=4, dim=64,
                               block_size=16, num_blocks=24, lens=[100, 40, 7], stride_pad=pad, pad_frac=0.05)
        case.note = f"padded strides {j}"
        _check(case)
    base = cases.make_case(2450, layout=PACKED, pack=8, v_pack=1, dtype=abi.DTYPE_BF16, heads=4, dim=64,
                           block_size=16, num_blocks=24, lens=[100, 40, 7], pad_frac=0.1)
    pitched = cases.to_pitched(base, 2 * 4 * 64, 64, seed=1)
    pitched.note = "pitched rows"
    _check(pitched)


def test_full_size_round_trip_paged_layout():
    """The Llama-3-70B shape with the paged-attention cache layout at its full token count:
    write, gather, and the benchmark's own byte check."""
    import torch
    from kvx_b200 import bench_support as bs, workloads
    for layout in ("packed", "paged"):
        dw = bs.setup_device_workload(workloads.SPECS["c4"], layers=1, layout=layout)
        stream = torch.cuda.current_stream().cuda_stream
        bs.fill_sentinel(dw)
        bs.launch_write(dw, 0, stream)
        bs.launch_gather(dw, 0, stream)
        torch.cuda.synchronize()
        res = bs.verify_layer(dw, 0)
        assert res["ok"], (layout, res)
        del dw
