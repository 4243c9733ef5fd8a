"""Randomised differential test: seeded random shapes, layouts, element types, strides, index
widths, padding and damaged tables through the C-ABI launchers, every result compared byte
for byte with the CPU checker.  Complements the hand-picked cases of test_gpu_parity.py: the
draw decides which kernel tier a case lands in (vector, 256-bit, segmented, packed, generic,
fp8), so the tiers' boundaries are crossed from both sides without being named here."""
import numpy as np
import pytest

import kvx_b200
from kvx_b200 import abi

import cases
from harness import gpu_gather, gpu_write, oracle_gather, oracle_write

pytestmark = pytest.mark.gpu

OK = abi.STATUS_OK
SEEDS_PER_GROUP = 40


def _draw(seed: int) -> dict:
    rng = np.random.default_rng(1000 + seed)
    layout = int(rng.choice([abi.LAYOUT_NHD, abi.LAYOUT_HND, abi.LAYOUT_HND_PACKED]))
    dtype = int(rng.choice([abi.DTYPE_F16, abi.DTYPE_BF16, abi.DTYPE_F32]))
    elem = 4 if dtype == abi.DTYPE_F32 else 2
    dim = int(rng.choice([8, 16, 24, 64, 80, 128, 256]))
    pack = 1
    if layout == abi.LAYOUT_HND_PACKED:
        pack = int(rng.choice([p for p in (2, 4, 8, 16 // elem) if dim % p == 0]))
    block_size = int(rng.choice([1, 2, 4, 8, 16, 32]))
    heads = int(rng.choice([1, 2, 3, 4, 8]))
    seqs = int(rng.integers(1, 7))
    lens = [int(x) for x in rng.integers(0, 5 * block_size + 2, seqs)]
    if rng.random() < 0.3:
        lens[int(rng.integers(0, seqs))] = 0
    need = sum(-(-n // block_size) for n in lens)
    kw = dict(layout=layout, dtype=dtype, pack=pack, dim=dim, heads=heads, block_size=block_size, lens=lens,
              num_blocks=need + int(rng.integers(1, 6)), pad_frac=float(rng.choice([0.0, 0.1, 0.5])),
              oob_slots=int(rng.integers(0, 3)), bad_blocks=int(rng.integers(0, 3)),
              slot_dtype=rng.choice([np.int32, np.int64]), index_dtype=rng.choice([np.int32, np.int64]))
    longest = max(lens)
    if longest > 1 and rng.random() < 0.3:   # the output holds fewer tokens than the longest context
        kw["max_seq_len"] = int(rng.integers(1, longest))
    if longest > block_size and rng.random() < 0.2:   # the table is narrower than the longest context
        kw["max_blocks"] = int(rng.integers(1, -(-longest // block_size)))
    if layout != abi.LAYOUT_HND_PACKED and rng.random() < 0.4:   # padded pool strides, in elements
        unit = int(rng.choice([1, 16 // elem, 32 // elem]))
        kw["stride_pad"] = tuple(int(unit * rng.integers(0, 4)) for _ in range(3))
    return kw


@pytest.mark.parametrize("group", range(5))
def test_random_copy_cases(group):
    for i in range(SEEDS_PER_GROUP):
        seed = group * SEEDS_PER_GROUP + i
        kw = _draw(seed)
        case = cases.make_case(seed, **kw)
        case.note = f"seed {seed}: {kw}"
        st, ek, ev = oracle_write(case)
        assert st == OK, case.note
        st, k, v = gpu_write(case, "dispatch", 1)
        assert st == OK, case.note
        assert np.array_equal(k, ek) and np.array_equal(v, ev), f"cache differs, {case.note}"
        st, eok, eov = oracle_gather(case, ek, ev)
        assert st == OK, case.note
        saved = {n: kvx_b200.get_option(n) for n in ("gather_rect_items", "gather_path", "wide")}
        kvx_b200.set_option("gather_path", seed % 3)       # CTA-granular, bulk-staged, warp-granular items
        kvx_b200.set_option("wide", (seed // 3) % 2)       # 128-bit / 256-bit accesses
        try:
            for rect in (0, 1 << 40):   # compacted and uncompacted (sequence, page) rectangle
                kvx_b200.set_option("gather_rect_items", rect)
                st, gk, gv = gpu_gather(case, ek, ev, "dispatch")
                assert st == OK, case.note
                assert np.array_equal(gk, eok) and np.array_equal(gv, eov), \
                    f"gather differs (rect {rect}, path {seed % 3}, wide {(seed // 3) % 2}), {case.note}"
        finally:
            for n, v in saved.items():
                kvx_b200.set_option(n, v)


@pytest.mark.parametrize("group", range(2))
def test_random_fp8_cases(group):
    for i in range(SEEDS_PER_GROUP):
        seed = 500 + group * SEEDS_PER_GROUP + i
        rng = np.random.default_rng(seed)
        kw = _draw(seed)
        kw.update(layout=int(rng.choice([abi.LAYOUT_NHD, abi.LAYOUT_HND])), pack=1,
                  dtype=int(rng.choice([abi.DTYPE_F16, abi.DTYPE_BF16, abi.DTYPE_F32])),
                  cache_dtype=abi.DTYPE_F8_E4M3, real_values=True,
                  scale_gran=int(rng.choice([abi.SCALE_PER_TENSOR, abi.SCALE_PER_HEAD])))
        kw.pop("stride_pad", None)
        case = cases.make_case(seed, **kw)
        case.note = f"seed {seed}: {kw}"
        st, ek, ev = oracle_write(case)
        assert st == OK, case.note
        st, k, v = gpu_write(case, "dispatch", 1)
        assert st == OK, case.note
        assert np.array_equal(k, ek) and np.array_equal(v, ev), f"fp8 cache differs, {case.note}"
        st, eok, eov = oracle_gather(case, ek, ev)
        assert st == OK, case.note
        st, gk, gv = gpu_gather(case, ek, ev, "dispatch")
        assert st == OK, case.note
        assert np.array_equal(gk, eok) and np.array_equal(gv, eov), f"fp8 gather differs, {case.note}"


@pytest.mark.parametrize("group_id", range(2))
def test_random_attention_cases(group_id):
    """Decode attention over random shapes against the checker's double-precision statement
    (tolerances of tests/test_gpu_attention.py): tensor-core and generic tier, 16-bit, f32 and
    fp8 caches, 1..16 query heads per KV head, contexts from empty to several chunks, truncated
    by max_seq_len, damaged tables."""
    from test_gpu_attention import check

    for i in range(20):
        seed = 900 + group_id * 20 + i
        rng = np.random.default_rng(seed)
        dtype = int(rng.choice([abi.DTYPE_BF16, abi.DTYPE_F16, abi.DTYPE_F32]))
        fp8 = dtype != abi.DTYPE_F32 and rng.random() < 0.3
        block_size = int(rng.choice([4, 16, 32, 64]))
        heads = int(rng.choice([1, 2, 4]))
        dim = int(rng.choice([32, 64, 128, 256]))
        seqs = int(rng.integers(1, 6))
        top = int(rng.choice([40, 300, 2500]))
        lens = [int(x) for x in rng.integers(0, top + 1, seqs)]
        need = sum(-(-n // block_size) for n in lens)
        kw = dict(layout=int(rng.choice([abi.LAYOUT_NHD, abi.LAYOUT_HND])), dtype=dtype, heads=heads, dim=dim,
                  block_size=block_size, lens=lens, num_blocks=need + 3, bad_blocks=int(rng.integers(0, 3)),
                  index_dtype=rng.choice([np.int32, np.int64]), real_values=True)
        if fp8:
            kw.update(cache_dtype=abi.DTYPE_F8_E4M3,
                      scale_gran=int(rng.choice([abi.SCALE_PER_TENSOR, abi.SCALE_PER_HEAD])))
        case = cases.make_case(seed, **kw)
        q_per_kv = int(rng.choice([1, 2, 4, 7, 8, 12, 16]))
        case.note = f"seed {seed}: group {q_per_kv}, {kw}"
        _, k, v = oracle_write(case)
        extra = {}
        if max(lens) > 2 and rng.random() < 0.3:
            extra["max_seq_len"] = int(rng.integers(1, max(lens)))
        check(case, k, v, q_per_kv, seed=seed, **extra)
