"""The synthetic-workload generators behind bench.py (slot mappings, block tables, lengths):
the counterpart of the reference's CPU test of its slot-mapping builder
(benchmarks/tests/fair_bench_slot_mapping_test.py), for the five benchmark configurations."""
import numpy as np
import pytest

from kvx_b200 import workloads


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4", "c5"])
def test_metadata_is_consistent(name):
    spec = workloads.SPECS[name]
    nb = None if spec.fixed_blocks else 3 * int(spec.seqs * (spec.len_hi // spec.block_size + 1))
    m = workloads.build_metadata(spec, num_blocks=nb)
    bs = spec.block_size
    assert m.lens.shape == (spec.seqs,) and m.lens.min() >= spec.len_lo and m.lens.max() <= spec.len_hi
    need = (m.lens.astype(np.int64) + bs - 1) // bs
    assert m.gather_pages == int(need.sum()) and m.gather_tokens == int(m.lens.sum())
    assert m.table.shape == (spec.seqs, int(need.max())) and m.max_seq_len == int(m.lens.max())
    # every sequence owns its own pages: used entries are distinct and inside the pool, the rest is -1
    used = m.table[m.table >= 0]
    assert used.size == m.gather_pages and np.unique(used).size == used.size and used.max() < m.num_blocks
    for s in range(spec.seqs):
        assert (m.table[s, : need[s]] >= 0).all() and (m.table[s, need[s]:] == -1).all()
    # slot = page * block_size + offset of the token's position, sequence-major; -1 = padding
    valid = m.slots >= 0
    assert m.valid_tokens == int(valid.sum()) and m.write_tokens == m.slots.shape[0]
    assert np.unique(m.slots[valid]).size == m.valid_tokens
    if spec.decode:
        assert m.write_tokens == spec.seqs
        pos = m.lens.astype(np.int64) - 1
        expect = m.table[np.arange(spec.seqs), pos // bs].astype(np.int64) * bs + pos % bs
    else:
        assert m.write_tokens == m.gather_tokens
        seq_of = np.repeat(np.arange(spec.seqs), m.lens)
        pos = np.concatenate([np.arange(n) for n in m.lens])
        expect = m.table[seq_of, pos // bs].astype(np.int64) * bs + pos % bs
    assert np.array_equal(m.slots[valid], expect[valid])
    if spec.pad_frac > 0:
        assert abs((~valid).mean() - spec.pad_frac) < 0.01
    else:
        assert valid.all()


def test_stated_sizes_of_the_configurations():
    c1 = workloads.build_metadata(workloads.SPECS["c1"])
    assert c1.num_blocks == 512 and c1.write_tokens == 1024 and (c1.lens == 128).all()
    c2 = workloads.SPECS["c2"]
    # 150 GB of K+V pages over 32 layers of 32 KiB pages
    assert workloads.build_metadata(c2).num_blocks == int(150e9 // (2 * 32 * 16 * 8 * 128 * 2)) == 71525
    c3 = workloads.build_metadata(workloads.SPECS["c3"], num_blocks=60000)
    assert c3.lens.min() >= 1 and c3.lens.max() <= 32768 and np.median(c3.lens) < 1000   # log-uniform
    c4 = workloads.build_metadata(workloads.SPECS["c4"], num_blocks=40000)
    assert c4.write_tokens == 32 * 8192 and c4.valid_tokens == c4.write_tokens


def test_algorithmic_byte_formulas():
    """write: 2 Tv (row_in + row_cache) + 8 T;  gather: 2 sum(len) (row_cache + row_out) + 4 pages + 4 S."""
    m = workloads.build_metadata(workloads.SPECS["c2"])
    row = 8 * 128 * 2
    assert m.write_bytes(8) == 2 * m.valid_tokens * 2 * row + 8 * m.write_tokens
    assert m.gather_bytes(8) == 2 * m.gather_tokens * 2 * row + 4 * m.gather_pages + 4 * 64
    assert m.write_bytes(1) * 8 - 7 * 8 * m.write_tokens == m.write_bytes(8)       # head shards add up
    f8 = workloads.build_metadata(workloads.SPECS["c5"], num_blocks=20000)
    assert f8.write_bytes(16) == 2 * f8.valid_tokens * (16 * 256 * 2 + 16 * 256) + 8 * f8.write_tokens


def test_seeds_are_reproducible_and_distinct():
    a = workloads.build_metadata(workloads.SPECS["c2"], num_blocks=20000)
    b = workloads.build_metadata(workloads.SPECS["c2"], num_blocks=20000)
    c = workloads.build_metadata(workloads.SPECS["c2"], num_blocks=20000, seed=5)
    assert np.array_equal(a.slots, b.slots) and np.array_equal(a.table, b.table)
    assert not np.array_equal(a.lens, c.lens)


def test_reference_arm_prints_the_gpu_arms_config():
    """`bench.py --impl reference` must describe the same workload as the other arm: the full
    configuration at its stated pool size, whatever bounded sample of it a CPU step runs."""
    import argparse
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    from kvx_b200 import workloads
    c = bench.reference_config(workloads.SPECS["c2"], argparse.Namespace(gpus=1, layers=None, pool_gb=None, layout="nhd"))
    assert (c["workload"], c["layers"], c["heads_per_gpu"], c["pool_blocks_per_tensor"], c["pool_gb_per_gpu"]) == \
        ("c2_llama3_8b_prefill", 32, 8, 71525, 150.0)
    assert (c["write_tokens"], c["valid_tokens"], c["gather_tokens"]) == (142060, 127653, 142060)
    c8 = bench.reference_config(workloads.SPECS["c2"], argparse.Namespace(gpus=8, layers=None, pool_gb=None, layout="nhd"))
    assert (c8["heads_per_gpu"], c8["pool_gb_per_gpu"], c8["parallelism"]) == (1, 18.75, "kv_head_shard8")
    assert set(c) == set(c8)
