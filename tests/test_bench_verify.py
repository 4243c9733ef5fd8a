"""The byte check `bench.py` runs on the buffers it timed (`bench_support.verify_layer`), on CPU
tensors: a workload whose write and gather are carried out here with plain torch indexing
through the same page views must pass, in every page layout the benchmark knows, and one
flipped bit of each kind (a written row, an untouched row, a gathered row, a row past a
sequence's end) must turn the matching flag red.  The fill pattern and the sentinel contain NaN
encodings, so the check must compare bit patterns, never floats."""
import dataclasses

import pytest
import torch

from kvx_b200 import bench_support as bs, workloads


def _workload(name: str, layout: str, heads: int = 2):
    spec = dataclasses.replace(workloads.SPECS[name], seqs=5, len_hi=300, len_lo=1 if name == "c3" else 50,
                               layers=2, pool_bytes=0)
    meta = workloads.build_metadata(spec, num_blocks=None)
    T, S, Lmax = meta.write_tokens, spec.seqs, meta.max_seq_len
    n = meta.num_blocks * spec.block_size * heads * spec.dim * 2
    g = torch.Generator().manual_seed(3)
    key = torch.randn(T, heads, spec.dim, generator=g).to(torch.bfloat16)
    value = torch.randn(T, heads, spec.dim, generator=g).to(torch.bfloat16)
    dw = bs.DeviceWorkload(meta=meta, heads=heads, layers=2, pool=torch.empty(2 * 2 * n, dtype=torch.uint8), key=key,
                           value=value, slots=torch.from_numpy(meta.slots), table=torch.from_numpy(meta.table),
                           lens=torch.from_numpy(meta.lens),
                           out_k=torch.empty(S, Lmax, heads, spec.dim, dtype=torch.bfloat16),
                           out_v=torch.empty(S, Lmax, heads, spec.dim, dtype=torch.bfloat16), layout=layout)
    bs.fill_sentinel(dw)
    return dw, n


def _write_and_gather(dw, layer: int) -> None:
    spec, meta = dw.meta.spec, dw.meta
    kp, vp = dw.layer_pages(layer)
    valid = dw.slots >= 0
    idx = dw.slots[valid]
    for pages, src in ((kp, dw.key), (vp, dw.value)):
        pages[idx // spec.block_size, idx % spec.block_size] = src[valid].reshape((-1,) + tuple(pages.shape[2:]))
    for s in range(spec.seqs):
        n = int(meta.lens[s])
        p = torch.arange(n)
        b = dw.table[s, p // spec.block_size].long()
        dw.out_k[s, :n] = kp[b, p % spec.block_size].reshape(n, dw.heads, spec.dim)
        dw.out_v[s, :n] = vp[b, p % spec.block_size].reshape(n, dw.heads, spec.dim)


@pytest.mark.parametrize("layout", ["nhd", "hnd", "packed", "paged"])
@pytest.mark.parametrize("name", ["c2", "c3"])
def test_verify_layer_accepts_good_buffers_and_sees_every_kind_of_damage(name, layout):
    dw, n = _workload(name, layout)
    _write_and_gather(dw, 1)
    assert bs.verify_layer(dw, 1)["ok"]
    spec = dw.meta.spec
    kp, vp = dw.layer_pages(1)
    slot = int(dw.slots[dw.slots >= 0][0])

    def flipped(tensor, index, flag):
        raw = tensor[index].clone()
        tensor[index] = (raw.view(torch.int16) ^ 1).view(torch.bfloat16)
        res = bs.verify_layer(dw, 1)
        tensor[index] = raw
        assert not res[flag] and not res["ok"], (flag, res)

    flipped(kp, (slot // spec.block_size, slot % spec.block_size, 0, 0), "write_rows")
    used = set((dw.slots[dw.slots >= 0]).tolist())
    free = next(r for r in range(dw.meta.num_blocks * spec.block_size) if r not in used)
    flipped(vp, (free // spec.block_size, free % spec.block_size, 1, 1), "untouched_pages")
    flipped(dw.out_v, (1, 0, 0, 3), "gather_live")
    short = int(dw.lens.argmin())
    if int(dw.lens[short]) < dw.meta.max_seq_len:
        flipped(dw.out_k, (short, dw.meta.max_seq_len - 1, 1, 0), "gather_dead")
    assert bs.verify_layer(dw, 1)["ok"]
    # the other layer was never written: its rows all hold the pattern, so a "written" check fails there
    assert not bs.verify_layer(dw, 0)["write_rows"]


def test_fill_pattern_is_position_dependent():
    dw, n = _workload("c2", "nhd")
    words = dw.pool.view(torch.int64)
    assert torch.equal(words, torch.arange(words.numel(), dtype=torch.int64))
    assert bool((dw.out_k.view(torch.uint8) == bs.SENTINEL).all())
