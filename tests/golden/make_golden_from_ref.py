"""Generates tests/golden/ref_*.npz on a machine with a B200: for a handful of small seeded
cases, runs the REFERENCE project's own kernels (oracle/_ref/libkvx_ref.so, compiled
unmodified for sm_100a by oracle/build.py) and stores inputs plus the bytes they produced.
The CPU checker is then pinned against these files without a GPU.

    python tests/golden/make_golden_from_ref.py [output_dir]

Cases avoid block-table ids >= num_blocks: the reference reads out of bounds for those.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from kvx_b200 import abi  # noqa: E402

import cases  # noqa: E402
from harness import Case  # noqa: E402

# name -> make_case keyword arguments (seed included)
GOLDEN_CASES = {
    "nhd_bf16_pad": dict(seed=11, dtype=abi.DTYPE_BF16, num_blocks=12, block_size=16, heads=2, dim=128,
                         lens=[40, 17, 5, 1], pad_frac=0.1, slot_dtype=np.int64, index_dtype=np.int32),
    "nhd_f16_s32": dict(seed=12, dtype=abi.DTYPE_F16, num_blocks=16, block_size=16, heads=4, dim=64,
                        lens=[30, 9], pad_frac=0.2, slot_dtype=np.int32, index_dtype=np.int64),
    "nhd_f32_odd": dict(seed=13, dtype=abi.DTYPE_F32, num_blocks=8, block_size=4, heads=1, dim=7,
                        lens=[9, 4, 0, 6], oob_slots=2),
    "hnd_bf16": dict(seed=14, layout=abi.LAYOUT_HND, dtype=abi.DTYPE_BF16, num_blocks=12, block_size=8,
                     heads=4, dim=32, lens=[20, 8, 31], pad_frac=0.1),
    "packed_f16": dict(seed=15, layout=abi.LAYOUT_HND_PACKED, pack=8, dtype=abi.DTYPE_F16, num_blocks=8,
                       block_size=8, heads=2, dim=32, lens=[13, 24]),
    "nhd_bf16_short_lens": dict(seed=16, dtype=abi.DTYPE_BF16, num_blocks=10, block_size=16, heads=2, dim=64,
                                lens=[50, 70], max_seq_len=40, max_blocks=3),
}

_ARRAYS = ("key", "value", "slots", "cache_k", "cache_v", "table", "lens", "out_k", "out_v")


def case_from_npz(z) -> Case:
    geom = abi.CacheGeometry(*[int(x) for x in z["geom"]])
    return Case(geom=geom, cache_dtype=int(z["dtype"]), io_dtype=int(z["dtype"]),
                max_seq_len=int(z["max_seq_len"]), **{f: z[f] for f in _ARRAYS})


def main(out_dir: str) -> None:
    import ctypes as C

    import torch

    from harness import gpu_gather, gpu_write
    from oracle.kvx_oracle import reference

    R = reference()
    if R is None:
        raise SystemExit("oracle/_ref/libkvx_ref.so is missing: build it where the reference checkout is")
    assert torch.cuda.is_available()
    os.makedirs(out_dir, exist_ok=True)
    for name, kw in GOLDEN_CASES.items():
        kw = dict(kw)
        case = cases.make_case(kw.pop("seed"), **kw)
        st, k, v = gpu_write(case, "dispatch", L=R)
        assert st == abi.STATUS_OK, (name, st)
        st, ok_, ov_ = gpu_gather(case, k, v, "dispatch", L=R)
        assert st == abi.STATUS_OK, (name, st)
        g = case.geom
        np.savez_compressed(os.path.join(out_dir, f"ref_{name}.npz"),
                            geom=np.array([g.num_blocks, g.block_size, g.num_kv_heads, g.head_dim, g.layout, g.pack]),
                            dtype=case.io_dtype, max_seq_len=case.max_seq_len,
                            ref_cache_k=k, ref_cache_v=v, ref_out_k=ok_, ref_out_v=ov_,
                            **{f: getattr(case, f) for f in _ARRAYS})
        print("wrote", name, C.sizeof(abi.CacheDesc))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
