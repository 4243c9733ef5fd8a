"""KV-head sharding over several ranks, on CPU with the gloo backend (world size 2): every
rank builds the same index metadata from the seed, owns its heads' slice of the batch and of
the pages, and the union of the per-rank results equals the unsharded result.  The data path
itself has no collective; gloo is used here only to bring the shards together for the check
and for the max-over-ranks reduction the benchmark does."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import dataclasses

    import torch
    import torch.distributed as dist

    from kvx_b200 import abi, workloads

    import cases
    from harness import oracle_gather, oracle_write

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        H = 8
        full = cases.make_case(4, dtype=abi.DTYPE_F16, num_blocks=32, block_size=16, heads=H, dim=32,
                               lens=[100, 48, 150], pad_frac=0.1, real_values=True)
        h0, h1 = workloads.head_range(H, rank, world)
        g = full.geom
        geom_r = abi.CacheGeometry(g.num_blocks, g.block_size, h1 - h0, g.head_dim)
        shard = dataclasses.replace(
            full, geom=geom_r, key=np.ascontiguousarray(full.key[:, h0:h1]),
            value=np.ascontiguousarray(full.value[:, h0:h1]),
            cache_k=cases.sentinel_fill(geom_r.elems, full.cache_dtype),
            cache_v=cases.sentinel_fill(geom_r.elems, full.cache_dtype),
            out_k=np.ascontiguousarray(full.out_k[:, :, h0:h1]), out_v=np.ascontiguousarray(full.out_v[:, :, h0:h1]))
        st, k, v = oracle_write(shard)
        assert st == 0
        st, ok_, ov_ = oracle_gather(shard, k, v)
        assert st == 0
        # bring the shards together: pages along the head axis, outputs along the head axis
        mine = torch.from_numpy(k.reshape(geom_r.shape).astype(np.int32))
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        pages = torch.cat(parts, dim=2).numpy().astype(np.uint16)
        mine_o = torch.from_numpy(ok_.astype(np.int32))
        parts_o = [torch.empty_like(mine_o) for _ in range(world)]
        dist.all_gather(parts_o, mine_o)
        outs = torch.cat(parts_o, dim=2).numpy().astype(np.uint16)
        # a timing-style reduction: max over ranks
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert float(t) == float(world)
        if rank == 0:
            _, fk, fv = oracle_write(full)
            _, fok, _ = oracle_gather(full, fk, fv)
            assert np.array_equal(pages.reshape(-1), fk)
            assert np.array_equal(outs, fok)
        out.put((rank, "ok"))
    except Exception as exc:  # report instead of hanging the peer
        out.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


def test_head_sharding_world_size_2():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_head_range_partitions_heads():
    from kvx_b200 import workloads
    for world in (1, 2, 4, 8):
        got = [workloads.head_range(8, r, world) for r in range(world)]
        assert got[0][0] == 0 and got[-1][1] == 8
        assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
    with pytest.raises(ValueError):
        workloads.head_range(8, 0, 3)


def test_metadata_is_identical_on_every_rank():
    """Index metadata depends on the seed only, never on the rank."""
    from kvx_b200 import workloads
    a = workloads.build_metadata(workloads.SPECS["c4"], num_blocks=40000)
    b = workloads.build_metadata(workloads.SPECS["c4"], num_blocks=40000)
    assert np.array_equal(a.slots, b.slots) and np.array_equal(a.table, b.table) and np.array_equal(a.lens, b.lens)
    assert a.write_bytes(8) == 8 * a.write_bytes(1) - 7 * a.write_tokens * 8
