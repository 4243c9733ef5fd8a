"""Host-buffer pipeline (kvx_host_write_kv / kvx_host_gather_kv): K/V, slots, block table,
lengths and outputs in host memory, pages on the device.  Results must equal the CPU checker's
byte for byte, including host output bytes the gather must leave untouched, with chunks small
enough that every call is split into several staged pieces."""
import ctypes as C

import numpy as np
import pytest

from kvx_b200 import abi

import cases
from harness import descriptors, host_buffers, oracle_gather, oracle_write

pytestmark = pytest.mark.gpu
OK = abi.STATUS_OK


def _run(case, chunk_bytes, device_scales=None, adjacent_outputs=False):
    import torch
    import kvx_b200
    L = kvx_b200.lib()
    hb = host_buffers(case)                      # numpy host buffers (inputs and outputs)
    if adjacent_outputs:                         # V output right behind the K output, in one array
        both = np.stack([hb["out_k"], hb["out_v"]])
        hb["out_k"], hb["out_v"] = both[0], both[1]
    if device_scales is not None:                # quantisation scales are read by the kernels
        hb["k_scale"], hb["v_scale"] = device_scales
    dev_k = torch.from_numpy(case.cache_k.view(np.uint8).copy()).cuda()
    dev_v = torch.from_numpy(case.cache_v.view(np.uint8).copy()).cuda()
    bufs = dict(hb, cache_k=dev_k, cache_v=dev_v)
    cache, write, gather, ks, vs = descriptors(case, bufs, abi.MEMORY_HOST)
    cache.k.memory = cache.v.memory = abi.MEMORY_DEVICE
    pipe = C.c_void_p()
    S, mb = case.table.shape
    assert L.kvx_host_pipe_create(chunk_bytes, S, mb, C.byref(pipe)) == OK
    try:
        assert L.kvx_host_write_kv(pipe, C.byref(cache), C.byref(write)) == OK
        assert L.kvx_host_gather_kv(pipe, C.byref(cache), C.byref(gather), C.byref(ks), C.byref(vs)) == OK
        assert L.kvx_host_pipe_sync(pipe) == OK
        h2d, d2h = C.c_uint64(), C.c_uint64()
        L.kvx_host_pipe_traffic(pipe, C.byref(h2d), C.byref(d2h))
        # a second round on the same pipe (staging sets are reused)
        assert L.kvx_host_write_kv(pipe, C.byref(cache), C.byref(write)) == OK
        assert L.kvx_host_gather_kv(pipe, C.byref(cache), C.byref(gather), C.byref(ks), C.byref(vs)) == OK
        assert L.kvx_host_pipe_sync(pipe) == OK
    finally:
        L.kvx_host_pipe_destroy(pipe)
    pages_k = dev_k.cpu().numpy().view(case.cache_k.dtype)
    pages_v = dev_v.cpu().numpy().view(case.cache_v.dtype)
    return pages_k, pages_v, hb["out_k"], hb["out_v"], h2d.value, d2h.value


@pytest.mark.parametrize("dtype", [abi.DTYPE_BF16, abi.DTYPE_F32])
def test_host_pipeline_matches_checker(dtype):
    for i, kw in enumerate([
        dict(heads=8, dim=128, block_size=16, num_blocks=80, lens=[300, 77, 512, 9, 0, 130], pad_frac=0.1, bad_blocks=3),
        dict(heads=2, dim=64, block_size=8, num_blocks=64, lens=[50, 70, 33], max_seq_len=40, max_blocks=6,
             slot_dtype=np.int32, index_dtype=np.int64, oob_slots=3),
    ]):
        case = cases.make_case(900 + i, dtype=dtype, **kw)
        _, ek, ev = oracle_write(case)
        _, eok, eov = oracle_gather(case, ek, ev)
        row = case.geom.num_kv_heads * case.geom.head_dim * case.key.dtype.itemsize
        seq_bytes = case.max_seq_len * row
        # one chunk holds a single sequence (and a fraction of the write batch)
        k, v, ok_, ov_, h2d, d2h = _run(case, max(seq_bytes, 4096))
        assert np.array_equal(k, ek) and np.array_equal(v, ev), f"pages differ (case {i})"
        assert np.array_equal(ok_, eok) and np.array_equal(ov_, eov), f"host outputs differ (case {i})"
        assert h2d >= 2 * case.T * row and d2h > 0


def test_host_pipeline_pairs_the_k_and_v_runs_of_a_sequence():
    """Where the V output lies a fixed distance behind the K output (one array for both), a
    sequence's K run and V run go back as the two rows of one 2-D copy; same bytes as with two
    copies (the knob) and as the checker's, untouched rows included; damaged table entries cut
    the runs."""
    import kvx_b200
    case = cases.make_case(950, dtype=abi.DTYPE_BF16, heads=8, dim=128, block_size=16, num_blocks=120,
                           lens=[300, 77, 512, 9, 0, 130, 511], pad_frac=0.1, bad_blocks=4)
    _, ek, ev = oracle_write(case)
    _, eok, eov = oracle_gather(case, ek, ev)
    row = case.geom.num_kv_heads * case.geom.head_dim * case.key.dtype.itemsize
    saved = kvx_b200.get_option("host_pair_kv")
    try:
        for pair in (1, 0):
            kvx_b200.set_option("host_pair_kv", pair)
            k, v, ok_, ov_, _, d2h = _run(case, 3 * case.max_seq_len * row, adjacent_outputs=True)
            assert np.array_equal(k, ek) and np.array_equal(v, ev)
            assert np.array_equal(ok_, eok) and np.array_equal(ov_, eov), f"host outputs differ (paired copies {pair})"
            assert d2h > 0
    finally:
        kvx_b200.set_option("host_pair_kv", saved)


def test_host_pipeline_fp8():
    import torch
    case = cases.make_case(950, dtype=abi.DTYPE_BF16, cache_dtype=abi.DTYPE_F8_E4M3, real_values=True, heads=4,
                           dim=64, block_size=16, num_blocks=24, lens=[100, 40, 7], scale_gran=abi.SCALE_PER_HEAD)
    _, ek, ev = oracle_write(case)
    _, eok, eov = oracle_gather(case, ek, ev)
    scales = (torch.from_numpy(case.k_scale).cuda(), torch.from_numpy(case.v_scale).cuda())
    k, v, ok_, ov_, _, _ = _run(case, 1 << 16, device_scales=scales)
    assert np.array_equal(k, ek) and np.array_equal(v, ev)
    assert np.array_equal(ok_, eok) and np.array_equal(ov_, eov)


def test_host_pipeline_takes_pitched_host_rows():
    """key / value in host memory whose token rows are further apart than heads * dim (slices of
    a fused projection output): the rows are copied with a pitched copy and staged densely, so
    the result equals the checker's on the same pitched descriptors; a row that is not dense
    inside is refused before anything is staged."""
    import kvx_b200
    L = kvx_b200.lib()
    base = cases.make_case(960, dtype=abi.DTYPE_BF16, heads=4, dim=64, block_size=16, num_blocks=40,
                           lens=[120, 9, 77], pad_frac=0.1)
    case = cases.to_pitched(base, 2 * 4 * 64, 24, seed=3)   # K rows 3x as far apart, V rows oddly so
    _, ek, ev = oracle_write(case)
    _, eok, eov = oracle_gather(case, ek, ev)
    k, v, ok_, ov_, h2d, _ = _run(case, 1 << 16)   # a chunk holds one padded sequence
    assert np.array_equal(k, ek) and np.array_equal(v, ev)
    assert np.array_equal(ok_, eok) and np.array_equal(ov_, eov)
    assert h2d < 2 * case.T * (3 * 4 * 64 * 2)              # only the rows themselves crossed the bus

    import torch
    hb = host_buffers(case)
    dev = torch.zeros(case.cache_k.nbytes, dtype=torch.uint8, device="cuda")
    cache, write, _, _, _ = descriptors(case, dict(hb, cache_k=dev, cache_v=dev), abi.MEMORY_HOST)
    cache.k.memory = cache.v.memory = abi.MEMORY_DEVICE
    write.io.key.stride[1] = 2 * 64                          # heads no longer adjacent inside a row
    pipe = C.c_void_p()
    assert L.kvx_host_pipe_create(1 << 16, 3, case.table.shape[1], C.byref(pipe)) == OK
    try:
        assert L.kvx_host_write_kv(pipe, C.byref(cache), C.byref(write)) == abi.STATUS_UNSUPPORTED
        assert L.kvx_host_pipe_sync(pipe) == OK
    finally:
        L.kvx_host_pipe_destroy(pipe)
    assert int(dev.max()) == 0
