"""The word a kernel sets when it abandons a bounded wait, and how the host learns of it.

The only kernels of the library that wait on anything are those of the bulk-async gather path
(tuning knob gather_path = 1): every wait on a staged copy has a time limit, after which the
waiting thread sets a word in device memory, lets its copies in flight finish and returns.
The test makes one wait run out in the harmless form: a test knob lets the first pipe of the
grid wait -- before it has issued any copy -- on a barrier that no copy will ever complete,
with the limit cut to a millisecond.  Nothing is in flight when that thread gives up, the other
pipes do their work as usual, the kernel ends normally and the context stays usable."""
import ctypes as C

import numpy as np
import pytest

from kvx_b200 import abi

import cases
from harness import descriptors, device_buffers, gpu_gather, host_buffers, oracle_gather, oracle_write

pytestmark = pytest.mark.gpu
OK = abi.STATUS_OK


@pytest.fixture
def stalled_bulk_path():
    import kvx_b200
    kvx_b200.lib().kvx_b200_device_error(1)
    saved = {k: kvx_b200.get_option(k) for k in ("gather_path", "bulk_test_stall", "bulk_wait_us")}
    kvx_b200.set_option("gather_path", 1)
    kvx_b200.set_option("bulk_test_stall", 1)
    kvx_b200.set_option("bulk_wait_us", 1000)
    yield
    for k, v in saved.items():
        kvx_b200.set_option(k, v)
    kvx_b200.lib().kvx_b200_device_error(1)


def _case():
    return cases.make_case(4100, dtype=abi.DTYPE_BF16, heads=8, dim=128, block_size=16, num_blocks=64,
                           lens=[200, 33, 150, 16])


def test_no_error_after_ordinary_launches():
    import kvx_b200
    L = kvx_b200.lib()
    case = _case()
    _, k, v = oracle_write(case)
    _, ek, ev = oracle_gather(case, k, v)
    saved = kvx_b200.get_option("gather_path")
    try:
        for path in (2, 1):  # the default path, then the bulk path with its usual one-second limit
            kvx_b200.set_option("gather_path", path)
            st, gk, gv = gpu_gather(case, k, v)
            assert st == OK and np.array_equal(gk, ek) and np.array_equal(gv, ev)
            assert L.kvx_b200_device_error(0) == 0
    finally:
        kvx_b200.set_option("gather_path", saved)


def test_abandoned_wait_sets_the_word_and_the_next_launch_works(stalled_bulk_path):
    import kvx_b200
    L = kvx_b200.lib()
    case = _case()
    _, k, v = oracle_write(case)
    _, ek, ev = oracle_gather(case, k, v)
    st, gk, gv = gpu_gather(case, k, v)          # synchronises the device before returning
    assert st == OK                               # the launcher cannot know: it returned long before
    assert L.kvx_b200_device_error(0) == 1        # read without clearing
    assert L.kvx_b200_device_error(1) == 1        # read and clear
    assert L.kvx_b200_device_error(0) == 0
    # rows the stalled pipe did not reach were left as they were; nothing else is wrong
    wrong_k = np.any(gk != ek, axis=(2, 3))
    assert np.all((gk == ek) | (gk == case.out_k))
    assert wrong_k.sum() < wrong_k.size
    # the context is intact: the same gather without the stall is bit-exact again
    kvx_b200.set_option("bulk_test_stall", 0)
    st, gk, gv = gpu_gather(case, k, v)
    assert st == OK and np.array_equal(gk, ek) and np.array_equal(gv, ev)
    assert L.kvx_b200_device_error(0) == 0


def test_host_pipeline_reports_the_abandoned_wait(stalled_bulk_path):
    import torch
    import kvx_b200
    L = kvx_b200.lib()
    case = _case()
    _, k, v = oracle_write(case)
    hb = host_buffers(case)
    dev_k = torch.from_numpy(k.view(np.uint8).copy()).cuda()
    dev_v = torch.from_numpy(v.view(np.uint8).copy()).cuda()
    cache, _, gather, ks, vs = descriptors(case, dict(hb, cache_k=dev_k, cache_v=dev_v), abi.MEMORY_HOST)
    cache.k.memory = cache.v.memory = abi.MEMORY_DEVICE
    pipe = C.c_void_p()
    S, mb = case.table.shape
    assert L.kvx_host_pipe_create(1 << 22, S, mb, C.byref(pipe)) == OK
    try:
        assert L.kvx_host_gather_kv(pipe, C.byref(cache), C.byref(gather), C.byref(ks), C.byref(vs)) == OK
        assert L.kvx_host_pipe_sync(pipe) == abi.STATUS_INTERNAL_ERROR
        assert L.kvx_b200_device_error(0) == 0    # the sync has cleared the word
        kvx_b200.set_option("bulk_test_stall", 0)
        assert L.kvx_host_gather_kv(pipe, C.byref(cache), C.byref(gather), C.byref(ks), C.byref(vs)) == OK
        assert L.kvx_host_pipe_sync(pipe) == OK
    finally:
        L.kvx_host_pipe_destroy(pipe)
    _, ek, ev = oracle_gather(case, k, v)
    assert np.array_equal(hb["out_k"], ek) and np.array_equal(hb["out_v"], ev)
