"""The allocation-free scale reduction, kvx_launch_kv_scales_static.

Some users of this library cannot give it device scratch: an engine that handed all free HBM
to its page pool when it started, or one that bans driver allocations while serving because
they stall the whole GPU.  For them the reduction's scratch is a fixed array inside the
library.  This file checks, through the C ABI, that the variant returns exactly what the
workspace-taking entry point returns -- on two calls in a row, since the second call finds
the array as the first one left it -- that the calls leave the device's free memory as they
found it (the property the variant exists for), that a call rejected for its arguments does
not disturb the shared array, and that head counts beyond the fixed size are refused.

Collected last on purpose (file name), so a run that stops at the first failure has already
run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from kvx_b200 import abi

from harness import f32_to_bits

pytestmark = pytest.mark.gpu

MAX_HEADS = 1024  # KVX_KV_SCALES_STATIC_MAX_HEADS in include/kvx_paged_kv.h


def _device_io(T, H, D, io, seed):
    import torch
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((T, H, D)).astype(np.float32)
    x[rng.random(x.shape) < 0.001] *= 50
    y = rng.standard_normal((T, H, D)).astype(np.float32) * 0.02
    dk = torch.from_numpy(f32_to_bits(x, io).view(np.uint8).reshape(-1)).cuda()
    dv = torch.from_numpy(f32_to_bits(y, io).view(np.uint8).reshape(-1)).cuda()
    desc = abi.write_desc(T, H, D, io, dk.data_ptr(), dv.data_ptr(), abi.DTYPE_S64, 0).io
    return desc, (dk, dv)


@pytest.mark.parametrize("io", [abi.DTYPE_BF16, abi.DTYPE_F16, abi.DTYPE_F32])
def test_static_scratch_variant_matches_workspace_variant(io):
    import torch
    import kvx_b200
    L = kvx_b200.lib()
    # different head counts back to back: each call must clear what the previous one used
    for call, (T, H, D, gran) in enumerate([(3000, 16, 256, abi.SCALE_PER_HEAD), (777, 4, 64, abi.SCALE_PER_HEAD),
                                            (1500, 32, 128, abi.SCALE_PER_TENSOR), (64, MAX_HEADS, 8, abi.SCALE_PER_HEAD)]):
        desc, keep = _device_io(T, H, D, io, 100 + call)
        n = H if gran == abi.SCALE_PER_HEAD else 1
        ws = torch.zeros(L.kvx_kv_scales_workspace_bytes(H), dtype=torch.uint8, device="cuda")
        want_k = torch.empty(n, dtype=torch.float32, device="cuda")
        want_v = torch.empty(n, dtype=torch.float32, device="cuda")
        st = L.kvx_launch_kv_scales(C.byref(desc), gran, want_k.data_ptr(), want_v.data_ptr(), ws.data_ptr(),
                                    ws.numel(), None)
        assert st == abi.STATUS_OK
        for repeat in range(2):  # two calls in a row on the shared array
            got_k = torch.full((n,), -1.0, dtype=torch.float32, device="cuda")
            got_v = torch.full((n,), -1.0, dtype=torch.float32, device="cuda")
            st = L.kvx_launch_kv_scales_static(C.byref(desc), gran, got_k.data_ptr(), got_v.data_ptr(), None)
            assert st == abi.STATUS_OK, (call, repeat, st)
            torch.cuda.synchronize()
            # same tolerance as the other parity tests: none (bit-for-bit)
            assert torch.equal(got_k.view(torch.int32), want_k.view(torch.int32)), (call, repeat)
            assert torch.equal(got_v.view(torch.int32), want_v.view(torch.int32)), (call, repeat)
        del keep


def test_static_scratch_variant_allocates_no_device_memory():
    """Free device memory, as the driver reports it, is the same before and after a series of
    calls (taken after one warm-up call, so that the one-time module and address look-up of the
    very first call on a device is not counted).  The buffers of the test are made beforehand."""
    import torch
    import kvx_b200
    L = kvx_b200.lib()
    desc, keep = _device_io(2048, 8, 128, abi.DTYPE_BF16, 31)
    big, keep2 = _device_io(512, MAX_HEADS, 8, abi.DTYPE_BF16, 32)
    out_k = torch.empty(MAX_HEADS, dtype=torch.float32, device="cuda")
    out_v = torch.empty(MAX_HEADS, dtype=torch.float32, device="cuda")
    assert L.kvx_launch_kv_scales_static(C.byref(desc), abi.SCALE_PER_HEAD, out_k.data_ptr(), out_v.data_ptr(),
                                         None) == abi.STATUS_OK
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for d in (desc, big, desc, big):
        for gran in (abi.SCALE_PER_HEAD, abi.SCALE_PER_TENSOR):
            assert L.kvx_launch_kv_scales_static(C.byref(d), gran, out_k.data_ptr(), out_v.data_ptr(),
                                                 None) == abi.STATUS_OK
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    del keep, keep2


def test_rejected_call_leaves_the_shared_array_alone():
    """A call that fails its argument checks must enqueue nothing: not the kernel and not the
    clearing of the shared array either, which an earlier call may still be using.  Seen from
    outside: the rejected call launches nothing, and the next good call is still right."""
    import torch
    import kvx_b200
    L = kvx_b200.lib()
    desc, keep = _device_io(999, 8, 128, abi.DTYPE_BF16, 41)
    n = 8
    ws = torch.zeros(L.kvx_kv_scales_workspace_bytes(n), dtype=torch.uint8, device="cuda")
    want_k = torch.empty(n, dtype=torch.float32, device="cuda")
    want_v = torch.empty(n, dtype=torch.float32, device="cuda")
    assert L.kvx_launch_kv_scales(C.byref(desc), abi.SCALE_PER_HEAD, want_k.data_ptr(), want_v.data_ptr(),
                                  ws.data_ptr(), ws.numel(), None) == abi.STATUS_OK
    got_k = torch.full((n,), -1.0, dtype=torch.float32, device="cuda")
    got_v = torch.full((n,), -1.0, dtype=torch.float32, device="cuda")
    before = L.kvx_b200_launch_count()
    assert L.kvx_launch_kv_scales_static(C.byref(desc), abi.SCALE_PER_HEAD, None, got_v.data_ptr(),
                                         None) == abi.STATUS_INVALID_ARGUMENT
    assert L.kvx_launch_kv_scales_static(C.byref(desc), 77, got_k.data_ptr(), got_v.data_ptr(),
                                         None) == abi.STATUS_UNSUPPORTED
    assert L.kvx_b200_launch_count() == before
    torch.cuda.synchronize()
    assert float(got_v.max()) == -1.0
    assert L.kvx_launch_kv_scales_static(C.byref(desc), abi.SCALE_PER_HEAD, got_k.data_ptr(), got_v.data_ptr(),
                                         None) == abi.STATUS_OK
    torch.cuda.synchronize()
    assert torch.equal(got_k.view(torch.int32), want_k.view(torch.int32))
    assert torch.equal(got_v.view(torch.int32), want_v.view(torch.int32))
    del keep


def test_static_scratch_variant_rejects_too_many_heads():
    import torch
    import kvx_b200
    L = kvx_b200.lib()
    desc, keep = _device_io(4, MAX_HEADS + 1, 8, abi.DTYPE_BF16, 5)
    out = torch.zeros(MAX_HEADS + 1, dtype=torch.float32, device="cuda")
    st = L.kvx_launch_kv_scales_static(C.byref(desc), abi.SCALE_PER_HEAD, out.data_ptr(), out.data_ptr(), None)
    assert st == abi.STATUS_OUT_OF_RANGE
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0  # nothing was launched
    del keep
