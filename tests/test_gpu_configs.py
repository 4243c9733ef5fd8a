"""GPU parity on the benchmark configurations' shapes (scaled to what the CPU checker
finishes in seconds), against the reference project's own kernels where its library is
available, the fp8-e4m3 variant, and size-independent properties at larger sizes."""
import ctypes as C
import os

import numpy as np
import pytest

import kvx_b200
from kvx_b200 import abi

import cases
from harness import (bits_to_f32, device_buffers, descriptors, f32_to_bits, gpu_gather, gpu_write, back,
                     oracle_gather, oracle_write)
from test_gpu_parity import check_gather, check_write

pytestmark = pytest.mark.gpu
OK = abi.STATUS_OK


# ------------------------------------------------------------------ config shapes --------

def test_config1_tinyllama_round_trip():
    """fp16, 4 heads x 64, block 16, 8 sequences x 128 tokens, 512-block pool, seeded page
    permutation: write everything, gather back, identity."""
    case = cases.make_case(1, dtype=abi.DTYPE_F16, num_blocks=512, block_size=16, heads=4, dim=64,
                           lens=[128] * 8, real_values=True)
    k, v = check_write(case)
    check_write(case, "prefill", 128)
    check_gather(case, k, v)
    st, gk, gv = gpu_gather(case, k, v)
    assert np.array_equal(gk.reshape(case.key.shape), case.key)
    assert np.array_equal(gv.reshape(case.value.shape), case.value)


def test_config2_llama3_8b_shape():
    """bf16, 8 heads x 128, block 16, ragged lengths, ~10 % of slots = -1."""
    rng = np.random.default_rng(2)
    lens = [int(x) for x in rng.integers(64, 513, size=12)]
    case = cases.make_case(2, dtype=abi.DTYPE_BF16, num_blocks=600, block_size=16, heads=8, dim=128,
                           lens=lens, pad_frac=0.10, slot_dtype=np.int64, index_dtype=np.int32)
    k, v = check_write(case)
    check_write(case, "prefill", 1)
    check_gather(case, k, v)


def test_config3_decode_shape():
    """bf16, block 32: one new token per sequence at position ctx-1 (log-uniform contexts),
    then the full-context gather, 1..many pages per sequence."""
    rng = np.random.default_rng(3)
    ctx = np.maximum(1, np.rint(np.exp(rng.random(48) * np.log(2048))).astype(int))
    full = cases.make_case(3, dtype=abi.DTYPE_BF16, num_blocks=int(sum(-(-c // 32) for c in ctx)) + 8,
                           block_size=32, heads=8, dim=128, lens=ctx.tolist())
    # decode write: keep only each sequence's last token
    last = np.cumsum(ctx) - 1
    import dataclasses
    dec = dataclasses.replace(full, key=full.key[last].copy(), value=full.value[last].copy(),
                              slots=full.slots[last].copy())
    check_write(dec)
    _, k, v = oracle_write(full)
    check_gather(full, k, v)


@pytest.mark.parametrize("shards", [1, 2, 4, 8])
def test_config4_head_sharded_shapes(shards):
    """fp16, 8 heads x 128 split over `shards` devices: each owns 8/shards heads' pages and
    its dense [T, 8/shards, 128] slice; slots / table / lens are replicated.  All shards run
    here one after the other; their union must equal the unsharded result."""
    H = 8
    case = cases.make_case(4, dtype=abi.DTYPE_F16, num_blocks=64, block_size=16, heads=H, dim=128,
                           lens=[200, 96, 300], real_values=True)
    _, ek, ev = oracle_write(case)
    _, eok, eov = oracle_gather(case, ek, ev)
    g = case.geom
    ek4 = ek.reshape(g.shape)
    hs = H // shards
    import dataclasses
    for r in range(shards):
        sl = slice(r * hs, (r + 1) * hs)
        geom_r = abi.CacheGeometry(g.num_blocks, g.block_size, hs, g.head_dim)
        sub = dataclasses.replace(case, geom=geom_r, key=np.ascontiguousarray(case.key[:, sl]),
                                  value=np.ascontiguousarray(case.value[:, sl]),
                                  cache_k=cases.sentinel_fill(geom_r.elems, case.cache_dtype),
                                  cache_v=cases.sentinel_fill(geom_r.elems, case.cache_dtype),
                                  out_k=np.ascontiguousarray(case.out_k[:, :, sl]),
                                  out_v=np.ascontiguousarray(case.out_v[:, :, sl]))
        st, k, v = gpu_write(sub)
        assert st == OK
        assert np.array_equal(k.reshape(geom_r.shape), ek4[:, :, sl])
        st, gk, gv = gpu_gather(sub, k, v)
        assert st == OK
        assert np.array_equal(gk, eok[:, :, sl]) and np.array_equal(gv, eov[:, :, sl])


# ------------------------------------------------------------------ vs the reference ------

def _reference_lib():
    from oracle.kvx_oracle import reference
    return reference()


@pytest.mark.parametrize("dtype", [abi.DTYPE_F32, abi.DTYPE_F16, abi.DTYPE_BF16])
def test_bit_exact_against_reference_kernels(dtype):
    """Same inputs through the reference project's own kernels (compiled unmodified for
    sm_100a) and through this library: identical bytes.  No block id >= num_blocks here
    (the reference reads out of bounds for those)."""
    R = _reference_lib()
    if R is None:
        pytest.skip("oracle/_ref/libkvx_ref.so not present")
    for i, kw in enumerate([
        dict(heads=8, dim=128, block_size=16, num_blocks=80, lens=[300, 77, 512, 9], pad_frac=0.1),
        dict(heads=4, dim=64, block_size=16, num_blocks=64, lens=[128] * 4, slot_dtype=np.int32, index_dtype=np.int64),
        dict(heads=1, dim=7, block_size=4, num_blocks=16, lens=[9, 4, 0, 6], oob_slots=2),
        dict(layout=abi.LAYOUT_HND, heads=4, dim=32, block_size=8, num_blocks=12, lens=[20, 8, 31], pad_frac=0.1),
        dict(layout=abi.LAYOUT_HND_PACKED, pack=8, heads=2, dim=32, block_size=8, num_blocks=8, lens=[13, 24]),
    ]):
        case = cases.make_case(600 + i, dtype=dtype, **kw)
        st, rk, rv = gpu_write(case, "dispatch", L=R)
        assert st == OK
        st, k, v = gpu_write(case, "dispatch")
        assert st == OK
        assert np.array_equal(k, rk) and np.array_equal(v, rv), f"write case {i}"
        if kw.get("heads") != 1:
            st, pk, _ = gpu_write(case, "prefill", 1, L=R)
            assert st == OK and np.array_equal(pk, rk)
        st, rok, rov = gpu_gather(case, rk, rv, L=R)
        assert st == OK
        st, gk, gv = gpu_gather(case, rk, rv)
        assert st == OK
        assert np.array_equal(gk, rok) and np.array_equal(gv, rov), f"gather case {i}"


# ------------------------------------------------------------------ fp8 e4m3 --------------

@pytest.mark.parametrize("io", [abi.DTYPE_BF16, abi.DTYPE_F16, abi.DTYPE_F32])
@pytest.mark.parametrize("layout,pack", [(abi.LAYOUT_NHD, 1), (abi.LAYOUT_HND, 1), (abi.LAYOUT_HND_PACKED, 4)])
def test_fp8_write_and_gather(io, layout, pack):
    for i, kw in enumerate([
        dict(heads=16, dim=256, block_size=64, num_blocks=6, lens=[100, 130, 7], scale_gran=abi.SCALE_PER_HEAD, pad_frac=0.1),
        dict(heads=3, dim=16, block_size=4, num_blocks=12, lens=[9, 5, 20], scale_gran=abi.SCALE_PER_TENSOR),
        dict(heads=2, dim=12, block_size=4, num_blocks=12, lens=[9, 5], scale_gran=abi.SCALE_PER_HEAD),  # generic tier
    ]):
        if layout == abi.LAYOUT_HND_PACKED and kw["dim"] % pack:
            continue
        case = cases.make_case(700 + i, layout=layout, pack=pack, dtype=io, cache_dtype=abi.DTYPE_F8_E4M3,
                               real_values=True, **kw)
        case.note = f"fp8 {i}"
        k, v = check_write(case)
        check_write(case, "typed")
        check_gather(case, k, v)


def test_fp8_quantise_every_bf16_value():
    """All 65 536 bf16 bit patterns (NaNs, infinities, denormals, -0 included) through the
    quantising write at several scales; then every e4m3 code back through the gather."""
    H, D = 4, 64
    n = 1 << 16
    T = n // (H * D)
    bits = np.arange(n, dtype=np.uint16).reshape(T, H, D)
    for scales in ([1.0, 0.37, 3.3, 1e-3], [0.013, 448.0, 2.0 ** -20, 7.0]):
        case = cases.make_case(9, dtype=abi.DTYPE_BF16, cache_dtype=abi.DTYPE_F8_E4M3, heads=H, dim=D,
                               block_size=16, num_blocks=T // 16 + 1, lens=[T], scale_gran=abi.SCALE_PER_HEAD)
        case.key, case.value = bits.copy(), bits[::-1].copy()
        case.k_scale = np.array(scales, np.float32)
        case.v_scale = np.array(scales[::-1], np.float32)
        k, v = check_write(case)
        check_gather(case, k, v)
    # every code through the dequantising gather for each IO type
    for io in (abi.DTYPE_BF16, abi.DTYPE_F16, abi.DTYPE_F32):
        case = cases.make_case(10, dtype=io, cache_dtype=abi.DTYPE_F8_E4M3, heads=2, dim=16, block_size=8,
                               num_blocks=1, lens=[8], scale_gran=abi.SCALE_PER_HEAD, real_values=True)
        codes = np.arange(256, dtype=np.uint8)
        case.k_scale = np.array([0.3, 1e-3], np.float32)
        case.v_scale = np.array([1.0, 3e4], np.float32)
        check_gather(case, codes.copy(), codes[::-1].copy())


def test_fp8_quantise_boundary_and_special_values_f32_io():
    """f32 inputs built to sit on and next to every e4m3 rounding boundary after the
    division (midpoints +- a few ulps, subnormal midpoints, +-448, +-464), plus infinities,
    NaNs with arbitrary payloads, +-0 and denormals, at awkward scales."""
    H, D = 2, 64
    rng = np.random.default_rng(77)
    codes = np.arange(0x7F, dtype=np.uint8)
    import ml_dtypes
    grid = codes.view(ml_dtypes.float8_e4m3fn).astype(np.float64)
    mids = np.concatenate([(grid[:-1] + grid[1:]) / 2, [464.0, 448.0, 2.0 ** -10, 2.0 ** -11]])
    for scales in ([1.0, 0.3], [0.0123, 7.7], [2.0 ** -30, 3e7]):
        vals = []
        for h, s in enumerate(scales):
            base = (mids * s).astype(np.float32)
            near = np.concatenate([np.nextafter(base, np.float32(np.inf)), np.nextafter(base, np.float32(-np.inf)), base,
                                   base * np.float32(1 + 3e-7), base * np.float32(1 - 3e-7)])
            near = np.concatenate([near, -near, [np.inf, -np.inf, 0.0, -0.0, 1e-45, -1e-45, 3e38]]).astype(np.float32)
            vals.append(near)
        n = max(len(v) for v in vals)
        T = -(-n // D) + 2
        x = rng.standard_normal((T, H, D)).astype(np.float32)
        bits = x.view(np.uint32).copy()
        for h, v in enumerate(vals):
            flat = bits[:, h, :].reshape(-1)
            flat[: len(v)] = v.view(np.uint32)
            flat[len(v): len(v) + 4] = [0x7FC00000, 0xFFC00001, 0x7F800001, 0xFFFFFFFF]  # NaNs
            bits[:, h, :] = flat.reshape(T, D)
        case = cases.make_case(9, dtype=abi.DTYPE_F32, cache_dtype=abi.DTYPE_F8_E4M3, heads=H, dim=D, block_size=16,
                               num_blocks=T // 16 + 1, lens=[T], scale_gran=abi.SCALE_PER_HEAD)
        case.key, case.value = bits.copy(), bits[::-1].copy()
        case.k_scale = np.array(scales, np.float32)
        case.v_scale = np.array(scales[::-1], np.float32)
        check_write(case)


@pytest.mark.parametrize("io", [abi.DTYPE_BF16, abi.DTYPE_F16, abi.DTYPE_F32])
@pytest.mark.parametrize("gran", [abi.SCALE_PER_HEAD, abi.SCALE_PER_TENSOR])
def test_scales_kernel_matches_oracle(io, gran):
    import torch
    from oracle.kvx_oracle import oracle
    rng = np.random.default_rng(5)
    for T, H, D in ((1000, 16, 256), (37, 4, 16), (1, 3, 24), (4096, 8, 128)):
        x = rng.standard_normal((T, H, D)).astype(np.float32)
        mask = rng.random(x.shape) < 0.001
        x[mask] *= 50
        y = rng.standard_normal((T, H, D)).astype(np.float32) * 0.01
        if T > 30:
            y[:, 1] = 0  # an all-zero head -> scale 1.0
        key, value = f32_to_bits(x, io), f32_to_bits(y, io)
        kio = abi.write_desc(T, H, D, io, key.ctypes.data, value.ctypes.data, abi.DTYPE_S64, 0, abi.MEMORY_HOST).io
        n = H if gran == abi.SCALE_PER_HEAD else 1
        eks, evs = np.zeros(n, np.float32), np.zeros(n, np.float32)
        assert oracle().kvx_oracle_kv_scales(C.byref(kio), gran, eks.ctypes.data, evs.ctypes.data) == OK
        dk = torch.from_numpy(key.view(np.uint8).reshape(-1)).cuda()
        dv = torch.from_numpy(value.view(np.uint8).reshape(-1)).cuda()
        dio = abi.write_desc(T, H, D, io, dk.data_ptr(), dv.data_ptr(), abi.DTYPE_S64, 0).io
        ks = torch.full((n,), -1.0, device="cuda")
        vs = torch.full((n,), -1.0, device="cuda")
        L = kvx_b200.lib()
        ws = torch.zeros(L.kvx_kv_scales_workspace_bytes(H), dtype=torch.uint8, device="cuda")
        for _ in range(2):  # the second call checks that the workspace was left zeroed
            st = L.kvx_launch_kv_scales(C.byref(dio), gran, ks.data_ptr(), vs.data_ptr(), ws.data_ptr(), ws.numel(), None)
            assert st == OK
            torch.cuda.synchronize()
            assert np.array_equal(ks.cpu().numpy(), eks) and np.array_equal(vs.cpu().numpy(), evs)
            assert int(ws.max()) == 0


def test_config5_fp8_shape_with_outliers():
    """bf16 in, 16 heads x 256, block 64, 0.1 % outliers x50, per-head scale = absmax / 448
    computed by the library's own reduction."""
    import torch
    from kvx_b200 import ops
    rng = np.random.default_rng(55)
    case = cases.make_case(55, dtype=abi.DTYPE_BF16, cache_dtype=abi.DTYPE_F8_E4M3, heads=16, dim=256,
                           block_size=64, num_blocks=8, lens=[200, 150, 64], scale_gran=abi.SCALE_PER_HEAD)
    for name in ("key", "value"):
        x = rng.standard_normal(case.key.shape).astype(np.float32)
        x[rng.random(x.shape) < 0.001] *= 50
        setattr(case, name, f32_to_bits(x, abi.DTYPE_BF16))
    dk = torch.from_numpy(case.key.view(np.int16)).cuda().view(torch.bfloat16)
    dv = torch.from_numpy(case.value.view(np.int16)).cuda().view(torch.bfloat16)
    ks, vs = ops.compute_kv_scales(dk, dv, per_head=True)
    case.k_scale, case.v_scale = ks.cpu().numpy(), vs.cpu().numpy()
    want = (np.abs(bits_to_f32(case.key, abi.DTYPE_BF16)).max(axis=(0, 2)) / np.float32(448)).astype(np.float32)
    assert np.array_equal(case.k_scale, want)
    k, v = check_write(case)
    check_gather(case, k, v)
    # dequantised values stay within half an e4m3 step of the input
    _, gk, _ = gpu_gather(case, k, v)
    t = 0
    for s, n in enumerate(case.lens.tolist()):
        got = bits_to_f32(gk[s, :n], abi.DTYPE_BF16)
        ref = bits_to_f32(case.key[t:t + n], abi.DTYPE_BF16)
        # e4m3 keeps 3 mantissa bits: relative error <= 2^-4 (+ the subnormal step)
        assert np.all(np.abs(got - ref) <= np.abs(ref) * 0.0625 + want[None, :, None] * 2.0 ** -9 * 1.01)
        t += n
