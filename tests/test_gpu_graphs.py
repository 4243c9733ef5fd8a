"""The launchers inside CUDA graphs: they allocate nothing, never synchronise and take the
stream they are given, so a decode step's per-layer calls can be captured once and replayed.
Checks that a captured write + gather (+ fused attention) sequence replays to the same bytes as
eager launches, on new inputs written into the same buffers."""
import ctypes as C

import numpy as np
import pytest

import kvx_b200
from kvx_b200 import abi

import cases
from harness import back, descriptors, device_buffers, oracle_gather, oracle_write

pytestmark = pytest.mark.gpu


def test_write_and_gather_replay_from_a_graph():
    import torch
    L = kvx_b200.lib()
    layers = 6
    case = cases.make_case(3100, dtype=abi.DTYPE_BF16, num_blocks=64, block_size=16, heads=4, dim=64,
                           lens=[100, 17, 0, 333, 16], pad_frac=0.1)
    bufs = [device_buffers(case) for _ in range(layers)]
    descs = [descriptors(case, b, abi.MEMORY_DEVICE) for b in bufs]
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            s = torch.cuda.current_stream().cuda_stream
            for cache, write, gather, _, _ in descs:
                assert L.kvx_launch_write_kv(C.byref(cache), C.byref(write), s) == abi.STATUS_OK
                assert L.kvx_launch_gather_kv(C.byref(cache), C.byref(gather), s) == abi.STATUS_OK
    # capture does not execute: the buffers still hold their initial bytes
    torch.cuda.synchronize()
    assert np.array_equal(back(bufs[0]["cache_k"], case.cache_k), case.cache_k)
    _, ek, ev = oracle_write(case)
    _, eok, eov = oracle_gather(case, ek, ev)
    for rounds in range(2):  # the second replay runs on caches that already hold the tokens
        graph.replay()
        torch.cuda.synchronize()
        for b in bufs:
            assert np.array_equal(back(b["cache_k"], case.cache_k), ek) and np.array_equal(back(b["cache_v"], case.cache_v), ev)
            assert np.array_equal(back(b["out_k"], case.out_k), eok) and np.array_equal(back(b["out_v"], case.out_v), eov)
    # new tokens in the same input buffers, same graph
    rng = np.random.default_rng(5)
    new_key = rng.integers(0, 2 ** 16, size=case.key.shape, dtype=np.uint16)
    import dataclasses
    case2 = dataclasses.replace(case, key=new_key)
    for b in bufs:
        b["key"].copy_(torch.from_numpy(new_key.view(np.uint8).reshape(-1)).cuda())
    graph.replay()
    torch.cuda.synchronize()
    _, ek2, _ = oracle_write(case2)
    assert np.array_equal(back(bufs[-1]["cache_k"], case.cache_k), ek2)


def test_fused_attention_replays_from_a_graph():
    import torch
    from kvx_b200 import ops
    torch.manual_seed(2)
    S, Hkv, G, D, bs, nb = 5, 2, 4, 128, 16, 600
    kc = torch.randn((nb, bs, Hkv, D), device="cuda").to(torch.bfloat16)
    vc = torch.randn((nb, bs, Hkv, D), device="cuda").to(torch.bfloat16)
    lens = torch.tensor([1, 16, 100, 3000, 411], dtype=torch.int32, device="cuda")   # 3000: split in chunks
    mb = 200
    table = torch.randperm(nb, device="cuda").to(torch.int32)[: S * mb // 2].repeat(2)[: S * mb].reshape(S, mb).contiguous()
    q = torch.randn((S, Hkv * G, D), device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    ws = torch.empty(ops.attention_workspace_bytes(S, Hkv * G, Hkv, D, mb * bs), dtype=torch.uint8, device="cuda")
    eager = ops.paged_attention_decode(q, kc, vc, table, lens, D ** -0.5, out=torch.empty_like(q), workspace=ws).clone()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            ops.paged_attention_decode(q, kc, vc, table, lens, D ** -0.5, out=out, workspace=ws)
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), eager.view(torch.int16))
