"""Full-size checks on the GPU: the benchmark configurations at their stated token counts,
page sizes and pool sizes (two layers each instead of all, so the run stays short), verified
through properties that need no CPU copy of the data: write -> gather round trip, padding and
untouched pages keep their sentinel, output rows past a sequence's length stay untouched, a
second identical write changes nothing, K and V never mix."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SENT = 0x5A  # byte pattern of untouched memory (bf16 0x5A5A is an ordinary finite number)


def _run(workload: str, layers: int, pool_gb):
    import torch

    from kvx_b200 import bench_support as bs, workloads

    import gc
    gc.collect()
    torch.cuda.empty_cache()  # memory cached by earlier tests must count as free when sizing the pool
    spec = workloads.SPECS[workload]
    dw = bs.setup_device_workload(spec, layers=layers, pool_gb=pool_gb)
    meta = dw.meta
    stream = torch.cuda.current_stream().cuda_stream
    dw.pool.fill_(SENT)
    dw.out_k.view(torch.uint8).fill_(SENT)
    dw.out_v.view(torch.uint8).fill_(SENT)
    for l in range(dw.layers):
        bs.launch_write(dw, l, stream)
    torch.cuda.synchronize()

    slots = dw.slots
    valid = slots >= 0
    n_valid = int(valid.sum())
    assert n_valid == meta.valid_tokens
    lens = torch.from_numpy(meta.lens.astype(np.int64)).cuda()
    S, Lmax = spec.seqs, meta.max_seq_len
    pos = torch.arange(Lmax, device="cuda")[None, :].expand(S, Lmax)
    live = pos < lens[:, None]                       # [S, Lmax] positions the gather defines
    sent16 = torch.tensor([SENT | (SENT << 8)], dtype=torch.int16, device="cuda")

    for l in range(dw.layers):
        kp, vp = dw.layer_pages(l)
        kp16, vp16 = kp.view(torch.int16), vp.view(torch.int16)
        # rows addressed by valid slots hold exactly the input rows
        flat_k = kp16.view(-1, dw.heads * spec.dim)
        flat_v = vp16.view(-1, dw.heads * spec.dim)
        src_k = dw.key.view(torch.int16).view(-1, dw.heads * spec.dim)
        src_v = dw.value.view(torch.int16).view(-1, dw.heads * spec.dim)
        idx = slots[valid]
        assert torch.equal(flat_k[idx], src_k[valid]), f"layer {l}: K rows differ"
        assert torch.equal(flat_v[idx], src_v[valid]), f"layer {l}: V rows differ"
        # every other row of the pool still holds the sentinel
        touched = torch.zeros(flat_k.shape[0], dtype=torch.bool, device="cuda")
        touched[idx] = True
        assert bool((flat_k[~touched] == sent16).all()) and bool((flat_v[~touched] == sent16).all())

    # a second identical write changes nothing
    before = dw.layer_pages(0)[0].clone()
    bs.launch_write(dw, 0, stream)
    torch.cuda.synchronize()
    assert torch.equal(before, dw.layer_pages(0)[0])
    del before

    bs.launch_gather(dw, dw.layers - 1, stream)
    torch.cuda.synchronize()
    ok16, ov16 = dw.out_k.view(torch.int16), dw.out_v.view(torch.int16)
    # rows past the sequence length are untouched (checked a few sequences at a time to bound
    # the temporaries: the decode configuration's outputs are 33 GB each)
    step = max(1, int(1e9 // (Lmax * dw.heads * spec.dim * 2)))
    for s0 in range(0, S, step):
        dead = ~live[s0:s0 + step]
        assert bool((ok16[s0:s0 + step][dead] == sent16).all())
        assert bool((ov16[s0:s0 + step][dead] == sent16).all())
    if not spec.decode:
        # token t of the batch is position (s, p) of the gather: valid tokens come back bit-exact,
        # padded tokens come back as what the page held (the sentinel)
        got_k, got_v = ok16[live], ov16[live]          # sequence-major == batch order
        src_k = dw.key.view(torch.int16).view(-1, dw.heads, spec.dim)
        src_v = dw.value.view(torch.int16).view(-1, dw.heads, spec.dim)
        assert torch.equal(got_k[valid], src_k[valid]) and torch.equal(got_v[valid], src_v[valid])
        assert bool((got_k[~valid] == sent16).all()) and bool((got_v[~valid] == sent16).all())
    else:
        # decode: only each sequence's last position was written
        last = (lens - 1)
        rows = torch.arange(S, device="cuda")
        assert torch.equal(ok16[rows, last], dw.key.view(torch.int16))
        assert torch.equal(ov16[rows, last], dw.value.view(torch.int16))
    return dw


def test_config2_llama3_8b_full_token_count_and_pool_geometry():
    """142 060 tokens (127 653 valid), 64 ragged sequences, 71 525-page pool per tensor."""
    dw = _run("c2", layers=2, pool_gb=None)
    assert dw.meta.num_blocks == 71525 and dw.meta.write_tokens > 140000


def test_config4_llama3_70b_full_token_count():
    """262 144 tokens, 32 sequences of 8 192, fp16."""
    dw = _run("c4", layers=2, pool_gb=None)
    assert dw.meta.write_tokens == 262144


def test_config3_decode_full_contexts():
    """512 sequences, contexts log-uniform up to 32 768 (about 1.5 M gathered tokens, 64 KiB
    pages, 1..998 pages per sequence)."""
    dw = _run("c3", layers=1, pool_gb=None)
    assert dw.meta.gather_tokens > 1_000_000


def test_config5_fp8_full_size_round_trip_within_quantisation_error():
    """262 144 tokens of 16 x 256 bf16, quantised to e4m3 pages with per-head absmax scales
    and read back: every value within half an e4m3 step of its input."""
    import torch

    from kvx_b200 import bench_support as bs, workloads

    spec = workloads.SPECS["c5"]
    dw = bs.setup_device_workload(spec, layers=1)
    stream = torch.cuda.current_stream().cuda_stream
    absmax = dw.key.float().abs().amax(dim=(0, 2)).cpu().numpy()
    want = (absmax / np.float32(448.0)).astype(np.float32)       # one IEEE division, on the host
    assert np.array_equal(dw.k_scale.cpu().numpy(), want)
    bs.launch_write(dw, 0, stream)
    bs.launch_gather(dw, 0, stream)
    torch.cuda.synchronize()
    T = dw.meta.write_tokens
    got = dw.out_k.view(T, dw.heads, spec.dim)[: 1 << 16].float()
    ref = dw.key[: 1 << 16].float()
    tol = ref.abs() * 0.0625 + dw.k_scale[None, :, None] * 2.0 ** -9 * 1.01
    assert bool(((got - ref).abs() <= tol).all())
    # quantisation is idempotent: writing the dequantised values again gives the same pages
    pages = dw.layer_pages(0)[0].clone()
    dw.key.copy_(dw.out_k.view(dw.key.shape))
    bs.launch_write(dw, 0, stream)
    torch.cuda.synchronize()
    same = (pages == dw.layer_pages(0)[0]).float().mean()
    assert float(same) > 0.999


def test_bench_byte_check_accepts_good_buffers_and_sees_damage():
    """The byte check the benchmark runs on its timed buffers (bench_support.verify_layer): green on
    a written and gathered layer, red as soon as one page byte, one gathered byte or one byte past
    a sequence's end is changed.  Small pool so the run is short; c2 (padded slots) and c3 (decode
    write, pages that keep their fill pattern are gathered)."""
    import torch

    from kvx_b200 import bench_support as bs, workloads

    for name in ("c2", "c3"):
        spec = workloads.SPECS[name]
        if name == "c3":
            import dataclasses
            spec = dataclasses.replace(spec, seqs=24)
        dw = bs.setup_device_workload(spec, layers=2, pool_gb=1.0)
        stream = torch.cuda.current_stream().cuda_stream
        bs.fill_sentinel(dw)
        for l in range(dw.layers):
            bs.launch_write(dw, l, stream)
            bs.launch_gather(dw, l, stream)
        torch.cuda.synchronize()
        res = bs.verify_layer(dw, dw.layers - 1)
        assert res["ok"], (name, res)
        kp, _ = dw.layer_pages(dw.layers - 1)
        flat = kp.view(torch.uint8).view(-1)
        slot = int(dw.slots[dw.slots >= 0][0])
        row = dw.heads * spec.dim * 2
        flat[slot * row + 5] ^= 1                              # a written row
        assert not bs.verify_layer(dw, dw.layers - 1)["write_rows"]
        flat[slot * row + 5] ^= 1
        untouched = int((~torch.isin(torch.arange(flat.shape[0] // row, device="cuda"), dw.slots)).nonzero()[0])
        flat[untouched * row + 9] ^= 1                         # a row no slot names
        assert not bs.verify_layer(dw, dw.layers - 1)["untouched_pages"]
        flat[untouched * row + 9] ^= 1
        out = dw.out_v.view(torch.uint8).view(spec.seqs, -1)
        out[1, 3] ^= 1                                         # a gathered byte
        assert not bs.verify_layer(dw, dw.layers - 1)["gather_live"]
        out[1, 3] ^= 1
        s_short = int(dw.lens.argmin())
        if int(dw.lens[s_short]) < dw.meta.max_seq_len:
            out[s_short, -1] ^= 1                              # a byte past the end of a sequence
            assert not bs.verify_layer(dw, dw.layers - 1)["gather_dead"]
            out[s_short, -1] ^= 1
        assert bs.verify_layer(dw, dw.layers - 1)["ok"]
        del dw
