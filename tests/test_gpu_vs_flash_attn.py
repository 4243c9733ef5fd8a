"""Cross-implementation check of the paged decode attention against the flash_attn package's
paged kv-cache kernel (library code in this image; `flash_attn_with_kvcache` with a block
table, pages of 256 tokens as that kernel requires): same inputs, outputs within bf16
rounding of each other, CUDA-event timings of both written to the folder named by
KVX_RESULTS_DIR, when set, for the record.
Runs in a child process and is skipped when flash_attn cannot be imported or run here."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SKIP_RC = 77


def _time(fn, iters=5):
    import torch
    fn(); fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters


def _compare():
    import numpy as np
    import torch

    from kvx_b200 import ops
    try:
        from flash_attn import flash_attn_with_kvcache
    except Exception as exc:
        print(f"flash_attn unavailable: {exc!r}"[:300])
        raise SystemExit(SKIP_RC)

    rows = []
    for label, S, max_ctx, group in (("decode_512_seqs", 512, 32768, 4), ("decode_64_seqs", 64, 4096, 4),
                                     ("mha_32_seqs", 32, 2048, 1)):
        torch.manual_seed(1)
        rng = np.random.default_rng(3)
        Hkv, D, bs = 8, 128, 256
        lens_np = np.maximum(1, np.rint(np.exp(rng.random(S) * np.log(max_ctx))).astype(np.int64))
        pages = [int(-(-n // bs)) for n in lens_np]
        nb, mb = sum(pages) + 4, max(pages)
        kc = torch.randn((nb, bs, Hkv, D), device="cuda", dtype=torch.bfloat16)
        vc = torch.randn((nb, bs, Hkv, D), device="cuda", dtype=torch.bfloat16)
        perm = rng.permutation(nb)
        table = np.zeros((S, mb), dtype=np.int32)
        at = 0
        for s, n in enumerate(pages):
            table[s, :n] = perm[at:at + n]
            at += n
        table = torch.from_numpy(table).cuda()
        lens = torch.from_numpy(lens_np.astype(np.int32)).cuda()
        q = torch.randn((S, Hkv * group, D), device="cuda", dtype=torch.bfloat16)
        scale = D ** -0.5
        Lmax = int(lens_np.max())
        ws = torch.empty(max(16, ops.attention_workspace_bytes(S, Hkv * group, Hkv, D, Lmax)), dtype=torch.uint8,
                         device="cuda")
        out = torch.empty_like(q)

        def ours():
            return ops.paged_attention_decode(q, kc, vc, table, lens, scale, max_seq_len=Lmax, out=out, workspace=ws)

        def theirs():
            return flash_attn_with_kvcache(q.unsqueeze(1), kc, vc, cache_seqlens=lens, block_table=table,
                                           softmax_scale=scale, causal=True)
        try:
            ref = theirs().squeeze(1).float()
        except Exception as exc:
            print(f"flash_attn cannot run here: {exc!r}"[:300])
            raise SystemExit(SKIP_RC)
        got = ours().float()
        torch.cuda.synchronize()
        # two bf16-rounded results of O(1) values: a few units in the last place apart at most
        assert torch.allclose(got, ref, atol=2e-2, rtol=2e-2), (label, (got - ref).abs().max().item())
        kv_bytes = int(lens_np.sum()) * 2 * Hkv * D * 2
        a, b = _time(ours), _time(theirs)
        rows.append({"case": label, "kv_gb": round(kv_bytes / 1e9, 3), "this_us": round(a, 1), "flash_attn_us": round(b, 1),
                     "this_kv_gbs": round(kv_bytes / a / 1e3, 1), "flash_attn_kv_gbs": round(kv_bytes / b / 1e3, 1)})
    out_dir = os.environ.get("KVX_RESULTS_DIR", "")
    if out_dir and os.path.isdir(out_dir):
        with open(os.path.join(out_dir, "vs_flash_attn.json"), "w") as f:
            json.dump(rows, f, indent=1)
    print(json.dumps(rows))


def test_attention_agrees_with_flash_attn_and_is_timed():
    p = subprocess.run([sys.executable, os.path.abspath(__file__)], capture_output=True, text=True, timeout=900)
    if p.returncode == SKIP_RC:
        pytest.skip(p.stdout.strip()[-300:] or "flash_attn unavailable")
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]


if __name__ == "__main__":
    sys.path.insert(0, ROOT)
    _compare()
