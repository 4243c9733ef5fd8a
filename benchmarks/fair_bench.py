#!/usr/bin/env python
"""fair_bench: the cache-write comparison table, this library against vLLM's own operator.

Follows the comparison the reference publishes (benchmarks/fair_bench.py:171-313): the same
eight decode-sized cases (:176-185), the same slot mapping (`build_kvx_like_slot_mapping`,
:19-34, pinned by benchmarks/tests/fair_bench_slot_mapping_test.py), the same columns of its
result file, and the native micro-benchmark program run as a subprocess and read through its
`write,` line (:120-146).  Differences, all in the direction of a fairer and fuller table:

* both operators are timed the same way -- CUDA events around `iters` back-to-back calls on the
  current stream (device time per call) and, next to it, wall-clock time per call with one
  synchronisation at the end (what a caller pays, dispatcher included).  The reference timed
  vLLM by wall clock and its own program by events;
* this library appears twice: through `torch.ops.kvx_b200.reshape_and_cache_flash_kvx`, the
  operator a serving engine would call, and through the native program `kvx_bench` (column
  `native`; skipped when the binary has not been built);
* the outputs of the two operators are compared bit for bit on every case;
* `--prefill` adds the Llama-3-8B prefill shape (one layer of the c2 configuration), where the
  call is bound by memory bandwidth rather than by launch latency, with GB/s and the fraction
  of the device's measured copy bandwidth (`--peak-gbs`).

    python benchmarks/fair_bench.py [--dtype bfloat16] [--iters 50] [--warmup 10] [--repeats 3]
                                    [--bin-path build/kvx_bench] [--output-csv out.csv] [--prefill]

Needs a CUDA device and vLLM's compiled cache operators; prints `vllm unavailable: ...` and
leaves the vLLM columns empty when they cannot be loaded.
"""
from __future__ import annotations

import argparse
import csv
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CASES = [
    {"num_heads": 8, "seq_count": 1, "seq_len": 128},
    {"num_heads": 8, "seq_count": 8, "seq_len": 512},
    {"num_heads": 8, "seq_count": 32, "seq_len": 128},
    {"num_heads": 32, "seq_count": 1, "seq_len": 128},
    {"num_heads": 32, "seq_count": 8, "seq_len": 512},
    {"num_heads": 32, "seq_count": 16, "seq_len": 1024},
    {"num_heads": 8, "seq_count": 8, "seq_len": 512, "tokens_per_seq": 16},
    {"num_heads": 32, "seq_count": 8, "seq_len": 1024, "tokens_per_seq": 32},
]


def build_kvx_like_slot_mapping(seq_count, seq_len, block_size, tokens_per_seq, device):
    """Slots of the last ``tokens_per_seq`` positions of ``seq_count`` sequences of ``seq_len``
    tokens, sequence s owning the consecutive pages ``s * ceil(seq_len / block_size) ...`` --
    the workload of the native program without ``--config``."""
    import torch
    if tokens_per_seq > seq_len:
        raise ValueError("tokens_per_seq cannot exceed seq_len")
    pages_per_seq = (seq_len + block_size - 1) // block_size
    pos = torch.arange(seq_len - tokens_per_seq, seq_len, dtype=torch.long)
    seq = torch.arange(seq_count, dtype=torch.long)
    slots = (seq[:, None] * pages_per_seq + pos[None, :] // block_size) * block_size + pos[None, :] % block_size
    return slots.reshape(-1).to(device)


def mean_std(values):
    return statistics.mean(values), (statistics.stdev(values) if len(values) > 1 else 0.0)


def time_call(fn, iters, warmup):
    """(device microseconds per call by CUDA events, wall microseconds per call)."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) * 1e6 / iters
    return a.elapsed_time(b) * 1e3 / iters, wall


def vllm_operator():
    """vLLM's reshape_and_cache_flash, or (None, reason)."""
    try:
        import torch
        from vllm import _custom_ops  # noqa: F401  (loads the compiled operators)
        return torch.ops._C_cache_ops.reshape_and_cache_flash, ""
    except Exception as exc:  # wheel missing, or its operators do not load on this box
        return None, repr(exc)[:200]


def run_native(bin_path, case, args):
    """tokens/s, GB/s and ms per call from the native program's `write,` line."""
    cmd = [bin_path, "--seq-count", str(case["seq_count"]), "--seq-len", str(case["seq_len"]),
           "--tokens-per-seq", str(case["tokens_per_seq"]), "--block-size", str(args.block_size),
           "--num-heads", str(case["num_heads"]), "--head-dim", str(args.head_dim), "--iters", str(args.iters),
           "--warmup", str(args.warmup), "--dtype", args.dtype]
    out = subprocess.run(cmd, check=True, text=True, capture_output=True).stdout
    for line in out.splitlines():
        if line.startswith("write,"):
            parts = line.split(",")
            return float(parts[10]), float(parts[11]), float(parts[9])
    raise RuntimeError("the native program printed no write line")


def run_case(case, args, vllm_op, rows):
    import torch

    from kvx_b200 import ops

    dtype = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}[args.dtype]
    heads, seqs, seq_len = case["num_heads"], case["seq_count"], case["seq_len"]
    tps, bs, dim = case["tokens_per_seq"], args.block_size, args.head_dim
    num_blocks = case.get("num_blocks", seqs * math.ceil(seq_len / bs))
    slots = case["slots"] if "slots" in case else build_kvx_like_slot_mapping(seqs, seq_len, bs, tps, "cuda")
    tokens = int(slots.numel())
    g = torch.Generator(device="cuda")
    g.manual_seed(42)
    key = torch.randn((tokens, heads, dim), generator=g, device="cuda", dtype=torch.float32).to(dtype)
    value = torch.randn((tokens, heads, dim), generator=g, device="cuda", dtype=torch.float32).to(dtype)
    shape = (num_blocks, bs, heads, dim)
    one = torch.ones(1, dtype=torch.float32, device="cuda")
    ours_k = torch.zeros(shape, dtype=dtype, device="cuda"); ours_v = torch.zeros_like(ours_k)
    elem = key.element_size()
    valid = int((slots >= 0).sum())
    moved = valid * heads * dim * elem * 4            # the reference's figure: K and V, read and written
    res = {"dtype": args.dtype, "num_heads": heads, "seq_count": seqs, "seq_len": seq_len, "tokens_per_seq": tps,
           "block_size": bs, "head_dim": dim, "num_blocks": num_blocks, "tokens": tokens}

    def ours():
        ops.reshape_and_cache_flash_kvx(key, value, ours_k, ours_v, slots, "auto", one, one)

    identical = None
    if vllm_op is not None:
        their_k = torch.zeros_like(ours_k); their_v = torch.zeros_like(ours_k)

        def theirs():
            vllm_op(key, value, their_k, their_v, slots, "auto", one, one)
        ours(); theirs()
        torch.cuda.synchronize()
        identical = bool(torch.equal(ours_k.view(torch.uint8), their_k.view(torch.uint8)) and
                         torch.equal(ours_v.view(torch.uint8), their_v.view(torch.uint8)))
    for name, fn in (("kvx", ours), ("vllm", theirs if vllm_op is not None else None)):
        if fn is None:
            continue
        dev, wall = zip(*[time_call(fn, args.iters, args.warmup) for _ in range(args.repeats)])
        for label, xs in (("device_us", dev), ("wall_us", wall)):
            res[f"{name}_{label}_mean"], res[f"{name}_{label}_std"] = mean_std(xs)
        res[f"{name}_tokens_per_s"] = valid / (res[f"{name}_device_us_mean"] * 1e-6)
        res[f"{name}_gb_per_s"] = moved / (res[f"{name}_device_us_mean"] * 1e-6) / 1e9
    if os.path.exists(args.bin_path) and "slots" not in case:
        runs = [run_native(args.bin_path, case, args) for _ in range(args.repeats)]
        res["native_ms_per_mean"], res["native_ms_per_std"] = mean_std([r[2] for r in runs])
        res["native_tokens_per_s"] = statistics.mean(r[0] for r in runs)
    res["identical"] = identical
    if vllm_op is not None:
        res["ratio_device"] = res["vllm_device_us_mean"] / res["kvx_device_us_mean"]
        res["ratio_wall"] = res["vllm_wall_us_mean"] / res["kvx_wall_us_mean"]
    if args.peak_gbs > 0:
        res["kvx_pct_of_peak"] = 100.0 * res["kvx_gb_per_s"] / args.peak_gbs
    rows.append(res)
    return res


def prefill_case(args):
    """One layer of the Llama-3-8B prefill configuration: 64 ragged sequences, about 10 % of
    the slots padded, pages drawn from a permuted pool."""
    import torch

    from kvx_b200 import workloads
    spec = workloads.SPECS["c2"]
    meta = workloads.build_metadata(spec, num_blocks=None, pool_budget_bytes=4e9 * spec.layers)
    return {"num_heads": spec.heads, "seq_count": spec.seqs, "seq_len": meta.max_seq_len,
            "tokens_per_seq": meta.write_tokens // spec.seqs, "num_blocks": meta.num_blocks,
            "slots": torch.from_numpy(meta.slots).cuda(), "label": "llama3-8b prefill, one layer"}


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--output-csv", default=os.path.join(ROOT, "benchmarks", "results", "fair_bench.csv"))
    ap.add_argument("--dtype", default="bfloat16", choices=["float32", "float16", "bfloat16"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--tokens-per-seq", type=int, default=1)
    ap.add_argument("--bin-path", default=os.path.join(ROOT, "build", "kvx_bench"))
    ap.add_argument("--peak-gbs", type=float, default=0.0, help="measured copy bandwidth of the device (GB/s)")
    ap.add_argument("--prefill", action="store_true", help="add the Llama-3-8B prefill shape")
    return ap.parse_args(argv)


def main(argv=None) -> int:
    args = parse_args(argv)
    import torch
    if not torch.cuda.is_available():
        print("fair_bench needs a CUDA device")
        return 1
    vllm_op, why = vllm_operator()
    print("env")
    print(f"torch_version={torch.__version__} device={torch.cuda.get_device_name(0)}")
    print("vllm_backend=reshape_and_cache_flash layout=NHD" if vllm_op is not None else f"vllm unavailable: {why}")
    print(f"dtype={args.dtype} iters={args.iters} warmup={args.warmup} repeats={args.repeats}")
    print()
    head = f"{'case':44s} {'kvx us':>9s} {'vllm us':>9s} {'ratio':>6s} {'kvx wall':>9s} {'vllm wall':>9s} {'native us':>9s} {'GB/s':>8s} same"
    print(head)
    rows = []
    cases = [dict(c, tokens_per_seq=c.get("tokens_per_seq", args.tokens_per_seq)) for c in CASES]
    if args.prefill:
        cases.append(prefill_case(args))
    for case in cases:
        r = run_case(case, args, vllm_op, rows)
        label = case.get("label") or (f"heads={r['num_heads']} seqs={r['seq_count']} len={r['seq_len']} "
                                      f"tokens/seq={r['tokens_per_seq']}")
        f = lambda k, scale=1.0: f"{r[k] * scale:9.2f}" if r.get(k) is not None else f"{'-':>9s}"
        ratio = f"{r['ratio_device']:5.2f}x" if "ratio_device" in r else f"{'-':>6s}"
        print(f"{label:44s} {f('kvx_device_us_mean')} {f('vllm_device_us_mean')} {ratio} {f('kvx_wall_us_mean')} "
              f"{f('vllm_wall_us_mean')} {f('native_ms_per_mean', 1e3)} {r['kvx_gb_per_s']:8.1f} "
              f"{ {True: 'yes', False: 'NO', None: '-'}[r['identical']] }")
    os.makedirs(os.path.dirname(os.path.abspath(args.output_csv)), exist_ok=True)
    fields = sorted({k for r in rows for k in r})
    with open(args.output_csv, "w", newline="", encoding="utf-8") as fh:
        w = csv.DictWriter(fh, fieldnames=fields)
        w.writeheader()
        w.writerows(rows)
    print(f"\nwrote {args.output_csv}")
    return 0 if all(r["identical"] is not False for r in rows) else 2


if __name__ == "__main__":
    sys.exit(main())
