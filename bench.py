#!/usr/bin/env python
"""Benchmark of the paged KV-cache write + gather hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

One step = one pass of the hot path over the configuration: `layers` prefill writes (one per
layer, each into its own page tensors) followed by `layers` full gathers.  Default workload
is the Llama-3-8B prefill configuration (bf16, 8 KV heads x 128, block 16, 64 sequences of
512..4096 tokens, ~10 % of slots = -1, pages drawn from a pool of up to 150 GB).  With N > 1
(launched by torch.distributed.run, one process per GPU) the cache is sharded by KV head:
rank r owns heads [r*8/N, (r+1)*8/N), index metadata is replicated, and no collective runs
on the data path (one barrier + one max-reduction of the measured time).

Prints ONE JSON line:  value = whole-job GB/s of algorithmic HBM bytes with inputs resident
in HBM; e2e = the same metric through the host-buffer C-ABI entry points (pinned host K/V in,
gathered K/V out, copies inside the timed region); roofline = dominant kernel against the
measured HBM copy peak; cpu_baseline = the CPU restatement timed on this box's cores.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def measured_peak() -> tuple[float, str]:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="kvx_b200", choices=["kvx_b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--layers", type=int, default=None, help="override the configuration's layer count")
    ap.add_argument("--pool-gb", type=float, default=None, help="cap the page pool (per device)")
    ap.add_argument("--seqs", type=int, default=None, help="override the number of sequences (small profiling cases)")
    ap.add_argument("--e2e-steps", type=int, default=None, help="steps of the host-buffer leg (default: min(steps, 3))")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-chunk-mb", type=int, default=64, help="staging chunk of the host-buffer pipeline")
    ap.add_argument("--no-attention", action="store_true", help="skip the informational fused decode-attention leg")
    ap.add_argument("--only-attention", action="store_true",
                    help="fill the pages with one write per layer, time only the fused decode attention and print its "
                         "numbers (the small command the attention kernel is profiled with)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-verify", action="store_true", help="skip the byte check of the timed buffers")
    ap.add_argument("--layout", default="nhd", choices=["nhd", "hnd", "packed", "paged"],
                    help="page layout of the headline workload: NHD (default), HND, HND_PACKED with 16-byte pack "
                         "groups for K and V, or 'paged' = packed K + [blocks, heads, dim, block_size] V")
    ap.add_argument("--configs", default="c4,c5,c3,c4:packed,c2:packed,c4:paged",
                    help="other configurations (name or name:layout) timed on a few layers each and verified after "
                         "the headline workload; '' = none")
    ap.add_argument("--no-reference-kernels", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU baseline budget")
    ap.add_argument("--option", action="append", default=[], help="tuning knob name=value")
    return ap.parse_args()


def config_dict(spec, meta, layers: int, heads_rank: int, pool_gb: float, world: int, layout: str) -> dict:
    """The `config` object of the JSON line; both arms print the same one for the same workload."""
    return {"workload": spec.name, "layout": layout, "layers": layers, "heads_global": spec.heads,
            "heads_per_gpu": heads_rank, "head_dim": spec.dim, "block_size": spec.block_size, "seqs": spec.seqs,
            "write_tokens": meta.write_tokens, "valid_tokens": meta.valid_tokens, "gather_tokens": meta.gather_tokens,
            "pool_blocks_per_tensor": meta.num_blocks, "pool_gb_per_gpu": pool_gb,
            "parallelism": f"kv_head_shard{world}",
            "l2": "inputs (K+V batch, page pool) larger than L2; every layer has its own pages"}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ------------------------------------------------------------------ CPU baseline ---------

def cpu_baseline(spec, seconds: float, threads: int | None = None) -> dict:
    """Times the CPU restatement (row memcpy per valid token, page-chunk memcpy per gathered
    page, pthreads) on ONE layer of the configuration with a pool of twice the needed pages,
    repeated until about `seconds` have passed.  This is test infrastructure timed as a
    baseline; the product never calls it."""
    import numpy as np
    from kvx_b200 import abi, workloads
    from kvx_b200.bench_support import DTYPE_CODE
    from oracle.kvx_oracle import oracle

    threads = threads or len(os.sched_getaffinity(0))
    cpu_spec = spec
    if spec.cache_dtype == "f8e4m3":
        return {"value": None, "unit": "GB/s", "cores": threads, "kind": "port",
                "sample": "not timed: the threaded CPU form covers the copy path only"}
    meta = workloads.build_metadata(cpu_spec, num_blocks=None, pool_budget_bytes=0)  # pool = needed pages
    meta = workloads.build_metadata(cpu_spec, num_blocks=2 * meta.gather_pages)
    H, D, bs = spec.heads, spec.dim, spec.block_size
    e = workloads.ELEM[spec.io_dtype]
    rng = np.random.default_rng(7)
    T, S, Lmax = meta.write_tokens, spec.seqs, meta.max_seq_len
    np_t = np.uint16 if e == 2 else np.uint32
    key = rng.integers(0, 65535, size=(T, H, D), dtype=np.uint16).astype(np_t) if e == 2 else rng.integers(0, 2 ** 32 - 1, size=(T, H, D), dtype=np.uint32)
    value = key[::-1].copy()
    geom = abi.CacheGeometry(meta.num_blocks, bs, H, D)
    ck, cv = np.zeros(geom.elems, np_t), np.zeros(geom.elems, np_t)
    ok_, ov_ = np.zeros((S, Lmax, H, D), np_t), np.zeros((S, Lmax, H, D), np_t)
    code = DTYPE_CODE[spec.io_dtype]
    cache = abi.cache_desc(geom, code, ck.ctypes.data, cv.ctypes.data, abi.MEMORY_HOST)
    w = abi.write_desc(T, H, D, code, key.ctypes.data, value.ctypes.data, abi.DTYPE_S64, meta.slots.ctypes.data, abi.MEMORY_HOST)
    g = abi.gather_desc(S, Lmax, H, D, code, ok_.ctypes.data, ov_.ctypes.data, abi.DTYPE_S32, meta.table.ctypes.data,
                        meta.table.shape[1], meta.lens.ctypes.data, abi.MEMORY_HOST)
    L = oracle()
    for _ in range(1):  # warm-up: touches every page once
        assert L.kvx_cpu_baseline_write_kv(C.byref(cache), C.byref(w), threads) == 0
        assert L.kvx_cpu_baseline_gather_kv(C.byref(cache), C.byref(g), threads) == 0
    reps, t_w, t_g = 0, 0.0, 0.0
    t_end = time.perf_counter() + seconds
    while reps < 3 or time.perf_counter() < t_end:
        t0 = time.perf_counter(); L.kvx_cpu_baseline_write_kv(C.byref(cache), C.byref(w), threads)
        t1 = time.perf_counter(); L.kvx_cpu_baseline_gather_kv(C.byref(cache), C.byref(g), threads)
        t2 = time.perf_counter()
        t_w += t1 - t0; t_g += t2 - t1; reps += 1
        if reps >= 200:
            break
    wb, gb = meta.write_bytes(H), meta.gather_bytes(H)
    return {"value": round((wb + gb) * reps / (t_w + t_g) / 1e9, 2), "unit": "GB/s", "cores": threads, "kind": "port",
            "write_gbs": round(wb * reps / t_w / 1e9, 2), "gather_gbs": round(gb * reps / t_g / 1e9, 2),
            "ms_per_layer": round((t_w + t_g) / reps * 1e3, 3),
            "sample": f"1 of {spec.layers} layers (all {H} heads), {T} write tokens / {meta.gather_tokens} gathered, "
                      f"pool = 2x needed pages in host RAM, {reps} repetitions; the reference has no CPU data "
                      f"path, this is the CPU restatement of its kernels"}


def reference_arm(args) -> None:
    """`--impl reference`: the reference's hot path on this box's host cores.  The reference
    moves data only in CUDA (its C entry points validate and return), so the CPU arm is the
    CPU restatement of its kernels, all host threads, one layer of the workload per step."""
    from kvx_b200 import workloads
    rank, world, _ = dist_env()
    if rank != 0:
        return
    spec = workloads.SPECS[args.workload]
    threads = len(os.sched_getaffinity(0))
    per_step = 1.0
    t0 = time.perf_counter()
    res = cpu_baseline(spec, seconds=max(2.0, min(60.0, per_step * (args.steps + args.warmup))), threads=threads)
    line = {"impl": "reference", "metric": "kv_write_gather_hbm_gbs", "value": res["value"], "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": res.get("ms_per_layer"), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            # the workload of the other arm at this many GPUs (the same object it prints); what a step
            # of THIS arm samples of it is said in cpu_baseline.sample
            "config": reference_config(spec, args),
            "cpu_baseline": res,
            "e2e": {"value": res["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": round(time.perf_counter() - t0, 1)}
    if not args.no_reference_kernels:
        line["reference_cuda"] = reference_cuda_column(args, spec)
    print(json.dumps(line), flush=True)


def reference_config(spec, args) -> dict:
    """The `config` the GPU arm prints for the same command line (the page pool at its stated
    size, which a B200 holds; the layers and layout of the command line)."""
    from kvx_b200 import workloads
    world = max(1, args.gpus)
    layers = spec.layers if args.layers is None else args.layers
    budget = None if args.pool_gb is None else args.pool_gb * 1e9 * spec.layers / layers
    meta = workloads.build_metadata(spec, pool_budget_bytes=budget, shards=world)
    heads_rank = spec.heads // world
    page_local = spec.block_size * heads_rank * spec.dim * workloads.ELEM[spec.cache_dtype]
    pool_gb = round(2 * layers * meta.num_blocks * page_local / 1e9, 2)
    return config_dict(spec, meta, layers, heads_rank, pool_gb, world, args.layout)


def reference_cuda_column(args, spec) -> dict:
    """Extra column of the reference arm: the reference project's own CUDA kernels (compiled
    unmodified for sm_100a) on device-resident inputs of the same workload, a few layers,
    CUDA-event timed.  Not the arm's headline value (that is the host-core run above)."""
    try:
        import torch
        if not torch.cuda.is_available():
            return {"unavailable": "no CUDA device"}
        from kvx_b200 import bench_support as bs
        torch.cuda.set_device(dist_env()[2])
        dw = bs.setup_device_workload(spec, 0, 1, layers=min(spec.layers, 4), pool_gb=args.pool_gb)
        res = time_reference_kernels(dw, measured_peak()[0])
        del dw
        torch.cuda.empty_cache()
        return res
    except Exception as exc:
        return {"unavailable": repr(exc)[:160]}


# ------------------------------------------------------------------ GPU arm --------------

def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import kvx_b200
    from kvx_b200 import abi, bench_support as bs, workloads

    rank, world, local = dist_env()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        # NCCL announces its version on stdout at start-up; stdout carries the one JSON line only.
        sys.stdout.flush()
        saved_fd = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            os.dup2(saved_fd, 1)
            os.close(saved_fd)
    for opt in args.option:
        name, val = opt.split("=")
        kvx_b200.set_option(name, int(val))
    L = kvx_b200.lib()
    spec = workloads.SPECS[args.workload]
    if args.seqs is not None:
        import dataclasses
        spec = dataclasses.replace(spec, seqs=args.seqs, name=f"{spec.name}_seqs{args.seqs}")
    peak, peak_kind = measured_peak()

    dw = bs.setup_device_workload(spec, rank, world, layers=args.layers, pool_gb=args.pool_gb, layout=args.layout)
    layers, meta = dw.layers, dw.meta
    stream = torch.cuda.current_stream().cuda_stream

    if args.only_attention:
        for l in range(layers):
            bs.launch_write(dw, l, stream)
        res = run_attention(dw, args.steps)
        res.update({"workload": spec.name, "layers": layers, "steps": args.steps, "gather_tokens": meta.gather_tokens})
        print(json.dumps({"fused_decode_attention": res}), flush=True)
        return

    def step(events=None):
        if events:
            events[0].record()
        for l in range(layers):
            bs.launch_write(dw, l, stream)
        if events:
            events[1].record()
        for l in range(layers):
            bs.launch_gather(dw, l, stream)
        if events:
            events[2].record()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    if not args.no_verify:
        bs.fill_sentinel(dw)  # before the warm-up: the check below looks at the buffers the timed steps used
    sampler = bs.ClockSampler(local, period_ms=20)
    sampler.start()  # sampled from the warm-up on: the timed region alone can be shorter than one period
    for _ in range(max(args.warmup, 3)):
        step()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier()
    launches0 = L.kvx_b200_launch_count()
    for i in range(args.steps):
        step(ev[i])
    barrier()
    launches = L.kvx_b200_launch_count() - launches0
    clocks = sampler.stop()

    total_ms = ev[0][0].elapsed_time(ev[-1][2])
    write_ms = sum(e[0].elapsed_time(e[1]) for e in ev)
    gather_ms = sum(e[1].elapsed_time(e[2]) for e in ev)
    t = torch.tensor([total_ms, write_ms, gather_ms], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, write_ms, gather_ms = [float(x) for x in t.tolist()]

    # ---- byte check of the buffers the timed steps wrote and gathered, on every rank -------
    verified, verify_detail = None, None
    if not args.no_verify:
        verify_detail = bs.verify_layer(dw, layers - 1)
        verified = all_ranks_true(verify_detail["ok"], dist)

    # ---- host-buffer leg (the call a user of the C ABI with host buffers makes) -------------
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, dw, dist)

    attention = None
    if world == 1 and not args.no_attention:
        attention = run_attention(dw, min(args.steps, 3))

    # ---- the other configurations, a few layers each, sharded over the same ranks -----------
    pool_gb_used = round(dw.pool.numel() / 1e9, 2)
    write_bytes_rank, gather_bytes_rank, heads_rank = dw.write_bytes, dw.gather_bytes, dw.heads
    configs = None
    wanted = [c for c in args.configs.split(",") if c and c != args.workload]
    if args.layers is not None or args.seqs is not None or args.pool_gb is not None:
        wanted = []  # a cut-down run (profiling, experiments) times its own workload only
    if wanted and not args.only_attention:
        del dw, step
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        configs = {}
        for name in wanted:
            configs[name] = run_config_leg(name, rank, world, dist, peak, verify=not args.no_verify)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    wb_all, gb_all = meta.write_bytes(spec.heads), meta.gather_bytes(spec.heads)  # all heads = all ranks
    steps = args.steps
    value = (wb_all + gb_all) * layers * steps / (total_ms * 1e-3) / 1e9
    write_gbs_rank = write_bytes_rank * layers * steps / (write_ms * 1e-3) / 1e9
    gather_gbs_rank = gather_bytes_rank * layers * steps / (gather_ms * 1e-3) / 1e9
    dom, dom_gbs, dom_bytes, dom_ms = ("gather", gather_gbs_rank, gather_bytes_rank, gather_ms) \
        if gather_bytes_rank >= write_bytes_rank else ("write", write_gbs_rank, write_bytes_rank, write_ms)
    traffic = TRAFFIC_PER_LAUNCH.get((args.workload, dom)) if args.layout == "nhd" else None
    if traffic is not None and args.seqs is not None:
        traffic = None  # the capture was taken on the configuration's own token counts
    line = {
        "metric": "kv_write_gather_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
        "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": round(total_ms / steps, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": config_dict(spec, meta, layers, heads_rank, pool_gb_used, world, args.layout),
        "pct_of_nominal_8tbs": round(100 * value / world / NOMINAL_HBM_GBS, 1),
        "write": {"gbs_per_gpu": round(write_gbs_rank, 1), "us_per_launch": round(write_ms * 1e3 / (layers * steps), 2),
                  "tokens_per_s": round(meta.valid_tokens * layers * steps / (write_ms * 1e-3)),
                  "frac_of_peak": round(write_gbs_rank / peak, 4)},
        "gather": {"gbs_per_gpu": round(gather_gbs_rank, 1), "us_per_launch": round(gather_ms * 1e3 / (layers * steps), 2),
                   "tokens_per_s": round(meta.gather_tokens * layers * steps / (gather_ms * 1e-3)),
                   "frac_of_peak": round(gather_gbs_rank / peak, 4)},
        "roofline": {"bound": "hbm", "kernel": dom, "achieved": round(dom_gbs, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(dom_gbs / peak, 4), "peak_kind": peak_kind,
                     "bytes_per_launch": dom_bytes, "us_per_launch": round(dom_ms * 1e3 / (layers * steps), 2),
                     # DRAM bytes of one launch; the capture is of all heads on one GPU and the traffic is
                     # proportional to the heads a rank owns
                     "traffic": None if traffic is None else traffic // world},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    if verified is not None:
        line["verified"] = verified
        line["verify"] = {"what": "last layer of the timed buffers, every rank: pool rows at valid slots == input rows, "
                                  "all other pool rows == fill pattern, gathered rows below len == pages[table], rows "
                                  "past len == sentinel", "rank0": verify_detail}
    if configs is not None:
        line["configs"] = configs
    if e2e is not None:
        line["e2e"] = e2e
    if attention is not None:
        line["fused_decode_attention"] = attention
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(spec, args.cpu_seconds)
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one launch on one GPU holding all KV heads, from
# an ncu capture of the kernel that the launcher picks for the workload (2 layers, 4 GB pool, the
# workload's own token counts per launch, so nothing is scaled).
TRAFFIC_PER_LAUNCH: dict = {
    ("c2", "gather"): 1_115_400_000,  # kvx_gather_pages_wide_kernel: 581.9 MB read + 533.5 MB written
    ("c2", "write"): 999_200_000,     # kvx_write_rows_kernel
}


def all_ranks_true(flag: bool, dist) -> bool:
    """Logical AND of a per-rank flag over the job."""
    import torch
    t = torch.tensor([1 if flag else 0], dtype=torch.int32, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(int(t.item()))


CONFIG_LEG_LAYERS = {"c1": 22, "c2": 2, "c3": 2, "c4": 4, "c5": 4}


def run_config_leg(name: str, rank: int, world: int, dist, peak: float, verify: bool = True, min_reps: int = 5) -> dict:
    """One of the other configurations on a few layers (each on its own pages), sharded by KV head
    over the job's ranks like the headline workload: writes and gathers timed separately with CUDA
    events (max over ranks), then the last layer byte-checked on every rank.  The fp8 configuration
    also times the absmax -> scale reduction that precedes its writes."""
    import torch
    import kvx_b200
    from kvx_b200 import abi, bench_support as bs, workloads
    L = kvx_b200.lib()
    name, _, layout = name.partition(":")
    layout = layout or "nhd"
    spec = workloads.SPECS[name]
    out = {"workload": spec.name, "layout": layout}
    if spec.heads % world:
        return {"workload": spec.name, "skipped": f"{world} GPUs do not divide {spec.heads} KV heads"}
    try:
        dw = bs.setup_device_workload(spec, rank, world, layers=CONFIG_LEG_LAYERS[name], layout=layout)
    except Exception as exc:  # e.g. out of memory on a smaller device
        return {"workload": spec.name, "error": repr(exc)[:160]}
    stream = torch.cuda.current_stream().cuda_stream
    if verify:
        bs.fill_sentinel(dw)
    legs = [("write", lambda l: bs.launch_write(dw, l, stream), dw.write_bytes),
            ("gather", lambda l: bs.launch_gather(dw, l, stream), dw.gather_bytes)]
    if spec.cache_dtype == "f8e4m3":
        io = abi.kv_io_desc(dw.meta.write_tokens, dw.heads, spec.dim, bs.DTYPE_CODE[spec.io_dtype],
                            dw.key.data_ptr(), dw.value.data_ptr())
        need = L.kvx_kv_scales_workspace_bytes(dw.heads)
        ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
        ks, vs = torch.empty_like(dw.k_scale), torch.empty_like(dw.v_scale)

        def scales(_l):
            st = L.kvx_launch_kv_scales(C.byref(io), abi.SCALE_PER_HEAD, ks.data_ptr(), vs.data_ptr(), ws.data_ptr(),
                                        need, stream)
            if st != abi.STATUS_OK:
                raise RuntimeError(f"kvx_launch_kv_scales status {st}")
        legs.insert(0, ("scales", scales, 2 * dw.key.numel() * dw.key.element_size()))

    def timed(fn, rounds):
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(rounds):
            for l in range(dw.layers):
                fn(l)
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # Warm-up: at least 3 rounds and about 0.15 s of the leg's own work, so that the clocks, which
    # drop while the device waits for the set-up above, are back up when the timing starts.
    for leg, fn, nbytes in legs:
        spent, rounds = 0.0, 0
        while rounds < 3 or (spent < 150.0 and rounds < 2000):
            spent += timed(fn, 1)
            rounds += 1
        per_round = spent / rounds
        reps = int(min(500, max(min_reps, 60.0 / max(per_round, 1e-3))))  # a timed region of about 60 ms
        us = timed(fn, reps) * 1e3 / (reps * dw.layers)
        gbs = nbytes / us / 1e3
        out[leg] = {"us_per_launch": round(us, 2), "gbs_per_gpu": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4),
                    "bytes_per_launch": int(nbytes), "launches_timed": reps * dw.layers}
    out["layers"] = dw.layers
    out["heads_per_gpu"] = dw.heads
    out["tokens"] = {"write": dw.meta.write_tokens, "valid": dw.meta.valid_tokens, "gathered": dw.meta.gather_tokens}
    if spec.cache_dtype == "f8e4m3":
        out["scales_match"] = all_ranks_true(bool(torch.equal(ks, dw.k_scale) and torch.equal(vs, dw.v_scale)), dist)
    if verify:
        res = bs.verify_layer(dw, dw.layers - 1)
        out["verified"] = all_ranks_true(res["ok"], dist)
        if not res["ok"]:
            out["verify_rank%d" % rank] = res
    del dw
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return out


def run_attention(dw, steps: int, group: int = 4) -> dict:
    """Informational: the gather fused into its consumer.  One decode query per sequence (4 query
    heads per KV head) attends over the workload's cached contexts through the same block table,
    every layer on its own pages; reported as K+V bytes of the live contexts per second."""
    import ctypes as C

    import torch
    import kvx_b200
    from kvx_b200 import abi, bench_support as bs
    L = kvx_b200.lib()
    spec, m = dw.meta.spec, dw.meta
    S, H, D = spec.seqs, dw.heads, spec.dim
    q = torch.randn((S, H * group, D), device="cuda").to(dw.key.dtype)
    out = torch.empty_like(q)
    need = L.kvx_paged_attention_workspace_bytes(S, H * group, H, D, m.max_seq_len)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    a = abi.attention_desc(S, H * group, D, bs.DTYPE_CODE[spec.io_dtype], q.data_ptr(), out.data_ptr(), D ** -0.5,
                           m.max_seq_len, abi.DTYPE_S32, dw.table.data_ptr(), m.table.shape[1], dw.lens.data_ptr())
    none = abi.scale_desc(None, abi.SCALE_NONE, H)
    ks, vs = (dw.ks_desc, dw.vs_desc) if dw.ks_desc is not None else (none, none)  # fp8 cache: per-head scales
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        for l in range(dw.layers):
            st = L.kvx_launch_paged_attention_decode(C.byref(dw.caches[l]), C.byref(a), C.byref(ks), C.byref(vs),
                                                     ws.data_ptr(), need, stream)
            if st != abi.STATUS_OK:
                raise RuntimeError(f"kvx_launch_paged_attention_decode status {st}")

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (steps * dw.layers)
    kv_bytes = m.gather_tokens * 2 * H * D * workloads_elem(spec.cache_dtype)
    return {"us_per_launch": round(us, 2), "kv_read_gbs": round(kv_bytes / us / 1e3, 1), "q_heads_per_kv_head": group,
            "note": "reads the pages in place; no gathered copy is written"}


def workloads_elem(dtype: str) -> int:
    from kvx_b200 import workloads
    return workloads.ELEM[dtype]


def run_e2e(args, dw, dist) -> dict:
    """Same workload through kvx_host_write_kv / kvx_host_gather_kv: K/V batch, slots, block
    table and lengths in pinned host memory, gathered K/V back to pinned host memory, every
    step, copies inside the timed region."""
    import torch
    import kvx_b200
    from kvx_b200 import abi, bench_support as bs
    L = kvx_b200.lib()
    meta, spec = dw.meta, dw.meta.spec
    steps = args.e2e_steps or min(args.steps, 3)
    hk = torch.empty(dw.key.shape, dtype=dw.key.dtype).pin_memory(); hk.copy_(dw.key)
    hv = torch.empty(dw.value.shape, dtype=dw.value.dtype).pin_memory(); hv.copy_(dw.value)
    hs = torch.from_numpy(meta.slots).pin_memory()
    ht = torch.from_numpy(meta.table).pin_memory()
    hl = torch.from_numpy(meta.lens).pin_memory()
    # one pinned array for both outputs: V a fixed distance behind K, which lets the pipeline bring
    # a sequence's K run and V run back as one 2-D copy
    hout = torch.empty((2, *dw.out_k.shape), dtype=dw.out_k.dtype).pin_memory()
    hok, hov = hout[0], hout[1]
    seq_bytes = dw.out_k[0].numel() * dw.out_k.element_size()
    chunk = max(args.e2e_chunk_mb << 20, seq_bytes)
    pipe = C.c_void_p()
    st = L.kvx_host_pipe_create(chunk, spec.seqs, meta.table.shape[1], C.byref(pipe))
    if st != abi.STATUS_OK:
        return {"value": None, "unit": "GB/s", "error": f"kvx_host_pipe_create status {st}"}
    code = bs.DTYPE_CODE[spec.io_dtype]
    w = abi.write_desc(meta.write_tokens, dw.heads, spec.dim, code, hk.data_ptr(), hv.data_ptr(), abi.DTYPE_S64,
                       hs.data_ptr(), abi.MEMORY_HOST, dw.ks_desc, dw.vs_desc)
    g = abi.gather_desc(spec.seqs, meta.max_seq_len, dw.heads, spec.dim, code, hok.data_ptr(), hov.data_ptr(),
                        abi.DTYPE_S32, ht.data_ptr(), meta.table.shape[1], hl.data_ptr(), abi.MEMORY_HOST)
    ks = C.byref(dw.ks_desc) if dw.ks_desc is not None else None
    vs = C.byref(dw.vs_desc) if dw.vs_desc is not None else None

    def step():
        for l in range(dw.layers):
            a = L.kvx_host_write_kv(pipe, C.byref(dw.caches[l]), C.byref(w))
            b = L.kvx_host_gather_kv(pipe, C.byref(dw.caches[l]), C.byref(g), ks, vs)
            if a != 0 or b != 0:
                raise RuntimeError(f"host pipeline status write={a} gather={b}")
        if L.kvx_host_pipe_sync(pipe) != 0:
            raise RuntimeError("host pipeline failed")

    step()  # warm-up
    h0, d0 = C.c_uint64(), C.c_uint64()
    L.kvx_host_pipe_traffic(pipe, C.byref(h0), C.byref(d0))
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    tt = torch.tensor([dt], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    dt = float(tt.item())
    h1, d1 = C.c_uint64(), C.c_uint64()
    L.kvx_host_pipe_traffic(pipe, C.byref(h1), C.byref(d1))
    # the last layer's gathered bytes must equal what the device-resident path produces
    check = bool(torch.equal(hok[0, : int(meta.lens[0])].cuda(), dw.out_k[0, : int(meta.lens[0])])) if dw.layers else True
    L.kvx_host_pipe_destroy(pipe)
    del hk, hv, hok, hov
    ceiling = pcie_ceiling(dist)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    bytes_all = (meta.write_bytes(spec.heads) + meta.gather_bytes(spec.heads)) * dw.layers * steps
    return {"value": round(bytes_all / dt / 1e9, 2), "unit": "GB/s", "steps": steps,
            "ms_per_step": round(dt / steps * 1e3, 2),
            "h2d_bytes_per_step": int((h1.value - h0.value) // steps),
            "d2h_bytes_per_step": int((d1.value - d0.value) // steps),
            "pcie_gbs_per_gpu": round(((h1.value - h0.value) + (d1.value - d0.value)) / dt / 1e9, 2),
            "pcie_ceiling": ceiling,
            "matches_device_path": check, "n_gpus": world,
            "api": "kvx_host_write_kv + kvx_host_gather_kv (pinned host buffers, staged in chunks)"}


def pcie_ceiling(dist, chunk_mb: int = 64, chunks: int = 16) -> dict:
    """What the box gives plain pinned copies: every rank at once moves `chunks` chunks of `chunk_mb` MB
    host -> device, then device -> host, then both directions at the same time (two streams, one
    asynchronous copy per chunk), wall-clock timed from a barrier to the last rank's completion.
    Twice: with one host chunk per direction used over and over (it stays in the host's caches: the
    most the links give), and with every chunk at its own place in `chunks` x `chunk_mb` MB of pinned
    memory per direction (streamed from and to host DRAM, as the host-buffer leg's data is).  The
    host-buffer leg above cannot beat the 'both' figures; it is reported next to them."""
    import torch
    n = chunk_mb << 20
    host_in = torch.empty(n * chunks, dtype=torch.uint8).pin_memory()
    host_out = torch.empty(n * chunks, dtype=torch.uint8).pin_memory()
    host_in.fill_(1)
    host_out.fill_(0)  # first touch by this process
    dev_in = torch.empty(n, dtype=torch.uint8, device="cuda")
    dev_out = torch.ones(n, dtype=torch.uint8, device="cuda")
    up, down = torch.cuda.Stream(), torch.cuda.Stream()

    def run(h2d: bool, d2h: bool, streamed: bool) -> float:
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        t0 = time.perf_counter()
        for i in range(chunks):
            at = i * n if streamed else 0
            if h2d:
                with torch.cuda.stream(up):
                    dev_in.copy_(host_in[at:at + n], non_blocking=True)
            if d2h:
                with torch.cuda.stream(down):
                    host_out[at:at + n].copy_(dev_out, non_blocking=True)
        torch.cuda.synchronize()
        t = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    run(True, True, True)  # warm-up
    gb = n * chunks / 1e9
    world = int(os.environ.get("WORLD_SIZE", "1"))
    t_up, t_down, t_both = run(True, False, False), run(False, True, False), run(True, True, False)
    s_up, s_down, s_both = run(True, False, True), run(False, True, True), run(True, True, True)
    return {"h2d_gbs_per_gpu": round(gb / t_up, 1), "d2h_gbs_per_gpu": round(gb / t_down, 1),
            "both_gbs_per_gpu": round(2 * gb / t_both, 1), "both_gbs_all_gpus": round(2 * gb * world / t_both, 1),
            "streamed": {"h2d_gbs_per_gpu": round(gb / s_up, 1), "d2h_gbs_per_gpu": round(gb / s_down, 1),
                         "both_gbs_per_gpu": round(2 * gb / s_both, 1),
                         "both_gbs_all_gpus": round(2 * gb * world / s_both, 1)},
            "how": f"{chunks} x {chunk_mb} MB pinned copies per direction and rank, all {world} ranks at once; "
                   f"'streamed': every chunk at its own place in {chunks * chunk_mb} MB per direction"}


def time_reference_kernels(dw, peak: float) -> dict:
    """The reference project's own CUDA kernels (compiled unmodified for sm_100a) on the same
    device-resident inputs, a few layers, CUDA-event timed.  Context for the numbers above."""
    import torch
    from oracle.kvx_oracle import reference
    try:
        R = reference()
    except Exception as exc:  # library missing or unloadable
        return {"unavailable": str(exc)[:120]}
    if R is None or dw.meta.spec.cache_dtype == "f8e4m3":
        return {"unavailable": "oracle/_ref/libkvx_ref.so not present" if R is None else "no fp8 path in the reference"}
    stream = torch.cuda.current_stream().cuda_stream
    n = min(dw.layers, 4)
    out = {}
    for name, fn, desc, nbytes in (("write", R.kvx_launch_write_kv, dw.write, dw.write_bytes),
                                   ("gather", R.kvx_launch_gather_kv, dw.gather, dw.gather_bytes)):
        for l in range(n):
            assert fn(C.byref(dw.caches[l]), C.byref(desc), stream) == 0
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            for l in range(n):
                fn(C.byref(dw.caches[l]), C.byref(desc), stream)
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / (3 * n)
        out[name] = {"us_per_launch": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
                     "frac_of_peak": round(nbytes / us / 1e3 / peak, 4)}
    return out


if __name__ == "__main__":
    main()
