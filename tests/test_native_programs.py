"""The native programs over the C ABI: `benchmarks/kvx_bench.cu` (the reference's benchmark
command line and CSV lines, plus configurations, layouts and devices), `tests/kvx_kernel_test.cu`
(the reference's nine records extended, byte-exact against host loops) and
`benchmarks/fair_bench.py` (the comparison table against vLLM's operator).

Without a GPU: they compile, the benchmark refuses bad arguments as the reference's does, and the
slot mapping of the comparison script is what the reference's test asks for
(benchmarks/tests/fair_bench_slot_mapping_test.py).  With one (-m gpu): all three run."""
import importlib.util
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def programs():
    from kvx_b200 import build
    return build.build_programs()


def _fair_bench():
    spec = importlib.util.spec_from_file_location("fair_bench", os.path.join(ROOT, "benchmarks", "fair_bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_programs_compile(programs):
    for name, path in programs.items():
        assert os.path.exists(path) and os.access(path, os.X_OK), name


def test_bench_refuses_bad_arguments(programs):
    """benchmarks/tests/kvx_bench_cli_test.py:43-47 and benchmarks/kvx_bench.cu:193-203 of the
    reference: a non-positive count, more written tokens than the sequence has, an unknown dtype."""
    exe = programs["kvx_bench"]
    for bad in (["--seq-count", "0"], ["--seq-len", "4", "--tokens-per-seq", "5"], ["--dtype=float64"],
                ["--iters=0"], ["--layout", "dhn"], ["--gpus", "3"]):
        proc = subprocess.run([exe] + bad, text=True, capture_output=True)
        assert proc.returncode != 0, bad
        assert "write," not in proc.stdout


def test_slot_mapping_of_the_comparison_script():
    fb = _fair_bench()
    for seq_count, seq_len, block_size, tps in ((2, 8, 4, 1), (2, 8, 4, 2), (4, 16, 8, 4), (1, 8, 16, 1), (2, 8, 4, 8)):
        slots = fb.build_kvx_like_slot_mapping(seq_count, seq_len, block_size, tps, device="cpu")
        assert slots.numel() == seq_count * tps
        pages = seq_count * ((seq_len + block_size - 1) // block_size)
        assert int(slots.max()) < pages * block_size and bool((slots >= 0).all())
        # the last tps positions of every sequence, sequence s on pages s * pages_per_seq ...
        want = [(s * (pages // seq_count) + p // block_size) * block_size + p % block_size
                for s in range(seq_count) for p in range(seq_len - tps, seq_len)]
        assert slots.tolist() == want
    with pytest.raises(ValueError):
        fb.build_kvx_like_slot_mapping(2, 8, 4, 9, device="cpu")
    assert len(fb.CASES) == 8


def _csv(stdout):
    lines = stdout.splitlines()
    head = next(l for l in lines if l.startswith("kernel,")).split(",")
    return {l.split(",")[0]: dict(zip(head, l.split(","))) for l in lines if l.startswith(("write,", "gather,"))}


@pytest.mark.gpu
def test_kernel_test_program_passes(programs):
    proc = subprocess.run([programs["kvx_kernel_test"]], text=True, capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "kvx_kernel_test passed" in proc.stdout
    records = [l for l in proc.stderr.splitlines() if l.endswith(": ok") or l.endswith(": fail")]
    assert len(records) == 11 and all(l.endswith(": ok") for l in records), records
    for name in ("write_f32", "write_f16", "write_bf16", "prefill_f32", "prefill_f16", "prefill_bf16",
                 "gather_f32", "gather_f16", "gather_bf16"):   # the reference's nine
        assert f"{name}: ok" in proc.stderr


@pytest.mark.gpu
def test_bench_program_keeps_the_reference_contract(programs):
    """The call of benchmarks/tests/kvx_bench_cli_test.py: arguments reflected in the `write,` line,
    13 leading columns in the reference's order."""
    exe = programs["kvx_bench"]
    proc = subprocess.run([exe, "--seq-count", "2", "--seq-len", "8", "--tokens-per-seq", "2", "--block-size", "4",
                           "--num-heads", "2", "--head-dim", "4", "--iters", "1", "--warmup", "1", "--dtype=float32",
                           "--check"], text=True, capture_output=True, timeout=300)
    assert proc.returncode == 0, proc.stderr
    line = next(l for l in proc.stdout.splitlines() if l.startswith("write,")).split(",")
    assert len(line) >= 13
    assert (int(line[1]), int(line[2]), int(line[3]), int(line[12])) == (2, 8, 4, 2)
    assert float(line[9]) > 0 and float(line[10]) > 0
    rows = _csv(proc.stdout)
    assert rows["write"]["checked"] == "1" and rows["gather"]["checked"] == "1"
    assert proc.stdout.splitlines()[0].startswith("write: ") and proc.stdout.splitlines()[1].startswith("gather: ")


@pytest.mark.gpu
@pytest.mark.parametrize("args", [
    ["--config", "c1", "--layers", "2", "--check"],
    ["--config", "c1", "--layout", "hnd", "--check"],
    ["--config", "c1", "--layout", "paged", "--check"],
    ["--config", "c2", "--pool-blocks", "9000", "--iters", "3", "--warmup", "1", "--check"],
    ["--config", "c2", "--pool-blocks", "9000", "--layout", "packed", "--iters", "3", "--warmup", "1", "--check"],
    ["--config", "c5", "--iters", "2", "--warmup", "1"],
])
def test_bench_program_configurations(programs, args):
    peak = 6548.5
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]
    except Exception:
        pass
    proc = subprocess.run([programs["kvx_bench"], "--peak-gbs", str(peak)] + args, text=True, capture_output=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    rows = _csv(proc.stdout)
    for kernel in ("write", "gather"):
        r = rows[kernel]
        assert float(r["gbs"]) > 0 and float(r["pct_of_8000"]) > 0 and float(r["pct_of_peak"]) > 0
        assert int(r["valid_tokens"]) > 0 and r["gpus"] == "1"
        if "--check" in args:
            assert r["checked"] == "1", r


@pytest.mark.gpu
def test_bench_program_shards_over_two_devices(programs):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("one CUDA device")
    proc = subprocess.run([programs["kvx_bench"], "--config", "c1", "--gpus", "2", "--check"], text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    rows = _csv(proc.stdout)
    assert rows["write"]["gpus"] == "2" and rows["write"]["checked"] == "1"


@pytest.mark.gpu
def test_comparison_script_prints_its_table(programs, tmp_path):
    out = tmp_path / "fair.csv"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "benchmarks", "fair_bench.py"), "--iters", "5", "--warmup", "2",
                           "--repeats", "1", "--bin-path", programs["kvx_bench"], "--output-csv", str(out), "--prefill"],
                          text=True, capture_output=True, timeout=900)
    assert proc.returncode == 0, (proc.stdout[-1500:], proc.stderr[-1500:])
    table = [l for l in proc.stdout.splitlines() if l.startswith("heads=") or l.startswith("llama3-8b")]
    assert len(table) == 9
    assert " NO" not in proc.stdout            # where vLLM's operator loads, the outputs are bit-identical
    import csv
    rows = list(csv.DictReader(open(out)))
    assert len(rows) == 9 and all(float(r["kvx_device_us_mean"]) > 0 for r in rows)
    assert all(float(r["native_ms_per_mean"]) > 0 for r in rows[:8])
