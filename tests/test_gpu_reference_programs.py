"""The reference project's own GPU programs, compiled unmodified (oracle/build.py) and linked
against THIS library instead of the reference kernels:

* its kernel test (tests/kvx_kernel_test.cu) must print "kvx_kernel_test passed";
* its micro-benchmark (benchmarks/kvx_bench.cu) must run the eight cases of its comparison
  script (benchmarks/fair_bench.py:176-185) and keep the CSV contract its tools parse
  (benchmarks/tests/kvx_bench_cli_test.py: a `write,` line of >= 13 fields reflecting the
  arguments).  Timings of both builds are written to the folder named by KVX_RESULTS_DIR, when set.

Skipped where the binaries were not built (no reference checkout at build time)."""
import json
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")

FAIR_CASES = [
    dict(num_heads=8, seq_count=1, seq_len=128), dict(num_heads=8, seq_count=8, seq_len=512),
    dict(num_heads=8, seq_count=32, seq_len=128), dict(num_heads=32, seq_count=1, seq_len=128),
    dict(num_heads=32, seq_count=8, seq_len=512), dict(num_heads=32, seq_count=16, seq_len=1024),
    dict(num_heads=8, seq_count=8, seq_len=512, tokens_per_seq=16),
    dict(num_heads=32, seq_count=8, seq_len=1024, tokens_per_seq=32),
]


def _exe(name):
    path = os.path.join(REF_DIR, name)
    if not os.path.exists(path):
        pytest.skip(f"{name} was not built")
    return path


def _bench(exe, case, dtype, iters=200, warmup=20):
    cmd = [exe, "--seq-count", str(case["seq_count"]), "--seq-len", str(case["seq_len"]),
           "--tokens-per-seq", str(case.get("tokens_per_seq", 1)), "--block-size", "16",
           "--num-heads", str(case["num_heads"]), "--head-dim", "128", "--iters", str(iters),
           "--warmup", str(warmup), "--dtype", dtype]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr[-500:]
    lines = {l.split(",")[0]: l.split(",") for l in p.stdout.splitlines() if l.startswith(("write,", "gather,"))}
    assert "write" in lines and "gather" in lines
    return lines


def test_reference_kernel_test_program_passes_on_this_library():
    p = subprocess.run([_exe("kvx_kernel_test_ours")], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout[-500:] + p.stderr[-1500:]
    assert "kvx_kernel_test passed" in p.stdout


def test_reference_bench_program_runs_on_this_library_and_keeps_its_csv_contract():
    ours, ref = _exe("kvx_bench_ours"), _exe("kvx_bench_ref")
    rows = []
    for dtype in ("bfloat16", "float16", "float32"):
        for case in FAIR_CASES:
            a, b = _bench(ours, case, dtype), _bench(ref, case, dtype)
            w = a["write"]
            assert len(w) >= 13
            assert int(w[1]) == case["seq_count"] and int(w[2]) == case["seq_len"] and int(w[4]) == case["num_heads"]
            assert int(w[12]) == case.get("tokens_per_seq", 1)
            assert float(w[9]) > 0 and float(w[10]) > 0
            rows.append({"dtype": dtype, **case,
                         "write_us": {"this": float(a["write"][9]) * 1e3, "reference": float(b["write"][9]) * 1e3},
                         "gather_us": {"this": float(a["gather"][9]) * 1e3, "reference": float(b["gather"][9]) * 1e3}})
    out_dir = os.environ.get("KVX_RESULTS_DIR", "")
    if out_dir and os.path.isdir(out_dir):
        with open(os.path.join(out_dir, "fair_bench_programs.json"), "w") as f:
            json.dump(rows, f, indent=1)
    # bad arguments still make the program fail (benchmarks/tests/kvx_bench_cli_test.py:44-53)
    bad = subprocess.run([ours, "--seq-count", "0"], capture_output=True, text=True, timeout=60)
    assert bad.returncode != 0
