"""bench.py contract pieces that need no GPU: the reference arm always prints one JSON line and exits 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ref(n):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", str(n), "--steps", "4",
                        "--warmup", "3"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_reference_arm_reports_unavailable_for_gpu_counts_it_has_no_driver_for():
    for n in (2, 4):
        line = _ref(n)
        assert line["impl"] == "reference" and "unavailable" in line and line["n_gpus"] == n


def test_reference_arm_prints_a_line_even_when_its_binary_cannot_run_here():
    line = _ref(8)
    assert line["impl"] == "reference"
    assert "unavailable" in line or line.get("metric") == "decode_tok_per_s"


def test_bench_flags_parse():
    sys.path.insert(0, ROOT)
    import importlib
    b = importlib.import_module("bench")
    old = sys.argv
    try:
        sys.argv = ["bench.py", "--gpus", "8", "--steps", "16", "--warmup", "3", "--plan", "hybrid", "--tp", "2", "--hot-experts", "8"]
        a = b.parse_args()
    finally:
        sys.argv = old
    assert (a.gpus, a.steps, a.warmup, a.plan, a.tp, a.hot_experts) == (8, 16, 3, "hybrid", 2, 8)
    sys.argv = ["bench.py"]
    try:
        d = b.parse_args()
    finally:
        sys.argv = old
    assert d.gpus == 1 and d.impl == "ours" and d.model == "qwen3-235b-a22b" and d.plan == "tp"
    assert d.kv == "bf16" and d.steps_per_launch == 1                     # the headline keeps bf16 KV rows, one token per launch
