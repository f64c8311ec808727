"""The parts of the benchmark contract that need no GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_and_exits_zero():
    """Either the reference's own result line or ``{"impl": "reference", "unavailable": "<why>"}``; never a crash."""
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1",
                        "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out["impl"] == "reference"
    assert ("unavailable" in out and isinstance(out["unavailable"], str) and "\n" not in out["unavailable"]) or "value" in out


def test_bench_defaults_and_flags():
    sys.path.insert(0, ROOT)
    import importlib

    bench = importlib.import_module("bench")
    src = open(os.path.join(ROOT, "bench.py")).read()
    for flag in ("--gpus", "--steps", "--warmup", "--impl"):
        assert flag in src
    # the model of the headline configuration
    assert bench.MODEL["hidden_size"] == 4096 and bench.MODEL["num_layers"] == 32 and bench.SEQ == 4096


def test_graft_entry_exposes_build_and_smoke():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as g

    assert callable(g.build) and callable(g.smoke)
