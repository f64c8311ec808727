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


def test_both_arms_run_the_same_searched_plan():
    """The plan of a run comes from the strategy JSON the search wrote for that GPU count; the reference arm's overrides
    carry the same micro-batching and data-parallel type, and every shipped plan matches the benchmark's batch."""
    import argparse

    sys.path.insert(0, ROOT)
    import bench
    from baseline import reference_arm as ra

    a = argparse.Namespace(warmup=3, steps=4, seq=4096, micro_batch=None, dp_type="zero2", layers=0, checkpoint=0,
                           strategy=None, pp=1, tp=1)
    for n in (1, 2, 4, 8):
        cfg, path, chunks, dp_type = bench.plan_knobs(n, a)
        assert cfg is not None and path.endswith("%dgpus_per_node_160GB_bf16.json" % n)
        assert cfg["global_bsz"] == bench.PER_GPU_BATCH * n and chunks == cfg["chunks"]
        assert cfg.get("predicted_time_cost", 0) > 0
        ov = ra.overrides_for(a, n, "/tmp/tok")
        assert "runtime.train.chunks=%d" % chunks in ov
        assert "runtime.parallel.default_dp_type=%s" % dp_type in ov
        assert "runtime.train.global_batch_size=%d" % (8 * n) in ov
    # debugging overrides fall back to plain flags but keep the searched micro-batching
    a.layers = 8
    cfg, _, chunks, _ = bench.plan_knobs(8, a)
    assert cfg is None and chunks == 2
