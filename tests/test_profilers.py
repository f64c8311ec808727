"""Model profiler (sweeps, command lists, post-processing against the reference's golden outputs), hardware
profiler (script generation, key names, a 2-rank sweep on CPU ranks) and the profile / search entry points."""
import json
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tests.dist_utils import run_distributed, worker_main  # noqa: E402

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fixtures")


def _profiler(tmp, **upd):
    from hetu_galvatron_b200.config.schema import GalvatronModelProfilerArgs
    from hetu_galvatron_b200.profiler.model import ModelProfiler

    upd.setdefault("runtime_yaml_template_path", "configs/profile_runtime.yaml")
    p = ModelProfiler(GalvatronModelProfilerArgs(**upd))
    p.set_profiler_launcher(str(tmp), "llama_search")
    return p


def test_sweep_lists(tmp_path):
    p = _profiler(tmp_path, profile_type="computation", profile_mode="sequence", profile_fixed_batch_size=1,
                  profile_min_seq_length=128, profile_max_seq_length=512, profile_seq_length_step=128)
    assert [t[0] for t in p.get_seq_length_tuple_list()] == [128, 256, 384, 512]
    p = _profiler(tmp_path, profile_type="memory", profile_mode="sequence", profile_fixed_batch_size=8,
                  profile_min_seq_length=128, profile_max_seq_length=512)
    assert [t[0] for t in p.get_seq_length_tuple_list()] == [128, 256, 512]
    p = _profiler(tmp_path, profile_mode="batch", profile_min_batch_size=16, profile_max_batch_size=64,
                  profile_batch_size_step=16)
    assert p.get_global_batch_size_list() == [16, 32, 48, 64]


@pytest.mark.parametrize("kind,mode,upd,count", [
    ("memory", "static", dict(profile_fixed_batch_size=8, profile_fixed_seq_length_list=[4096]), 24),
    ("memory", "sequence", dict(profile_fixed_batch_size=8, profile_min_seq_length=128, profile_max_seq_length=512), 18),
    ("computation", "static", dict(profile_fixed_batch_size=32, profile_fixed_seq_length_list=[4096]), 2),
    ("computation", "batch", dict(profile_min_batch_size=16, profile_max_batch_size=32, profile_batch_size_step=16,
                                  profile_fixed_seq_length_list=[4096]), 4),
    ("computation", "sequence", dict(profile_fixed_batch_size=8, profile_min_seq_length=128, profile_max_seq_length=512,
                                     profile_seq_length_step=128), 8),
])
def test_command_lists(tmp_path, monkeypatch, kind, mode, upd, count):
    monkeypatch.setenv("NUM_NODES", "1")
    monkeypatch.setenv("NUM_GPUS_PER_NODE", "8")
    monkeypatch.setenv("RUNTIME_LAUNCHER", "echo")
    p = _profiler(tmp_path, profile_type=kind, profile_mode=mode, **upd)
    ran = []
    cmds = p.launch_profiling_scripts(run=lambda c: ran.append(c) or 0)
    assert len(cmds) == count == len(ran)
    assert all("runtime.profile.profile=1" in c and "runtime.model.num_layers=" in c for c in cmds)
    # scripts_only writes the same list to a shell file
    p2 = _profiler(tmp_path, profile_type=kind, profile_mode=mode, profile_flow_control="scripts_only", **upd)
    p2.launch_profiling_scripts(run=lambda c: pytest.fail("must not launch"))
    script = tmp_path / "scripts" / ("%s_profile_scripts_all.sh" % kind)
    assert script.read_text().count("sleep 1") == count


def _same(a, b, path=""):
    if isinstance(b, dict):
        for k, v in b.items():
            assert str(k) in {str(x) for x in a}, (path, k)
            _same({str(x): y for x, y in a.items()}[str(k)], v, path + "/" + str(k))
    else:
        assert abs(a - b) < 1e-6, (path, a, b)


@pytest.mark.parametrize("kind,mode,upd,raw_key,gold_key", [
    ("computation", "static", dict(profile_fixed_batch_size=8, profile_layernum_min=2, profile_layernum_max=4,
                                   profile_fixed_seq_length_list=[4096]), "computation_static_config", "static_time_config"),
    ("computation", "batch", dict(profile_min_batch_size=1, profile_max_batch_size=10, profile_batch_size_step=1,
                                  profile_layernum_min=2, profile_layernum_max=4, profile_fixed_seq_length_list=[4096]),
     "computation_batch_config", "batch_time_config"),
    ("computation", "sequence", dict(profile_fixed_batch_size=1, profile_min_seq_length=4096, profile_max_seq_length=32768,
                                     profile_seq_length_step=4096, profile_layernum_min=1, profile_layernum_max=2),
     "computation_sequence_config", "sequence_time_config"),
    ("memory", "static", dict(profile_fixed_batch_size=8, sequence_parallel=False, profile_fixed_seq_length_list=[4096]),
     "memory_static_config", "static_memory_config"),
    ("memory", "static", dict(profile_fixed_batch_size=8, sequence_parallel=True, profile_fixed_seq_length_list=[4096]),
     "memory_static_config_sp", "static_memory_config_sp"),
    ("memory", "sequence", dict(profile_fixed_batch_size=8, profile_min_seq_length=512, profile_max_seq_length=8192,
                                sequence_parallel=True), "memory_sequence_config_sp", "sequence_memory_config_sp"),
])
def test_post_processing_reproduces_reference_outputs(tmp_path, monkeypatch, kind, mode, upd, raw_key, gold_key):
    monkeypatch.setenv("NUM_NODES", "1")
    monkeypatch.setenv("NUM_GPUS_PER_NODE", "8")
    raw = json.load(open(os.path.join(FIX, "profiler_raw.json")))[raw_key]
    gold = json.load(open(os.path.join(FIX, "search_profiles.json")))[gold_key]
    p = _profiler(tmp_path, profile_type=kind, profile_mode=mode, **upd)
    path = p.time_profiling_path() if kind == "computation" else p.memory_profiling_path()
    os.makedirs(os.path.dirname(path), exist_ok=True)
    json.dump(raw, open(path, "w"))
    p.process_profiled_data()
    _same(json.load(open(path)), gold)


# ---- hardware profiler ----------------------------------------------------------------------------------------------
def test_hardware_scripts_and_sweeps(tmp_path):
    from hetu_galvatron_b200.config.schema import ProfilerHardwareArgs
    from hetu_galvatron_b200.profiler import hardware as hw

    assert hw.halving_degrees(8, 8) == [8, 4, 2] and hw.halving_degrees(16, 8) == [8, 4, 2]
    assert hw.halving_batch_sizes(8) == [8, 4, 2, 1] and hw.pp_degree_sweep(8, 4) == [2, 4]
    assert hw.bandwidth_jobs(8, [8, 4, 2]) == [(8, 1), (4, 1), (4, 0), (2, 1), (2, 0)]
    prof = hw.HardwareProfiler(ProfilerHardwareArgs(envs=["export NCCL_DEBUG=WARN"]))
    prof.set_path(str(tmp_path))
    prof.profile_bandwidth()
    prof.profile_sp_bandwidth()
    d = tmp_path / "scripts"
    ar = (d / "profile_allreduce.sh").read_text()
    assert "export NUM_GPUS_PER_NODE=8" in ar and "--global_tp_deg 8 4 2" in ar and "--profile_time 0" in ar
    assert "--pp_deg 2 4 8" in (d / "profile_p2p.sh").read_text()
    sp = (d / "profile_allreduce_sp.sh").read_text()
    assert "--local_batch_size 1024 512 256 128 64 32 16 8 4 2 1" in sp and "--profile_time 1" in sp
    assert "all2all" in (d / "profile_all2all_sp.sh").read_text()
    ran = []
    prof.profile_overlap(run=lambda c: ran.append(c) or 0)
    assert "overlap" in ran[0] and "--overlap_time_multiply 4" in ran[0]


def hw_sweep(payload):
    from hetu_galvatron_b200.profiler import hardware as hw

    out = payload["out"]
    res = {}
    res.update(hw.profile_allreduce([2], [1], 0, out, 1, 2, measurements=6, seq=64, hidden=64))
    res.update(hw.profile_allreduce([2], [2, 1], 1, out, 1, 2, measurements=6, seq=64, hidden=64))
    res.update(hw.profile_all2all([2], [1], out, 1, 2, measurements=6, seq=64, hidden=64))
    res.update(hw.profile_p2p([2], out, 1, 2, batch_size=1, measurements=6, seq=64, hidden=64))
    res["overlap_coe"] = hw.profile_overlap(out, 2, n=64, iters=2)
    return res


REGISTRY = {"hw_sweep": hw_sweep}


def test_hardware_sweep_on_two_cpu_ranks(tmp_path):
    res = run_distributed(__file__, "hw_sweep", 2, {"out": str(tmp_path)}, timeout=180)
    for key in ("allreduce_size_2_consec_1", "allreduce_size_2_2MB_time", "allreduce_size_2_1MB_time",
                "all2all_size_2_1MB_time", "pp_size_2", "overlap_coe"):
        assert res[0][key] > 0, key
    bw = json.load(open(tmp_path / "allreduce_bandwidth_1nodes_2gpus_per_node.json"))
    assert list(bw) == ["allreduce_size_2_consec_1"]
    sp = json.load(open(tmp_path / "sp_time_1nodes_2gpus_per_node.json"))
    assert set(sp) == {"allreduce_size_2_2MB_time", "allreduce_size_2_1MB_time", "all2all_size_2_1MB_time"}
    assert "pp_size_2" in json.load(open(tmp_path / "p2p_bandwidth_1nodes_2gpus_per_node.json"))
    assert json.load(open(tmp_path / "overlap_coefficient.json"))["overlap_coe"] >= 1.0
    # the files are what the search engine's readers expect
    from hetu_galvatron_b200.utils.config_utils import read_allreduce_bandwidth_config, read_p2p_bandwidth_config, remap_config

    b, c = read_allreduce_bandwidth_config(bw, 2)
    assert "2_1" in b and c["1"] == 0
    assert 2 in read_p2p_bandwidth_config(str(tmp_path / "p2p_bandwidth_1nodes_2gpus_per_node.json"))[0]
    assert "popt" in remap_config(sp, "allreduce")[2]


def test_profile_entry_points(tmp_path, monkeypatch):
    from hetu_galvatron_b200.cli import profile_hardware, profiler

    cfg = os.path.join(os.path.dirname(FIX), "..", "hetu_galvatron_b200", "cli", "configs")
    monkeypatch.setenv("HG_PROFILE_DIR", str(tmp_path))
    monkeypatch.setenv("NUM_NODES", "1")
    monkeypatch.setenv("NUM_GPUS_PER_NODE", "8")
    monkeypatch.setenv("RUNTIME_LAUNCHER", "echo")
    p = profiler.main([os.path.join(cfg, "profile_memory.yaml"), "model_profiler.profile_flow_control=scripts_only"])
    assert (tmp_path / "scripts" / "memory_profile_scripts_all.sh").exists() and p.model_name
    profile_hardware.main([os.path.join(cfg, "profile_hardware.yaml")], run_overlap=False)
    assert (tmp_path / "scripts" / "profile_allreduce.sh").exists()


def test_refit_ratio_and_optimizer_term():
    from hetu_galvatron_b200.profiler import refit
    from hetu_galvatron_b200.search.cost_model import (LayerTimeCost, ModelArgs, ParallelArgs, ProfileHardwareArgs,
                                                       ProfileModelArgs, TrainArgs)
    from hetu_galvatron_b200.search.strategy import DPType, LayerStrategy

    fwd = {"layernum2_bsz2_seq4096": 10.0, "layernum4_bsz2_seq4096": 18.0}
    full = {"layernum2_bsz2_seq4096": 40.0, "layernum4_bsz2_seq4096": 70.0}
    assert refit.ratio_from_times(fwd, full, 2, 4, 2, 4096) == pytest.approx(30.0 / 8.0 - 1.0)
    assert refit.ratio_from_times(fwd, full, 2, 4, 2, 4096, optimizer_ms=1.0) == pytest.approx(28.0 / 8.0 - 1.0)
    with pytest.raises(ValueError):
        refit.ratio_from_times(fwd, fwd, 2, 4, 2, 4096)
    # 18 bytes of state per parameter are streamed as 34 bytes per step
    assert refit.optimizer_ms_per_layer(900.0, 6500.0) == pytest.approx(3600.0 * 34 / 18 / 1024 / 6500 * 1e3)
    # the per-step term from one and two micro-batches per step: d1 = x + o = 13, d2 = 2x + o = 24 -> o = 2
    full2 = {"layernum2_bsz2_seq4096": 30.0, "layernum4_bsz2_seq4096": 56.0,
             "layernum2_bsz4_seq4096": 50.0, "layernum4_bsz4_seq4096": 98.0}
    assert refit.optimizer_ms_from_accumulation(full2, 2, 4, 2, 4096) == pytest.approx(2.0)
    assert refit.optimizer_ms_from_accumulation(full, 2, 4, 2, 4096) is None

    def cost(opt_ms, ratio, dp_type, dp):
        hw = ProfileHardwareArgs(allreduce_latency_per_MB_dict={"%d_1" % dp: 0.0, "%d_0" % dp: 0.0, "1_1": 0.0},
                                 optimizer_ms_per_layer=opt_ms)
        pm = ProfileModelArgs(forward_computation_time=2.0, backward_forward_ratio=ratio)
        st = LayerStrategy(pp_size=1, tp_size=1, sp_size=1, dp_size=dp, dp_type=dp_type, checkpoint=False)
        return LayerTimeCost(st, 8 * dp, 1, ModelArgs(parameter_size=48, seq_length=1024, hidden_size=1024, layer_num=4),
                             TrainArgs(), ParallelArgs(), pm, hw).gen_result()[0]

    base = cost(0.0, 2.0, DPType.DDP, 1)
    assert cost(0.0, 3.0, DPType.DDP, 1) == pytest.approx(base * 4.0 / 3.0)       # fwd * (1 + ratio)
    assert cost(1.0, 2.0, DPType.DDP, 1) == pytest.approx(base + 1e-3)            # + 1 ms per layer, unsharded
    assert cost(8.0, 2.0, DPType.ZERO2, 8) - cost(0.0, 2.0, DPType.ZERO2, 8) == pytest.approx(1e-3)  # / sdp under ZeRO


RUNTIME_YAML = """
runtime:
  parallel: {mixed_precision: fp32}
  model: {model_size: llama-test, hidden_size: 64, num_layers: 2, num_attention_heads: 4, ffn_hidden_size: 128,
          vocab_size: 512, normalization: RMSNorm, gated_linear_unit: true, activation_func: torch.nn.functional.silu}
  profile: {profile: 1}
  train: {train_iters: 25, lr: 1.0e-3, global_batch_size: 2, chunks: 1, seq_length: 32}
  data: {use_random_dataset: true}
"""
PROFILE_YAML = """
model_profiler:
  profile_type: computation
  profile_mode: static
  profile_mixed_precision: fp32
  profile_fixed_batch_size: 2
  profile_fixed_seq_length_list: [32]
  profile_layernum_min: 1
  profile_layernum_max: 3
  runtime_yaml_template_path: %s
  model_info: {model_size: llama-test, hidden_size: 64, num_attention_heads: 4, vocab_size: 512}
"""


def test_computation_profiling_end_to_end_on_cpu(tmp_path):
    """The whole flow: the model profiler launches two forward-only training runs (1 and 3 layers) through the
    training entry point, each writes its raw time, and post-processing derives the per-layer numbers."""
    import subprocess

    rt = tmp_path / "runtime.yaml"
    rt.write_text(RUNTIME_YAML)
    pf = tmp_path / "profile.yaml"
    pf.write_text(PROFILE_YAML % rt)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, HG_QUIET="1", HG_PROFILE_DIR=str(tmp_path), PYTHONPATH=root, OMP_NUM_THREADS="2",
               RUNTIME_LAUNCHER="%s -m hetu_galvatron_b200.cli.train_dist" % sys.executable)
    r = subprocess.run([sys.executable, "-m", "hetu_galvatron_b200.cli.profiler", str(pf)], env=env, cwd=str(tmp_path),
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    out = json.load(open(tmp_path / "configs" / "computation_profiling_fp32_llama-test_all.json"))
    assert out["layernum1_bsz2_seq32"] > 0 and out["layernum3_bsz2_seq32"] > out["layernum1_bsz2_seq32"]
    assert out["layertype_0_bsz2_seq32"] > 0 and out["layertype_other_bsz2_seq32"] >= 0


if __name__ == "__main__":
    worker_main(REGISTRY)
