"""Strategy search: strategy-space goldens, golden search results on canned profiles, native vs Python DP."""
import glob
import json
import os

import numpy as np
import pytest

from hetu_galvatron_b200.config.model_config import model_layer_configs, model_name, resolve_model_config
from hetu_galvatron_b200.config.schema import GalvatronSearchArgs
from hetu_galvatron_b200.search.dp import DPAlg, load_native_core
from hetu_galvatron_b200.search.engine import GalvatronSearchEngine
from hetu_galvatron_b200.search.strategy import strategies_from_config

FIX = json.load(open(os.path.join(os.path.dirname(__file__), "fixtures", "search_profiles.json")))


def write_profiles(tmp, model, time_mode, memory_mode, sp):
    cfg, hw, out = tmp / "configs", tmp / "hardware", tmp / "output"
    for d in (cfg, hw, out):
        d.mkdir(exist_ok=True)
    json.dump(FIX["%s_time_config" % time_mode], open(cfg / ("computation_profiling_bf16_%s_all.json" % model), "w"))
    mem_key = {"static": "static_memory_config_sp" if sp else "static_memory_config",
               "sequence": "sequence_memory_config_sp"}[memory_mode]
    json.dump(FIX[mem_key], open(cfg / ("memory_profiling_bf16_%s_all.json" % model), "w"))
    h = FIX["hardware_configs"]
    json.dump(h["allreduce"], open(hw / "allreduce_bandwidth_1nodes_8gpus_per_node.json", "w"))
    json.dump(h["p2p"], open(hw / "p2p_bandwidth_1nodes_8gpus_per_node.json", "w"))
    json.dump(h["overlap"], open(hw / "overlap_coefficient.json", "w"))
    json.dump(h["sp"], open(hw / "sp_time_1nodes_8gpus_per_node.json", "w"))
    return cfg, hw, out


def make_engine(tmp, time_mode="static", memory_mode="static", sp=False, seqlen=None, **kw):
    args = GalvatronSearchArgs()
    args.model_info.model_config_path = "llama2-7b"
    for key, val in kw.items():
        for section in (args.batch_size_info, args.hardware_info, args.parallelism_info, args.common_train_info,
                        args.options_info, args.search_space_info, args.model_info):
            if key in type(section).model_fields:
                setattr(section, key, val)
                break
        else:
            raise KeyError(key)
    resolve_model_config(args)
    name = model_name(args)
    cfg, hw, out = write_profiles(tmp, name, time_mode, memory_mode, sp)
    p = args.profiling_info
    p.memory_profiling_path = p.time_profiling_path = str(cfg)
    p.allreduce_bandwidth_config_path = p.p2p_bandwidth_config_path = p.overlap_coe_path = p.sp_time_path = str(hw)
    p.time_profile_mode, p.memory_profile_mode = time_mode, memory_mode
    args.common_train_info.sequence_parallel = sp
    args.options_info.log_dir = str(tmp / "logs")
    args.options_info.output_config_path = str(out)
    eng = GalvatronSearchEngine(args)
    eng.verbose = False
    eng.set_search_engine_info(str(cfg), model_layer_configs(args), name)
    if seqlen is not None:
        eng.seqlen_list = seqlen
    eng.initialize_search_engine()
    return eng, out


def test_strategy_space_for_8_gpus(tmp_path):
    eng, _ = make_engine(tmp_path, seqlen=[4096], default_dp_type="zero2")
    got = ", ".join(s.to_simple_string() for s in eng.layer_strategy_list)
    expect = ("1-1-8, 1-1-8-c, 1-1-8f, 1-1-8f-c, 1-2*-4-sp, 1-2*-4-c-sp, 1-2*-4f-sp, 1-2*-4f-c-sp, 1-4*-2-sp, "
              "1-4*-2-c-sp, 1-4*-2f-sp, 1-4*-2f-c-sp, 1-8*-1-sp, 1-8*-1-c-sp, 1-2*-4, 1-2*-4-c, 1-2*-4f, 1-2*-4f-c, "
              "1-4*-2, 1-4*-2-c, 1-4*-2f, 1-4*-2f-c, 1-8*-1, 1-8*-1-c, 2-1-4, 2-1-4-c, 2-1-4f, 2-1-4f-c, 2-2*-2-sp, "
              "2-2*-2-c-sp, 2-2*-2f-sp, 2-2*-2f-c-sp, 2-4*-1-sp, 2-4*-1-c-sp, 2-2*-2, 2-2*-2-c, 2-2*-2f, 2-2*-2f-c, "
              "2-4*-1, 2-4*-1-c, 4-1-2, 4-1-2-c, 4-1-2f, 4-1-2f-c, 4-2*-1-sp, 4-2*-1-c-sp, 4-2*-1, 4-2*-1-c, 8-1-1, "
              "8-1-1-c")
    assert len(eng.layer_strategy_list) == 50
    assert got == expect


@pytest.mark.parametrize("chunk,fine,throughput,vtp,embed_sdp", [
    (32, 1, 2.6485091403918064, 8, 0),
    (8, 0, 2.5246283459057333, 1, 1),
])
def test_golden_search(tmp_path, chunk, fine, throughput, vtp, embed_sdp):
    eng, out = make_engine(tmp_path, "sequence", "sequence", True, [8192], settle_bsz=64, settle_chunk=chunk,
                           memory_constraint=36, default_dp_type="zero2", pipeline_type="pipedream_flush",
                           async_grad_reduce=False, fine_grained_mode=fine, num_layers=28)
    got = eng.parallelism_optimization()
    assert abs(got - throughput) < 1e-6
    files = glob.glob(os.path.join(out, "galvatron_config_*.json"))
    assert len(files) == 1
    cfg = json.load(open(files[0]))
    for k in ("pp_deg", "tp_sizes_enc", "tp_consecutive_flags", "dp_types_enc", "use_sp", "checkpoint", "global_bsz",
              "chunks", "pp_division", "pipeline_type", "default_dp_type", "vtp", "vsp"):
        assert k in cfg
    assert (cfg["pp_deg"], cfg["global_bsz"], cfg["chunks"], cfg["pp_division"]) == (1, 64, chunk, "28")
    assert (cfg["vtp"], cfg["vsp"], cfg["embed_sdp"]) == (vtp, 0, embed_sdp)
    names = [s.to_simple_string() for s in strategies_from_config(cfg, "zero2")]
    if fine:
        assert names == ["1-4*-2f-c"] * 14 + ["1-4*-2f"] * 12 + ["1-4*-2"] * 2
    else:
        assert names == ["1-1-8f-c"] * 28


def test_native_dp_core_matches_python():
    assert load_native_core() is not None, "the native dp core must build"
    rng = np.random.default_rng(0)
    L, S, M = 6, 5, 300
    v = rng.integers(5, 60, size=(L, S)).astype(np.int32)
    intra = rng.random((L, S))
    inter = rng.random((L, S, S)) * 0.1
    inter[0] = 0
    other_mem, other_time = {1: 20, 2: 45, 4: 290}, {1: 0.5, 2: 0.25, 4: 0.1}
    outs = []
    for native, threads in ((False, 1), (True, 1), (True, 4)):
        alg = DPAlg(M, other_mem, other_time, L, S, use_cpp_core=native, threads=threads)
        alg.set_v_and_cost(v, intra, inter)
        outs.append(alg.fit())
    for total, res, remain in outs[1:]:
        for k in other_mem:
            assert total[k] == outs[0][0][k] or (np.isinf(total[k]) and np.isinf(outs[0][0][k]))
            assert [int(x) for x in res[k]] == [int(x) for x in outs[0][1][k]]
            assert int(remain[k]) == int(outs[0][2][k])


def test_memory_balanced_stage_division():
    from hetu_galvatron_b200.search.engine import balance_stages, pp_division_even

    # a heavy first stage (embedding) pushes layers to the later stages; nothing is left empty
    div, cost = balance_stages([10.0] * 12, [35.0, 0.0, 0.0, 15.0], 4)
    assert sum(div) == 12 and min(div) >= 1 and div[0] < div[1]
    assert max(cost) <= 1.3 * (120 + 50) / 4 + 10.0
    # uniform costs without extras reproduce the even split
    div, _ = balance_stages([1.0] * 8, [0.0] * 4, 4)
    assert div == pp_division_even([8], 4)
    # more stages than a greedy fill would populate: every stage still gets a layer
    div, _ = balance_stages([5.0, 1.0, 1.0, 1.0], [0.0, 0.0, 0.0, 0.0], 4)
    assert div == [1, 1, 1, 1]


def test_shipped_b200_profiles_reproduce_the_shipped_plan(tmp_path, monkeypatch):
    """The B200 hardware profile, model profiles and refit under ``cli/`` give the strategy file that ships beside them
    (search space cut to the data-parallel strategies, which contain the optimum, to keep the test short)."""
    import hetu_galvatron_b200.cli as cli_pkg
    from hetu_galvatron_b200.cli import search_dist

    cli = os.path.dirname(cli_pkg.__file__)
    monkeypatch.setenv("HG_PROFILE_DIR", cli)
    thr = search_dist.main([os.path.join(cli, "configs", "search_dist.yaml"),
                            "search_engine.search_space_info.max_pp_deg=1", "search_engine.search_space_info.max_tp_deg=1",
                            "search_engine.search_space_info.max_sp_deg=1",
                            "search_engine.options_info.output_config_path=%s" % tmp_path,
                            "search_engine.options_info.log_dir=%s" % tmp_path])
    assert 1.2 < 64 / thr < 1.6                                   # seconds per iteration of 64 sequences on 8 GPUs
    name = "galvatron_config_llama2-7b_1nodes_8gpus_per_node_160GB_bf16.json"
    got = json.load(open(tmp_path / name))
    shipped = json.load(open(os.path.join(cli, "configs", name)))
    assert got == shipped
