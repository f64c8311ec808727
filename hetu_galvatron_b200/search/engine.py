"""Strategy search engine: enumerate -> filter -> load profiles -> cost models -> task sweep -> JSON.

    engine = GalvatronSearchEngine(args)                       # args: GalvatronSearchArgs
    engine.set_search_engine_info(path, model_layer_configs(args), model_name(args))
    engine.initialize_search_engine()
    throughput = engine.parallelism_optimization()            # writes galvatron_config_*.json

Capability parity: galvatron/core/search_engine/search_engine.py:22-103 (setup), :106-255 (strategy
space), :286-462 (profile ingestion: static / batch / sequence modes, bandwidth + latency tables),
:464-509 (cost-model bundles), :520-644 (task grid, optional thread pool, selection), :646-727 (one task),
:729-785 (batch sizes, output file), :788-899 (cost-model check), :954-1099 (pipeline divisions).
"""
from __future__ import annotations

import copy
import logging
import os
import threading
from typing import Any, Dict, List, Optional, Sequence, Union

import numpy as np
from scipy.optimize import curve_fit

from .cost_model import (LayerMemoryCost, ModelArgs, ParallelArgs, ProfileHardwareArgs, ProfileModelArgs, TrainArgs,
                         EmbeddingLMHeadMemoryCost, EmbeddingLMHeadTimeCost, pipeline_costmodel)
from .dp import DpOnModel
from .strategy import (AttentionStrategy, DPType, EmbeddingLMHeadStrategy, FFNStrategy, LayerStrategy, array2str,
                       format_strategy_list, is_power_of_two, read_json_config, strategy_list2config,
                       write_json_config)

TP_SP_MODES = ("tp_only", "sp_only", "tp_with_sp")


def _line(x, m, c):
    return m * x + c


def _quad(x, a, b, c):
    return a * x * x + b * x + c


def _int_keys(d):
    if isinstance(d, dict):
        return {(int(k) if isinstance(k, str) and k.isdigit() else k): _int_keys(v) for k, v in d.items()}
    return d


def num2str(num, name: str) -> str:
    if isinstance(num, (list, tuple)):
        return name + "_".join(str(v) for v in num)
    return "%s%s" % (name, num)


# ---- hardware profile readers --------------------------------------------------------------------------
def read_allreduce_bandwidth_config(config: Union[str, dict], gpu_num: int):
    """``allreduce_size_{n}_consec_{0|1}`` (MB/ms) -> ({key: bandwidth}, {key: ms per MB}); the full-world
    group has one layout, stored under ``n``, ``n_0`` and ``n_1``."""
    env = read_json_config(config) if isinstance(config, str) else config
    bw: Dict[str, float] = {}
    n = gpu_num
    if n >= 2:
        full = env["allreduce_size_%d_consec_1" % n]
        for key in ("%d" % n, "%d_1" % n, "%d_0" % n):
            bw[key] = full
    n //= 2
    while n >= 2:
        bw["%d_0" % n] = env["allreduce_size_%d_consec_0" % n]
        bw["%d_1" % n] = env["allreduce_size_%d_consec_1" % n]
        n //= 2
    coe = {k: 1.0 / v for k, v in bw.items()}
    for key in ("1", "1_1", "1_0"):
        bw[key], coe[key] = np.inf, 0
    return bw, coe


def read_p2p_bandwidth_config(config: Union[str, dict]):
    env = read_json_config(config) if isinstance(config, str) else config
    bw = {int(k.split("_")[-1]): v for k, v in env.items() if "pp_size_" in k}
    return bw, {k: 1.0 / v for k, v in bw.items()}


def _latency_tables(config: dict, prefix: str, factor: float, bytes_keys: bool):
    """``{prefix}_{n}_{m}MB_time`` -> {n: {size: ms, "popt": (slope, intercept)}}."""
    out: Dict[int, Dict] = {}
    for key, val in config.items():
        if key.startswith(prefix):
            parts = key.split("_")
            n, mb = int(parts[-3]), int(parts[-2][:-2])
            out.setdefault(n, {})[mb * 1024 * 1024 if bytes_keys else mb] = val * factor
    for n, table in out.items():
        xs = [(k // 1024 // 1024 if bytes_keys else k) for k in table]
        ys = list(table.values())
        if len(xs) < 8:
            raise AssertionError("need at least 8 message sizes in the %s profile of group size %d" % (prefix, n))
        table["popt"] = curve_fit(_line, xs, ys)[0]
    return out


def remap_config(config: dict, op: str):
    """Byte-keyed tables; all-reduce times are halved (all-gather / reduce-scatter equivalent)."""
    return _latency_tables(config, op, 0.5 if op == "allreduce" else 1.0, True)


def remap_config_for_latency(config: dict, op: str):
    prefix = {"allreduce": "allreduce_size", "all2all": "all2all_size", "allgather": "allreduce_size"}[op]
    return _latency_tables(config, prefix, 0.5 if op == "allgather" else 1.0, False)


def pp_division_even(layernum_list: Sequence[int], pp_deg: int) -> List[int]:
    total = int(np.sum(layernum_list))
    avg = total // pp_deg
    return [avg] * (pp_deg - 1) + [total - avg * (pp_deg - 1)]


def balance_stages(layer_costs: Sequence[float], other_costs: Sequence[float], pp_deg: int):
    """Split ``len(layer_costs)`` consecutive layers over ``pp_deg`` stages so that stage memory
    (``other_costs[stage]`` + its layers) is even: a stage takes layers until it is within half a layer of the
    average, no early stage may exceed 1.3x the average, and no stage is left empty.  Returns (division, stage costs)."""
    n = len(layer_costs)
    avg = (float(np.sum(layer_costs)) + float(np.sum(other_costs))) / pp_deg
    division = [0] * pp_deg
    acc = [float(x) for x in other_costs]
    idx = 0
    for i in range(pp_deg):
        while idx < n and not (i < pp_deg - 1 and avg - acc[i] < 0.5 * layer_costs[idx]):
            acc[i] += layer_costs[idx]
            division[i] += 1
            idx += 1
    for i in range(pp_deg - 1):
        left, right = int(np.sum(division[:i])), int(np.sum(division[:i + 1]))
        cur = float(np.sum(layer_costs[left:right])) + other_costs[i]
        while cur > avg * 1.3 and division[i] > 0:
            division[i] -= 1
            division[i + 1] += 1
            right -= 1
            cur -= layer_costs[right]
    for i in range(pp_deg - 1):
        while division[i] <= 0:
            division[i] += 1
            division[i + 1] -= 1
    for i in range(pp_deg - 1, 0, -1):
        while division[i] <= 0:
            division[i] += 1
            division[i - 1] -= 1
    stage = []
    for i in range(pp_deg):
        left, right = int(np.sum(division[:i])), int(np.sum(division[:i + 1]))
        stage.append(float(other_costs[i]) + float(np.sum(layer_costs[left:right])))
    return division, stage


def pp_division_memory_balanced(model_args_list, train_args_list, parallel_args_list, profile_model_args_list,
                                layer_num: Sequence[int], pp_deg: int, bsz: int, mbsz: int, strategies):
    """Pipeline division balanced by the memory of the cheapest uniform strategy (tp 1, ZeRO-2 over the remaining
    ranks, GPipe accounting), for models with several layer types
    (galvatron/core/search_engine/search_engine.py:954-1058).  Returns ``(division, stage memory)`` or
    ``(None, None)`` when no strategy uses ``pp_deg`` stages."""
    import copy as _copy

    from .cost_model import EmbeddingLMHeadMemoryCost, LayerMemoryCost
    from .strategy import DPType, EmbeddingLMHeadStrategy, LayerStrategy

    if pp_deg == 1:
        return [int(np.sum(layer_num))], None
    cand = [s for s in strategies if s.pp_size == pp_deg]
    if not cand:
        return None, None
    world = cand[0].world_size
    pa = [_copy.deepcopy(p) for p in parallel_args_list]
    for p in pa:
        p.pipeline_type = "gpipe"
    chunks = max(1, bsz // mbsz)
    per_type = []
    for i in range(len(layer_num)):
        st = LayerStrategy(pp_size=pp_deg, tp_size=1, sp_size=1, dp_size=world // pp_deg, dp_type=DPType.ZERO2, checkpoint=False)
        per_type.append(LayerMemoryCost(st, bsz, chunks, 0, model_args_list[i], train_args_list[i], pa[i],
                                        profile_model_args_list[i]).get_memory_cost()["enc_total"])
    est = EmbeddingLMHeadStrategy(pp_size=pp_deg, tp_size=1, sp_size=1, dp_size=world // pp_deg, dp_type=DPType.ZERO2)
    other = EmbeddingLMHeadMemoryCost(est, bsz, chunks, model_args_list[0], train_args_list[0], pa[0],
                                      profile_model_args_list[0]).get_memory_cost()["enc_total"]
    layers: List[float] = []
    for i, n in enumerate(layer_num):
        layers += [per_type[i]] * int(n)
    return balance_stages(layers, other, pp_deg)


def ensure_log_dir(log_dir: str) -> str:
    """Create the directory of the per-task search logs (galvatron/core/search_engine/utils.py:33-40)."""
    os.makedirs(log_dir, exist_ok=True)
    return log_dir


def _task_logger(log_dir: str, gbsz, chunks, pp, buffer_tp, mode) -> logging.Logger:
    d = ensure_log_dir(os.path.join(log_dir, "search_gbsz%d_chunks%d" % (gbsz, chunks)))
    name = "hg.search.%s.%d.%d.%d.%s.%d.%d" % (log_dir, gbsz, chunks, pp, mode, buffer_tp, threading.get_ident())
    logger = logging.getLogger(name)
    logger.setLevel(logging.INFO)
    logger.propagate = False
    for h in list(logger.handlers):
        logger.removeHandler(h)
        h.close()
    fh = logging.FileHandler(os.path.join(d, "pp%d_%s_buffer_tp%d.log" % (pp, mode, buffer_tp)), mode="w")
    fh.setFormatter(logging.Formatter("%(message)s"))
    logger.addHandler(fh)
    return logger


class GalvatronSearchEngine:
    def __init__(self, args):
        self.args = args
        self.world_size = args.hardware_info.num_nodes * args.hardware_info.num_gpus_per_node
        self.memory_constraint = args.hardware_info.memory_constraint * 1024
        self.mem_path = self.time_path = self.model_name = self.path = None
        self.verbose = True

    def _say(self, *a):
        if self.verbose:
            print(*a, flush=True)

    # ---- basic info ----------------------------------------------------------------------------------------
    def set_search_engine_info(self, path: str, model_layer_configs, model_name: str):
        self.set_model_layer_configs(model_layer_configs)
        self.path, self.model_name = path, model_name
        self.memory_profiling_path()
        self.time_profiling_path()

    def set_model_layer_configs(self, configs):
        if configs is None:
            return
        self.hiddensize_list = [c["hidden_size"] for c in configs]
        self.layernum_list = [c["layer_num"] for c in configs]
        self.seqlen_list = [c["seq_len"] for c in configs]
        self.num_layertype = len(self.layernum_list)
        self.total_layernum = sum(self.layernum_list)

    def _profile_path(self, kind: str, override: Optional[str]) -> str:
        name = "%s_profiling_%s_%s_all.json" % (kind, self.args.parallelism_info.mixed_precision, self.model_name)
        return os.path.join(override if override is not None else os.path.join(self.path, "configs"), name)

    def memory_profiling_path(self):
        if self.mem_path is None:
            self.mem_path = self._profile_path("memory", self.args.profiling_info.memory_profiling_path)
        return self.mem_path

    def time_profiling_path(self):
        if self.time_path is None:
            self.time_path = self._profile_path("computation", self.args.profiling_info.time_profiling_path)
        return self.time_path

    def initialize_search_engine(self, show_all_strategy_list: bool = False):
        self.generate_strategy_list()
        self.filter_strategy_list()
        if show_all_strategy_list:
            self.show_all_strategy_list()
        self.get_profiled_model_configs()
        self.get_profiled_hardware_configs()
        self.set_cost_models()

    # ---- strategy space ------------------------------------------------------------------------------------
    def generate_strategy_list(self):
        sp_info, default = self.args.search_space_info, self.args.parallelism_info.default_dp_type
        world = self.world_size
        degrees = []
        d = 1
        while d <= world:
            degrees.append(d)
            d *= 2
        found = set()
        for pp in degrees:
            if pp > self.total_layernum or pp > sp_info.max_pp_deg:
                continue
            for flavour, limit in (("tp", sp_info.max_tp_deg), ("sp", sp_info.max_sp_deg)):
                for width in degrees:
                    if (limit != -1 and width > limit) or width * pp > world:
                        continue
                    for cp in degrees:
                        if (sp_info.max_cp_deg != -1 and cp > sp_info.max_cp_deg) or pp * width * cp > world:
                            continue
                        dp = world // pp // width // cp
                        if dp == 1:
                            dp_types = [DPType.DDP]
                        elif default == "ddp":
                            dp_types = [DPType.DDP, DPType.ZERO3]
                        else:
                            dp_types = [DPType.ZERO2, DPType.ZERO3]
                        tp, sp = (width, 1) if flavour == "tp" else (1, width)
                        for dpt in dp_types:
                            for ckpt in (False, True):
                                found.add(AttentionStrategy(pp, tp, sp, cp, dp, dpt, ckpt))
        self.attention_strategy_list = sorted(found)
        self.ffn_strategy_list = sorted({s.to_ffn_strategy() for s in found})
        self.layer_strategy_list = sorted({s.to_layer_strategy() for s in found})
        self.embedding_lmhead_strategy_list = sorted({s.to_embedding_lmhead_strategy() for s in found})

    def filter_strategy_list(self, **overrides):
        """Apply the ``disable_*`` switches (keyword overrides update ``args.search_space_info`` first)."""
        info = self.args.search_space_info
        for k, v in overrides.items():
            if v is not None:
                setattr(info, k, v)
        rules = [("disable_pp", lambda s: s.pp_size == 1), ("disable_tp", lambda s: s.tp_size == 1),
                 ("disable_sp", lambda s: s.sp_size == 1), ("disable_cp", lambda s: s.cp_size == 1),
                 ("disable_dp", lambda s: s.dp_size == 1),
                 ("disable_fsdp", lambda s: s.dp_type != DPType.ZERO3)]
        names = ("embedding_lmhead_strategy_list", "attention_strategy_list", "ffn_strategy_list",
                 "layer_strategy_list")
        for flag, keep in rules:
            if getattr(info, flag):
                for n in names:
                    setattr(self, n, [s for s in getattr(self, n) if keep(s)])
        if info.disable_ckpt:
            for n in names[1:]:
                setattr(self, n, [s for s in getattr(self, n) if not s.checkpoint])
        if info.disable_embedding_lmhead_tp:
            self.embedding_lmhead_strategy_list = [s for s in self.embedding_lmhead_strategy_list if s.tp_size == 1]
        if info.disable_embedding_lmhead_sp:
            self.embedding_lmhead_strategy_list = [s for s in self.embedding_lmhead_strategy_list if s.sp_size == 1]
        for n in names:
            setattr(self, n, sorted(set(getattr(self, n))))

    def show_all_strategy_list(self):
        for n in ("attention_strategy_list", "ffn_strategy_list", "embedding_lmhead_strategy_list",
                  "layer_strategy_list"):
            lst = getattr(self, n)
            self._say("%s (%d): %s" % (n, len(lst), format_strategy_list(lst)))

    # ---- profiles --------------------------------------------------------------------------------------------
    def _fit_times(self, prefix_fn, mode):
        """Per layer type: a float (static / sequence) or the (slope, intercept) of time*bsz over bsz (batch)."""
        out = []
        for i in range(self.num_layertype):
            prefix = prefix_fn(i)
            if mode == "static":
                out.extend(t for s, t in self.time_config.items() if s.startswith(prefix))
                continue
            xs, ys = [], []
            for s, t in self.time_config.items():
                if not s.startswith(prefix):
                    continue
                if mode == "batch" and "_seq%d" % self.seqlen_list[i] in s:
                    xs.append(int(s.split("_")[-2][3:]))
                    ys.append(t * xs[-1])
                elif mode == "sequence" and "_bsz1_" in s:
                    xs.append(int(s.split("seq")[-1]))
                    ys.append(t)
            if mode == "batch":
                if len(xs) < 3:    # a line through fewer points says nothing about its own error
                    raise AssertionError("the computation profile of %s needs at least 3 batch sizes" % prefix)
                out.append(curve_fit(_line, xs, ys)[0])
            else:
                fn = _quad if prefix.startswith("layertype_%d_" % i) and "other" not in prefix else _line
                out.append(fn(self.seqlen_list[i], *curve_fit(fn, xs, ys)[0]))
        return out

    def get_profiled_model_configs(self):
        prof = self.args.profiling_info
        self.time_config = read_json_config(self.time_profiling_path())
        self.memory_config = _int_keys(read_json_config(self.memory_profiling_path()))
        mode = prof.time_profile_mode
        if mode == "static":
            self.time_profiled_list, self.other_time_profiled_list = [], []
            for i in range(self.num_layertype):
                for s, t in self.time_config.items():
                    if s.startswith("layertype_%d_" % i):
                        self.time_profiled_list.append(t)
                    if s.startswith("layertype_other_"):
                        self.other_time_profiled_list.append(t)
        else:
            self.time_profiled_list = self._fit_times(lambda i: "layertype_%d_" % i, mode)
            self.other_time_profiled_list = self._fit_times(lambda i: "layertype_other_", mode)
        n = self.num_layertype
        self.param_sizes, self.act_sizes = [0] * n, [{} for _ in range(n)]
        mem = self.memory_config
        sp = self.args.common_train_info.sequence_parallel
        if prof.memory_profile_mode == "sequence":
            if not sp or n != 1:
                raise AssertionError("sequence-mode memory profiles need sequence parallelism and one layer type")
            maxseqs = []
            for i in range(n):
                cfg = mem["layertype_%d_sp" % i]
                hi, lo = max(int(k) for k in cfg), min(int(k) for k in cfg)
                maxseqs.append(hi)
                self.param_sizes[i] = cfg[lo]["parameter_size"]
                self.act_sizes[i] = {tp: a / hi * self.seqlen_list[i]
                                     for tp, a in cfg[hi]["tp_activation_per_bsz_dict"].items()}
            self.other_memory_pp_off = mem["other_memory_pp_off_sp"][maxseqs[0]]
            self.other_memory_pp_on = {"first_stage": mem["other_memory_pp_on_first_sp"][maxseqs[0]],
                                       "last_stage": mem["other_memory_pp_on_last_sp"][maxseqs[-1]]}
            for tp in self.other_memory_pp_off["activation"]:
                self.other_memory_pp_off["activation"][tp] = self.other_memory_pp_off["activation"][tp] / maxseqs[0] * self.seqlen_list[0]
                first, last = self.other_memory_pp_on["first_stage"]["activation"], self.other_memory_pp_on["last_stage"]["activation"]
                first[tp] = first[tp] / maxseqs[0] * self.seqlen_list[0]
                last[tp] = last[tp] / maxseqs[-1] * self.seqlen_list[-1]
        else:
            tag = "_sp" if sp else ""
            for i in range(n):
                cfg = mem["layertype_%d%s" % (i, tag)][self.seqlen_list[i]]
                self.param_sizes[i] = cfg["parameter_size"]
                self.act_sizes[i] = cfg["tp_activation_per_bsz_dict"].copy()
            seq_key = num2str(self.seqlen_list, "seq")[3:]
            seq_key = int(seq_key) if seq_key.isdigit() else seq_key
            self.other_memory_pp_off = mem["other_memory_pp_off" + tag][seq_key]
            self.other_memory_pp_on = {"first_stage": mem["other_memory_pp_on_first" + tag][seq_key],
                                       "last_stage": mem["other_memory_pp_on_last" + tag][seq_key]}
        return self.time_config, self.memory_config

    def _hw_file(self, override: Optional[str], name: str) -> str:
        if override is not None:
            return override if override.endswith(".json") else os.path.join(override, name)
        # default: next to the search configuration, then the reference's tree layout, then the profile measured
        # on 8 x B200 that ships with the package
        here = os.path.dirname(os.path.abspath(__file__))
        candidates = [os.path.join(self.path, "hardware_configs"),
                      os.path.join(self.path, "../../profile_hardware/hardware_configs/"),
                      os.path.join(here, "..", "profiler", "hardware_configs")]
        for base in candidates:
            if os.path.exists(os.path.join(base, name)):
                return os.path.join(base, name)
        return os.path.join(candidates[0], name)

    def get_profiled_hardware_configs(self):
        prof, hw = self.args.profiling_info, self.args.hardware_info
        tag = "%dnodes_%dgpus_per_node.json" % (hw.num_nodes, hw.num_gpus_per_node)
        prof.allreduce_bandwidth_config_path = self._hw_file(prof.allreduce_bandwidth_config_path, "allreduce_bandwidth_" + tag)
        self.allreduce_bandwidth, self.allreduce_comm_coe = read_allreduce_bandwidth_config(
            prof.allreduce_bandwidth_config_path, self.world_size)
        prof.p2p_bandwidth_config_path = self._hw_file(prof.p2p_bandwidth_config_path, "p2p_bandwidth_" + tag)
        self.p2p_bandwidth, self.p2p_comm_coe = read_p2p_bandwidth_config(prof.p2p_bandwidth_config_path)
        prof.overlap_coe_path = self._hw_file(prof.overlap_coe_path, "overlap_coefficient.json")
        self.overlap_coe = read_json_config(prof.overlap_coe_path)["overlap_coe"]
        prof.sp_time_path = self._hw_file(prof.sp_time_path, "sp_time_" + tag)
        sp_cfg = read_json_config(prof.sp_time_path)
        self.sp_allreduce = remap_config(sp_cfg, "allreduce")
        self.sp_all2all = remap_config(sp_cfg, "all2all")
        self.allreduce_latency = remap_config_for_latency(sp_cfg, "allreduce")
        self.allgather_latency = remap_config_for_latency(sp_cfg, "allgather")
        self.all2all_latency = remap_config_for_latency(sp_cfg, "all2all")
        # optional B200 refit inputs stored next to the hardware profile
        self.bwd_fwd_ratio, self.fused_hidden = None, 0.0
        refit = os.path.join(os.path.dirname(prof.overlap_coe_path), "b200_refit.json")
        if os.path.exists(refit):
            r = read_json_config(refit)
            self.bwd_fwd_ratio = r.get("backward_forward_ratio")
            # scalar, or one measured value per tensor-parallel degree (profiler/hardware.py::profile_fused_tp)
            per_tp = {int(k.rsplit("tp", 1)[1]): float(v) for k, v in r.items()
                      if k.startswith("fused_comm_hidden_fraction_tp")}
            self.fused_hidden = per_tp if per_tp else r.get("fused_comm_hidden_fraction", 0.0)
            self.optimizer_ms = r.get("optimizer_ms_per_layer", 0.0)
            self.cache_fraction = r.get("allocator_cache_fraction")
        return self.allreduce_bandwidth, self.p2p_bandwidth, self.overlap_coe, self.sp_allreduce, self.sp_all2all

    def set_cost_models(self):
        a = self.args
        self.model_args_list, self.train_args_list, self.parallel_args_list = [], [], []
        self.profile_model_args_list, self.profile_hardware_args_list = [], []
        for i in range(self.num_layertype):
            self.model_args_list.append(ModelArgs(self.param_sizes[i], self.seqlen_list[i], self.hiddensize_list[i],
                                                  self.layernum_list[i]))
            self.train_args_list.append(TrainArgs(mixed_precision=a.parallelism_info.mixed_precision != "fp32",
                                                  async_grad_reduce=a.parallelism_info.async_grad_reduce))
            self.parallel_args_list.append(ParallelArgs(use_zero2_for_dp=a.parallelism_info.default_dp_type == "zero2",
                                                        sequence_parallel=a.common_train_info.sequence_parallel,
                                                        pipeline_type=a.parallelism_info.pipeline_type))
            self.profile_model_args_list.append(ProfileModelArgs(
                tp_activation_per_bsz_dict=self.act_sizes[i], other_memory_pp_off=self.other_memory_pp_off,
                other_memory_pp_on=self.other_memory_pp_on, forward_computation_time=self.time_profiled_list[i],
                other_time_profiled=self.other_time_profiled_list[0],
                backward_forward_ratio=getattr(self, "bwd_fwd_ratio", None)))
            self.profile_hardware_args_list.append(ProfileHardwareArgs(
                bct_fct_coe=2, extra_overhead=0, comm_coe_dict=self.allreduce_comm_coe, dp_overlap_coe=self.overlap_coe,
                bct_overlap_coe=self.overlap_coe, p2p_comm_coe_dict=self.p2p_comm_coe,
                costmodel_coe=a.debug_info.debug_costmodel_coe, allreduce_dict=self.sp_allreduce,
                all2all_dict=self.sp_all2all, overlap_slowdown_coe=self.overlap_coe,
                allreduce_latency_per_MB_dict=self.allreduce_comm_coe,
                allreduce_message_size_to_latency_dict_dict=self.allreduce_latency,
                allgather_message_size_to_latency_dict_dict=self.allgather_latency,
                all2all_message_size_to_latency_dict_dict=self.all2all_latency,
                fused_comm_hidden_fraction=getattr(self, "fused_hidden", 0.0),
                optimizer_ms_per_layer=getattr(self, "optimizer_ms", 0.0)))

    # ---- the sweep -----------------------------------------------------------------------------------------------
    def set_searching_bsz(self):
        b = self.args.batch_size_info
        if b.settle_bsz is not None and b.settle_bsz > 0:
            self.min_bsz = self.max_bsz = b.settle_bsz
            self.bsz_scale = 0
            self.BSZs = [b.settle_bsz]
        else:
            if not (b.min_bsz > 0 and b.max_bsz >= b.min_bsz and b.bsz_scale > 0):
                raise AssertionError("bad batch-size range")
            self.min_bsz = max(b.min_bsz, b.bsz_scale)
            self.bsz_scale = b.bsz_scale
            self.BSZs = list(range(self.min_bsz, b.max_bsz + 1, self.bsz_scale))
            self.max_bsz = self.BSZs[-1]

    def _tasks(self):
        a = self.args
        pp_range = sorted({s.pp_size for s in self.embedding_lmhead_strategy_list})
        tasks = []
        for gbsz in self.BSZs:
            chunk_list = [a.batch_size_info.settle_chunk] if a.batch_size_info.settle_chunk != -1 else range(1, gbsz + 1)
            for chunks in chunk_list:
                if gbsz % chunks:
                    continue
                for pp in pp_range:
                    if pp > chunks or pp > self.total_layernum:
                        continue
                    max_tp = max(self.world_size // pp, 1)
                    if a.search_space_info.max_tp_deg != -1:
                        max_tp = min(max_tp, a.search_space_info.max_tp_deg)
                    max_dp = max(min(gbsz // chunks, self.world_size // pp), 1)
                    min_tp = max(self.world_size // pp // max_dp, 1)
                    for mode in TP_SP_MODES:
                        if mode == "sp_only":
                            widths = [max_tp]
                        else:
                            widths = [w for w in range(min_tp, max_tp + 1) if is_power_of_two(w) and w * pp <= self.world_size]
                        tasks.extend((gbsz, chunks, pp, mode, w) for w in widths)
        return tasks

    def parallelism_optimization(self) -> float:
        self._say("=" * 25, "strategy search: memory budget %d MB" % self.memory_constraint, "=" * 25)
        self.set_searching_bsz()
        tasks = self._tasks()
        results: Dict[tuple, Dict[str, Any]] = {}
        opt = self.args.options_info
        if opt.parallel_search and len(tasks) > 1:
            import concurrent.futures

            workers = opt.worker if opt.worker > 0 else 2 * (os.cpu_count() or 1)
            with concurrent.futures.ThreadPoolExecutor(max_workers=min(workers, len(tasks))) as ex:
                futs = {ex.submit(self.search_for_single_task, t[0], t[1], t[2], t[4], t[3]): t for t in tasks}
                for fut in concurrent.futures.as_completed(futs):
                    results[futs[fut]] = copy.deepcopy(fut.result())
        else:
            for i, t in enumerate(tasks):
                self._say("task %d/%d: gbsz=%d chunks=%d pp=%d mode=%s buffer_tp=%d" % (i + 1, len(tasks), *t))
                results[t] = self.search_for_single_task(t[0], t[1], t[2], t[4], t[3])
        best, best_task = -1, None
        for t in tasks:  # task order decides ties, as in a sequential sweep
            thr = results[t]["throughput"]
            if thr > best:
                best, best_task = thr, t
        if best > 0:
            r = results[best_task]
            self._say("optimal: gbsz=%d chunks=%d pp=%d mode=%s buffer_tp=%d" % best_task)
            self._say("time cost %s s, memory remaining %s MB, memory cost %s MB" % (
                r["time_cost"], r["memory_remain"], r["memory_cost"]))
            self._say("vocab tp|sp=%s sp=%s sdp=%s" % (r["embedding_lmhead_tp_sp_size"], r["embedding_lmhead_sp"],
                                                      r["embedding_lmhead_sdp"]))
            self._say(format_strategy_list(r["strategy_list"]))
            self.optimal = r
            self.save_results(r, best_task[0], best_task[1])
        else:
            self._say("no valid configuration found")
        return best

    def search_for_single_task(self, gbsz, chunks, pp_size, global_buffer_tp_size, tp_sp_mode) -> Dict[str, Any]:
        a = self.args
        log_dir = os.path.join(a.options_info.log_dir, "%s_%dnodes_%dgpus_%dGB" % (
            self.model_name, a.hardware_info.num_nodes, a.hardware_info.num_gpus_per_node, self.memory_constraint // 1024))
        logger = _task_logger(log_dir, gbsz, chunks, pp_size, global_buffer_tp_size, tp_sp_mode)
        logger.info("search start: gbsz=%d chunks=%d pp=%d buffer_tp=%d mode=%s" % (
            gbsz, chunks, pp_size, global_buffer_tp_size, tp_sp_mode))
        max_dp = max(min(gbsz // chunks, self.world_size // pp_size), 1)

        def pick(lst):
            out = [s for s in lst if s.pp_size == pp_size and s.tp_sp_size <= global_buffer_tp_size and s.dp_size <= max_dp]
            if tp_sp_mode == "tp_only":
                out = [s for s in out if s.sp_size == 1]
            elif tp_sp_mode == "sp_only":
                out = [s for s in out if s.tp_size == 1]
            return out

        layers, embeds = pick(self.layer_strategy_list), pick(self.embedding_lmhead_strategy_list)
        if not layers or not embeds:
            logger.info("no strategies for this task")
            return {"throughput": -1}
        division = pp_division_even(self.layernum_list, pp_size)
        dp = DpOnModel(self.model_args_list, self.train_args_list, self.parallel_args_list, self.profile_model_args_list,
                       self.profile_hardware_args_list, max_mem=self.memory_constraint, layer_num=self.layernum_list,
                       sequence_len=self.seqlen_list, comm_coe_dict=self.allreduce_comm_coe, world_size=self.world_size,
                       pipeline_type=a.parallelism_info.pipeline_type, config=a, logger=logger,
                       threads=getattr(self, "dp_threads", 1),
                       mem_cache_fraction=getattr(self, "cache_fraction", None) or 0.2)
        best = dp.fit(gbsz, chunks, pp_size, division, global_buffer_tp_size, tp_sp_mode, layers, embeds)
        throughput = gbsz / best["time_cost"]
        logger.info("optimal: %s" % best)
        logger.info("max throughput = %s samples/s" % throughput)
        logger.info(format_strategy_list(best["strategy_list"]))
        for h in list(logger.handlers):
            h.close()
            logger.removeHandler(h)
        return {"throughput": throughput, "time_cost": best["time_cost"], "strategy_list": best["strategy_list"],
                "pp_size": pp_size, "pp_stage_list": division, "memory_remain": best["memory_remain"],
                "memory_cost": best["memory_used"], "embedding_lmhead_tp_sp_size": best["embedding_lmhead_tp_sp_size"],
                "embedding_lmhead_sp": best["embedding_lmhead_sp"], "embedding_lmhead_sdp": best["embedding_lmhead_sdp"]}

    # ---- output --------------------------------------------------------------------------------------------------
    def output_config_name(self) -> str:
        a = self.args
        name = "galvatron_config_%s_%dnodes_%dgpus_per_node_%dGB_%s" % (
            self.model_name, a.hardware_info.num_nodes, a.hardware_info.num_gpus_per_node, self.memory_constraint // 1024,
            a.parallelism_info.mixed_precision)
        if a.batch_size_info.settle_bsz > 0:
            name += "_bsz%d" % a.batch_size_info.settle_bsz
        off = [k for k in ("dp", "tp", "pp", "fsdp", "ckpt") if getattr(a.search_space_info, "disable_" + k)]
        if off:
            name += "_[%s_off]" % "_".join(off)
        return name + ".json"

    def save_results(self, optimal, optimal_bsz, chunk) -> str:
        a = self.args
        cfg = strategy_list2config(optimal["strategy_list"])
        cfg.update(global_bsz=optimal_bsz, chunks=chunk, pp_division=array2str(optimal["pp_stage_list"]),
                   pipeline_type=a.parallelism_info.pipeline_type, default_dp_type=a.parallelism_info.default_dp_type,
                   vtp=optimal["embedding_lmhead_tp_sp_size"], vsp=optimal["embedding_lmhead_sp"],
                   embed_sdp=optimal["embedding_lmhead_sdp"], vocab_sdp=optimal["embedding_lmhead_sdp"],
                   predicted_time_cost=float(optimal["time_cost"]))
        out_dir = a.options_info.output_config_path or os.path.join(self.path, "configs/")
        path = os.path.join(out_dir, self.output_config_name())
        write_json_config(cfg, path)
        self._say("wrote the searched strategy to %s" % path)
        return path

    # ---- diagnostics ----------------------------------------------------------------------------------------------
    def check_cost_model(self, gbsz: int, chunks: int, strategy_list: Optional[List[LayerStrategy]] = None):
        """Per-strategy predicted time / memory for a uniform assignment (to compare with measurements)."""
        if self.num_layertype != 1:
            raise AssertionError("only for single-layer-type (decoder-only) models")
        rows = []
        for s in (strategy_list or self.layer_strategy_list):
            if chunks < s.pp_size or gbsz // chunks // s.dp_size < 1:
                continue
            es = s.to_embedding_lmhead_strategy()
            _, other_nosync = EmbeddingLMHeadTimeCost(es, gbsz, chunks, self.seqlen_list, self.model_args_list[0],
                                                      self.train_args_list[0], self.parallel_args_list[0],
                                                      self.profile_model_args_list[0],
                                                      self.profile_hardware_args_list[0]).gen_result()
            division = pp_division_even(self.layernum_list, s.pp_size)
            t = pipeline_costmodel(self.layernum_list, self.model_args_list, self.train_args_list,
                                   self.parallel_args_list, self.profile_model_args_list,
                                   self.profile_hardware_args_list, [s] * self.total_layernum, division, chunks, gbsz,
                                   s.pp_size, other_nosync)
            mem = []
            other = EmbeddingLMHeadMemoryCost(es, gbsz, chunks, self.model_args_list[0], self.train_args_list[0],
                                              self.parallel_args_list[0], self.profile_model_args_list[0]
                                              ).get_memory_cost()["enc_total"]
            for stage in range(s.pp_size):
                lm = LayerMemoryCost(s, gbsz, chunks, stage, self.model_args_list[0], self.train_args_list[0],
                                     self.parallel_args_list[0], self.profile_model_args_list[0]
                                     ).get_memory_cost()["enc_total"]
                mem.append(lm * division[stage] + other[stage])
            rows.append({"strategy": s.to_simple_string(), "time_s": float(t), "memory_mb": [float(m) for m in mem]})
        return rows
