"""Model profiler: plans the profiling runs and turns their raw measurements into the per-layer numbers that the
search engine reads.

*Planning.*  Every run is one launch of the training entry point (``$RUNTIME_LAUNCHER <runtime yaml> k=v ...``) with
``runtime.profile.profile=1``; :class:`~hetu_galvatron_b200.profiler.runtime.RuntimeProfiler` inside that run writes
raw keys into ``configs/{computation,memory}_profiling_<precision>_<model>_<unit>.json``:

* computation -- 1 GPU, forward only, for every (batch size, layer count in {min, max}, sequence length);
* memory -- N GPUs: (1) pp=1, tp in {1,2,..}, vocab-tp off/on, layer count in {min, max}; (2) the same without tp but
  with activation checkpointing; (3) pp in {2,4} with one layer per stage, tp in {1,2,..}, vocab-tp off/on.

*Post-processing.*  With ``T(L)`` the forward time and ``ms(L) / act(L)`` the model-state / activation megabytes of
a run with ``L`` layers::

    layertype_0_bsz{b}_seq{s}        = (T(Lmax) - T(Lmin)) / b / (Lmax - Lmin)                       ms per sample per layer
    layertype_other_bsz{b}_seq{s}    = max(0, (T(Lmin) - Lmin * b * per_layer) / b)
    parameter_size                   = max_tp( tp * (ms(Lmax) - ms(Lmin)) / dL * pp / 4 [* dp for ZeRO-3] )       MB
    tp_activation_per_bsz_dict[tp]   = (act(Lmax) - act(Lmin)) / dL / tp * world / bsz                            MB per sample
    tp_activation_per_bsz_dict["checkpoint"] = max over tp of the same from the checkpointed runs
    other_memory_pp_{off,on_first,on_last}[_sp][seq] = {model_states: {vtp: MB}, activation: {vtp: MB per sample}}

(the "other" part is what remains on the first / last rank after subtracting the layers of that stage).
Capability parity: galvatron/core/profiler/model_profiler.py:58-138 (sweeps), :140-200 (overrides), :231-391
(command lists), :422-471 (time), :473-803 (memory), :805-880 (helpers).
"""
from __future__ import annotations

import copy
import os
from collections import defaultdict
from typing import Any, Callable, Dict, List, Optional, Tuple

from ..utils.config_utils import num2str, read_json_config, write_json_config
from .runtime import BaseProfiler


class ModelProfiler(BaseProfiler):
    def __init__(self, args):
        super().__init__()
        self.args = args
        self.num_layertype = 1
        self.global_batch_size_list = self.layernum_tuple_list = self.seq_length_tuple_list = None
        self.basic_overrides_dict = None

    def set_profiler_launcher(self, path: str, model_name: Optional[str] = None):
        self.set_work_dir(path)
        self.set_model_name(model_name)
        self.set_profile_unit(self.args.profile_unit)
        self.set_mixed_precision(self.args.profile_mixed_precision)

    # ---- sweeps ---------------------------------------------------------------------------------------------
    def get_global_batch_size_list(self) -> List[int]:
        if self.global_batch_size_list is None:
            a = self.args
            if a.profile_mode == "batch":
                if None in (a.profile_min_batch_size, a.profile_max_batch_size, a.profile_batch_size_step):
                    raise AssertionError("batch mode needs profile_{min,max}_batch_size and profile_batch_size_step")
                self.global_batch_size_list = list(range(a.profile_min_batch_size, a.profile_max_batch_size + 1,
                                                         a.profile_batch_size_step))
            else:
                if a.profile_fixed_batch_size is None:
                    raise AssertionError("%s mode needs profile_fixed_batch_size" % a.profile_mode)
                self.global_batch_size_list = [a.profile_fixed_batch_size]
        return self.global_batch_size_list

    def get_layernum_tuple_list(self) -> List[Tuple[int, ...]]:
        if self.layernum_tuple_list is None:
            a = self.args
            self.layernum_tuple_list = [(a.profile_layernum_min,), (a.profile_layernum_max,)]
        return self.layernum_tuple_list

    def get_seq_length_tuple_list(self) -> List[Tuple[int, ...]]:
        if self.seq_length_tuple_list is None:
            a = self.args
            if a.profile_mode in ("static", "batch"):
                if not a.profile_fixed_seq_length_list or len(a.profile_fixed_seq_length_list) != 1:
                    raise AssertionError("profile_fixed_seq_length_list must hold one sequence length")
                seqs = [a.profile_fixed_seq_length_list[0]]
            elif a.profile_type == "computation":
                if None in (a.profile_min_seq_length, a.profile_max_seq_length, a.profile_seq_length_step):
                    raise AssertionError("sequence mode needs profile_{min,max}_seq_length and profile_seq_length_step")
                seqs = list(range(a.profile_min_seq_length, a.profile_max_seq_length + 1, a.profile_seq_length_step))
            else:
                lo, hi = a.profile_min_seq_length, a.profile_max_seq_length
                if lo is None or hi is None or lo & (lo - 1) or hi & (hi - 1):
                    raise AssertionError("memory profiling over sequence lengths needs power-of-two bounds")
                seqs = [1 << s for s in range(lo.bit_length() - 1, hi.bit_length())]
            self.seq_length_tuple_list = [(s,) for s in seqs]
        return self.seq_length_tuple_list

    def get_basic_overrides_dict(self) -> Dict[str, Any]:
        if self.basic_overrides_dict is None:
            a = self.args
            common_tail = {
                "runtime.model.model_size": a.model_info.model_size,
                "runtime.model.is_moe_model": a.model_info.is_moe_model,
                "runtime.model.model_config_path": a.model_info.model_config_path,
                "runtime.model.set_layernum_manually": 1,
                "runtime.model.set_seqlen_manually": 1,
                "runtime.data.use_random_dataset": True,
            }
            if a.profile_type == "computation":
                d = {"runtime.parallel.pp_deg": 1, "runtime.parallel.global_tp_deg": 1, "runtime.parallel.global_cp_deg": 1,
                     "runtime.parallel.global_checkpoint": 0, "runtime.parallel.vocab_tp": 1, "runtime.parallel.vocab_cp": 1,
                     "runtime.parallel.default_dp_type": "ddp", "runtime.parallel.sdp": 0,
                     "runtime.parallel.pipeline_type": "gpipe", "runtime.parallel.mixed_precision": a.profile_mixed_precision,
                     "runtime.train.chunks": 1, "runtime.train.use_flash_attn": True, "runtime.train.sequence_parallel": True,
                     "runtime.profile.profile": 1, "runtime.profile.profile_mode": a.profile_mode,
                     "runtime.profile.profile_unit": a.profile_unit, "runtime.profile.profile_forward": 1}
            else:
                bsz = self.get_global_batch_size_list()
                if len(bsz) != 1:
                    raise AssertionError("memory profiling uses one batch size")
                d = {"runtime.parallel.default_dp_type": a.profile_dp_type, "runtime.parallel.pipeline_type": "gpipe",
                     "runtime.parallel.mixed_precision": a.profile_mixed_precision,
                     "runtime.train.global_batch_size": bsz[0], "runtime.train.chunks": 1,
                     "runtime.train.use_flash_attn": True, "runtime.train.sequence_parallel": True,
                     "runtime.profile.profile": 1, "runtime.profile.profile_mode": a.profile_mode,
                     "runtime.profile.profile_unit": a.profile_unit, "runtime.profile.profile_forward": 0,
                     "runtime.profile.save_profiled_memory": 1}
            d.update(common_tail)
            self.basic_overrides_dict = d
        return self.basic_overrides_dict

    def get_envs_dict(self) -> Dict[str, Any]:
        # stream issue order is explicit in this framework; the variable is kept for launchers that expect it.
        # Memory runs keep the gradient / parameter buffers in the caching allocator (not in symmetric memory) so
        # that the allocator statistics the runtime profiler reads see them.
        env = {"CUDA_DEVICE_MAX_CONNECTIONS": 1}
        if self.args.profile_type == "memory":
            env["HG_FUSED_ZERO"] = 0
        return env

    @staticmethod
    def dict_to_str(d: Dict, sep: str = "=") -> str:
        return "".join("%s%s%s " % (k, sep, "null" if v is None else v) for k, v in d.items())

    # ---- command lists ----------------------------------------------------------------------------------------
    def _command(self, overrides: Dict[str, Any], log_dir: str, log_name: str) -> str:
        launcher = os.getenv("RUNTIME_LAUNCHER")
        if launcher is None:
            raise AssertionError("RUNTIME_LAUNCHER is not set")
        return "%s %s %s %s 2>&1 | tee %s/%s.log" % (self.dict_to_str(self.get_envs_dict()), launcher,
                                                     self.args.runtime_yaml_template_path, self.dict_to_str(overrides),
                                                     log_dir, log_name)

    def memory_commands(self) -> List[str]:
        a = self.args
        if a.profile_mode not in ("static", "sequence"):
            raise AssertionError("memory profiling supports the static and sequence modes")
        nodes, gpn = int(os.getenv("NUM_NODES", -1)), int(os.getenv("NUM_GPUS_PER_NODE", -1))
        if nodes < 0 or gpn < 0:
            raise AssertionError("NUM_NODES and NUM_GPUS_PER_NODE are not set")
        world = nodes * gpn
        max_tp = min(world, a.profile_max_tp_deg) if a.profile_mode == "static" else 1
        base = self.get_basic_overrides_dict()
        log_dir = os.path.join(self.path, "logs/profile_memory")
        cmds = []

        def add(pp, tp, vtp_on, ckpt, layers, seq, name_vocab):
            ov = {"runtime.parallel.pp_deg": pp, "runtime.parallel.global_tp_deg": tp,
                  "runtime.parallel.global_checkpoint": ckpt, "runtime.parallel.vocab_tp": tp if vtp_on else 1,
                  "runtime.model.num_layers": layers, "runtime.train.seq_length": seq}
            ov.update(base)
            cmds.append(self._command(ov, log_dir, "pp%d_tp%d_vocab%d_ckpt%d_layernum%d_seq%d" % (pp, tp, name_vocab, ckpt, layers, seq)))

        def tp_degrees(limit):
            t = 1
            while t <= limit:
                yield t
                t *= 2

        for (seq,) in self.get_seq_length_tuple_list():
            for tp in tp_degrees(max_tp):
                for vtp_on in (0, 1):
                    if tp == 1 and vtp_on:
                        continue
                    for (layers,) in self.get_layernum_tuple_list():
                        add(1, tp, vtp_on, 0, layers, seq, vtp_on)
        for (seq,) in self.get_seq_length_tuple_list():
            for (layers,) in self.get_layernum_tuple_list():
                add(1, 1, 0, 1, layers, seq, 1)
        for (seq,) in self.get_seq_length_tuple_list():
            for pp in (2, 4):
                for tp in tp_degrees(max_tp):
                    if pp * tp > world:
                        continue
                    for vtp_on in (0, 1):
                        if tp == 1 and vtp_on:
                            continue
                        add(pp, tp, vtp_on, 0, pp, seq, vtp_on)
        return cmds

    def computation_commands(self) -> List[str]:
        base = self.get_basic_overrides_dict()
        log_dir = os.path.join(self.path, "logs/profile_computation")
        cmds = []
        for gbsz in self.get_global_batch_size_list():
            for (layers,) in self.get_layernum_tuple_list():
                for (seq,) in self.get_seq_length_tuple_list():
                    ov = {"runtime.train.global_batch_size": gbsz, "runtime.model.num_layers": layers,
                          "runtime.train.seq_length": seq}
                    ov.update(base)
                    cmds.append(self._command(ov, log_dir, "layernum_%d_seq_%d_gbsz_%d" % (layers, seq, gbsz)))
        return cmds

    def launch_profiling_scripts(self, run: Optional[Callable[[str], int]] = None):
        a = self.args
        if a.profile_flow_control == "data_only":
            return []
        run = run or os.system
        kind = a.profile_type
        cmds = self.memory_commands() if kind == "memory" else self.computation_commands()
        os.makedirs(os.path.join(self.path, "logs/profile_%s" % kind), exist_ok=True)
        if a.profile_flow_control == "scripts_only":
            d = os.path.join(self.path, "scripts")
            os.makedirs(d, exist_ok=True)
            script = os.path.join(d, "%s_profile_scripts_%s.sh" % (kind, a.profile_unit))
            with open(script, "w") as f:
                for c in cmds:
                    f.write(c + "\nsleep 1\n")
            print("%s profiling scripts written to %s" % (kind, script))
        else:
            for c in cmds:
                print(c)
                run(c)
        return cmds

    # ---- post-processing -------------------------------------------------------------------------------------------
    def env_args(self) -> Dict[str, str]:
        mem = self.args.profile_type == "memory"
        return {"NUM_NODES": os.getenv("NUM_NODES", "1") if mem else "1",
                "NUM_GPUS_PER_NODE": os.getenv("NUM_GPUS_PER_NODE", "8") if mem else "1"}

    def process_profiled_data(self):
        if self.args.profile_flow_control in ("scripts_only", "launch_only"):
            return
        env = self.env_args()
        world = int(env["NUM_NODES"]) * int(env["NUM_GPUS_PER_NODE"])
        layer_lists = [list(t) for t in self.get_layernum_tuple_list()]
        if self.args.profile_type == "computation":
            self._process_computation(layer_lists)
        else:
            self._process_memory(world, layer_lists)

    @staticmethod
    def key_format(layernum, bsz=None, seq=None, rank=None, type=None) -> str:
        s = "layernum" + ("_".join(str(v) for v in layernum) if isinstance(layernum, (list, tuple)) else str(layernum))
        if bsz is not None:
            s += "_bsz%d" % bsz
        if seq is not None:
            s += "_%s" % seq if isinstance(seq, str) else "_seq%d" % seq
        if rank is not None and type is not None:
            s += "_rank%d_%s" % (rank, type)
        return s

    def _process_computation(self, layer_lists: List[List[int]]):
        path = self.time_profiling_path()
        cfg = read_json_config(path)
        a = self.args
        dL = a.profile_layernum_max - a.profile_layernum_min
        for bsz in self.get_global_batch_size_list():
            for seq in self.get_seq_length_tuple_list():
                info = num2str(list(seq), "seq")
                t_min = cfg[self.key_format(layer_lists[0], bsz, info)]
                per_layer = []
                for idx, layers in enumerate(layer_lists[1:]):
                    t = (cfg[self.key_format(layers, bsz, info)] - t_min) / bsz / dL
                    cfg["layertype_%d_bsz%d_seq%d" % (idx, bsz, seq[idx])] = t
                    per_layer.append(t)
                other = t_min
                for idx, t in enumerate(per_layer):
                    other -= layer_lists[0][idx] * t * bsz
                cfg["layertype_other_bsz%d_%s" % (bsz, info)] = max(other / bsz, 0)
        write_json_config(cfg, path)

    @staticmethod
    def total_memcost(pp_deg: int, layernum: int, layertype: int, per_layer_cost: List[float], stage_idx: int) -> float:
        costs: List[float] = []
        for l in range(layertype):
            costs.extend([per_layer_cost[l]] * layernum)
        per_stage = len(costs) // pp_deg
        if per_stage * pp_deg != len(costs):
            raise AssertionError("layers must divide evenly over the pipeline stages")
        return float(sum(costs[stage_idx * per_stage:(stage_idx + 1) * per_stage]))

    def _process_memory(self, world: int, layer_lists: List[List[int]]):
        a = self.args
        if a.profile_mode not in ("static", "sequence"):
            raise AssertionError("memory profiling supports the static and sequence modes")
        path = self.memory_profiling_path()
        cfg = read_json_config(path)
        for seq in self.get_seq_length_tuple_list():
            self._process_memory_one_seq(cfg, seq, world, layer_lists)
        write_json_config(cfg, path)

    def _process_memory_one_seq(self, cfg: Dict, seq: Tuple[int, ...], world: int, layer_lists: List[List[int]]):
        a = self.args
        bsz = a.profile_fixed_batch_size
        if bsz is None:
            raise AssertionError("memory post-processing needs profile_fixed_batch_size")
        dL = a.profile_layernum_max - a.profile_layernum_min
        l_min, l_max = layer_lists[0], layer_lists[1]
        info = num2str(list(seq), "seq")
        sp = "_sp" if a.sequence_parallel else ""
        K = self.key_format

        def strategy_key(pp, tp, ckpt=False, vtp=False):
            s = "%d_%d_%d" % (pp, tp, world // pp // tp)
            if ckpt:
                s += "_c"
            if vtp:
                s += "_vtp"
            return s + sp

        def powers(limit):
            t = 1
            while t <= limit:
                yield t
                t *= 2

        # per-layer parameters and activations by tensor-parallel degree (pp = 1 runs)
        param_by_tp: Dict[int, float] = {}
        act_by_tp: Dict[Any, float] = {}
        param_size = -1.0
        for tp in powers(world):
            re = cfg.get(strategy_key(1, tp))
            if re is None:
                continue
            p = (re[K(l_max, bsz, info, 0, "ms")] - re[K(l_min, bsz, info, 0, "ms")]) / dL / 4
            act = (re[K(l_max, bsz, info, 0, "act")] - re[K(l_min, bsz, info, 0, "act")]) / dL / tp * world / bsz
            if a.profile_dp_type == "zero3":
                p *= world // tp
            param_by_tp[tp], act_by_tp[tp] = p, act
            param_size = max(param_size, p * tp)
        # checkpointed runs
        act_ckpt = -1.0
        for tp in powers(world):
            re = cfg.get(strategy_key(1, tp, ckpt=True))
            if re is None:
                continue
            act = (re[K(l_max, bsz, info, 0, "act")] - re[K(l_min, bsz, info, 0, "act")]) / dL / tp * world / bsz
            act_ckpt = max(act_ckpt, act)
        act_by_tp["checkpoint"] = act_ckpt

        # what is left on the first / last rank besides the decoder layers
        inf = 1e6
        new = lambda: {"model_states": defaultdict(lambda: inf), "activation": defaultdict(lambda: inf)}  # noqa: E731
        off, first, last = new(), new(), new()
        for pp in powers(world):
            for tp in powers(world // pp):
                for vtp_on in (0, 1):
                    if tp == 1 and vtp_on:
                        continue
                    re = cfg.get(strategy_key(pp, tp, vtp=bool(vtp_on)))
                    if re is None:
                        continue
                    layernum = pp if pp > 1 else l_min[0]
                    lkey = [layernum] if pp > 1 else l_min
                    dp = world // pp // tp
                    ms_first = self.total_memcost(pp, layernum, 1, [param_by_tp[tp] * 4], 0)
                    ms_last = self.total_memcost(pp, layernum, 1, [param_by_tp[tp] * 4], pp - 1)
                    act_first = self.total_memcost(pp, layernum, 1, [act_by_tp[tp]], 0)
                    act_last = self.total_memcost(pp, layernum, 1, [act_by_tp[tp]], pp - 1)
                    r0, rl = re[K(lkey, bsz, info, 0, "ms")], re[K(lkey, bsz, info, world - 1, "ms")]
                    if a.profile_dp_type == "zero3":
                        scale = (world // pp) / (tp if vtp_on else 1)
                        o_ms_first = (r0 - ms_first / dp) * scale
                        o_ms_last = (rl - ms_last / dp) * scale
                    else:
                        o_ms_first, o_ms_last = r0 - ms_first, rl - ms_last
                    peak0 = max(re[K(lkey, bsz, info, 0, "act_peak")], re[K(lkey, bsz, info, 0, "act")])
                    peakl = max(re[K(lkey, bsz, info, world - 1, "act_peak")], re[K(lkey, bsz, info, world - 1, "act")])
                    local_b = bsz / (world // (pp * tp))
                    div = bsz / world * pp * (tp if vtp_on else 1)
                    o_act_first = (peak0 - act_first * local_b) / div
                    o_act_last = (peakl - act_last * local_b) / div
                    vals = [max(v, 0) for v in (o_ms_first, o_ms_last, o_act_first, o_act_last)]
                    key = tp if vtp_on else 1
                    if pp == 1:
                        off["model_states"][key] = min(off["model_states"][key], vals[0])
                        off["activation"][key] = min(off["activation"][key], vals[2])
                    else:
                        first["model_states"][key] = min(first["model_states"][key], vals[0])
                        first["activation"][key] = min(first["activation"][key], vals[2])
                        last["model_states"][key] = min(last["model_states"][key], vals[1])
                        last["activation"][key] = min(last["activation"][key], vals[3])
        if a.sequence_parallel:
            # degrees that were not measured: halve from the next smaller one (activations are sharded by sequence)
            for tp in (2, 4, 8):
                if tp not in act_by_tp:
                    act_by_tp[tp] = act_by_tp[tp // 2] / 2
                for d in (off, first, last):
                    for k in ("model_states", "activation"):
                        if tp not in d[k]:
                            d[k][tp] = d[k][tp // 2] / 2
        cfg.setdefault("layertype_0" + sp, {})[str(seq[0])] = {"parameter_size": param_size,
                                                              "tp_activation_per_bsz_dict": act_by_tp}
        seq_key = info[3:] if info.startswith("seq") else info
        for name, d in (("other_memory_pp_off", off), ("other_memory_pp_on_first", first), ("other_memory_pp_on_last", last)):
            cfg.setdefault(name + sp, {})[seq_key] = {k: dict(v) for k, v in copy.deepcopy(d).items()}
