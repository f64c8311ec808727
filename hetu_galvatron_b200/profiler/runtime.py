"""In-training profiler: memory at fixed stages, device-timed iterations, the console line.

Hooks called from the training loop (same call sites as the reference, models/gpt/train_dist.py:43-68 and
hybrid_parallel_model.py:69-70): ``profile_time_start(it)`` / ``profile_time_end(it, loss, lr, grad_norm)``,
``profile_memory(it, stage)`` with stage in {"Before Forward", "After Forward", "After Backward"} and
``post_profile_memory(it)``.  Results go to the model-profiler JSON files the search engine reads:

* time   ``computation_profiling_{prec}_{model}_{unit}.json`` : ``layernum{L}_bsz{b}_seq{s}`` -> ms of a
          forward-only iteration (``profile_forward = 1``)
* memory ``memory_profiling_{prec}_{model}_{unit}.json`` : under the strategy key
          ``"{pp}_{tp}_{dp}[_c][_vtp][_sp]"``: ``layernum.._bsz.._seq.._rank{r}_{ms,act,act_peak}`` in MB.

Iteration time is taken with CUDA events on the training stream (wall clock on CPU), the first iteration is
dropped and samples outside 3 sigma are filtered.  Capability parity:
galvatron/core/profiler/runtime_profiler.py:24-62, :105-194, :218-258, :290-370; profiler/utils.py:22-64;
profiler/base_profiler.py:31-63.
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Dict, List, Optional

import numpy as np
import torch


def num2str(num, name: str) -> str:
    if isinstance(num, (list, tuple)):
        return name + "_".join(str(v) for v in num)
    return "%s%s" % (name, num)


def _read(path):
    return json.load(open(path)) if os.path.exists(path) else {}


def _write(cfg, path):
    d = os.path.dirname(path)
    if d:
        os.makedirs(d, exist_ok=True)
    with open(path, "w") as f:
        json.dump(cfg, f, indent=4)


def memory_strategy_key(pp_deg, tp_deg, world_size, checkpoint, sequence_parallel, vocab_tp) -> str:
    key = "%d_%d_%d" % (pp_deg, tp_deg, world_size // pp_deg // tp_deg)
    if checkpoint:
        key += "_c"
    if vocab_tp == tp_deg and tp_deg != 1:
        key += "_vtp"
    if sequence_parallel:
        key += "_sp"
    return key


def save_profiled_memory(path, pp_deg, tp_deg, world_size, layer_num, bsz, rank, model_states, activation,
                         activation_peak, cpt, sequence_parallel=False, vocab_tp=1, seq=None):
    cfg = _read(path)
    key = memory_strategy_key(pp_deg, tp_deg, world_size, cpt, sequence_parallel, vocab_tp)
    prefix = "%s_bsz%d_%s_rank%d" % (num2str(layer_num, "layernum"), bsz, num2str(seq, "seq"), rank)
    entry = cfg.setdefault(key, {})
    entry[prefix + "_ms"], entry[prefix + "_act"], entry[prefix + "_act_peak"] = model_states, activation, activation_peak
    _write(cfg, path)


def save_profiled_time(path, time_ms, bsz, layer_num, seq):
    cfg = _read(path)
    cfg["%s_bsz%d_%s" % (num2str(layer_num, "layernum"), bsz, num2str(seq, "seq"))] = time_ms
    _write(cfg, path)


def memory_mb(device=None, kind="allocated"):
    """(max, current) MB of the CUDA caching allocator; zeros on CPU."""
    if not torch.cuda.is_available():
        return 0.0, 0.0
    if kind == "reserved":
        return torch.cuda.max_memory_reserved(device) / 2 ** 20, torch.cuda.memory_reserved(device) / 2 ** 20
    return torch.cuda.max_memory_allocated(device) / 2 ** 20, torch.cuda.memory_allocated(device) / 2 ** 20


class BaseProfiler:
    def __init__(self):
        self.path = self.model_name = None
        self.profile_unit, self.mixed_precision = "all", "bf16"

    def set_work_dir(self, path):
        self.path = path

    def set_model_name(self, name):
        self.model_name = name

    def set_profile_unit(self, unit):
        self.profile_unit = unit

    def set_mixed_precision(self, mp):
        self.mixed_precision = mp

    def _config_path(self, kind: str) -> str:
        name = "%s_profiling_%s_%s_%s.json" % (kind, self.mixed_precision, self.model_name, self.profile_unit)
        return os.path.join(self.path or ".", "configs", name)

    def memory_profiling_path(self):
        return self._config_path("memory")

    def time_profiling_path(self):
        return self._config_path("computation")


class RuntimeProfiler(BaseProfiler):
    def __init__(self, args):
        super().__init__()
        self.args = args
        self.rank, self.world_size = 0, 1
        self.profile_ranks: List[int] = [0]
        self.mem_dict: Dict[str, float] = {}
        self.max_profile_iter = 5
        self.layernum_list = self.seqlen_list = self.hiddensize_list = None
        self.time_list: List[float] = []
        self.start_iter, self.end_iter, self.exit = 10, 20, False
        self._t0 = None
        self._ev = None
        self.last_iter_time = None

    # ---- setup -----------------------------------------------------------------------------------------
    def set_profiler_dist(self, path=None, model_layer_configs=None, model_name=None, profile_ranks=None,
                          start_iter=10, end_iter=20, rank=None):
        import torch.distributed as dist

        a = self.args
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = (dist.get_rank() if dist.is_initialized() else 0) if rank is None else rank
        self.set_work_dir(path)
        self.set_model_name(model_name)
        self.set_profile_unit(a.profile.profile_unit)
        self.set_mixed_precision(a.parallel.mixed_precision)
        self.set_model_layer_configs(model_layer_configs)
        self.set_memory_profiler(rank, profile_ranks if profile_ranks is not None else [0, world - 1])
        self.set_time_profiler(start_iter, end_iter, bool(a.profile.exit_after_profiling))

    def set_profiler_single(self, start_iter=10, end_iter=20):
        self.set_memory_profiler(0)
        self.set_time_profiler(start_iter, end_iter, bool(self.args.profile.exit_after_profiling))

    def set_model_layer_configs(self, cfgs):
        if cfgs is None:
            return
        self.hiddensize_list = [c["hidden_size"] for c in cfgs]
        self.layernum_list = [c["layer_num"] for c in cfgs]
        self.seqlen_list = [c["seq_len"] for c in cfgs]

    def set_memory_profiler(self, rank, profile_ranks=(), max_profile_iter=5):
        self.rank = rank
        self.profile_ranks = list(profile_ranks) if len(profile_ranks) else [rank]
        self.mem_dict, self.max_profile_iter = {}, max_profile_iter

    def set_time_profiler(self, start_iter, end_iter, exit=False):
        import torch.distributed as dist

        if end_iter <= start_iter:
            raise AssertionError("end_iter must be greater than start_iter")
        self.start_iter, self.end_iter, self.exit = start_iter, end_iter, exit
        self.time_list = []
        self.world_size = dist.get_world_size() if dist.is_initialized() else 1

    # ---- memory ------------------------------------------------------------------------------------------
    def profile_memory(self, iter: int, stage: str = ""):
        a = self.args
        if not (a.profile.profile and self.rank in self.profile_ranks and iter <= self.max_profile_iter):
            return
        dev = a.local_rank if torch.cuda.is_available() else None
        if stage == "Before Forward":
            if torch.cuda.is_available():
                torch.cuda.reset_peak_memory_stats(dev)
            self.mem_dict["iter_%d_before_forward" % iter] = memory_mb(dev)[1]
        elif stage == "After Forward":
            self.mem_dict["iter_%d_after_forward" % iter] = memory_mb(dev)[1]
        elif stage == "After Backward":
            mx, cur = memory_mb(dev)
            self.mem_dict["iter_%d_after_backward" % iter] = cur
            self.mem_dict["iter_%d_after_backward_max" % iter] = mx

    def post_profile_memory(self, iter: int):
        a = self.args
        if not (a.profile.profile and iter == self.max_profile_iter):
            return
        save = bool(a.profile.save_profiled_memory)
        if self.rank in self.profile_ranks:
            m, k = self.mem_dict, self.max_profile_iter - 1
            m["model_states"] = m.get("iter_%d_after_backward" % k, 0.0)
            if "iter_%d_after_forward" % k in m:
                m["model_states_and_activation"] = m["iter_%d_after_forward" % k]
                m["activation"] = m["iter_%d_after_forward" % k] - m.get("iter_%d_before_forward" % k, 0.0)
            m["model_states_and_peak_activation"] = m.get("iter_%d_after_backward_max" % k, 0.0)
            m["peak_activation"] = m["model_states_and_peak_activation"] - m["model_states"]
            time.sleep(0.05 * self.rank)
            print("[Profiled memory for rank %d]:" % self.rank)
            for key, val in m.items():
                print("\t%s: %.2f MB" % (key, val))
            if save:
                save_profiled_memory(self.memory_profiling_path(), a.parallel.pp_deg, a.parallel.global_tp_deg,
                                     self.world_size, self.layernum_list, a.train.global_batch_size, self.rank,
                                     m["model_states"], m.get("activation", 0.0), m["peak_activation"],
                                     a.parallel.global_checkpoint, a.train.sequence_parallel, a.parallel.vocab_tp,
                                     self.seqlen_list)
        if save:
            sys.exit(0)

    # ---- time --------------------------------------------------------------------------------------------
    def _now(self):
        if torch.cuda.is_available():
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            return ev
        return time.perf_counter()

    def profile_time_start(self, iter: int):
        if not self.args.profile.profile:
            return
        if self.start_iter <= iter < self.end_iter:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self._t0 = self._now()
        elif iter == self.end_iter:
            self._process_time_results()

    def profile_time_end(self, iter: int, loss=None, learning_rate=None, grad_norm=None):
        if not self.args.profile.profile or not (self.start_iter <= iter < self.end_iter):
            return
        t1 = self._now()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            dt = self._t0.elapsed_time(t1) / 1e3
        else:
            dt = t1 - self._t0
        self.time_list.append(dt)
        self.last_iter_time = dt
        if self.rank == self.world_size - 1:
            print(self.format_iteration(iter, dt, loss, learning_rate, grad_norm))

    def format_iteration(self, iter, iter_time, loss, learning_rate, grad_norm) -> str:
        if loss is None:
            return str(iter_time)
        a = self.args
        lr = (a.train.lr or 0.0) if learning_rate is None else learning_rate
        lv = loss.item() if hasattr(loss, "item") else float(loss)
        return ("| Iteration: {:6d} | Consumed samples: {:12d} | Elapsed time per iteration (ms): {:.1f} | "
                "Learning rate: {:.6e} | Loss: {:.6e} | grad norm: {:.2f} |").format(
            iter + 1, (iter + 1) * a.train.global_batch_size, iter_time * 1e3, lr, lv,
            0.0 if grad_norm is None else grad_norm)

    def filtered_time_samples(self) -> List[float]:
        if not self.time_list:
            raise RuntimeError("no timing samples")
        s = list(self.time_list)
        if self.start_iter == 0 and len(s) > 1:
            s = s[1:]
        if len(s) <= 2:
            return s
        mean, std = float(np.mean(s)), float(np.std(s))
        if std == 0:
            return s
        kept = [x for x in s if mean - 3 * std <= x <= mean + 3 * std]
        return kept or s

    def average_time(self) -> float:
        s = self.filtered_time_samples()
        return sum(s) / len(s)

    def _process_time_results(self):
        avg = self.average_time()
        print("Average iteration time is: %.4f s" % avg)
        a = self.args
        if a.profile.profile_forward:
            save_profiled_time(self.time_profiling_path(), avg * 1e3, a.train.global_batch_size, self.layernum_list,
                               self.seqlen_list)
        elif getattr(a.profile, "save_profiled_iteration_time", 0) and self.rank == 0:
            save_profiled_time(self._config_path("iteration"), avg * 1e3, a.train.global_batch_size, self.layernum_list,
                               self.seqlen_list)
        if self.exit:
            sys.exit(0)
        span = self.end_iter - self.start_iter
        self.time_list = []
        self.start_iter, self.end_iter = self.end_iter, self.end_iter + span
        self._t0 = self._now()
