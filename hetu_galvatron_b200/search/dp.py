"""Dynamic-programming driver of the strategy search.

For one task ``(global batch, chunks, pp, pipeline division, search mode)`` it builds, per pipeline stage,
the integer memory table ``v[layer, strategy]`` (MB, rounded up), the per-layer time ``intra[layer,
strategy]`` and the transition cost ``inter[layer, prev, cur]`` (activation resharding when the
sequence-sharding width changes, otherwise tiny tie-breakers that prefer the simpler strategy), runs the
native core once per (embedding / LM-head candidate, stage), and re-scores the concatenated per-layer
assignment with the pipeline cost model.  Coarse mode (``fine_grained_mode = 0``) gives every layer the
same strategy.

Capability parity: galvatron/core/search_engine/dynamic_programming.py:12-115 (DPAlg incl. the pure-Python
fallback), :117-360 (budget, coarse mode), :362-610 (fine-grained tables and the per-candidate loop).
"""
from __future__ import annotations

import copy
import math
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

from .cost_model import (EmbeddingLMHeadMemoryCost, EmbeddingLMHeadTimeCost, LayerMemoryCost, LayerTimeCost,
                         pipeline_costmodel)
from .strategy import DPType, EmbeddingLMHeadStrategy, LayerStrategy, format_strategy_list


def load_native_core():
    try:
        from .._lib import hg_dp_core  # type: ignore

        return hg_dp_core
    except Exception:
        try:
            from ..csrc import build as _build

            _build.build_host()
            import importlib

            return importlib.import_module("hetu_galvatron_b200._lib.hg_dp_core")
        except Exception:
            return None


MEM_TABLE_ROWS = 32768


class DPAlg:
    """One stage's knapsack: memory budget ``max_mem`` MB, ``layer_num`` layers, ``S`` strategies."""

    def __init__(self, max_mem: int, other_mem_cost: Dict[int, int], other_time_cost: Dict[int, float],
                 layer_num: int, layer_strategy_num: int, use_cpp_core: bool = True, threads: int = 1):
        self.max_mem = max_mem + 1
        self.layer_num, self.S = layer_num, layer_strategy_num
        self.other_mem_cost, self.other_time_cost = other_mem_cost, other_time_cost
        self.use_cpp_core, self.threads = use_cpp_core, threads
        self._f = np.zeros((self.max_mem, self.S), dtype=np.float64)
        self._mark = np.full((layer_num, self.max_mem, self.S), -1, dtype=np.int32)
        self.v = self.inter = self.intra = None

    def set_v_and_cost(self, v: np.ndarray, intra_layer_cost: np.ndarray, inter_layer_cost: np.ndarray):
        if v.shape != (self.layer_num, self.S) or intra_layer_cost.shape != (self.layer_num, self.S) or \
                inter_layer_cost.shape != (self.layer_num, self.S, self.S):
            raise AssertionError("table shapes do not match (layers=%d, strategies=%d)" % (self.layer_num, self.S))
        self.v = np.ascontiguousarray(v.astype(np.int32))
        self.inter = np.ascontiguousarray(inter_layer_cost, dtype=np.float64)
        self.intra = np.ascontiguousarray(intra_layer_cost, dtype=np.float64)

    def fit(self):
        core = load_native_core() if self.use_cpp_core else None
        if core is not None:
            res = {k: np.full(self.layer_num, -1, dtype=np.int32) for k in self.other_mem_cost}
            total, remain = core.dynamic_programming_core(
                self.layer_num, self.max_mem, self.S, self.v, self._mark, self._f, self.inter, self.intra,
                {int(k): int(v) for k, v in self.other_mem_cost.items()},
                {int(k): float(v) for k, v in self.other_time_cost.items()}, res, self.threads)
            return total, {k: list(v) for k, v in res.items()}, remain
        return self._fit_python()

    def _fit_python(self):
        """Reference semantics in NumPy (row-vectorised over the previous strategy); used when the native
        module cannot be built, and as the oracle of the native core's test."""
        f, mark, v = self._f, self._mark, self.v
        for i in range(self.layer_num):
            for m in range(self.max_mem - 1, -1, -1):
                for s in range(self.S):
                    if m < v[i, s]:
                        mark[i, m, s] = -1
                        f[m, s] = np.inf
                        continue
                    cand = f[m - v[i, s], :] + self.inter[i, :, s] + self.intra[i, s]
                    k = int(np.argmin(cand))
                    mark[i, m, s] = k
                    f[m, s] = cand[k]
        total, res, remain = {}, {}, {}
        for key, om in self.other_mem_cost.items():
            res[key] = [-1] * self.layer_num
            m0 = self.max_mem - 1 - om
            if m0 < 0 or not np.min(f[m0]) < np.inf:
                total[key], remain[key] = np.inf, -1
                continue
            s = int(np.argmin(f[m0]))
            total[key] = f[m0, s] + self.other_time_cost[key]
            res[key][-1] = s
            m = m0
            for i in range(self.layer_num - 1, 0, -1):
                cur = s
                s = int(mark[i, m, cur])
                m -= v[i, cur]
                res[key][i - 1] = s
            remain[key] = int(m - v[0, s])
        return total, res, remain


def _differs_only_in(a: LayerStrategy, b: LayerStrategy, what: Sequence[str]) -> bool:
    """True when ``a`` and ``b`` agree on everything except the listed aspects, and differ in at least one of
    them.  Aspects: ``sp`` (tensor- vs sequence-parallel flavour of the same width), ``fsdp`` (ZeRO type),
    ``cpt`` (checkpoint flag)."""
    what = sorted(what)
    if what == ["sp"]:
        same = (a.pp_size, a.tp_sp_size, a.dp_size, a.checkpoint, a.dp_type) == \
               (b.pp_size, b.tp_sp_size, b.dp_size, b.checkpoint, b.dp_type)
        return same and a.sp_size != b.sp_size
    base = (a.pp_size, a.tp_size, a.sp_size, a.dp_size) == (b.pp_size, b.tp_size, b.sp_size, b.dp_size)
    if what == ["fsdp"]:
        return base and a.checkpoint == b.checkpoint and a.dp_type != b.dp_type
    if what == ["cpt"]:
        return base and a.dp_type == b.dp_type and a.checkpoint != b.checkpoint
    if what == ["cpt", "fsdp"]:
        return base and not (a.dp_type == b.dp_type and a.checkpoint == b.checkpoint)
    return True


class DpOnModel:
    def __init__(self, model_args_list, train_args_list, parallel_args_list, profile_model_args_list,
                 profile_hardware_args_list, max_mem: int = 8192, layer_num: List[int] = None,
                 sequence_len: List[int] = None, comm_coe_dict: Dict[str, float] = None, world_size: int = 8,
                 mem_cache: bool = True, pipeline_type: str = "gpipe", config=None, logger=None, threads: int = 1,
                 mem_cache_fraction: float = 0.2):
        n = len(layer_num)
        for lst in (model_args_list, train_args_list, parallel_args_list, profile_model_args_list,
                    profile_hardware_args_list):
            if not isinstance(lst, list) or len(lst) != n:
                raise AssertionError("one argument bundle per layer type is required")
        self.margs, self.targs, self.pargs = model_args_list, train_args_list, parallel_args_list
        self.pmargs, self.hwargs = profile_model_args_list, profile_hardware_args_list
        self.layer_num, self.sequence_len = layer_num, sequence_len
        self.comm_coe_dict, self.world_size = comm_coe_dict or {}, world_size
        self.config, self.logger, self.pipeline_type, self.threads = config, logger, pipeline_type, threads
        self.max_mem = max_mem
        self.mem_cache = 0
        if max_mem // 1024 > 20 and mem_cache:
            # part of a large budget is left to the caching allocator (fragmentation, transient buffers): a fifth, as
            # in the reference, unless the hardware refit measured this framework's own overhead
            self.mem_cache = int(max_mem * mem_cache_fraction)
            self.max_mem -= self.mem_cache
        self.mem_sub_cache = self.max_mem

    def log(self, msg):
        if self.logger is not None:
            self.logger.info(msg)

    # ---- shared pieces ---------------------------------------------------------------------------------------
    def _global_buffer_mb(self, gbsz, chunks, pp_size, buffer_tp, mode) -> float:
        """Persistent all-gather buffer of Megatron sequence parallelism ([S, b, H] at the largest tp)."""
        cfg = self.config
        if not (cfg.common_train_info.sequence_parallel and cfg.common_train_info.global_memory_buffer) or mode == "sp_only":
            return 0
        dp = self.world_size // pp_size // buffer_tp
        mb = gbsz / chunks / dp * cfg.model_info.hidden_size * max(self.sequence_len) * 4 / 1024 / 1024
        # (the precision field is a non-empty string for every precision, so the halving always applies --
        #  kept because the golden search results depend on it)
        return mb / 2 if cfg.parallelism_info.mixed_precision else mb

    def _embed_costs(self, strategy, gbsz, chunks):
        t = EmbeddingLMHeadTimeCost(strategy, gbsz, chunks, self.sequence_len, self.margs[0], self.targs[0],
                                    self.pargs[0], self.pmargs[0], self.hwargs[0], self.logger).gen_result()
        m = EmbeddingLMHeadMemoryCost(strategy, gbsz, chunks, self.margs[0], self.targs[0], self.pargs[0],
                                      self.pmargs[0], self.logger).get_memory_cost()["enc_total"]
        return t, m

    def _layer_memory(self, strategy, gbsz, chunks, stage, t):
        return LayerMemoryCost(strategy, gbsz, chunks, stage, self.margs[t], self.targs[t], self.pargs[t],
                               self.pmargs[t], self.logger).get_memory_cost()["enc_total"]

    def _pipeline(self, strategy_list, partition, chunks, gbsz, pp_size, other_time):
        return pipeline_costmodel(self.layer_num, self.margs, self.targs, self.pargs, self.pmargs, self.hwargs,
                                  strategy_list, partition, chunks, gbsz, pp_size, other_time, self.logger)

    @staticmethod
    def _empty(pp_size):
        return {"time_cost": np.inf, "memory_used": [-1] * pp_size, "memory_remain": [-1] * pp_size,
                "strategy_list": None, "embedding_lmhead_tp_sp_size": -1, "embedding_lmhead_sp": -1,
                "embedding_lmhead_sdp": -1, "pp_size": pp_size}

    @staticmethod
    def _record(opt, cost, used, remain, strategies, es: EmbeddingLMHeadStrategy):
        opt.update(time_cost=cost, memory_used=copy.deepcopy(used), memory_remain=copy.deepcopy(remain),
                   strategy_list=copy.deepcopy(strategies), embedding_lmhead_tp_sp_size=es.tp_sp_size,
                   embedding_lmhead_sp=1 if es.sp_size > 1 else 0,
                   embedding_lmhead_sdp=1 if es.dp_type == DPType.ZERO3 else 0)

    # ---- coarse: one strategy for the whole model -------------------------------------------------------------
    def _coarse(self, gbsz, chunks, pp_size, division, global_mb, layer_strategies):
        opt = self._empty(pp_size)
        total_layers = sum(self.layer_num)
        for idx, ls in enumerate(layer_strategies):
            es = ls.to_embedding_lmhead_strategy()
            (_, other_nosync), other_mem = self._embed_costs(es, gbsz, chunks)
            used, ok, start = [0] * pp_size, True, 0
            for stage in range(pp_size):
                per_layer = []
                for t, n in enumerate(self.layer_num):
                    per_layer += [self._layer_memory(ls, gbsz, chunks, stage, t)] * n
                u = math.ceil(global_mb) + math.ceil(other_mem[stage])
                u += sum(math.ceil(per_layer[i]) for i in range(start, start + division[stage]))
                used[stage] = u
                start += division[stage]
                if u > self.mem_sub_cache:
                    ok = False
                    break
            if not ok:
                self.log("strategy %d %s: out of memory" % (idx, ls))
                continue
            remain = [self.mem_sub_cache - u for u in used]
            used = [u + self.mem_cache for u in used]
            strategies = [ls] * total_layers
            cost = self._pipeline(strategies, division, chunks, gbsz, pp_size, other_nosync)
            if opt["time_cost"] > cost:
                self._record(opt, cost, used, remain, strategies, es)
            self.log("strategy %d %s: pipeline_cost %s, memory_used %s" % (idx, ls, cost, used))
        return opt

    # ---- fine-grained: per-layer strategies by dynamic programming --------------------------------------------
    def _transition_costs(self, gbsz, chunks, pp_size, strategies) -> np.ndarray:
        cfg = self.config
        S, total = len(strategies), sum(self.layer_num)
        inter = np.zeros((total, S, S))
        start = 0
        for t, n in enumerate(self.layer_num):
            res = np.zeros((S, S))
            for a_i, a in enumerate(strategies):
                for b_i, b in enumerate(strategies):
                    if a_i == b_i:
                        continue
                    if cfg.common_train_info.sequence_parallel and a.tp_sp_size != b.tp_sp_size:
                        g = max(a.tp_sp_size, b.tp_sp_size)
                        dp = self.world_size // pp_size // g
                        lbsz = gbsz / chunks / dp
                        sample = self.sequence_len[t] * cfg.model_info.hidden_size * \
                            (4 if cfg.parallelism_info.mixed_precision == "fp32" else 2)
                        res[a_i, b_i] = (g - 1) / g * lbsz * sample
                        key = "%d" % g if ((g == 1 or dp == 1) and "%d" % g in self.comm_coe_dict) else "%d_1" % g
                        res[a_i, b_i] *= self.comm_coe_dict[key] * 1e-7
                    else:
                        # equal width: no data moves; nudge ties towards the plainer strategy
                        if _differs_only_in(a, b, ["sp"]) and b.sp_size > 1:
                            res[a_i, b_i] = 1e-10
                        if _differs_only_in(a, b, ["fsdp"]) and b.dp_type == DPType.ZERO3:
                            res[a_i, b_i] = 1e-9
                        if _differs_only_in(a, b, ["cpt"]) and b.checkpoint:
                            res[a_i, b_i] = 2e-9
                        both = _differs_only_in(a, b, ["fsdp", "cpt"])
                        if both and b.dp_type == DPType.ZERO3 and b.checkpoint:
                            res[a_i, b_i] = 3e-9
                        if both and not _differs_only_in(a, b, ["fsdp"]) and not _differs_only_in(a, b, ["cpt"]) \
                                and a.dp_type == DPType.ZERO3 and b.checkpoint:
                            res[a_i, b_i] = 1e-9
            inter[start:start + n] = res
            start += n
        inter[0] = 0  # nothing precedes the first layer
        return inter

    def _fine(self, gbsz, chunks, pp_size, division, global_mb, strategies, embed_strategies):
        S, total = len(strategies), sum(self.layer_num)
        intra = np.zeros((total, S))
        start = 0
        for t, n in enumerate(self.layer_num):
            row = [LayerTimeCost(s, gbsz, chunks, self.margs[t], self.targs[t], self.pargs[t], self.pmargs[t],
                                 self.hwargs[t], self.logger).gen_result()[0] for s in strategies]
            intra[start:start + n] = np.array(row, dtype=np.float64).reshape(1, -1).repeat(n, axis=0)
            start += n
        # The knapsack table has one row per memory unit.  Budgets up to MEM_TABLE_ROWS MB use 1 MB units (what the
        # reference does for its 24-40 GB budgets); a 180 GB part uses coarser units so that the table keeps that
        # size.  Every amount is rounded up to whole units, so the plan can only over-estimate memory (by less than
        # one unit per layer).
        unit = max(1, math.ceil(self.max_mem / MEM_TABLE_ROWS))
        budget = self.max_mem // unit
        memory = [np.zeros((total, S)) for _ in range(pp_size)]
        for stage in range(pp_size):
            start = 0
            for t, n in enumerate(self.layer_num):
                st = 0 if self.pipeline_type == "gpipe" else stage
                row = np.ceil(np.array([self._layer_memory(s, gbsz, chunks, st, t) for s in strategies]) / unit).astype(np.int32)
                memory[stage][start:start + n] = row.reshape(1, -1).repeat(n, axis=0)
                start += n
        inter = self._transition_costs(gbsz, chunks, pp_size, strategies)
        embed = [self._embed_costs(es, gbsz, chunks) for es in embed_strategies]
        opt = self._empty(pp_size)
        for es, ((other_sync, other_nosync), other_mem) in zip(embed_strategies, embed):
            other_mem = np.ceil((np.asarray(other_mem, dtype=np.float64) + float(global_mb)) / unit).astype(int)
            key = es.tp_sp_size
            chosen, remain_l, used_l, start = [], [], [], 0
            for stage in range(pp_size):
                n = division[stage]
                alg = DPAlg(budget, {key: int(other_mem[stage])}, {key: other_sync[stage]}, n, S, threads=self.threads)
                alg.set_v_and_cost(memory[stage][start:start + n], intra[start:start + n], inter[start:start + n])
                _, picks, remain = alg.fit()
                picks, remain = picks[key], remain[key]
                if remain == -1:
                    chosen.append(None)
                    used_l.append(np.inf)
                else:
                    chosen.append([strategies[i] for i in picks])
                    used_l.append((budget - remain) * unit + self.mem_cache)
                remain_l.append(remain if remain == -1 else remain * unit)
                start += n
            if any(c is None for c in chosen):
                self.log("embedding/lm-head %s: no solution" % es)
                continue
            flat = [s for c in chosen for s in c]
            cost = self._pipeline(flat, division, chunks, gbsz, pp_size, other_nosync)
            if opt["time_cost"] > cost:
                self._record(opt, cost, used_l, remain_l, flat, es)
            self.log("embedding/lm-head %s: pipeline_cost %s" % (es, cost))
        return opt

    def fit(self, gbsz: int, chunks: int, pp_size: int, pp_stage_list: List[int], global_buffer_tp_size: int,
            tp_sp_mode: str, layer_strategy_list: List[LayerStrategy] = None,
            embedding_lmhead_strategy_list: List[EmbeddingLMHeadStrategy] = None) -> Dict[str, Any]:
        self.log("layer strategies: " + format_strategy_list(layer_strategy_list))
        self.log("embedding/lm-head strategies: " + format_strategy_list(embedding_lmhead_strategy_list))
        global_mb = self._global_buffer_mb(gbsz, chunks, pp_size, global_buffer_tp_size, tp_sp_mode)
        if self.config.options_info.fine_grained_mode == 0:
            return self._coarse(gbsz, chunks, pp_size, pp_stage_list, global_mb, layer_strategy_list)
        return self._fine(gbsz, chunks, pp_size, pp_stage_list, global_mb, layer_strategy_list,
                          sorted(embedding_lmhead_strategy_list))
