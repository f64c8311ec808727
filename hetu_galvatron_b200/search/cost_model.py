"""Analytic time / memory cost models of the planner.

Inputs come from the profilers: per-layer forward time (ms per sample, or a linear fit in the local
batch), per-layer parameter size and per-sample activation footprint per tensor-parallel degree, the
embedding + LM-head ("other") time / model states / activations, all-reduce bandwidth coefficients
(ms per MB per group size), message-size -> latency tables for all-gather and all-to-all, p2p
coefficients and the compute / communication overlap slow-down.

Outputs: seconds per layer (with and without gradient synchronisation), MB per layer, and the
pipeline-composed iteration time.  The formulas follow the reference term by term so that its golden
search results are reproduced (galvatron/core/cost_model/components/layer_cost.py:58-328,
components/embedding_lmhead_cost.py:9-313, cost_model_handler.py:16-98, cost_model_args.py:5-51); the
B200 refit changes the *inputs* (measured fused-kernel tables, backward/forward ratio, overlap
coefficient), not the structure.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from .strategy import DPType, EmbeddingLMHeadStrategy, LayerStrategy

Number = Union[float, np.ndarray]


# ---- argument bundles (one set per layer type) -----------------------------------------------------
@dataclass
class ModelArgs:
    parameter_size: float = 48          # MB of one layer's parameters (fp32)
    seq_length: int = 1024
    hidden_size: int = 4096
    layer_num: int = 16


@dataclass
class TrainArgs:
    mixed_precision: bool = False
    checkpoint: bool = False
    async_grad_reduce: bool = True
    pytorch_context_mem: int = 1024     # MB held by the CUDA context / allocator per process


@dataclass
class ParallelArgs:
    use_zero2_for_dp: bool = False
    sequence_parallel: bool = False
    pipeline_type: str = "gpipe"
    optimal_chunk_func: Optional[Callable] = None
    chunks: Optional[int] = None


@dataclass
class ProfileModelArgs:
    tp_activation_per_bsz_dict: dict = field(default_factory=lambda: {1: 85, 2: 47, 4: 28, 8: 18.5})
    other_memory_pp_off: dict = field(default_factory=lambda: {"model_states": 640, "activation": 320})
    other_memory_pp_on: dict = field(default_factory=lambda: {
        "first_stage": {"model_states": 640, "activation": 320},
        "last_stage": {"model_states": 640, "activation": 320}})
    forward_computation_time: Optional[Number] = 35 / 24
    other_time_profiled: Optional[Number] = 0
    # B200 refit: measured backward/forward ratio of a layer (the reference fixes it to 2)
    backward_forward_ratio: Optional[float] = None


@dataclass
class ProfileHardwareArgs:
    bct_fct_coe: float = 2
    extra_overhead: float = 0
    comm_coe_dict: dict = field(default_factory=dict)
    dp_overlap_coe: float = 1.3
    bct_overlap_coe: float = 1.3
    p2p_comm_coe_dict: dict = field(default_factory=dict)
    allreduce_dict: dict = field(default_factory=dict)
    all2all_dict: dict = field(default_factory=dict)
    costmodel_coe: float = 1.0
    overlap_slowdown_coe: float = 1.0
    allreduce_latency_per_MB_dict: dict = field(default_factory=dict)
    allreduce_message_size_to_latency_dict_dict: dict = field(default_factory=dict)
    allgather_message_size_to_latency_dict_dict: dict = field(default_factory=dict)
    all2all_message_size_to_latency_dict_dict: dict = field(default_factory=dict)
    # B200 refit: fraction of the TP/SP collective time that the fused compute+collective kernels hide
    fused_comm_hidden_fraction: object = 0.0      # a float, or {tp degree: float}
    # B200 refit: optimizer step of one unsharded layer in ms (memory-bound AdamW + norm; scales with 1/sdp under ZeRO)
    optimizer_ms_per_layer: float = 0.0


def _line(x, m, c):
    return m * x + c


def _lookup_latency(table: dict, size_mb: float) -> float:
    """Measured latency of a message of ``size_mb`` MB, or the table's linear fit."""
    if size_mb in table:
        return table[size_mb]
    return _line(size_mb, *table["popt"])


def zero_ratios(chunks: int, mixed_precision: bool, async_grad_reduce: bool):
    """Fractions of the 4x-parameter model states a rank keeps under ZeRO-2 / ZeRO-3 over ``d`` ranks.

    With more than one micro-batch and deferred reduction the full gradient buffer survives the
    accumulation (ZeRO-2 behaves like ZeRO-1, ZeRO-3 keeps unsharded gradients); with immediate
    reduction an fp32 reduction buffer adds a quarter."""
    if chunks == 1:
        z2 = (lambda d: 7 / 8 * (1 / d + 0.003) + 1 / 8) if mixed_precision else (lambda d: 3 / 4 * (1 / d + 0.003) + 1 / 4)
        z3 = lambda d: 1 / d + 0.003
    elif async_grad_reduce:
        z2 = (lambda d: 6 / 8 * (1 / d + 0.003) + 2 / 8) if mixed_precision else (lambda d: 2 / 4 * (1 / d + 0.003) + 2 / 4)
        z3 = (lambda d: 7 / 8 * (1 / d + 0.003) + 1 / 8) if mixed_precision else (lambda d: 3 / 4 * (1 / d + 0.003) + 1 / 4)
    else:
        z2 = (lambda d: (7 / 8 * (1 / d + 0.003) + 1 / 8) * 5 / 4) if mixed_precision else (lambda d: 3 / 4 * (1 / d + 0.003) + 1 / 4)
        z3 = lambda d: (1 / d + 0.003) * 5 / 4
    return z2, z3


def in_flight_microbatches(pp: int, stage: int, chunks: int, pipeline_type: str) -> int:
    if pp == 1:
        return 1
    if chunks < pp:
        raise AssertionError("chunks %d must be >= pp_size %d" % (chunks, pp))
    return pp - stage if pipeline_type == "pipedream_flush" else chunks


# ---- per-layer time ------------------------------------------------------------------------------------
class LayerTimeCost:
    """Seconds per layer for one strategy."""

    def __init__(self, strategy: LayerStrategy, global_batch_size: int, chunks: int, model_args: ModelArgs,
                 train_args: TrainArgs, parallel_args: ParallelArgs, profile_model_args: ProfileModelArgs,
                 profile_hardware_args: ProfileHardwareArgs, logger=None):
        s, hw, pm = strategy, profile_hardware_args, profile_model_args
        self.s, self.hw = s, hw
        L = model_args.layer_num
        self.L = L
        self.lbsz = global_batch_size // chunks // s.dp_size  # data-parallel (not sdp) split of the batch
        self.chunks = max(1, int(chunks))
        w = s.tp_sp_size
        # computation
        fwd = pm.forward_computation_time
        if isinstance(fwd, np.ndarray):
            self.fct = _line(self.lbsz / w, *fwd) * L
        else:
            self.fct = fwd * self.lbsz / w * L
        ratio = pm.backward_forward_ratio if pm.backward_forward_ratio is not None else hw.bct_fct_coe
        self.bct = self.fct * ratio
        if s.checkpoint:
            self.bct += self.fct
        # data-parallel gradient traffic
        param_mb = model_args.parameter_size / s.tp_size
        sdp = s.sdp_size
        self.dp_msg = 2 * (sdp - 1) * (param_mb / sdp) * L
        if train_args.mixed_precision:
            self.dp_msg /= 2
        self.zero3_gather_msg = self.dp_msg * 0.5
        key = "%d_0" % sdp if s.tp_size != 1 else "%d_1" % sdp
        self.dc = hw.allreduce_latency_per_MB_dict[key]
        self.dc_overlap = self.dc * hw.dp_overlap_coe
        # tensor / sequence-parallel collectives
        if w == 1:
            self.tp_time = 0
        else:
            if s.tp_size == 1:   # Ulysses: 2 all-to-all forward + 2 backward per layer
                n, table = 4 * L, hw.all2all_message_size_to_latency_dict_dict[s.sp_size]
            else:                # Megatron TP+SP: 3 exposed all-gather-sized collectives in attention, 3 in the MLP
                n, table = 6 * L, hw.allgather_message_size_to_latency_dict_dict[s.tp_size]
            if s.checkpoint:
                n *= 1.5
            msg = self.lbsz * model_args.seq_length * model_args.hidden_size * (2 if train_args.mixed_precision else 4) / 1024 / 1024
            hidden = hw.fused_comm_hidden_fraction
            if isinstance(hidden, dict):      # measured per degree; only the Megatron-TP path has fused GEMM kernels
                hidden = hidden.get(s.tp_size, 0.0) if s.tp_size > 1 else 0.0
            self.tp_time = _lookup_latency(table, msg) * n * (1.0 - hidden)
        # pipeline p2p
        self.p2p_coe = None
        if s.pp_size > 1 and hw.p2p_comm_coe_dict is not None:
            self.p2p_coe = hw.p2p_comm_coe_dict[s.pp_size]
            self.p2p_msg = s.pp_size * 2 * self.lbsz * model_args.seq_length * model_args.hidden_size * 4 / 1024 / 1024
            if train_args.mixed_precision:
                self.p2p_msg /= 2

    def _overlap(self, dp_msg, bct) -> Tuple[float, float]:
        """Backward compute and gradient reduction slow each other down while they overlap."""
        comm_t = dp_msg * self.dc_overlap
        comp_t = bct * self.hw.bct_overlap_coe
        if comm_t > comp_t:
            return comp_t, (dp_msg - comp_t / self.dc_overlap) * self.dc
        if comm_t < comp_t:
            return comm_t, bct - comm_t / self.hw.bct_overlap_coe
        return comp_t, 0

    def result(self, no_gradient_sync: bool = False) -> float:
        s, hw = self.s, self.hw
        factor = 0 if no_gradient_sync else 1
        w = s.tp_sp_size
        if w == 1 and s.dp_size > 1:
            a, b = self._overlap(self.dp_msg * factor, self.bct)
            res = self.fct + a + b + hw.extra_overhead
        elif s.dp_size == 1 and w > 1:
            res = self.fct + self.bct + self.tp_time
        elif s.dp_size == 1 and w == 1:
            res = self.fct + self.bct
        else:
            a, b = self._overlap(self.dp_msg * factor, self.bct)
            res = self.fct + a + b + self.tp_time + hw.extra_overhead
        if s.dp_type == DPType.ZERO3:
            res = res + self.zero3_gather_msg * self.dc
        if hw.optimizer_ms_per_layer:
            shard = s.sdp_size if s.dp_type in (DPType.ZERO2, DPType.ZERO3) else 1
            # a per-step cost; this result is one micro-batch's share (the pipeline model multiplies it by `chunks`)
            res = res + hw.optimizer_ms_per_layer * self.L / (s.tp_size * shard) / self.chunks
        if s.pp_size > 1 and self.p2p_coe is not None:
            res = res + self.p2p_msg * self.p2p_coe
        return res * 0.001 * hw.costmodel_coe / self.L

    def gen_result(self) -> Tuple[float, float]:
        return self.result(False), self.result(True)


# ---- per-layer memory ----------------------------------------------------------------------------------
class LayerMemoryCost:
    def __init__(self, strategy: LayerStrategy, global_batch_size: int, chunks: int, stage_idx: int = 0,
                 model_args: ModelArgs = None, train_args: TrainArgs = None, parallel_args: ParallelArgs = None,
                 profile_model_args: ProfileModelArgs = None, logger=None):
        s = strategy
        lbsz = global_batch_size // chunks // s.dp_size
        held = in_flight_microbatches(s.pp_size, stage_idx, chunks, parallel_args.pipeline_type) * lbsz
        z2, z3 = zero_ratios(chunks, train_args.mixed_precision, train_args.async_grad_reduce)
        self.parameter = model_args.parameter_size / s.tp_size
        self.model_states = 4 * self.parameter
        if s.dp_type == DPType.ZERO3:
            self.model_states *= z3(s.sdp_size)
        elif s.dp_type == DPType.ZERO2:
            self.model_states *= z2(s.sdp_size)
        acts = profile_model_args.tp_activation_per_bsz_dict
        if s.checkpoint:
            self.activation = acts["checkpoint"] * held
            if s.sp_size > 1 or (s.tp_size > 1 and parallel_args.sequence_parallel):
                self.activation /= s.tp_sp_size
        else:
            self.activation = acts[s.tp_sp_size] * held

    def get_memory_cost(self) -> Dict[str, float]:
        return {"parameter": self.parameter, "model_states": self.model_states, "activation": self.activation,
                "enc_total": self.model_states + self.activation}


# ---- embedding + LM head ---------------------------------------------------------------------------------
class EmbeddingLMHeadTimeCost:
    """Seconds per pipeline stage spent in the embedding (first stage) and norm + LM head (last stage)."""

    def __init__(self, strategy: EmbeddingLMHeadStrategy, global_batch_size: int, chunks: int,
                 sequence_length_list: Sequence[int], model_args: ModelArgs, train_args: TrainArgs,
                 parallel_args: ParallelArgs, profile_model_args: ProfileModelArgs,
                 profile_hardware_args: ProfileHardwareArgs, logger=None):
        s, hw, pm = strategy, profile_hardware_args, profile_model_args
        self.s, self.hw = s, hw
        pp = s.pp_size
        lbsz = global_batch_size // chunks // s.dp_size
        other = pm.other_time_profiled
        if isinstance(other, np.ndarray):
            t = _line(lbsz / s.tp_sp_size / s.cp_size, *other)
        else:
            t = other * lbsz / s.tp_sp_size / s.cp_size
        self.fct = [0] * pp
        if pp == 1:
            self.fct[0] = t
        else:
            self.fct[0] = self.fct[-1] = t / 2
        key = "%d_0" % s.sdp_size if s.tp_size != 1 else "%d_1" % s.sdp_size
        self.dp_coe = hw.allreduce_latency_per_MB_dict[key] * (s.sdp_size - 1) / s.sdp_size
        f = 0.5 if train_args.mixed_precision else 1.0
        self.dp_msg = [0] * pp
        if pp == 1:
            self.dp_msg[0] = pm.other_memory_pp_off["model_states"][s.tp_size] / 4 * f
        else:
            self.dp_msg[0] = pm.other_memory_pp_on["first_stage"]["model_states"][s.tp_size] / 4 * f
            self.dp_msg[-1] = pm.other_memory_pp_on["last_stage"]["model_states"][s.tp_size] / 4 * f
        self.fwd_factor, self.bwd_factor = (0.5, 1.0) if s.dp_type == DPType.ZERO3 else (0.0, 0.5)
        per_seq = []
        for seq in sequence_length_list:
            if s.tp_sp_size == 1 or s.tp_size == 1:
                per_seq.append(0)
            else:
                if not parallel_args.sequence_parallel:
                    raise AssertionError("sequence_parallel must be on when the vocab layers use tp > 1")
                msg = lbsz * seq * model_args.hidden_size * (2 if train_args.mixed_precision else 4) / 1024 / 1024
                per_seq.append(_lookup_latency(hw.allgather_message_size_to_latency_dict_dict[s.tp_size], msg))
        self.tp_time = [0] * pp
        if pp == 1:
            self.tp_time[0] = per_seq[0] + per_seq[-1]
        else:
            self.tp_time[0], self.tp_time[-1] = per_seq[0], per_seq[-1]

    def _overlapped(self, fwd_comm, fwd_comp, bwd_comm, bwd_comp, tp_time):
        k = self.hw.dp_overlap_coe
        fc, bc = fwd_comp * k, bwd_comp * k
        fwd = fwd_comm + (fc - fwd_comm) / k if fc > fwd_comm else fwd_comm
        bwd = bwd_comm + (bc - bwd_comm) / k if bc > bwd_comm else bwd_comm
        return fwd + bwd + tp_time

    def gen_result(self) -> Tuple[List[float], List[float]]:
        pp = self.s.pp_size
        with_sync, no_sync = [0] * pp, [0] * pp
        for i in ([0] if pp == 1 else [0, -1]):
            comm = self.dp_msg[i] * self.dp_coe
            bwd_comp = self.fct[i] * self.hw.bct_fct_coe
            with_sync[i] = 0.001 * self._overlapped(comm * self.fwd_factor, self.fct[i], comm * self.bwd_factor,
                                                    bwd_comp, self.tp_time[i])
            no_sync[i] = 0.001 * self._overlapped(comm * self.fwd_factor, self.fct[i], comm * (self.bwd_factor - 0.5),
                                                  bwd_comp, self.tp_time[i])
        return with_sync, no_sync


class EmbeddingLMHeadMemoryCost:
    def __init__(self, strategy: EmbeddingLMHeadStrategy, global_batch_size: int, chunks: int,
                 model_args: ModelArgs = None, train_args: TrainArgs = None, parallel_args: ParallelArgs = None,
                 profile_model_args: ProfileModelArgs = None, logger=None):
        s, pm = strategy, profile_model_args
        pp = s.pp_size
        lbsz = global_batch_size // chunks // s.dp_size
        z2, z3 = zero_ratios(chunks, train_args.mixed_precision, train_args.async_grad_reduce)
        scale = z3(s.sdp_size) if s.dp_type == DPType.ZERO3 else (z2(s.sdp_size) if s.dp_type == DPType.ZERO2 else 1.0)
        self.model_states, self.activation = [0] * pp, [0] * pp
        if pp == 1:
            self.model_states[0] = pm.other_memory_pp_off["model_states"][s.tp_size] * scale
            self.activation[0] = pm.other_memory_pp_off["activation"][s.tp_sp_size] * lbsz
        else:
            if chunks < pp:
                raise AssertionError("chunks %d must be >= pp_size %d" % (chunks, pp))
            first, last = (pp, 1) if parallel_args.pipeline_type == "pipedream_flush" else (chunks, chunks)
            self.model_states[0] = pm.other_memory_pp_on["first_stage"]["model_states"][s.tp_size] * scale
            self.model_states[-1] = pm.other_memory_pp_on["last_stage"]["model_states"][s.tp_size] * scale
            self.activation[0] = pm.other_memory_pp_on["first_stage"]["activation"][s.tp_sp_size] * first * lbsz
            self.activation[-1] = pm.other_memory_pp_on["last_stage"]["activation"][s.tp_sp_size] * last * lbsz
        self.context = [train_args.pytorch_context_mem] * pp

    def get_memory_cost(self) -> Dict[str, List[float]]:
        return {"model_states": self.model_states, "activation": self.activation,
                "pytorch_context_mem": self.context,
                "enc_total": [a + b + c for a, b, c in zip(self.model_states, self.activation, self.context)]}


# ---- pipeline composition ----------------------------------------------------------------------------------
def stage_sums(layer_costs: Sequence[float], division: Sequence[int]) -> List[float]:
    if int(np.sum(division)) != len(layer_costs):
        raise AssertionError("pipeline division does not cover the layers")
    out, start = [], 0
    for n in division:
        out.append(np.sum(layer_costs[start:start + n]))
        start += n
    return out


def pipeline_costmodel(layer_num_list, model_args_list, train_args_list, parallel_args_list, profile_model_args_list,
                       profile_hardware_args_list, strategy_list: List[LayerStrategy], partition, chunks, gbsz,
                       pp_size, other_time_cost, logger=None, return_stage_cost=False):
    """Iteration time (s) of a per-layer strategy assignment under a pipeline partition.

    Steady state: every stage's compute once plus ``chunks - 1`` repetitions of the last stage; lower
    bounded by the warm-up / cool-down schedule of the first stage; plus the part of the gradient
    reduction that sticks out behind the last backward."""
    types = []
    for t, n in enumerate(layer_num_list):
        types += [t] * n
    if len(strategy_list) != len(types):
        raise AssertionError("strategy list (%d) != layers (%d)" % (len(strategy_list), len(types)))
    cache: Dict[Tuple[int, LayerStrategy], Tuple[float, float]] = {}
    sync, nosync = [], []
    for t, s in zip(types, strategy_list):
        if (t, s) not in cache:
            cache[(t, s)] = LayerTimeCost(s, gbsz, chunks, model_args_list[t], train_args_list[t], parallel_args_list[t],
                                          profile_model_args_list[t], profile_hardware_args_list[t], logger).gen_result()
        sync.append(cache[(t, s)][0])
        nosync.append(cache[(t, s)][1])
    stage_sync = stage_sums(sync, partition)
    stage_comp = stage_sums(nosync, partition)
    if len(other_time_cost) != len(stage_comp):
        raise AssertionError("other_time_cost must have one entry per stage")
    for i, t in enumerate(other_time_cost):
        stage_comp[i] += t
    result = np.sum(stage_comp) + stage_comp[-1] * (chunks - 1)
    ramp = min(pp_size - 1, chunks - 1) * stage_comp[0]
    rest = np.sum(stage_comp[1:])
    result = max(result, max(ramp * 1 / 3, rest * 1 / 3) + max(ramp * 2 / 3, rest * 2 / 3) +
                 stage_comp[0] * max(0, chunks + 1 - pp_size))
    tail = [stage_sync[i] - np.sum(stage_comp[:i + 1]) for i in range(pp_size)]
    reduce_time = np.max(tail)
    result += reduce_time if reduce_time > 0 else 0
    if return_stage_cost:
        return stage_sync, result
    return result
