"""Arch list -> modules of this rank's pipeline stage, each wrapped as a ZeRO unit.

The model is the sequence ``embedding_0, decoder_1 .. decoder_L, prenorm_{L+1}, lm_head_{L+2}`` (MoE:
``moe_decoder_i``) -- the names double as the checkpoint directory names.  Families ``gpt``, ``llama``,
``qwen`` are dense decoders that differ only in their :class:`ModelSpec` (norm, activation, position
embedding, biases); ``mistral`` / ``mixtral`` use the MoE decoder layer.

Capability parity: galvatron/core/runtime/models/builder.py:42-121 (arch list, sequential build),
:124-155 (wrap units), models/arch.py:41-120 (registry / layer shapes),
galvatron/core/runtime/hybrid_parallel_model.py:99-301 (assembly order: groups -> modules -> relocation ->
pipeline -> data-parallel wrap -> checkpoint wrap).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..parallel.groups import GroupFactory, LayerGroups, build_layer_groups, dense_layout, embedding_group_ranks
from ..parallel.reshard import build_reshard
from ..parallel.zero import link_prefetch, ShardedUnit, UnitWrapper
from ..runtime.plan import HybridPlan, LayerPlan
from .modules import (GalvatronCausalLMHead, GalvatronDecoderLayer, GalvatronEmbedding, GalvatronFinalNorm)
from .spec import LayerCtx, ModelSpec

FAMILIES = {"gpt": "decoder", "llama": "decoder", "qwen": "decoder", "mistral": "moe_decoder",
            "mixtral": "moe_decoder"}


def build_causal_lm_arch(spec: ModelSpec) -> List[str]:
    body = "moe_decoder" if spec.is_moe else "decoder"
    return ["embedding"] + [body] * spec.layers + ["prenorm", "lm_head"]


class StageModel(nn.Module):
    """The units of one pipeline stage, with the resharding modules between them."""

    def __init__(self):
        super().__init__()
        self.units = nn.ModuleList()      # UnitWrapper per arch entry of this stage
        self.reshards = nn.ModuleList()   # Reshard or Identity applied *before* the unit of the same index
        self.plans: List[LayerPlan] = []
        self.sharded: List[ShardedUnit] = []
        self.has_embedding = False
        self.has_head = False

    def forward(self, x, labels=None):
        for plan, re, unit in zip(self.plans, self.reshards, self.units):
            if not isinstance(re, nn.Identity):
                x = re(x)
            if plan.kind == "lm_head":
                x = unit(x, labels)
            else:
                x = unit(x)
        return x


class ModelGroups:
    """Process groups of the whole model as seen from this rank."""

    def __init__(self, factory: GroupFactory, plan: HybridPlan, rank: int):
        self.factory, self.plan, self.rank = factory, plan, rank
        self._cache: Dict[Tuple, LayerGroups] = {}
        self.per_layer: List[LayerGroups] = []
        for lp in plan.layers:
            key = (lp.tp, lp.sp, lp.cp, lp.ep if lp.kind == "moe_decoder" else None, lp.etp)
            if key not in self._cache:
                self._cache[key] = build_layer_groups(factory, plan.world_size, plan.pp_deg, lp.tp, lp.sp, lp.cp,
                                                      lp.ep if lp.kind == "moe_decoder" else None, lp.etp)
            self.per_layer.append(self._cache[key])
        base = dense_layout(plan.world_size, plan.pp_deg)
        self.pp = factory.make(base.groups(("pp",)))
        # gradients travel on a communicator of their own, so that each of the two is a one-way FIFO
        self.pp_bwd = factory.make(base.groups(("pp",)), tag="pp_bwd") if plan.pp_deg > 1 else self.pp
        self.embedding = factory.make(embedding_group_ranks(base), allow_absent=True)
        self.stage = base.coord(rank, "pp")
        self.stage_ranks = plan.world_size // plan.pp_deg
        self.layout = base

    def ctx(self, lp: LayerPlan, seq_len: int, fused_comm: bool = False) -> LayerCtx:
        g = self.per_layer[lp.index]
        return LayerCtx(tp=g.tp, sp=g.sp, cp=g.cp, dp=g.dp, sdp=g.sdp, tsp_cp=g.tsp_cp, ep=g.ep, tp_of_ep=g.tp_of_ep,
                        tp_and_ep=g.tp_and_ep, dp_of_ep=g.dp_of_ep, dp_type=lp.dp_type, checkpoint=lp.checkpoint,
                        sequence_parallel=True, seq_len=seq_len, fused_comm=fused_comm, layer_index=lp.index)


def _make_module(lp: LayerPlan, spec: ModelSpec, ctx: LayerCtx, device, tied_weight=None) -> nn.Module:
    if lp.kind == "embedding":
        return GalvatronEmbedding(spec, ctx, device, lp.name)
    if lp.kind == "decoder":
        return GalvatronDecoderLayer(spec, ctx, device, lp.name)
    if lp.kind == "moe_decoder":
        from .moe import GalvatronMoEDecoderLayer

        return GalvatronMoEDecoderLayer(spec, ctx, device, lp.name)
    if lp.kind == "prenorm":
        return GalvatronFinalNorm(spec, ctx, device, lp.name)
    if lp.kind == "lm_head":
        return GalvatronCausalLMHead(spec, ctx, device, lp.name, tied_weight)
    raise KeyError(lp.kind)


def build_stage(spec: ModelSpec, plan: HybridPlan, groups: ModelGroups, device, seed: int = 1234,
                full_init: bool = False, fused_comm: bool = False, reduce_in_fp32: bool = True,
                fused_zero: bool = False) -> StageModel:
    """Instantiate, initialise and wrap the units of this rank's stage."""
    stage = StageModel()
    mine = plan.stage_layers(groups.stage)
    embed_weight = None
    prev_lp = None
    for lp in plan.layers:
        # reshard groups are created collectively by every rank, in arch order
        # (also across a stage boundary: the receiver re-lays-out what the sender shipped in its own layout)
        if prev_lp is not None:
            re = build_reshard(groups.factory, plan.world_size, plan.pp_deg, groups.rank,
                               groups.per_layer[prev_lp.index], groups.per_layer[lp.index], prev_lp, lp,
                               peer=fused_comm)
        else:
            re = None
        if lp.stage == groups.stage:
            ctx = groups.ctx(lp, spec.seq_len, fused_comm)
            tied = embed_weight if (lp.kind == "lm_head" and spec.tied and plan.pp_deg == 1) else None
            mod = _make_module(lp, spec, ctx, device, tied)
            mod.reset_parameters(seed, full_init)
            if lp.kind == "embedding":
                embed_weight = mod.embed_tokens.weight
                stage.has_embedding = True
            if lp.kind == "lm_head":
                stage.has_head = True
            # every gradient is a sum over samples weighted by 1/(samples per *loss* replica): one divisor for
            # all units, the data-parallel degree of the vocab (loss) layers
            dp_size = plan.dp_size(plan.layers[0])
            if lp.kind == "moe_decoder":
                from .moe import wrap_moe_units

                unit = wrap_moe_units(mod, lp, ctx, plan, reduce_in_fp32, fused_zero)
            else:
                tied_over_pp = spec.tied and plan.pp_deg > 1 and lp.kind in ("embedding", "lm_head")
                # a weight tied across stages is summed over the two stages first (engine.sync_tied_embedding_grads):
                # its unit accumulates the whole step in main_grad whatever the reduction mode of the other units
                su = ShardedUnit(mod, lp.name, ctx.sdp, dp_size, lp.dp_type, reduce_in_fp32, tp=ctx.tp,
                                 defer_sync=plan.async_grad_reduce or tied_over_pp, fused_zero=fused_zero)
                su.reduce_at_step_only = tied_over_pp
                if lp.kind == "lm_head" and spec.tied and plan.pp_deg > 1:
                    su.count_in_norm = False  # the first stage's copy of the tied weight carries the norm
                stage.sharded.append(su)
                unit = UnitWrapper(mod, su, checkpoint=lp.checkpoint)
                if tied is not None:
                    unit.extra_units.append(tied._hg_unit)
            if hasattr(unit, "sharded_units"):
                stage.sharded.extend(unit.sharded_units)
            stage.units.append(unit)
            stage.reshards.append(re if re is not None else nn.Identity())
            stage.plans.append(lp)
        prev_lp = lp
    flat = []
    for u in stage.units:
        flat.extend(getattr(u, "wrappers", [u]))
    link_prefetch(flat)
    return stage
