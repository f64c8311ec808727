"""From arguments (GLOBAL flags or a searched strategy JSON) to the per-layer execution plan.

``build_plan(args, world_size)`` returns a :class:`HybridPlan`: one :class:`LayerPlan` per entry of the
model's arch list (embedding, L decoder layers, final norm, LM head) with its pipeline stage, tensor /
sequence / context-parallel degrees, ZeRO type and checkpoint flag, plus batch geometry (global batch,
chunks) and pipeline division.  ``plan.as_config_dict()`` gives the dictionary layout of the
reference (``pp_deg, tp_sizes_enc, tp_consecutive_flags, cp_sizes_enc, dp_types_enc, ep_sizes_enc,
tp_of_ep_sizes_enc, checkpoint_flags_enc, pp_ranks_enc, pp_division, use_sp, vocab_tp, vocab_sp, vocab_cp,
default_dp_type, global_batch_size``), which is also what is written to ``hybrid_parallel_configs.json``
next to a distributed checkpoint and compared on resume.

Capability parity: galvatron/core/runtime/hybrid_parallel_config.py:18-184 (modes, validation),
:229-314 (whole-model expansion, Ulysses swap), :359-369 (chunks heuristic).  One deliberate fix: the
searched ``embed_sdp`` flag is honoured (the reference writes ``embed_sdp`` but reads ``vocab_sdp``).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..search.strategy import array2str, config2strategy, str2array


@dataclass
class LayerPlan:
    kind: str                 # embedding | decoder | moe_decoder | prenorm | lm_head
    name: str                 # module name in the checkpoint layout, e.g. decoder_3
    stage: int
    tp: int = 1
    sp: int = 1
    cp: int = 1
    dp_type: str = "ddp"
    checkpoint: bool = False
    ep: int = 1
    etp: int = 1
    index: int = 0            # position in the arch list


@dataclass
class HybridPlan:
    world_size: int
    pp_deg: int
    layers: List[LayerPlan]
    pp_division: List[int]
    global_batch_size: int
    chunks: int
    pipeline_type: str
    default_dp_type: str
    vocab_tp: int
    vocab_sp: int
    vocab_cp: int
    vocab_sdp: int
    mixed_precision: str = "bf16"
    async_grad_reduce: bool = True
    is_moe: bool = False
    source: str = "GLOBAL"

    @property
    def decoder_layers(self) -> List[LayerPlan]:
        return [l for l in self.layers if l.kind in ("decoder", "moe_decoder")]

    def stage_layers(self, stage: int) -> List[LayerPlan]:
        return [l for l in self.layers if l.stage == stage]

    def dp_size(self, lp: LayerPlan) -> int:
        return self.world_size // self.pp_deg // (lp.tp * lp.sp * lp.cp)

    def as_config_dict(self) -> Dict[str, Any]:
        dec = self.decoder_layers
        return {
            "is_moe_model": self.is_moe,
            "pp_deg": self.pp_deg,
            "tp_sizes_enc": [max(l.tp, l.sp) for l in dec],
            "tp_consecutive_flags": [1] * len(dec),
            "cp_sizes_enc": [l.cp for l in dec],
            "dp_types_enc": [1 if l.dp_type == "zero3" else 0 for l in dec],
            "ep_sizes_enc": [l.ep for l in dec],
            "tp_of_ep_sizes_enc": [l.etp for l in dec],
            "checkpoint_flags_enc": [int(l.checkpoint) for l in dec],
            "pp_ranks_enc": [l.stage for l in dec],
            "pp_division": list(self.pp_division),
            "use_sp": [1 if l.sp > 1 else 0 for l in dec],
            "vocab_tp": self.vocab_tp,
            "vocab_sp": self.vocab_sp,
            "vocab_cp": self.vocab_cp,
            "default_dp_type": self.default_dp_type,
            "global_batch_size": self.global_batch_size,
        }

    def short_name(self) -> str:
        """One-line name of the plan, e.g. ``dp8-zero2``, ``pp2-tp2-dp2-zero3-ckpt16`` (decoder layers only; a
        mixed plan lists each distinct layer strategy with its layer count)."""
        kinds: Dict[str, int] = {}
        for l in self.layers:
            if l.kind not in ("decoder", "moe_decoder"):
                continue
            parts = []
            if l.tp > 1:
                parts.append("tp%d" % l.tp)
            if l.sp > 1:
                parts.append("sp%d" % l.sp)
            if l.cp > 1:
                parts.append("cp%d" % l.cp)
            if l.kind == "moe_decoder" and l.ep > 1:
                parts.append("ep%d" % l.ep)
            d = self.dp_size(l)
            parts.append("dp%d" % d)
            if d > 1 or l.dp_type != "ddp":
                parts.append(l.dp_type if d > 1 else "ddp")
            if l.checkpoint:
                parts.append("ckpt")
            key = "-".join(p for p in parts if p != "ddp")
            kinds[key] = kinds.get(key, 0) + 1
        body = "+".join(k if len(kinds) == 1 else "%sx%d" % (k, c) for k, c in kinds.items())
        return ("pp%d-" % self.pp_deg if self.pp_deg > 1 else "") + body

    def describe(self) -> str:
        lines = ["pp=%d  gbsz=%d  chunks=%d  pipeline=%s  default_dp=%s  vocab(tp=%d sp=%d cp=%d sdp=%d)" % (
            self.pp_deg, self.global_batch_size, self.chunks, self.pipeline_type, self.default_dp_type, self.vocab_tp,
            self.vocab_sp, self.vocab_cp, self.vocab_sdp)]
        for l in self.layers:
            lines.append("  %-12s stage %d  tp %d sp %d cp %d dp %d %-5s%s%s" % (
                l.name, l.stage, l.tp, l.sp, l.cp, self.dp_size(l), l.dp_type, " ckpt" if l.checkpoint else "",
                (" ep %d etp %d" % (l.ep, l.etp)) if l.kind == "moe_decoder" else ""))
        return "\n".join(lines)


def default_chunks(local_bsz: int, pp_deg: int) -> int:
    """``chunks = -1``: one micro-batch without pipelining, else micro-batches of (about) 4 samples."""
    if pp_deg <= 1:
        return 1
    return max(1, math.ceil(local_bsz / 4))


def pp_division_even(num_layers: int, pp_deg: int) -> List[int]:
    avg = num_layers // pp_deg
    return [avg] * (pp_deg - 1) + [num_layers - avg * (pp_deg - 1)]


def build_plan(args, world_size: int) -> HybridPlan:
    par, model, train = args.parallel, args.model, args.train
    L = model.num_layers
    is_moe = bool(model.is_moe_model or model.num_moe_experts)
    path = par.galvatron_config_path
    if path in (None, "None"):
        source = "GLOBAL"
        pp = par.pp_deg
        tps = [max(1, par.global_tp_deg)] * L
        cps = [max(1, par.global_cp_deg)] * L
        dpt = [int(par.sdp)] * L
        eps_, etps = [par.global_ep_deg] * L, [par.global_tp_of_ep_deg] * L
        ckpt = [int(par.global_checkpoint)] * L
        use_sp = [1 if par.use_ulysses else 0] * L
        division = None
        vtp, vcp = par.vocab_tp, par.vocab_cp
        vsp = 1 if par.use_ulysses else 0
        gbsz, chunks = train.global_batch_size, train.chunks
        vocab_sdp = int(par.vocab_sdp)
    else:
        cfg = path if isinstance(path, dict) else json.load(open(path))
        source = "JSON" if isinstance(path, dict) else "JSON %s" % path
        pp, tps, cps, _consec, dpt, use_sp, vtp, vsp, vcp = config2strategy(cfg)
        if len(tps) != L:
            raise ValueError("strategy JSON has %d layers, the model has %d" % (len(tps), L))
        gbsz, chunks = cfg["global_bsz"], cfg["chunks"]
        ckpt = str2array(cfg["checkpoint"]) if "checkpoint" in cfg else [0] * L
        division = str2array(cfg["pp_division"]) if "pp_division" in cfg else None
        eps_ = str2array(cfg["ep_sizes_enc"]) if "ep_sizes_enc" in cfg else [1] * L
        etps = str2array(cfg["tp_of_ep_sizes_enc"]) if "tp_of_ep_sizes_enc" in cfg else [1] * L
        par.pipeline_type = cfg.get("pipeline_type", par.pipeline_type)
        par.default_dp_type = cfg.get("default_dp_type", par.default_dp_type)
        vocab_sdp = int(cfg.get("vocab_sdp", cfg.get("embed_sdp", par.vocab_sdp)))
        par.vocab_sdp = vocab_sdp
        train.global_batch_size, train.chunks = gbsz, chunks
        par.pp_deg, par.vocab_tp, par.vocab_sp, par.vocab_cp = pp, vtp, vsp, vcp
        for key in ("fused_comm", "fused_zero", "async_grad_reduce", "reduce_in_fp32"):   # optional runtime switches
            if key in cfg and cfg[key] is not None:
                setattr(par, key, bool(cfg[key]))
    if division is None:
        division = pp_division_even(L, pp)
    if sum(division) != L or len(division) != pp:
        raise ValueError("pp_division %s does not cover %d layers in %d stages" % (division, L, pp))
    if world_size % pp:
        raise ValueError("world size %d not divisible by pp_deg %d" % (world_size, pp))
    per_stage = world_size // pp
    min_tp = min(min(tps), max(1, vtp))
    min_cp = min(min(cps), max(1, vcp))
    if gbsz is None:
        raise ValueError("global_batch_size is not set")
    if gbsz % (per_stage // min_tp // min_cp):
        raise ValueError("global_batch_size %d must be a multiple of world/pp/min_tp/min_cp = %d" % (
            gbsz, per_stage // min_tp // min_cp))
    stage_of = []
    for s, n in enumerate(division):
        stage_of += [s] * n
    default = par.default_dp_type
    layers: List[LayerPlan] = []
    vocab_dp_type = "zero3" if vocab_sdp else default
    v_tp, v_sp = (1, max(1, vtp)) if vsp else (max(1, vtp), 1)
    layers.append(LayerPlan("embedding", "embedding_0", 0, v_tp, v_sp, max(1, vcp), vocab_dp_type, False, index=0))
    for i in range(L):
        width = tps[i]
        if width * cps[i] > per_stage:
            raise ValueError("layer %d: tp*cp = %d exceeds the %d ranks of a stage" % (i, width * cps[i], per_stage))
        tp, sp = (1, width) if use_sp[i] else (width, 1)
        kind = "moe_decoder" if is_moe else "decoder"
        layers.append(LayerPlan(kind, "%s_%d" % (kind, i + 1), stage_of[i], tp, sp, cps[i],
                                "zero3" if dpt[i] else default, bool(ckpt[i]), eps_[i], etps[i], index=i + 1))
    layers.append(LayerPlan("prenorm", "prenorm_%d" % (L + 1), pp - 1, v_tp, v_sp, max(1, vcp), vocab_dp_type, False,
                            index=L + 1))
    layers.append(LayerPlan("lm_head", "lm_head_%d" % (L + 2), pp - 1, v_tp, v_sp, max(1, vcp), vocab_dp_type, False,
                            index=L + 2))
    if chunks is None or chunks < 1:
        local = gbsz // (per_stage // min_tp // min_cp)
        chunks = default_chunks(local, pp)
    return HybridPlan(world_size, pp, layers, division, gbsz, chunks, par.pipeline_type, default, max(1, vtp),
                      int(bool(vsp)), max(1, vcp), vocab_sdp, par.mixed_precision, par.async_grad_reduce, is_moe,
                      source)


def check_checkpoint_compatibility(plan: HybridPlan, ckpt_dir: str):
    """A distributed checkpoint stores per-rank optimizer shards, so it can only be resumed under the very
    same strategy: compare with the ``hybrid_parallel_configs.json`` saved beside it."""
    path = os.path.join(ckpt_dir, "hybrid_parallel_configs.json")
    if not os.path.exists(path):
        return
    saved = json.load(open(path))
    mine = json.loads(json.dumps(plan.as_config_dict()))
    diff = [k for k in mine if k in saved and saved[k] != mine[k] and k != "global_batch_size"]
    if diff:
        raise ValueError("the checkpoint in %s was written under a different parallel strategy (differs in: %s)" % (
            ckpt_dir, ", ".join(diff)))
