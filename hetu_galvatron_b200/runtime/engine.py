"""``GalvatronModel``: the assembled hybrid-parallel model and its training step.

    model = build_model(args)                      # groups, stage modules, ZeRO units, pipeline engine
    loss  = model.forward_backward(batch, iter, profiler, loss_func, labels=..., loss_mask=...)
    optimizer.step()

``batch`` is this rank's share of the global batch (``[B_local, S]`` token ids, split over the vocab
layers' data-parallel group by the data loader); the engine slices the sequence for context parallelism,
cuts micro-batches, runs the schedule (no-PP accumulation / GPipe / 1F1B-flush) and returns the mean loss
of the step (a 0-dim device tensor; the caller decides when to read it).

Capability parity: galvatron/core/runtime/hybrid_parallel_model.py:51-97 (``forward_backward``, loss
reduction), :99-301 (assembly), models/builder.py:158-187 (``build_model``).
"""
from __future__ import annotations

import os
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from ..config.model_config import resolve_model_config
from ..models.builder import ModelGroups, StageModel, build_stage
from ..models.spec import ModelSpec, spec_from_args
from ..parallel.groups import GroupFactory
from ..parallel.pipeline import PipelineEngine, chunk_batch
from .plan import HybridPlan, build_plan


def default_loss_func(loss_mask: Optional[torch.Tensor], cp: int = 1) -> Callable:
    """``sum(loss * mask) / sum(mask)`` over this rank's tokens, pre-divided by the context-parallel
    degree because gradients are summed (not averaged) over the cp ranks."""

    def fn(per_token_loss: torch.Tensor) -> torch.Tensor:
        if loss_mask is None:
            return per_token_loss.float().mean() / cp
        m = loss_mask.to(per_token_loss.dtype)
        return (per_token_loss * m).sum() / m.sum().clamp(min=1) / cp

    return fn


class GalvatronModel:
    def __init__(self, args, spec: ModelSpec, plan: HybridPlan, groups: ModelGroups, stage: StageModel, device):
        self.args, self.spec, self.plan, self.groups, self.model, self.device = args, spec, plan, groups, stage, device
        self.engine = PipelineEngine(stage, groups, plan, spec, device)
        self.vocab_ctx = groups.ctx(plan.layers[0], spec.seq_len)
        self.iter = 0

    # ---- introspection ------------------------------------------------------------------------------------
    @property
    def sharded_units(self):
        return self.model.sharded

    def parameters(self):
        return self.model.parameters()

    def named_units(self):
        return [(lp.name, u) for lp, u in zip(self.model.plans, self.model.units)]

    @property
    def is_first_stage(self):
        return self.engine.first

    @property
    def is_last_stage(self):
        return self.engine.last

    def local_batch_size(self) -> int:
        lp = self.plan.layers[0]
        return self.plan.global_batch_size // self.plan.dp_size(lp)

    # ---- training step ------------------------------------------------------------------------------------
    def forward_backward(self, batch, iter: int = 0, profiler=None, loss_func: Optional[Callable] = None,
                         labels: Optional[torch.Tensor] = None, loss_mask: Optional[torch.Tensor] = None,
                         forward_only: bool = False, **kwargs):
        tokens = batch[0] if isinstance(batch, (list, tuple)) else batch
        c = self.vocab_ctx
        if labels is None:
            labels = kwargs.get("labels")
        chunks = max(1, min(self.plan.chunks, tokens.shape[0]))
        from ..utils.runtime_utils import get_batch_on_this_cp_rank

        part = get_batch_on_this_cp_rank({"tokens": tokens, "labels": labels, "loss_mask": loss_mask}, c.cp_size, c.cp_rank)
        tok, lab, msk = part["tokens"], part["labels"], part["loss_mask"]
        toks, labs, msks = chunk_batch(tok, chunks), chunk_batch(lab, chunks), chunk_batch(msk, chunks)
        chunks = len(toks)
        d_vocab = self.plan.dp_size(self.plan.layers[0])
        mb_sizes = [t.shape[0] * d_vocab for t in toks]
        if loss_func is None:
            fns = [default_loss_func(m, c.cp_size) for m in msks]
        else:
            fns = [loss_func] * chunks
        if profiler is not None:
            profiler.profile_memory(iter, "Before Forward")
            self.engine.after_forward = lambda: profiler.profile_memory(iter, "After Forward")
        losses = self.engine.run(toks, labs, fns, mb_sizes, forward_only=forward_only)
        if profiler is not None:
            self.engine.after_forward = None
            profiler.profile_memory(iter, "After Backward")
        self.iter = iter
        return self._reduce_loss(losses)

    def _reduce_loss(self, losses: List[torch.Tensor]):
        """Step loss for logging: sum of the (already 1/chunks-scaled) micro-batch losses, summed over cp,
        averaged over the vocab layers' dp group; valid on the last pipeline stage (``None`` elsewhere)."""
        if not losses:
            return None
        total = torch.stack([l.float() for l in losses]).sum()
        c = self.vocab_ctx
        if c.cp_size > 1:
            dist.all_reduce(total, group=c.cp.group)
        if c.dp is not None and c.dp.size > 1 and c.dp.group is not None:
            from ..utils.runtime_utils import average_losses_across_data_parallel_group

            total = average_losses_across_data_parallel_group([total], c.dp)[0]
        return total

    # ---- tied embeddings across pipeline stages ---------------------------------------------------------
    def sync_tied_embedding_grads(self):
        """First and last stage hold a copy of the tied embedding / LM-head weight: sum their gradients."""
        if not self.spec.tied or self.plan.pp_deg == 1:
            return
        g = self.groups.embedding
        if g.size < 2 or g.group is None:
            return
        for lp, u in zip(self.model.plans, self.model.units):
            if lp.kind in ("embedding", "lm_head"):
                w = u.inner.embed_tokens.weight if lp.kind == "embedding" else u.inner.lm_head.weight
                # these units keep the whole step's gradient in main_grad and reduce over their sharding group only
                # in optimizer.step() (ShardedUnit.reduce_at_step_only), i.e. after this sum over the two stages
                w._hg_unit.prepare_grads()
                dist.all_reduce(w.main_grad, group=g.group)


def build_model(args, device=None, full_init: bool = False, fused_comm: Optional[bool] = None,
                fused_zero: Optional[bool] = None) -> GalvatronModel:
    """Resolve the configuration, create the process groups and instantiate this rank's stage."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    resolve_model_config(args, vocab_tp=None)
    if getattr(args.model, "shape_order", "SBH") != "SBH":
        # same restriction as the reference (hybrid_parallel_model.py:198): activations are [sequence, batch, hidden]
        raise ValueError("Shape order must be SBH for the hybrid parallel model")
    if getattr(args.model, "multi_latent_attention", False):
        raise NotImplementedError("multi_latent_attention: the reference only carries the flag (rope_utils.py); "
                                  "no latent-attention layer exists there or here")
    plan = build_plan(args, world)
    # pad the vocabulary for the vocab tensor-parallel degree
    from ..config.model_config import finalize_model_args

    finalize_model_args(args.model, vocab_tp=plan.vocab_tp if not plan.vocab_sp else 1)
    spec = spec_from_args(args)
    if device is None:
        if torch.cuda.is_available():
            device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", args.local_rank)))
        else:
            device = torch.device("cpu")
    backend = None
    factory = GroupFactory(rank, world, backend)
    groups = ModelGroups(factory, plan, rank)
    # named random streams: one per distinct tensor/sequence-parallel group size (dropout on sharded activations)
    from ..parallel.random import set_seed_with_group

    ctxs = [groups.ctx(lp, spec.seq_len) for lp in plan.layers]
    shard_groups = [(c.tp if c.tp_size >= c.sp_size else c.sp) for c in ctxs]
    set_seed_with_group([g for g in shard_groups if g is not None and g.size > 1], None, args.train.seed or 1234,
                        cuda=device.type == "cuda")
    # own kernels over peer memory instead of NCCL: argument > configuration field > environment > on (CUDA only)
    if fused_comm is None:
        fused_comm = getattr(args.parallel, "fused_comm", None)
    if fused_comm is None:
        fused_comm = bool(int(os.environ.get("HG_FUSED_COMM", "1")))
    if fused_zero is None:
        fused_zero = getattr(args.parallel, "fused_zero", None)
    if fused_zero is None:
        fused_zero = bool(int(os.environ.get("HG_FUSED_ZERO", "1")))
    fused_comm = bool(fused_comm) and device.type == "cuda" and spec.dtype in (torch.bfloat16, torch.float16)
    fused_zero = bool(fused_zero) and device.type == "cuda"
    if device.type == "cuda" and spec.dtype in (torch.bfloat16, torch.float16):
        from ..ops import _lib

        _lib.select_precision("fp16" if spec.dtype == torch.float16 else "bf16")   # one kernel build per process
    stage = build_stage(spec, plan, groups, device, seed=args.train.seed or 1234, full_init=full_init,
                        fused_comm=fused_comm, reduce_in_fp32=bool(args.parallel.reduce_in_fp32),
                        fused_zero=fused_zero)
    if os.environ.get("HG_QUIET", "0") != "1":
        from ..utils.runtime_utils import print_rank_0

        print_rank_0("================ hybrid-parallel plan (%s) ================" % plan.source)
        print_rank_0(plan.describe())
    return GalvatronModel(args, spec, plan, groups, stage, device)
