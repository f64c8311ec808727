"""Sharded-parameter manager: DDP / ZeRO-2 / ZeRO-3 per wrap unit, with its own flat buffers.

Each wrap unit (one decoder layer, the embedding, the final norm, the LM head, an expert block) gets

* ``flat``        the working-precision parameters in one buffer (the module's parameters are views);
* ``main_grad``   an fp32 gradient buffer of the same layout (``param.main_grad`` views): the weight-
                  gradient GEMM epilogue accumulates straight into it;
* ``master/exp_avg/exp_avg_sq``  fp32 optimizer state of the *local shard* (whole buffer for DDP);

and, per ZeRO type over the unit's ``sdp`` group (dp x sp x cp):

=========  =====================================  ==========================================
type       parameters                              gradients
=========  =====================================  ==========================================
ddp        replicated                              all-reduce
zero2      replicated, refreshed by all-gather     reduce-scatter -> shard
           after the sharded optimizer step
zero3      sharded; all-gathered before the        reduce-scatter -> shard
           unit's forward and again before its
           backward, storage released in between
=========  =====================================  ==========================================

With ``defer_sync`` (the reference's ``async_grad_reduce=True``) the reduction runs once, after the last
micro-batch; otherwise after every micro-batch's backward of the unit.  Gradients are *summed* over the
sequence/context-parallel part of the group and *averaged* over the data-parallel replicas.

This replaces torch FSDP as used by the reference (galvatron/core/runtime/parallel.py:100-210,
pipeline/grad_reduce.py:48-149, pipeline/sp_grad_reduce.py:48-132) so that the collectives can be fused
with our own kernels.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.checkpoint import checkpoint as _torch_checkpoint

from .. import ops
from . import mappings as mp

ALIGN = 64  # elements; keeps every parameter 128-byte aligned inside the flat buffers


def _group_info(g):
    if g is None or g.size == 1 or g.group is None:
        return None, 1, 0
    return g.group, g.size, g.rank


class ShardedUnit:
    def __init__(self, module: nn.Module, name: str, sdp, dp_size: int, dp_type: str = "ddp",
                 reduce_in_fp32: bool = True, tp=None, defer_sync: bool = True, grad_sum_group=None,
                 fused_zero: bool = False):
        self.module, self.name = module, name
        self.pg, self.n, self.rank = _group_info(sdp)
        self.dp_size = max(1, dp_size)
        self.dp_type = dp_type if self.n > 1 else "ddp"
        self.reduce_in_fp32 = reduce_in_fp32
        self.tp_pg, self.tp_n, _ = _group_info(tp)
        self.defer_sync = defer_sync
        params = []
        for p in module.parameters():
            if getattr(p, "_hg_unit", None) is None:
                p._hg_unit = self
                params.append(p)
        # tensor-parallel-replicated parameters (norm weights, replicated biases, router) first
        params.sort(key=lambda p: 0 if getattr(p, "tp_replicated", False) else 1)
        self.params: List[nn.Parameter] = params
        self.offsets: List[int] = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        self.replicated_numel = 0
        for p, o in zip(params, self.offsets):
            if getattr(p, "tp_replicated", False):
                self.replicated_numel = o + p.numel()
        mult = ALIGN * self.n
        self.numel = max(mult, (off + mult - 1) // mult * mult)
        self.shard_numel = self.numel // self.n
        self.device = params[0].device if params else torch.device("cpu")
        self.dtype = params[0].dtype if params else torch.float32
        self.flat: Optional[torch.Tensor] = None
        self.main_grad: Optional[torch.Tensor] = None
        self.gathered = True
        self.step_count = 0
        self._reduced = False
        self._bwd_pending = False
        self.count_in_norm = True  # False for the second copy of a weight tied across pipeline stages
        # own reduce-scatter / AdamW+all-gather kernels over peer memory instead of NCCL (parallel/fused_zero.py)
        self.fused = False
        if fused_zero and params and self.dp_type in ("zero2", "zero3"):
            from . import fused_zero as fz

            self.fused = fz.available(self.device, self.n)
        if params:
            self._materialise()

    # ---- construction ----------------------------------------------------------------------------
    def _materialise(self):
        dev = self.device
        self._sym_grad = self._sym_flat = None
        if self.fused:
            from . import fused_zero as fz

            # peers read the gradient buffer and (ZeRO-2) write the parameter buffer: both symmetric
            self._sym_grad = fz.SymmetricBuffer(self.numel, torch.float32, dev, self.pg)
            if self.dp_type == "zero2" and self.dtype == torch.bfloat16:
                self._sym_flat = fz.SymmetricBuffer(self.numel, self.dtype, dev, self.pg)
        self.flat = self._sym_flat.tensor if self._sym_flat is not None else torch.zeros(self.numel, dtype=self.dtype, device=dev)
        for p, o in zip(self.params, self.offsets):
            self.flat[o:o + p.numel()].copy_(p.data.reshape(-1))
        self._bind_params()
        self.main_grad = self._sym_grad.tensor if self._sym_grad is not None else \
            torch.zeros(self.numel, dtype=torch.float32, device=dev)
        for p, o in zip(self.params, self.offsets):
            p.main_grad = self.main_grad[o:o + p.numel()].view(p.shape)
            p.mg_fresh = True
        lo, hi = self.shard_range()
        self.master = self.flat[lo:hi].float().clone()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.grad_shard = None  # fp32 view / buffer holding this rank's reduced gradient
        self._sym_shard = None
        if self.dp_type == "zero3":
            if self.fused and self.dtype == torch.bfloat16:
                # the bf16 shard is what peers pull from when they re-assemble the unit's parameters: it changes only
                # in the optimizer step, which ends with a rendezvous, so gathers need no synchronisation of their own
                from . import fused_zero as fz

                self._sym_shard = fz.SymmetricBuffer(self.shard_numel, self.dtype, dev, self.pg)
                self.shard_lp = self._sym_shard.tensor
                self.shard_lp.copy_(self.flat[lo:hi])
                self.sync_peers()
            else:
                self.shard_lp = self.flat[lo:hi].clone()
            self.release()
        else:
            self.shard_lp = self.flat[lo:hi]

    def _bind_params(self):
        for p, o in zip(self.params, self.offsets):
            p.data = self.flat[o:o + p.numel()].view(p.shape)

    def shard_range(self):
        if self.dp_type == "ddp":
            return 0, self.numel
        return self.rank * self.shard_numel, (self.rank + 1) * self.shard_numel

    def sync_params_from(self, src_rank_in_group: int = 0):
        """Broadcast the working parameters from one rank of the sdp group (after a non-deterministic
        initialisation) and rebuild the master copy."""
        if self.n > 1:
            was = self.gathered
            if self.dp_type == "zero3" and not was:
                self.flat.untyped_storage().resize_(self.numel * self.flat.element_size())
            if self.dp_type != "zero3" or was:
                src = dist.get_global_rank(self.pg, src_rank_in_group)
                dist.broadcast(self.flat, src=src, group=self.pg)
                lo, hi = self.shard_range()
                self.master.copy_(self.flat[lo:hi])

    def reload_master(self):
        """Re-derive master weights / bf16 shard from ``flat`` (after a checkpoint load into the params)."""
        if not self.gathered:
            raise RuntimeError("gather the unit before reloading")
        lo, hi = self.shard_range()
        self.master.copy_(self.flat[lo:hi])
        if self.dp_type == "zero3":
            self.shard_lp.copy_(self.flat[lo:hi])
            if self._sym_shard is not None:
                self.sync_peers()        # peers pull from this shard

    # ---- ZeRO-3 gather / release --------------------------------------------------------------------
    def gather(self):
        if self.dp_type != "zero3" or self.gathered:
            return
        nbytes = self.numel * self.flat.element_size()
        st = self.flat.untyped_storage()
        if st.size() != nbytes:
            st.resize_(nbytes)
        if self.flat.device.type == "cpu":
            parts = [torch.empty_like(self.shard_lp) for _ in range(self.n)]
            dist.all_gather(parts, self.shard_lp, group=self.pg)
            self.flat.copy_(torch.cat(parts))
        elif self._sym_shard is not None:
            from . import fused_zero as fz

            fz.all_gather_peer(self._sym_shard, self.shard_numel, self.flat)   # pull every rank's shard over NVLink
        else:
            dist.all_gather_into_tensor(self.flat, self.shard_lp, group=self.pg)
        self.gathered = True

    def release(self):
        if self.dp_type != "zero3" or not self.gathered:
            return
        # views held by autograd's saved tensors stay attached to the storage object; it is re-filled by
        # the next gather() before anything reads it
        self.flat.untyped_storage().resize_(0)
        self.gathered = False

    # ---- gradients --------------------------------------------------------------------------------------
    def zero_grad(self):
        for p in self.params:
            p.mg_fresh = True
            p.grad = None
        self._reduced = False
        self._acc_used = False

    def _finish_accumulation(self):
        """Fold stray ``.grad`` tensors (bias / generic autograd paths) into ``main_grad`` and zero what
        received nothing."""
        for p in self.params:
            if p.grad is not None:
                if getattr(p, "mg_fresh", False):
                    p.main_grad.copy_(p.grad)
                    p.mg_fresh = False
                else:
                    p.main_grad.add_(p.grad)
                p.grad = None

    def prepare_grads(self):
        """Make ``main_grad`` complete for the micro-batches seen so far: fold autograd ``.grad`` tensors in
        and zero the parameters that received nothing."""
        self._finish_accumulation()
        for p in self.params:
            if getattr(p, "mg_fresh", False):  # received nothing since the last reset
                p.main_grad.zero_()
                p.mg_fresh = False

    def sync_peers(self):
        """Stream-ordered rendezvous of the sharding group (fused path only)."""
        if self.fused:
            from . import fused_zero as fz

            fz.peer_barrier(self.pg, self.device)

    def _reduce_now(self, presynced: bool = False) -> torch.Tensor:
        """Sum the current ``main_grad`` over the sdp group; returns the buffer holding this rank's part."""
        self.prepare_grads()
        if self.tp_n > 1 and self.replicated_numel > 0:
            # norm weights / replicated biases saw only this rank's S/t tokens: sum over the tp group
            dist.all_reduce(self.main_grad[: self.replicated_numel], group=self.tp_pg)
        if self.n == 1:
            return self.main_grad
        if self.dp_type == "ddp":
            dist.all_reduce(self.main_grad, group=self.pg)
            return self.main_grad
        if getattr(self, "_rs_out", None) is None:
            self._rs_out = torch.empty(self.shard_numel, dtype=torch.float32, device=self.device)
        if self.fused:
            from . import fused_zero as fz

            if not presynced:
                self.sync_peers()        # every rank's gradients are complete
            fz.reduce_scatter_peer(self._sym_grad, self.rank, self.shard_numel, self._rs_out)
            if not self.defer_sync:
                self.sync_peers()        # main_grad is reused by the next micro-batch right away
            return self._rs_out
        if self.main_grad.device.type == "cpu":
            tmp = self.main_grad.clone()
            dist.all_reduce(tmp, group=self.pg)
            self._rs_out.copy_(tmp[self.rank * self.shard_numel:(self.rank + 1) * self.shard_numel])
        else:
            dist.reduce_scatter_tensor(self._rs_out, self.main_grad, group=self.pg)
        return self._rs_out

    def reduce_grads(self, final: bool = True, presynced: bool = False):
        """Gradient synchronisation.  Deferred mode: one reduction at the end of the step.  Immediate mode:
        every micro-batch's gradient is reduced right after the unit's backward and added to the running
        shard, and ``main_grad`` starts fresh for the next micro-batch."""
        if self._reduced:
            return
        if self.defer_sync:
            if final:
                self.grad_shard = self._reduce_now(presynced)
                self._reduced = True
            return
        if not final:
            red = self._reduce_now()
            if getattr(self, "_acc", None) is None:
                self._acc = torch.zeros_like(red)
                self._acc_used = False
            if self._acc_used:
                self._acc.add_(red)
            else:
                self._acc.copy_(red)
                self._acc_used = True
            for p in self.params:
                p.mg_fresh = True
        else:
            if getattr(self, "_acc", None) is None or not self._acc_used:
                self.grad_shard = self._reduce_now()
            else:
                self.grad_shard = self._acc
            self._reduced = True

    def grad_sumsq(self, out: torch.Tensor):
        """Add this rank's share of the squared gradient norm to ``out[0]`` so that a SUM over all ranks
        counts every parameter element exactly once."""
        if not self.count_in_norm:
            return
        g = self.grad_shard
        inv = 1.0 / (self.dp_size * self.dp_size)  # gradients are still dp-sums here
        rep = self.n if self.dp_type == "ddp" else 1  # identical copies held by the sdp group
        ops.sumsq(g, out, accumulate=True, scale=inv / rep)
        if self.tp_n > 1 and self.replicated_numel > 0:
            lo, hi = self.shard_range()
            a, b = max(lo, 0), min(hi, self.replicated_numel)
            if b > a:
                ops.sumsq(g[a - lo:b - lo], out, accumulate=True, scale=inv / rep * (1.0 / self.tp_n - 1.0))

    # ---- optimizer --------------------------------------------------------------------------------------
    def optimizer_step(self, lr, beta1, beta2, eps, weight_decay, clip_coef: Optional[torch.Tensor] = None):
        if not self.params:
            return
        self.step_count += 1
        g = self.grad_shard
        # fold the 1/dp average into the device-side gradient scale
        self._ensure_scale(clip_coef)
        if self.fused and self.dtype == torch.bfloat16:
            from . import fused_zero as fz

            # ZeRO-2: the updated bf16 values go straight into every rank's parameter buffer (no all-gather);
            # ZeRO-3: into the local bf16 shard.  The caller rendezvouses the group afterwards (sync_peers).
            target = self._sym_flat if self.dp_type == "zero2" else self.shard_lp
            off = self.rank * self.shard_numel if self.dp_type == "zero2" else 0
            fz.adamw_allgather_peer(self.master, g, self.exp_avg, self.exp_avg_sq, target, off, lr=lr, beta1=beta1,
                                    beta2=beta2, eps=eps, weight_decay=weight_decay, step=self.step_count,
                                    gscale=self._scale)
            return
        lp = self.shard_lp if self.dtype != torch.float32 else None
        ops.adamw_step(self.master, g, self.exp_avg, self.exp_avg_sq, lp, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                       weight_decay=weight_decay, step=self.step_count, gscale=self._scale)
        if self.dtype == torch.float32:
            self.shard_lp.copy_(self.master)
        if self.dp_type == "zero2":
            if self.flat.device.type == "cpu":
                parts = [torch.empty_like(self.shard_lp) for _ in range(self.n)]
                dist.all_gather(parts, self.shard_lp.contiguous(), group=self.pg)
                self.flat.copy_(torch.cat(parts))
            else:
                dist.all_gather_into_tensor(self.flat, self.shard_lp, group=self.pg)

    def _ensure_scale(self, clip_coef):
        if not hasattr(self, "_scale"):
            self._scale = torch.ones(1, dtype=torch.float32, device=self.device)
        if clip_coef is None:
            self._scale.fill_(1.0 / self.dp_size)
        else:
            torch.mul(clip_coef, 1.0 / self.dp_size, out=self._scale)

    # ---- state dict -------------------------------------------------------------------------------------
    def optimizer_state(self) -> Dict[str, torch.Tensor]:
        return {"master": self.master, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq,
                "step": torch.tensor(self.step_count)}

    def load_optimizer_state(self, sd):
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.step_count = int(sd["step"])

    def full_state_dict(self) -> Dict[str, torch.Tensor]:
        """Unsharded parameters of the unit keyed by their module-relative names (collective for zero3)."""
        was = self.gathered
        self.gather()
        out = {k: v.detach().clone().cpu() for k, v in self.module.state_dict().items()}
        if not was:
            self.release()
        return out


class _Boundary(torch.autograd.Function):
    """Identity in the forward; runs a callback when the gradient passes in the backward."""

    @staticmethod
    def forward(ctx, x, cb):
        ctx.cb = cb
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.cb()
        return g, None


class UnitWrapper(nn.Module):
    """Runs a unit's module between the ZeRO hooks (gather before forward / backward, release after,
    gradient reduction after the backward) and optional activation recomputation."""

    def __init__(self, inner: nn.Module, unit: ShardedUnit, checkpoint: bool = False):
        super().__init__()
        self.inner, self.unit, self.checkpoint = inner, unit, checkpoint
        self.sync_this_backward = True
        self.extra_units: List[ShardedUnit] = []  # units owning parameters this module borrows (tied weights)

    def _pre_backward(self):
        self.unit.gather()
        for e in self.extra_units:
            e.gather()
        self.unit._bwd_pending = True

    def _post_backward(self):
        u = self.unit
        if not u._bwd_pending:
            return
        u._bwd_pending = False
        u.release()
        for e in self.extra_units:
            e.release()
        if self.sync_this_backward and not u.defer_sync:
            u.reduce_grads(final=False)

    def finish_backward(self):
        """Called by the engine after the whole backward: covers units whose inputs carry no gradient."""
        self._post_backward()

    def forward(self, *args, **kwargs):
        u = self.unit
        u.gather()
        for e in self.extra_units:
            e.gather()
        grad_mode = torch.is_grad_enabled()
        if grad_mode:
            # the unit's backward is over once the gradient has left through *every* differentiable input
            pending = [sum(1 for a in args if torch.is_tensor(a) and a.requires_grad)]

            def _one_input_done():
                pending[0] -= 1
                if pending[0] <= 0:
                    self._post_backward()

            args = tuple(_Boundary.apply(a, _one_input_done) if torch.is_tensor(a) and a.requires_grad else a
                         for a in args)
        if self.checkpoint and grad_mode:
            out = _torch_checkpoint(self.inner, *args, use_reentrant=False, **kwargs)
        else:
            out = self.inner(*args, **kwargs)
        u.release()
        for e in self.extra_units:
            e.release()
        if grad_mode:
            if torch.is_tensor(out) and out.requires_grad:
                out = _Boundary.apply(out, self._pre_backward)
            elif isinstance(out, tuple):
                out = tuple(_Boundary.apply(o, self._pre_backward) if torch.is_tensor(o) and o.requires_grad else o
                            for o in out)
        return out
