"""Optimizer over the ZeRO units: fused AdamW on flat shards, global gradient-norm clipping, schedules.

``ShardedAdamW.step()``:  reduce gradients (if the engine has not already) -> squared norm of every
unit's shard (device scalars) -> one scalar all-reduce over WORLD -> clip coefficient on the device ->
AdamW on each shard with the coefficient and the 1/dp average folded into the gradient scale -> bf16
parameter refresh (ZeRO-2 all-gather).  The host never reads the norm unless asked to (``grad_norm()``).

The norm is the mathematically exact global L2 norm: every parameter element is counted once
(replicated parameters are down-weighted by their replication factor); the reference sums whatever each
rank holds (galvatron/core/runtime/optimizer/utils.py:14-40, optimizer/clip_grads.py:66-151), which
over-counts replicated parameters.

Capability parity: optimizer/utils.py:43-71 (AdamW construction, state restore),
optimizer/clip_grads.py:154-194 (clip coefficient ``max_norm / (norm + 1e-6)``).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .. import ops


class ShardedAdamW:
    def __init__(self, units: List, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 clip_grad: float = 1.0, device=None, expert_units: Optional[List] = None):
        self.units = [u for u in units if u.params]
        self.param_groups = [{"lr": lr, "weight_decay": weight_decay, "betas": betas, "eps": eps}]
        self.clip_grad = clip_grad
        dev = device if device is not None else (self.units[0].device if self.units else "cpu")
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._coef = torch.ones(1, dtype=torch.float32, device=dev)
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)

    def zero_grad(self, set_to_none: bool = True):
        for u in self.units:
            u.zero_grad()

    def _sync_fused_groups(self):
        """One rendezvous per distinct sharding group among the units that use the peer-memory kernels."""
        seen = set()
        for u in self.units:
            if getattr(u, "fused", False) and id(u.pg) not in seen:
                seen.add(id(u.pg))
                u.sync_peers()

    def reduce_gradients(self):
        """Finish the step's gradient synchronisation: units whose reduction was launched from their backward hook
        (the usual case) only need the reduction stream joined; the rest (forward-only units, weights tied across
        stages, CPU runs) reduce here."""
        from ..parallel.zero import REDUCE

        pending = [u for u in self.units if not u._reduced]
        if pending and self.units:
            # what the backward hooks queued on the reduction stream comes first: the in-kernel rendezvous counts calls,
            # so the reductions of a group must run in one order on every rank
            REDUCE.join(self.units[0].device)
        if any(getattr(u, "fused", False) and u.defer_sync and u.wire_dtype == torch.float32 for u in pending):
            self._sync_fused_groups()      # every rank's backward has written its gradients
            presynced = True
        else:
            presynced = False
        for u in pending:
            u.reduce_grads(final=True, presynced=presynced)
        if self.units:
            REDUCE.join(self.units[0].device)

    def compute_grad_norm(self):
        self._sumsq.zero_()
        for u in self.units:
            u.grad_sumsq(self._sumsq)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(self._sumsq)
        ops.clip_coefficient(self._sumsq, self.clip_grad, self._coef, self._norm)

    def grad_norm(self) -> float:
        """Host read of the last computed norm (synchronises)."""
        return float(self._norm.item())

    def step(self):
        g = self.param_groups[0]
        self.reduce_gradients()
        self.compute_grad_norm()
        coef = self._coef if self.clip_grad > 0 else None
        for u in self.units:
            u.optimizer_step(g["lr"], g["betas"][0], g["betas"][1], g["eps"], g["weight_decay"], coef)
        self._sync_fused_groups()          # peers' parameter stores have landed before the next forward

    def state_dict(self) -> Dict:
        return {"param_groups": self.param_groups, "state": {u.name: u.optimizer_state() for u in self.units}}

    def load_state_dict(self, sd: Dict):
        self.param_groups[0].update({k: v for k, v in sd["param_groups"][0].items()})
        missing = [u.name for u in self.units if u.name not in sd["state"]]
        for u in self.units:
            if u.name in sd["state"]:
                u.load_optimizer_state(sd["state"][u.name])
        if missing:
            import warnings

            warnings.warn("optimizer state has no entry for %d unit(s) (%s%s): they keep freshly initialised moments"
                          % (len(missing), ", ".join(missing[:4]), ", ..." if len(missing) > 4 else ""))
