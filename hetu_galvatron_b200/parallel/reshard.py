"""Activation resharding between neighbouring layers whose strategies differ.

Between layers an activation is ``[S / g, B / d, H]`` with ``g = (tp | sp) * cp`` ranks sharing one
sample's sequence and ``d = stage_ranks / g`` data-parallel replicas.  When ``(tp|sp, cp)`` changes from
one layer to the next the tensor is re-laid-out:

1. the sequence is gathered over the old layer's ``tsp_cp`` group (and un-zig-zagged if it was
   context-parallel),
2. the batch is gathered over the "fused" group when the new layer has fewer replicas, or sliced when
   it has more,
3. the sequence is (zig-zagged and) sliced for the new layer's ``tsp_cp`` group.

Every step is one of the autograd-symmetric mappings, so the backward re-lays-out the gradient the
opposite way.  Integer / non-float inputs take the same path without autograd.

Capability parity: galvatron/core/runtime/redistribute.py:5-41 (zig-zag), :223-341 (fused
split / all-gather), :345-415 (autograd + module); group derivation comm_groups.py:225-263.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import mappings as mp
from .groups import CommGroup, GroupFactory, Layout


def zigzag_order(cp: int) -> list:
    """Chunk ids (of ``2*cp``) in the order a gather over the cp group concatenates them."""
    order = []
    for r in range(cp):
        order += [r, 2 * cp - 1 - r]
    return order


def undo_zigzag(x: torch.Tensor, cp: int) -> torch.Tensor:
    """``x`` = concat over cp ranks of their two chunks -> natural sequence order (dim 0)."""
    if cp == 1:
        return x
    chunks = x.chunk(2 * cp, dim=0)
    order = zigzag_order(cp)
    nat = [None] * (2 * cp)
    for pos, cid in enumerate(order):
        nat[cid] = chunks[pos]
    return torch.cat(nat, dim=0)


def apply_zigzag(x: torch.Tensor, cp: int) -> torch.Tensor:
    """natural order -> concat over cp ranks of (chunk r, chunk 2c-1-r)."""
    if cp == 1:
        return x
    chunks = x.chunk(2 * cp, dim=0)
    return torch.cat([chunks[c] for c in zigzag_order(cp)], dim=0)


class Reshard(nn.Module):
    """Moves ``[S/g_old, B/d_old, H]`` to ``[S/g_new, B/d_new, H]``."""

    def __init__(self, old_groups, new_groups, old_width: int, old_cp: int, new_width: int, new_cp: int,
                 fused: Optional[CommGroup], rank_in_stage: int):
        super().__init__()
        self.old, self.new = old_groups, new_groups
        self.g_old, self.g_new = old_width * old_cp, new_width * new_cp
        self.cp_old, self.cp_new = old_cp, new_cp
        self.fused = fused
        self.j = rank_in_stage % max(self.g_old, self.g_new)  # index inside the larger block
        self.identity = (old_width == new_width and old_cp == new_cp)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.identity:
            return x
        floating = x.is_floating_point()
        gather = (lambda t, g: mp.gather_first_dim(t, g, grad_is_partial=True)) if floating else \
            (lambda t, g: mp.all_gather_first(t, g))
        # 1. full sequence of my batch shard, natural order
        full = gather(x, self.old.tsp_cp) if self.g_old > 1 else x
        full = undo_zigzag(full, self.cp_old)
        # 2. batch re-split
        if self.g_new > self.g_old:       # fewer replicas afterwards: gather the batch shards of the block
            k = self.g_new // self.g_old
            if k > 1:
                fb = full.transpose(0, 1).contiguous()          # [B, S, H]
                fb = gather(fb, self.fused)
                full = fb.transpose(0, 1).contiguous()
        elif self.g_new < self.g_old:     # more replicas afterwards: keep my slice of the batch
            k = self.g_old // self.g_new
            b = self.j // self.g_new
            full = full.chunk(k, dim=1)[b].contiguous()
        # 3. sequence slice for the new layer
        full = apply_zigzag(full, self.cp_new)
        if self.g_new > 1:
            i = self.new.tsp_cp.rank
            full = full.chunk(self.g_new, dim=0)[i].contiguous()
        return full


def build_reshard(factory: GroupFactory, world: int, pp: int, rank: int, old_groups, new_groups, old_plan,
                  new_plan) -> Optional[Reshard]:
    ow, ocp = max(old_plan.tp, old_plan.sp), old_plan.cp
    nw, ncp = max(new_plan.tp, new_plan.sp), new_plan.cp
    if ow == nw and ocp == ncp:
        return None
    g_old, g_new = ow * ocp, nw * ncp
    big, small = max(g_old, g_new), min(g_old, g_new)
    fused = None
    if g_new > g_old:
        # ranks holding the same sequence chunk in the g_new/g_old old-groups of one block
        lay = Layout(("pp", "blk", "a", "i"), (pp, world // pp // big, big // small, small))
        fused = factory.make(lay.groups(("a",)))
    stage_ranks = world // pp
    return Reshard(old_groups, new_groups, ow, ocp, nw, ncp, fused, rank % stage_ranks)
