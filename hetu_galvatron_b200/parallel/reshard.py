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


# ---- one-kernel resharding over peer memory -------------------------------------------------------------------
def _global_pos(i: torch.Tensor, s_local: torch.Tensor, width: int, cp: int, S: int) -> torch.Tensor:
    """Natural sequence position of local row ``s_local`` on sequence-shard index ``i`` (``i = c * width + t``)."""
    g = width * cp
    c, t = i // width, i % width
    p = t * (S // g) + s_local                      # position inside the cp rank's part
    if cp == 1:
        return p
    half = S // (2 * cp)
    return torch.where(p < half, c * half + p, (2 * cp - 1 - c) * half + (p - half))


def _owner(pos: torch.Tensor, width: int, cp: int, S: int):
    """Inverse of :func:`_global_pos`: (sequence-shard index, local row) holding natural position ``pos``."""
    g = width * cp
    if cp == 1:
        p, c = pos, torch.zeros_like(pos)
    else:
        half = S // (2 * cp)
        chunk = pos // half
        first = chunk < cp
        c = torch.where(first, chunk, 2 * cp - 1 - chunk)
        p = torch.where(first, pos - chunk * half, half + pos - chunk * half)
    per = S // g
    return c * width + p // per, p % per


def pull_lists(S: int, rows_dst: int, b_dst: int, b_src: int, j_dst: int, src, dst, device):
    """For every output row ``(s', b')`` of block rank ``j_dst``: the block rank and the row that hold it in the
    source layout.  ``src`` / ``dst`` are ``(width, cp)``; rows are numbered ``s * batch + b``."""
    (w_s, cp_s), (w_d, cp_d) = src, dst
    g_s, g_d = w_s * cp_s, w_d * cp_d
    a_d, i_d = j_dst // g_d, j_dst % g_d
    s_loc = torch.arange(rows_dst, device=device).repeat_interleave(b_dst)
    b_loc = torch.arange(b_dst, device=device).repeat(rows_dst)
    pos = _global_pos(torch.full_like(s_loc, i_d), s_loc, w_d, cp_d, S)
    sample = a_d * b_dst + b_loc
    a_s, b_s = sample // b_src, sample % b_src
    i_s, s_s = _owner(pos, w_s, cp_s, S)
    return (a_s * g_s + i_s).to(torch.int32), (s_s * b_src + b_s).to(torch.int32)


class _PeerReshard(torch.autograd.Function):
    """Forward pulls the rows of the new layout from the block's ranks; backward pulls the gradient rows of the old
    layout the same way (the move is a permutation inside the block, so no reduction is needed)."""

    @staticmethod
    def forward(ctx, x, mod, S):
        ctx.mod, ctx.S, ctx.shape = mod, S, x.shape
        return mod._pull(x, S, mod.src, mod.dst)

    @staticmethod
    def backward(ctx, g):
        return ctx.mod._pull(g, ctx.S, ctx.mod.dst, ctx.mod.src), None, None


class Reshard(nn.Module):
    """Moves ``[S/g_old, B/d_old, H]`` to ``[S/g_new, B/d_new, H]``.

    With ``peer`` set (bf16 activations on a GPU, block of at most 8 ranks) the whole move is one pull kernel over
    NVLink peer memory: every rank publishes its tensor, computes for each of its new rows which block rank holds
    it, and gathers them (``parallel/fused_a2a.py``)."""

    def __init__(self, old_groups, new_groups, old_width: int, old_cp: int, new_width: int, new_cp: int,
                 fused: Optional[CommGroup], rank_in_stage: int, peer: bool = False):
        super().__init__()
        self.peer = peer
        self.src, self.dst = (old_width, old_cp), (new_width, new_cp)
        self._lists = {}
        self.old, self.new = old_groups, new_groups
        self.g_old, self.g_new = old_width * old_cp, new_width * new_cp
        self.cp_old, self.cp_new = old_cp, new_cp
        self.fused = fused
        self.j = rank_in_stage % max(self.g_old, self.g_new)  # index inside the larger block
        self.identity = (old_width == new_width and old_cp == new_cp)

    def _peer_block_ok(self, x: torch.Tensor) -> bool:
        """Symmetric memory works over the block of ranks this move spans (probed once, agreed over the block)."""
        from .fused_zero import available

        grp = self.old.tsp_cp if self.g_old >= self.g_new else self.new.tsp_cp
        return grp is not None and grp.group is not None and available(x.device, grp.size, grp.group)

    def _pull(self, x: torch.Tensor, S: int, src, dst) -> torch.Tensor:
        from . import fused_a2a as fa

        g_s, g_d = src[0] * src[1], dst[0] * dst[1]
        big = max(g_s, g_d)
        grp = self.old.tsp_cp if self.g_old >= self.g_new else self.new.tsp_cp   # the block
        rows_s, b_s, H = x.shape
        b_d = b_s * g_d // g_s
        rows_d = S // g_d
        key = (S, rows_s, b_s, src, dst)
        lists = self._lists.get(key)
        if lists is None:
            lists = self._lists[key] = pull_lists(S, rows_d, b_d, b_s, self.j % big if big else 0, src, dst, x.device)
        slot = fa.staging_for(grp, x.numel() * 2, x.device).publish(x)
        out = fa.gather_rows(slot, lists[0], lists[1], rows_d * b_d, H, H)
        return out.view(rows_d, b_d, H)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.identity:
            return x
        floating = x.is_floating_point()
        if self.peer and floating and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and x.dim() == 3 and x.shape[-1] % 8 == 0 \
                and max(self.g_old, self.g_new) <= 8 and self._peer_block_ok(x):
            S = x.shape[0] * self.g_old
            return _PeerReshard.apply(x, self, S)
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
                  new_plan, peer: bool = False) -> Optional[Reshard]:
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
    return Reshard(old_groups, new_groups, ow, ocp, nw, ncp, fused, rank % stage_ranks, peer=peer)
