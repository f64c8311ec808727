"""Rank <-> parallel-coordinate algebra and per-layer process groups.

A layer's strategy fixes the sizes of the ``pp, dp, cp, tp, sp`` axes (their product is the world
size).  Ranks are laid out in the order ``pp-dp-cp-tp-sp`` with the rightmost axis fastest, so
``coord(axis) = (rank // stride(axis)) % size(axis)``; a group of some axes = the ranks that agree on
every *other* axis.  MoE layers use the order ``pp-ep-edp-etp``.  The algebra is pure Python (testable
without a process group); :class:`GroupFactory` turns rank lists into ``torch.distributed`` groups,
creating each distinct rank set once (``new_group`` is collective, so every rank walks the same list).

Capability parity: galvatron/core/runtime/comm_groups.py:39-116 (coordinates), :119-203 (groups),
:206-221 (embedding group), :225-263 (resharding groups), :266-442 (per-layer lists).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

DENSE_ORDER = ("pp", "dp", "cp", "tp", "sp")
MOE_ORDER = ("pp", "ep", "edp", "etp")


@dataclass(frozen=True)
class Layout:
    """Sizes of the axes, slowest first."""

    order: Tuple[str, ...]
    sizes: Tuple[int, ...]

    @property
    def world(self) -> int:
        w = 1
        for s in self.sizes:
            w *= s
        return w

    def stride(self, axis: str) -> int:
        i = self.order.index(axis)
        st = 1
        for s in self.sizes[i + 1:]:
            st *= s
        return st

    def size(self, axis: str) -> int:
        return self.sizes[self.order.index(axis)]

    def coord(self, rank: int, axis: str) -> int:
        return (rank // self.stride(axis)) % self.size(axis)

    def coords(self, rank: int) -> Dict[str, int]:
        return {a: self.coord(rank, a) for a in self.order}

    def rank_of(self, coords: Dict[str, int]) -> int:
        return sum(coords[a] * self.stride(a) for a in self.order)

    def groups(self, axes: Sequence[str]) -> List[List[int]]:
        """All groups spanned by ``axes``: ranks equal on every other axis, each list ascending."""
        axes = tuple(a for a in self.order if a in axes)
        buckets: Dict[Tuple[int, ...], List[int]] = {}
        for r in range(self.world):
            key = tuple(self.coord(r, a) for a in self.order if a not in axes)
            buckets.setdefault(key, []).append(r)
        return [buckets[k] for k in sorted(buckets)]

    def group_of(self, rank: int, axes: Sequence[str]) -> List[int]:
        for g in self.groups(axes):
            if rank in g:
                return g
        raise ValueError("rank %d outside the layout" % rank)


def dense_layout(world: int, pp: int, tp: int = 1, sp: int = 1, cp: int = 1) -> Layout:
    denom = pp * tp * sp * cp
    if world % denom:
        raise ValueError("world size %d is not divisible by pp*tp*sp*cp = %d" % (world, denom))
    return Layout(DENSE_ORDER, (pp, world // denom, cp, tp, sp))


def moe_layout(world: int, pp: int, ep: int = 1, etp: int = 1) -> Layout:
    denom = pp * ep * etp
    if world % denom:
        raise ValueError("world size %d is not divisible by pp*ep*etp = %d" % (world, denom))
    return Layout(MOE_ORDER, (pp, ep, world // denom, etp))


# which axes span each named group of a dense layer
DENSE_GROUP_AXES = {
    "tp": ("tp",), "sp": ("sp",), "cp": ("cp",), "dp": ("dp",),
    "sdp": ("dp", "sp", "cp"),        # parameters are sharded / reduced over dp x sp x cp
    "tsp_cp": ("tp", "sp", "cp"),     # the ranks that together hold one sample's full sequence
    "tp_sp": ("tp", "sp"),
    "pp": ("pp",),
}
MOE_GROUP_AXES = {"ep": ("ep",), "tp_of_ep": ("etp",), "tp_and_ep": ("ep", "etp"), "dp_of_ep": ("edp",)}


def embedding_group_ranks(layout: Layout) -> List[List[int]]:
    """First and last pipeline stage of every pipeline chain (tied embedding / LM-head weights)."""
    pp = layout.size("pp")
    out = []
    for chain in layout.groups(("pp",)):
        out.append([chain[0]] if pp == 1 else [chain[0], chain[-1]])
    return out


def reshard_plan(world: int, pp: int, old: Tuple[int, int], new: Tuple[int, int]):
    """Groups needed to move activations between two neighbouring layers whose sequence-sharding width
    ``g = (tp|sp) * cp`` differs.  ``old`` / ``new`` are ``(tp_or_sp, cp)``.

    The activation of a layer is sharded along the sequence over its tsp_cp group and along the batch
    over its dp group.  Going from width ``g_old`` to ``g_new``:
      * ``g_new > g_old``: the batch shards of ``g_new/g_old`` neighbouring old groups are gathered
        (all-gather over the strided "fused" group) and the sequence is split finer (a local slice);
      * ``g_new < g_old``: the sequence is gathered over the part of the old group that merges
        (all-gather over the fused group) and the batch is split (a local slice).
    Returns ``(old_groups, new_groups, fused_groups)`` as rank lists; the fused groups have
    ``max(g)/min(g)`` members with stride ``min(g)`` inside a block of ``max(g)`` consecutive ranks."""
    g_old, g_new = old[0] * old[1], new[0] * new[1]
    lay_old = Layout(("pp", "dp", "g"), (pp, world // pp // g_old, g_old))
    lay_new = Layout(("pp", "dp", "g"), (pp, world // pp // g_new, g_new))
    old_groups, new_groups = lay_old.groups(("g",)), lay_new.groups(("g",))
    big, small = max(g_old, g_new), min(g_old, g_new)
    fused = []
    for block in Layout(("pp", "dp", "g"), (pp, world // pp // big, big)).groups(("g",)):
        for off in range(small):
            fused.append([block[off + k * small] for k in range(big // small)])
    return old_groups, new_groups, fused


# --------------------------------------------------------------------------------------------
# torch.distributed side
# --------------------------------------------------------------------------------------------
@dataclass
class CommGroup:
    """One process group as seen by this rank."""

    ranks: List[int]
    group: object = None  # torch.distributed.ProcessGroup or None for single-rank groups
    rank: int = 0          # this process's index inside `ranks`

    @property
    def size(self) -> int:
        return len(self.ranks)

    def has(self, r: int) -> bool:
        return r in self.ranks

    def __repr__(self):
        return "CommGroup(size=%d, ranks=%s)" % (self.size, self.ranks)


class GroupFactory:
    """Creates every distinct rank set once.  All ranks must call :meth:`make` with the same sequence
    of rank-list collections (``new_group`` is a collective over the default group)."""

    def __init__(self, rank: int, world: int, backend: Optional[str] = None):
        self.rank, self.world, self.backend = rank, world, backend
        self._cache: Dict[tuple, object] = {}

    def make(self, all_groups: List[List[int]], tag: str = "", allow_absent: bool = False) -> CommGroup:
        """``tag`` asks for a communicator of its own over a rank set that may already have one (a second,
        independent channel between the same ranks, e.g. the backward direction of the pipeline)."""
        import torch.distributed as dist

        mine = None
        for ranks in all_groups:
            key = tuple(ranks) if not tag else (tag,) + tuple(ranks)
            if key not in self._cache:
                if len(ranks) == 1 or not dist.is_initialized():
                    self._cache[key] = None
                elif len(ranks) == self.world and ranks == list(range(self.world)) and not tag:
                    self._cache[key] = dist.group.WORLD
                else:
                    self._cache[key] = dist.new_group(ranks, backend=self.backend)
            if self.rank in ranks:
                mine = CommGroup(list(ranks), self._cache[key], ranks.index(self.rank))
        if mine is None:
            if allow_absent:     # e.g. a middle pipeline stage and the first/last-stage embedding groups
                return CommGroup([self.rank], None, 0)
            raise RuntimeError("rank %d is in none of the groups" % self.rank)
        return mine


@dataclass
class LayerGroups:
    """Process groups of one layer (dense part + MoE part when the layer has experts)."""

    tp: CommGroup
    sp: CommGroup
    cp: CommGroup
    dp: CommGroup
    sdp: CommGroup
    tsp_cp: CommGroup
    ep: Optional[CommGroup] = None
    tp_of_ep: Optional[CommGroup] = None
    tp_and_ep: Optional[CommGroup] = None
    dp_of_ep: Optional[CommGroup] = None
    layout: Optional[Layout] = None
    moe_layout: Optional[Layout] = None


def build_layer_groups(factory: GroupFactory, world: int, pp: int, tp: int, sp: int, cp: int,
                       ep: Optional[int] = None, etp: int = 1) -> LayerGroups:
    lay = dense_layout(world, pp, tp, sp, cp)
    made = {name: factory.make(lay.groups(axes)) for name, axes in DENSE_GROUP_AXES.items()
            if name in ("tp", "sp", "cp", "dp", "sdp", "tsp_cp")}
    lg = LayerGroups(layout=lay, **made)
    if ep is not None:
        ml = moe_layout(world, pp, ep, etp)
        lg.moe_layout = ml
        for name, axes in MOE_GROUP_AXES.items():
            setattr(lg, name, factory.make(ml.groups(axes)))
    return lg


def describe(lay: Layout, rank: int = 0) -> str:
    parts = ["%s=%d" % (a, s) for a, s in zip(lay.order, lay.sizes)]
    return "layout[%s] rank %d at %s" % (" ".join(parts), rank, lay.coords(rank))
