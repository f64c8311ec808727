"""Autograd-symmetric collectives over ``torch.distributed`` (NCCL on GPUs, gloo on CPU).

These are the *baseline* communication path and the oracle of the fused compute+collective kernels:
every mapping is a pair (forward collective, backward collective) such that the pair is its own
transpose.  A ``None`` group or a group of one rank turns every mapping into the identity.

Capability parity: galvatron/core/runtime/tensor_parallel/mappings.py:18-214 (copy / reduce / scatter /
gather / reduce-scatter along the first and the last dimension, unequal splits), :217-481 (all-to-all,
equal and ``-v``), :489-548 (functional wrappers).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


def _pg(group):
    """Accepts a CommGroup, a ProcessGroup or None -> (process_group | None, size, rank)."""
    if group is None:
        return None, 1, 0
    if hasattr(group, "ranks"):
        if group.size == 1 or group.group is None:
            return None, 1, 0
        return group.group, group.size, group.rank
    n = dist.get_world_size(group)
    return (group if n > 1 else None), n, dist.get_rank(group)


# ---- raw collectives (no autograd) ------------------------------------------------------------
def all_reduce_(t: torch.Tensor, group, op=dist.ReduceOp.SUM) -> torch.Tensor:
    pg, n, _ = _pg(group)
    if n > 1:
        dist.all_reduce(t, op=op, group=pg)
    return t


def all_gather_first(t: torch.Tensor, group, sizes: Optional[Sequence[int]] = None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    pg, n, _ = _pg(group)
    if n == 1:
        return t
    t = t.contiguous()
    if sizes is None:
        if out is None:
            out = torch.empty((n * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=pg)
        return out
    parts = [torch.empty((s,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device) for s in sizes]
    dist.all_gather(parts, t, group=pg)
    return torch.cat(parts, dim=0)


def reduce_scatter_first(t: torch.Tensor, group, sizes: Optional[Sequence[int]] = None) -> torch.Tensor:
    pg, n, r = _pg(group)
    if n == 1:
        return t
    t = t.contiguous()
    if sizes is None:
        if t.shape[0] % n:
            raise ValueError("first dimension %d is not divisible by the group size %d" % (t.shape[0], n))
        out = torch.empty((t.shape[0] // n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        if t.device.type == "cpu":  # gloo has no reduce_scatter_tensor
            tmp = t.clone()
            dist.all_reduce(tmp, group=pg)
            out.copy_(tmp.chunk(n, dim=0)[r])
        else:
            dist.reduce_scatter_tensor(out, t, group=pg)
        return out
    tmp = t.clone()
    dist.all_reduce(tmp, group=pg)
    return tmp.split(list(sizes), dim=0)[r].contiguous()


def all_to_all_first(t: torch.Tensor, group, out_splits: Optional[List[int]] = None,
                     in_splits: Optional[List[int]] = None) -> torch.Tensor:
    pg, n, _ = _pg(group)
    if n == 1:
        return t
    t = t.contiguous()
    if out_splits is None:
        out = torch.empty_like(t)
    else:
        out = torch.empty((sum(out_splits),) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    if t.device.type == "cpu":
        # gloo has no all-to-all: pairwise isend / irecv between the members of the group
        ins = list(t.split(in_splits, 0)) if in_splits is not None else list(t.chunk(n, 0))
        outs = list(out.split(out_splits, 0)) if out_splits is not None else list(out.chunk(n, 0))
        me = dist.get_rank(pg)
        outs[me].copy_(ins[me])
        reqs, keep = [], []
        for peer in range(n):
            if peer == me:
                continue
            g_peer = dist.get_global_rank(pg, peer)
            if outs[peer].numel():
                buf = torch.empty_like(outs[peer])
                keep.append((outs[peer], buf))
                reqs.append(dist.irecv(buf, src=g_peer))
            if ins[peer].numel():
                reqs.append(dist.isend(ins[peer].contiguous(), dst=g_peer))
        for r in reqs:
            r.wait()
        for dst, buf in keep:
            dst.copy_(buf)
    else:
        dist.all_to_all_single(out, t, output_split_sizes=out_splits, input_split_sizes=in_splits, group=pg)
    return out


# ---- autograd pairs ---------------------------------------------------------------------------------
class _Copy(torch.autograd.Function):  # fwd identity, bwd all-reduce
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        return all_reduce_(g.contiguous().clone(), ctx.group), None


class _Reduce(torch.autograd.Function):  # fwd all-reduce, bwd identity
    @staticmethod
    def forward(ctx, x, group):
        return all_reduce_(x.contiguous().clone(), group)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _ScatterFirst(torch.autograd.Function):  # fwd local slice, bwd all-gather
    @staticmethod
    def forward(ctx, x, group, sizes):
        ctx.group, ctx.sizes = group, sizes
        _, n, r = _pg(group)
        if n == 1:
            return x
        if sizes is None:
            return x.chunk(n, dim=0)[r].contiguous()
        return x.split(list(sizes), dim=0)[r].contiguous()

    @staticmethod
    def backward(ctx, g):
        return all_gather_first(g, ctx.group, ctx.sizes), None, None


class _GatherFirst(torch.autograd.Function):  # fwd all-gather, bwd reduce-scatter (or slice)
    @staticmethod
    def forward(ctx, x, group, sizes, grad_is_partial):
        ctx.group, ctx.sizes, ctx.partial = group, sizes, grad_is_partial
        return all_gather_first(x, group, sizes)

    @staticmethod
    def backward(ctx, g):
        if ctx.partial:
            return reduce_scatter_first(g, ctx.group, ctx.sizes), None, None, None
        _, n, r = _pg(ctx.group)
        if n == 1:
            return g, None, None, None
        if ctx.sizes is None:
            return g.chunk(n, dim=0)[r].contiguous(), None, None, None
        return g.split(list(ctx.sizes), dim=0)[r].contiguous(), None, None, None


class _ReduceScatterFirst(torch.autograd.Function):  # fwd reduce-scatter, bwd all-gather
    @staticmethod
    def forward(ctx, x, group, sizes):
        ctx.group, ctx.sizes = group, sizes
        return reduce_scatter_first(x, group, sizes)

    @staticmethod
    def backward(ctx, g):
        return all_gather_first(g, ctx.group, ctx.sizes), None, None


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, out_splits, in_splits):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        return all_to_all_first(x, group, out_splits, in_splits)

    @staticmethod
    def backward(ctx, g):
        return all_to_all_first(g, ctx.group, ctx.in_splits, ctx.out_splits), None, None, None


def copy_to_group(x, group):
    """Identity forward, all-reduce backward (input of a column-parallel linear without SP)."""
    return x if _pg(group)[1] == 1 else _Copy.apply(x, group)


def reduce_from_group(x, group):
    """All-reduce forward, identity backward (output of a row-parallel linear without SP)."""
    return x if _pg(group)[1] == 1 else _Reduce.apply(x, group)


all_reduce_sum = reduce_from_group


def scatter_first_dim(x, group, sizes=None):
    return x if _pg(group)[1] == 1 else _ScatterFirst.apply(x, group, sizes)


def gather_first_dim(x, group, sizes=None, grad_is_partial: bool = True):
    """All-gather along dim 0.  ``grad_is_partial=True`` (Megatron-SP): every rank's output gradient
    is a partial sum, so the backward is a reduce-scatter; ``False``: the gradients are replicas."""
    return x if _pg(group)[1] == 1 else _GatherFirst.apply(x, group, sizes, grad_is_partial)


def reduce_scatter_first_dim(x, group, sizes=None):
    return x if _pg(group)[1] == 1 else _ReduceScatterFirst.apply(x, group, sizes)


def all_to_all(x, group, out_splits=None, in_splits=None):
    return x if _pg(group)[1] == 1 else _AllToAll.apply(x, group, out_splits, in_splits)


def scatter_last_dim(x, group):
    pg, n, r = _pg(group)
    if n == 1:
        return x
    return scatter_first_dim(x.movedim(-1, 0).contiguous(), group).movedim(0, -1).contiguous()


def gather_last_dim(x, group, grad_is_partial: bool = False):
    pg, n, r = _pg(group)
    if n == 1:
        return x
    return gather_first_dim(x.movedim(-1, 0).contiguous(), group, None, grad_is_partial).movedim(0, -1).contiguous()


def reduce_scatter_last_dim(x, group):
    pg, n, r = _pg(group)
    if n == 1:
        return x
    return reduce_scatter_first_dim(x.movedim(-1, 0).contiguous(), group).movedim(0, -1).contiguous()


def broadcast_(t: torch.Tensor, src_global_rank: int, group) -> torch.Tensor:
    pg, n, _ = _pg(group)
    if n > 1:
        dist.broadcast(t, src=src_global_rank, group=pg)
    return t
