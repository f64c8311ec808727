"""DeepSpeed-Ulysses sequence parallelism: heads <-> sequence exchange around a local attention.

Between layers the activation is sequence-sharded ``[S/p, B, H]`` and the weights are whole.  Inside the
attention, one all-to-all turns ``[S/p, B, n, hd]`` into ``[S, B, n/p, hd]`` (every rank sees the whole
sequence for ``n/p`` heads), attention runs locally, and a second all-to-all restores the sequence
sharding.  In the ``[S, B, ...]`` layout the received blocks are already in sequence order, so each
direction needs a single permute copy (the reference's ``[B, S, ...]`` path needs two;
galvatron/core/runtime/transformer/attention_impl.py:115-198, :278-405).  When there are fewer kv heads than
ranks they are replicated ``p / ng`` times first (attention_impl.py:339-345).
"""
from __future__ import annotations

import torch

from .. import ops
from . import mappings as mp


def seq_to_heads(x: torch.Tensor, group, p: int) -> torch.Tensor:
    """``[S_loc, B, n, hd]`` -> ``[S_loc * p, B, n / p, hd]``"""
    S, B, n, hd = x.shape
    xs = x.reshape(S, B, p, n // p, hd).permute(2, 0, 1, 3, 4).contiguous().view(p * S, B, n // p, hd)
    return mp.all_to_all(xs, group)


def heads_to_seq(y: torch.Tensor, group, p: int) -> torch.Tensor:
    """``[S_loc * p, B, n / p, hd]`` -> ``[S_loc, B, n, hd]``"""
    Sp, B, m, hd = y.shape
    S = Sp // p
    z = mp.all_to_all(y.contiguous(), group).view(p, S, B, m, hd)
    return z.permute(1, 2, 0, 3, 4).reshape(S, B, p * m, hd)


def ulysses_attention(q, k, v, ctx, S_full: int):
    """q ``[S_loc, B, nh, hd]``, k / v ``[S_loc, B, ng, hd]`` (RoPE already applied) -> ``[S_loc, B, nh, hd]``."""
    p = ctx.sp_size
    nh, ng = q.shape[2], k.shape[2]
    if nh % p:
        raise ValueError("query heads (%d) must be divisible by the Ulysses degree %d" % (nh, p))
    if getattr(ctx, "fused_comm", False) and (ng % p == 0 or p % ng == 0):
        from . import fused_a2a as fa

        if fa.usable(q, ctx.sp):
            # peer-memory path: the exchange and the layout change are one pull kernel per tensor; kv heads that
            # would be replicated are pulled from their single owner instead
            rep = p // ng if ng < p else 1
            qg = fa.seq_to_heads(q, ctx.sp, p)
            kg = fa.seq_to_heads(k, ctx.sp, p, rep)
            vg = fa.seq_to_heads(v, ctx.sp, p, rep)
            if ctx.cp_size > 1:
                from .ring_attention import ring_attention

                og = ring_attention(qg, kg, vg, ctx.cp, S_full)
            else:
                og = ops.flash_attention(qg, kg, vg, causal=True)
            return fa.heads_to_seq(og, ctx.sp, p)
    if ng < p:
        rep = p // ng
        k = k.repeat_interleave(rep, dim=2)
        v = v.repeat_interleave(rep, dim=2)
    elif ng % p:
        raise ValueError("kv heads (%d) must be divisible by the Ulysses degree %d" % (ng, p))
    qg, kg, vg = seq_to_heads(q, ctx.sp, p), seq_to_heads(k, ctx.sp, p), seq_to_heads(v, ctx.sp, p)
    if ctx.cp_size > 1:
        from .ring_attention import ring_attention

        og = ring_attention(qg, kg, vg, ctx.cp, S_full)
    else:
        og = ops.flash_attention(qg, kg, vg, causal=True)
    return heads_to_seq(og, ctx.sp, p)
