"""Context parallelism over a zig-zag split of the sequence.

The sequence is cut into ``2c`` chunks; rank ``r`` owns chunks ``r`` and ``2c-1-r`` (so that causal work is
balanced).  Two implementations of the attention over the whole sequence:

``ring_attention`` (default)
    K/V blocks travel around the ring of the ``c`` ranks, one hop per step, while every rank keeps only its own
    block plus the one in flight: K/V memory is O(S/c) per rank.  Step ``t`` works on the block of rank
    ``(r - t) mod c``; of the four (query chunk, key chunk) pairs of a step only the causally visible ones are
    computed, each with one flash-attention call at the chunks' global positions, and the partial results are
    merged through their log-sum-exp.  The exchange of step ``t + 1`` is posted before the compute of step ``t``.
    The backward recomputes the probabilities from the *global* log-sum-exp, so every pair yields exact partial
    gradients: dQ accumulates locally, dK/dV accumulators travel with their block and arrive at its owner after
    the last hop.

``allgather_attention`` (``HG_CP_ALLGATHER=1``)
    K and V of the whole group are all-gathered once and put into natural order; each local query chunk attends
    to its causal prefix in one call.  Fewer, larger kernels, but O(S) K/V memory per rank.

Capability parity: galvatron/core/runtime/transformer/attention_impl.py:564-780 (zig-zag ring forward /
backward with LSE merging), :437-478 (merge), utils/utils.py:295-325 (batch slicing).
"""
from __future__ import annotations

import math
import os
from typing import List, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..ops.attention import flash_backward
from . import mappings as mp
from .reshard import undo_zigzag


def step_pairs(r: int, src: int, c: int) -> List[Tuple[int, int]]:
    """Causally visible (query half, key half) pairs when rank ``r`` holds the K/V block of rank ``src``.

    Halves: 0 = the rank's early chunk (index ``rank``), 1 = its late chunk (index ``2c-1-rank``).  A query chunk
    sees a key chunk with a smaller or equal index."""
    q_chunks = (r, 2 * c - 1 - r)
    k_chunks = (src, 2 * c - 1 - src)
    return [(qi, kj) for qi in (0, 1) for kj in (0, 1) if k_chunks[kj] <= q_chunks[qi]]


def merge_partial(out_acc: torch.Tensor, lse_acc: torch.Tensor, out_new: torch.Tensor, lse_new: torch.Tensor):
    """Fold a partial attention result over a disjoint key set into the running one, in place.
    ``out_acc`` fp32 ``[S, B, h, d]``, ``lse_acc`` fp32 ``[B, h, S]`` (``-inf`` where nothing was seen yet)."""
    if out_acc.is_cuda:
        return ops.attention_merge(out_acc, lse_acc, out_new, lse_new)
    lse = torch.logaddexp(lse_acc, lse_new)
    wa = torch.exp(lse_acc - lse).permute(2, 0, 1).unsqueeze(-1)
    wb = torch.exp(lse_new - lse).permute(2, 0, 1).unsqueeze(-1)
    out_acc.mul_(wa).add_(out_new.float() * wb)
    lse_acc.copy_(lse)


def _exchange(send: torch.Tensor, recv: torch.Tensor, group):
    """Send ``send`` to the next rank of the ring and receive ``recv`` from the previous one; returns the requests."""
    ranks = group.ranks
    nxt, prv = ranks[(group.rank + 1) % group.size], ranks[(group.rank - 1) % group.size]
    if send.is_cuda:
        # one NCCL group: with two ranks the previous and the next rank are the same peer, and a receive queued in
        # front of the matching send on that peer's stream would wait forever
        return dist.batch_isend_irecv([dist.P2POp(dist.isend, send, nxt, group=group.group),
                                       dist.P2POp(dist.irecv, recv, prv, group=group.group)])
    return [dist.isend(send, dst=nxt, group=group.group), dist.irecv(recv, src=prv, group=group.group)]


def _wait(reqs):
    for r in reqs:
        r.wait()


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, scale):
        c, r = group.size, group.rank
        S_loc, B, nh, hd = q.shape
        half = S_loc // 2
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        cur = torch.stack([k, v])                                   # one message per hop
        out_acc = torch.zeros((S_loc, B, nh, hd), dtype=torch.float32, device=q.device)
        lse_acc = torch.full((B, nh, S_loc), float("-inf"), dtype=torch.float32, device=q.device)
        for t in range(c):
            nxt, reqs = None, []
            if t + 1 < c:
                nxt = torch.empty_like(cur)
                reqs = _exchange(cur, nxt, group)                   # travels under this step's compute
            src = (r - t) % c
            qc, kc = (r, 2 * c - 1 - r), (src, 2 * c - 1 - src)
            for qi, kj in step_pairs(r, src, c):
                qs, ks = slice(qi * half, (qi + 1) * half), slice(kj * half, (kj + 1) * half)
                o, lse = ops.flash_attention(q[qs], cur[0][ks], cur[1][ks], causal=True, scale=scale,
                                             q_pos0=qc[qi] * half, k_pos0=kc[kj] * half, return_lse=True)
                merge_partial(out_acc[qs], lse_acc[:, :, qs], o, lse)
            _wait(reqs)
            if nxt is not None:
                cur = nxt
        out = out_acc.to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse_acc)
        ctx.group, ctx.scale = group, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        group, scale = ctx.group, ctx.scale
        c, r = group.size, group.rank
        S_loc, B, nh, hd = q.shape
        half = S_loc // 2
        dout = dout.contiguous()
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        cur = torch.stack([k, v])
        acc = None                                                   # fp32 dK/dV of the block in hand, travelling with it
        for t in range(c):
            nxt, reqs = None, []
            if t + 1 < c:
                nxt = torch.empty_like(cur)
                reqs = _exchange(cur, nxt, group)
            src = (r - t) % c
            qc, kc = (r, 2 * c - 1 - r), (src, 2 * c - 1 - src)
            part = torch.zeros((2,) + tuple(k.shape), dtype=torch.float32, device=q.device)
            for qi, kj in step_pairs(r, src, c):
                qs, ks = slice(qi * half, (qi + 1) * half), slice(kj * half, (kj + 1) * half)
                if q.is_cuda:
                    dq_p, dk_p, dv_p = flash_backward(q[qs], cur[0][ks], cur[1][ks], out[qs], dout[qs],
                                                      lse[:, :, qs].contiguous(), True, scale, qc[qi] * half, kc[kj] * half)
                else:
                    dq_p, dk_p, dv_p = _reference_backward(q[qs], cur[0][ks], cur[1][ks], dout[qs], out[qs], lse[:, :, qs],
                                                           scale, qc[qi] * half, kc[kj] * half)
                dq[qs] += dq_p
                part[0][ks] += dk_p
                part[1][ks] += dv_p
            if acc is not None:
                _wait(acc_reqs)
                part += acc_in
            _wait(reqs)
            if nxt is not None:
                cur = nxt
            # hand the block's accumulator to the next rank, which works on the same block in its next step; after the
            # last step one more hop brings every accumulator to the block's owner
            acc_in = torch.empty_like(part)
            acc_reqs = _exchange(part, acc_in, group)
            acc = part
        _wait(acc_reqs)
        dk, dv = acc_in[0].to(k.dtype), acc_in[1].to(v.dtype)
        return dq.to(q.dtype), dk, dv, None, None


def _reference_backward(q, k, v, dout, out, lse, scale, q_pos0, k_pos0):
    """fp32 backward of one (query chunk, key chunk) pair from the global log-sum-exp (CPU oracle path)."""
    S, B, nh, hd = q.shape
    Skv, ng = k.shape[0], k.shape[2]
    rep = nh // ng
    qf, dof, of = (t.float().permute(1, 2, 0, 3) for t in (q, dout, out))
    kf = k.float().permute(1, 2, 0, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(1, 2, 0, 3).repeat_interleave(rep, dim=1)
    s = torch.einsum("bhqd,bhkd->bhqk", qf, kf) * scale
    qp = torch.arange(S, device=q.device) + q_pos0
    kp = torch.arange(Skv, device=q.device) + k_pos0
    s = s.masked_fill(kp[None, :] > qp[:, None], float("-inf"))
    p = torch.exp(s - lse[..., None])
    dsum = (dof * of).sum(-1, keepdim=True)
    dp = torch.einsum("bhqd,bhkd->bhqk", dof, vf)
    ds = p * (dp - dsum) * scale
    dq = torch.einsum("bhqk,bhkd->bhqd", ds, kf).permute(2, 0, 1, 3)
    dk = torch.einsum("bhqk,bhqd->bhkd", ds, qf).view(B, ng, rep, Skv, hd).sum(2).permute(2, 0, 1, 3)
    dv = torch.einsum("bhqk,bhqd->bhkd", p, dof).view(B, ng, rep, Skv, hd).sum(2).permute(2, 0, 1, 3)
    return dq, dk, dv


def allgather_attention(q, k, v, cp_group, S_full: int):
    """All-gather variant: K / V of the whole group in natural order, one flash call per local query chunk."""
    c, r = cp_group.size, cp_group.rank
    half = q.shape[0] // 2
    k_all = undo_zigzag(mp.gather_first_dim(k, cp_group, grad_is_partial=True), c)
    v_all = undo_zigzag(mp.gather_first_dim(v, cp_group, grad_is_partial=True), c)
    outs = []
    for qi, chunk in ((0, r), (1, 2 * c - 1 - r)):
        qc = q[qi * half:(qi + 1) * half]
        hi = (chunk + 1) * half
        outs.append(ops.flash_attention(qc, k_all[:hi], v_all[:hi], causal=True, q_pos0=chunk * half, k_pos0=0))
    return torch.cat(outs, dim=0)


def ring_attention(q, k, v, cp_group, S_full: int):
    """q ``[S/c, B, nh, hd]``, k / v ``[S/c, B, ng, hd]`` in zig-zag order -> ``[S/c, B, nh, hd]``."""
    c = cp_group.size if cp_group is not None else 1
    if c == 1:
        return ops.flash_attention(q, k, v, causal=True)
    if os.environ.get("HG_CP_ALLGATHER", "0") == "1":
        return allgather_attention(q, k, v, cp_group, S_full)
    return _RingAttention.apply(q, k, v, cp_group, 1.0 / math.sqrt(q.shape[-1]))
