"""Peer-memory all-to-all with the layout transform folded in (``csrc/sm100/fused_a2a.cu``).

Ulysses sequence parallelism exchanges heads for sequence around the attention:

    seq_to_heads   ``[S/p, B, n, hd]``  ->  ``[S, B, n/p, hd]``
    heads_to_seq   ``[S, B, n/p, hd]``  ->  ``[S/p, B, n, hd]``

With NCCL each direction is a permute copy plus ``all_to_all_single``.  Here every rank publishes its tensor in a
symmetric staging buffer and the destination pulls its chunks from all peers straight into their final position of
a fresh local tensor (one kernel, peer loads over NVLink).  When there are fewer key/value heads than ranks, the
replication is never materialised: rank ``d`` simply pulls head ``d // (p / ng)``.

Staging has two parities.  Per call: copy into staging[parity] -> ``peer_barrier`` (one-element all-reduce: every
rank's staging is complete) -> pull.  A parity is rewritten two calls later, after the next call's rendezvous has
shown that every rank finished pulling from it, so one rendezvous per call is enough.
The kernels never wait on another GPU.

Capability parity: galvatron/core/runtime/transformer/attention_impl.py:139-198 (layout pre/post), :316-405
(``DistributedAttention``, GQA replication :339-345), moe/token_dispatcher.py:510-689 for the row-list variant.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Tuple

import torch

from ..ops import _lib
from .fused_zero import SymmetricBuffer, peer_barrier

_STAGING: Dict[Tuple[int, ...], "A2AStaging"] = {}


class A2AStaging:
    """Two symmetric staging slots per process group, grown on demand (growth is a collective: every rank of the
    group sees the same sizes in the same order, so they grow together)."""

    def __init__(self, group, nbytes: int, device):
        self.group, self.device = group, device
        self.capacity = nbytes
        self.slots = [SymmetricBuffer(nbytes, torch.uint8, device, group.group) for _ in range(2)]
        self.calls = 0

    def publish(self, x: torch.Tensor) -> SymmetricBuffer:
        """Copy ``x`` (contiguous) into the next slot and rendezvous; returns the slot."""
        self.calls += 1
        slot = self.slots[self.calls & 1]
        nbytes = x.numel() * x.element_size()
        slot.tensor[:nbytes].view(x.dtype).copy_(x.reshape(-1))
        peer_barrier(self.group.group, self.device)
        return slot


def staging_for(group, nbytes: int, device) -> A2AStaging:
    key = tuple(group.ranks)
    st = _STAGING.get(key)
    if st is None or st.capacity < nbytes:
        if st is not None:
            # peers may still be pulling from the old slots: rendezvous before dropping them
            peer_barrier(group.group, device)
            torch.cuda.synchronize(device)
        st = _STAGING[key] = A2AStaging(group, max(nbytes, 2 * st.capacity if st else nbytes), device)
    return st


def usable(x: torch.Tensor, group) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and group is not None and 1 < group.size <= 8
            and (x.shape[-1] % 8 == 0))


def _gather(slot: SymmetricBuffer, rows, chunk, src_off, src_stride, out, out_peer_stride, out_row_stride):
    lib = _lib.load()
    rc = lib.hg_peer_gather_bf16(slot.ptr_array(), slot.t, rows, chunk, src_off, src_stride, out.data_ptr(),
                                 out_peer_stride, out_row_stride, _lib.stream())
    _lib.check(rc, "hg_peer_gather_bf16")
    _lib.count_launch()


def _seq_to_heads(x: torch.Tensor, group, p: int, rep: int) -> torch.Tensor:
    """``x [S, B, n, hd]`` on every rank -> ``[p*S, B, m, hd]`` with ``m = n*rep/p`` heads of the whole sequence."""
    S, B, n, hd = x.shape
    d = group.rank
    m = max(1, n * rep // p)
    first_head = (d // rep) if rep > 1 else d * m
    slot = staging_for(group, x.numel() * 2, x.device).publish(x.contiguous())
    out = torch.empty((p * S, B, m, hd), dtype=x.dtype, device=x.device)
    _gather(slot, S * B, m * hd, first_head * hd, n * hd, out, S * B * m * hd, m * hd)
    return out


def _heads_to_seq(y: torch.Tensor, group, p: int) -> torch.Tensor:
    """``y [p*S, B, m, hd]`` on every rank -> ``[S, B, p*m, hd]`` (this rank's sequence chunk, all heads)."""
    Sp, B, m, hd = y.shape
    S = Sp // p
    d = group.rank
    slot = staging_for(group, y.numel() * 2, y.device).publish(y.contiguous())
    out = torch.empty((S, B, p * m, hd), dtype=y.dtype, device=y.device)
    _gather(slot, S * B, m * hd, d * S * B * m * hd, m * hd, out, m * hd, p * m * hd)
    return out


class _SeqToHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, p, rep):
        ctx.group, ctx.p, ctx.rep, ctx.n = group, p, rep, x.shape[2]
        return _seq_to_heads(x, group, p, rep)

    @staticmethod
    def backward(ctx, g):
        z = _heads_to_seq(g, ctx.group, ctx.p)        # [S, B, p*m, hd]
        if ctx.rep > 1:                               # replicated kv heads: sum the replicas' gradients
            S, B, _, hd = z.shape
            z = z.view(S, B, ctx.n, ctx.rep, hd).float().sum(3).to(g.dtype)
        return z, None, None, None


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, group, p):
        ctx.group, ctx.p = group, p
        return _heads_to_seq(y, group, p)

    @staticmethod
    def backward(ctx, g):
        return _seq_to_heads(g, ctx.group, ctx.p, 1), None, None


def seq_to_heads(x, group, p: int, rep: int = 1):
    return _SeqToHeads.apply(x, group, p, rep)


def heads_to_seq(y, group, p: int):
    return _HeadsToSeq.apply(y, group, p)


# ---- row lists (mixture-of-experts dispatch / combine) ----------------------------------------------------------
def gather_rows(slot: SymmetricBuffer, peer: torch.Tensor, row: torch.Tensor, n_out: int, width: int,
                src_row_stride: int, topk: int = 1, scale: torch.Tensor = None) -> torch.Tensor:
    """``out[o] = sum_k scale[o, k] * src_{peer[o, k]}[row[o, k]]`` over the peers' staging slots (bf16 rows)."""
    lib = _lib.load()
    out = torch.empty((n_out, width), dtype=torch.bfloat16, device=peer.device)
    rc = lib.hg_peer_gather_rows_bf16(slot.ptr_array(), slot.t, peer.data_ptr(), row.data_ptr(), n_out, topk, width,
                                      src_row_stride, out.data_ptr(), _lib.ptr(scale), _lib.stream())
    _lib.check(rc, "hg_peer_gather_rows_bf16")
    _lib.count_launch()
    return out
