"""Peer-memory all-to-all with the layout transform folded in (``csrc/sm100/fused_a2a.cu``).

Ulysses sequence parallelism exchanges heads for sequence around the attention:

    seq_to_heads   ``[S/p, B, n, hd]``  ->  ``[S, B, n/p, hd]``
    heads_to_seq   ``[S, B, n/p, hd]``  ->  ``[S/p, B, n, hd]``

With NCCL each direction is a permute copy plus ``all_to_all_single``.  Here every rank publishes its tensor in a
symmetric staging buffer and the destination pulls its chunks from all peers straight into their final position of
a fresh local tensor (one kernel, peer loads over NVLink).  When there are fewer key/value heads than ranks, the
replication is never materialised: rank ``d`` simply pulls head ``d // (p / ng)``.

Staging has two parities.  Per call: copy into staging[parity] -> pull kernel, which carries the cross-rank rendezvous
itself (signal slots in symmetric memory, bounded wait; ``HG_A2A_RENDEZVOUS=nccl`` restores the older form below).
Older form: copy into staging[parity] -> ``peer_barrier`` (one-element all-reduce: every
rank's staging is complete) -> pull.  A parity is rewritten two calls later, after the next call's rendezvous has
shown that every rank finished pulling from it, so one rendezvous per call is enough.

Capability parity: galvatron/core/runtime/transformer/attention_impl.py:139-198 (layout pre/post), :316-405
(``DistributedAttention``, GQA replication :339-345), moe/token_dispatcher.py:510-689 for the row-list variant.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Tuple

import torch

from ..ops import _lib
from .fused_zero import SignalSlots, SymmetricBuffer, peer_barrier

_STAGING: Dict[Tuple[int, ...], "A2AStaging"] = {}


class A2AStaging:
    """Two symmetric staging slots per process group, grown on demand (growth is a collective: every rank of the
    group sees the same sizes in the same order, so they grow together)."""

    def __init__(self, group, nbytes: int, device):
        self.group, self.device = group, device
        self.capacity = nbytes
        self.slots = [SymmetricBuffer(nbytes, torch.uint8, device, group.group) for _ in range(2)]
        self.calls = 0
        # HG_A2A_RENDEZVOUS=nccl: a stream-ordered one-element all-reduce after the copy instead of the pull kernel's
        # own signal-slot rendezvous
        self.signals = SignalSlots.get(device, group.group, "a2a") if os.environ.get("HG_A2A_RENDEZVOUS", "kernel") == "kernel" else None
        for s in self.slots:
            s.signals, s.epoch, s.me = self.signals, 0, group.rank

    def publish(self, x: torch.Tensor) -> SymmetricBuffer:
        """Copy ``x`` into the next slot; returns the slot.  The pull kernel that follows waits until every rank of the
        group has published (``slot.epoch``); each publish must be followed by at least one pull on every rank.  The two
        slots alternate: a slot is written again only after the pull of the publish in between, whose rendezvous every
        peer enters after its reads of this one."""
        self.calls += 1
        slot = self.slots[self.calls & 1]
        nbytes = x.numel() * x.element_size()
        # one pass even when ``x`` is a strided view (e.g. q / k / v inside the packed QKV buffer)
        slot.tensor[:nbytes].view(x.dtype).view(x.shape).copy_(x)
        if self.signals is None:
            peer_barrier(self.group.group, self.device)
        else:
            slot.epoch = self.signals.next_epoch()
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
    from .fused_zero import available

    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and group is not None and 1 < group.size <= 8
            and (x.shape[-1] % 8 == 0) and available(x.device, group.size, group.group))


def _rendezvous_args(slot: SymmetricBuffer):
    sig = getattr(slot, "signals", None)
    if sig is None:
        return None, 0, 0
    return sig.buf.ptr_array(), slot.me, slot.epoch


def _gather(slot: SymmetricBuffer, rows, chunk, src_off, src_stride, out, out_peer_stride, out_row_stride):
    lib = _lib.load()
    sig, me, epoch = _rendezvous_args(slot)
    rc = lib.hg_peer_gather_bf16_rv(slot.ptr_array(), slot.t, rows, chunk, src_off, src_stride, out.data_ptr(),
                                    out_peer_stride, out_row_stride, sig, me, epoch, _lib.stream())
    _lib.check(rc, "hg_peer_gather_bf16")
    _lib.count_launch()


def _seq_to_heads(x: torch.Tensor, group, p: int, rep: int) -> torch.Tensor:
    """``x [S, B, n, hd]`` on every rank -> ``[p*S, B, m, hd]`` with ``m = n*rep/p`` heads of the whole sequence."""
    S, B, n, hd = x.shape
    d = group.rank
    m = max(1, n * rep // p)
    first_head = (d // rep) if rep > 1 else d * m
    slot = staging_for(group, x.numel() * 2, x.device).publish(x)
    out = torch.empty((p * S, B, m, hd), dtype=x.dtype, device=x.device)
    _gather(slot, S * B, m * hd, first_head * hd, n * hd, out, S * B * m * hd, m * hd)
    return out


def _heads_to_seq(y: torch.Tensor, group, p: int) -> torch.Tensor:
    """``y [p*S, B, m, hd]`` on every rank -> ``[S, B, p*m, hd]`` (this rank's sequence chunk, all heads)."""
    Sp, B, m, hd = y.shape
    S = Sp // p
    d = group.rank
    slot = staging_for(group, y.numel() * 2, y.device).publish(y)
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
    out = torch.empty((n_out, width), dtype=slot.tensor.dtype if slot.tensor.dtype.is_floating_point else _lib.lp_dtype(), device=peer.device)
    if _lib.DEBUG_KERNELS:     # the debug build checks every routed row against the size of the peers' buffers
        lib.hg_debug_set_gather_row_limit(slot.tensor.numel() * slot.tensor.element_size() // (2 * max(1, src_row_stride)))
    sig, me, epoch = _rendezvous_args(slot)
    rc = lib.hg_peer_gather_rows_bf16_rv(slot.ptr_array(), slot.t, peer.data_ptr(), row.data_ptr(), n_out, topk, width,
                                         src_row_stride, out.data_ptr(), _lib.ptr(scale), sig, me, epoch, _lib.stream())
    _lib.check(rc, "hg_peer_gather_rows_bf16")
    _lib.count_launch()
    return out


# Routed (token, expert) pairs dropped because a statically sized expert buffer was full, summed over the layers and
# iterations since the last read (a device scalar per device; see MoERouting(bound=...)).
OVERFLOW: Dict[str, torch.Tensor] = {}


def note_overflow(count: torch.Tensor):
    key = str(count.device)
    if key not in OVERFLOW:
        OVERFLOW[key] = torch.zeros((), dtype=torch.int64, device=count.device)
    OVERFLOW[key] += count


def read_overflow(device) -> int:
    """Host read (synchronises) and reset of the dropped-pair counter of ``device``."""
    t = OVERFLOW.get(str(device))
    if t is None:
        return 0
    v = int(t.item())
    t.zero_()
    return v


def static_bound(tokens: int, topk: int, experts_local: int, align: int, factor: float) -> int:
    """Rows of a statically sized expert buffer: ``factor`` times the balanced load of a rank (``tokens * topk``
    pairs) plus the worst-case alignment padding of its local experts, rounded up to ``align``."""
    rows = int(factor * tokens * topk) + experts_local * align
    return (rows + align - 1) // align * align


class MoERouting:
    """Placement of every routed (rank, token, slot) of an expert-parallel group, computed identically on every rank
    from the all-gathered top-k expert indices.

    Destination rank ``D`` lays its local experts out as aligned, zero-padded segments; within an expert the rows
    are ordered by (source rank, token, slot).  From that one table follow

    * ``peer_d / tok_d / slot_d`` ``[total_D]``: for each row of this rank's expert buffer, where it comes from
      (``-1`` for padding rows);
    * ``peer_s / row_s`` ``[T*k]``: for each of this rank's (token, slot) pairs, where its expert output lives
      (``-1`` for dropped pairs);
    * ``row_start`` ``[E_loc + 1]`` int32 segment starts for the grouped GEMM; ``totals`` rows per rank (host list).
    """

    def __init__(self, idx: torch.Tensor, group, num_experts: int, align: int, bound: int = 0):
        """``bound`` > 0: every rank's expert buffer has exactly ``bound`` rows (a static size), the whole table is
        built on the device and nothing is read back on the host; pairs that would land beyond ``bound`` are dropped
        and counted in :data:`OVERFLOW` (checked once per iteration by the training loop).  ``bound`` = 0: the
        buffers are sized exactly, which costs one host read of the per-rank totals per layer call."""
        import torch.distributed as dist

        ep, me = group.size, group.rank
        T, k = idx.shape
        E, E_loc = num_experts, num_experts // ep
        dev = idx.device
        idx_all = torch.empty((ep, T, k), dtype=idx.dtype, device=dev)
        dist.all_gather_into_tensor(idx_all, idx.contiguous(), group=group.group)
        flat = idx_all.reshape(-1).long()
        valid = flat >= 0
        key = torch.where(valid, flat, torch.full_like(flat, E))
        order = torch.argsort(key, stable=True)
        key_sorted = key[order]
        # (not torch.bincount: it reads the largest key back on the host)
        counts = torch.zeros(E + 1, dtype=torch.int64, device=dev).scatter_add_(0, key, torch.ones_like(key))[:E]
        ustart = torch.cumsum(counts, 0) - counts
        padded = (counts + align - 1) // align * align
        per_rank = padded.view(ep, E_loc)
        astart = (torch.cumsum(per_rank, 1) - per_rank).reshape(-1)            # start of each expert on its rank
        totals_t = per_rank.sum(1).clamp(min=align)
        n_valid_sorted = key_sorted < E
        ks = key_sorted.clamp(max=E - 1)
        pos = torch.arange(flat.numel(), device=dev) - ustart[ks]
        dest_row_sorted = torch.where(n_valid_sorted, astart[ks] + pos, torch.full_like(pos, -1))
        dest_row = torch.empty_like(dest_row_sorted)
        dest_row[order] = dest_row_sorted
        dest_rank = torch.where(valid, flat // E_loc, torch.full_like(flat, -1))
        self.T, self.k, self.ep, self.me = T, k, ep, me
        n = T * k
        local_astart = astart.view(ep, E_loc)[me]
        self.group = group
        if bound > 0:
            # static buffers, no host reads: rows beyond the bound are dropped (and reported), the rows of this rank's
            # buffer are filled by a scatter over all (rank, token, slot) entries with a dump slot for foreign ones
            self.total = self.max_total = int(bound)
            self.totals = [int(bound)] * ep
            fits = dest_row < bound
            note_overflow(((dest_rank >= 0) & ~fits).sum())
            dest_rank = torch.where(fits, dest_rank, torch.full_like(dest_rank, -1))
            self.peer_s = dest_rank[me * n:(me + 1) * n].to(torch.int32).contiguous()
            self.row_s = dest_row[me * n:(me + 1) * n].clamp(min=0, max=bound - 1).to(torch.int32).contiguous()
            every = torch.arange(flat.numel(), device=dev)
            tgt = torch.where(dest_rank == me, dest_row, torch.full_like(dest_row, bound))
            r_of, rem = (every // n).to(torch.int32), every % n
            self.peer_d = torch.full((bound + 1,), -1, dtype=torch.int32, device=dev).scatter_(0, tgt, r_of)[:bound].contiguous()
            self.tok_d = torch.zeros((bound + 1,), dtype=torch.int32, device=dev).scatter_(0, tgt, (rem // k).to(torch.int32))[:bound].contiguous()
            self.slot_d = torch.zeros((bound + 1,), dtype=torch.int32, device=dev).scatter_(0, tgt, rem.to(torch.int32))[:bound].contiguous()
            ends = torch.cat([local_astart, per_rank[me].sum().reshape(1)]).clamp(max=bound)
            self.row_start = ends.to(torch.int32)
            return
        self.totals = [int(x) for x in totals_t.tolist()]                      # one host read per layer call
        self.total, self.max_total = self.totals[me], max(self.totals)
        self.peer_s = dest_rank[me * n:(me + 1) * n].to(torch.int32).contiguous()
        self.row_s = dest_row[me * n:(me + 1) * n].clamp(min=0).to(torch.int32).contiguous()
        mine = dest_rank == me
        src_flat = torch.nonzero(mine, as_tuple=False).squeeze(1)              # index into (r, t, slot)
        rows = dest_row[src_flat]
        self.peer_d = torch.full((self.total,), -1, dtype=torch.int32, device=dev)
        self.tok_d = torch.zeros((self.total,), dtype=torch.int32, device=dev)
        self.slot_d = torch.zeros((self.total,), dtype=torch.int32, device=dev)
        r_of, rem = src_flat // n, src_flat % n
        self.peer_d[rows] = r_of.to(torch.int32)
        self.tok_d[rows] = (rem // k).to(torch.int32)
        self.slot_d[rows] = rem.to(torch.int32)
        self.row_start = torch.cat([local_astart, per_rank[me].sum().reshape(1)]).to(torch.int32)


def _publish_sized(group, x: torch.Tensor, rows_bound: int) -> SymmetricBuffer:
    """Publish ``x [rows, width]``; the staging is sized by ``rows_bound`` (the same number on every rank)."""
    st = staging_for(group, rows_bound * x.shape[1] * 2, x.device)
    return st.publish(x)


class _MoEDispatch(torch.autograd.Function):
    """``x [T, H]`` on every rank -> this rank's expert buffer ``[total, H]`` (aligned, zero-padded segments)."""

    @staticmethod
    def forward(ctx, x, plan: MoERouting):
        ctx.plan = plan
        slot = _publish_sized(plan.group, x, plan.T)
        return gather_rows(slot, plan.peer_d, plan.tok_d, plan.total, x.shape[1], x.shape[1])

    @staticmethod
    def backward(ctx, g):
        p = ctx.plan
        slot = _publish_sized(p.group, g, p.max_total)
        # every token sums the gradients of its k copies, wherever they were processed
        return gather_rows(slot, p.peer_s.view(p.T, p.k), p.row_s.view(p.T, p.k), p.T, g.shape[1], g.shape[1], p.k), None


class _MoECombine(torch.autograd.Function):
    """Expert outputs ``[total, H]`` on every rank -> ``[T*k, H]``: each (token, slot) pair's output back home
    (zeros for dropped pairs)."""

    @staticmethod
    def forward(ctx, y, plan: MoERouting):
        ctx.plan = plan
        slot = _publish_sized(plan.group, y, plan.max_total)
        return gather_rows(slot, plan.peer_s, plan.row_s, plan.T * plan.k, y.shape[1], y.shape[1])

    @staticmethod
    def backward(ctx, g):
        p = ctx.plan
        slot = _publish_sized(p.group, g, p.T * p.k)
        return gather_rows(slot, p.peer_d, p.slot_d, p.total, g.shape[1], g.shape[1]), None


class _MoECombineWeighted(torch.autograd.Function):
    """``out[t] = sum_k w[t, k] * y_{peer}[row(t, k)]``: the combine with the routing weights applied inside the pull
    kernel.  Backward: ``dy[row] = w(row) * g[token(row)]`` (one weighted pull of the token gradients, the weights of
    a row's (token, slot) pair looked up in the gathered weight table) and ``dw[t, k] = <g[t], y_row(t, k)>`` (the
    rows are pulled once more; nothing of size ``[T, k, H]`` is kept between forward and backward)."""

    @staticmethod
    def forward(ctx, y, w, plan: MoERouting):
        ctx.plan = plan
        ctx.save_for_backward(y, w)
        slot = _publish_sized(plan.group, y, plan.max_total)
        p = plan
        return gather_rows(slot, p.peer_s.view(p.T, p.k), p.row_s.view(p.T, p.k), p.T, y.shape[1], y.shape[1], p.k,
                           scale=w.contiguous())

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist

        p = ctx.plan
        y, w = ctx.saved_tensors
        g = g.contiguous()
        H = g.shape[1]
        # weights of the rows of this rank's expert buffer: w_all[source rank, token * k + slot]
        w_all = torch.empty((p.ep, p.T * p.k), dtype=w.dtype, device=w.device)
        dist.all_gather_into_tensor(w_all, w.reshape(-1).contiguous(), group=p.group.group)
        src = p.peer_d.clamp(min=0).long()
        w_d = torch.where(p.peer_d >= 0, w_all[src, p.slot_d.long()], torch.zeros((), dtype=w.dtype, device=w.device))
        slot = _publish_sized(p.group, g, p.T)
        dy = gather_rows(slot, p.peer_d, p.tok_d, p.total, H, H, 1, scale=w_d.float().contiguous())
        slot_y = _publish_sized(p.group, y, p.max_total)
        rows = gather_rows(slot_y, p.peer_s, p.row_s, p.T * p.k, H, H).view(p.T, p.k, H)
        dw = (rows.float() * g.float().unsqueeze(1)).sum(-1).to(w.dtype)
        return dy, dw, None


def moe_combine_weighted(y, w, plan: MoERouting):
    return _MoECombineWeighted.apply(y, w, plan)


def moe_dispatch(x, plan: MoERouting):
    return _MoEDispatch.apply(x, plan)


def moe_combine(y, plan: MoERouting):
    return _MoECombine.apply(y, plan)
