"""ZeRO gradient reduce-scatter and "AdamW + parameter all-gather" as our own kernels over NVLink peer memory
(``csrc/sm100/fused_zero.cu``).

A wrap unit that uses this path keeps its flat fp32 gradient buffer and its flat bf16 parameter buffer in symmetric
memory (same size on every rank of the sharding group, mapped into every peer).  Per optimizer step:

1. ``peer_barrier``          one-element all-reduce: every rank's backward has finished writing its gradients
                             (bf16 wire: has finished rounding them into the staging buffer);
2. ``reduce_scatter_peer`` / ``reduce_scatter_staged``
                             this rank's shard = sum over ranks of their buffers' slice (peer loads, fp32 or bf16);
3. (global gradient norm -- a scalar all-reduce over all ranks, which also orders step 2 on every rank before 4)
4. ``adamw_allgather_peer``  AdamW on the shard; bf16 results stored into every rank's parameter buffer;
5. ``peer_barrier``          every rank's stores have landed before anyone's next forward.

The kernels never wait on another GPU; the ordering comes from the stream-ordered collectives of steps 1, 3, 5.
This replaces FSDP's reduce-scatter / all-gather around the optimizer in the reference
(galvatron/core/runtime/parallel.py:119-152, pipeline/grad_reduce.py:48-65, optimizer/utils.py:43-52).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib

MAX_PEERS = 8


GUARD_BYTES = 512          # debug build: canary region before and after every symmetric buffer
GUARD_BYTE = 0xA5
_GUARDED: List["SymmetricBuffer"] = []


class SymmetricBuffer:
    """A tensor allocated identically on every rank of ``pg`` and mapped into all of them.

    With ``HG_DEBUG_KERNELS=1`` the allocation carries a canary region on both sides that peers and local kernels must
    never write; :func:`verify_guards` checks them (a peer store that ran past its slice lands there first)."""

    def __init__(self, numel: int, dtype, device, pg):
        from .symm_vmm import allocate

        esize = torch.empty(0, dtype=dtype).element_size()
        guard = GUARD_BYTES // esize if _lib.DEBUG_KERNELS else 0
        raw, base, self.handle = allocate((numel + 2 * guard) * esize, device, pg)
        self._raw = raw.view(dtype)
        self.tensor = self._raw[guard:guard + numel]
        self.ptrs: List[int] = [int(p) + guard * esize for p in base]
        self.t = len(self.ptrs)
        self._guard = guard
        if guard:
            for g in self._guards():
                g.view(torch.uint8).fill_(GUARD_BYTE)
            _GUARDED.append(self)

    def _guards(self):
        g = self._guard
        return (self._raw[:g], self._raw[self._raw.numel() - g:])

    def guards_intact(self) -> bool:
        return self._guard == 0 or all(bool((g.view(torch.uint8) == GUARD_BYTE).all()) for g in self._guards())

    def ptr_array(self, byte_offset: int = 0):
        return (ctypes.c_void_p * self.t)(*[p + byte_offset for p in self.ptrs])


def verify_guards() -> int:
    """Number of symmetric buffers whose canary regions were overwritten (always 0 outside the debug build)."""
    return sum(0 if b.guards_intact() else 1 for b in _GUARDED)


_PROBED: Dict[tuple, bool] = {}


def symmetric_memory_works(device, pg) -> bool:
    """Whether symmetric memory can really be set up over ``pg`` on this machine: a one-time probe that allocates a
    small buffer, runs the rendezvous and reads the peer pointers, then agrees on the outcome over the group (a rank
    where the probe failed makes every rank of the group fall back to NCCL together, with one warning).  Collective
    over ``pg``; the answer is cached."""
    key = (str(device), id(pg))
    if key in _PROBED:
        return _PROBED[key]
    ok = 1
    why = ""
    try:
        from .symm_vmm import allocate

        _buf, ptrs, _owner = allocate(256, device, pg)
        if len(ptrs) != dist.get_world_size(pg):
            ok, why = 0, "the allocator returned %d peer pointers" % len(ptrs)
        if hasattr(_owner, "close"):
            torch.cuda.synchronize(device)
            dist.barrier(group=pg)
            _owner.close()
    except Exception as e:     # no peer access, no fabric handle support, an older torch, ...
        ok, why = 0, "%s: %s" % (type(e).__name__, str(e)[:200])
    flag = torch.tensor([ok], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=pg)
    works = bool(int(flag.item()))
    if not works and dist.get_rank(pg) == 0:
        import warnings

        warnings.warn("symmetric memory is not usable over this group (%s): the peer-memory kernels are off for it and "
                      "NCCL carries the traffic" % (why or "a peer rank could not set it up"))
    _PROBED[key] = works
    return works


def available(device, n: int, pg=None) -> bool:
    """Peer-memory kernels can serve a group of ``n`` ranks on ``device`` (2..8 ranks of one node, CUDA, and, when the
    process group is given, a successful :func:`symmetric_memory_works` probe)."""
    if device.type != "cuda" or n < 2 or n > MAX_PEERS:
        return False
    from ..utils.runtime_utils import is_torch_min_version

    if not is_torch_min_version("2.5.0"):      # torch.distributed._symmetric_memory appeared in 2.5
        return False
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception:
        return False
    return True if pg is None else symmetric_memory_works(device, pg)


_TICKS: Dict[Tuple[int, int], torch.Tensor] = {}


def peer_barrier(pg, device):
    """Stream-ordered rendezvous of the group: when it completes on this rank's stream, everything queued before
    it on every rank's stream has completed."""
    key = (id(pg), device.index if device.index is not None else 0)
    t = _TICKS.get(key)
    if t is None:
        t = _TICKS[key] = torch.zeros(1, dtype=torch.float32, device=device)
    dist.all_reduce(t, group=pg)


def reduce_scatter_peer(grads: SymmetricBuffer, me: int, shard_numel: int, out: torch.Tensor, max_ctas: int = 0):
    """fp32 on the wire: ``out = sum_r grads_r[me*S:(me+1)*S]`` by peer loads.  ``max_ctas`` caps the grid (0 = none)."""
    lib = _lib.load()
    rc = lib.hg_zero_reduce_scatter_capped(grads.ptr_array(), grads.t, me, shard_numel, out.data_ptr(), int(max_ctas),
                                           _lib.stream())
    _lib.check(rc, "hg_zero_reduce_scatter")
    _lib.count_launch()
    return out


class SignalSlots:
    """Per-group signal words in symmetric memory (``int32[8]`` per rank) and the call counter that the ranks of the
    group advance in lockstep: the bf16-wire reduce-scatter publishes / awaits ``epoch`` through them."""

    _by_group: Dict[tuple, "SignalSlots"] = {}

    def __init__(self, device, pg, channel: str = "zero"):
        self.buf = SymmetricBuffer(8, torch.int32, device, pg)
        self.channel = channel
        self.epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=pg)           # every rank's slots are zero before anybody publishes

    @classmethod
    def get(cls, device, pg, channel: str = "zero") -> "SignalSlots":
        """One set of slots per (group, channel).  A channel is a sequence of kernels that every rank runs in the same
        order on one stream (the call counter is only meaningful within such a sequence): the gradient reductions on
        the reduction stream are one channel, the all-to-all exchanges on the compute stream another."""
        key = (str(device), id(pg), channel)
        if key not in cls._by_group:
            cls._by_group[key] = SignalSlots(device, pg, channel)
        return cls._by_group[key]

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch


class StagingPair:
    """Two symmetric buffers of the wire dtype, used alternately by consecutive reductions."""

    def __init__(self, numel: int, dtype, device, pg):
        self.bufs = [SymmetricBuffer(numel, dtype, device, pg) for _ in range(2)]
        self.turn = 0
        self.signals = SignalSlots.get(device, pg)

    def next(self) -> SymmetricBuffer:
        b = self.bufs[self.turn]
        self.turn ^= 1
        return b


_STAGING: Dict[tuple, StagingPair] = {}


def staging_buffers(numel: int, dtype, device, pg) -> StagingPair:
    """The staging pair for units of ``numel`` elements over ``pg`` (one pair per size and group, shared by every unit
    of that size): a unit rounds its gradient into the pair's next buffer right before its reduce-scatter
    (``ShardedUnit._reduce_into`` explains why alternating needs no extra rendezvous)."""
    key = (numel, dtype, str(device), id(pg))
    pair = _STAGING.get(key)
    if pair is None:
        pair = _STAGING[key] = StagingPair(numel, dtype, device, pg)
    return pair


def round_into_staging(grad32: torch.Tensor, staging: SymmetricBuffer, me: int, shard_numel: int):
    """bf16 copy of every slice of the fp32 gradient buffer except this rank's own (which nobody reads remotely)."""
    from ..ops.optim import cast_bf16

    lo, hi = me * shard_numel, (me + 1) * shard_numel
    if lo > 0:
        cast_bf16(grad32[:lo], staging.tensor[:lo])
    if hi < grad32.numel():
        cast_bf16(grad32[hi:], staging.tensor[hi:])


def reduce_scatter_staged(staging: SymmetricBuffer, own32: torch.Tensor, me: int, shard_numel: int, out: torch.Tensor,
                          accumulate: bool = False, max_ctas: int = 0, signals: "SignalSlots" = None):
    """bf16 on the wire: ``out (+)= own32[slice] + sum_{r != me} staging_r[slice]`` (fp32 sum in rank order).

    With ``signals`` the kernel itself waits until every rank of the group has reached the same call (each rank
    publishes the call's epoch in its peers' signal slots after its rounding kernel, bounded wait); without, the caller
    must have ordered the ranks (``peer_barrier``)."""
    lib = _lib.load()
    sig_arr, epoch = (signals.buf.ptr_array(), signals.next_epoch()) if signals is not None else (None, 0)
    rc = lib.hg_zero_reduce_scatter_bf16wire(staging.ptr_array(), own32.data_ptr(), staging.t, me, shard_numel,
                                             out.data_ptr(), int(bool(accumulate)), int(max_ctas), sig_arr, epoch,
                                             _lib.stream())
    _lib.check(rc, "hg_zero_reduce_scatter_bf16wire")
    _lib.count_launch()
    return out


def add_inplace(out: torch.Tensor, x: torch.Tensor):
    lib = _lib.load()
    _lib.check(lib.hg_add_inplace_f32(out.data_ptr(), x.data_ptr(), out.numel(), _lib.stream()), "hg_add_inplace_f32")
    _lib.count_launch()
    return out


def adamw_allgather_peer(master, grad, exp_avg, exp_avg_sq, targets, dst_off: int, *, lr, beta1, beta2, eps,
                         weight_decay, step, gscale=None, skip=None):
    """``targets``: a ``SymmetricBuffer`` of bf16 parameters (stores go to every rank) or a local bf16 tensor."""
    lib = _lib.load()
    if isinstance(targets, SymmetricBuffer):
        arr, t_out = targets.ptr_array(), targets.t
    else:
        arr, t_out = (ctypes.c_void_p * 1)(targets.data_ptr()), 1
    rc = lib.hg_zero_adamw_allgather(master.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), arr,
                                     t_out, dst_off, master.numel(), float(lr), float(beta1), float(beta2), float(eps),
                                     float(weight_decay), int(step), _lib.ptr(gscale), _lib.ptr(skip), _lib.stream())
    _lib.check(rc, "hg_zero_adamw_allgather")
    _lib.count_launch()


def all_gather_peer(shards: SymmetricBuffer, shard_numel: int, out: torch.Tensor):
    """``out[r*S:(r+1)*S] = shard_r`` for every rank ``r``: this rank pulls all shards through their peer mappings
    (bf16, ``S`` a multiple of 8).  The shards must be quiescent (see ``ShardedUnit``: they change only inside the
    optimizer step, which ends with a rendezvous)."""
    lib = _lib.load()
    rc = lib.hg_peer_gather_bf16(shards.ptr_array(), shards.t, 1, shard_numel, 0, shard_numel, out.data_ptr(), shard_numel,
                                 shard_numel, _lib.stream())
    _lib.check(rc, "hg_peer_gather_bf16")
    _lib.count_launch()
    return out
