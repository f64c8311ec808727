"""Sharded-parameter manager: DDP / ZeRO-2 / ZeRO-3 per wrap unit, with its own flat buffers.

Each wrap unit (one decoder layer, the embedding, the final norm, the LM head, an expert block) gets

* ``flat``        the working-precision parameters in one buffer (the module's parameters are views);
* ``main_grad``   an fp32 gradient buffer of the same layout (``param.main_grad`` views): the weight-
                  gradient GEMM epilogue accumulates straight into it;
* ``master/exp_avg/exp_avg_sq``  fp32 optimizer state of the *local shard* (whole buffer for DDP);

and, per ZeRO type over the unit's ``sdp`` group (dp x sp x cp):

=========  =====================================  ==========================================
type       parameters                              gradients
=========  =====================================  ==========================================
ddp        replicated                              all-reduce
zero2      replicated, refreshed by all-gather     reduce-scatter -> shard
           after the sharded optimizer step
zero3      sharded; all-gathered before the        reduce-scatter -> shard
           unit's forward and again before its
           backward, storage released in between
=========  =====================================  ==========================================

With ``defer_sync`` (the reference's ``async_grad_reduce=True``) the reduction runs once per step: it is launched
from the unit's post-backward hook of the *last* micro-batch, on a side stream, so that it overlaps the backward
of the layers below (the reference does the same through FSDP's post-backward hook:
pipeline/sp_grad_reduce.py:48-132).  Otherwise it runs after every micro-batch's backward of the unit, also on the
side stream, and the unit's unsharded fp32 gradient buffer is *transient*: it comes from a small pool
(:class:`GradPool`) shared by all units of the same size and goes back once its reduce-scatter has run, so a rank
holds ``pool x layer`` unsharded gradients plus its own shards instead of a whole model's worth (FSDP's
``SHARD_GRAD_OP`` / ``FULL_SHARD`` memory behaviour, parallel.py:119-152).  Gradients are *summed* over the
sequence/context-parallel part of the group and *averaged* over the data-parallel replicas.

On the wire the gradients travel in the working precision (bf16) unless ``reduce_in_fp32`` is set, as in the
reference (parallel.py:128-131); they are accumulated over micro-batches and summed over ranks in fp32 either way.

This replaces torch FSDP as used by the reference (galvatron/core/runtime/parallel.py:100-210,
pipeline/grad_reduce.py:48-149, pipeline/sp_grad_reduce.py:48-132) so that the collectives can be fused
with our own kernels.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.checkpoint import checkpoint as _torch_checkpoint

from .. import ops
from . import mappings as mp

ALIGN = 64  # elements; keeps every parameter 128-byte aligned inside the flat buffers
POOL_BUFFERS = 3  # unsharded gradient buffers per (size, group) in the per-micro-batch reduction mode


class _ReduceState:
    """Process-wide state of the overlapped gradient reduction."""

    def __init__(self):
        self.last_microbatch = True       # set by the pipeline engine before each backward
        self.overlap = os.environ.get("HG_OVERLAP_REDUCE", "1") == "1"
        self.max_ctas = int(os.environ.get("HG_REDUCE_CTAS", "48"))   # grid cap of a reduction that runs beside GEMMs
        self._streams: Dict[int, "torch.cuda.Stream"] = {}
        self._gather_streams: Dict[int, "torch.cuda.Stream"] = {}
        self.used = False                 # something was queued on a side stream since the last join

    def stream(self, device):
        if device.type != "cuda" or not self.overlap:
            return None
        idx = device.index if device.index is not None else torch.cuda.current_device()
        st = self._streams.get(idx)
        if st is None:
            st = self._streams[idx] = torch.cuda.Stream(device=device)
        return st

    def gather_stream(self, device):
        """Side stream of the ZeRO-3 parameter prefetch (separate from the reduction stream, so that the parameters
        of the next unit never queue behind a gradient reduction)."""
        if device.type != "cuda" or os.environ.get("HG_PREFETCH_PARAMS", "1") != "1":
            return None
        idx = device.index if device.index is not None else torch.cuda.current_device()
        st = self._gather_streams.get(idx)
        if st is None:
            st = self._gather_streams[idx] = torch.cuda.Stream(device=device)
        return st

    def join(self, device):
        """The current stream waits for everything queued on the reduction stream."""
        if device.type == "cuda" and self.used:
            idx = device.index if device.index is not None else torch.cuda.current_device()
            st = self._streams.get(idx)
            if st is not None:
                torch.cuda.current_stream(device).wait_stream(st)
            self.used = False


REDUCE = _ReduceState()
_WIRE_SCRATCH: Dict[tuple, torch.Tensor] = {}


def set_last_microbatch(flag: bool):
    """Called by the schedule before a micro-batch's backward: deferred units reduce during the last one."""
    REDUCE.last_microbatch = bool(flag)


class GradPool:
    """Unsharded fp32 gradient buffers shared by the units of one size and sharding group.

    A unit takes the next buffer (round-robin) when its backward starts and hands it back when its reduce-scatter
    has been queued; ``free[k]`` is the event after which buffer ``k`` may be overwritten (on the fused fp32-wire
    path that is after a rendezvous of the group, because peers read the buffer)."""

    _pools: Dict[tuple, "GradPool"] = {}

    def __init__(self, numel: int, device, pg, symmetric: bool):
        self.bufs, self.sym = [], []
        for _ in range(POOL_BUFFERS):
            if symmetric:
                from . import fused_zero as fz

                sb = fz.SymmetricBuffer(numel, torch.float32, device, pg)
                self.sym.append(sb)
                self.bufs.append(sb.tensor)
            else:
                self.sym.append(None)
                self.bufs.append(torch.zeros(numel, dtype=torch.float32, device=device))
        self.free: List[Optional[object]] = [None] * POOL_BUFFERS
        self.next = 0

    @classmethod
    def get(cls, numel: int, device, pg, symmetric: bool) -> "GradPool":
        key = (numel, str(device), id(pg), symmetric)
        if key not in cls._pools:
            cls._pools[key] = GradPool(numel, device, pg, symmetric)
        return cls._pools[key]

    def acquire(self) -> int:
        k = self.next
        self.next = (k + 1) % len(self.bufs)
        ev = self.free[k]
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            self.free[k] = None
        return k


def _group_info(g):
    if g is None or g.size == 1 or g.group is None:
        return None, 1, 0
    return g.group, g.size, g.rank


class ShardedUnit:
    def __init__(self, module: nn.Module, name: str, sdp, dp_size: int, dp_type: str = "ddp",
                 reduce_in_fp32: bool = False, tp=None, defer_sync: bool = True, grad_sum_group=None,
                 fused_zero: bool = False):
        self.module, self.name = module, name
        self.pg, self.n, self.rank = _group_info(sdp)
        self.dp_size = max(1, dp_size)
        self.dp_type = dp_type if self.n > 1 else "ddp"
        self.reduce_in_fp32 = reduce_in_fp32
        self.tp_pg, self.tp_n, _ = _group_info(tp)
        self.defer_sync = defer_sync
        params = []
        for p in module.parameters():
            if getattr(p, "_hg_unit", None) is None:
                p._hg_unit = self
                params.append(p)
        # tensor-parallel-replicated parameters (norm weights, replicated biases, router) first
        params.sort(key=lambda p: 0 if getattr(p, "tp_replicated", False) else 1)
        self.params: List[nn.Parameter] = params
        self.offsets: List[int] = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        self.replicated_numel = 0
        for p, o in zip(params, self.offsets):
            if getattr(p, "tp_replicated", False):
                self.replicated_numel = o + p.numel()
        mult = ALIGN * self.n
        self.numel = max(mult, (off + mult - 1) // mult * mult)
        self.shard_numel = self.numel // self.n
        self.device = params[0].device if params else torch.device("cpu")
        self.dtype = params[0].dtype if params else torch.float32
        # dtype in which gradients cross the links; accumulation and the sum over ranks are fp32 regardless
        self.wire_dtype = torch.float32 if (reduce_in_fp32 or self.dtype == torch.float32) else self.dtype
        self.flat: Optional[torch.Tensor] = None
        self.main_grad: Optional[torch.Tensor] = None
        self.gathered = True
        self.step_count = 0
        self._reduced = False
        self._bwd_pending = False
        self._acc_used = False
        self._gather_event = None
        self.count_in_norm = True  # False for the second copy of a weight tied across pipeline stages
        # a weight tied across pipeline stages is summed over the two stages before the sharding group reduces it:
        # its unit keeps the whole-step gradient and reduces at the optimizer step
        self.reduce_at_step_only = False
        # own reduce-scatter / AdamW+all-gather kernels over peer memory instead of NCCL (parallel/fused_zero.py)
        self.fused = False
        if fused_zero and params and self.dp_type in ("zero2", "zero3") and self.dtype in (torch.bfloat16, torch.float16):
            from . import fused_zero as fz

            self.fused = fz.available(self.device, self.n, self.pg)
        # per-micro-batch reduction of a sharded unit: the unsharded gradient buffer is borrowed from a pool
        self.pooled = bool(params) and not defer_sync and self.dp_type in ("zero2", "zero3")
        if params:
            self._materialise()

    # ---- construction ----------------------------------------------------------------------------
    def _materialise(self):
        dev = self.device
        self._sym_grad = self._sym_flat = None
        self._pool: Optional[GradPool] = None
        self._pool_slot = -1
        self._staging = None            # bf16 wire: buffer pair the gradient is rounded into before it is reduced
        peers_read_fp32 = self.fused and self.wire_dtype == torch.float32
        if self.fused:
            from . import fused_zero as fz

            if self.dp_type == "zero2":
                self._sym_flat = fz.SymmetricBuffer(self.numel, self.dtype, dev, self.pg)   # peers write parameters
            if self.wire_dtype != torch.float32:
                self._staging = fz.staging_buffers(self.numel, self.wire_dtype, dev, self.pg)
        self.flat = self._sym_flat.tensor if self._sym_flat is not None else torch.zeros(self.numel, dtype=self.dtype, device=dev)
        for p, o in zip(self.params, self.offsets):
            self.flat[o:o + p.numel()].copy_(p.data.reshape(-1))
        self._bind_params()
        if self.pooled:
            self._pool = GradPool.get(self.numel, dev, self.pg, peers_read_fp32)
            self._bind_grads(self._pool.bufs[0])       # placeholder views until the first backward borrows a buffer
            self.main_grad = None
        else:
            if peers_read_fp32:
                from . import fused_zero as fz

                self._sym_grad = fz.SymmetricBuffer(self.numel, torch.float32, dev, self.pg)   # peers read gradients
                self.main_grad = self._sym_grad.tensor
            else:
                self.main_grad = torch.zeros(self.numel, dtype=torch.float32, device=dev)
            self._bind_grads(self.main_grad)
        lo, hi = self.shard_range()
        self.master = self.flat[lo:hi].float().clone()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        # this rank's reduced gradient of the step (fp32): the whole buffer for ddp, the shard otherwise
        self.grad_shard = None
        self._red_buf = None if self.dp_type == "ddp" and self.defer_sync else \
            torch.zeros(hi - lo, dtype=torch.float32, device=dev)
        self._sym_shard = None
        if self.dp_type == "zero3":
            if self.fused:
                # the bf16 shard is what peers pull from when they re-assemble the unit's parameters: it changes only
                # in the optimizer step, which ends with a rendezvous, so gathers need no synchronisation of their own
                from . import fused_zero as fz

                self._sym_shard = fz.SymmetricBuffer(self.shard_numel, self.dtype, dev, self.pg)
                self.shard_lp = self._sym_shard.tensor
                self.shard_lp.copy_(self.flat[lo:hi])
                self.sync_peers()
            else:
                self.shard_lp = self.flat[lo:hi].clone()
            self.release()
        else:
            self.shard_lp = self.flat[lo:hi]

    def _bind_params(self):
        for p, o in zip(self.params, self.offsets):
            p.data = self.flat[o:o + p.numel()].view(p.shape)

    def _bind_grads(self, buf: torch.Tensor):
        for p, o in zip(self.params, self.offsets):
            p.main_grad = buf[o:o + p.numel()].view(p.shape)
            p.mg_fresh = True

    def shard_range(self):
        if self.dp_type == "ddp":
            return 0, self.numel
        return self.rank * self.shard_numel, (self.rank + 1) * self.shard_numel

    def reload_master(self):
        """Re-derive master weights / bf16 shard from ``flat`` (after a checkpoint load into the params)."""
        if not self.gathered:
            raise RuntimeError("gather the unit before reloading")
        lo, hi = self.shard_range()
        self.master.copy_(self.flat[lo:hi])
        if self.dp_type == "zero3":
            self.shard_lp.copy_(self.flat[lo:hi])
            if self._sym_shard is not None:
                self.sync_peers()        # peers pull from this shard

    # ---- ZeRO-3 gather / release --------------------------------------------------------------------
    def gather(self, prefetch: bool = False):
        """Re-assemble the unit's parameters from the shards of its group.  ``prefetch=True`` queues the gather on a
        side stream (ordered after what the current stream holds so far) and returns at once; the plain call that
        follows before the unit runs only makes the current stream wait for it."""
        if self.dp_type != "zero3":
            return
        if self.gathered:
            if not prefetch and self._gather_event is not None:
                torch.cuda.current_stream(self.device).wait_event(self._gather_event)
                self._gather_event = None
            return
        nbytes = self.numel * self.flat.element_size()
        st = self.flat.untyped_storage()
        if st.size() != nbytes:
            st.resize_(nbytes)          # allocated (and later released) on the current stream in both modes
        side = REDUCE.gather_stream(self.device) if prefetch else None
        if side is not None:
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                self._gather_now()
                self._gather_event = torch.cuda.Event()
                self._gather_event.record(side)
        else:
            self._gather_now()
        self.gathered = True

    def _gather_now(self):
        if self.flat.device.type == "cpu":
            parts = [torch.empty_like(self.shard_lp) for _ in range(self.n)]
            dist.all_gather(parts, self.shard_lp, group=self.pg)
            self.flat.copy_(torch.cat(parts))
        elif self._sym_shard is not None:
            from . import fused_zero as fz

            fz.all_gather_peer(self._sym_shard, self.shard_numel, self.flat)   # pull every rank's shard over NVLink
        else:
            dist.all_gather_into_tensor(self.flat, self.shard_lp, group=self.pg)

    def release(self):
        if self.dp_type != "zero3" or not self.gathered:
            return
        if self._gather_event is not None:      # prefetched but never used: the copy must land before the storage goes
            torch.cuda.current_stream(self.device).wait_event(self._gather_event)
            self._gather_event = None
        # views held by autograd's saved tensors stay attached to the storage object; it is re-filled by
        # the next gather() before anything reads it
        self.flat.untyped_storage().resize_(0)
        self.gathered = False

    # ---- gradients --------------------------------------------------------------------------------------
    def zero_grad(self):
        for p in self.params:
            p.mg_fresh = True
            p.grad = None
        self._reduced = False
        self._acc_used = False

    def begin_backward(self):
        """Before the unit's backward of a micro-batch: a pooled unit borrows its gradient buffer."""
        if self.pooled and self.main_grad is None:
            self._pool_slot = self._pool.acquire()
            self.main_grad = self._pool.bufs[self._pool_slot]
            self._bind_grads(self.main_grad)

    def _finish_accumulation(self):
        """Fold stray ``.grad`` tensors (bias / generic autograd paths) into ``main_grad``."""
        for p in self.params:
            if p.grad is not None:
                if getattr(p, "mg_fresh", False):
                    p.main_grad.copy_(p.grad)
                    p.mg_fresh = False
                else:
                    p.main_grad.add_(p.grad)
                p.grad = None

    def prepare_grads(self):
        """Make ``main_grad`` complete for the micro-batches seen so far: fold autograd ``.grad`` tensors in
        and zero the parameters that received nothing."""
        self.begin_backward()
        self._finish_accumulation()
        for p in self.params:
            if getattr(p, "mg_fresh", False):  # received nothing since the last reset
                p.main_grad.zero_()
                p.mg_fresh = False

    def sync_peers(self):
        """Stream-ordered rendezvous of the sharding group (fused path only)."""
        if self.fused:
            from . import fused_zero as fz

            fz.peer_barrier(self.pg, self.device)

    def _wire_scratch(self, numel: int) -> torch.Tensor:
        """A reusable buffer of the wire dtype (NCCL / gloo path; all its uses are ordered on one stream)."""
        key = (numel, self.wire_dtype, str(self.device))
        buf = _WIRE_SCRATCH.get(key)
        if buf is None:
            buf = _WIRE_SCRATCH[key] = torch.empty(numel, dtype=self.wire_dtype, device=self.device)
        return buf

    def _reduce_into(self, out: torch.Tensor, accumulate: bool, presynced: bool = False, capped: bool = False):
        """``out (+)= sum over the sharding group of main_grad`` (this rank's slice for zero2 / zero3).  Runs on the
        current stream; ``main_grad`` must be complete (``prepare_grads``)."""
        mg = self.main_grad
        if self.tp_n > 1 and self.replicated_numel > 0:
            # norm weights / replicated biases saw only this rank's S/t tokens: sum over the tp group
            dist.all_reduce(mg[: self.replicated_numel], group=self.tp_pg)
        if self.n == 1:
            if out is not mg:
                out.add_(mg) if accumulate else out.copy_(mg)
            return
        lowp = self.wire_dtype != torch.float32
        max_ctas = REDUCE.max_ctas if capped else 0
        if self.dp_type == "ddp":
            if lowp:
                w = self._wire_scratch(self.numel)
                w.copy_(mg)
                dist.all_reduce(w, group=self.pg)
                red = w
            else:
                dist.all_reduce(mg, group=self.pg)
                red = mg
            if out is not red:
                out.add_(red) if accumulate else out.copy_(red)
            return
        lo, hi = self.shard_range()
        if self.fused:
            from . import fused_zero as fz

            if lowp:
                st = self._staging.next()
                fz.round_into_staging(mg, st, self.rank, self.shard_numel)
                # the kernel waits for every rank's staged gradients itself (signal slots, bounded wait)
                fz.reduce_scatter_staged(st, mg, self.rank, self.shard_numel, out, accumulate, max_ctas,
                                         signals=self._staging.signals)
                # no rendezvous afterwards: the staging buffers alternate, and a rank rounds into a buffer again only
                # after the rendezvous of the unit in between, which every peer enters after its reads of this one
            else:
                if not presynced:
                    self.sync_peers()    # every rank's gradients are complete
                src = self._sym_grad if self._pool is None else self._pool.sym[self._pool_slot]
                if accumulate:
                    tmp = self._wire_scratch(self.shard_numel)
                    fz.reduce_scatter_peer(src, self.rank, self.shard_numel, tmp, max_ctas)
                    fz.add_inplace(out, tmp)
                else:
                    fz.reduce_scatter_peer(src, self.rank, self.shard_numel, out, max_ctas)
                if not self.defer_sync:
                    self.sync_peers()    # peers have finished reading before the buffer is written again
            return
        if mg.device.type == "cpu":
            tmp = mg.to(self.wire_dtype) if lowp else mg.clone()
            dist.all_reduce(tmp, group=self.pg)
            red = tmp[lo:hi]
        else:
            src = mg
            if lowp:
                src = self._wire_scratch(self.numel)
                src.copy_(mg)
            red = self._wire_scratch(self.shard_numel) if (accumulate or lowp) else out
            dist.reduce_scatter_tensor(red, src, group=self.pg)
        if red is not out:
            out.add_(red) if accumulate else out.copy_(red)

    def _target(self) -> torch.Tensor:
        return self.main_grad if self._red_buf is None else self._red_buf

    def _launch_reduce(self, accumulate: bool, presynced: bool = False, overlap: bool = True):
        """Queue the reduction of the current ``main_grad``: on the side stream (ordered after everything queued so
        far on the current one) when overlap is on, else in place.  A pooled unit hands its buffer back."""
        self.prepare_grads()          # on the current stream: autograd's tensors live there
        has_comm = self.n > 1 or (self.tp_n > 1 and self.replicated_numel > 0)
        side = REDUCE.stream(self.device) if (overlap and has_comm) else None
        out = self._target()
        if side is None:
            self._reduce_into(out, accumulate, presynced)
            if self.pooled:
                self.main_grad = None
            return
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self._reduce_into(out, accumulate, presynced, capped=True)
            if self.pooled:
                ev = torch.cuda.Event()
                ev.record(side)
                self._pool.free[self._pool_slot] = ev
                self.main_grad = None
        REDUCE.used = True

    def on_backward_done(self):
        """Post-backward hook of one micro-batch of this unit."""
        if self._reduced or self.reduce_at_step_only:
            return
        if not self.defer_sync:
            self._launch_reduce(accumulate=self._acc_used)
            self._acc_used = True
        elif REDUCE.last_microbatch and REDUCE.overlap and self.device.type == "cuda":
            self._launch_reduce(accumulate=False)
            self.grad_shard = self._target()
            self._reduced = True

    def reduce_grads(self, final: bool = True, presynced: bool = False):
        """Whatever of the step's gradient synchronisation has not been launched from the backward hooks."""
        if self._reduced or not final:
            return
        if self.defer_sync or not self._acc_used:
            self._launch_reduce(accumulate=False, presynced=presynced, overlap=False)
        self.grad_shard = self._target()
        self._reduced = True

    def grad_sumsq(self, out: torch.Tensor):
        """Add this rank's share of the squared gradient norm to ``out[0]`` so that a SUM over all ranks
        counts every parameter element exactly once."""
        if not self.count_in_norm:
            return
        g = self.grad_shard
        inv = 1.0 / (self.dp_size * self.dp_size)  # gradients are still dp-sums here
        rep = self.n if self.dp_type == "ddp" else 1  # identical copies held by the sdp group
        ops.sumsq(g, out, accumulate=True, scale=inv / rep)
        if self.tp_n > 1 and self.replicated_numel > 0:
            lo, hi = self.shard_range()
            a, b = max(lo, 0), min(hi, self.replicated_numel)
            if b > a:
                ops.sumsq(g[a - lo:b - lo], out, accumulate=True, scale=inv / rep * (1.0 / self.tp_n - 1.0))

    # ---- optimizer --------------------------------------------------------------------------------------
    def optimizer_step(self, lr, beta1, beta2, eps, weight_decay, clip_coef: Optional[torch.Tensor] = None):
        if not self.params:
            return
        self.step_count += 1
        g = self.grad_shard
        # fold the 1/dp average into the device-side gradient scale
        self._ensure_scale(clip_coef)
        if self.fused:
            from . import fused_zero as fz

            # ZeRO-2: the updated bf16 values go straight into every rank's parameter buffer (no all-gather);
            # ZeRO-3: into the local bf16 shard.  The caller rendezvouses the group afterwards (sync_peers).
            target = self._sym_flat if self.dp_type == "zero2" else self.shard_lp
            off = self.rank * self.shard_numel if self.dp_type == "zero2" else 0
            fz.adamw_allgather_peer(self.master, g, self.exp_avg, self.exp_avg_sq, target, off, lr=lr, beta1=beta1,
                                    beta2=beta2, eps=eps, weight_decay=weight_decay, step=self.step_count,
                                    gscale=self._scale)
            return
        lp = self.shard_lp if self.dtype != torch.float32 else None
        ops.adamw_step(self.master, g, self.exp_avg, self.exp_avg_sq, lp, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                       weight_decay=weight_decay, step=self.step_count, gscale=self._scale)
        if self.dtype == torch.float32:
            self.shard_lp.copy_(self.master)
        if self.dp_type == "zero2":
            if self.flat.device.type == "cpu":
                parts = [torch.empty_like(self.shard_lp) for _ in range(self.n)]
                dist.all_gather(parts, self.shard_lp.contiguous(), group=self.pg)
                self.flat.copy_(torch.cat(parts))
            else:
                dist.all_gather_into_tensor(self.flat, self.shard_lp, group=self.pg)

    def _ensure_scale(self, clip_coef):
        if not hasattr(self, "_scale"):
            self._scale = torch.ones(1, dtype=torch.float32, device=self.device)
        if clip_coef is None:
            self._scale.fill_(1.0 / self.dp_size)
        else:
            torch.mul(clip_coef, 1.0 / self.dp_size, out=self._scale)

    # ---- state dict -------------------------------------------------------------------------------------
    def optimizer_state(self) -> Dict[str, torch.Tensor]:
        return {"master": self.master, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq,
                "step": torch.tensor(self.step_count)}

    def load_optimizer_state(self, sd):
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.step_count = int(sd["step"])

    def full_state_dict(self) -> Dict[str, torch.Tensor]:
        """Unsharded parameters of the unit keyed by their module-relative names (collective for zero3)."""
        was = self.gathered
        self.gather()
        out = {k: v.detach().clone().cpu() for k, v in self.module.state_dict().items()}
        if not was:
            self.release()
        return out


class _Boundary(torch.autograd.Function):
    """Identity in the forward; runs a callback when the gradient passes in the backward."""

    @staticmethod
    def forward(ctx, x, cb):
        ctx.cb = cb
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.cb()
        return g, None


class UnitWrapper(nn.Module):
    """Runs a unit's module between the ZeRO hooks (gather before forward / backward, release after,
    gradient reduction after the backward) and optional activation recomputation."""

    def __init__(self, inner: nn.Module, unit: ShardedUnit, checkpoint: bool = False):
        super().__init__()
        self.inner, self.unit, self.checkpoint = inner, unit, checkpoint
        self.extra_units: List[ShardedUnit] = []  # units owning parameters this module borrows (tied weights)
        # ZeRO-3: the unit that runs after this one in the forward / in the backward; its parameters are gathered
        # on a side stream while this unit computes (set by link_prefetch)
        self.next_unit: Optional[ShardedUnit] = None
        self.prev_unit: Optional[ShardedUnit] = None

    def _pre_backward(self):
        self.unit.gather()
        for e in self.extra_units:
            e.gather()
        if self.prev_unit is not None and not self.unit._bwd_pending:
            self.prev_unit.gather(prefetch=True)
        if not self.unit._bwd_pending:
            self.unit.begin_backward()
        self.unit._bwd_pending = True

    def _post_backward(self):
        u = self.unit
        if not u._bwd_pending:
            return
        u._bwd_pending = False
        u.release()
        for e in self.extra_units:
            e.release()
        u.on_backward_done()

    def finish_backward(self):
        """Called by the engine after the whole backward: covers units whose inputs carry no gradient."""
        self._post_backward()

    def forward(self, *args, **kwargs):
        u = self.unit
        u.gather()
        for e in self.extra_units:
            e.gather()
        if self.next_unit is not None:
            self.next_unit.gather(prefetch=True)
        grad_mode = torch.is_grad_enabled()
        if grad_mode:
            # the unit's backward is over once the gradient has left through *every* differentiable input
            pending = [sum(1 for a in args if torch.is_tensor(a) and a.requires_grad)]

            def _one_input_done():
                pending[0] -= 1
                if pending[0] <= 0:
                    self._post_backward()

            args = tuple(_Boundary.apply(a, _one_input_done) if torch.is_tensor(a) and a.requires_grad else a
                         for a in args)
        if self.checkpoint and grad_mode:
            out = _torch_checkpoint(self.inner, *args, use_reentrant=False, **kwargs)
        else:
            out = self.inner(*args, **kwargs)
        u.release()
        for e in self.extra_units:
            e.release()
        if grad_mode:
            if torch.is_tensor(out) and out.requires_grad:
                out = _Boundary.apply(out, self._pre_backward)
            elif isinstance(out, tuple):
                out = tuple(_Boundary.apply(o, self._pre_backward) if torch.is_tensor(o) and o.requires_grad else o
                            for o in out)
        return out


def link_prefetch(wrappers: List[UnitWrapper]):
    """Chain the wrappers of a stage in execution order so that each ZeRO-3 unit is gathered one unit ahead."""
    for a, b in zip(wrappers, wrappers[1:]):
        if b.unit.dp_type == "zero3" and b.unit is not a.unit:
            a.next_unit = b.unit
        if a.unit.dp_type == "zero3" and b.unit is not a.unit:
            b.prev_unit = a.unit
