"""Pipeline-parallel schedules (no-PP gradient accumulation, GPipe, 1F1B-flush) over NCCL / gloo p2p.

A stage runs ``StageModel`` on micro-batches; activations cross a stage boundary in the *sender's*
layout ``[S/g, mb/d, H]`` between ranks with the same index inside their stage, and the receiver
re-lays them out for its first layer.  Sends are asynchronous (``isend``) and are only waited for when
their buffer is about to be reused, receives are posted before the compute they feed; nothing calls a
device-wide synchronise.

Capability parity: galvatron/core/runtime/pipeline/pipeline.py:307-385 (no pipeline), :387-713
(1F1B-flush: warm-up / steady / cool-down), :730-895 (GPipe), :907-981 (forward / backward step),
:1092-1269 (p2p), :276-305 (uneven last micro-batch), pipeline/utils.py:12-64 (chunking).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

from .zero import set_last_microbatch


def chunk_batch(t: Optional[torch.Tensor], chunks: int) -> List[Optional[torch.Tensor]]:
    """Split along the batch dimension into at most ``chunks`` micro-batches (the last may be smaller)."""
    if t is None:
        return [None] * chunks
    parts = list(t.chunk(chunks, dim=0))
    return parts


class P2P:
    """Point-to-point activations / gradients between neighbouring stages."""

    def __init__(self, pp_group, stage: int, num_stages: int):
        self.stage, self.n = stage, num_stages
        ranks = pp_group.ranks
        self.prev = ranks[stage - 1] if stage > 0 else None
        self.next = ranks[stage + 1] if stage < num_stages - 1 else None
        self._pending: List = []

    def recv(self, shape, dtype, device, src) -> (torch.Tensor, object):
        buf = torch.empty(shape, dtype=dtype, device=device)
        return buf, dist.irecv(buf, src=src)

    def send(self, t: torch.Tensor, dst):
        t = t.contiguous()
        work = dist.isend(t, dst=dst)
        self._pending.append((work, t))  # keep the buffer alive until the send completed

    def drain(self):
        for work, _ in self._pending:
            work.wait()
        self._pending.clear()


class PipelineEngine:
    """Runs one training step of a stage under the chosen schedule."""

    def __init__(self, stage_model, groups, plan, spec, device):
        self.model, self.groups, self.plan, self.spec, self.device = stage_model, groups, plan, spec, device
        self.stage, self.n = groups.stage, plan.pp_deg
        self.p2p = P2P(groups.pp, self.stage, self.n) if self.n > 1 else None
        self.first, self.last = self.stage == 0, self.stage == self.n - 1
        self.after_forward = None  # optional hook (memory profiling): after the first forward / after all GPipe forwards

    # ---- shapes ---------------------------------------------------------------------------------------
    def _boundary_shape(self, lp, mb_global: int):
        """Activation shape after layer ``lp`` for a micro-batch of ``mb_global`` samples over the stage."""
        g = max(lp.tp, lp.sp) * lp.cp
        d = self.plan.dp_size(lp)
        return (self.spec.seq_len // g, max(1, mb_global // d), self.spec.hidden)

    def _recv_shape(self, mb_global):
        first_lp = self.model.plans[0]
        prev_lp = self.plan.layers[first_lp.index - 1]
        return self._boundary_shape(prev_lp, mb_global)

    def _send_shape(self, mb_global):
        return self._boundary_shape(self.model.plans[-1], mb_global)

    # ---- one micro-batch ----------------------------------------------------------------------------------
    def _forward(self, x, labels, loss_fn, scale):
        out = self.model(x, labels)
        if self.last:
            loss = loss_fn(out) * scale
            return loss
        return out

    def run(self, tokens: List, labels: List, loss_fns: List[Callable], mb_sizes: Sequence[int],
            forward_only: bool = False):
        """``tokens[i]`` / ``labels[i]``: micro-batch i of this rank (``None`` where the stage does not need
        them); ``mb_sizes[i]``: its *global-per-stage* sample count.  Returns the list of micro-batch losses
        (last stage) or an empty list."""
        chunks = len(mb_sizes)
        scale = 1.0 / chunks
        if self.n == 1:
            return self._run_no_pp(tokens, labels, loss_fns, scale, forward_only)
        if self.plan.pipeline_type == "gpipe" or forward_only:
            return self._run_gpipe(tokens, labels, loss_fns, mb_sizes, scale, forward_only)
        return self._run_1f1b(tokens, labels, loss_fns, mb_sizes, scale)

    def _finish_backward(self):
        for u in self.model.units:
            for w in getattr(u, "wrappers", [u]):
                w.finish_backward()

    def _run_no_pp(self, tokens, labels, loss_fns, scale, forward_only):
        losses = []
        for i in range(len(tokens)):
            with torch.set_grad_enabled(not forward_only):
                loss = self._forward(tokens[i], labels[i], loss_fns[i], scale)
            if i == 0 and self.after_forward is not None:
                self.after_forward()
            if not forward_only:
                set_last_microbatch(i == len(tokens) - 1)   # deferred units launch their reduction in this backward
                loss.backward()
                self._finish_backward()
            losses.append(loss.detach())
        return losses

    # ---- GPipe ---------------------------------------------------------------------------------------------
    def _run_gpipe(self, tokens, labels, loss_fns, mb_sizes, scale, forward_only):
        chunks = len(mb_sizes)
        dtype = self.spec.dtype
        inputs, outputs, losses = [], [], []
        for i in range(chunks):
            if self.first:
                x = tokens[i]
            else:
                x, w = self.p2p.recv(self._recv_shape(mb_sizes[i]), dtype, self.device, self.p2p.prev)
                w.wait()
                x.requires_grad_(not forward_only)
            with torch.set_grad_enabled(not forward_only):
                out = self._forward(x, labels[i], loss_fns[i], scale)
            if not self.last:
                self.p2p.send(out.detach(), self.p2p.next)
            else:
                losses.append(out.detach())
            inputs.append(x)
            outputs.append(out)
        if self.after_forward is not None:
            self.after_forward()
        if forward_only:
            self.p2p.drain()
            return losses
        for i in range(chunks):
            set_last_microbatch(i == chunks - 1)
            self._backward_step(inputs[i], outputs[i], mb_sizes[i])
            inputs[i] = outputs[i] = None
        self.p2p.drain()
        return losses

    def _backward_step(self, x, out, mb):
        if self.last:
            out.backward()
        else:
            g, w = self.p2p.recv(tuple(out.shape), out.dtype, self.device, self.p2p.next)
            w.wait()
            torch.autograd.backward(out, grad_tensors=g)
        self._finish_backward()
        if not self.first:
            self.p2p.send(x.grad, self.p2p.prev)

    # ---- 1F1B with flush ---------------------------------------------------------------------------------
    def _run_1f1b(self, tokens, labels, loss_fns, mb_sizes, scale):
        chunks = len(mb_sizes)
        dtype = self.spec.dtype
        warm = min(self.n - self.stage - 1, chunks)
        inputs, outputs, losses = [], [], []

        def fwd(i):
            if self.first:
                x = tokens[i]
            else:
                x, w = self.p2p.recv(self._recv_shape(mb_sizes[i]), dtype, self.device, self.p2p.prev)
                w.wait()
                x.requires_grad_(True)
            out = self._forward(x, labels[i], loss_fns[i], scale)
            if not self.last:
                self.p2p.send(out.detach(), self.p2p.next)
            else:
                losses.append(out.detach())
            inputs.append(x)
            outputs.append(out)

        done = [0]

        def bwd():
            x, out = inputs.pop(0), outputs.pop(0)
            done[0] += 1
            set_last_microbatch(done[0] == chunks)
            self._backward_step(x, out, None)

        for i in range(warm):
            fwd(i)
        for i in range(warm, chunks):
            fwd(i)
            bwd()
        for _ in range(warm):
            bwd()
        self.p2p.drain()
        return losses
