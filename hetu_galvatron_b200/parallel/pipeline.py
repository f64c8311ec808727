"""Pipeline-parallel schedules (no-PP gradient accumulation, GPipe, 1F1B-flush) over NCCL / gloo p2p.

A stage runs ``StageModel`` on micro-batches; activations cross a stage boundary in the *sender's*
layout ``[S/g, mb/d, H]`` between ranks with the same index inside their stage, and the receiver
re-lays them out for its first layer.

Communication.  A schedule is a list of steps ``("F", i)`` / ``("B", i)``.  Activations travel on one
communicator, gradients on a second one over the same ranks, so each is a one-way FIFO between neighbours:
a stage can post the receive of step ``k+1`` *before* it computes step ``k`` (the transfer then runs under
the compute) and send its result with a plain ``isend`` right after the compute, and no ordering of those
calls can make two neighbours wait on each other.  (With one communicator for both directions the
steady state of 1F1B, where both neighbours send first, needs the send and the receive fused into one
``batch_isend_irecv`` group, as the reference does in pipeline.py:1108-1139, and that rules out the early
receive.)  Sends are only waited for when their buffer is dropped at the end of the step; nothing calls
a device-wide synchronise.

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
    """Point-to-point activations (forward channel) and gradients (backward channel) between neighbouring stages."""

    def __init__(self, pp_group, stage: int, num_stages: int, bwd_group=None):
        self.stage, self.n = stage, num_stages
        ranks = pp_group.ranks
        self.prev = ranks[stage - 1] if stage > 0 else None
        self.next = ranks[stage + 1] if stage < num_stages - 1 else None
        self.fwd = pp_group.group
        self.bwd = bwd_group.group if bwd_group is not None else pp_group.group
        self._pending: List = []

    def recv_activation(self, shape, dtype, device):
        buf = torch.empty(shape, dtype=dtype, device=device)
        return buf, dist.irecv(buf, src=self.prev, group=self.fwd)

    def recv_gradient(self, shape, dtype, device):
        buf = torch.empty(shape, dtype=dtype, device=device)
        return buf, dist.irecv(buf, src=self.next, group=self.bwd)

    def send_activation(self, t: torch.Tensor):
        t = t.contiguous()
        self._pending.append((dist.isend(t, dst=self.next, group=self.fwd), t))  # keeps the buffer alive

    def send_gradient(self, t: torch.Tensor):
        t = t.contiguous()
        self._pending.append((dist.isend(t, dst=self.prev, group=self.bwd), t))

    def drain(self):
        for work, _ in self._pending:
            work.wait()
        self._pending.clear()


class PipelineEngine:
    """Runs one training step of a stage under the chosen schedule."""

    def __init__(self, stage_model, groups, plan, spec, device):
        self.model, self.groups, self.plan, self.spec, self.device = stage_model, groups, plan, spec, device
        self.stage, self.n = groups.stage, plan.pp_deg
        self.p2p = P2P(groups.pp, self.stage, self.n, getattr(groups, "pp_bwd", None)) if self.n > 1 else None
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
            steps = [("F", i) for i in range(chunks)] + ([] if forward_only else [("B", i) for i in range(chunks)])
        else:
            steps = one_f_one_b_steps(self.stage, self.n, chunks)
        return self._run_steps(steps, tokens, labels, loss_fns, mb_sizes, scale, forward_only)

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

    # ---- pipelined schedules ------------------------------------------------------------------------------
    def _post_recv(self, step, mb_sizes):
        """Post the receive a step needs (``None`` when its input is local)."""
        kind, i = step
        if kind == "F":
            if self.first:
                return None
            return self.p2p.recv_activation(self._recv_shape(mb_sizes[i]), self.spec.dtype, self.device)
        if self.last:
            return None
        return self.p2p.recv_gradient(self._send_shape(mb_sizes[i]), self.spec.dtype, self.device)

    def _run_steps(self, steps, tokens, labels, loss_fns, mb_sizes, scale, forward_only):
        chunks = len(mb_sizes)
        inputs, outputs, losses = {}, {}, []
        n_bwd = sum(1 for k, _ in steps if k == "B")
        done_bwd = 0
        first_fwd_hook = self.after_forward
        nxt = self._post_recv(steps[0], mb_sizes) if steps else None
        for k, (kind, i) in enumerate(steps):
            cur = nxt
            # the next step's input starts travelling while this step computes
            nxt = self._post_recv(steps[k + 1], mb_sizes) if k + 1 < len(steps) else None
            if kind == "F":
                if cur is None:
                    x = tokens[i]
                else:
                    x, work = cur
                    work.wait()
                    x.requires_grad_(not forward_only)
                with torch.set_grad_enabled(not forward_only):
                    out = self._forward(x, labels[i], loss_fns[i], scale)
                if not self.last:
                    self.p2p.send_activation(out.detach())
                else:
                    losses.append(out.detach())
                inputs[i], outputs[i] = x, out
                last_fwd = k + 1 == len(steps) or all(kk != "F" for kk, _ in steps[k + 1:])
                if first_fwd_hook is not None and (last_fwd if self.plan.pipeline_type == "gpipe" else i == 0):
                    first_fwd_hook()
                    first_fwd_hook = None
            else:
                x, out = inputs.pop(i), outputs.pop(i)
                done_bwd += 1
                set_last_microbatch(done_bwd == n_bwd)
                if cur is None:
                    out.backward()
                else:
                    g, work = cur
                    work.wait()
                    torch.autograd.backward(out, grad_tensors=g)
                self._finish_backward()
                if not self.first:
                    self.p2p.send_gradient(x.grad)
        self.p2p.drain()
        return losses


def one_f_one_b_steps(stage: int, num_stages: int, chunks: int):
    """1F1B with flush for one stage: ``num_stages - stage - 1`` warm-up forwards, then forward / backward pairs,
    then the remaining backwards."""
    warm = min(num_stages - stage - 1, chunks)
    steps = [("F", i) for i in range(warm)]
    for i in range(warm, chunks):
        steps += [("F", i), ("B", i - warm)]
    steps += [("B", i) for i in range(chunks - warm, chunks)]
    return steps
