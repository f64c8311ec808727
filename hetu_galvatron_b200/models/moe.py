"""Mixture-of-experts decoder layer: attention block, top-k router, token dispatch, expert MLPs.

Units / parameter names (checkpoint contract, reference models/moe_modules.py:19-155):

    GalvatronMoEAttention   attn.* (as the dense attention block) + pre_router_norm.weight
    GalvatronMoERouter      router.weight [E, H] fp32 (+ router.expert_bias)
    GalvatronMoEMLP         experts.linear_fc1.weight [E_loc, 2F/etp, H], experts.linear_fc2.weight [E_loc, H, F/etp]
                            (exported per expert as experts.local_experts.{j}.linear_fc{1,2}.weight)

Routing (reference moe/router.py:98-438, moe/moe_utils.py:430-544): fp32 gate, softmax-then-top-k or
top-k-then-softmax, sigmoid scores with optional selection bias, group-limited top-k, capacity dropping
(``probs`` / ``position`` policy), switch-style auxiliary load-balancing loss, z-loss.

Dispatch: tokens are sorted by expert (expert-major, token-minor -- moe_utils.py:219-353), exchanged with
an all-to-all-v over the expert-parallel group (``alltoall``) or all-gathered (``allgather``), re-sorted
``[source][local expert] -> [local expert][source]`` into 128-row-aligned, zero-padded segments, run
through the grouped tcgen05 GEMM (fc1 -> SwiGLU -> fc2), and returned by the mirror path where the
routing weights are applied in fp32 (token_dispatcher.py:116-284, :287-740; moe/mlp.py:26-211).
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..ops.gemm import OUT_F32, OUT_F32_ACC
from ..parallel import mappings as mp
from ..parallel.zero import ShardedUnit, UnitWrapper
from .modules import GalvatronAttention, Norm, _param, init_normal_sharded_, ops_add
from .spec import LayerCtx, ModelSpec

SEG_ALIGN = 128  # rows; expert segments start on tile boundaries and are zero padded


# --------------------------------------------------------------------------------------------
# aux-loss plumbing
# --------------------------------------------------------------------------------------------
class _AuxLossScaler(torch.autograd.Function):
    """Attaches an auxiliary loss to an activation: identity forward, injects d(aux)=scale in the backward."""

    scale = 1.0

    @staticmethod
    def forward(ctx, x, aux):
        ctx.save_for_backward(aux)
        return x

    @staticmethod
    def backward(ctx, g):
        (aux,) = ctx.saved_tensors
        return g, torch.ones_like(aux) * _AuxLossScaler.scale


def set_aux_loss_scale(scale: float):
    _AuxLossScaler.scale = float(scale)


# --------------------------------------------------------------------------------------------
# router
# --------------------------------------------------------------------------------------------
def topk_routing(logits: torch.Tensor, spec: ModelSpec, expert_bias: Optional[torch.Tensor] = None):
    """logits [T, E] (fp32) -> (probs [T, k], idx [T, k]); differentiable in probs."""
    k, E = spec.topk, logits.shape[1]
    if logits.is_cuda and not (spec.router_groups and spec.router_group_topk) and E <= 256 and k <= 8:
        # one kernel per direction: scores, selection, probabilities (ops/fused.py::router_topk)
        probs, idx, _, _ = ops.router_topk(logits, k, spec.router_score, spec.router_pre_softmax, expert_bias,
                                           spec.router_scaling)
        return probs, idx

    def limited_topk(scores):
        if spec.router_groups and spec.router_group_topk:
            T = scores.shape[0]
            g = spec.router_groups
            grouped = scores.view(T, g, E // g)
            gscore = grouped.topk(max(1, k // spec.router_group_topk), dim=-1).values.sum(-1)
            keep = gscore.topk(spec.router_group_topk, dim=-1).indices
            mask = torch.zeros(T, g, dtype=torch.bool, device=scores.device).scatter_(1, keep, True)
            scores = scores.masked_fill(~mask.unsqueeze(-1).expand(T, g, E // g).reshape(T, E), float("-inf"))
        return scores.topk(k, dim=-1)

    if spec.router_score == "softmax":
        if spec.router_pre_softmax:
            scores = torch.softmax(logits, dim=-1)
            probs, idx = limited_topk(scores)
        else:
            vals, idx = limited_topk(logits)
            probs = torch.softmax(vals, dim=-1)
    else:
        scores = torch.sigmoid(logits)
        sel = scores + expert_bias if expert_bias is not None else scores
        _, idx = limited_topk(sel)
        probs = scores.gather(1, idx)
        if k > 1:
            probs = probs / (probs.sum(-1, keepdim=True) + 1e-20)
    if spec.router_scaling:
        probs = probs * spec.router_scaling
    return probs, idx


def apply_capacity(probs, idx, E: int, capacity: int, policy: str):
    """Drop assignments beyond ``capacity`` per expert; dropped slots get probability 0 and index -1."""
    T, k = idx.shape
    flat_e = idx.reshape(-1)
    if policy == "probs":
        order = torch.argsort(probs.reshape(-1), descending=True, stable=True)
    else:
        order = torch.arange(T * k, device=idx.device)
    e_sorted = flat_e[order]
    onehot = torch.nn.functional.one_hot(e_sorted, E)
    rank_in_e = (onehot.cumsum(0) - 1).gather(1, e_sorted[:, None])[:, 0]
    keep_sorted = rank_in_e < capacity
    keep = torch.zeros(T * k, dtype=torch.bool, device=idx.device)
    keep[order] = keep_sorted
    keep = keep.view(T, k)
    return probs * keep, torch.where(keep, idx, torch.full_like(idx, -1))


def switch_aux_loss(logits, idx, E, k, coeff, group=None):
    """``sum_e mean_prob_e * fraction_e * E * coeff`` with counts summed over the sequence-partition group."""
    T = logits.shape[0]
    scores = torch.softmax(logits, dim=-1)
    counts = torch.zeros(E, dtype=torch.float32, device=logits.device)
    valid = idx.reshape(-1)
    valid = valid[valid >= 0]
    counts.index_add_(0, valid, torch.ones_like(valid, dtype=torch.float32))
    total_T = T
    if group is not None and group.size > 1 and group.group is not None:
        dist.all_reduce(counts, group=group.group)
        total_T = T * group.size
    agg = scores.sum(0)
    return (agg * counts).sum() * (E * coeff / (k * total_T * T))


def sequence_aux_loss(logits, idx, E, k, coeff, batch: int):
    """Load-balancing loss computed per sequence and averaged over the batch (rows are ordered ``s * batch + b``):
    for every sequence, ``sum_e mean_prob_e * fraction_e * E / k`` (moe/moe_utils.py:62-112)."""
    T = logits.shape[0]
    S = T // batch
    scores = torch.softmax(logits, dim=-1).view(S, batch, E)
    valid = (idx >= 0)
    onehot = torch.zeros(T, E, dtype=torch.float32, device=logits.device)
    onehot.scatter_add_(1, idx.clamp(min=0), valid.to(torch.float32))
    frac = onehot.view(S, batch, E).sum(0) / (S * k)            # [batch, E] fraction of the sequence's slots
    mean_prob = scores.mean(0)                                     # [batch, E]
    return (mean_prob * frac).sum(-1).mean() * (E * coeff)


def sinkhorn(cost: torch.Tensor, tol: float = 1e-4, max_iter: int = 100) -> torch.Tensor:
    """Sinkhorn-Knopp normalisation of ``exp(cost)`` towards uniform row and column sums (moe/moe_utils.py:14-59)."""
    cost = torch.exp(cost)
    d0 = torch.ones(cost.size(0), device=cost.device, dtype=cost.dtype)
    d1 = torch.ones(cost.size(1), device=cost.device, dtype=cost.dtype)
    eps = 1e-8
    err = 1e9
    it = 0
    while err > tol and it < max_iter:
        d1_old = d1
        d0 = (1.0 / d0.size(0)) / (torch.sum(d1 * cost, 1) + eps)
        d1 = (1.0 / d1.size(0)) / (torch.sum(d0.unsqueeze(1) * cost, 0) + eps)
        err = float(torch.mean(torch.abs(d1_old - d1)))
        it += 1
    return d1 * cost * d0.unsqueeze(1)


def sinkhorn_routing(logits: torch.Tensor, k: int, training: bool):
    """Selection by the balanced assignment (no gradient), probabilities from the raw logits: sigmoid for top-1,
    softmax otherwise (moe/router.py:236-262)."""
    act = (lambda x: torch.sigmoid(x)) if k == 1 else (lambda x: torch.softmax(x, dim=-1, dtype=torch.float32))
    if training:
        with torch.no_grad():
            idx = sinkhorn(logits.float()).topk(k, dim=1).indices
        return act(logits).gather(1, idx), idx
    scores = act(logits)
    probs, idx = scores.topk(k, dim=1)
    return probs, idx


def z_loss(logits, coeff):
    return torch.logsumexp(logits, dim=-1).pow(2).mean() * coeff


class GalvatronMoERouter(nn.Module):
    def __init__(self, spec: ModelSpec, ctx: LayerCtx, device, name: str):
        super().__init__()
        self.spec, self.ctx, self.name = spec, ctx, name
        self.router = nn.Module()
        self.router.weight = _param((spec.experts, spec.hidden), torch.float32, device)
        self.router.weight.tp_replicated = True
        if spec.router_expert_bias:
            self.router.register_buffer("expert_bias", torch.zeros(spec.experts, device=device))
            self.router.register_buffer("local_tokens_per_expert", torch.zeros(spec.experts, device=device))

    def reset_parameters(self, seed=1234, full_init=False):
        init_normal_sharded_(self.router.weight, self.spec.init_std, (self.spec.experts, self.spec.hidden), None, 0, 1,
                             seed, self.name + ".router.weight", full_init)

    def update_expert_bias(self, rate: float, group=None):
        """Aux-loss-free balancing: after an optimizer step, raise the selection bias of under-loaded experts and
        lower that of over-loaded ones by ``rate`` (token counts summed over ``group``), then reset the counters
        (moe/moe_utils.py:547-571)."""
        if not hasattr(self.router, "expert_bias"):
            return
        with torch.no_grad():
            load = self.router.local_tokens_per_expert.clone()
            if group is not None and dist.is_initialized():
                dist.all_reduce(load, group=group)
            self.router.expert_bias += torch.sign(load.mean() - load) * rate
            self.router.local_tokens_per_expert.zero_()

    def forward(self, x2d: torch.Tensor):
        """x2d [T, H] -> (probs [T, k] fp32, idx [T, k] int64 with -1 for dropped, x2d possibly carrying aux losses)."""
        s = self.spec
        xin = x2d
        if s.jitter_eps and self.training:
            noise = torch.empty_like(xin).uniform_(1.0 - s.jitter_eps, 1.0 + s.jitter_eps)
            xin = xin * noise
        if xin.is_cuda and xin.dtype in (torch.bfloat16, torch.float16) and s.router_dtype != "fp64" and s.experts % 8 == 0:
            logits = _GateLinear.apply(xin, self.router.weight)     # tcgen05 GEMM, fp32 accumulation and output
        else:
            dt = torch.float64 if s.router_dtype == "fp64" else torch.float32
            logits = torch.nn.functional.linear(xin.to(dt), self.router.weight.to(dt)).float()
        # `calculate_per_token_loss`: the trainer then divides every gradient by the token count, so the auxiliary
        # losses are multiplied by the local token count to keep their weight (reference: moe/router.py:303-312, 334-342)
        tok_scale = float(x2d.shape[0]) if s.per_token_loss else 1.0
        if s.z_loss_coeff and self.training:
            logits = _AuxLossScaler.apply(logits, z_loss(logits, s.z_loss_coeff) * tok_scale)
        bias = getattr(self.router, "expert_bias", None)
        if s.load_balancing == "sinkhorn":
            probs, idx = sinkhorn_routing(logits, s.topk, self.training)
        else:
            probs, idx = topk_routing(logits, s, bias)
        if s.capacity_factor is not None:
            cap = math.ceil(x2d.shape[0] * s.topk / s.experts * s.capacity_factor)
            probs, idx = apply_capacity(probs, idx, s.experts, cap, s.drop_policy)
        if s.aux_loss_coeff and s.load_balancing == "seq_aux_loss" and self.training and getattr(self, "batch_hint", 0):
            probs = _AuxLossScaler.apply(probs, sequence_aux_loss(logits, idx, s.experts, s.topk, s.aux_loss_coeff,
                                                                  self.batch_hint) * tok_scale)
        elif s.aux_loss_coeff and s.load_balancing in ("aux_loss", "seq_aux_loss") and self.training:
            grp = self.ctx.tp if self.ctx.tp_size > 1 else (self.ctx.sp if self.ctx.sp_size > 1 else None)
            probs = _AuxLossScaler.apply(probs, switch_aux_loss(logits, idx, s.experts, s.topk, s.aux_loss_coeff, grp) * tok_scale)
        if bias is not None:
            with torch.no_grad():
                v = idx.reshape(-1)
                self.router.local_tokens_per_expert.index_add_(0, v[v >= 0], torch.ones_like(v[v >= 0], dtype=torch.float32))
        return probs, idx


# --------------------------------------------------------------------------------------------
# experts
# --------------------------------------------------------------------------------------------
class _GroupedLinear(torch.autograd.Function):
    """Per-segment ``y = x @ w[g].T`` on the grouped tcgen05 GEMM; weight gradients go to ``main_grad``."""

    @staticmethod
    def forward(ctx, x, w, row_start):
        ctx.save_for_backward(x, w, row_start)
        return ops.grouped_gemm(x, w, row_start)

    @staticmethod
    def backward(ctx, dy):
        x, w, row_start = ctx.saved_tensors
        dy = dy.contiguous()
        dx = ops.grouped_gemm(dy, w, row_start, b_mn=True)
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            fresh = getattr(w, "mg_fresh", False)
            ops.grouped_wgrad(dy, x, row_start, mg, accumulate=not fresh)
            w.mg_fresh = False
            return dx, None, None
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        ops.grouped_wgrad(dy, x, row_start, dw, accumulate=False)
        return dx, dw.to(w.dtype), None


def grouped_linear(x, w, row_start):
    if not x.is_cuda:
        rs = row_start.tolist()
        outs = [torch.nn.functional.linear(x[rs[g]:rs[g + 1]], w[g]) for g in range(w.shape[0])]
        pad = x.new_zeros((x.shape[0] - rs[-1], w.shape[1]))
        return torch.cat(outs + [pad], dim=0)
    return _GroupedLinear.apply(x, w, row_start)


class _GateLinear(torch.autograd.Function):
    """Router logits ``x [T, H] (bf16) @ W[E, H]^T -> [T, E]`` in fp32 on the tcgen05 GEMM (bf16 operands, fp32
    accumulator written out unrounded), with both gradients on the same kernel; replaces the fp32 library GEMM on a
    widened copy of the activations (galvatron/core/runtime/moe/router.py gating)."""

    @staticmethod
    def forward(ctx, x, w):
        wl = w.detach().to(x.dtype)
        ctx.save_for_backward(x, wl)
        ctx.w = w
        return ops.gemm(x, wl, out_mode=OUT_F32)

    @staticmethod
    def backward(ctx, dlogits):
        x, wl = ctx.saved_tensors
        w = ctx.w
        dl = dlogits.to(x.dtype).contiguous()
        dx = ops.gemm(dl, wl, b_mn=True)
        mg = getattr(w, "main_grad", None)
        if mg is not None and mg.dtype == torch.float32:
            fresh = getattr(w, "mg_fresh", False)
            ops.gemm(dl, x, a_mn=True, b_mn=True, out=mg, out_mode=OUT_F32 if fresh else OUT_F32_ACC)
            w.mg_fresh = False
            return dx, None
        dw = ops.gemm(dl, x, a_mn=True, b_mn=True, out_mode=OUT_F32)
        return dx, dw.to(w.dtype)


class _ExpertSliceLinear(torch.autograd.Function):
    """``y = x @ w[j].T`` for one expert ``j`` of a stacked weight ``[E, N, K]`` on the dense tcgen05 GEMM; the weight
    gradient goes into expert ``j``'s slice of the stacked weight's ``main_grad`` (or of a dense gradient)."""

    @staticmethod
    def forward(ctx, x, w, j, first_use):
        ctx.save_for_backward(x, w)
        ctx.j, ctx.first_use = j, first_use
        return ops.gemm(x, w[j])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        j = ctx.j
        dy = dy.contiguous()
        dx = ops.gemm(dy, w[j], b_mn=True)
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            fresh = getattr(w, "mg_fresh", False)
            if fresh and ctx.first_use:
                mg.zero_()               # the experts run one by one: clear the stack once, then every slice accumulates
                w.mg_fresh = False
            ops.gemm(dy, x, a_mn=True, b_mn=True, out=mg[j], out_mode=OUT_F32_ACC)
            return dx, None, None, None
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        ops.gemm(dy, x, a_mn=True, b_mn=True, out=dw[j], out_mode=OUT_F32)
        return dx, dw.to(w.dtype), None, None


def sequential_expert_mlp(x, w1, w2, row_start, activation):
    """The experts one after the other on the rows ``[row_start[g], row_start[g+1])`` (``moe_grouped_gemm: false``;
    galvatron/core/runtime/moe/mlp.py:128-211).  The segment bounds are read on the host (one synchronisation per
    layer), which the grouped form avoids."""
    rs = row_start.tolist()
    out = x.new_zeros((x.shape[0], w2.shape[1]))
    order = [g for g in range(w1.shape[0]) if rs[g + 1] > rs[g]]
    for n, g in enumerate(order):
        xs = x[rs[g]:rs[g + 1]]
        # autograd runs the experts in reverse: the last expert of the forward is the first to touch main_grad
        first_in_backward = n == len(order) - 1
        if x.is_cuda:
            y = _ExpertSliceLinear.apply(xs, w1, g, first_in_backward)
            o = _ExpertSliceLinear.apply(ops.activation(y, activation), w2, g, first_in_backward)
        else:
            o = torch.nn.functional.linear(ops.activation(torch.nn.functional.linear(xs, w1[g]), activation), w2[g])
        out = _WriteRows.apply(out, o, rs[g])
    return out


class _WriteRows(torch.autograd.Function):
    """``out[start : start + rows] = part`` as a differentiable in-place write into a buffer built for it."""

    @staticmethod
    def forward(ctx, out, part, start):
        ctx.start, ctx.rows = start, part.shape[0]
        out[start:start + part.shape[0]] = part
        ctx.mark_dirty(out)
        return out

    @staticmethod
    def backward(ctx, g):
        return g, g[ctx.start:ctx.start + ctx.rows], None


class ExpertMLP(nn.Module):
    def __init__(self, spec: ModelSpec, ctx: LayerCtx, device, name: str):
        super().__init__()
        self.spec, self.ctx, self.name = spec, ctx, name
        if spec.experts % ctx.ep_size:
            raise ValueError("experts (%d) must be divisible by ep=%d" % (spec.experts, ctx.ep_size))
        self.E_loc = spec.experts // ctx.ep_size
        t = ctx.etp_size
        self.Fl = spec.moe_ffn // t
        mult = 2 if spec.gated else 1
        self.linear_fc1 = nn.Module()
        self.linear_fc1.weight = _param((self.E_loc, mult * self.Fl, spec.hidden), spec.dtype, device)
        self.linear_fc2 = nn.Module()
        self.linear_fc2.weight = _param((self.E_loc, spec.hidden, self.Fl), spec.dtype, device)

    def reset_parameters(self, seed, full_init):
        s, c = self.spec, self.ctx
        for j in range(self.E_loc):
            e = c.ep_rank * self.E_loc + j
            base = "%s.local_experts.%d" % (self.name, e)
            w1 = self.linear_fc1.weight[j]
            if s.gated:
                init_normal_sharded_(w1[: self.Fl], s.init_std, (s.moe_ffn, s.hidden), 0, c.etp_rank, c.etp_size, seed,
                                     base + ".gate", full_init)
                init_normal_sharded_(w1[self.Fl:], s.init_std, (s.moe_ffn, s.hidden), 0, c.etp_rank, c.etp_size, seed,
                                     base + ".up", full_init)
            else:
                init_normal_sharded_(w1, s.init_std, (s.moe_ffn, s.hidden), 0, c.etp_rank, c.etp_size, seed,
                                     base + ".fc1", full_init)
            init_normal_sharded_(self.linear_fc2.weight[j], s.init_std, (s.hidden, s.moe_ffn), 1, c.etp_rank, c.etp_size,
                                 seed, base + ".fc2", full_init)

    def forward(self, x: torch.Tensor, row_start: torch.Tensor) -> torch.Tensor:
        if not self.spec.grouped_gemm:
            return sequential_expert_mlp(x, self.linear_fc1.weight, self.linear_fc2.weight, row_start,
                                         self.spec.activation)
        y = grouped_linear(x, self.linear_fc1.weight, row_start)
        a = ops.activation(y, self.spec.activation)
        return grouped_linear(a, self.linear_fc2.weight, row_start)


# --------------------------------------------------------------------------------------------
# dispatch
# --------------------------------------------------------------------------------------------
def _aligned_starts(counts: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """Segment starts (int32 [G+1]) with every start a multiple of SEG_ALIGN; needs the host total."""
    padded = (counts + SEG_ALIGN - 1) // SEG_ALIGN * SEG_ALIGN
    starts = torch.zeros(counts.numel() + 1, dtype=torch.int64, device=counts.device)
    starts[1:] = padded.cumsum(0)
    return starts, int(starts[-1].item())


class GalvatronMoEMLP(nn.Module):
    """Token dispatch + experts + combine."""

    def __init__(self, spec: ModelSpec, ctx: LayerCtx, device, name: str):
        super().__init__()
        self.spec, self.ctx = spec, ctx
        self.experts = ExpertMLP(spec, ctx, device, name + ".experts")

    def reset_parameters(self, seed=1234, full_init=False):
        self.experts.reset_parameters(seed, full_init)

    def forward(self, x2d: torch.Tensor, probs: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        """``x2d [T, H]``, ``probs / idx [T, k]`` -> ``[T, H]``.

        Expert tensor parallelism (each expert's FFN dimension split over the ``tp_of_ep`` group): the tokens of the
        group are gathered, every rank runs the routed experts on its weight slice, and the partial sums are
        reduce-scattered back to the token owners (moe/token_dispatcher.py:560-600 does the gather after the
        all-to-all; gathering first keeps one code path for both dispatchers).
        All-gather dispatcher: tokens, probabilities and indices of the whole expert-parallel group are gathered,
        each rank serves the pairs routed to its local experts, and a reduce-scatter returns the weighted sums
        (moe/token_dispatcher.py:116-284)."""
        s, c = self.spec, self.ctx
        etp = c.etp_size
        if etp > 1:
            x2d = mp.gather_first_dim(x2d, c.tp_of_ep, grad_is_partial=True)
            probs = mp.gather_first_dim(probs, c.tp_of_ep, grad_is_partial=True)
            idx = mp.all_gather_first(idx.contiguous(), c.tp_of_ep)
        if s.dispatcher == "allgather" and c.ep_size > 1:
            E_loc = self.experts.E_loc
            lo = c.ep_rank * E_loc
            xa = mp.gather_first_dim(x2d, c.ep, grad_is_partial=True)
            pa = mp.gather_first_dim(probs, c.ep, grad_is_partial=True)
            ia = mp.all_gather_first(idx.contiguous(), c.ep)
            local = (ia >= lo) & (ia < lo + E_loc)
            il = torch.where(local, ia - lo, torch.full_like(ia, -1))
            out = self._routed(xa, pa, il, local_only=True)
            out = mp.reduce_scatter_first_dim(out, c.ep)
        else:
            out = self._routed(x2d, probs, idx)
        if etp > 1:
            out = mp.reduce_scatter_first_dim(out, c.tp_of_ep)
        return out

    def _routed(self, x2d: torch.Tensor, probs: torch.Tensor, idx: torch.Tensor, local_only: bool = False) -> torch.Tensor:
        """Dispatch to the experts and combine.  ``local_only``: ``idx`` already names local experts (``-1`` for
        pairs served elsewhere) and no exchange is needed."""
        s, c = self.spec, self.ctx
        T, H = x2d.shape
        k, E, ep, E_loc = s.topk, s.experts, c.ep_size, self.experts.E_loc
        if local_only:
            E, ep = E_loc, 1
        # "flex" is the reference's fused dispatcher (DeepEP, moe/token_dispatcher.py:743-1037); here it selects the
        # peer-memory pull kernels, which the fused-communication switch also turns on for "alltoall"
        if ep > 1 and (getattr(c, "fused_comm", False) or s.dispatcher == "flex"):
            from ..parallel import fused_a2a as fa

            if fa.usable(x2d, c.ep):
                # peer-memory path: tokens are pulled from their source ranks straight into the aligned expert
                # segments (all-to-all + permute in one kernel) and the outputs are pulled back home the same way
                bound = fa.static_bound(T, k, E_loc, SEG_ALIGN, s.expert_buffer_factor) if s.expert_buffer_factor else 0
                plan = fa.MoERouting(idx.to(torch.int32), c.ep, E, SEG_ALIGN, bound=bound)
                buf = fa.moe_dispatch(x2d, plan)
                out_buf = self.experts(buf, plan.row_start)
                w = torch.where(idx >= 0, probs, torch.zeros_like(probs)).to(torch.float32)
                # the routing weights are applied inside the pull kernel: no [T, k, H] intermediate
                return fa.moe_combine_weighted(out_buf, w, plan)
        flat_e = idx.reshape(-1)
        valid = flat_e >= 0
        sort_key = torch.where(valid, flat_e, torch.full_like(flat_e, E))
        order = torch.argsort(sort_key, stable=True)               # expert-major, token-minor
        n_valid = int(valid.sum().item()) if (s.capacity_factor is not None or local_only) else T * k
        order = order[:n_valid]
        tok_of = order // k
        e_sorted = flat_e[order]
        counts = torch.bincount(e_sorted, minlength=E)              # tokens per (global) expert from this rank
        send = x2d.index_select(0, tok_of)                           # [n_valid, H]
        if ep > 1:
            all_counts = mp.all_gather_first(counts, c.ep).view(ep, E)
            mine = all_counts[:, c.ep_rank * E_loc:(c.ep_rank + 1) * E_loc]          # [src, local expert]
            in_splits = counts.view(ep, E_loc).sum(1).tolist()
            out_splits = mine.sum(1).tolist()
            recv = mp.all_to_all(send, c.ep, out_splits, in_splits)                  # [src][local expert] order
        else:
            mine = counts.view(1, E_loc)
            recv = send
        # [src][local expert] -> [local expert][src], into aligned zero-padded segments
        per_expert = mine.sum(0)
        starts, total = _aligned_starts(per_expert)
        seg = mine.t().contiguous()                                   # [local expert, src]
        within = torch.cumsum(seg, dim=1) - seg                       # offset of each src block inside its expert
        src_block_start = (torch.cumsum(mine.reshape(-1), 0) - mine.reshape(-1)).view(mine.shape)  # in recv order
        n_src = mine.shape[0]
        rows = torch.arange(recv.shape[0], device=recv.device)
        blk_ends = torch.cumsum(mine.reshape(-1), 0)
        blk = torch.bucketize(rows, blk_ends, right=True)             # which (src, expert) block a row is in
        b_src, b_exp = blk // E_loc, blk % E_loc
        dest = starts[b_exp] + within[b_exp, b_src] + (rows - src_block_start.reshape(-1)[blk])
        buf = recv.new_zeros((max(total, SEG_ALIGN), H)).index_copy(0, dest, recv)
        row_start = starts.to(torch.int32)
        out_buf = self.experts(buf, row_start)
        back = out_buf.index_select(0, dest)
        if ep > 1:
            back = mp.all_to_all(back, c.ep, in_splits, out_splits)
        w = probs.reshape(-1)[order].to(torch.float32)
        out = torch.zeros((T, H), dtype=torch.float32, device=x2d.device)
        out = out.index_add(0, tok_of, back.float() * w[:, None])
        return out.to(x2d.dtype)


# --------------------------------------------------------------------------------------------
# layer + wrapping
# --------------------------------------------------------------------------------------------
class GalvatronMoEAttention(nn.Module):
    def __init__(self, spec, ctx, device, name):
        super().__init__()
        self.attn = GalvatronAttention(spec, ctx, device, name + ".attn")
        self.pre_router_norm = Norm(spec, device)
        # shared experts are dense parameters (replicated over the expert-parallel group, sharded over tp), so they
        # live in this unit and are reduced over the layer's full data-parallel group (moe/mlp.py:215-400)
        self.shared_experts = None
        if spec.shared_ffn > 0:
            from .modules import MLP

            self.shared_experts = MLP(spec, ctx, device, name + ".mlp.shared_experts", ffn=spec.shared_ffn)

    def reset_parameters(self, seed=1234, full_init=False):
        self.attn.reset_parameters(seed, full_init)
        self.pre_router_norm.reset_parameters()
        if self.shared_experts is not None:
            self.shared_experts.reset_parameters(seed, full_init)

    def forward(self, x):
        a = self.attn(x)
        n, h = self.pre_router_norm(a, residual=x)
        if self.shared_experts is not None:
            return n, h, self.shared_experts(n)
        return n, h


class GalvatronMoEDecoderLayer(nn.Module):
    def __init__(self, spec: ModelSpec, ctx: LayerCtx, device, name: str):
        super().__init__()
        self.spec, self.ctx = spec, ctx
        self.attention = GalvatronMoEAttention(spec, ctx, device, name)
        self.router = GalvatronMoERouter(spec, ctx, device, name)
        self.mlp = GalvatronMoEMLP(spec, ctx, device, name + ".mlp")

    def reset_parameters(self, seed=1234, full_init=False):
        self.attention.reset_parameters(seed, full_init)
        self.router.reset_parameters(seed, full_init)
        self.mlp.reset_parameters(seed, full_init)


class MoELayerRunner(nn.Module):
    """Runs the three units of an MoE layer in order (each between its own ZeRO hooks)."""

    def __init__(self, attention: UnitWrapper, router: UnitWrapper, mlp: UnitWrapper, units: List[ShardedUnit]):
        super().__init__()
        self.attention, self.router, self.mlp = attention, router, mlp
        self.sharded_units = units
        self.wrappers = [attention, router, mlp]

    @property
    def inner(self):
        return self

    def finish_backward(self):
        for w in self.wrappers:
            w.finish_backward()

    def forward(self, x):
        res = self.attention(x)
        n, h = res[0], res[1]
        S, B, H = n.shape
        n2 = n.reshape(S * B, H)
        self.router.inner.batch_hint = B
        probs, idx = self.router(n2)
        y = self.mlp(n2, probs, idx).view(S, B, H)
        if len(res) > 2:
            y = y + res[2]
        return ops_add(h, y)


def wrap_moe_units(layer: GalvatronMoEDecoderLayer, lp, ctx: LayerCtx, plan, reduce_in_fp32: bool,
                   fused_zero: bool = False):
    dp_size = plan.dp_size(plan.layers[0])
    defer = plan.async_grad_reduce
    u_attn = ShardedUnit(layer.attention, lp.name + "_attention", ctx.sdp, dp_size, lp.dp_type, reduce_in_fp32, tp=ctx.tp,
                         defer_sync=defer, fused_zero=fused_zero)
    u_router = ShardedUnit(layer.router, lp.name + "_router", ctx.sdp, dp_size, "ddp", reduce_in_fp32, tp=ctx.tp,
                           defer_sync=defer)
    u_mlp = ShardedUnit(layer.mlp, lp.name + "_mlp", ctx.dp_of_ep, dp_size, lp.dp_type, reduce_in_fp32, tp=None,
                        defer_sync=defer, fused_zero=fused_zero)
    return MoELayerRunner(UnitWrapper(layer.attention, u_attn, lp.checkpoint), UnitWrapper(layer.router, u_router),
                          UnitWrapper(layer.mlp, u_mlp, lp.checkpoint), [u_attn, u_router, u_mlp])
