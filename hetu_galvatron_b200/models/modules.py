"""The generic decoder stack: embedding, attention block, MLP block, decoder layer, final norm, LM head.

Module and parameter names are the checkpoint contract (one unit per entry of the model's arch list):

    GalvatronEmbedding      embed_tokens.weight [V/vtp, H] (+ embed_positions.weight [S, H])
    GalvatronDecoderLayer   attn.input_layernorm.weight[/bias]
                            attn.attention.linear_qkv.weight[/bias]   [(nh+2ng)hd/t, H], grouped per kv head
                            attn.attention.linear_proj.weight[/bias]  [H, nh*hd/t]
                            ffn.post_attention_layernorm.weight[/bias]
                            ffn.mlp.linear_fc1.weight[/bias]          [2F/t, H] = cat(gate shard, up shard)
                            ffn.mlp.linear_fc2.weight[/bias]          [H, F/t]
    GalvatronFinalNorm      norm.weight[/bias]
    GalvatronCausalLMHead   lm_head.weight [V/vtp, H]

(reference: galvatron/core/runtime/models/modules.py:35-338, transformer/attention.py:515-926,
transformer/mlp.py:23-133).  Activations travel as ``[S_local, B, H]``.  Every layer gets its own
:class:`LayerCtx`, so neighbouring layers may use different tensor / sequence / context-parallel
degrees; the resharding between them lives in ``parallel/reshard.py``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..parallel import mappings as mp
from .spec import LayerCtx, ModelSpec


# --------------------------------------------------------------------------------------------
# parameter helpers
# --------------------------------------------------------------------------------------------
def _param(shape, dtype, device) -> nn.Parameter:
    return nn.Parameter(torch.empty(shape, dtype=dtype, device=device))


def init_normal_sharded_(p: torch.Tensor, std: float, full_shape, dim: Optional[int], rank: int, world: int,
                         seed: int, name: str, full_init: bool):
    """N(0, std) initialisation of a (possibly tensor-parallel) shard.

    ``full_init``: draw the *whole* tensor from a generator seeded by the parameter's name and slice
    this rank's shard -- identical to a single-process model with the same seed (used by the parity
    tests).  Otherwise draw only the shard, on the parameter's device, from a seed that depends on the
    rank (shards differ across tensor-parallel ranks, as with the reference's RNG tracker,
    galvatron/core/runtime/tensor_parallel/random.py:279-317)."""
    h = (hash_name(name) + seed) % (2 ** 31)
    if full_init:
        g = torch.Generator(device="cpu").manual_seed(h)
        full = torch.empty(full_shape, dtype=torch.float32).normal_(0.0, std, generator=g)
        if dim is not None and world > 1:
            full = full.chunk(world, dim=dim)[rank]
        p.data.copy_(full.to(p.dtype))
    else:
        g = torch.Generator(device=p.device).manual_seed((h + 7919 * rank) % (2 ** 31))
        p.data.normal_(0.0, std, generator=g)


def hash_name(name: str) -> int:
    v = 2166136261
    for ch in name.encode():
        v = ((v ^ ch) * 16777619) % (2 ** 32)
    return v


class Norm(nn.Module):
    def __init__(self, spec: ModelSpec, device, size: int = 0):
        super().__init__()
        self.rms = spec.norm == "RMSNorm"
        self.eps = spec.eps
        size = size or spec.hidden
        self.weight = _param((size,), spec.dtype, device)
        self.bias = None if self.rms else _param((size,), spec.dtype, device)
        self.weight.tp_replicated = True
        if self.bias is not None:
            self.bias.tp_replicated = True

    def reset_parameters(self):
        nn.init.ones_(self.weight)
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def forward(self, x, residual=None):
        return ops.norm(x, self.weight, self.bias, self.eps, self.rms, residual=residual)


class _Linear(nn.Module):
    """Holds ``weight [out_local, in_local]`` (+ bias); the parallel wiring is done by the caller."""

    def __init__(self, out_f, in_f, bias, spec: ModelSpec, device):
        super().__init__()
        self.weight = _param((out_f, in_f), spec.dtype, device)
        self.bias = _param((out_f,), spec.dtype, device) if bias else None


# --------------------------------------------------------------------------------------------
# positions
# --------------------------------------------------------------------------------------------
def zigzag_positions(S: int, cp: int, cp_rank: int, device) -> torch.Tensor:
    """Global positions of the tokens a context-parallel rank holds: chunks ``r`` and ``2c-1-r`` of
    the sequence cut into ``2c`` chunks (load-balanced causal split)."""
    half = S // (2 * cp)
    a = torch.arange(half, device=device)
    return torch.cat([cp_rank * half + a, (2 * cp - 1 - cp_rank) * half + a])


def local_positions(ctx: LayerCtx, S_full: int, S_rows: int, row0: int, device):
    """Positions of ``S_rows`` consecutive local rows starting at row ``row0`` of this rank's
    context-parallel portion.  Returns ``(pos_tensor | None, scalar_offset)``."""
    if ctx.cp_size > 1:
        zz = zigzag_positions(S_full, ctx.cp_size, ctx.cp_rank, device)
        return zz[row0:row0 + S_rows].to(torch.int32), 0
    return None, row0


# --------------------------------------------------------------------------------------------
# attention block
# --------------------------------------------------------------------------------------------
_WARNED_ATTN_DROPOUT = False


class SelfAttention(nn.Module):
    def __init__(self, spec: ModelSpec, ctx: LayerCtx, device, name: str):
        super().__init__()
        self.spec, self.ctx, self.name = spec, ctx, name
        t = ctx.tp_size
        if spec.heads % t or spec.kv_heads % t:
            raise ValueError("heads (%d) and kv heads (%d) must be divisible by tp=%d" % (spec.heads, spec.kv_heads, t))
        self.nh, self.ng, self.hd = spec.heads // t, spec.kv_heads // t, spec.head_dim
        self.linear_qkv = _Linear((self.nh + 2 * self.ng) * self.hd, spec.hidden, spec.qkv_bias, spec, device)
        self.linear_proj = _Linear(spec.hidden, self.nh * self.hd, spec.bias, spec, device)
        qpg = self.nh // self.ng
        rot = [g * (qpg + 2) + j for g in range(self.ng) for j in range(qpg + 1)]  # q heads and the k head
        self.register_buffer("rope_slots", torch.tensor(rot, dtype=torch.int32, device=device), persistent=False)
        self.rot_dim = int(self.hd * spec.rope_pct)
        # Optional per-head normalisation of queries and keys (the model's norm type over head_dim, one weight shared by
        # all heads, hence replicated over the tensor-parallel ranks and its gradient summed over them).
        # Reference: transformer/attention.py:705-742, 900-913 (q_layernorm / k_layernorm).
        self.q_layernorm = Norm(spec, device, size=self.hd) if spec.qk_layernorm else None
        self.k_layernorm = Norm(spec, device, size=self.hd) if spec.qk_layernorm else None
        # set by models.inference.forward_step for the duration of a cached forward; None in training
        self.inference_context = None
        self.layer_number = ctx.layer_index

    def reset_parameters(self, seed: int, full_init: bool):
        s, c = self.spec, self.ctx
        # the packed QKV rows are grouped per kv head, so a tensor-parallel shard is a contiguous row range
        init_normal_sharded_(self.linear_qkv.weight, s.init_std, (s.qkv_out, s.hidden), 0, c.tp_rank, c.tp_size, seed,
                             self.name + ".linear_qkv.weight", full_init)
        init_normal_sharded_(self.linear_proj.weight, s.init_std, (s.hidden, s.heads * s.head_dim), 1, c.tp_rank,
                             c.tp_size, seed, self.name + ".linear_proj.weight", full_init)
        for lin in (self.linear_qkv, self.linear_proj):
            if lin.bias is not None:
                nn.init.zeros_(lin.bias)
        if self.linear_proj.bias is not None:
            self.linear_proj.bias.tp_replicated = True
        for n in (self.q_layernorm, self.k_layernorm):
            if n is not None:
                n.reset_parameters()

    def _qk_norm(self, qkv2):
        """Normalise the query heads and the key head of every group inside the packed projection ``[T, P]``."""
        T = qkv2.shape[0]
        qpg = self.nh // self.ng
        g = qkv2.view(T, self.ng, qpg + 2, self.hd)
        q, _ = self.q_layernorm(g[:, :, :qpg].reshape(-1, self.hd))
        k, _ = self.k_layernorm(g[:, :, qpg].reshape(-1, self.hd))
        return torch.cat([q.view(T, self.ng, qpg, self.hd), k.view(T, self.ng, 1, self.hd), g[:, :, qpg + 1:]],
                         dim=2).reshape(T, -1)

    def run_realtime_tests(self):
        """``train.test_mode``: the query / key norm parameters must be identical on every data- and tensor-parallel
        rank (they are replicated, and a silent corruption of one copy would otherwise go unnoticed).
        Reference: transformer/attention.py:805-874."""
        if self.q_layernorm is None:
            return
        import torch.distributed as dist

        mine = torch.stack([p.detach().float() for n in (self.q_layernorm, self.k_layernorm)
                            for p in (n.weight, n.bias) if p is not None])
        for name, grp in (("dp", self.ctx.dp), ("tp", self.ctx.tp)):
            if grp is None or grp.size < 2 or grp.group is None:
                continue
            got = [torch.empty_like(mine) for _ in range(grp.size)]
            dist.all_gather(got, mine, group=grp.group)
            for r, other in enumerate(got):
                if not torch.equal(other, got[0]):
                    raise AssertionError("%s: query / key norm parameters of %s rank %d differ from rank 0's" %
                                         (self.name, name, r))

    def forward(self, x):
        """x: normalised hidden states ``[S_local, B, H]`` -> attention output ``[S_local, B, H]``."""
        s, c = self.spec, self.ctx
        from ..parallel.tp_layers import column_parallel_linear, row_parallel_linear

        qkv = column_parallel_linear(x, self.linear_qkv.weight, self.linear_qkv.bias, c)  # [S_att, B, P]
        S_att, B = qkv.shape[0], qkv.shape[1]
        S_full = c.seq_len or S_att * c.cp_size * c.sp_size
        qkv2 = qkv.reshape(S_att * B, -1)
        if self.q_layernorm is not None:
            if s.test_mode:
                self.run_realtime_tests()
            qkv2 = self._qk_norm(qkv2)
        if self.inference_context is not None:
            ctxv = self._cached_attention(qkv2, S_att, B)
            return row_parallel_linear(ctxv, self.linear_proj.weight, self.linear_proj.bias, c)
        if s.pos == "rope":
            row0 = c.sp_rank * S_att if c.sp_size > 1 else 0
            pos, off = local_positions(c, S_full, S_att, row0, qkv.device)
            if pos is not None:
                pos = pos.repeat_interleave(B)
            cos, sin = ops.rope_tables(max(S_full, 1), self.rot_dim, s.rope_base, str(qkv.device), s.rope_interp,
                                        s.rope_scaling_factor)
            qkv2 = ops.rope_packed(qkv2, self.rope_slots, self.hd, cos, sin, B, pos, off, s.rope_interleaved)
        if s.attention_dropout > 0.0 and self.training:
            ctxv = self._attention_with_dropout(qkv2, S_att, B)
        elif c.sp_size == 1 and c.cp_size == 1:
            ctxv = ops.flash_attention_packed(qkv2, S_att, B, self.nh, self.ng, self.hd, causal=True)
            ctxv = ctxv.view(S_att, B, self.nh * self.hd)
        else:
            q, k, v = ops.attention.split_packed(qkv2, self.nh, self.ng, self.hd)
            q = q.reshape(S_att, B, self.nh, self.hd)
            k = k.reshape(S_att, B, self.ng, self.hd)
            v = v.reshape(S_att, B, self.ng, self.hd)
            if c.sp_size > 1:
                from ..parallel.ulysses import ulysses_attention

                o = ulysses_attention(q, k, v, c, S_full)
            else:
                from ..parallel.ring_attention import ring_attention

                o = ring_attention(q, k, v, c.cp, S_full)
            ctxv = o.reshape(S_att, B, self.nh * self.hd)
        return row_parallel_linear(ctxv, self.linear_proj.weight, self.linear_proj.bias, c)


    def _attention_with_dropout(self, qkv2, S_att: int, B: int):
        """``attention_dropout`` > 0 while training: the flash kernels have no dropout, so the probabilities are formed
        explicitly (fp32, O(S^2) memory per head) and dropped from the tensor-parallel random stream (every rank holds
        different heads).  Reference: attention_impl.py:40-111 passes the rate to flash-attn's ``dropout_p``."""
        s, c = self.spec, self.ctx
        if c.sp_size > 1 or c.cp_size > 1:
            raise NotImplementedError("attention dropout with Ulysses or context parallelism")
        global _WARNED_ATTN_DROPOUT
        if not _WARNED_ATTN_DROPOUT:
            import warnings

            warnings.warn("attention_dropout = %g: attention runs on the unfused path (explicit probabilities) while "
                          "training" % s.attention_dropout)
            _WARNED_ATTN_DROPOUT = True
        q, k, v = ops.attention.split_packed(qkv2, self.nh, self.ng, self.hd)
        q = q.reshape(S_att, B, self.nh, self.hd)
        k = k.reshape(S_att, B, self.ng, self.hd)
        v = v.reshape(S_att, B, self.ng, self.hd)

        def run():
            return ops.attention.attention_reference(q, k, v, True, dropout_p=s.attention_dropout)[0]

        if c.tp_size > 1:
            from ..parallel.random import get_rng_tracker, tensor_parallel_rng_name

            tracker, name = get_rng_tracker(), tensor_parallel_rng_name(c.tp_size)
            if not tracker.check(name):
                with tracker.fork(name):
                    return run().reshape(S_att, B, self.nh * self.hd)
        return run().reshape(S_att, B, self.nh * self.hd)

    def _cached_attention(self, qkv2, S_new: int, B: int):
        """Incremental forward with a key / value cache (static batching): the new keys and values are written
        behind the ``sequence_len_offset`` tokens already cached for this layer and the new queries attend to
        everything up to their own position.  Counterpart of ``_adjust_key_value_for_inference`` and the
        cached branches of the reference's attention (transformer/attention.py:253-389, 398-513), which no entry
        point of the reference reaches; here ``models.inference`` drives it."""
        s, c, ic = self.spec, self.ctx, self.inference_context
        if c.sp_size > 1 or c.cp_size > 1:
            raise NotImplementedError("cached attention needs sp = cp = 1")
        past = ic.sequence_len_offset
        b0 = ic.batch_size_offset
        if past + S_new > ic.max_sequence_length or b0 + B > ic.max_batch_size:
            raise ValueError("inference context too small: %d + %d tokens of %d, batch %d + %d of %d" %
                             (past, S_new, ic.max_sequence_length, b0, B, ic.max_batch_size))
        if s.pos == "rope":
            cos, sin = ops.rope_tables(ic.max_sequence_length, self.rot_dim, s.rope_base, str(qkv2.device),
                                        s.rope_interp, s.rope_scaling_factor)
            qkv2 = ops.rope_packed(qkv2, self.rope_slots, self.hd, cos, sin, B, None, past, s.rope_interleaved)
        q, k, v = ops.attention.split_packed(qkv2, self.nh, self.ng, self.hd)
        q = q.reshape(S_new, B, self.nh, self.hd)
        k = k.reshape(S_new, B, self.ng, self.hd)
        v = v.reshape(S_new, B, self.ng, self.hd)
        key = self.layer_number
        if key not in ic.key_value_memory_dict:
            shape = (ic.max_sequence_length, ic.max_batch_size, self.ng, self.hd)
            ic.key_value_memory_dict[key] = (torch.zeros(shape, dtype=k.dtype, device=k.device),
                                             torch.zeros(shape, dtype=v.dtype, device=v.device))
        kc, vc = ic.key_value_memory_dict[key]
        kc[past:past + S_new, b0:b0 + B] = k
        vc[past:past + S_new, b0:b0 + B] = v
        o = ops.flash_attention(q, kc[:past + S_new, b0:b0 + B], vc[:past + S_new, b0:b0 + B], causal=True,
                                q_pos0=past, k_pos0=0)
        return o.reshape(S_new, B, self.nh * self.hd)


class CrossAttention(nn.Module):
    """Attention of the hidden states over another sequence: queries from ``x``, keys and values from
    ``key_value_states`` (``linear_q`` and a fused ``linear_kv``, both column-parallel over the layer's tp group),
    no mask, row-parallel output projection.  Same restriction as the reference's class
    (transformer/attention.py:929-1017): no grouped-query attention."""

    def __init__(self, spec: ModelSpec, ctx: LayerCtx, device, name: str):
        super().__init__()
        if spec.kv_heads != spec.heads:
            raise ValueError("Group query attention is not currently supported in cross attention.")
        if ctx.sp_size > 1 or ctx.cp_size > 1:
            raise NotImplementedError("cross attention with Ulysses or context parallelism")
        self.spec, self.ctx, self.name = spec, ctx, name
        t = ctx.tp_size
        if spec.heads % t:
            raise ValueError("heads (%d) must be divisible by tp=%d" % (spec.heads, t))
        self.nh, self.hd = spec.heads // t, spec.head_dim
        self.linear_q = _Linear(self.nh * self.hd, spec.hidden, spec.bias, spec, device)
        self.linear_kv = _Linear(2 * self.nh * self.hd, spec.hidden, spec.bias, spec, device)   # per head: [k | v]
        self.linear_proj = _Linear(spec.hidden, self.nh * self.hd, spec.bias, spec, device)

    def reset_parameters(self, seed: int, full_init: bool):
        s, c = self.spec, self.ctx
        full = s.heads * s.head_dim
        init_normal_sharded_(self.linear_q.weight, s.init_std, (full, s.hidden), 0, c.tp_rank, c.tp_size, seed,
                             self.name + ".linear_q.weight", full_init)
        init_normal_sharded_(self.linear_kv.weight, s.init_std, (2 * full, s.hidden), 0, c.tp_rank, c.tp_size, seed,
                             self.name + ".linear_kv.weight", full_init)
        init_normal_sharded_(self.linear_proj.weight, s.init_std, (s.hidden, full), 1, c.tp_rank, c.tp_size, seed,
                             self.name + ".linear_proj.weight", full_init)
        for lin in (self.linear_q, self.linear_kv, self.linear_proj):
            if lin.bias is not None:
                nn.init.zeros_(lin.bias)
        if self.linear_proj.bias is not None:
            self.linear_proj.bias.tp_replicated = True

    def forward(self, x, key_value_states):
        """``x [Sq_local, B, H]``, ``key_value_states [Sk_local, B, H]`` -> ``[Sq_local, B, H]``."""
        c = self.ctx
        from ..parallel.tp_layers import column_parallel_linear, row_parallel_linear

        q = column_parallel_linear(x, self.linear_q.weight, self.linear_q.bias, c)                       # [Sq, B, np*hn]
        kv = column_parallel_linear(key_value_states, self.linear_kv.weight, self.linear_kv.bias, c)    # [Sk, B, np*2*hn]
        Sq, B = q.shape[0], q.shape[1]
        Sk = kv.shape[0]
        q = q.reshape(Sq, B, self.nh, self.hd)
        kv = kv.reshape(Sk, B, self.nh, 2 * self.hd)
        k, v = kv[..., :self.hd], kv[..., self.hd:]
        o = ops.flash_attention(q, k.contiguous(), v.contiguous(), causal=False)
        return row_parallel_linear(o.reshape(Sq, B, self.nh * self.hd), self.linear_proj.weight,
                                   self.linear_proj.bias, c)


class GalvatronAttention(nn.Module):
    def __init__(self, spec, ctx, device, name):
        super().__init__()
        self.input_layernorm = Norm(spec, device)
        self.attention = SelfAttention(spec, ctx, device, name + ".attention")

    def reset_parameters(self, seed, full_init):
        self.input_layernorm.reset_parameters()
        self.attention.reset_parameters(seed, full_init)

    def forward(self, x):
        n, _ = self.input_layernorm(x)
        return self.attention(n)


# --------------------------------------------------------------------------------------------
# MLP block
# --------------------------------------------------------------------------------------------
class MLP(nn.Module):
    def __init__(self, spec: ModelSpec, ctx: LayerCtx, device, name: str, ffn: Optional[int] = None,
                 tp_group="tp"):
        super().__init__()
        self.spec, self.ctx, self.name = spec, ctx, name
        self.F = ffn or spec.ffn
        t = ctx.tp_size
        if self.F % t:
            raise ValueError("ffn size %d not divisible by tp=%d" % (self.F, t))
        self.Fl = self.F // t
        mult = 2 if spec.gated else 1
        self.linear_fc1 = _Linear(mult * self.Fl, spec.hidden, spec.bias, spec, device)
        self.linear_fc2 = _Linear(spec.hidden, self.Fl, spec.bias, spec, device)

    def reset_parameters(self, seed, full_init):
        s, c = self.spec, self.ctx
        w1 = self.linear_fc1.weight
        if s.gated:
            # rows = [gate shard ; up shard]: each half is a row-shard of its own full matrix
            init_normal_sharded_(w1[: self.Fl], s.init_std, (self.F, s.hidden), 0, c.tp_rank, c.tp_size, seed,
                                 self.name + ".linear_fc1.gate", full_init)
            init_normal_sharded_(w1[self.Fl:], s.init_std, (self.F, s.hidden), 0, c.tp_rank, c.tp_size, seed,
                                 self.name + ".linear_fc1.up", full_init)
        else:
            init_normal_sharded_(w1, s.init_std, (self.F, s.hidden), 0, c.tp_rank, c.tp_size, seed,
                                 self.name + ".linear_fc1.weight", full_init)
        init_normal_sharded_(self.linear_fc2.weight, s.init_std, (s.hidden, self.F), 1, c.tp_rank, c.tp_size, seed,
                             self.name + ".linear_fc2.weight", full_init)
        for lin in (self.linear_fc1, self.linear_fc2):
            if lin.bias is not None:
                nn.init.zeros_(lin.bias)
        if self.linear_fc2.bias is not None:
            self.linear_fc2.bias.tp_replicated = True

    def forward(self, x):
        from ..parallel.tp_layers import column_parallel_linear, row_parallel_linear

        y = column_parallel_linear(x, self.linear_fc1.weight, self.linear_fc1.bias, self.ctx)
        a = ops.activation(y, self.spec.activation)
        return row_parallel_linear(a, self.linear_fc2.weight, self.linear_fc2.bias, self.ctx)


class GalvatronMLP(nn.Module):
    def __init__(self, spec, ctx, device, name):
        super().__init__()
        self.post_attention_layernorm = Norm(spec, device)
        self.mlp = MLP(spec, ctx, device, name + ".mlp")

    def reset_parameters(self, seed, full_init):
        self.post_attention_layernorm.reset_parameters()
        self.mlp.reset_parameters(seed, full_init)

    def forward(self, attn_out, residual):
        p = self.mlp.spec.hidden_dropout
        n, h = self.post_attention_layernorm(hidden_dropout(attn_out, p, self.mlp.ctx, self.training),
                                             residual=residual)  # h = residual + attn_out
        return ops_add(h, hidden_dropout(self.mlp(n), p, self.mlp.ctx, self.training))


def hidden_dropout(x, p: float, ctx, training: bool):
    """Dropout on a block output.  Under tensor/sequence parallelism every rank of the group holds a different
    slice of the sequence, so the mask comes from the group's own random stream (``parallel/random.py``)."""
    if p <= 0.0 or not training:
        return x
    shard = max(ctx.tp_size, getattr(ctx, "sp_size", 1))
    if shard > 1:
        from ..parallel.random import get_rng_tracker, tensor_parallel_rng_name

        tracker = get_rng_tracker()
        name = tensor_parallel_rng_name(shard)
        if not tracker.check(name):
            with tracker.fork(name):
                return torch.nn.functional.dropout(x, p, True)
    return torch.nn.functional.dropout(x, p, True)


class _Add(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        from ..ops import _lib

        out = torch.empty_like(a)
        lib = _lib.load()
        _lib.check(lib.hg_add_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _lib.stream()), "hg_add")
        _lib.count_launch()
        return out

    @staticmethod
    def backward(ctx, g):
        return g, g


def ops_add(a, b):
    if a.is_cuda and a.dtype in (torch.bfloat16, torch.float16) and a.is_contiguous() and b.is_contiguous() and a.shape == b.shape:
        return _Add.apply(a, b)
    return a + b


# --------------------------------------------------------------------------------------------
# units
# --------------------------------------------------------------------------------------------
class GalvatronDecoderLayer(nn.Module):
    def __init__(self, spec: ModelSpec, ctx: LayerCtx, device, name: str):
        super().__init__()
        self.ctx = ctx
        self.attn = GalvatronAttention(spec, ctx, device, name + ".attn")
        self.ffn = GalvatronMLP(spec, ctx, device, name + ".ffn")

    def reset_parameters(self, seed=1234, full_init=False):
        self.attn.reset_parameters(seed, full_init)
        self.ffn.reset_parameters(seed, full_init)

    def forward(self, x):
        return self.ffn(self.attn(x), x)


class GalvatronEmbedding(nn.Module):
    """Vocab-parallel token embedding (+ learned absolute positions), output ``[S_local, B, H]``."""

    def __init__(self, spec: ModelSpec, ctx: LayerCtx, device, name: str):
        super().__init__()
        self.spec, self.ctx, self.name = spec, ctx, name
        from ..utils.training_utils import VocabUtility

        # this rank's rows of the (padded) vocabulary; raises when the vocab tp degree does not divide it
        self.v0, v1 = VocabUtility.vocab_range_from_global_vocab_size(spec.padded_vocab, ctx.tp_rank, ctx.tp_size)
        self.Vl = v1 - self.v0
        self.embed_tokens = nn.Module()
        self.embed_tokens.weight = _param((self.Vl, spec.hidden), spec.dtype, device)
        self.embed_positions = None
        if spec.pos == "learned_absolute":
            self.embed_positions = nn.Module()
            self.embed_positions.weight = _param((spec.seq_len, spec.hidden), spec.dtype, device)
            self.embed_positions.weight.tp_replicated = True

    def reset_parameters(self, seed=1234, full_init=False):
        s, c = self.spec, self.ctx
        init_normal_sharded_(self.embed_tokens.weight, s.init_std, (s.padded_vocab, s.hidden), 0, c.tp_rank, c.tp_size,
                             seed, "embed_tokens.weight", full_init)
        if self.embed_positions is not None:
            init_normal_sharded_(self.embed_positions.weight, s.init_std, (s.seq_len, s.hidden), None, 0, 1, seed,
                                 "embed_positions.weight", True if full_init else False)

    def forward(self, tokens):
        """tokens ``[B, S_cp]`` (already sliced for context parallelism) -> ``[S_local, B, H]``."""
        s, c = self.spec, self.ctx
        B, S_in = tokens.shape
        ids = tokens.t().contiguous()  # [S, B]
        row0 = 0
        if c.sp_size > 1:  # Ulysses-style vocab layers: slice the sequence locally, weights are whole
            S_loc = S_in // c.sp_size
            row0 = c.sp_rank * S_loc
            ids = ids[row0:row0 + S_loc]
        S_rows = ids.shape[0]
        pos_w = self.embed_positions.weight if self.embed_positions is not None else None
        if pos_w is not None and c.cp_size > 1:
            raise NotImplementedError("learned absolute positions with context parallelism")
        x = ops.embedding(ids.reshape(-1), self.embed_tokens.weight, v0=self.v0, pos_emb=pos_w, batch=B,
                          pos_offset=row0)
        x = x.view(S_rows, B, s.hidden)
        if c.tp_size > 1:
            if pos_w is not None:
                raise NotImplementedError("learned absolute positions with vocab tensor parallelism > 1")
            x = mp.reduce_scatter_first_dim(x, c.tp) if c.sequence_parallel else mp.reduce_from_group(x, c.tp)
        return x


class GalvatronFinalNorm(nn.Module):
    def __init__(self, spec, ctx, device, name):
        super().__init__()
        self.ctx = ctx
        self.norm = Norm(spec, device)

    def reset_parameters(self, seed=1234, full_init=False):
        self.norm.reset_parameters()

    def forward(self, x):
        return self.norm(x)[0]


class GalvatronCausalLMHead(nn.Module):
    """Vocab-parallel LM head + cross entropy; returns the per-token loss ``[B, S_local_tokens]``."""

    def __init__(self, spec: ModelSpec, ctx: LayerCtx, device, name: str, tied_weight: Optional[nn.Parameter] = None):
        super().__init__()
        self.spec, self.ctx, self.name = spec, ctx, name
        from ..utils.training_utils import VocabUtility

        self.v0, v1 = VocabUtility.vocab_range_from_global_vocab_size(spec.padded_vocab, ctx.tp_rank, ctx.tp_size)
        self.Vl = v1 - self.v0
        self.lm_head = nn.Module()
        if tied_weight is not None:
            self.lm_head.weight = tied_weight
            self.owns_weight = False
        else:
            self.lm_head.weight = _param((self.Vl, spec.hidden), spec.dtype, device)
            self.owns_weight = True

    def reset_parameters(self, seed=1234, full_init=False):
        if self.owns_weight:
            s, c = self.spec, self.ctx
            nm = "embed_tokens.weight" if s.tied else "lm_head.weight"
            init_normal_sharded_(self.lm_head.weight, s.init_std, (s.padded_vocab, s.hidden), 0, c.tp_rank, c.tp_size,
                                 seed, nm, full_init)

    def forward(self, x, labels=None):
        """x ``[S_local, B, H]``; labels ``[B, S_cp]``.  Without labels returns the local logits."""
        s, c = self.spec, self.ctx
        from ..parallel.tp_layers import column_parallel_linear

        logits = column_parallel_linear(x, self.lm_head.weight, None, c)  # [S_rows, B, V/t]
        S_rows, B = logits.shape[0], logits.shape[1]
        if labels is None:
            return logits
        lab = labels.t().contiguous()  # [S_cp, B]
        if c.sp_size > 1:
            lab = lab[c.sp_rank * S_rows:(c.sp_rank + 1) * S_rows]
        loss = ops.cross_entropy(logits.reshape(S_rows * B, -1), lab.reshape(-1), v0=self.v0,
                                 group=c.tp if c.tp_size > 1 else None)
        loss = loss.view(S_rows, B)
        if c.sp_size > 1:  # every rank returns the loss of the whole (cp-local) sequence
            loss = mp.gather_first_dim(loss, c.sp, grad_is_partial=False)
        return loss.t().contiguous()  # [B, S]
