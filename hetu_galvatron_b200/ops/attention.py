"""Flash attention (tcgen05 kernels of csrc/sm100/attention.cu) with autograd.

Two entry points:

* :func:`flash_attention_packed` -- reads Q, K, V straight out of the fused QKV projection
  ``[S*B, (nh + 2*ng) * hd]`` whose columns are grouped per kv head as ``[ng, (nh/ng + 2), hd]``
  (the layout of the reference's ``linear_qkv``, galvatron/core/runtime/transformer/attention.py:876-926)
  and writes the context as ``[S*B, nh*hd]`` ready for the output projection.  No split / transpose
  copies exist in either direction: the backward writes dQ, dK, dV into one packed gradient buffer.
* :func:`flash_attention` -- separate ``[S, B, heads, hd]`` tensors with optional global position
  offsets and LSE output; the building block of the Ulysses and ring (context-parallel) paths.

Oracle: fp32 ``softmax(Q K^T / sqrt(hd) + causal mask) V``.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib
from ._lib import AttnTensor


def _desc(t: torch.Tensor, ss: int, sb: int, slots: int, gs: int, hs: int, off: int) -> AttnTensor:
    return AttnTensor(t.data_ptr(), ss, sb, slots, gs, hs, off)


def attention_reference(q, k, v, causal=True, scale=None, q_pos0=0, k_pos0=0, dropout_p: float = 0.0):
    """q: [S,B,nh,hd], k/v: [Skv,B,ng,hd] -> (out [S,B,nh,hd], lse [B,nh,S]); fp32 math.  ``dropout_p`` drops
    attention probabilities (after the softmax, rescaled by 1 / (1 - p)) from the current random stream."""
    S, B, nh, hd = q.shape
    Skv, ng = k.shape[0], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    qf = q.float().permute(1, 2, 0, 3)
    kf = k.float().permute(1, 2, 0, 3).repeat_interleave(nh // ng, dim=1)
    vf = v.float().permute(1, 2, 0, 3).repeat_interleave(nh // ng, dim=1)
    s = torch.einsum("bhqd,bhkd->bhqk", qf, kf) * scale
    if causal:
        qp = torch.arange(S, device=q.device) + q_pos0
        kp = torch.arange(Skv, device=q.device) + k_pos0
        s = s.masked_fill(kp[None, :] > qp[:, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    p = torch.nan_to_num(p, nan=0.0)
    if dropout_p > 0.0:
        p = torch.nn.functional.dropout(p, dropout_p, True)
    o = torch.einsum("bhqk,bhkd->bhqd", p, vf)
    return o.permute(2, 0, 1, 3).to(q.dtype), lse


class _FlashPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, S, B, nh, ng, hd, causal, scale):
        lib = _lib.load()
        T, P = qkv.shape
        qpg = nh // ng
        slots = nh + 2 * ng
        out = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty((B, nh, S), dtype=torch.float32, device=qkv.device)
        ss, sb = B * P, P
        q = _desc(qkv, ss, sb, slots, qpg + 2, 1, 0)
        k = _desc(qkv, ss, sb, slots, qpg + 2, 0, qpg)
        v = _desc(qkv, ss, sb, slots, qpg + 2, 0, qpg + 1)
        o = _desc(out, B * nh * hd, nh * hd, nh, qpg, 1, 0)
        rc = lib.hg_flash_fwd(ctypes.byref(q), ctypes.byref(k), ctypes.byref(v), ctypes.byref(o), lse.data_ptr(), S, S,
                              B, nh, ng, hd, int(causal), 0, 0, float(scale), _lib.stream())
        _lib.check(rc, "hg_flash_fwd")
        _lib.count_launch()
        ctx.save_for_backward(qkv, out, lse)
        ctx.cfg = (S, B, nh, ng, hd, causal, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        S, B, nh, ng, hd, causal, scale = ctx.cfg
        lib = _lib.load()
        T, P = qkv.shape
        qpg = nh // ng
        slots = nh + 2 * ng
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        dsum = torch.empty((B, nh, S), dtype=torch.float32, device=qkv.device)
        ss, sb = B * P, P
        q = _desc(qkv, ss, sb, slots, qpg + 2, 1, 0)
        k = _desc(qkv, ss, sb, slots, qpg + 2, 0, qpg)
        v = _desc(qkv, ss, sb, slots, qpg + 2, 0, qpg + 1)
        o = _desc(out, B * nh * hd, nh * hd, nh, qpg, 1, 0)
        do = _desc(dout, B * nh * hd, nh * hd, nh, qpg, 1, 0)
        dq = _desc(dqkv, ss, sb, slots, qpg + 2, 1, 0)
        dk = _desc(dqkv, ss, sb, slots, qpg + 2, 0, qpg)
        dv = _desc(dqkv, ss, sb, slots, qpg + 2, 0, qpg + 1)
        rc = lib.hg_flash_bwd(ctypes.byref(q), ctypes.byref(k), ctypes.byref(v), ctypes.byref(o), ctypes.byref(do),
                              lse.data_ptr(), dsum.data_ptr(), ctypes.byref(dq), ctypes.byref(dk), ctypes.byref(dv), S,
                              S, B, nh, ng, hd, int(causal), 0, 0, float(scale), _lib.stream())
        _lib.check(rc, "hg_flash_bwd")
        _lib.count_launch(3)
        return dqkv, None, None, None, None, None, None, None


def split_packed(qkv, nh, ng, hd):
    """Views of q [T,nh,hd], k [T,ng,hd], v [T,ng,hd] inside the packed projection (reference layout)."""
    T = qkv.shape[0]
    qpg = nh // ng
    g = qkv.view(T, ng, qpg + 2, hd)
    return g[:, :, :qpg].reshape(T, nh, hd), g[:, :, qpg], g[:, :, qpg + 1]


def flash_attention_packed(qkv: torch.Tensor, S: int, B: int, nh: int, ng: int, hd: int, causal: bool = True,
                           scale: float | None = None) -> torch.Tensor:
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if not qkv.is_cuda:
        q, k, v = split_packed(qkv, nh, ng, hd)
        o, _ = attention_reference(q.reshape(S, B, nh, hd), k.reshape(S, B, ng, hd), v.reshape(S, B, ng, hd), causal,
                                   scale)
        return o.reshape(S * B, nh * hd)
    if hd not in (64, 128):
        raise ValueError("the sm_100a flash attention kernels support head_dim 64 and 128")
    return _FlashPacked.apply(qkv.contiguous(), S, B, nh, ng, hd, causal, scale)


class _Flash(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, q_pos0, k_pos0):
        lib = _lib.load()
        S, B, nh, hd = q.shape
        Skv, ng = k.shape[0], k.shape[2]
        qpg = nh // ng
        out = torch.empty_like(q)
        lse = torch.empty((B, nh, S), dtype=torch.float32, device=q.device)
        qd = _desc(q, q.stride(0), q.stride(1), nh, qpg, 1, 0)
        kd = _desc(k, k.stride(0), k.stride(1), ng, 1, 0, 0)
        vd = _desc(v, v.stride(0), v.stride(1), ng, 1, 0, 0)
        od = _desc(out, out.stride(0), out.stride(1), nh, qpg, 1, 0)
        rc = lib.hg_flash_fwd(ctypes.byref(qd), ctypes.byref(kd), ctypes.byref(vd), ctypes.byref(od), lse.data_ptr(),
                              S, Skv, B, nh, ng, hd, int(causal), q_pos0, k_pos0, float(scale), _lib.stream())
        _lib.check(rc, "hg_flash_fwd")
        _lib.count_launch()
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (causal, scale, q_pos0, k_pos0)
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, k, v, out, lse = ctx.saved_tensors
        causal, scale, q_pos0, k_pos0 = ctx.cfg
        dq, dk, dv = flash_backward(q, k, v, out, dout.contiguous(), lse, causal, scale, q_pos0, k_pos0)
        return dq, dk, dv, None, None, None, None


def flash_backward(q, k, v, out, dout, lse, causal, scale, q_pos0=0, k_pos0=0):
    """Raw backward with an externally supplied (possibly global) LSE -- used by ring attention."""
    lib = _lib.load()
    S, B, nh, hd = q.shape
    Skv, ng = k.shape[0], k.shape[2]
    qpg = nh // ng
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dsum = torch.empty((B, nh, S), dtype=torch.float32, device=q.device)
    qd = _desc(q, q.stride(0), q.stride(1), nh, qpg, 1, 0)
    kd = _desc(k, k.stride(0), k.stride(1), ng, 1, 0, 0)
    vd = _desc(v, v.stride(0), v.stride(1), ng, 1, 0, 0)
    od = _desc(out, out.stride(0), out.stride(1), nh, qpg, 1, 0)
    dod = _desc(dout, dout.stride(0), dout.stride(1), nh, qpg, 1, 0)
    dqd = _desc(dq, dq.stride(0), dq.stride(1), nh, qpg, 1, 0)
    dkd = _desc(dk, dk.stride(0), dk.stride(1), ng, 1, 0, 0)
    dvd = _desc(dv, dv.stride(0), dv.stride(1), ng, 1, 0, 0)
    rc = lib.hg_flash_bwd(ctypes.byref(qd), ctypes.byref(kd), ctypes.byref(vd), ctypes.byref(od), ctypes.byref(dod),
                          lse.data_ptr(), dsum.data_ptr(), ctypes.byref(dqd), ctypes.byref(dkd), ctypes.byref(dvd), S,
                          Skv, B, nh, ng, hd, int(causal), q_pos0, k_pos0, float(scale), _lib.stream())
    _lib.check(rc, "hg_flash_bwd")
    _lib.count_launch(3)
    return dq, dk, dv


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
                    scale: float | None = None, q_pos0: int = 0, k_pos0: int = 0, return_lse: bool = False):
    """q ``[S,B,nh,hd]``, k/v ``[Skv,B,ng,hd]`` -> out ``[S,B,nh,hd]`` (and LSE ``[B,nh,S]``)."""
    hd = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if not q.is_cuda:
        o, lse = attention_reference(q, k, v, causal, scale, q_pos0, k_pos0)
        return (o, lse) if return_lse else o

    def fix(t):
        return t if (t.stride(-1) == 1 and t.stride(-2) == hd) else t.contiguous()

    out, lse = _Flash.apply(fix(q), fix(k), fix(v), causal, scale, q_pos0, k_pos0)
    return (out, lse) if return_lse else out


def attention_merge(out_acc: torch.Tensor, lse_acc: torch.Tensor, out_new: torch.Tensor, lse_new: torch.Tensor):
    """In-place log-sum-exp merge of a partial attention result over a disjoint key set (CUDA):
    ``out_acc`` fp32 ``[S, B, h, d]`` contiguous, ``lse_acc`` fp32 ``[B, h, S]`` whose last dimension may be a slice of a
    longer sequence, ``out_new`` bf16 ``[S, B, h, d]``, ``lse_new`` fp32 ``[B, h, S]``.  Oracle:
    ``l = logaddexp(lse_acc, lse_new); out = exp(lse_acc - l) * out_acc + exp(lse_new - l) * out_new``."""
    S, B, h, d = out_acc.shape
    if not (out_acc.is_contiguous() and lse_acc.stride(2) == 1 and lse_acc.stride(0) == h * lse_acc.stride(1)):
        raise ValueError("attention_merge: unsupported layout")
    out_new, lse_new = out_new.contiguous(), lse_new.contiguous()
    lib = _lib.load()
    rc = lib.hg_attn_merge(out_acc.data_ptr(), lse_acc.data_ptr(), lse_acc.stride(1), out_new.data_ptr(),
                           lse_new.data_ptr(), S, B * h, d, _lib.stream())
    _lib.check(rc, "hg_attn_merge")
    _lib.count_launch()
