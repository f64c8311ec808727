"""bf16 GEMM on the tcgen05 kernel (csrc/sm100/gemm.cu) and the autograd ``linear`` built on it.

The three products of a linear layer read the tensors exactly as PyTorch stores them:

* forward  ``y = x @ w.T``      : A = x [T,K] (K-major),  B = w [N,K] (K-major)
* dgrad    ``dx = dy @ w``      : A = dy [T,N] (K-major), B = w [N,K] read N-major
* wgrad    ``dw = dy.T @ x``    : A = dy [T,N] read M-major, B = x [T,K] read N-major

so no transpose pass ever runs.  With ``w.main_grad`` (an fp32 buffer owned by the sharded-parameter
manager) the weight gradient is accumulated there by the GEMM epilogue (``C += acc``), which is what
gradient accumulation over micro-batches and the ZeRO reduce-scatter consume.

Reference call sites replaced: galvatron/core/runtime/tensor_parallel/layers.py:300 (fwd), :342
(dgrad), :414 (wgrad).
"""
from __future__ import annotations

import os

import torch

from . import _lib

OUT_BF16, OUT_F32, OUT_F32_ACC, OUT_BF16_ACC = 0, 1, 2, 3


def _rowmajor(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        raise ValueError("expected a matrix")
    if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


# CTA-pair kernel (tcgen05.mma.cta_group::2, 256x256 tiles): "auto" uses it for problems of at least one pair tile,
# "0" never, "1" always.  The one-CTA kernel is the fallback when the device cannot co-schedule a pair.
_PAIR_MODE = os.environ.get("HG_GEMM_PAIR", "auto")
_pair_ok = True


def _use_pair(M: int, N: int, pair) -> bool:
    if pair is not None:
        return bool(pair)
    if not _pair_ok or _PAIR_MODE == "0":
        return False
    return _PAIR_MODE == "1" or (M >= 256 and N >= 256)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: torch.Tensor | None = None,
         out_mode: int = OUT_BF16, bias: torch.Tensor | None = None, max_ctas: int = 0, pair=None) -> torch.Tensor:
    """``C[M,N] = op(A) op(B)`` with fp32 accumulation.

    ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn``), ``b`` is ``[N,K]`` (or ``[K,N]`` when ``b_mn``).
    ``pair``: force (True) / forbid (False) the CTA-pair kernel; ``None`` follows ``HG_GEMM_PAIR``.
    """
    if not a.is_cuda:
        A = a.t() if a_mn else a
        Bm = b if b_mn else b.t()
        acc = A.float() @ Bm.float()
        if bias is not None:
            acc = acc + bias.float()
        if out is None:
            return acc.to(torch.float32 if out_mode in (OUT_F32, OUT_F32_ACC) else a.dtype)
        if out_mode in (OUT_F32_ACC, OUT_BF16_ACC):
            out.add_(acc.to(out.dtype))
        else:
            out.copy_(acc.to(out.dtype))
        return out
    lp = _lib.lp_dtype()
    if a.dtype != lp or b.dtype != lp:
        raise TypeError("the tcgen05 GEMM of this build takes %s operands, got %s and %s" % (lp, a.dtype, b.dtype))
    a, b = _rowmajor(a), _rowmajor(b)
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError("contraction mismatch: %s vs %s" % (tuple(a.shape), tuple(b.shape)))
    if out is None:
        dt = torch.float32 if out_mode in (OUT_F32, OUT_F32_ACC) else lp
        if out_mode in (OUT_F32_ACC, OUT_BF16_ACC):
            raise ValueError("accumulating output modes need `out`")
        out = torch.empty((M, N), dtype=dt, device=a.device)
    else:
        if out.shape[0] != M or out.shape[1] != N or out.stride(1) != 1:
            raise ValueError("bad output tensor")
    lib = _lib.load()
    if _use_pair(M, N, pair):
        rc = lib.hg_gemm2_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(bias), M, N, K, a.stride(0),
                               b.stride(0), out.stride(0), int(a_mn), int(b_mn), out_mode, max_ctas, _lib.stream())
        if rc == 0:
            _lib.count_launch()
            return out
        if rc != -2 or pair:
            raise _lib.KernelError("hg_gemm2_bf16 failed with code %d (M=%d N=%d K=%d a_mn=%d b_mn=%d)" % (rc, M, N, K, a_mn, b_mn))
        global _pair_ok
        _pair_ok = False  # this device cannot co-schedule the pair: one-CTA kernel from now on
    rc = lib.hg_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(bias), M, N, K, a.stride(0),
                          b.stride(0), out.stride(0), int(a_mn), int(b_mn), out_mode, max_ctas, _lib.stream())
    if rc != 0:
        raise _lib.KernelError(
            "hg_gemm_bf16 failed with code %d (M=%d N=%d K=%d a_mn=%d b_mn=%d a=%s/%s b=%s/%s out=%s/%s mode=%d)" %
            (rc, M, N, K, a_mn, b_mn, tuple(a.shape), a.stride(), tuple(b.shape), b.stride(), tuple(out.shape),
             out.stride(), out_mode))
    _lib.count_launch()
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        return gemm(x, w, bias=bias)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = _rowmajor(dy)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy, w, b_mn=True)
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                fresh = getattr(w, "mg_fresh", False)
                gemm(dy, x, a_mn=True, b_mn=True, out=mg, out_mode=OUT_F32 if fresh else OUT_F32_ACC)
                w.mg_fresh = False
                dw = None
            else:
                dw = gemm(dy, x, a_mn=True, b_mn=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w.T (+ bias)`` over the last dimension; leading dimensions are flattened."""
    if not x.is_cuda:
        return torch.nn.functional.linear(x, w, bias)
    shp = x.shape
    y = _Linear.apply(x.reshape(-1, shp[-1]), w, bias)
    return y.view(*shp[:-1], w.shape[0])


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, row_start: torch.Tensor, *, b_mn: bool = False,
                 out: torch.Tensor | None = None) -> torch.Tensor:
    """Per-group product for the MoE experts.

    ``a``: ``[rows, K]``; ``row_start``: int32 ``[G+1]`` on the device (segment boundaries, ascending);
    ``b``: ``[G, N, K]`` (or ``[G, K, N]`` when ``b_mn``).  Rows outside every segment are left untouched.
    """
    G = b.shape[0]
    if b_mn:
        K, N = b.shape[1], b.shape[2]
    else:
        N, K = b.shape[1], b.shape[2]
    if out is None:
        out = torch.zeros((a.shape[0], N), dtype=a.dtype, device=a.device)
    if not a.is_cuda:
        rs = row_start.tolist()
        for g in range(G):
            Bm = b[g] if b_mn else b[g].t()
            out[rs[g]:rs[g + 1]] = (a[rs[g]:rs[g + 1]].float() @ Bm.float()).to(out.dtype)
        return out
    if b_mn and K % 64 != 0:
        raise ValueError("grouped GEMM with an N-major B needs K % 64 == 0")
    a = _rowmajor(a)
    b2 = b.reshape(G * b.shape[1], b.shape[2])
    lib = _lib.load()
    rc = lib.hg_grouped_gemm_bf16(a.data_ptr(), b2.data_ptr(), out.data_ptr(), row_start.data_ptr(), G, a.shape[0], N,
                                  K, a.stride(0), b2.stride(0), out.stride(0), int(b_mn), OUT_BF16, _lib.stream())
    _lib.check(rc, "hg_grouped_gemm_bf16")
    _lib.count_launch()
    return out


def grouped_wgrad(dy: torch.Tensor, x: torch.Tensor, row_start: torch.Tensor, out: torch.Tensor,
                  accumulate: bool = True) -> torch.Tensor:
    """``out[g] (+)= dy[seg_g].T @ x[seg_g]``;  ``out``: fp32 ``[G, N, K]``.  Segment boundaries must be
    multiples of 64 rows (the permutation pads every expert's segment and zero-fills the padding)."""
    G = out.shape[0]
    if not dy.is_cuda:
        rs = row_start.tolist()
        for g in range(G):
            acc = dy[rs[g]:rs[g + 1]].float().t() @ x[rs[g]:rs[g + 1]].float()
            if accumulate:
                out[g] += acc.to(out.dtype)
            else:
                out[g] = acc.to(out.dtype)
        return out
    dy, x = _rowmajor(dy), _rowmajor(x)
    lib = _lib.load()
    rc = lib.hg_grouped_wgrad_bf16(dy.data_ptr(), x.data_ptr(), out.data_ptr(), row_start.data_ptr(), G, dy.shape[0],
                                   out.shape[1], out.shape[2], dy.stride(0), x.stride(0),
                                   OUT_F32_ACC if accumulate else OUT_F32, 0, _lib.stream())
    _lib.check(rc, "hg_grouped_wgrad_bf16")
    _lib.count_launch()
    return out


