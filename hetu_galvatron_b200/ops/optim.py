"""Flat-buffer optimizer kernels: fused AdamW, squared-norm reduction, clip coefficient and scaling.

CUDA tensors go through csrc/sm100/optim.cu; CPU tensors through the same math in PyTorch (the oracle).
Oracle for AdamW: ``torch.optim.AdamW`` (decoupled weight decay, bias-corrected moments).
"""
from __future__ import annotations

import torch

from . import _lib


def adamw_step(p32: torch.Tensor, grad: torch.Tensor, m: torch.Tensor, v: torch.Tensor, p_lp: torch.Tensor | None,
               *, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
               gscale: torch.Tensor | None = None, skip: torch.Tensor | None = None):
    """One AdamW step on flat buffers (fp32 master ``p32`` and moments; ``grad`` fp32 or bf16).

    ``gscale`` is an optional 1-element fp32 device tensor multiplied into the gradient (clip
    coefficient), ``skip`` an optional int32 flag that turns the step into a no-op; both stay on the
    device, so a clipped step needs no host synchronisation.  ``p_lp`` receives the bf16 copy."""
    n = p32.numel()
    if not p32.is_cuda:
        if skip is not None and int(skip.item()) != 0:
            return
        g = grad.float()
        if gscale is not None:
            g = g * gscale.float()
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        b1 = 1 - beta1 ** step
        b2 = 1 - beta2 ** step
        p32.mul_(1 - lr * weight_decay)
        p32.addcdiv_(m, (v.sqrt() / (b2 ** 0.5)).add_(eps), value=-lr / b1)
        if p_lp is not None:
            p_lp.copy_(p32)
        return
    lib = _lib.load()
    rc = lib.hg_adamw(p32.data_ptr(), grad.data_ptr(), m.data_ptr(), v.data_ptr(), _lib.ptr(p_lp), n,
                      int(grad.dtype == _lib.lp_dtype()), lr, beta1, beta2, eps, weight_decay, step,
                      _lib.ptr(gscale), _lib.ptr(skip), _lib.stream())
    _lib.check(rc, "hg_adamw")
    _lib.count_launch()


_scratch = {}


def _partials(device):
    key = str(device)
    if key not in _scratch:
        _scratch[key] = torch.empty(2048, dtype=torch.float32, device=device)
    return _scratch[key]


def sumsq(x: torch.Tensor, out: torch.Tensor, accumulate: bool = True, scale: float = 1.0):
    """``out[0] (+)= scale * sum(x^2)`` with a fixed reduction order (deterministic)."""
    if not x.is_cuda:
        val = scale * x.float().pow(2).sum()
        if accumulate:
            out[0] += val
        else:
            out[0] = val
        return out
    lib = _lib.load()
    x = x.contiguous()
    rc = lib.hg_sumsq(x.data_ptr(), x.numel(), int(x.dtype == _lib.lp_dtype()), _partials(x.device).data_ptr(),
                      out.data_ptr(), int(accumulate), float(scale), _lib.stream())
    _lib.check(rc, "hg_sumsq")
    _lib.count_launch(2)
    return out


def clip_coefficient(total_sumsq: torch.Tensor, max_norm: float, coef: torch.Tensor, norm_out: torch.Tensor):
    """``norm = sqrt(total)``, ``coef = min(1, max_norm / (norm + 1e-6))`` (1 when ``max_norm <= 0``)."""
    if not total_sumsq.is_cuda:
        nrm = total_sumsq[0].sqrt()
        norm_out[0] = nrm
        c = max_norm / (nrm + 1e-6)
        coef[0] = c if (max_norm > 0 and c < 1) else 1.0
        return
    lib = _lib.load()
    _lib.check(lib.hg_clip_coef(total_sumsq.data_ptr(), float(max_norm), coef.data_ptr(), norm_out.data_ptr(),
                                _lib.stream()), "hg_clip_coef")
    _lib.count_launch()


def scale_(x: torch.Tensor, coef: torch.Tensor | None = None, host_coef: float = 1.0):
    if not x.is_cuda:
        c = host_coef * (float(coef[0]) if coef is not None else 1.0)
        x.mul_(c)
        return x
    lib = _lib.load()
    _lib.check(lib.hg_scale(x.data_ptr(), x.numel(), int(x.dtype == _lib.lp_dtype()), _lib.ptr(coef), host_coef,
                            _lib.stream()), "hg_scale")
    _lib.count_launch()
    return x


def cast_bf16(src32: torch.Tensor, dst16: torch.Tensor):
    if not src32.is_cuda:
        dst16.copy_(src32)
        return dst16
    lib = _lib.load()
    _lib.check(lib.hg_cast_f32_bf16(src32.data_ptr(), dst16.data_ptr(), src32.numel(), _lib.stream()), "hg_cast")
    _lib.count_launch()
    return dst16
