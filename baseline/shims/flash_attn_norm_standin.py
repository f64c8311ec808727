"""Stand-ins for ``flash_attn.ops.rms_norm`` and ``flash_attn.ops.layer_norm``.

Both modules of the image's flash-attn 2.8 import ``dropout_layer_norm``, a CUDA extension built from
flash-attention's ``csrc/layer_norm`` that this image does not carry, and the reference imports them at module load
(``galvatron/core/runtime/transformer/norm.py:3-4``).  ``install()`` registers two replacement modules under those
names whose classes come from flash-attn itself:

* ``RMSNorm``: ``flash_attn.ops.triton.layer_norm.RMSNorm`` (flash-attn's own Triton kernel, same constructor
  arguments ``hidden_size, eps, device, dtype`` that the reference passes);
* ``DropoutAddLayerNorm``: ``torch.nn.LayerNorm`` under the constructor signature the reference uses
  (``hidden_size, eps, device, dtype``); only GPT-2-style models (``normalization: LayerNorm``) reach it.

None of this repository's kernels is involved.  The Triton module needs a CUDA driver at import, so the lookup is
deferred until the attribute is first read.
"""
from __future__ import annotations

import sys
import types


def _rms_norm_getattr(name):
    if name in ("RMSNorm", "rms_norm", "rms_norm_fn"):
        from flash_attn.ops.triton import layer_norm as tl_norm
        return {"RMSNorm": tl_norm.RMSNorm, "rms_norm": tl_norm.rms_norm_fn, "rms_norm_fn": tl_norm.rms_norm_fn}[name]
    raise AttributeError(name)


def _layer_norm_getattr(name):
    if name == "DropoutAddLayerNorm":
        import torch

        class DropoutAddLayerNorm(torch.nn.LayerNorm):
            def __init__(self, hidden_size, prenorm=False, p=0.0, eps=1e-5, residual_in_fp32=False,
                         device=None, dtype=None):
                super().__init__(hidden_size, eps=eps, device=device, dtype=dtype)
                assert not prenorm and p == 0.0

            def forward(self, x0, residual=None):
                return super().forward(x0 if residual is None else x0 + residual)

        return DropoutAddLayerNorm
    raise AttributeError(name)


def install():
    for modname, getter in (("flash_attn.ops.rms_norm", _rms_norm_getattr),
                            ("flash_attn.ops.layer_norm", _layer_norm_getattr)):
        if modname in sys.modules:
            continue
        m = types.ModuleType(modname)
        m.__getattr__ = getter
        sys.modules[modname] = m
