"""Python face of the fused tensor-parallel kernels (csrc/sm100/fused_tp2.cu on the CTA-pair tile when a rank's slab
is a multiple of 256 rows, csrc/sm100/fused_tp.cu on the one-CTA tile otherwise).

``all_gather_linear``      sequence-sharded ``[S/t, B, K]`` x column-parallel weight  -> ``[S, B, N/t]``
``linear_reduce_scatter``  ``[S, B, K/t]`` x row-parallel weight -> partial sums reduced to ``[S/t, B, N]``

Each is one kernel launch per direction: the all-gather / reduce-scatter traffic runs over NVLink peer
memory from inside the persistent tcgen05 GEMM.  The backward of each is the other (dgrad through the dual
fused kernel, wgrad on the gathered operand the forward already produced).

Buffers that peers touch live in one symmetric-memory workspace per tensor-parallel group
(``torch.distributed._symmetric_memory`` does the allocation and the handle exchange); the layout is

    [ signal slots | reduce-scatter tile flags x2 | all-gather staging x2 | reduce-scatter staging x2 ]

with two parities so that call ``n + 1`` never overwrites what a slower peer still reads from call ``n``.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _lib
from ..ops.gemm import OUT_BF16, OUT_F32, OUT_F32_ACC

_WORKSPACES: Dict[Tuple[int, ...], "TPWorkspace"] = {}
_SIGNAL_BYTES = 256


def _round_up(x, m):
    return (x + m - 1) // m * m


class TPWorkspace:
    def __init__(self, group, slab_rows: int, cols: int, device):
        from .symm_vmm import allocate

        self.group, self.t, self.me = group, group.size, group.rank
        self.slab_rows, self.cols = slab_rows, cols
        self.max_tiles = (slab_rows // 128) * ((cols + 255) // 256)
        t = self.t
        self.flag_bytes = _round_up(t * self.max_tiles * 4, 256)
        self.ag_bytes = _round_up(slab_rows * cols * 2, 256)
        self.rs_bytes = t * self.max_tiles * 128 * 256 * 2   # whole 128x256 tiles, wire layout
        self.off_flags = [_SIGNAL_BYTES + i * self.flag_bytes for i in range(2)]
        base = _SIGNAL_BYTES + 2 * self.flag_bytes
        self.off_ag = [base + i * self.ag_bytes for i in range(2)]
        base += 2 * self.ag_bytes
        self.off_rs = [base + i * self.rs_bytes for i in range(2)]
        total = base + 2 * self.rs_bytes
        self.buf, self.ptrs, self.handle = allocate(total, device, group.group)
        self.ag_epoch = 0
        self.rs_epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group.group)      # every rank's flags are zero before anybody's kernel polls them

    def fits(self, slab_rows, cols):
        return slab_rows <= self.slab_rows and cols <= self.cols

    def ptr_array(self, offset):
        arr = (ctypes.c_void_p * self.t)(*[p + offset for p in self.ptrs])
        return arr

    def local_view(self, offset, nbytes):
        return self.buf[offset:offset + nbytes]


def workspace_for(group, slab_rows: int, cols: int, device) -> TPWorkspace:
    key = tuple(group.ranks)
    ws = _WORKSPACES.get(key)
    if ws is None or not ws.fits(slab_rows, cols):
        ws = TPWorkspace(group, max(slab_rows, ws.slab_rows if ws else 0), max(cols, ws.cols if ws else 0), device)
        _WORKSPACES[key] = ws
    return ws


def usable(x2d_rows_per_rank: int, cols: int) -> bool:
    return x2d_rows_per_rank % 128 == 0 and cols % 8 == 0


def _pair_tile(slab_rows: int) -> bool:
    """The CTA-pair kernels tile 256 rows per cluster: a rank's slab must be made of whole pair tiles."""
    return slab_rows % 256 == 0 and os.environ.get("HG_FUSED_PAIR", "1") == "1"


# ---- raw launches ------------------------------------------------------------------------------------------
def ag_gemm(x_local: torch.Tensor, w: torch.Tensor, group, b_mn: bool = False, bias=None):
    """x_local ``[slab, K]`` (this rank's rows) -> (``[t*slab, N]``, gathered ``[t*slab, K]``)."""
    lib = _lib.load()
    slab, K = x_local.shape
    N = w.shape[1] if b_mn else w.shape[0]
    ws = workspace_for(group, slab, K, x_local.device)
    ws.ag_epoch += 1
    par = ws.ag_epoch & 1
    stage = ws.local_view(ws.off_ag[par], slab * K * 2).view(x_local.dtype).view(slab, K)
    stage.copy_(x_local)
    t = ws.t
    gathered = torch.empty((t * slab, K), dtype=x_local.dtype, device=x_local.device)
    ready = torch.zeros(t * slab // 128, dtype=torch.int32, device=x_local.device)
    out = torch.empty((t * slab, N), dtype=x_local.dtype, device=x_local.device)
    fn = lib.hg_ag_gemm2_bf16 if _pair_tile(slab) else lib.hg_ag_gemm_bf16
    rc = fn(ws.ptr_array(ws.off_ag[par]), ws.ptr_array(0), gathered.data_ptr(), ready.data_ptr(),
            w.data_ptr(), out.data_ptr(), _lib.ptr(bias), t, ws.me, ws.ag_epoch, slab, N, K,
            w.stride(0), out.stride(0), int(b_mn), OUT_BF16, _lib.stream())
    _lib.check(rc, "hg_ag_gemm_bf16")
    _lib.count_launch()
    return out, gathered


def gemm_rs(x: torch.Tensor, w: torch.Tensor, group, b_mn: bool = False) -> torch.Tensor:
    """x ``[t*slab, K]``, w ``[N, K]`` (or ``[K, N]``) -> this rank's ``[slab, N]`` of the summed product."""
    lib = _lib.load()
    M, K = x.shape
    N = w.shape[1] if b_mn else w.shape[0]
    t = group.size
    slab = M // t
    ws = workspace_for(group, slab, N, x.device)
    ws.rs_epoch += 1
    par = ws.rs_epoch & 1
    out = torch.empty((slab, N), dtype=x.dtype, device=x.device)
    fn = lib.hg_gemm_rs2_bf16 if _pair_tile(slab) else lib.hg_gemm_rs_bf16
    rc = fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), ws.ptr_array(ws.off_rs[par]),
            ws.ptr_array(ws.off_flags[par]), t, ws.me, ws.rs_epoch, slab, N, K, x.stride(0),
            w.stride(0), out.stride(0), int(b_mn), _lib.stream())
    _lib.check(rc, "hg_gemm_rs_bf16")
    _lib.count_launch()
    return out


# ---- autograd ----------------------------------------------------------------------------------------------
def _wgrad(dy, x, w):
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        fresh = getattr(w, "mg_fresh", False)
        ops.gemm(dy, x, a_mn=True, b_mn=True, out=mg, out_mode=OUT_F32 if fresh else OUT_F32_ACC)
        w.mg_fresh = False
        return None
    return ops.gemm(dy, x, a_mn=True, b_mn=True)


class _AllGatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, group):
        out, gathered = ag_gemm(x, w, group, False, bias)
        ctx.save_for_backward(gathered, w)
        ctx.group, ctx.has_bias = group, bias is not None
        return out

    @staticmethod
    def backward(ctx, dy):
        gathered, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm_rs(dy, w, ctx.group, b_mn=True)          # dgrad, partial sums reduced to our rows
        dw = _wgrad(dy, gathered, w)
        db = dy.float().sum(0).to(dy.dtype) if ctx.has_bias else None
        return dx, dw, db, None


class _LinearReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, group):
        ctx.save_for_backward(x, w)
        ctx.group = group
        return gemm_rs(x, w, group, False)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx, dy_all = ag_gemm(dy.contiguous(), w, ctx.group, b_mn=True)   # gather dy, dgrad in one kernel
        dw = _wgrad(dy_all, x, w)
        return dx, dw, None


def _peer_ok(x: torch.Tensor, group) -> bool:
    from .fused_zero import available

    return available(x.device, group.size, group.group)


def all_gather_linear(x: torch.Tensor, w: torch.Tensor, bias, group) -> torch.Tensor:
    """``[S_loc, B, K]`` -> ``[S_loc * t, B, N_loc]``"""
    S, B, K = x.shape
    if not usable(S * B, K) or not _peer_ok(x, group):
        from . import mappings as mp

        return ops.linear(mp.gather_first_dim(x, group, grad_is_partial=True), w, bias)
    out = _AllGatherLinear.apply(x.reshape(S * B, K).contiguous(), w, bias, group)
    return out.view(S * group.size, B, -1)


def linear_reduce_scatter(x: torch.Tensor, w: torch.Tensor, group) -> torch.Tensor:
    """``[S, B, K_loc]`` -> ``[S / t, B, N]``"""
    S, B, K = x.shape
    t = group.size
    if S % t or not usable(S // t * B, w.shape[0]) or K % 8 or not _peer_ok(x, group):
        from . import mappings as mp

        return mp.reduce_scatter_first_dim(ops.linear(x, w, None), group)
    out = _LinearReduceScatter.apply(x.reshape(S * B, K).contiguous(), w, group)
    return out.view(S // t, B, -1)
