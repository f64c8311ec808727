"""Tensor-parallel linear layers (Megatron TP with sequence parallelism) as functions of explicit weights.

Column-parallel: the input is sequence-sharded ``[S/t, B, K]``; it is all-gathered along the sequence and
multiplied by the local weight rows ``[N/t, K]``.  Row-parallel: the local product ``[S, B, K/t] x [N, K/t]^T``
is a partial sum that is reduce-scattered back to ``[S/t, B, N]``.

Two implementations of each:
  * baseline  -- NCCL collective (``parallel.mappings``) followed / preceded by the tcgen05 GEMM;
  * fused     -- one sm_100a kernel that moves the slabs over NVLink peer memory while the tensor cores
                 work (``parallel.fused_comm``), selected by ``ctx.fused_comm`` when the layer's tp group
                 has a symmetric-memory workspace.

Reference: galvatron/core/runtime/tensor_parallel/layers.py:262-427 (linear with async communication),
:547-816 (column parallel), :819-988 (row parallel).
"""
from __future__ import annotations

import torch

from .. import ops
from . import mappings as mp


def column_parallel_linear(x: torch.Tensor, w: torch.Tensor, bias, ctx) -> torch.Tensor:
    """x ``[S_local, B, K]`` -> ``[S_gathered, B, N_local]``."""
    if ctx.tp_size > 1:
        if ctx.fused_comm and x.is_cuda:
            from .fused_comm import all_gather_linear

            return all_gather_linear(x, w, bias, ctx.tp)
        if ctx.sequence_parallel:
            x = mp.gather_first_dim(x, ctx.tp, grad_is_partial=True)
        else:
            x = mp.copy_to_group(x, ctx.tp)
    return ops.linear(x, w, bias)


def row_parallel_linear(x: torch.Tensor, w: torch.Tensor, bias, ctx) -> torch.Tensor:
    """x ``[S, B, K_local]`` -> ``[S_local, B, N]`` (bias added once, after the reduction)."""
    if ctx.tp_size > 1:
        if ctx.fused_comm and x.is_cuda and ctx.sequence_parallel:
            from .fused_comm import linear_reduce_scatter

            y = linear_reduce_scatter(x, w, ctx.tp)
        else:
            y = ops.linear(x, w, None)
            y = mp.reduce_scatter_first_dim(y, ctx.tp) if ctx.sequence_parallel else mp.reduce_from_group(y, ctx.tp)
        if bias is not None:
            y = y + bias
        return y
    return ops.linear(x, w, bias)
