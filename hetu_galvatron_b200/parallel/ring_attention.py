"""Context parallelism over a zig-zag split of the sequence.

The sequence is cut into ``2c`` chunks; rank ``r`` owns chunks ``r`` and ``2c-1-r`` (so that causal work
is balanced).  K and V of the whole group are all-gathered once (NVSwitch gives every pair full
bandwidth, so a ring of ``c`` point-to-point steps buys nothing on one node) and put into natural order;
each of the two local query chunks then attends to its causal prefix ``K[0 : (chunk+1) * half]`` in one
flash-attention call with the chunk's global position offset, which needs no partial-softmax merging.
The backward is autograd's transpose: flash-attention backward per chunk, then a reduce-scatter of dK/dV.

Capability parity: galvatron/core/runtime/transformer/attention_impl.py:564-780 (zig-zag ring forward /
backward with LSE merging), :437-478 (merge), utils/utils.py:295-325 (batch slicing).
"""
from __future__ import annotations

import torch

from .. import ops
from . import mappings as mp
from .reshard import apply_zigzag, undo_zigzag


def merge_attention(out_a, lse_a, out_b, lse_b):
    """Combine two partial softmax-attention results over disjoint key sets (fp32).
    ``out``: [S, B, h, d], ``lse``: [B, h, S]."""
    lse = torch.logaddexp(lse_a, lse_b)
    wa = torch.exp(lse_a - lse).permute(2, 0, 1).unsqueeze(-1)
    wb = torch.exp(lse_b - lse).permute(2, 0, 1).unsqueeze(-1)
    return out_a.float() * wa + out_b.float() * wb, lse


def ring_attention(q, k, v, cp_group, S_full: int):
    """q ``[S/c, B, nh, hd]``, k / v ``[S/c, B, ng, hd]`` in zig-zag order -> ``[S/c, B, nh, hd]``."""
    c = cp_group.size if cp_group is not None else 1
    if c == 1:
        return ops.flash_attention(q, k, v, causal=True)
    r = cp_group.rank
    S_loc = q.shape[0]
    half = S_loc // 2
    k_all = undo_zigzag(mp.gather_first_dim(k, cp_group, grad_is_partial=True), c)
    v_all = undo_zigzag(mp.gather_first_dim(v, cp_group, grad_is_partial=True), c)
    outs = []
    for qi, chunk in ((0, r), (1, 2 * c - 1 - r)):
        qc = q[qi * half:(qi + 1) * half]
        hi = (chunk + 1) * half
        outs.append(ops.flash_attention(qc, k_all[:hi], v_all[:hi], causal=True, q_pos0=chunk * half, k_pos0=0))
    return torch.cat(outs, dim=0)
