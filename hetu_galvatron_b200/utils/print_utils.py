"""Rank-aware printing (galvatron/utils/print_utils.py)."""
from __future__ import annotations

import os


def is_rank0() -> bool:
    return int(os.environ.get("RANK", "0")) == 0


def print_rank0(*a, **kw):
    if is_rank0():
        print(*a, **kw)


def print_single_rank(message, rank: int = 0):
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_rank() == rank:
        print(message, flush=True)


def form_strategy(strategy) -> str:
    """``[pp, tp, dp, {flags}]`` -> ``"pp-tp-dp[f|*][-c][-sp]"`` as in search logs."""
    pp, tp, dp = strategy[0], strategy[1], strategy[2]
    info = strategy[3] if len(strategy) > 3 else {}
    s = "%d-%d%s-%d%s" % (pp, tp, "*" if info.get("tp") == 0 else "", dp, "f" if info.get("fsdp") else "")
    if info.get("cpt"):
        s += "-c"
    if info.get("sp"):
        s += "-sp"
    return s
