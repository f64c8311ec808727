"""Device-memory reporting helpers (galvatron/utils/memory_utils.py)."""
from __future__ import annotations

import torch


def _mb(x: int) -> float:
    return x / 2 ** 20


def print_peak_memory(prefix: str, device, kind: str = "allocated"):
    if not torch.cuda.is_available():
        return None
    if kind == "allocated":
        cur, peak = torch.cuda.memory_allocated(device), torch.cuda.max_memory_allocated(device)
    else:
        cur, peak = torch.cuda.memory_reserved(device), torch.cuda.max_memory_reserved(device)
    print("%s: %.2f MB %s, peak %.2f MB" % (prefix, _mb(cur), kind, _mb(peak)))
    return _mb(cur), _mb(peak)


def print_param_num(model) -> int:
    n = sum(p.numel() for p in model.parameters())
    print("Total number of parameters on this rank: %.2f M" % (n / 1e6))
    return n
