"""Small runtime helpers under the names the reference's users know
(galvatron/core/runtime/utils/utils.py:28-52, 54-70, 97-152, 170-192, 295-337).

Nested attribute access that sees through this framework's unit wrappers, rank-filtered printing / logging, torch
version checks, the zig-zag slice of a batch for context parallelism, the loss average over the data-parallel group
and the offsets of the norm parameters inside a unit's flat buffer.
"""
from __future__ import annotations

import logging
from functools import reduce
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
from packaging.version import Version


# ---- nested attributes -----------------------------------------------------------------------------------------
def _unwrap(obj):
    """``UnitWrapper`` (the ZeRO / checkpointing wrapper around a unit's module) is transparent, as FSDP is in the
    reference."""
    from ..parallel.zero import UnitWrapper

    return obj.inner if isinstance(obj, UnitWrapper) else obj


def rgetattr(obj, attr: str):
    """``rgetattr(m, "a.b.c")`` = ``m.a.b.c``; the empty path returns ``obj``."""
    if attr == "":
        return obj
    return reduce(lambda o, name: getattr(_unwrap(o), name), [obj] + attr.split("."))


def rsetattr(obj, attr: str, val) -> None:
    pre, _, post = attr.rpartition(".")
    setattr(_unwrap(rgetattr(obj, pre)) if pre else obj, post, val)


def rhasattr(obj, attr: str) -> bool:
    try:
        rgetattr(obj, attr)
        return True
    except AttributeError:
        return False


# ---- rank-filtered output ---------------------------------------------------------------------------------------
def _rank() -> int:
    import torch.distributed as dist

    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def print_rank_0(message) -> None:
    if _rank() == 0:
        print(message, flush=True)


def log_single_rank(logger: logging.Logger, *args: Any, rank: int = 0, **kwargs: Any) -> None:
    """``logger.log(*args, **kwargs)`` on one rank only (every rank when torch.distributed is not initialised)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == rank:
        logger.log(*args, **kwargs)


# ---- versions -----------------------------------------------------------------------------------------------------
def get_torch_version() -> Version:
    try:
        return Version(torch.__version__.split("+")[0])
    except Exception:
        return Version("0.0.0")


def is_torch_min_version(version: str, check_equality: bool = True) -> bool:
    have, want = get_torch_version(), Version(version)
    return have >= want if check_equality else have > want


# ---- batches ------------------------------------------------------------------------------------------------------
def get_batch_on_this_cp_rank(batch: Dict[str, Optional[torch.Tensor]], cp_size: int, cp_rank: int) -> Dict:
    """Zig-zag split of every tensor of ``batch`` along its sequence dimension (dimension 1; 2 for
    ``attention_mask``): the sequence is cut into ``2 * cp_size`` chunks and rank ``r`` keeps chunks ``r`` and
    ``2 * cp_size - 1 - r``, which balances the causal-attention work."""
    if cp_size <= 1:
        return batch
    out = {}
    for key, val in batch.items():
        if val is None:
            out[key] = None
            continue
        d = 2 if key == "attention_mask" else 1
        v = val.view(*val.shape[:d], 2 * cp_size, val.shape[d] // (2 * cp_size), *val.shape[d + 1:])
        idx = torch.tensor([cp_rank, 2 * cp_size - 1 - cp_rank], device=val.device)
        v = v.index_select(d, idx)
        out[key] = v.reshape(*val.shape[:d], -1, *val.shape[d + 1:])
    return out


def get_batch_on_this_tp_rank(data_iterator, group, device, shape):
    """Only the first rank of the tensor-parallel ``group`` reads from ``data_iterator``; the others receive the
    tokens and labels by broadcast.  Returns ``(tokens, {"labels": ...})``."""
    from ..runtime.data import broadcast_batch, get_batch

    tokens, kw = None, {}
    if group is None or group.size == 1 or group.rank == 0:
        tokens, kw, _ = get_batch(data_iterator, device)
    return broadcast_batch(tokens, kw, group, device, shape)


def average_losses_across_data_parallel_group(losses: Sequence[torch.Tensor], group=None) -> torch.Tensor:
    """Mean over the ranks of ``group`` (a ``CommGroup``; default: the vocabulary layers' data-parallel group) of
    each loss in ``losses``, as one 1-D tensor."""
    import torch.distributed as dist

    if group is None:
        from ..parallel import state

        try:
            group = state.get_vocab_groups()[3]
        except Exception:
            group = None
    avg = torch.cat([l.clone().detach().view(1) for l in losses])
    if group is not None and group.size > 1:
        dist.all_reduce(avg, group=group.group)
        avg = avg / group.size
    return avg


# ---- norm parameters inside flat buffers -------------------------------------------------------------------------
def get_layernorm_offset(modules: Iterable[torch.nn.Module], layernorm_name: Sequence[str] = ()) -> Tuple[List, List]:
    """For every module: element offsets and sizes, in ``named_parameters`` order, of the parameters that belong to a
    sub-module whose name contains one of ``layernorm_name`` (these are replicated over tensor-parallel ranks and
    their gradients need the extra reduction)."""
    total_off, total_size = [], []
    for module in modules:
        offs, sizes, offset = [], [], 0
        for sub_name, sub in _unwrap(module).named_modules(remove_duplicate=False):
            is_ln = any(n in sub_name for n in layernorm_name)
            for _, p in sub.named_parameters(recurse=False):
                if is_ln:
                    offs.append(offset)
                    sizes.append(p.numel())
                offset += p.numel()
        total_off.append(offs)
        total_size.append(sizes)
    return total_off, total_size
