"""Small helpers shared by the profilers and the entry points."""
from __future__ import annotations

from typing import List, Optional

import torch.distributed as dist


def profiling_group_ranks(world_size: int, group_size: int, consecutive: bool) -> List[List[int]]:
    """Rank lists of the tensor-parallel-like groups used by the hardware sweep: consecutive groups are
    ``[k*g, (k+1)*g)``; strided groups take every ``world/g``-th rank (the layout of ``global_tp_consec=0``)."""
    n = world_size // group_size
    if consecutive:
        return [list(range(i * group_size, (i + 1) * group_size)) for i in range(n)]
    return [list(range(i, world_size, n)) for i in range(n)]


def gen_profiling_groups(group_size: int, consecutive: bool):
    """Create every group of the layout (collective on all ranks) and return this rank's
    (galvatron/utils/training_utils.py:43-60)."""
    world, rank = dist.get_world_size(), dist.get_rank()
    mine: Optional[object] = None
    for ranks in profiling_group_ranks(world, group_size, consecutive):
        g = dist.new_group(ranks=ranks)
        if rank in ranks:
            mine = g
    return mine


def set_seed(seed: int = 1234):
    from ..runtime.initialize import set_seed as _s

    _s(seed)


def print_loss(loss, ep: int, iter: int):
    if loss is None:
        return
    if ep == -1:
        print("(Iteration %d): Loss = %.3f" % (iter, float(loss)))
    else:
        print("[Epoch %d] (Iteration %d): Loss = %.3f" % (ep, iter, float(loss)))


def divide(numerator: int, denominator: int) -> int:
    if numerator % denominator:
        raise ValueError("%d is not divisible by %d" % (numerator, denominator))
    return numerator // denominator


class VocabUtility:
    """Vocabulary range ``[first, last)`` owned by a rank of a vocab-parallel group
    (galvatron/core/runtime/tensor_parallel/utils.py:32-82)."""

    @staticmethod
    def vocab_range_from_per_partition_vocab_size(per_partition: int, rank: int, world_size: int = None):
        return rank * per_partition, (rank + 1) * per_partition

    @staticmethod
    def vocab_range_from_global_vocab_size(global_vocab: int, rank: int, world_size: int):
        return VocabUtility.vocab_range_from_per_partition_vocab_size(divide(global_vocab, world_size), rank, world_size)
