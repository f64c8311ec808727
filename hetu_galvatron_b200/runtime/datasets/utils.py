"""Dataset helpers of the reference's ``datasets/megatron/utils.py`` (:21-87): the split enum, weight normalisation
and the build of the native index helpers."""
from __future__ import annotations

from enum import Enum
from typing import List, Sequence


class Split(Enum):
    train = 0
    valid = 1
    test = 2


def normalize(weights: Sequence[float]) -> List[float]:
    from .blended import normalize as _n

    return _n(weights)


