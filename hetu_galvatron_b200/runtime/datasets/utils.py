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


def compile_helpers() -> str:
    """Build (if stale) and return the path of the native dataset helpers (``csrc/host/dataset_helpers.cpp``).  The
    reference shells out to ``make`` in its source tree; here the package's own build step does it."""
    from ...csrc import build as _build

    built = _build.build_host()
    for path in built:
        if "dataset_helpers" in str(path):
            return str(path)
    raise RuntimeError("the dataset helpers were not built: %s" % (built,))
