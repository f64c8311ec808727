"""Named random-number streams for hybrid parallelism.

Dropout inside a tensor-parallel region must differ across the ranks of the group (each holds a different slice),
while dropout outside it must agree across them.  ``RNGStatesTracker`` keeps one generator state per name;
``with tracker.fork(name):`` runs a region on that stream and puts the default stream back afterwards.  Works for
CUDA and for CPU generators (the CPU path serves the gloo tests).

``set_seed_with_group(tp_groups, tp_and_ep_groups, seed)`` registers the streams the way the reference does
(galvatron/core/runtime/tensor_parallel/random.py:120-226, :279-317): ``data-parallel-rng`` = ``seed``;
one ``model-parallel-rng-<g>`` per distinct tensor-parallel group size ``g`` seeded ``seed + 917 + 100*k + rank_in_group``
(``k`` counts distinct sizes in registration order); likewise ``expert-parallel-rng-<g>`` per tensor x expert group size.

Parameter initialisation in this framework does not depend on these streams: every parameter is drawn from a
generator keyed by (seed, parameter name) and then sliced, so the initial weights are identical under every
strategy (``models/modules.py``).
"""
from __future__ import annotations

import contextlib
from typing import Dict, Iterable, Optional

import torch

DATA_PARALLEL = "data-parallel-rng"
MODEL_PARALLEL = "model-parallel-rng"
EXPERT_PARALLEL = "expert-parallel-rng"


def _get_state(cuda: bool):
    return torch.cuda.get_rng_state() if cuda else torch.get_rng_state()


def _set_state(state, cuda: bool):
    if cuda:
        torch.cuda.set_rng_state(state)
    else:
        torch.set_rng_state(state)


class RNGStatesTracker:
    def __init__(self, cuda: Optional[bool] = None):
        self.cuda = torch.cuda.is_available() if cuda is None else cuda
        self.reset()

    def reset(self):
        self.states_: Dict[str, torch.Tensor] = {}
        self.seeds_ = set()

    def is_initialized(self) -> bool:
        return bool(self.states_)

    def get_states(self) -> Dict[str, torch.Tensor]:
        return {k: v.clone() for k, v in self.states_.items()}

    def set_states(self, states: Dict[str, torch.Tensor]):
        self.states_ = {k: v.clone() for k, v in states.items()}

    def check(self, name: str) -> bool:
        """True when ``name`` is still free."""
        return name not in self.states_

    def add(self, name: str, seed: int):
        if seed in self.seeds_:
            raise ValueError("seed %d already used" % seed)
        if name in self.states_:
            raise ValueError("rng state %s already exists" % name)
        self.seeds_.add(seed)
        keep = _get_state(self.cuda)
        if self.cuda:
            torch.cuda.manual_seed(seed)
        else:
            torch.manual_seed(seed)
        self.states_[name] = _get_state(self.cuda)
        _set_state(keep, self.cuda)

    @contextlib.contextmanager
    def fork(self, name: str = MODEL_PARALLEL):
        if name not in self.states_:
            raise KeyError("rng state %s was never added" % name)
        keep = _get_state(self.cuda)
        _set_state(self.states_[name], self.cuda)
        try:
            yield
        finally:
            self.states_[name] = _get_state(self.cuda)
            _set_state(keep, self.cuda)


_TRACKER: Optional[RNGStatesTracker] = None


def get_rng_tracker() -> RNGStatesTracker:
    global _TRACKER
    if _TRACKER is None:
        _TRACKER = RNGStatesTracker()
    return _TRACKER


# name kept for users of the reference API
get_cuda_rng_tracker = get_rng_tracker


def tensor_parallel_rng_name(group_size: Optional[int] = None) -> str:
    return MODEL_PARALLEL if group_size is None else "%s-%d" % (MODEL_PARALLEL, group_size)


def expert_parallel_rng_name(group_size: Optional[int] = None) -> str:
    return EXPERT_PARALLEL if group_size is None else "%s-%d" % (EXPERT_PARALLEL, group_size)


def set_seed_with_group(tp_groups: Iterable = (), tp_and_ep_groups: Optional[Iterable] = None, seed: int = 1234,
                        cuda: Optional[bool] = None) -> RNGStatesTracker:
    """``tp_groups`` / ``tp_and_ep_groups``: objects with ``.size`` and ``.rank`` (``CommGroup``), one per layer."""
    global _TRACKER
    _TRACKER = RNGStatesTracker(cuda)
    t = _TRACKER
    offset = seed + 917
    if t.cuda:
        torch.cuda.manual_seed(seed)
    else:
        torch.manual_seed(seed)
    t.add(DATA_PARALLEL, seed)
    for prefix, groups in ((MODEL_PARALLEL, tp_groups or ()), (EXPERT_PARALLEL, tp_and_ep_groups or ())):
        for g in groups:
            name = "%s-%d" % (prefix, g.size)
            if t.check(name):
                t.add(name, offset + g.rank)
                offset += 100
    return t
