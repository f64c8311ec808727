"""Rerun state machine: attribute an unexpected result (NaN / spike) to a transient fault, a persistent fault
of this device, or a genuinely correct computation -- by re-running the step.

Protocol per training step (the loop drives it):

    while rsm.should_run_forward_backward(data_iterator):
        loss = forward_backward(...)                      # inside: rsm.validate_result(loss, rejection_func=...)
    should_ckpt, should_exit, code = rsm.should_checkpoint_and_exit()

1. *Initial run.*  ``validate_result`` records the value; a rejected value arms a re-run.
2. *Re-run in place* with the very same batches (``RerunDataIterator`` replays them).  A different value means
   the fault did not repeat: **transient error** -- logged, training goes on.  The same value cannot be told
   apart yet: the step is checkpointed and the job asked to restart elsewhere (exit code 16).
3. *Re-run from the checkpoint* (ideally on another device).  The same value again: the computation is
   **correct** (the spike is real); a different one: the first device has a **persistent error** (exit code 17
   when the check was fatal).

Every decision is agreed between ranks with a MAX all-reduce of one flag, so all ranks take the same branch.
``RerunErrorInjector`` flips results on the host at a configurable rate to exercise all three diagnoses;
nothing is ever injected on the device.  ``REPORT_DETERMINISM_STATS`` mode re-runs every step and keeps
statistics of the relative difference.

Capability parity: galvatron/core/runtime/utils/rerun_state_machine.py:34-37 (exit codes), :72-109 (modes,
states), :308-371 (rank agreement), :374-432 (checkpoint / exit decision), :434-649 (``validate_result``),
:930-986 (tracker file), :989-1055 (replaying iterator), :1058-1140 (``QuickStats``), :1143-1238 (injector).
"""
from __future__ import annotations

import enum
import json
import math
import os
import random
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple

import torch

EXIT_CODE_RESUME_TO_DISAMBIGUATE = 16
EXIT_CODE_FAILED_ON_RESULT_VALIDATION = 17


class RerunMode(str, enum.Enum):
    DISABLED = "disabled"
    VALIDATE_RESULTS = "validate_results"
    REPORT_DETERMINISM_STATS = "report_determinism_stats"


class RerunState(enum.Enum):
    NOT_RUNNING_YET = 0
    INITIAL_RUN = 1
    RERUNNING_IN_PLACE = 2
    WILL_RERUN_FROM_CHECKPOINT = 3
    RERUNNING_FROM_CHECKPOINT = 4
    RERUNNING_AGAIN_FROM_CHECKPOINT = 5


class RerunDiagnostic(str, enum.Enum):
    CORRECT_RESULT = "correct_result"
    TRANSIENT_ERROR = "transient_error"
    PERSISTENT_ERROR = "persistent_error"


class QuickStats:
    """Running max / mean / median-ish summary over a bounded window."""

    def __init__(self, max_size: int = 100000):
        self.max_size, self.samples, self.pos, self.zero_cnt, self.max = max_size, [], 0, 0, 0.0

    def record(self, x: float):
        if x == 0.0:
            self.zero_cnt += 1
            return
        if len(self.samples) < self.max_size:
            self.samples.append(x)
        else:
            self.samples[self.pos] = x
            self.pos = (self.pos + 1) % self.max_size
        self.max = max(self.max, x)

    def combine(self, others: List["QuickStats"]):
        for o in others:
            self.zero_cnt += o.zero_cnt
            self.max = max(self.max, o.max)
            self.samples = (self.samples + o.samples)[-self.max_size:]

    def print_stats(self) -> str:
        n = len(self.samples)
        if n == 0:
            return "no non-zero samples (%d zeros)" % self.zero_cnt
        s = sorted(self.samples)
        return "zeros %d, n %d, max %.3g, mean %.3g, median %.3g, p95 %.3g" % (
            self.zero_cnt, n, self.max, sum(s) / n, s[n // 2], s[min(n - 1, int(0.95 * n))])


class RerunDataIterator:
    """Wraps a data iterator, remembers what it handed out during a step and replays it on a re-run."""

    def __init__(self, iterable: Iterable):
        self.it = iter(iterable)
        self.saved: List[Any] = []
        self.replaying = False
        self.pos = 0

    def __iter__(self):
        return self

    def __next__(self):
        if self.replaying:
            if self.pos < len(self.saved):
                item = self.saved[self.pos]
                self.pos += 1
                return item
            self.replaying = False
        item = next(self.it)
        self.saved.append(item)
        return item

    def rewind(self):
        self.replaying, self.pos = True, 0

    def advance(self):
        self.saved, self.replaying, self.pos = [], False, 0

    def state_dict(self):
        return {"saved": self.saved, "replaying": self.replaying, "pos": self.pos}

    def load_state_dict(self, sd):
        self.saved, self.replaying, self.pos = sd["saved"], sd["replaying"], sd["pos"]


class RerunErrorInjector:
    """Host-side fault injection: with probability ``rate / 1e6`` per validation, one rank's result is replaced
    so that the state machine reaches the chosen diagnosis."""

    def __init__(self, error_injection_rate: int = 0, error_injection_type: RerunDiagnostic = RerunDiagnostic.TRANSIENT_ERROR,
                 seed: int = 0):
        self.rate, self.type = error_injection_rate, RerunDiagnostic(error_injection_type)
        self.rng = random.Random(seed)
        self.should_inject = False
        self.injected_rank: Optional[int] = None
        self.injected_device: Optional[int] = None

    def maybe_arm(self, rank: int, device: int):
        if self.rate > 0 and not self.should_inject and self.rng.randint(0, 999999) < self.rate:
            self.should_inject, self.injected_rank, self.injected_device = True, rank, device

    def maybe_inject(self, result, state: RerunState, rank: int, device: int):
        if not self.should_inject or rank != self.injected_rank:
            return result
        if self.type == RerunDiagnostic.TRANSIENT_ERROR:
            hit = state == RerunState.INITIAL_RUN          # does not repeat
            if state != RerunState.INITIAL_RUN:
                self.should_inject = False                  # one fault per arming
        elif self.type == RerunDiagnostic.PERSISTENT_ERROR:
            hit = device == self.injected_device            # repeats only on the original device
        else:
            hit = True                                      # repeats everywhere: the value is "real"
        return float("nan") if hit else result

    def state_dict(self):
        return {"rate": self.rate, "type": self.type.value, "should_inject": self.should_inject,
                "rank": self.injected_rank, "device": self.injected_device}

    def load_state_dict(self, sd):
        self.rate, self.type, self.should_inject = sd["rate"], RerunDiagnostic(sd["type"]), sd["should_inject"]
        self.injected_rank, self.injected_device = sd["rank"], sd["device"]


def _agree(flag: bool) -> bool:
    """True on every rank if true on any rank (host-side decision; a CPU tensor on gloo, CUDA on NCCL)."""
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size() == 1:
        return flag
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return bool(t.item())


class RerunStateMachine:
    def __init__(self, mode: RerunMode = RerunMode.DISABLED, error_injector: Optional[RerunErrorInjector] = None,
                 result_rejected_tracker_filename: Optional[str] = None):
        self.mode = RerunMode(mode)
        self.state = RerunState.NOT_RUNNING_YET
        self.injector = error_injector or RerunErrorInjector()
        self.tracker_file = result_rejected_tracker_filename
        self.current_iteration = -1
        self.rerun_requested = False
        self.checkpoint_requested = False
        self.restart_again_requested = False
        self.continue_requested = False
        self.saved_results: Dict[int, Any] = {}
        self.validation_counts = 0
        self.failed_validation_call: Optional[int] = None
        self.initial_result: Any = None
        self.suspicious_device: Optional[int] = None
        self.suspicious_node: Optional[str] = None
        self.fatal = True
        self.stats: Dict[str, QuickStats] = {}
        self.log: List[Tuple[int, str, str]] = []
        self.data_iterators: List[RerunDataIterator] = []

    # ---- helpers -----------------------------------------------------------------------------------------
    @staticmethod
    def _rank() -> int:
        import torch.distributed as dist

        return dist.get_rank() if dist.is_initialized() else 0

    @staticmethod
    def _device() -> int:
        return torch.cuda.current_device() if torch.cuda.is_available() else -1

    def get_mode(self):
        return self.mode

    def set_mode(self, mode):
        self.mode = RerunMode(mode)

    def _record(self, diag: RerunDiagnostic, msg: str):
        self.log.append((self.current_iteration, diag.value, msg))
        if self._rank() == 0:
            print("[rerun] iteration %d: %s (%s)" % (self.current_iteration, diag.value, msg))
        if self.tracker_file and self._rank() == 0:
            entries = []
            if os.path.exists(self.tracker_file):
                entries = json.load(open(self.tracker_file))
            entries.append({"iteration": self.current_iteration, "diagnostic": diag.value, "message": msg})
            with open(self.tracker_file, "w") as f:
                json.dump(entries, f)

    # ---- loop control ------------------------------------------------------------------------------------------
    def should_run_forward_backward(self, data_iterator=None) -> bool:
        """Call in a ``while`` around the step's forward-backward.  Returns True for the initial run and for
        each requested re-run, False when the step is settled."""
        its = data_iterator if isinstance(data_iterator, (list, tuple)) else [data_iterator]
        self.data_iterators = [it for it in its if isinstance(it, RerunDataIterator)]
        if self.mode == RerunMode.DISABLED:
            if self.state == RerunState.NOT_RUNNING_YET:
                self.state = RerunState.INITIAL_RUN
                self.current_iteration += 1
                return True
            self.state = RerunState.NOT_RUNNING_YET
            for it in self.data_iterators:
                it.advance()
            return False
        if self.state == RerunState.NOT_RUNNING_YET:
            self.state = RerunState.INITIAL_RUN
            self.current_iteration += 1
            self.validation_counts, self.rerun_requested, self.saved_results = 0, False, {}
            self.injector.maybe_arm(self._rank(), self._device())
            return True
        if self.state == RerunState.WILL_RERUN_FROM_CHECKPOINT:
            # restored from a checkpoint: run the suspicious step again (possibly on another device)
            self.state = RerunState.RERUNNING_FROM_CHECKPOINT
            self.validation_counts = 0
            for it in self.data_iterators:
                it.rewind()
            return True
        if self.state == RerunState.INITIAL_RUN:
            want = self.rerun_requested or self.mode == RerunMode.REPORT_DETERMINISM_STATS
            if _agree(want):
                self.state = RerunState.RERUNNING_IN_PLACE
                self.validation_counts = 0
                for it in self.data_iterators:
                    it.rewind()
                return True
        elif self.state == RerunState.RERUNNING_IN_PLACE:
            if _agree(self.checkpoint_requested):
                self.checkpoint_requested = True
                self.state = RerunState.WILL_RERUN_FROM_CHECKPOINT
                return False  # the caller checkpoints and exits; the data iterators stay rewound in the state
        elif self.state == RerunState.RERUNNING_FROM_CHECKPOINT:
            if _agree(self.restart_again_requested):
                self.state = RerunState.RERUNNING_AGAIN_FROM_CHECKPOINT
        # step settled
        self.state = RerunState.NOT_RUNNING_YET
        self.rerun_requested = False
        for it in self.data_iterators:
            it.advance()
        return False

    def should_checkpoint_and_exit(self) -> Tuple[bool, bool, int]:
        """(save a checkpoint now?, exit now?, exit code)."""
        if self.mode == RerunMode.DISABLED:
            return False, False, 0
        if self.state == RerunState.WILL_RERUN_FROM_CHECKPOINT and self.checkpoint_requested:
            self.checkpoint_requested = False
            return True, True, EXIT_CODE_RESUME_TO_DISAMBIGUATE
        if _agree(self.failed_validation_call is not None and self.fatal and
                  any(d == RerunDiagnostic.PERSISTENT_ERROR.value for _, d, _ in self.log[-1:])):
            return False, True, EXIT_CODE_FAILED_ON_RESULT_VALIDATION
        return False, False, 0

    # ---- validation ------------------------------------------------------------------------------------------------
    def validate_result(self, result, rejection_func: Callable[[Any], bool], message: str = "unexpected result",
                        comparison_func: Optional[Callable[[Any, Any], float]] = None, tolerance: float = 0.0,
                        fatal: bool = True):
        """Check ``result`` (a float or 0-dim tensor read on the host) with ``rejection_func``; drives the
        re-run protocol described in the module docstring."""
        if self.mode == RerunMode.DISABLED:
            return
        if self.state == RerunState.NOT_RUNNING_YET:
            raise RuntimeError("validate_result must be called inside the should_run_forward_backward loop")
        self.validation_counts += 1
        call = self.validation_counts
        value = result.item() if torch.is_tensor(result) else result
        value = self.injector.maybe_inject(value, self.state, self._rank(), self._device())
        compare = comparison_func or _relative_difference
        if self.state == RerunState.INITIAL_RUN:
            self.saved_results[call] = value
            if self.mode == RerunMode.VALIDATE_RESULTS and rejection_func(value):
                self.rerun_requested, self.failed_validation_call = True, call
                self.initial_result, self.fatal = value, fatal
                self.suspicious_device, self.suspicious_node = self._device(), os.uname().nodename
            return
        if self.state == RerunState.RERUNNING_IN_PLACE:
            first = self.saved_results.get(call)
            diff = compare(first, value)
            if self.mode == RerunMode.REPORT_DETERMINISM_STATS:
                self.stats.setdefault(message, QuickStats()).record(diff)
                return
            if call != self.failed_validation_call:
                return
            if diff > tolerance:
                self._record(RerunDiagnostic.TRANSIENT_ERROR, "%s: %r on the first run, %r on the re-run" % (message, first, value))
                self.failed_validation_call = None
            else:
                self.checkpoint_requested = True   # reproducible here: needs another device to tell apart
            return
        if self.state in (RerunState.RERUNNING_FROM_CHECKPOINT, RerunState.RERUNNING_AGAIN_FROM_CHECKPOINT):
            if call != self.failed_validation_call:
                return
            diff = compare(self.initial_result, value)
            same_device = (self._device() == self.suspicious_device and os.uname().nodename == self.suspicious_node)
            if diff <= tolerance and same_device and self.state == RerunState.RERUNNING_FROM_CHECKPOINT:
                # nothing learnt on the same device: ask for one more restart elsewhere
                self.restart_again_requested = True
                self._record(RerunDiagnostic.CORRECT_RESULT, "%s reproduced on the same device; treated as correct" % message)
            elif diff <= tolerance:
                self._record(RerunDiagnostic.CORRECT_RESULT, "%s reproduced on another device: the value is real" % message)
            else:
                self._record(RerunDiagnostic.PERSISTENT_ERROR, "%s: %r on device %s, %r elsewhere" % (
                    message, self.initial_result, self.suspicious_device, value))
            if not self.restart_again_requested:
                self.failed_validation_call = None if diff <= tolerance else self.failed_validation_call

    def is_unexpectedly_large(self, threshold: float, context: str = "loss"):
        return lambda x: (x != x) or math.isinf(x) or abs(x) > threshold

    # ---- persistence ------------------------------------------------------------------------------------------------
    def state_dict(self, data_iterator=None) -> Dict:
        its = data_iterator if isinstance(data_iterator, (list, tuple)) else [data_iterator]
        return {"mode": self.mode.value, "state": self.state.value, "current_iteration": self.current_iteration,
                "failed_validation_call": self.failed_validation_call, "initial_result": self.initial_result,
                "suspicious_device": self.suspicious_device, "suspicious_node": self.suspicious_node,
                "fatal": self.fatal, "injector": self.injector.state_dict(), "log": self.log,
                "data_iterators": [it.state_dict() for it in its if isinstance(it, RerunDataIterator)]}

    def load_state_dict(self, sd: Dict, data_iterator=None):
        self.mode, self.state = RerunMode(sd["mode"]), RerunState(sd["state"])
        self.current_iteration = sd["current_iteration"]
        self.failed_validation_call, self.initial_result = sd["failed_validation_call"], sd["initial_result"]
        self.suspicious_device, self.suspicious_node = sd["suspicious_device"], sd["suspicious_node"]
        self.fatal, self.log = sd["fatal"], [tuple(x) for x in sd["log"]]
        self.injector.load_state_dict(sd["injector"])
        its = data_iterator if isinstance(data_iterator, (list, tuple)) else [data_iterator]
        for it, s in zip([i for i in its if isinstance(i, RerunDataIterator)], sd.get("data_iterators", [])):
            it.load_state_dict(s)


def _relative_difference(a, b) -> float:
    if a is None or b is None:
        return float("inf")
    if a != a and b != b:
        return 0.0
    if a != a or b != b or math.isinf(a) or math.isinf(b):
        return 0.0 if a == b else float("inf")
    return abs(a - b) / max(abs(a), abs(b), 1e-30)


def get_skipped_iterations_from_tracker_file(path: str) -> List[int]:
    """Iterations whose result was rejected and finally judged real (to be skipped on the next run)."""
    if not path or not os.path.exists(path):
        return []
    return sorted({e["iteration"] for e in json.load(open(path)) if e["diagnostic"] == RerunDiagnostic.CORRECT_RESULT.value})


_MACHINE: Optional[RerunStateMachine] = None


def initialize_rerun_state_machine(**kwargs) -> RerunStateMachine:
    global _MACHINE
    _MACHINE = RerunStateMachine(**kwargs)
    return _MACHINE


def get_rerun_state_machine() -> RerunStateMachine:
    global _MACHINE
    if _MACHINE is None:
        _MACHINE = RerunStateMachine()
    return _MACHINE


def destroy_rerun_state_machine():
    global _MACHINE
    _MACHINE = None
