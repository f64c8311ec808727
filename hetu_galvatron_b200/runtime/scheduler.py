"""Learning-rate / weight-decay schedules and micro-batch calculators.

``OptimizerParamScheduler`` is stepped in *samples* (``step(increment=global_batch_size)``): linear warm-up
from ``init_lr`` to ``max_lr`` over ``lr_warmup_steps``, then constant / linear / cosine / inverse-square-root /
WSD (warm-up, stable, decay with an exponential, linear or cosine tail) decay to ``min_lr`` over
``lr_decay_steps``; weight decay ramps constant / linear / cosine from ``start_wd`` to ``end_wd``.  ``state_dict``
round-trips through ``opt_param_scheduler.json`` in a checkpoint.

Capability parity: galvatron/core/runtime/optimizer/param_scheduler.py:45-100 (construction), :102-281
(schedules), :283-385 (state), optimizer/num_microbatches_calculator.py:266-508 (constant / ramp-up batch size).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional


class OptimizerParamScheduler:
    def __init__(self, optimizer, init_lr: float, max_lr: float, min_lr: float, lr_warmup_steps: int,
                 lr_decay_steps: int, lr_decay_style: str, start_wd: float, end_wd: float, wd_incr_steps: int,
                 wd_incr_style: str, use_checkpoint_opt_param_scheduler: bool = True,
                 override_opt_param_scheduler: bool = False, wsd_decay_steps: Optional[int] = None,
                 lr_wsd_decay_style: Optional[str] = None):
        self.optimizer = optimizer
        self.init_lr, self.max_lr, self.min_lr = init_lr, float(max_lr), min_lr
        if not (0.0 <= self.min_lr <= self.max_lr and self.init_lr <= self.max_lr):
            raise AssertionError("need 0 <= min_lr <= max_lr and init_lr <= max_lr")
        self.lr_warmup_steps, self.lr_decay_steps = lr_warmup_steps, lr_decay_steps
        if self.lr_decay_steps <= 0 or self.lr_warmup_steps >= self.lr_decay_steps:
            raise AssertionError("need 0 <= lr_warmup_steps < lr_decay_steps")
        self.lr_decay_style, self.wsd_decay_steps, self.lr_wsd_decay_style = lr_decay_style, wsd_decay_steps, lr_wsd_decay_style
        if lr_decay_style == "WSD" and wsd_decay_steps is None:
            raise AssertionError("WSD needs wsd_decay_steps")
        self.start_wd, self.end_wd, self.wd_incr_steps, self.wd_incr_style = start_wd, end_wd, wd_incr_steps, wd_incr_style
        if not (0.0 <= start_wd <= end_wd):
            raise AssertionError("need 0 <= start_wd <= end_wd")
        self.override = override_opt_param_scheduler
        self.use_checkpoint = use_checkpoint_opt_param_scheduler
        if self.override and self.use_checkpoint:
            raise AssertionError("override and use-checkpoint are exclusive")
        self.num_steps = 0
        self.step(0)

    def get_wd(self) -> float:
        if self.num_steps > self.wd_incr_steps:
            return self.end_wd
        if self.wd_incr_style == "constant":
            return self.end_wd
        r = self.num_steps / self.wd_incr_steps
        if self.wd_incr_style == "linear":
            coeff = r
        elif self.wd_incr_style == "cosine":
            coeff = 0.5 * (math.cos(math.pi * (1 - r)) + 1.0)
        else:
            raise ValueError(self.wd_incr_style)
        return self.start_wd + coeff * (self.end_wd - self.start_wd)

    def get_lr(self, max_lr: Optional[float] = None, min_lr: Optional[float] = None) -> float:
        max_lr = self.max_lr if max_lr is None else max_lr
        min_lr = self.min_lr if min_lr is None else min_lr
        n = self.num_steps
        if self.lr_warmup_steps > 0 and n <= self.lr_warmup_steps:
            return self.init_lr + (max_lr - self.init_lr) * n / self.lr_warmup_steps
        style = self.lr_decay_style
        if style == "constant":
            return max_lr
        if n > self.lr_decay_steps:
            return min_lr
        if style == "inverse-square-root":
            w = max(self.lr_warmup_steps, 1)
            return max(min_lr, max_lr * w ** 0.5 / max(n, 1) ** 0.5)
        span = self.lr_decay_steps - self.lr_warmup_steps
        r = (n - self.lr_warmup_steps) / span
        delta = max_lr - min_lr
        if style == "linear":
            coeff = 1.0 - r
        elif style == "cosine":
            coeff = 0.5 * (math.cos(math.pi * r) + 1.0)
        elif style == "WSD":
            anneal_start = self.lr_decay_steps - self.wsd_decay_steps
            if n <= anneal_start:
                coeff = 1.0
            else:
                wr = (n - anneal_start) / self.wsd_decay_steps
                tail = self.lr_wsd_decay_style or "exponential"
                if tail == "linear":
                    coeff = 1.0 - wr
                elif tail == "cosine":
                    coeff = 0.5 * (math.cos(math.pi * wr) + 1.0)
                else:
                    coeff = 2.0 * math.pow(0.5, wr) - 1.0
        else:
            raise ValueError(style)
        return min_lr + coeff * delta

    def step(self, increment: int):
        self.num_steps += increment
        wd = self.get_wd()
        for g in self.optimizer.param_groups:
            g["lr"] = self.get_lr(g.get("max_lr"), g.get("min_lr")) * g.get("lr_mult", 1.0)
            g["weight_decay"] = wd * g.get("wd_mult", 1.0)

    def state_dict(self) -> Dict:
        return {"max_lr": self.max_lr, "lr_warmup_steps": self.lr_warmup_steps, "num_steps": self.num_steps,
                "lr_decay_style": self.lr_decay_style, "lr_decay_steps": self.lr_decay_steps, "min_lr": self.min_lr,
                "start_wd": self.start_wd, "end_wd": self.end_wd, "wd_incr_style": self.wd_incr_style,
                "wd_incr_steps": self.wd_incr_steps}

    def _pick(self, mine, saved, name):
        if self.override:
            return mine
        if not self.use_checkpoint and mine != saved:
            raise AssertionError("scheduler value for %s differs from the checkpoint (%s vs %s)" % (name, mine, saved))
        return saved

    def load_state_dict(self, sd: Dict):
        self.max_lr = self._pick(self.max_lr, sd.get("max_lr", sd.get("start_lr")), "max_lr")
        self.min_lr = self._pick(self.min_lr, sd["min_lr"], "min_lr")
        self.lr_warmup_steps = self._pick(self.lr_warmup_steps, sd.get("lr_warmup_steps", sd.get("warmup_iter")), "warmup")
        self.lr_decay_steps = self._pick(self.lr_decay_steps, sd.get("lr_decay_steps", sd.get("end_iter")), "decay steps")
        self.lr_decay_style = self._pick(self.lr_decay_style, sd.get("lr_decay_style", sd.get("decay_style")), "decay style")
        if "start_wd" in sd:
            self.start_wd = self._pick(self.start_wd, sd["start_wd"], "start_wd")
            self.end_wd = self._pick(self.end_wd, sd["end_wd"], "end_wd")
            self.wd_incr_steps = self._pick(self.wd_incr_steps, sd["wd_incr_steps"], "wd steps")
            self.wd_incr_style = self._pick(self.wd_incr_style, sd["wd_incr_style"], "wd style")
        self.num_steps = 0
        self.step(sd.get("num_steps", sd.get("num_iters", 0)))


def get_optimizer_param_scheduler(optimizer, args) -> OptimizerParamScheduler:
    """Build the scheduler from ``args.train`` (iteration- or sample-based horizons, warm-up fraction)."""
    t = args.train
    gbsz = t.global_batch_size
    if t.train_iters:
        decay_iters = t.lr_decay_iters if t.lr_decay_iters is not None else t.train_iters
        decay_steps = decay_iters * gbsz
        wd_steps = t.train_iters * gbsz
        wsd_steps = t.lr_wsd_decay_iters * gbsz if t.lr_wsd_decay_iters is not None else None
        warmup = t.lr_warmup_fraction * decay_steps if t.lr_warmup_fraction is not None else (t.lr_warmup_iters or 0) * gbsz
    elif t.train_samples:
        decay_steps = t.lr_decay_samples if t.lr_decay_samples is not None else t.train_samples
        wd_steps = t.train_samples
        wsd_steps = t.lr_wsd_decay_samples
        warmup = t.lr_warmup_fraction * decay_steps if t.lr_warmup_fraction is not None else (t.lr_warmup_samples or 0)
    else:
        raise ValueError("either train_iters or train_samples must be set")
    start_wd = t.start_weight_decay if t.start_weight_decay is not None else t.weight_decay
    end_wd = t.end_weight_decay if t.end_weight_decay is not None else t.weight_decay
    return OptimizerParamScheduler(
        optimizer, init_lr=t.lr_warmup_init, max_lr=t.lr, min_lr=t.min_lr if t.min_lr is not None else 0.0,
        lr_warmup_steps=int(warmup), lr_decay_steps=int(decay_steps), lr_decay_style=t.lr_decay_style,
        start_wd=start_wd, end_wd=end_wd, wd_incr_steps=int(wd_steps), wd_incr_style=t.weight_decay_incr_style,
        use_checkpoint_opt_param_scheduler=t.use_checkpoint_opt_param_scheduler,
        override_opt_param_scheduler=t.override_opt_param_scheduler, wsd_decay_steps=wsd_steps,
        lr_wsd_decay_style=t.lr_wsd_decay_style)


# ---- micro-batch calculators -------------------------------------------------------------------------------
class ConstantNumMicroBatchesCalculator:
    def __init__(self, global_batch_size: int, micro_batch_size: int, data_parallel_size: int):
        per_step = micro_batch_size * data_parallel_size
        if global_batch_size % per_step:
            raise AssertionError("global batch %d is not divisible by micro batch %d x dp %d" % (
                global_batch_size, micro_batch_size, data_parallel_size))
        self.num_micro_batches = global_batch_size // per_step
        self.current_global_batch_size = global_batch_size
        self.micro_batch_size = micro_batch_size

    def get(self):
        return self.num_micro_batches

    def get_current_global_batch_size(self):
        return self.current_global_batch_size

    def update(self, consumed_samples, consistency_check=True):
        pass


class RampupBatchsizeNumMicroBatchesCalculator:
    """Global batch grows from ``start`` by ``increment`` every ``ramp_samples / steps`` consumed samples."""

    def __init__(self, global_batch_size, micro_batch_size, data_parallel_size, start_batch_size, batch_size_increment,
                 ramup_samples):
        self.global_batch_size, self.micro_batch_size, self.dp = global_batch_size, micro_batch_size, data_parallel_size
        self.per_step = micro_batch_size * data_parallel_size
        self.start, self.incr, self.ramp = start_batch_size, batch_size_increment, ramup_samples
        diff = global_batch_size - start_batch_size
        if diff < 0 or diff % batch_size_increment:
            raise AssertionError("global batch must be start + k * increment")
        n = diff // batch_size_increment
        self.samples_per_increment = ramup_samples / n if n > 0 else 0
        self.update(0, False)

    def update(self, consumed_samples, consistency_check=True):
        if consumed_samples > self.ramp or self.samples_per_increment == 0:
            cur = self.global_batch_size
        else:
            cur = min(self.global_batch_size, self.start + int(consumed_samples / self.samples_per_increment) * self.incr)
        if consistency_check and cur % self.per_step:
            raise AssertionError("current global batch %d not divisible by micro batch x dp = %d" % (cur, self.per_step))
        self.current_global_batch_size = cur
        self.num_micro_batches = max(1, cur // self.per_step)

    def get(self):
        return self.num_micro_batches

    def get_current_global_batch_size(self):
        return self.current_global_batch_size


def build_num_microbatches_calculator(global_batch_size, micro_batch_size, data_parallel_size,
                                      rampup_batch_size: Optional[List[int]] = None):
    if rampup_batch_size is None:
        return ConstantNumMicroBatchesCalculator(global_batch_size, micro_batch_size, data_parallel_size)
    if len(rampup_batch_size) != 3:
        raise AssertionError("rampup_batch_size = [start, increment, ramp_samples]")
    return RampupBatchsizeNumMicroBatchesCalculator(global_batch_size, micro_batch_size, data_parallel_size,
                                                    *[int(x) for x in rampup_batch_size])
