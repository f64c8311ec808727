"""The training loop shared by the dense and MoE entry points.

Per iteration: next batch (pinned host memory -> device, asynchronous), forward-backward through the engine,
gradient reduction + exact global-norm clipping + fused AdamW (:class:`ShardedAdamW.step`), schedule step, profiler
hooks, periodic checkpoint, re-run validation of the loss when the state machine is enabled.  The loss is read on
the host once per iteration (for logging and validation), which is the only forced synchronisation.

Capability parity: galvatron/models/gpt/train_dist.py:21-73, models/moe/train_dist.py:36-111 (adds the
load-balancing loss report), core/runtime/optimizer/utils.py:43-71 (optimizer + scheduler construction).
"""
from __future__ import annotations

import os
import sys
from typing import Optional

import torch
import torch.distributed as dist

from ..config.model_config import model_layer_configs, model_name, resolve_model_config
from ..profiler.runtime import RuntimeProfiler
from . import checkpoint as ckpt
from .data import get_batch, get_train_valid_test_data_iterators
from .engine import build_model
from .optimizer import ShardedAdamW
from .rerun import RerunDataIterator, get_rerun_state_machine
from .scheduler import get_optimizer_param_scheduler


def _nvtx_push(name: str):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)


def _nvtx_pop():
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_pop()


def _update_expert_bias(model, args):
    """Aux-loss-free load balancing: nudge every router's selection bias after the optimizer step."""
    m = args.model
    if not getattr(m, "moe_router_enable_expert_bias", False):
        return
    rate = getattr(m, "moe_router_bias_update_rate", 1e-3) or 1e-3
    for unit in model.model.units:
        router = getattr(unit, "router", None)
        if router is not None and hasattr(router.inner, "update_expert_bias"):
            ctx = router.inner.ctx
            grp = ctx.sdp.group if (ctx.sdp is not None and ctx.sdp.size > 1) else None
            router.inner.update_expert_bias(rate, grp)


def _device_status_code(device) -> int:
    """The device status word of this process (0 = healthy; always 0 without a GPU).  Reading it clears it."""
    if getattr(device, "type", "cpu") != "cuda":
        return 0
    from ..ops import _lib

    return _lib.read_status(clear=True)


def check_device_status(device) -> None:
    """Raise ``KernelError`` on every rank if any kernel of any rank recorded a failure since the last check.

    Every wait inside the kernels (mbarrier, tensor memory, peer flag) gives up after a bounded time, records a code
    in a device status word and lets the kernel unwind with incomplete output.  The loop reads that word once per
    iteration, right after the loss has been read (the device is idle then), and takes the maximum over the ranks,
    so that a step computed from incomplete tiles is rejected everywhere before its parameters are kept or
    checkpointed, and no rank is left waiting in a collective for one that raised."""
    code = _device_status_code(device)
    if code == 0 and getattr(device, "type", "cpu") == "cuda":
        from ..ops import _lib
        from ..parallel import fused_zero

        if _lib.DEBUG_KERNELS and fused_zero.verify_guards():
            code = 6     # something wrote outside a symmetric buffer: same class as a bad argument
    if dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([code], dtype=torch.int32, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        code = int(t.item())
    if code != 0:
        from ..ops import _lib

        raise _lib.KernelError("device status word = %d (%s): the step used incomplete kernel output and is rejected"
                               % (code, _lib._STATUS_NAMES.get(code, "?")))


def get_optimizer_and_param_scheduler(model, args):
    t = args.train
    opt = ShardedAdamW(model.sharded_units, lr=t.lr, betas=(t.adam_beta1, t.adam_beta2), eps=t.adam_eps,
                       weight_decay=t.weight_decay, clip_grad=t.clip_grad or 0.0, device=model.device)
    sched = None
    if t.train_iters or t.train_samples:
        sched = get_optimizer_param_scheduler(opt, args)
    return opt, sched


def get_runtime_profiler(args, model, start_iter: int = 10, end_iter: int = 20) -> RuntimeProfiler:
    prof = RuntimeProfiler(args)
    # raw measurements land in <dir>/configs/, where the model profiler looks for them
    prof.set_profiler_dist(path=os.environ.get("HG_PROFILE_DIR") or os.getcwd(), model_layer_configs=model_layer_configs(args), model_name=model_name(args),
                           start_iter=start_iter, end_iter=end_iter)
    return prof


def _profile_window(default):
    """``HG_PROFILE_WINDOW="start,end"`` moves the iterations that the runtime profiler times (default 10..20)."""
    v = os.environ.get("HG_PROFILE_WINDOW")
    if not v:
        return default
    a, b = (int(x) for x in v.split(","))
    return a, b


def evaluate(model, data_iterator, iters: int) -> Optional[float]:
    """Mean loss over ``iters`` forward-only batches of ``data_iterator`` (``None`` on ranks without the last pipeline
    stage or when there is nothing to evaluate).  Gradients are neither computed nor touched."""
    if data_iterator is None or iters <= 0:
        return None
    total, n = 0.0, 0
    for _ in range(iters):
        tokens, kw, loss_fn = get_batch(data_iterator, model.device)
        loss = model.forward_backward([tokens], 0, None, loss_fn, labels=kw.get("labels"), loss_mask=kw.get("loss_mask"),
                                      forward_only=True)
        if loss is not None:
            total += float(loss)
            n += 1
    return total / n if n else None


def train(args, max_iters: Optional[int] = None, profile_window=None):
    """Runs ``args.train.train_iters`` iterations (or ``max_iters``); returns the list of per-iteration losses seen
    on this rank (``None`` entries on ranks that do not hold the last pipeline stage)."""
    resolve_model_config(args)
    model = build_model(args)
    rank = dist.get_rank() if dist.is_initialized() else 0
    optimizer, scheduler = get_optimizer_and_param_scheduler(model, args)
    start = 0
    c = args.ckpt
    if c.load is not None:
        if c.distributed_checkpoint:
            it = c.load_iteration or 0
            ckpt.load_distributed_checkpoint(model, optimizer, scheduler, c.load, it)
            start = it
        else:
            ckpt.load_hf_split(model, c.load)
    args.train.iteration = start
    train_it, valid_it, _ = get_train_valid_test_data_iterators(args, model)
    machine = get_rerun_state_machine()
    train_it = RerunDataIterator(train_it)
    profile_window = profile_window or _profile_window((10, 20))
    profiler = get_runtime_profiler(args, model, start_iter=profile_window[0], end_iter=profile_window[1])
    profiler.profile_memory(0, "After creating model")
    total = max_iters if max_iters is not None else (args.train.train_iters or 0)
    if args.train.skip_train:
        total = start      # evaluation / checkpoint conversion only
    gbsz = args.train.global_batch_size
    losses = []
    for it in range(start, total):
        profiler.profile_time_start(it)
        forward_only = bool(args.profile.profile_forward)
        loss = None
        while machine.should_run_forward_backward(train_it):
            _nvtx_push("forward_backward")
            tokens, kw, loss_fn = get_batch(train_it, model.device)
            optimizer.zero_grad()
            loss = model.forward_backward([tokens], it, profiler, loss_fn, labels=kw.get("labels"),
                                          loss_mask=kw.get("loss_mask"), forward_only=forward_only)
            if loss is not None and machine.get_mode().value != "disabled":
                machine.validate_result(loss, machine.is_unexpectedly_large(1e4), "loss", tolerance=0.0, fatal=True)
            _nvtx_pop()
        if not forward_only:
            _nvtx_push("optimizer")
            model.sync_tied_embedding_grads()
            optimizer.step()
            _update_expert_bias(model, args)
            _nvtx_pop()
            if scheduler is not None:
                scheduler.step(increment=gbsz)
        profiler.profile_memory(it, "After optimizer_step")
        lr = optimizer.param_groups[0]["lr"]
        loss_val = float(loss) if loss is not None else None
        check_device_status(model.device)
        losses.append(loss_val)
        if getattr(args.model, "print_loss", 0) and loss_val is not None:
            from ..utils.training_utils import print_loss

            print_loss(loss_val, -1, it)          # the model scripts' per-iteration loss line (`model.print_loss`)
        if loss_val is not None:
            from ..parallel import state as _state

            _state.log_scalars(it + 1, **{"train/loss": loss_val, "train/lr": lr})
        profiler.post_profile_memory(it)
        profiler.profile_time_end(it, loss_val, lr, optimizer.grad_norm() if (optimizer.clip_grad > 0 and not forward_only) else None)
        if args.train.do_valid and args.train.eval_interval and (it + 1) % args.train.eval_interval == 0:
            val = evaluate(model, valid_it, args.train.eval_iters or 0)
            if val is not None:
                from ..parallel import state as _state

                _state.log_scalars(it + 1, **{"validation/loss": val})
                # the loss lives on the last pipeline stage; its last rank reports, like the iteration line
                if not dist.is_initialized() or rank == dist.get_world_size() - 1:
                    print("| Iteration: %6d | validation loss: %.6e |" % (it + 1, val), flush=True)
        save, leave, code = machine.should_checkpoint_and_exit()
        if c.save is not None and (save or (c.save_interval and (it + 1) % c.save_interval == 0)):
            ckpt.save_distributed_checkpoint(model, optimizer, scheduler, it + 1, c.save,
                                             extra={"rerun": machine.state_dict(train_it)})
        if leave:
            if dist.is_initialized():
                dist.barrier()
            sys.exit(code)
        if dist.is_initialized():
            dist.barrier()
    return losses
