"""Process-wide state: arguments, tokenizer, metric writers, the named reusable-buffer pool.

Capability parity: galvatron/core/runtime/parallel_state.py:31-141 (globals and writers), :143-306 (group
getters -- here the groups live on the model object, ``GalvatronModel.groups``), core/runtime/utils/utils.py:73-94
(``GlobalMemoryBuffer``).
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

_ARGS = None
_TOKENIZER = None
_TB_WRITER = None
_WANDB = None
_BUFFER = None
_MODEL = None


class GlobalMemoryBuffer:
    """Named flat buffers reused across calls (e.g. the sequence-parallel all-gather target ``"mpu"``): a
    request returns a view of the first ``numel`` elements, growing the allocation when needed."""

    def __init__(self):
        self.buffers: Dict[Tuple[str, torch.dtype, str], torch.Tensor] = {}

    def get_tensor(self, shape, dtype, name: str, device=None) -> torch.Tensor:
        n = int(math.prod(shape))
        dev = device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu")
        key = (name, dtype, str(dev))
        buf = self.buffers.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(n, dtype=dtype, device=dev, requires_grad=False)
            self.buffers[key] = buf
        return buf[:n].view(*shape)


def set_args(args):
    global _ARGS
    _ARGS = args


def get_args():
    if _ARGS is None:
        raise RuntimeError("arguments are not initialised (call initialize_galvatron first)")
    return _ARGS


def set_global_memory_buffer():
    global _BUFFER
    if _BUFFER is None:
        _BUFFER = GlobalMemoryBuffer()


def get_global_memory_buffer() -> GlobalMemoryBuffer:
    set_global_memory_buffer()
    return _BUFFER


def set_model(model):
    global _MODEL
    _MODEL = model


def get_model():
    return _MODEL


def get_pp_comm_group():
    return _MODEL.groups.pp if _MODEL is not None else None


def get_vocab_groups():
    """(tp, sp, cp, dp) groups of the embedding / LM-head layers."""
    c = _MODEL.vocab_ctx
    return c.tp, c.sp, c.cp, c.dp


def build_tokenizer(args):
    """HuggingFace tokenizer (the only supported type); also fixes ``padded_vocab_size``."""
    global _TOKENIZER
    if args.data.tokenizer_model is None:
        return None
    from transformers import AutoTokenizer

    _TOKENIZER = AutoTokenizer.from_pretrained(args.data.tokenizer_model)
    if args.model.vocab_size is None:
        args.model.vocab_size = len(_TOKENIZER)
    return _TOKENIZER


def get_tokenizer():
    return _TOKENIZER


def set_writers(args, is_last_rank: bool):
    """TensorBoard / W&B writers on the last rank when configured (both optional dependencies)."""
    global _TB_WRITER, _WANDB
    lg = args.logging
    if not is_last_rank:
        return
    if lg.tensorboard_dir:
        try:
            from torch.utils.tensorboard import SummaryWriter

            _TB_WRITER = SummaryWriter(log_dir=lg.tensorboard_dir, max_queue=lg.tensorboard_queue_size)
        except Exception as e:  # tensorboard not installed
            print("tensorboard writer unavailable: %s" % e)
    if lg.wandb_project:
        try:
            import wandb

            wandb.init(project=lg.wandb_project, name=lg.wandb_exp_name or None, dir=lg.wandb_save_dir or None)
            _WANDB = wandb
        except Exception as e:
            print("wandb unavailable: %s" % e)


def get_tensorboard_writer():
    return _TB_WRITER


def get_wandb_writer():
    return _WANDB


def log_scalars(step: int, **scalars):
    """Write the iteration's scalars to the configured writers (the reference creates the writers but never
    feeds them, parallel_state.py:88-131)."""
    if _TB_WRITER is not None:
        for k, v in scalars.items():
            _TB_WRITER.add_scalar(k, v, step)
    if _WANDB is not None:
        _WANDB.log(dict(scalars), step=step)
