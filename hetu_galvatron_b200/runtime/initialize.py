"""Process start-up: ranks from the environment, argument checks, process group, seeds, global state.

Capability parity: galvatron/core/runtime/initialize.py:114-139 (process group), :142-187 (initialisation
order incl. building the native dataset helpers on one rank), :190-237 (argument validation), :240-247 (args
dump); parallel_state globals (parallel_state.py:31-141).
"""
from __future__ import annotations

import datetime
import json
import os
import random

import numpy as np
import torch
import torch.distributed as dist

from ..parallel import state


def set_seed(seed: int):
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def validate_args(args):
    p, m, t = args.parallel, args.model, args.train
    if t.global_batch_size is None:
        raise ValueError("train.global_batch_size must be set")
    if p.use_ulysses and p.global_tp_deg > 1 and m.num_attention_heads and m.num_attention_heads % p.global_tp_deg:
        raise ValueError("Ulysses degree must divide the number of attention heads")
    if p.mixed_precision == "fp16" and torch.cuda.is_available():
        raise ValueError("the sm_100a kernels are bf16; use mixed_precision=bf16 (fp32 runs on the CPU oracle path)")
    if p.pp_deg > 1 and t.chunks not in (-1,) and t.chunks is not None and 0 < t.chunks < p.pp_deg \
            and p.pipeline_type == "pipedream_flush":
        raise ValueError("1F1B needs chunks >= pp_deg")
    if p.global_cp_deg > 1 and t.seq_length and t.seq_length % (2 * p.global_cp_deg):
        raise ValueError("seq_length must be divisible by 2 * cp for the zig-zag split")
    return args


def print_args_rank0(args):
    if int(os.environ.get("RANK", "0")) == 0:
        print("------------------------ arguments ------------------------")
        print(json.dumps(json.loads(args.model_dump_json()), indent=2, default=str))
        print("-----------------------------------------------------------")


def initialize_galvatron(args, backend: str = None):
    """Fill rank fields from the environment, validate, create the default process group, seed, and publish
    ``args`` in ``parallel.state``.  Idempotent with respect to an existing process group."""
    args.rank = int(os.environ.get("RANK", "0"))
    args.world_size = int(os.environ.get("WORLD_SIZE", "1"))
    args.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    validate_args(args)
    state.set_args(args)
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(args.local_rank)
    if args.world_size > 1 and not dist.is_initialized():
        be = backend or (args.distributed_backend if use_cuda else "gloo")
        kw = dict(timeout=datetime.timedelta(minutes=args.distributed_timeout_minutes))
        if use_cuda and be == "nccl":
            kw["device_id"] = torch.device("cuda", args.local_rank)
        dist.init_process_group(be, **kw)
    set_seed(args.train.seed or 1234)
    state.set_global_memory_buffer()
    state.set_writers(args, is_last_rank=(args.rank == args.world_size - 1))
    from .rerun import initialize_rerun_state_machine

    initialize_rerun_state_machine()
    from ..models.moe import set_aux_loss_scale

    set_aux_loss_scale(1.0)
    if (args.data.data_path or args.data.train_data_path) and not args.data.use_random_dataset:
        # build the native index helpers on one rank, everybody waits
        if args.rank == 0:
            from ..csrc import build as _build

            _build.build_host()
        if dist.is_initialized():
            dist.barrier()
    return args
