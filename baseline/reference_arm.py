"""``bench.py --impl reference``: the unmodified reference (installed by ``baseline/install_reference.sh`` into
``baseline/_ref``) trained through its own public API on the benchmark's configuration.

What runs is the reference's stock training loop, call for call (``galvatron/models/gpt/train_dist.py:21-72``):
``load_with_hydra`` on its own ``scripts/train_dist.yaml`` with dotted overrides, ``initialize_galvatron``,
``resolve_model_config``, ``build_model``, ``get_train_valid_test_data_iterators`` (its synthetic
``FakeCausalLMDataset``, ``runtime.data.use_random_dataset``), ``get_optimizer_and_param_scheduler`` and per step
``get_batch`` -> ``model.forward_backward`` -> ``clip_grad_norm`` -> ``optimizer.step`` -> scheduler step ->
``zero_grad``.  Kernels on that path are the reference's: cuBLAS through ``torch.nn.functional.linear``, flash-attn 2,
its Triton cross-entropy, NCCL through FSDP.  Nothing of ``hetu_galvatron_b200`` is imported here.

Stand-ins (each is a loader or a norm layer the image lacks, none is code of this repository's engine):

* ``baseline/shims/{hydra,omegaconf}``: the three calls of the reference's YAML loader;
* ``baseline/shims/flash_attn_norm_standin.py``: ``flash_attn.ops.rms_norm`` / ``layer_norm`` import a CUDA extension
  (``dropout_layer_norm``) the image does not carry; the stand-in serves flash-attn's own Triton ``RMSNorm``;
* a word-level tokenizer of 32000 entries written to a scratch directory (the reference builds a HuggingFace
  tokenizer at start-up only to learn the vocabulary size; no text is tokenized with synthetic data);
* ``apply_rope_fusion=false``: the fused RoPE needs apex or Transformer Engine, neither is installed; the reference's
  own unfused RoPE runs.

The timed loop differs from ``train_dist.py`` in two ways only: the runtime profiler is switched off
(``runtime.profile.profile=0``; it synchronizes the device twice per iteration) and the K timed steps are bracketed by
a barrier + device synchronize with CUDA events, as the benchmark's contract asks.  Every step includes the
reference's own host->device copy of the batch (``FakeCausalLMDataset.__getitem__``) and its ``loss.item()``.

If any of this fails, one JSON line ``{"impl": "reference", "unavailable": "<exception from inside galvatron>"}`` is
printed and the exit code is 0.
"""
from __future__ import annotations

import json
import os
import sys
import tempfile
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
SHIMS = os.path.join(HERE, "shims")
VOCAB = 32000
PER_GPU_BATCH = 8


def _write_tokenizer(path: str, vocab_size: int) -> None:
    """A HuggingFace fast tokenizer directory with ``vocab_size`` word-level entries (eos = id 2)."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    vocab = {"<unk>": 0, "<s>": 1, "</s>": 2}
    for i in range(3, vocab_size):
        vocab["t%d" % i] = i
    tok = Tokenizer(models.WordLevel(vocab=vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", bos_token="<s>", eos_token="</s>").save_pretrained(path)


def overrides_for(a, world: int, tokenizer_dir: str):
    """Dotted overrides that turn the reference's ``scripts/train_dist.yaml`` into the benchmark's configuration."""
    # same micro-batching and data-parallel type as the other arm (bench.plan_knobs: the searched strategy's values)
    sys.path.insert(0, os.path.dirname(HERE))
    from bench import plan_knobs

    _, _, chunks, dp_type = plan_knobs(world, a)
    layers = getattr(a, "layers", 0) or 32
    iters = a.warmup + a.steps + 1
    return [
        "paths.tokenizer_model=%s" % tokenizer_dir,
        "paths.data_path=null",
        "runtime.parallel.pp_deg=1", "runtime.parallel.global_tp_deg=1", "runtime.parallel.vocab_tp=1",
        "runtime.parallel.sdp=%d" % (1 if dp_type == "zero3" else 0),
        "runtime.parallel.default_dp_type=%s" % dp_type,
        "runtime.parallel.mixed_precision=bf16",
        "runtime.parallel.global_checkpoint=%d" % int(getattr(a, "checkpoint", 0)),
        # the model, inline (the reference's third documented way, galvatron/utils/hf_config_adapter.py:1-20): its
        # model_configs/llama2-7b.yaml always writes apply_rope_fusion=true and tied embeddings over inline values
        "paths.model_config_path=null", "runtime.model.model_size=llama2-7b",
        "++runtime.model.hidden_size=4096", "++runtime.model.num_attention_heads=32",
        "++runtime.model.ffn_hidden_size=11008", "++runtime.model.vocab_size=%d" % VOCAB,
        "++runtime.model.normalization=RMSNorm", "++runtime.model.norm_epsilon=1.0e-5",
        "++runtime.model.activation_func=torch.nn.functional.silu", "++runtime.model.gated_linear_unit=true",
        "++runtime.model.position_embedding_type=rope", "++runtime.model.rotary_base=10000",
        "++runtime.model.add_bias_linear=false", "++runtime.model.add_qkv_bias=false",
        "++runtime.model.make_vocab_size_divisible_by=128",
        "++runtime.model.apply_rope_fusion=false",
        # false is the value of the reference's own llama2-7b.yaml.  In the reference this flag being FALSE leaves
        # the embedding and the LM head as two independent matrices (models/builder.py:184 passes the tied-weight
        # names only when it is true), which is the benchmark's architecture (Llama-2 does not tie them).
        "++runtime.model.untie_embeddings_and_output_weights=false",
        "runtime.model.num_layers=%d" % layers, "runtime.model.set_layernum_manually=1",
        "runtime.profile.profile=0", "runtime.profile.exit_after_profiling=0",
        "runtime.train.train_iters=%d" % iters,
        "runtime.train.seq_length=%d" % a.seq, "runtime.model.set_seqlen_manually=1",
        "runtime.train.global_batch_size=%d" % (PER_GPU_BATCH * world),
        "runtime.train.micro_batch_size=%d" % PER_GPU_BATCH,   # batch per rank of the synthetic loader
        "runtime.train.chunks=%d" % chunks,
        "runtime.train.lr=1.0e-4", "runtime.train.min_lr=1.0e-5",
        "++runtime.train.seed=1234",
        "++runtime.data.use_random_dataset=true",
    ]


def _train(a):
    """The reference's ``train()`` with the benchmark's timing brackets; returns the result dict on every rank."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.setdefault("RANK", "0"))
    world = int(os.environ.setdefault("WORLD_SIZE", "1"))
    local_rank = int(os.environ.setdefault("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29517")
    # the reference's launcher script exports these (galvatron/models/gpt/scripts/train_yaml.sh:5-8)
    os.environ.setdefault("TORCH_NCCL_AVOID_RECORD_STREAMS", "1")
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "1")
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

    sys.path.insert(0, REF_DIR)
    sys.path.insert(0, SHIMS)
    import flash_attn_norm_standin
    flash_attn_norm_standin.install()

    tok_dir = os.path.join(tempfile.gettempdir(), "hg_ref_tokenizer_%d_r%d" % (os.getppid(), rank))
    if not os.path.exists(os.path.join(tok_dir, "tokenizer.json")):
        _write_tokenizer(tok_dir, VOCAB)

    from galvatron.core.arguments import load_with_hydra
    from galvatron.core.runtime.dataloader import get_batch, get_train_valid_test_data_iterators
    from galvatron.core.runtime.initialize import initialize_galvatron
    from galvatron.core.runtime.models.builder import build_model, get_runtime_profiler
    from galvatron.core.runtime.optimizer.utils import clip_grad_norm, get_optimizer_and_param_scheduler
    from galvatron.core.runtime.utils.utils import set_megatron_args_for_dataset
    from galvatron.utils.hf_config_adapter import resolve_model_config

    gpt_dir = os.path.join(REF_DIR, "galvatron", "models", "gpt")
    os.chdir(gpt_dir)   # the YAML names its model file relative to this directory, as the reference's launcher does
    args = load_with_hydra(os.path.join("scripts", "train_dist.yaml"), overrides=overrides_for(a, world, tok_dir),
                           mode="train_dist")
    initialize_galvatron(args)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)

    resolve_model_config(args)
    model = build_model(args)
    set_megatron_args_for_dataset(args)
    train_it, _, _ = get_train_valid_test_data_iterators()
    optimizer, sched = get_optimizer_and_param_scheduler(model, args)
    profiler = get_runtime_profiler(args, gpt_dir, start_iter=0, end_iter=max(1, args.train.train_iters - 1))

    def step(i):
        tokens, kwargs, loss_func = get_batch(train_it)
        profiler.profile_time_start(i)
        loss = model.forward_backward([tokens], i, profiler, loss_func=loss_func, **kwargs)
        grad_norm = clip_grad_norm(model, args.train.clip_grad)
        optimizer.step()
        sched.step(increment=args.train.global_batch_size)
        optimizer.zero_grad()
        profiler.profile_time_end(i, loss, optimizer.param_groups[0]["lr"], grad_norm)
        return loss, tokens

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    it = 0
    for _ in range(a.warmup):
        step(it)
        it += 1
    barrier()
    sampler = None
    if rank == 0:
        sys.path.insert(0, os.path.dirname(HERE))
        from bench import ClockSampler   # nvidia-smi sampling only, no model code
        sampler = ClockSampler(local_rank)
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.perf_counter()
    e0.record()
    loss, tokens = None, None
    for _ in range(a.steps):
        loss, tokens = step(it)
        it += 1
    e1.record()
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1000 / a.steps
    dev_ms = e0.elapsed_time(e1) / a.steps
    clocks = sampler.stop() if sampler is not None else {}
    if world > 1:
        t = torch.tensor([dev_ms, wall_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, wall_ms = float(t[0]), float(t[1])
    B, S = int(tokens.shape[0]), int(tokens.shape[1])
    gbsz = B * world
    ntok = gbsz * S
    e2e_ms = max(dev_ms, wall_ms)
    out = {
        "metric": "tokens/sec", "value": ntok / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "impl": "reference",
        "data": "synthetic uniform-random token ids (the reference's FakeCausalLMDataset); random-init weights",
        "config": {"model": "llama2-7b (%dL h4096 32 heads ffn 11008 vocab 32000)" % args.model.num_layers,
                   "global_batch": gbsz, "seq_len": S, "micro_batch": B // max(1, args.train.chunks),
                   "parallelism": "dp%d%s" % (world, "" if world == 1 else "-" + args.parallel.default_dp_type),
                   "l2": "working set far larger than the 126 MB L2",
                   "optimizer": "the reference's AdamW + global-norm clip inside the timed region"},
        "clocks": clocks,
        "e2e": {"value": ntok / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(B * (S + 1) * 8), "d2h_bytes_per_step": 4 * max(1, args.train.chunks)},
        "gpu_launches": 0,
        "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30,
        "peak_reserved_gib": torch.cuda.max_memory_reserved() / 2 ** 30,
        # cudaMalloc failures that made the caching allocator free its cache and retry (each one stalls the device)
        "alloc_retries": int(torch.cuda.memory_stats().get("num_alloc_retries", 0)),
        "final_loss": float(loss) if loss is not None else None,
    }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out


def run(a):
    rank = int(os.environ.get("RANK", "0"))
    if not os.path.isdir(os.path.join(REF_DIR, "galvatron")):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable":
                              "baseline/_ref is empty: run baseline/install_reference.sh <reference checkout>"}))
        return 0
    try:
        out = _train(a)
        if rank == 0:
            print(json.dumps(out), flush=True)
    except BaseException as e:   # SystemExit from the reference's own exit() calls included
        if rank == 0:
            tb = traceback.extract_tb(e.__traceback__)
            where = next(("%s:%d" % (f.filename.split("baseline/_ref/")[-1], f.lineno) for f in reversed(tb)
                          if "galvatron" in f.filename), "%s:%d" % (os.path.basename(tb[-1].filename), tb[-1].lineno)
                         if tb else "?")
            traceback.print_exc(file=sys.stderr)
            print(json.dumps({"impl": "reference", "unavailable": "reference failed at %s: %s: %s"
                              % (where, type(e).__name__, " ".join(str(e).split())[:300])}), flush=True)
    return 0
