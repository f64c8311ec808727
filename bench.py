"""Headline benchmark: Llama-2-7B-shaped training throughput (tokens/s), bf16, seq 4096.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched once per rank by torchrun)
    python bench.py --impl reference ...                      (the unmodified reference, when installable)

Weak scaling: 8 sequences per GPU (global batch 8*N -- 64 at N = 8, the configuration the baseline names).
Synthetic uniform-random token ids (a fresh batch every step), random-init N(0, 0.02) weights.  The parallel plan is
the one the strategy search wrote for N GPUs from the shipped B200 profiles
(``hetu_galvatron_b200/cli/configs/galvatron_config_llama2-7b_1nodes_<N>gpus_per_node_160GB_bf16.json``, produced by
``python -m hetu_galvatron_b200.cli.search_dist``); its predicted iteration time is printed beside the measured one.
Per step: forward + backward of all micro-batches, gradient reduction, global-norm clipping, AdamW.  Two timed
regions of K steps each:

  * ``value``      device-timed with CUDA events (inputs resident on the device), max over ranks;
  * ``e2e.value``  the same step through the public API with the step's inputs copied host->device from
                   pinned memory and the loss read back device->host every step.

Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEQ = 4096
PER_GPU_BATCH = 8
MODEL = dict(model_size="llama2-7b", hidden_size=4096, num_layers=32, num_attention_heads=32, ffn_hidden_size=11008,
             vocab_size=32000, normalization="RMSNorm", norm_epsilon=1e-5, activation_func="torch.nn.functional.silu",
             gated_linear_unit=True, position_embedding_type="rope", untie_embeddings_and_output_weights=True,
             make_vocab_size_divisible_by=128)


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def searched_strategy(n: int, a):
    """The strategy JSON the search engine wrote for ``n`` GPUs (``--strategy PATH`` overrides, ``--strategy none``
    falls back to plain flags).  Returns ``(dict or None, path or None)``."""
    if a.strategy == "none":
        return None, None
    path = a.strategy or os.path.join(ROOT, "hetu_galvatron_b200", "cli", "configs",
                                      "galvatron_config_llama2-7b_1nodes_%dgpus_per_node_160GB_bf16.json" % n)
    if not os.path.exists(path):
        return None, None
    with open(path) as f:
        return json.load(f), path


def plan_knobs(n: int, a):
    """``(strategy dict or None, path, chunks, dp_type)`` used by both arms, so that they run the same plan."""
    cfg, path = searched_strategy(n, a)
    if cfg is not None and a.micro_batch is None:
        chunks = int(cfg["chunks"])
        dp_type = cfg.get("default_dp_type", a.dp_type)
    else:
        chunks = PER_GPU_BATCH // (a.micro_batch or 2)
        dp_type = a.dp_type
    if a.layers or a.micro_batch is not None or a.checkpoint or a.pp > 1 or a.tp > 1 or \
            (cfg is not None and cfg.get("global_bsz") != PER_GPU_BATCH * n):
        cfg = None      # debugging overrides: plain flags with the strategy's micro-batching
    return cfg, path, max(1, chunks), (dp_type if n > 1 else "ddp")


def run_reference(a):
    """The unmodified reference through its own public path, when it can be imported on this image."""
    from baseline import reference_arm

    return reference_arm.run(a)


def run_ours(a):
    import torch
    import torch.distributed as dist

    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs
    from hetu_galvatron_b200.ops import _lib
    from hetu_galvatron_b200.runtime.engine import build_model
    from hetu_galvatron_b200.runtime.optimizer import ShardedAdamW

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    if world != a.gpus and rank == 0:
        print("warning: --gpus %d but WORLD_SIZE=%d" % (a.gpus, world), file=sys.stderr)
    n = world
    gbsz = PER_GPU_BATCH * n
    strategy, strategy_path, chunks, dp_type = plan_knobs(n, a)
    model_cfg = dict(MODEL)
    if a.layers:
        model_cfg["num_layers"] = a.layers
    parallel = dict(pp_deg=a.pp, global_tp_deg=a.tp, vocab_tp=a.tp, pipeline_type="pipedream_flush",
                    default_dp_type=dp_type if n > a.pp * a.tp else "ddp", sdp=1 if dp_type == "zero3" else 0,
                    mixed_precision="bf16", async_grad_reduce=True, global_checkpoint=int(a.checkpoint))
    if strategy is not None:
        parallel["galvatron_config_path"] = strategy      # JSON mode: the per-layer plan comes from the search
    args = GalvatronRuntimeArgs(
        parallel=parallel,
        model=model_cfg,
        train=dict(seq_length=a.seq, global_batch_size=gbsz, chunks=chunks, lr=1e-4, adam_beta1=0.9, adam_beta2=0.95,
                   weight_decay=0.1, clip_grad=1.0, seed=1234),
        rank=rank, world_size=n, local_rank=local_rank)
    os.environ.setdefault("HG_QUIET", "1")   # stdout carries the one JSON line only; the plan is in its "config"
    model = build_model(args, device=dev)
    opt = ShardedAdamW(model.sharded_units, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, clip_grad=1.0,
                       device=dev)
    B = model.local_batch_size()
    S = a.seq
    chunks = model.plan.chunks
    mbs = max(1, B // chunks)
    g = torch.Generator().manual_seed(1234 + rank)
    # a fresh batch of uniform-random tokens for every step of the run (warm-up, device-timed, end-to-end)
    n_host = a.warmup + 2 * a.steps
    host = [torch.randint(0, MODEL["vocab_size"], (B, S + 1), generator=g).pin_memory() for _ in range(n_host)]
    dev_batches = [h.to(dev) for h in host[:a.warmup + a.steps]]
    cursor = [0]

    def step_device(i):
        t = dev_batches[cursor[0]]
        cursor[0] += 1
        opt.zero_grad()
        loss = model.forward_backward(t[:, :-1], i, labels=t[:, 1:])
        opt.step()
        return loss

    def step_e2e(i):
        t = host[a.warmup + a.steps + i].to(dev, non_blocking=True)
        opt.zero_grad()
        loss = model.forward_backward(t[:, :-1], i, labels=t[:, 1:])
        opt.step()
        # the loss lives on the last pipeline stage; the other stages have nothing to read back
        return float(loss.item()) if loss is not None else None

    def barrier():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(a.warmup):
        step_device(i)
    barrier()
    _lib.assert_healthy()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    _lib.reset_launches()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    last = None
    for i in range(a.steps):
        last = step_device(i)
    ev1.record()
    barrier()
    launches = _lib.launches()
    ms = ev0.elapsed_time(ev1) / a.steps
    # end to end: H2D of the inputs and D2H of the loss inside the timed region
    barrier()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    loss_val = None
    for i in range(a.steps):
        loss_val = step_e2e(i)
    e1.record()
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1000 / a.steps
    e2e_ms = max(e0.elapsed_time(e1) / a.steps, wall_ms)
    clocks = sampler.stop() if rank == 0 else {}
    _lib.assert_healthy()
    if n > 1:
        t = torch.tensor([ms, e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    if n > 1 and model.plan.pp_deg > 1:
        # rank 0 prints; with pipeline stages the loss is on the last stage
        vals = [None] * n
        dist.all_gather_object(vals, loss_val)
        loss_val = next((v for v in reversed(vals) if v is not None), None)
    tokens = gbsz * S
    value = tokens / (ms / 1000.0)
    peak_mem = torch.cuda.max_memory_allocated() / 2 ** 30
    flops = model.spec.flops_per_token(S) * tokens
    out = {
        "metric": "tokens/sec", "value": value, "unit": "tokens/s", "n_gpus": n, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform-random token ids; random-init N(0,0.02) weights",
        "impl": "ours",
        "config": {"model": "llama2-7b (32L h4096 32 heads ffn 11008 vocab 32000)" if not a.layers else
                   "llama2-7b-shaped, %d layers" % a.layers,
                   "global_batch": gbsz, "seq_len": S, "micro_batch": mbs, "chunks": chunks,
                   "parallelism": model.plan.short_name() + ("-ckpt" if a.checkpoint else ""),
                   "strategy": ("searched: " + os.path.relpath(strategy_path, ROOT)) if strategy is not None else "flags",
                   "l2": "working set (13.5 GB of bf16 weights + activations per step) is far larger than the 126 MB L2",
                   "optimizer": "AdamW fp32 master + global-norm clip inside the timed region"},
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms / 1000.0), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(B * (S + 1) * 8), "d2h_bytes_per_step": 4},
        "gpu_launches": launches,
        "model_tflops_per_gpu": flops / (ms / 1000.0) / 1e12 / n,
        "peak_mem_gib": peak_mem,
        "peak_reserved_gib": torch.cuda.max_memory_reserved() / 2 ** 30,
        "alloc_retries": int(torch.cuda.memory_stats().get("num_alloc_retries", 0)),
        "final_loss": loss_val,
    }
    if strategy is not None and strategy.get("predicted_time_cost"):
        pred = float(strategy["predicted_time_cost"]) * 1000.0
        out.update(predicted_ms=pred, measured_ms=ms, pred_error=(pred - ms) / ms)
    if rank == 0:
        print(json.dumps(out))
    if n > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seq", type=int, default=SEQ)
    ap.add_argument("--micro-batch", type=int, default=(int(os.environ["HG_BENCH_MBS"]) if "HG_BENCH_MBS" in os.environ else None),
                    help="sequences per micro-batch (default: what the searched strategy says)")
    ap.add_argument("--strategy", default=os.environ.get("HG_BENCH_STRATEGY"),
                    help="strategy JSON to run (default: the shipped searched plan for N GPUs; 'none' = plain flags)")
    ap.add_argument("--dp-type", default=os.environ.get("HG_BENCH_DP", "zero2"))
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (result is not a headline number)")
    ap.add_argument("--checkpoint", type=int, default=0)
    ap.add_argument("--pp", type=int, default=1, help="debug only: pipeline stages of a plain-flags plan")
    ap.add_argument("--tp", type=int, default=1, help="debug only: tensor-parallel degree of a plain-flags plan")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
