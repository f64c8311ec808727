"""Device-timed comparison of the peer-memory all-to-all (layout transform folded in) with "permute + NCCL
all_to_all_single" for the Ulysses head/sequence exchange.

    torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 -m hetu_galvatron_b200.profiler.fused_a2a_bench \
        --seq 32768 --batch 1 --heads 40 --head-dim 128

Each rank holds ``[seq/p, batch, heads, head_dim]`` bf16.  Arms (CUDA events, 3 warm-ups, median of ``--iters``,
maximum over ranks, 256 MiB L2 flush between runs): ``s2h`` sequence->heads and ``h2s`` heads->sequence, each as the
peer kernel (staging copy + rendezvous + pull) and as the NCCL path (permute copy + all-to-all).  Roofline: the bytes
that cross NVLink per direction, ``(p-1)/p`` of the tensor, at 770 GB/s.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def run(seq: int, batch: int, heads: int, hd: int, iters: int = 10):
    from ..ops import _lib
    from ..parallel import fused_a2a as fa
    from ..parallel import ulysses as ul
    from ..parallel.groups import CommGroup

    p, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    grp = CommGroup(list(range(p)), dist.group.WORLD, rank)
    x = torch.randn(seq // p, batch, heads, hd, device=dev, dtype=torch.bfloat16)
    y = torch.randn(seq, batch, heads // p, hd, device=dev, dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        v = torch.tensor([ts[len(ts) // 2]], device=dev)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v)

    with torch.no_grad():
        res = {"gpus": p, "seq": seq, "batch": batch, "heads": heads, "head_dim": hd,
               "s2h_peer_ms": timed(lambda: fa.seq_to_heads(x, grp, p)), "s2h_nccl_ms": timed(lambda: ul.seq_to_heads(x, grp, p)),
               "h2s_peer_ms": timed(lambda: fa.heads_to_seq(y, grp, p)), "h2s_nccl_ms": timed(lambda: ul.heads_to_seq(y, grp, p))}
    link_bytes = x.numel() * 2 * (p - 1) / p
    res["roofline_ms"] = link_bytes / (NVLINK_GBS * 1e9) * 1e3
    res["s2h_frac_of_roofline"] = res["roofline_ms"] / res["s2h_peer_ms"]
    res["h2s_frac_of_roofline"] = res["roofline_ms"] / res["h2s_peer_ms"]
    res["status"] = _lib.read_status()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=32768)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=40)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    rank = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank), timeout=datetime.timedelta(seconds=120))
    res = run(a.seq, a.batch, a.heads, a.head_dim, a.iters)
    if dist.get_rank() == 0:
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
