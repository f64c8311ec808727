"""Device-timed comparison of the peer-memory ZeRO kernels with the NCCL path, on a flat buffer the size of one
decoder layer (or any ``--numel``).

    torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 -m hetu_galvatron_b200.profiler.fused_zero_bench

Arms, each timed with CUDA events after 3 warm-ups, median of ``--iters`` runs, maximum over ranks, with a 256 MiB
buffer rewritten between runs (nothing is served from L2):

* ``rs_peer``   rendezvous + ``hg_zero_reduce_scatter`` (peer loads)          vs ``rs_nccl``  ``reduce_scatter_tensor`` (fp32)
* ``opt_peer``  ``hg_zero_adamw_allgather`` (peer stores) + rendezvous        vs ``opt_nccl`` ``hg_adamw`` + ``all_gather_into_tensor`` (bf16)

Roofline of each arm = the slower of its local HBM bytes at the measured copy bandwidth and its NVLink bytes
(per direction) at 770 GB/s.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def measured_hbm_gbs(default: float = 6650.0) -> float:
    here = os.path.dirname(os.path.abspath(__file__))
    for up in (os.path.join(here, "..", ".."), os.getcwd()):
        p = os.path.join(up, "MEASURED_PEAKS.json")
        if os.path.exists(p):
            return float(json.load(open(p)).get("hbm_gbs", default))
    return default


def run(numel: int, iters: int = 10):
    from .. import ops
    from ..ops import _lib
    from ..parallel import fused_zero as fz

    t, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    numel = (numel + 64 * t - 1) // (64 * t) * (64 * t)
    S = numel // t
    pg = dist.group.WORLD
    grads = fz.SymmetricBuffer(numel, torch.float32, dev, pg)
    params = fz.SymmetricBuffer(numel, torch.bfloat16, dev, pg)
    grads.tensor.normal_()
    shard = torch.empty(S, dtype=torch.float32, device=dev)
    master, m, v = (torch.randn(S, device=dev) for _ in range(3))
    v.abs_()
    lp = torch.empty(S, dtype=torch.bfloat16, device=dev)
    full = torch.empty(numel, dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    hp = dict(lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3)

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
        x = torch.tensor([ts[len(ts) // 2]], device=dev)
        dist.all_reduce(x, op=dist.ReduceOp.MAX)
        return float(x)

    def rs_peer():
        fz.peer_barrier(pg, dev)
        fz.reduce_scatter_peer(grads, rank, S, shard)

    def opt_peer():
        fz.adamw_allgather_peer(master, shard, m, v, params, rank * S, **hp)
        fz.peer_barrier(pg, dev)

    def opt_nccl():
        ops.adamw_step(master, shard, m, v, lp, **hp)
        dist.all_gather_into_tensor(full, lp)

    res = {"gpus": t, "numel": numel,
           "rs_peer_ms": timed(rs_peer), "rs_nccl_ms": timed(lambda: dist.reduce_scatter_tensor(shard, grads.tensor)),
           "opt_peer_ms": timed(opt_peer), "opt_nccl_ms": timed(opt_nccl)}
    hbm = measured_hbm_gbs() * 1e9
    link = NVLINK_GBS * 1e9
    rs_link, rs_hbm = (t - 1) * S * 4, (S * 4) * 2           # pulls from t-1 peers; local read + shard write
    opt_link, opt_hbm = (t - 1) * S * 2, S * (4 * 4 + 3 * 4 + 2)  # bf16 stores to t-1 peers; 4 reads + 3 writes fp32 + local bf16
    res["rs_roofline_ms"] = max(rs_link / link, rs_hbm / hbm) * 1e3
    res["opt_roofline_ms"] = max(opt_link / link, opt_hbm / hbm) * 1e3
    res["rs_frac_of_roofline"] = res["rs_roofline_ms"] / res["rs_peer_ms"]
    res["opt_frac_of_roofline"] = res["opt_roofline_ms"] / res["opt_peer_ms"]
    res["status"] = _lib.read_status()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--numel", type=int, default=202383360, help="elements of the flat buffer (default: one Llama-2-7B layer)")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    rank = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank), timeout=datetime.timedelta(seconds=120))
    res = run(a.numel, a.iters)
    if dist.get_rank() == 0:
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
