"""Device-timed comparison of the fused tensor-parallel kernels with "NCCL collective + the same GEMM".

    torchrun --nnodes 1 --nproc-per-node 2 --master-addr 127.0.0.1 -m hetu_galvatron_b200.profiler.fused_tp_bench \
        --slab 4096 --kdim 4096 --ndim 6144

Per configuration: all-gather -> GEMM (``[t*slab, K] x [N, K]^T`` with the input sharded by rows) and GEMM ->
reduce-scatter (``[t*slab, K] x [N, K]^T`` summed over ranks, output sharded by rows).  Each variant is timed with
CUDA events on the launching stream after 3 warm-ups; a 256 MiB buffer is rewritten between iterations so that
nothing is served from L2; the figure is the median over iterations and the maximum over ranks.  The roofline is
the slower of FLOPs at the measured cuBLAS bf16 burst rate and the bytes that must cross NVLink at 770 GB/s per
direction.  One JSON line per configuration is printed by rank 0.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def measured_bf16_tflops(default: float = 1590.0) -> float:
    here = os.path.dirname(os.path.abspath(__file__))
    for up in (os.path.join(here, "..", ".."), os.getcwd()):
        p = os.path.join(up, "MEASURED_PEAKS.json")
        if os.path.exists(p):
            return float(json.load(open(p)).get("bf16_tflops", default))
    return default


def fused_vs_nccl(group, slab: int, K: int, N: int, iters: int = 10):
    from .. import ops
    from ..ops import _lib
    from ..parallel import fused_comm as fc

    t = group.size
    dev = torch.device("cuda", torch.cuda.current_device())
    x = torch.randn(slab, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
    x2 = torch.randn(t * slab, K, device=dev, dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            dist.barrier(group=group.group)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        v = torch.tensor([ts[len(ts) // 2]], device=dev)
        dist.all_reduce(v, op=dist.ReduceOp.MAX, group=group.group)
        return float(v)

    def nccl_ag():
        xg = torch.empty(t * slab, K, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(xg, x, group=group.group)
        return ops.gemm(xg, w)

    def nccl_rs():
        y = ops.gemm(x2, w)
        o = torch.empty(slab, N, device=dev, dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(o, y, group=group.group)
        return o

    res = {"ag_fused_ms": timed(lambda: fc.ag_gemm(x, w, group)), "ag_nccl_ms": timed(nccl_ag),
           "rs_fused_ms": timed(lambda: fc.gemm_rs(x2, w, group)), "rs_nccl_ms": timed(nccl_rs),
           "gemm_only_ms": timed(lambda: ops.gemm(x2, w))}
    flops = 2.0 * t * slab * K * N
    peak = measured_bf16_tflops()
    res["ag_fused_tflops"] = flops / res["ag_fused_ms"] / 1e9
    res["rs_fused_tflops"] = flops / res["rs_fused_ms"] / 1e9
    ag_bytes = (t - 1) * slab * K * 2
    rs_bytes = (t - 1) * slab * N * 2
    res["ag_roofline_ms"] = max(flops / peak / 1e9, ag_bytes / (NVLINK_GBS * 1e9) * 1e3)
    res["rs_roofline_ms"] = max(flops / peak / 1e9, rs_bytes / (NVLINK_GBS * 1e9) * 1e3)
    res["ag_frac_of_roofline"] = res["ag_roofline_ms"] / res["ag_fused_ms"]
    res["rs_frac_of_roofline"] = res["rs_roofline_ms"] / res["rs_fused_ms"]
    res["status"] = _lib.read_status()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--slab", type=int, default=4096)
    ap.add_argument("--kdim", type=int, default=4096)   # not --k / --n: torchrun would read them as its own
    ap.add_argument("--ndim", type=int, default=6144)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    rank = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank), timeout=datetime.timedelta(seconds=120))
    from ..parallel.groups import CommGroup

    world = dist.get_world_size()
    grp = CommGroup(list(range(world)), dist.group.WORLD, dist.get_rank())
    res = fused_vs_nccl(grp, a.slab, a.kdim, a.ndim, a.iters)
    if dist.get_rank() == 0:
        print(json.dumps({"gpus": world, "slab": a.slab, "K": a.kdim, "N": a.ndim, **res}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
