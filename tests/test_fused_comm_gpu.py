"""Fused tensor-parallel kernels (all-gather -> GEMM, GEMM -> reduce-scatter) against the NCCL + fp32 reference,
forward and backward, on 2 GPUs (one process per GPU)."""
import json
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tests.dist_utils import run_distributed  # noqa: E402

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _init():
    import datetime

    import torch.distributed as dist

    rank = int(os.environ["RANK"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank), timeout=datetime.timedelta(seconds=60))
    from hetu_galvatron_b200.parallel.groups import CommGroup

    world = dist.get_world_size()
    return rank, world, CommGroup(list(range(world)), dist.group.WORLD, rank)


def rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def fused_vs_reference(cfg):
    import torch.distributed as dist

    from hetu_galvatron_b200.ops import _lib
    from hetu_galvatron_b200.parallel import fused_comm as fc

    rank, t, grp = _init()
    dev = torch.device("cuda", rank)
    slab, K, N = cfg["slab"], cfg["K"], cfg["N"]
    out = {}
    for rep in range(2):  # twice: exercises both staging parities and the epoch protocol
        g = torch.Generator(device=dev).manual_seed(100 + rank + 10 * rep)
        x = torch.randn(slab, K, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_()
        w = (torch.randn(N, K, device=dev, dtype=torch.bfloat16, generator=g) * 0.05).requires_grad_()
        # all-gather -> GEMM
        y = fc._AllGatherLinear.apply(x, w, None, grp)
        xs = [torch.empty_like(x) for _ in range(t)]
        dist.all_gather(xs, x.detach())
        xg = torch.cat(xs).float()
        ref = xg @ w.detach().float().t()
        out["ag_fwd_%d" % rep] = rel(y, ref)
        dy = torch.randn(t * slab, N, device=dev, dtype=torch.bfloat16, generator=g)
        y.backward(dy)
        dx_full = dy.float() @ w.detach().float()
        dist.all_reduce(dx_full)
        out["ag_dx_%d" % rep] = rel(x.grad, dx_full[rank * slab:(rank + 1) * slab])
        out["ag_dw_%d" % rep] = rel(w.grad, dy.float().t() @ xg)
        # GEMM -> reduce-scatter
        x2 = torch.randn(t * slab, K, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_()
        w2 = (torch.randn(N, K, device=dev, dtype=torch.bfloat16, generator=g) * 0.05).requires_grad_()
        z = fc._LinearReduceScatter.apply(x2, w2, grp)
        full = x2.detach().float() @ w2.detach().float().t()
        dist.all_reduce(full)
        out["rs_fwd_%d" % rep] = rel(z, full[rank * slab:(rank + 1) * slab])
        dz = torch.randn(slab, N, device=dev, dtype=torch.bfloat16, generator=g)
        z.backward(dz)
        dzs = [torch.empty_like(dz) for _ in range(t)]
        dist.all_gather(dzs, dz)
        dzg = torch.cat(dzs).float()
        out["rs_dx_%d" % rep] = rel(x2.grad, dzg @ w2.detach().float())
        out["rs_dw_%d" % rep] = rel(w2.grad, dzg.t() @ x2.detach().float())
    torch.cuda.synchronize()
    out["status"] = _lib.read_status()
    return out


def fused_vs_nccl_timing(cfg):
    """Device-timed fused kernels vs NCCL collective + the same GEMM (see profiler/fused_tp_bench.py)."""
    from hetu_galvatron_b200.profiler.fused_tp_bench import fused_vs_nccl

    rank, t, grp = _init()
    return fused_vs_nccl(grp, cfg["slab"], cfg["K"], cfg["N"])


REGISTRY = {"fused_vs_reference": fused_vs_reference, "fused_vs_nccl_timing": fused_vs_nccl_timing}


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip("needs %d GPUs" % n)


@pytest.mark.parametrize("slab,K,N", [(256, 512, 768), (1024, 4096, 1536), (384, 1024, 1000), (512, 1024, 1320)])
def test_fused_tp_kernels_match_reference(slab, K, N):
    """Slabs of whole 256-row tiles run on the CTA-pair kernels (fused_tp2.cu), the 384-row slab on the one-CTA kernels
    (fused_tp.cu); N = 1000 / 1320 leave a partial last column tile."""
    _need(2)
    res = run_distributed(__file__, "fused_vs_reference", 2, {"slab": slab, "K": K, "N": N}, timeout=240,
                          extra_env={"HG_BACKEND": "nccl", "NCCL_NVLS_ENABLE": "0"})
    for r in res:
        assert r["status"] == 0, r
        for k, v in r.items():
            if k != "status":
                assert v < 2e-2, (k, r)


if __name__ == "__main__":
    func, payload = sys.argv[2], json.loads(sys.argv[3])
    out = REGISTRY[func](payload)
    with open(os.environ["HG_OUT"], "w") as f:
        json.dump(out, f)
    import torch.distributed as dist

    dist.barrier()
    dist.destroy_process_group()
