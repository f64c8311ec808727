"""ZeRO reduce-scatter and AdamW+all-gather over NVLink peer memory (2 GPUs): kernel numerics against
NCCL + the plain AdamW kernel, and whole-model training parity with the NCCL path."""
import json
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tests.dist_utils import run_distributed  # noqa: E402

pytestmark = pytest.mark.gpu


def _init():
    import datetime

    import torch.distributed as dist

    rank = int(os.environ["RANK"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank), timeout=datetime.timedelta(seconds=60))
    return rank, dist.get_world_size()


def kernels_vs_nccl(cfg):
    import torch.distributed as dist

    from hetu_galvatron_b200 import ops
    from hetu_galvatron_b200.ops import _lib
    from hetu_galvatron_b200.parallel import fused_zero as fz

    rank, t = _init()
    dev = torch.device("cuda", rank)
    S = cfg["shard"]
    n = S * t
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    grads = fz.SymmetricBuffer(n, torch.float32, dev, dist.group.WORLD)
    params = fz.SymmetricBuffer(n, torch.bfloat16, dev, dist.group.WORLD)
    out = {}
    for rep in range(2):
        grads.tensor.copy_(torch.randn(n, device=dev, generator=g))
        ref = torch.empty(S, device=dev)
        dist.reduce_scatter_tensor(ref, grads.tensor.clone())
        got = torch.empty(S, device=dev)
        fz.peer_barrier(dist.group.WORLD, dev)
        fz.reduce_scatter_peer(grads, rank, S, got)
        fz.peer_barrier(dist.group.WORLD, dev)
        out["rs_%d" % rep] = float((got - ref).abs().max() / ref.abs().max())
        # bf16 on the wire: peers' slices rounded to bf16, own slice exact, fp32 sum; then the accumulating form
        pair = fz.staging_buffers(n, torch.bfloat16, dev, dist.group.WORLD)
        st = pair.next()
        fz.round_into_staging(grads.tensor, st, rank, S)
        fz.peer_barrier(dist.group.WORLD, dev)
        got16 = torch.empty(S, device=dev)
        fz.reduce_scatter_staged(st, grads.tensor, rank, S, got16, accumulate=False, max_ctas=8 if rep else 0)
        fz.reduce_scatter_staged(st, grads.tensor, rank, S, got16, accumulate=True)
        fz.peer_barrier(dist.group.WORLD, dev)
        # the same reduction with the kernel's own rendezvous instead of a collective before it
        st2 = pair.next()
        fz.round_into_staging(grads.tensor, st2, rank, S)
        got16b = torch.empty(S, device=dev)
        fz.reduce_scatter_staged(st2, grads.tensor, rank, S, got16b, signals=pair.signals)
        rounded = [torch.empty(n, device=dev) for _ in range(t)]
        dist.all_gather(rounded, grads.tensor.clone())
        lo, hi = rank * S, (rank + 1) * S
        want = sum((x[lo:hi] if r == rank else x[lo:hi].bfloat16().float()) for r, x in enumerate(rounded))
        out["rs16_%d" % rep] = float((got16 - 2 * want).abs().max() / want.abs().max())
        out["rs16_flags_%d" % rep] = float((got16b - want).abs().max() / want.abs().max())
        # AdamW + all-gather against the plain kernel + NCCL all-gather
        master = torch.randn(S, device=dev, generator=g)
        m0, v0 = torch.randn(S, device=dev, generator=g) * 0.1, torch.rand(S, device=dev, generator=g) * 0.01
        scale = torch.full((1,), 0.5, device=dev)
        a = [master.clone(), m0.clone(), v0.clone()]
        lp = torch.empty(S, dtype=torch.bfloat16, device=dev)
        ops.adamw_step(a[0], got, a[1], a[2], lp, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=rep + 1,
                       gscale=scale)
        full = torch.empty(n, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(full, lp)
        b = [master.clone(), m0.clone(), v0.clone()]
        fz.adamw_allgather_peer(b[0], got, b[1], b[2], params, rank * S, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8,
                                weight_decay=0.1, step=rep + 1, gscale=scale)
        fz.peer_barrier(dist.group.WORLD, dev)
        torch.cuda.synchronize()
        out["adam_state_%d" % rep] = max(float((x - y).abs().max()) for x, y in zip(a, b))
        out["gathered_%d" % rep] = float((params.tensor.float() - full.float()).abs().max())
    out["status"] = _lib.read_status()
    out["allocator"] = "vmm" if type(grads.handle).__name__ == "VmmSymmetricBuffer" else "torch"
    return out


def train(cfg):
    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs
    from hetu_galvatron_b200.runtime.engine import build_model
    from hetu_galvatron_b200.runtime.optimizer import ShardedAdamW

    rank, t = _init()
    dev = torch.device("cuda", rank)
    args = GalvatronRuntimeArgs(
        parallel=dict(mixed_precision="bf16", default_dp_type=cfg["dp_type"], sdp=1 if cfg["dp_type"] == "zero3" else 0,
                      async_grad_reduce=cfg.get("defer", True), reduce_in_fp32=cfg.get("fp32_wire", False)),
        model=dict(model_size="llama-test", hidden_size=256, num_layers=3, num_attention_heads=4, ffn_hidden_size=768,
                   vocab_size=1024, make_vocab_size_divisible_by=8, normalization="RMSNorm",
                   activation_func="torch.nn.functional.silu", gated_linear_unit=True, num_query_groups=2),
        train=dict(seq_length=256, global_batch_size=8, chunks=2, lr=1e-3))
    model = build_model(args, device=dev, full_init=True, fused_zero=cfg["fused"])
    assert all(u.fused == cfg["fused"] for u in model.sharded_units if u.params)
    assert all(u.pooled == (not cfg.get("defer", True)) for u in model.sharded_units if u.params)
    opt = ShardedAdamW(model.sharded_units, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.01, clip_grad=1.0, device=dev)
    tok = torch.randint(0, 1024, (8, 257), generator=torch.Generator().manual_seed(3))
    mine = tok[rank * 4:(rank + 1) * 4].to(dev)
    out = []
    for it in range(4):
        opt.zero_grad()
        loss = model.forward_backward(mine[:, :-1], it, labels=mine[:, 1:])
        opt.step()
        out.append([float(loss), opt.grad_norm()])
    if cfg.get("report_guards"):
        from hetu_galvatron_b200.ops import _lib
        from hetu_galvatron_b200.parallel import fused_zero as fz

        _lib.assert_healthy()
        out.append(["guards", fz.verify_guards()])
    return out


REGISTRY = {"kernels_vs_nccl": kernels_vs_nccl, "train": train}
ENV = {"NCCL_NVLS_ENABLE": "0"}


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip("needs %d GPUs" % n)


@pytest.mark.parametrize("shard", [4096, 1 << 20])
def test_peer_kernels_match_nccl(shard):
    _need(2)
    res = run_distributed(__file__, "kernels_vs_nccl", 2, {"shard": shard}, timeout=240, extra_env=ENV)
    for r in res:
        assert r["status"] == 0, r
        for rep in range(2):
            assert r["rs_%d" % rep] < 1e-6 and r["adam_state_%d" % rep] < 1e-5 and r["gathered_%d" % rep] < 0.04, r
            assert r["rs16_%d" % rep] < 1e-6 and r["rs16_flags_%d" % rep] < 1e-6, r


def test_own_vmm_allocator_backs_the_peer_kernels():
    """HG_SYMM_ALLOC=vmm: the buffers come from this framework's own cuMemCreate / export / import / map allocator
    (descriptors passed between the ranks over Unix sockets); kernels and a training run give the same results."""
    _need(2)
    env = dict(ENV, HG_SYMM_ALLOC="vmm")
    res = run_distributed(__file__, "kernels_vs_nccl", 2, {"shard": 1 << 18}, timeout=240, extra_env=env)
    for r in res:
        assert r["status"] == 0 and r["allocator"] == "vmm", r
        for rep in range(2):
            assert r["rs_%d" % rep] < 1e-6 and r["adam_state_%d" % rep] < 1e-5 and r["gathered_%d" % rep] < 0.04, r
            assert r["rs16_%d" % rep] < 1e-6 and r["rs16_flags_%d" % rep] < 1e-6, r
    cfg = {"dp_type": "zero2", "defer": True, "fp32_wire": False}
    ref = run_distributed(__file__, "train", 2, dict(cfg, fused=True), timeout=300, extra_env=ENV)
    got = run_distributed(__file__, "train", 2, dict(cfg, fused=True), timeout=300, extra_env=env)
    for r in range(2):
        for (l0, n0), (l1, n1) in zip(ref[r], got[r]):
            assert abs(l0 - l1) / abs(l0) < 1e-4 and abs(n0 - n1) / n0 < 1e-3, (ref, got)


@pytest.mark.parametrize("dp_type,defer,fp32_wire", [("zero2", True, False), ("zero2", True, True), ("zero3", True, False),
                                                     ("zero2", False, False), ("zero3", False, True)])
def test_training_matches_nccl_path(dp_type, defer, fp32_wire):
    """Peer-memory reduce-scatter / AdamW + all-gather against the NCCL path of the same step, for both wire dtypes,
    with the reduction launched from the last backward (deferred) or after every micro-batch from pooled buffers."""
    _need(2)
    cfg = {"dp_type": dp_type, "defer": defer, "fp32_wire": fp32_wire}
    ref = run_distributed(__file__, "train", 2, dict(cfg, fused=False), timeout=300, extra_env=ENV)
    got = run_distributed(__file__, "train", 2, dict(cfg, fused=True), timeout=300, extra_env=ENV)
    for r in range(2):
        for (l0, n0), (l1, n1) in zip(ref[r], got[r]):
            assert abs(l0 - l1) / abs(l0) < 2e-3 and abs(n0 - n1) / n0 < 2e-2, (ref, got)


if __name__ == "__main__":
    func, payload = sys.argv[2], json.loads(sys.argv[3])
    out = REGISTRY[func](payload)
    with open(os.environ["HG_OUT"], "w") as f:
        json.dump(out, f)
    import torch.distributed as dist

    dist.barrier()
    torch.cuda.synchronize()
    dist.destroy_process_group()
