"""Peer-memory all-to-all kernels (2 GPUs): the Ulysses head/sequence exchange against the NCCL path, forward and
backward, including fewer kv heads than ranks; and the row-list gather used by the MoE dispatch."""
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
    from hetu_galvatron_b200.parallel.groups import CommGroup

    world = dist.get_world_size()
    return rank, world, CommGroup(list(range(world)), dist.group.WORLD, rank)


def rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def ulysses_vs_nccl(cfg):
    from types import SimpleNamespace

    from hetu_galvatron_b200.ops import _lib
    from hetu_galvatron_b200.parallel import fused_a2a as fa
    from hetu_galvatron_b200.parallel import ulysses as ul

    rank, p, grp = _init()
    dev = torch.device("cuda", rank)
    S, B, nh, ng, hd = cfg["S"], cfg["B"], cfg["nh"], cfg["ng"], cfg["hd"]
    out = {}
    for rep in range(3):  # three rounds: both staging parities and their reuse
        g = torch.Generator(device=dev).manual_seed(17 + rank + 10 * rep)
        mk = lambda n: torch.randn(S, B, n, hd, device=dev, dtype=torch.bfloat16, generator=g)  # noqa: E731
        q0, k0, v0 = mk(nh), mk(ng), mk(ng)
        # exchange alone (bitwise: both paths only move data)
        a = ul.seq_to_heads(q0, grp, p)
        b = fa.seq_to_heads(q0, grp, p)
        out["s2h_%d" % rep] = float((a.float() - b.float()).abs().max())
        out["h2s_%d" % rep] = float((ul.heads_to_seq(a, grp, p).float() - fa.heads_to_seq(b, grp, p).float()).abs().max())
        res = []
        for fused in (False, True):
            ctx = SimpleNamespace(sp_size=p, sp=grp, cp_size=1, cp=None, fused_comm=fused)
            q, k, v = (t.clone().requires_grad_() for t in (q0, k0, v0))
            o = ul.ulysses_attention(q, k, v, ctx, S * p)
            go = torch.randn(o.shape, device=dev, dtype=torch.bfloat16, generator=torch.Generator(device=dev).manual_seed(99 + rank))
            o.backward(go)
            res.append((o.detach(), q.grad, k.grad, v.grad))
        for name, x, y in zip(("o", "dq", "dk", "dv"), res[1], res[0]):
            out["%s_%d" % (name, rep)] = rel(x, y)
    torch.cuda.synchronize()
    out["status"] = _lib.read_status()
    return out


def rows_vs_torch(cfg):
    import torch.distributed as dist

    from hetu_galvatron_b200.ops import _lib
    from hetu_galvatron_b200.parallel import fused_a2a as fa

    rank, t, grp = _init()
    dev = torch.device("cuda", rank)
    T, H, K, n_out = cfg["T"], cfg["H"], cfg["K"], cfg["n_out"]
    g = torch.Generator(device=dev).manual_seed(3 + rank)
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16, generator=g)
    xs = [torch.empty_like(x) for _ in range(t)]
    dist.all_gather(xs, x)
    allx = torch.stack(xs)                                         # [t, T, H]
    gi = torch.Generator(device=dev).manual_seed(100 + rank)
    peer = torch.randint(-1, t, (n_out, K), device=dev, generator=gi, dtype=torch.int32)
    row = torch.randint(0, T, (n_out, K), device=dev, generator=gi, dtype=torch.int32)
    scale = torch.rand(n_out, K, device=dev, generator=gi)
    slot = fa.staging_for(grp, x.numel() * 2, dev).publish(x)
    out = {}
    got = fa.gather_rows(slot, peer, row, n_out, H, H, K, scale)
    picked = allx[peer.clamp(min=0).long(), row.long()].float() * (scale * (peer >= 0))[..., None]
    out["weighted"] = rel(got, picked.sum(1))
    if K == 1:
        plain = fa.gather_rows(slot, peer, row, n_out, H, H, 1, None)
        ref = allx[peer.clamp(min=0).long(), row.long()][:, 0] * (peer >= 0).to(torch.bfloat16)
        out["plain"] = float((plain.float() - ref.float()).abs().max())
    torch.cuda.synchronize()
    out["status"] = _lib.read_status()
    return out


def train_moe(cfg):
    """A small MoE / Ulysses model for 4 steps; cfg["fused"] switches the peer-memory kernels on."""
    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs
    from hetu_galvatron_b200.ops import _lib
    from hetu_galvatron_b200.runtime.engine import build_model
    from hetu_galvatron_b200.runtime.optimizer import ShardedAdamW

    rank, t, _ = _init()
    dev = torch.device("cuda", rank)
    model = dict(model_size="llama-test", hidden_size=256, num_layers=2, num_attention_heads=4, ffn_hidden_size=768,
                 vocab_size=1024, make_vocab_size_divisible_by=8, normalization="RMSNorm",
                 activation_func="torch.nn.functional.silu", gated_linear_unit=True, num_query_groups=2)
    model.update(cfg.get("model", {}))
    args = GalvatronRuntimeArgs(parallel=dict(mixed_precision="bf16", **cfg.get("parallel", {})), model=model,
                                train=dict(seq_length=cfg.get("seq", 256), global_batch_size=8, chunks=2, lr=1e-3))
    m = build_model(args, device=dev, full_init=True, fused_comm=cfg["fused"])
    opt = ShardedAdamW(m.sharded_units, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.01, clip_grad=1.0, device=dev)
    tok = torch.randint(0, 1024, (8, cfg.get("seq", 256) + 1), generator=torch.Generator().manual_seed(3))
    B = m.local_batch_size()
    d = m.vocab_ctx.dp.rank if m.vocab_ctx.dp is not None else 0
    mine = tok[d * B:(d + 1) * B].to(dev)
    out = []
    for it in range(4):
        opt.zero_grad()
        loss = m.forward_backward(mine[:, :-1], it, labels=mine[:, 1:])
        opt.step()
        out.append([float(loss), opt.grad_norm()])
    _lib.assert_healthy()
    return out


REGISTRY = {"ulysses_vs_nccl": ulysses_vs_nccl, "rows_vs_torch": rows_vs_torch, "train_moe": train_moe}
ENV = {"NCCL_NVLS_ENABLE": "0"}


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip("needs %d GPUs" % n)


@pytest.mark.parametrize("nh,ng", [(8, 8), (8, 2), (4, 1)])
def test_ulysses_exchange_matches_nccl(nh, ng):
    _need(2)
    res = run_distributed(__file__, "ulysses_vs_nccl", 2, {"S": 256, "B": 2, "nh": nh, "ng": ng, "hd": 64}, timeout=240,
                          extra_env=ENV)
    for r in res:
        assert r["status"] == 0, r
        for rep in range(3):
            assert r["s2h_%d" % rep] == 0.0 and r["h2s_%d" % rep] == 0.0, r
            for name in ("o", "dq", "dk", "dv"):
                assert r["%s_%d" % (name, rep)] < 1e-2, (name, r)


@pytest.mark.parametrize("K", [1, 2])
def test_row_gather_matches_indexing(K):
    _need(2)
    res = run_distributed(__file__, "rows_vs_torch", 2, {"T": 512, "H": 256, "K": K, "n_out": 777}, timeout=240, extra_env=ENV)
    for r in res:
        assert r["status"] == 0 and r["weighted"] < 5e-3, r
        if K == 1:
            assert r["plain"] == 0.0, r


MOE = {"num_moe_experts": 4, "moe_ffn_hidden_size": 256, "moe_router_topk": 2, "is_moe_model": True,
       "moe_token_dispatcher_type": "alltoall", "moe_aux_loss_coeff": 1e-2}


@pytest.mark.parametrize("name,cfg", [
    ("moe_ep2", {"parallel": {"global_ep_deg": 2}, "model": MOE}),
    ("ulysses_sp2", {"parallel": {"global_tp_deg": 2, "use_ulysses": True}}),
    ("reshard_tp_1_2_2_1", {"parallel": {"galvatron_config_path": {
        "pp_deg": 1, "tp_sizes_enc": "1,2", "tp_consecutive_flags": "1,1", "dp_types_enc": "0,0", "use_sp": "0,0",
        "checkpoint": "0,0", "global_bsz": 8, "chunks": 2, "pp_division": "2", "pipeline_type": "gpipe",
        "default_dp_type": "ddp", "vtp": 1, "vsp": 0, "embed_sdp": 0}}}),
])
def test_model_training_matches_nccl_path(name, cfg):
    _need(2)
    ref = run_distributed(__file__, "train_moe", 2, dict(cfg, fused=False), timeout=300, extra_env=ENV)
    got = run_distributed(__file__, "train_moe", 2, dict(cfg, fused=True), timeout=300, extra_env=ENV)
    for r in range(2):
        for (l0, n0), (l1, n1) in zip(ref[r], got[r]):
            assert abs(l0 - l1) / abs(l0) < 5e-3 and abs(n0 - n1) / n0 < 5e-2, (name, ref, got)


def test_ring_context_parallel_matches_the_all_gather_variant():
    """Zig-zag context parallelism over 2 GPUs: K/V blocks exchanged hop by hop with log-sum-exp merging (flash kernels
    at chunk offsets, merge kernel, dK/dV accumulators travelling with their block) against the all-gather variant."""
    _need(2)
    cfg = {"parallel": {"global_cp_deg": 2, "vocab_cp": 2}, "fused": False, "seq": 512}
    ref = run_distributed(__file__, "train_moe", 2, cfg, timeout=300, extra_env=dict(ENV, HG_CP_ALLGATHER="1"))
    got = run_distributed(__file__, "train_moe", 2, cfg, timeout=300, extra_env=ENV)
    for r in range(2):
        for (l0, n0), (l1, n1) in zip(ref[r], got[r]):
            assert abs(l0 - l1) / abs(l0) < 5e-3 and abs(n0 - n1) / n0 < 5e-2, (ref, got)


def moe_layer_without_host_syncs(cfg):
    """One MoE decoder layer, forward + backward, under ``set_sync_debug_mode("error")`` after a warm-up pass: the
    statically sized peer-memory dispatcher builds its routing table on the device."""
    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs
    from hetu_galvatron_b200.ops import _lib
    from hetu_galvatron_b200.parallel import fused_a2a as fa
    from hetu_galvatron_b200.runtime.engine import build_model

    rank, t, _ = _init()
    dev = torch.device("cuda", rank)
    model = dict(model_size="llama-test", hidden_size=256, num_layers=1, num_attention_heads=4, ffn_hidden_size=768,
                 vocab_size=1024, make_vocab_size_divisible_by=8, normalization="RMSNorm",
                 activation_func="torch.nn.functional.silu", gated_linear_unit=True, **MOE)
    model.update(moe_token_dispatcher_type="flex", moe_grouped_gemm=True, moe_expert_buffer_factor=2.0,
                 moe_aux_loss_coeff=0.0)
    args = GalvatronRuntimeArgs(parallel=dict(mixed_precision="bf16", global_ep_deg=2), model=model,
                                train=dict(seq_length=256, global_batch_size=4, chunks=1, lr=1e-3))
    m = build_model(args, device=dev, full_init=True, fused_comm=True)
    layer = [u for lp, u in m.named_units() if lp.startswith("moe_decoder")][0]
    x = torch.randn(256, 2, 256, device=dev, dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(256, 2, 256, device=dev, dtype=torch.bfloat16)
    layer(x).backward(g)                   # warm-up: staging buffers, workspaces, kernel modules
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        y = layer(x)
        y.backward(g)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.cuda.synchronize()
    _lib.assert_healthy()
    return {"dropped": fa.read_overflow(dev), "finite": bool(torch.isfinite(x.grad.float()).all())}


REGISTRY["moe_layer_without_host_syncs"] = moe_layer_without_host_syncs


def test_moe_layer_has_no_host_synchronisation_with_static_expert_buffers():
    _need(2)
    res = run_distributed(__file__, "moe_layer_without_host_syncs", 2, {}, timeout=300, extra_env=ENV)
    for r in res:
        assert r["dropped"] == 0 and r["finite"], res


def test_static_expert_buffers_train_like_exact_ones():
    """``moe_expert_buffer_factor`` (device-built routing table, static buffers) against the exactly sized buffers."""
    _need(2)
    base = {"parallel": {"global_ep_deg": 2}, "fused": True}
    ref = run_distributed(__file__, "train_moe", 2, dict(base, model=dict(MOE, moe_grouped_gemm=True)), timeout=300, extra_env=ENV)
    got = run_distributed(__file__, "train_moe", 2, dict(base, model=dict(MOE, moe_grouped_gemm=True, moe_expert_buffer_factor=2.0)),
                          timeout=300, extra_env=ENV)
    for r in range(2):
        for (l0, n0), (l1, n1) in zip(ref[r], got[r]):
            assert abs(l0 - l1) / abs(l0) < 2e-3 and abs(n0 - n1) / n0 < 2e-2, (ref, got)


def test_flex_dispatcher_selects_the_pull_kernels():
    """``moe_token_dispatcher_type: flex`` runs the fused dispatcher without the global switch and trains like
    the all-to-all dispatcher."""
    _need(2)
    ref = run_distributed(__file__, "train_moe", 2, {"parallel": {"global_ep_deg": 2}, "model": MOE, "fused": False},
                          timeout=300, extra_env=ENV)
    got = run_distributed(__file__, "train_moe", 2,
                          {"parallel": {"global_ep_deg": 2}, "model": dict(MOE, moe_token_dispatcher_type="flex"),
                           "fused": False}, timeout=300, extra_env=ENV)
    for r in range(2):
        for (l0, n0), (l1, n1) in zip(ref[r], got[r]):
            assert abs(l0 - l1) / abs(l0) < 5e-3 and abs(n0 - n1) / n0 < 5e-2, (ref, got)


if __name__ == "__main__":
    func, payload = sys.argv[2], json.loads(sys.argv[3])
    out = REGISTRY[func](payload)
    with open(os.environ["HG_OUT"], "w") as f:
        json.dump(out, f)
    import torch.distributed as dist

    dist.barrier()
    torch.cuda.synchronize()
    dist.destroy_process_group()
