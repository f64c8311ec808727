"""Every parallelism path on CPU ranks (gloo, fp32): loss parity against the single-process model.

DP / ZeRO-2 / ZeRO-3 (deferred and immediate reduction), Megatron TP+SP, vocab TP, Ulysses SP (incl. fewer kv
heads than ranks), zig-zag context parallelism, GPipe and 1F1B-flush pipelines, layer-wise heterogeneous
strategies with resharding, tied embeddings across pipeline stages, activation checkpointing, MoE with
expert parallelism."""
import json
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tests.dist_utils import run_distributed, worker_main  # noqa: E402

STEPS = 3
GBSZ, SEQ, VOCAB = 8, 128, 1024


def make_args(cfg):
    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs

    model = dict(model_size="llama-test", hidden_size=256, num_layers=4, num_attention_heads=4, ffn_hidden_size=688,
                 vocab_size=VOCAB, normalization="RMSNorm", activation_func="torch.nn.functional.silu",
                 gated_linear_unit=True, make_vocab_size_divisible_by=8)
    model.update(cfg.get("model", {}))
    parallel = dict(mixed_precision="fp32")
    parallel.update(cfg.get("parallel", {}))
    train = dict(seq_length=SEQ, global_batch_size=GBSZ, chunks=cfg.get("chunks", 1), lr=1e-3, seed=1234)
    train.update(cfg.get("train", {}))
    return GalvatronRuntimeArgs(parallel=parallel, model=model, train=train)


def train(cfg):
    import torch
    import torch.distributed as dist

    from hetu_galvatron_b200.runtime.engine import build_model
    from hetu_galvatron_b200.runtime.optimizer import ShardedAdamW

    torch.manual_seed(0)
    args = make_args(cfg)
    model = build_model(args, device=torch.device("cpu"), full_init=True)
    opt = ShardedAdamW(model.sharded_units, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.01, clip_grad=1.0)
    g = torch.Generator().manual_seed(7)
    tok = torch.randint(0, VOCAB, (GBSZ, SEQ + 1), generator=g)
    B = model.local_batch_size()
    d = model.vocab_ctx.dp.rank if model.vocab_ctx.dp is not None else 0
    mine = tok[d * B:(d + 1) * B]
    out = []
    for it in range(STEPS):
        opt.zero_grad()
        loss = model.forward_backward(mine[:, :-1], it, labels=mine[:, 1:])
        model.sync_tied_embedding_grads()
        opt.step()
        val = float(loss) if loss is not None else None
        out.append([val, opt.grad_norm()])
    return out


def generate(cfg):
    """Greedy continuation through the key / value cache on this strategy; returns the generated tokens."""
    import torch

    from hetu_galvatron_b200.models.inference import StaticInferenceContext, forward_step, greedy_generate
    from hetu_galvatron_b200.runtime.engine import build_model

    torch.manual_seed(0)
    args = make_args(cfg)
    model = build_model(args, device=torch.device("cpu"), full_init=True)
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, VOCAB, (2, 16), generator=g)
    out = greedy_generate(model, prompt, 4, vocab_group=model.vocab_ctx.tp, new_tokens_per_step=cfg.get("per_step", 1))
    # the cached logits of the prompt equal the plain forward's
    ctx = StaticInferenceContext(2, 32)
    cached = forward_step(model, prompt, ctx)
    with torch.no_grad():
        plain = model.model(prompt, None)
    return {"tokens": out.tolist(), "diff": float((cached - plain).abs().max())}


REGISTRY = {"train": train, "generate": generate}

_baselines = {}


def baseline(key, cfg):
    if key not in _baselines:
        _baselines[key] = run_distributed(__file__, "train", 1, cfg)[0]
    return _baselines[key]


def check(world, cfg, base_cfg=None, key="dense", rtol=2e-4, norm_rtol=2e-3):
    ref = baseline(key, base_cfg or {"chunks": 1})
    res = run_distributed(__file__, "train", world, cfg)
    seen = False
    for r in res:
        for (l, n), (l0, n0) in zip(r, ref):
            if l is not None:
                seen = True
                assert abs(l - l0) / abs(l0) < rtol, (cfg, res, ref)
            assert abs(n - n0) / abs(n0) < norm_rtol, (cfg, res, ref)
    assert seen


@pytest.mark.parametrize("dp_type,async_reduce,chunks", [("ddp", True, 1), ("zero2", True, 2), ("zero3", True, 2),
                                                         ("zero3", False, 2), ("zero2", False, 1)])
def test_data_parallel_and_zero(dp_type, async_reduce, chunks):
    check(2, {"chunks": chunks, "parallel": {"default_dp_type": dp_type, "sdp": 1 if dp_type == "zero3" else 0,
                                             "async_grad_reduce": async_reduce}})


@pytest.mark.parametrize("mp", ["bf16", "fp16"])
def test_mixed_precision_data_parallel(mp):
    """16-bit parameters and activations with fp32 master weights and fp32 gradient reduction: two ZeRO-2 ranks
    against one process at the same precision (the counterpart of the reference's tests/core/test_mixed_precision.py)."""
    base = {"chunks": 1, "parallel": {"mixed_precision": mp}}
    check(2, {"chunks": 2, "parallel": {"mixed_precision": mp, "default_dp_type": "zero2"}}, base, key="mp_" + mp,
          rtol=2e-3, norm_rtol=2e-2)


def test_tensor_parallel_with_sequence_parallel_and_vocab_tp():
    check(2, {"parallel": {"global_tp_deg": 2, "vocab_tp": 2}})


def test_tp2_dp2_zero3_checkpoint():
    check(4, {"chunks": 2, "parallel": {"global_tp_deg": 2, "vocab_tp": 1, "sdp": 1, "global_checkpoint": 1}})


def test_qk_layernorm_under_tensor_and_data_parallelism():
    """Per-head query / key normalisation: its weights are replicated over the tensor-parallel ranks (each sees its own
    heads), so their gradients are summed over tp; with ``test_mode`` every forward cross-checks the copies."""
    model = {"qk_layernorm": True, "num_query_groups": 2}
    base = {"chunks": 1, "model": model}
    check(4, {"chunks": 2, "parallel": {"global_tp_deg": 2, "vocab_tp": 2, "default_dp_type": "zero2"}, "model": model,
              "train": {"test_mode": True}}, base, key="qkln")
    check(2, {"parallel": {"global_tp_deg": 2, "use_ulysses": True, "vocab_tp": 2}, "model": model}, base, key="qkln")


@pytest.mark.parametrize("kv", [None, 1])
def test_ulysses(kv):
    model = {"num_query_groups": kv} if kv else {}
    base = {"chunks": 1, "model": model}
    check(2, {"parallel": {"global_tp_deg": 2, "use_ulysses": True, "vocab_tp": 2}, "model": model}, base,
          key="kv%s" % kv)


def test_context_parallel_zigzag():
    check(2, {"parallel": {"global_cp_deg": 2, "vocab_cp": 2}})


def test_context_parallel_ring_of_four_and_all_gather_variant():
    """Four ranks: K/V blocks make three hops, the dK/dV accumulators four; the all-gather variant gives the same."""
    check(4, {"parallel": {"global_cp_deg": 4, "vocab_cp": 4}})
    res = run_distributed(__file__, "train", 4, {"parallel": {"global_cp_deg": 4, "vocab_cp": 4}},
                          extra_env={"HG_CP_ALLGATHER": "1"})
    ref = baseline("dense", {"chunks": 1})
    assert abs(res[0][0][0] - ref[0][0]) / ref[0][0] < 2e-4 and abs(res[0][2][1] - ref[2][1]) / ref[2][1] < 2e-3


def test_ring_step_pairs_cover_the_causal_triangle_once():
    from hetu_galvatron_b200.parallel.ring_attention import step_pairs

    for c in (2, 3, 4, 8):
        seen = {}
        for r in range(c):
            for t in range(c):
                src = (r - t) % c
                qc, kc = (r, 2 * c - 1 - r), (src, 2 * c - 1 - src)
                for qi, kj in step_pairs(r, src, c):
                    key = (qc[qi], kc[kj])
                    assert key not in seen
                    seen[key] = True
        assert set(seen) == {(i, j) for i in range(2 * c) for j in range(i + 1)}
        # balanced: every rank computes the same number of pairs
        assert len({sum(len(step_pairs(r, (r - t) % c, c)) for t in range(c)) for r in range(c)}) == 1


@pytest.mark.parametrize("ptype,chunks", [("gpipe", 2), ("pipedream_flush", 4)])
def test_pipeline(ptype, chunks):
    check(2, {"chunks": chunks, "parallel": {"pp_deg": 2, "pipeline_type": ptype}})


def test_pipeline_four_stages():
    """Four stages (middle stages belong to no embedding group): 1F1B-flush and GPipe, receives posted one step
    ahead on direction-separated communicators."""
    check(4, {"chunks": 4, "parallel": {"pp_deg": 4, "pipeline_type": "pipedream_flush"}})
    check(4, {"chunks": 2, "parallel": {"pp_deg": 4, "pipeline_type": "gpipe"}})


def test_one_f_one_b_step_lists():
    from hetu_galvatron_b200.parallel.pipeline import one_f_one_b_steps

    assert one_f_one_b_steps(0, 2, 3) == [("F", 0), ("F", 1), ("B", 0), ("F", 2), ("B", 1), ("B", 2)]
    assert one_f_one_b_steps(1, 2, 3) == [("F", 0), ("B", 0), ("F", 1), ("B", 1), ("F", 2), ("B", 2)]
    for stage in range(4):     # every micro-batch once forward, once backward, backward after its forward
        st = one_f_one_b_steps(stage, 4, 2)
        assert sorted(st) == sorted([("F", 0), ("F", 1), ("B", 0), ("B", 1)])
        assert all(st.index(("F", i)) < st.index(("B", i)) for i in range(2))


def test_reduce_in_fp32_and_low_precision_wire():
    """bf16 parameters: gradients cross the links in bf16 by default and in fp32 with ``reduce_in_fp32``; both match
    one process at the same precision."""
    base = {"chunks": 1, "parallel": {"mixed_precision": "bf16"}}
    for fp32 in (False, True):
        for dp_type, defer in (("zero3", False), ("ddp", True)):
            check(2, {"chunks": 2, "parallel": {"mixed_precision": "bf16", "default_dp_type": dp_type,
                                                "sdp": 1 if dp_type == "zero3" else 0, "reduce_in_fp32": fp32,
                                                "async_grad_reduce": defer}},
                  base, key="mp_bf16", rtol=2e-3, norm_rtol=2e-2)


def test_pipeline_tied_embeddings_immediate_reduction():
    """Tied embedding / LM-head copies on two stages exchange their gradients also when every other unit reduces
    after each micro-batch (``async_grad_reduce=False``)."""
    model = {"untie_embeddings_and_output_weights": False}
    check(4, {"chunks": 2, "parallel": {"pp_deg": 2, "pipeline_type": "gpipe", "default_dp_type": "zero2",
                                        "async_grad_reduce": False}, "model": model},
          {"chunks": 1, "model": model}, key="tied")


def test_pipeline_tied_embeddings_tp():
    model = {"untie_embeddings_and_output_weights": False}
    check(4, {"chunks": 2, "parallel": {"pp_deg": 2, "pipeline_type": "pipedream_flush", "global_tp_deg": 2,
                                        "vocab_tp": 2}, "model": model}, {"chunks": 1, "model": model}, key="tied")


def test_layerwise_heterogeneous_strategy():
    strategy = {"pp_deg": 1, "tp_sizes_enc": "1,2,4,2", "tp_consecutive_flags": "1,1,1,1", "dp_types_enc": "0,1,0,1",
                "use_sp": "0,0,0,1", "checkpoint": "0,1,0,0", "global_bsz": GBSZ, "chunks": 2, "pp_division": "4",
                "pipeline_type": "gpipe", "default_dp_type": "zero2", "vtp": 2, "vsp": 0, "embed_sdp": 1}
    check(4, {"parallel": {"galvatron_config_path": strategy}})


def test_cached_generation_under_tensor_parallelism():
    """Vocab- and tensor-parallel ranks generate the same tokens as one process (two tokens per step keep the
    sequence-parallel activations divisible by the tp degree)."""
    one = run_distributed(__file__, "generate", 1, {"per_step": 2})
    two = run_distributed(__file__, "generate", 2, {"per_step": 2, "parallel": {"global_tp_deg": 2, "vocab_tp": 2}})
    assert one[0]["diff"] < 1e-5 and all(r["diff"] < 1e-5 for r in two)
    assert two[0]["tokens"] == two[1]["tokens"] == one[0]["tokens"]


def test_moe_expert_parallel():
    model = {"num_moe_experts": 4, "moe_ffn_hidden_size": 256, "moe_router_topk": 2, "is_moe_model": True,
             "moe_token_dispatcher_type": "alltoall", "moe_aux_loss_coeff": 1e-2}
    base = {"chunks": 1, "model": model}
    check(2, {"parallel": {"global_ep_deg": 2}, "model": model}, base, key="moe", rtol=1e-3, norm_rtol=2e-2)


MOE = {"num_moe_experts": 4, "moe_ffn_hidden_size": 256, "moe_router_topk": 2, "is_moe_model": True,
       "moe_token_dispatcher_type": "alltoall", "moe_aux_loss_coeff": 1e-2}


def test_moe_grouped_and_sequential_experts_agree():
    """``moe_grouped_gemm`` selects one grouped contraction over all experts or a loop over them: same training."""
    base = {"chunks": 1, "model": MOE}
    check(2, {"parallel": {"global_ep_deg": 2}, "model": dict(MOE, moe_grouped_gemm=True)}, base, key="moe", rtol=1e-3,
          norm_rtol=2e-2)


def test_moe_allgather_dispatcher():
    base = {"chunks": 1, "model": MOE}
    check(2, {"parallel": {"global_ep_deg": 2}, "model": dict(MOE, moe_token_dispatcher_type="allgather")}, base,
          key="moe", rtol=1e-3, norm_rtol=2e-2)


def test_moe_flex_dispatcher_name_is_accepted():
    # "flex" picks the peer-memory kernels on GPUs; on CPU ranks it takes the all-to-all path
    base = {"chunks": 1, "model": MOE}
    check(2, {"parallel": {"global_ep_deg": 2}, "model": dict(MOE, moe_token_dispatcher_type="flex")}, base,
          key="moe", rtol=1e-3, norm_rtol=2e-2)


def test_moe_expert_tensor_parallel():
    base = {"chunks": 1, "model": MOE}
    check(4, {"parallel": {"global_ep_deg": 2, "global_tp_of_ep_deg": 2}, "model": MOE}, base, key="moe", rtol=1e-3,
          norm_rtol=2e-2)


def test_moe_shared_experts():
    model = dict(MOE, moe_shared_expert_intermediate_size=128)
    base = {"chunks": 1, "model": model}
    check(2, {"parallel": {"global_ep_deg": 2}, "model": model}, base, key="moe_shared", rtol=1e-3, norm_rtol=2e-2)
    check(2, {"parallel": {"global_tp_deg": 2, "vocab_tp": 2}, "model": model}, base, key="moe_shared", rtol=1e-3, norm_rtol=2e-2)


if __name__ == "__main__":
    worker_main(REGISTRY)
