"""Checkpoints on CPU: HuggingFace -> split files -> (tensor-parallel) shards with loss parity against the
HuggingFace model itself, distributed save -> resume giving the same losses as an uninterrupted run, and export back
to HuggingFace names."""
import json
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tests.dist_utils import run_distributed, worker_main  # noqa: E402

H, L, NH, NKV, FFN, V, SEQ, GB = 64, 2, 4, 2, 96, 256, 32, 4


def make_args(parallel=None, ckpt=None, train=None):
    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs

    p = dict(mixed_precision="fp32")
    p.update(parallel or {})
    t = dict(seq_length=SEQ, global_batch_size=GB, chunks=1, lr=1e-3, seed=3, train_iters=4, lr_warmup_fraction=0.25,
             min_lr=1e-4, clip_grad=1.0)
    t.update(train or {})
    return GalvatronRuntimeArgs(
        parallel=p, ckpt=ckpt or {}, train=t, data=dict(use_random_dataset=True),
        model=dict(model_size="llama-test", hidden_size=H, num_layers=L, num_attention_heads=NH, num_query_groups=NKV,
                   ffn_hidden_size=FFN, vocab_size=V, normalization="RMSNorm", gated_linear_unit=True,
                   activation_func="torch.nn.functional.silu", untie_embeddings_and_output_weights=True,
                   make_vocab_size_divisible_by=8, norm_epsilon=1e-5))


def hf_model():
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(11)
    cfg = LlamaConfig(hidden_size=H, num_hidden_layers=L, num_attention_heads=NH, num_key_value_heads=NKV,
                      intermediate_size=FFN, vocab_size=V, rms_norm_eps=1e-5, max_position_embeddings=SEQ,
                      tie_word_embeddings=False, attention_bias=False, rope_theta=10000.0)
    return LlamaForCausalLM(cfg).eval()


def batch():
    g = torch.Generator().manual_seed(5)
    return torch.randint(0, V, (GB, SEQ + 1), generator=g)


def loss_from_split(cfg):
    """Build the model under cfg["parallel"], load the split files, return the loss on the fixed batch."""
    from hetu_galvatron_b200.runtime import checkpoint as ck
    from hetu_galvatron_b200.runtime.engine import build_model

    model = build_model(make_args(cfg.get("parallel")), device=torch.device("cpu"))
    ck.load_hf_split(model, cfg["dir"])
    tok = batch()
    B = model.local_batch_size()
    d = model.vocab_ctx.dp.rank if model.vocab_ctx.dp is not None else 0
    mine = tok[d * B:(d + 1) * B]
    loss = model.forward_backward(mine[:, :-1], 0, labels=mine[:, 1:], forward_only=True)
    return float(loss) if loss is not None else None


def train_and_resume(cfg):
    """cfg["phase"]: "full" trains 4 iterations saving at 2; "resume" loads iteration 2 and trains 2 more."""
    from hetu_galvatron_b200.runtime.initialize import initialize_galvatron
    from hetu_galvatron_b200.runtime.trainer import train

    ck = dict(save=cfg["dir"], save_interval=2) if cfg["phase"] == "full" else \
        dict(load=cfg["dir"], load_iteration=2, distributed_checkpoint=True)
    args = make_args(cfg.get("parallel"), ckpt=ck)
    initialize_galvatron(args, backend="gloo")
    return train(args)


def moe_args(parallel=None, model=None):
    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs

    p = dict(mixed_precision="fp32")
    p.update(parallel or {})
    m = dict(model_size="mixtral-test", hidden_size=H, num_layers=L, num_attention_heads=NH, num_query_groups=NKV,
             vocab_size=V, normalization="RMSNorm", gated_linear_unit=True, activation_func="torch.nn.functional.silu",
             untie_embeddings_and_output_weights=True, make_vocab_size_divisible_by=8, norm_epsilon=1e-5,
             is_moe_model=True, num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=FFN, rotary_base=1000000)
    m.update(model or {})
    return GalvatronRuntimeArgs(parallel=p, model=m, data=dict(use_random_dataset=True),
                                train=dict(seq_length=SEQ, global_batch_size=GB, chunks=1, lr=1e-3, seed=3))


def moe_loss_from_split(cfg):
    from hetu_galvatron_b200.runtime import checkpoint as ck
    from hetu_galvatron_b200.runtime.engine import build_model

    model = build_model(moe_args(cfg.get("parallel"), cfg.get("model")), device=torch.device("cpu"))
    ck.load_hf_split(model, cfg["dir"])
    tok = batch()
    B = model.local_batch_size()
    d = model.vocab_ctx.dp.rank if model.vocab_ctx.dp is not None else 0
    mine = tok[d * B:(d + 1) * B]
    loss = model.forward_backward(mine[:, :-1], 0, labels=mine[:, 1:], forward_only=True)
    return float(loss) if loss is not None else None


REGISTRY = {"loss_from_split": loss_from_split, "train_and_resume": train_and_resume,
            "moe_loss_from_split": moe_loss_from_split}


@pytest.fixture(scope="module")
def split_dir(tmp_path_factory):
    from hetu_galvatron_b200.runtime import checkpoint as ck

    d = tmp_path_factory.mktemp("split")
    m = hf_model()
    files = ck.convert_hf_to_split(m.state_dict(), "llama", str(d))
    assert "model_embed_tokens.pt" in files and "model_layers_1.pt" in files and "model_norm.pt" in files and "lm_head.pt" in files
    keys = set(torch.load(d / "model_layers_0.pt", weights_only=True))
    assert {"self_attn.q_proj.weight", "mlp.gate_proj.weight", "input_layernorm.weight"} <= keys
    tok = batch()
    with torch.no_grad():
        ref = m(input_ids=tok[:, :-1], labels=None).logits.float()
    loss = torch.nn.functional.cross_entropy(ref.reshape(-1, V), tok[:, 1:].reshape(-1)).item()
    return str(d), loss, m


@pytest.fixture(scope="module")
def mixtral_split(tmp_path_factory):
    from transformers import MixtralConfig, MixtralForCausalLM

    from hetu_galvatron_b200.runtime import checkpoint as ck

    torch.manual_seed(21)
    cfg = MixtralConfig(hidden_size=H, num_hidden_layers=L, num_attention_heads=NH, num_key_value_heads=NKV,
                        intermediate_size=FFN, vocab_size=V, rms_norm_eps=1e-5, max_position_embeddings=SEQ,
                        num_local_experts=4, num_experts_per_tok=2, tie_word_embeddings=False, router_aux_loss_coef=0.0,
                        sliding_window=None, rope_theta=1000000.0)
    m = MixtralForCausalLM(cfg).eval()
    d = tmp_path_factory.mktemp("mixtral_split")
    ck.convert_hf_to_split(m.state_dict(), "mixtral", str(d))
    tok = batch()
    with torch.no_grad():
        logits = m(input_ids=tok[:, :-1]).logits.float()
    loss = torch.nn.functional.cross_entropy(logits.reshape(-1, V), tok[:, 1:].reshape(-1)).item()
    return str(d), loss


@pytest.mark.parametrize("world,parallel,model", [
    (1, {}, {}),
    (2, dict(global_ep_deg=2), dict(moe_token_dispatcher_type="alltoall")),
    (2, dict(global_ep_deg=2), dict(moe_token_dispatcher_type="allgather")),
])
def test_mixtral_hf_weights_give_hf_loss(mixtral_split, world, parallel, model):
    """Router, dispatch, experts and combine against HuggingFace's Mixtral with the same weights."""
    d, hf_loss = mixtral_split
    res = run_distributed(__file__, "moe_loss_from_split", world, {"dir": d, "parallel": parallel, "model": model})
    seen = [r for r in res if r is not None]
    assert seen and all(abs(r - hf_loss) / hf_loss < 1e-4 for r in seen), (res, hf_loss)


def test_qkv_pack_roundtrip():
    from hetu_galvatron_b200.runtime.checkpoint import pack_qkv, unpack_qkv

    q, k, v = torch.randn(NH * 16, H), torch.randn(NKV * 16, H), torch.randn(NKV * 16, H)
    q2, k2, v2 = unpack_qkv(pack_qkv(q, k, v, NH, NKV, 16), NH, NKV, 16)
    assert torch.equal(q, q2) and torch.equal(k, k2) and torch.equal(v, v2)


def test_hf_weights_give_hf_loss_single_process(split_dir):
    d, hf_loss, _ = split_dir
    ours = run_distributed(__file__, "loss_from_split", 1, {"dir": d})[0]
    assert abs(ours - hf_loss) / hf_loss < 1e-4, (ours, hf_loss)


@pytest.mark.parametrize("parallel", [dict(global_tp_deg=2, vocab_tp=2), dict(pp_deg=2, pipeline_type="gpipe"),
                                      dict(default_dp_type="zero3", sdp=1)])
def test_hf_weights_give_hf_loss_when_sharded(split_dir, parallel):
    d, hf_loss, _ = split_dir
    res = run_distributed(__file__, "loss_from_split", 2, {"dir": d, "parallel": parallel})
    seen = [r for r in res if r is not None]
    assert seen and all(abs(r - hf_loss) / hf_loss < 1e-4 for r in seen), (res, hf_loss)


@pytest.mark.parametrize("world,parallel", [(1, {}), (2, dict(global_tp_deg=2, vocab_tp=2, default_dp_type="zero2"))])
def test_save_resume_continues_identically(tmp_path, world, parallel):
    d = str(tmp_path / "ckpt")
    full = run_distributed(__file__, "train_and_resume", world, {"dir": d, "phase": "full", "parallel": parallel})
    assert os.path.exists(os.path.join(d, "hybrid_parallel_configs.json"))
    assert os.path.exists(os.path.join(d, "iter_2", "model_layers_0", "0.pt"))
    assert os.path.exists(os.path.join(d, "iter_2", "optimizer", "%d.pt" % (world - 1)))
    sched = json.load(open(os.path.join(d, "iter_2", "opt_param_scheduler.json")))
    assert sched["num_steps"] == 2 * GB
    resumed = run_distributed(__file__, "train_and_resume", world, {"dir": d, "phase": "resume", "parallel": parallel})
    for r in range(world):
        assert len(resumed[r]) == 2
        for a, b in zip(resumed[r], full[r][2:]):
            assert abs(a - b) / abs(b) < 1e-5, (resumed, full)


def test_strategy_mismatch_is_refused(tmp_path):
    d = str(tmp_path / "ckpt")
    run_distributed(__file__, "train_and_resume", 1, {"dir": d, "phase": "full"})
    with pytest.raises(AssertionError):
        run_distributed(__file__, "train_and_resume", 2, {"dir": d, "phase": "resume", "parallel": dict(global_tp_deg=2, vocab_tp=2)})


def test_export_back_to_hf_names(split_dir, tmp_path):
    from hetu_galvatron_b200.models.spec import spec_from_args
    from hetu_galvatron_b200.config.model_config import resolve_model_config
    from hetu_galvatron_b200.runtime import checkpoint as ck
    from hetu_galvatron_b200.runtime.engine import build_model
    from hetu_galvatron_b200.runtime.optimizer import ShardedAdamW

    d, _, m = split_dir
    args = make_args()
    model = build_model(args, device=torch.device("cpu"))
    ck.load_hf_split(model, d)
    opt = ShardedAdamW(model.sharded_units, lr=1e-3)
    out = str(tmp_path / "dist")
    ck.save_distributed_checkpoint(model, opt, None, 7, out)
    sd = ck.export_to_hf(out, 7, model.spec)
    ref = m.state_dict()
    for k, v in ref.items():
        if "rotary" in k:
            continue
        assert k in sd, k
        assert torch.allclose(sd[k].float(), v.float(), atol=1e-6), k


if __name__ == "__main__":
    worker_main(REGISTRY)


def test_bert_mlm_checkpoint_is_regrouped_like_the_reference_tool(tmp_path):
    """Key layout of the reference's tests/models/test_checkpoint_convert.py."""
    import torch

    from hetu_galvatron_b200.cli import checkpoint_convert_h2g as h2g

    src, dst = tmp_path / "hf", tmp_path / "split"
    src.mkdir()
    keys = ["bert.embeddings.word_embeddings.weight", "bert.embeddings.LayerNorm.bias",
            "bert.encoder.layer.0.attention.self.query.weight", "bert.encoder.layer.0.output.LayerNorm.bias",
            "bert.encoder.layer.1.intermediate.dense.weight", "bert.pooler.dense.weight",
            "cls.predictions.transform.dense.weight", "cls.predictions.decoder.weight", "cls.predictions.bias"]
    torch.save({k: torch.randn(3, 2) for k in keys}, src / "bert_model.bin")
    files = h2g.main(["--model_type", "bert-mlm", "--input_checkpoint", str(src), "--output_dir", str(dst)])
    assert files == ["bert_embeddings.pt", "bert_encoder_layer_0.pt", "bert_encoder_layer_1.pt", "bert_pooler.pt",
                     "cls_predictions.pt"]
    assert set(torch.load(dst / "bert_embeddings.pt")) == {"word_embeddings.weight", "LayerNorm.bias"}
    assert set(torch.load(dst / "bert_encoder_layer_0.pt")) == {"attention.self.query.weight", "output.LayerNorm.bias"}
    assert set(torch.load(dst / "cls_predictions.pt")) == {"transform.dense.weight", "decoder.weight", "bias"}


def _family_loss(model_type, model_kw, state_dict, tmp):
    """Split an HF state dict, load it into our model of the same shape, return the loss on the fixed batch."""
    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs
    from hetu_galvatron_b200.runtime import checkpoint as ck
    from hetu_galvatron_b200.runtime.engine import build_model

    ck.convert_hf_to_split(state_dict, model_type, str(tmp))
    args = GalvatronRuntimeArgs(parallel=dict(mixed_precision="fp32"), data=dict(use_random_dataset=True),
                                train=dict(seq_length=SEQ, global_batch_size=GB, chunks=1, lr=1e-3, seed=3),
                                model=model_kw)
    m = build_model(args, device=torch.device("cpu"))
    ck.load_hf_split(m, str(tmp))
    tok = batch()
    return float(m.forward_backward(tok[:, :-1], 0, labels=tok[:, 1:], forward_only=True))


def _hf_loss(m):
    tok = batch()
    with torch.no_grad():
        lg = m(input_ids=tok[:, :-1]).logits.float()
    return torch.nn.functional.cross_entropy(lg.reshape(-1, lg.shape[-1]), tok[:, 1:].reshape(-1)).item()


def test_gpt2_hf_weights_give_hf_loss(tmp_path):
    """GPT-2 family: learned positions, LayerNorm, biases, tanh-GELU, tied embeddings, HF's transposed Conv1D weights."""
    from transformers import GPT2Config, GPT2LMHeadModel

    torch.manual_seed(31)
    hf = GPT2LMHeadModel(GPT2Config(n_embd=H, n_layer=L, n_head=NH, n_inner=4 * H, vocab_size=V, n_positions=SEQ,
                                    resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0,
                                    activation_function="gelu_new")).eval()
    with torch.no_grad():                      # biases and norm weights away from their 0 / 1 initial values
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.05 * torch.randn_like(p))
    ours = _family_loss("gpt", dict(model_size="gpt-test", hidden_size=H, num_layers=L, num_attention_heads=NH,
                                    ffn_hidden_size=4 * H, vocab_size=V, normalization="LayerNorm",
                                    activation_func="torch.nn.functional.gelu", gated_linear_unit=False,
                                    position_embedding_type="learned_absolute", add_bias_linear=True,
                                    add_qkv_bias=True, make_vocab_size_divisible_by=8, norm_epsilon=1e-5),
                        hf.state_dict(), tmp_path)
    ref = _hf_loss(hf)
    assert abs(ours - ref) / ref < 1e-4, (ours, ref)


def test_qwen2_hf_weights_give_hf_loss(tmp_path):
    """Qwen-2 family: Llama-style layers with biases on q / k / v only, GQA, rope base 1e6."""
    from transformers import Qwen2Config, Qwen2ForCausalLM

    torch.manual_seed(32)
    hf = Qwen2ForCausalLM(Qwen2Config(hidden_size=H, num_hidden_layers=L, num_attention_heads=NH,
                                      num_key_value_heads=NKV, intermediate_size=FFN, vocab_size=V, rms_norm_eps=1e-6,
                                      max_position_embeddings=SEQ, tie_word_embeddings=False, rope_theta=1000000.0,
                                      use_sliding_window=False)).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias"):
                p.copy_(0.1 * torch.randn_like(p))
    ours = _family_loss("qwen", dict(model_size="qwen-test", hidden_size=H, num_layers=L, num_attention_heads=NH,
                                     num_query_groups=NKV, ffn_hidden_size=FFN, vocab_size=V, normalization="RMSNorm",
                                     gated_linear_unit=True, activation_func="torch.nn.functional.silu",
                                     untie_embeddings_and_output_weights=True, make_vocab_size_divisible_by=8,
                                     norm_epsilon=1e-6, add_qkv_bias=True, rotary_base=1000000),
                        hf.state_dict(), tmp_path)
    ref = _hf_loss(hf)
    assert abs(ours - ref) / ref < 1e-4, (ours, ref)
