"""End-to-end model steps on one GPU: the CUDA-kernel path against the PyTorch (CPU, fp32) oracle path."""
import copy

import pytest
import torch

from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs
from hetu_galvatron_b200.ops import _lib
from hetu_galvatron_b200.runtime.engine import build_model
from hetu_galvatron_b200.runtime.optimizer import ShardedAdamW

pytestmark = pytest.mark.gpu


def make_args(mp, family="llama", ckpt=0, chunks=2):
    model = dict(model_size=family + "-test", hidden_size=256, num_layers=3, num_attention_heads=4, ffn_hidden_size=768,
                 vocab_size=1024, make_vocab_size_divisible_by=8)
    if family == "llama":
        model.update(normalization="RMSNorm", activation_func="torch.nn.functional.silu", gated_linear_unit=True,
                     num_query_groups=2)
    else:
        model.update(normalization="LayerNorm", activation_func="torch.nn.functional.gelu", gated_linear_unit=False,
                     position_embedding_type="learned_absolute", add_bias_linear=True, add_qkv_bias=True)
    return GalvatronRuntimeArgs(parallel=dict(mixed_precision=mp, global_checkpoint=ckpt), model=model,
                                train=dict(seq_length=256, global_batch_size=4, chunks=chunks, lr=1e-3))


def run(args, device, tok, steps=3):
    model = build_model(args, device=torch.device(device), full_init=True)
    opt = ShardedAdamW(model.sharded_units, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.01, clip_grad=1.0,
                       device=torch.device(device))
    out = []
    for it in range(steps):
        opt.zero_grad()
        loss = model.forward_backward(tok[:, :-1].to(device), it, labels=tok[:, 1:].to(device))
        opt.step()
        out.append((float(loss.item()), opt.grad_norm()))
    return out


@pytest.mark.parametrize("family", ["llama", "gpt"])
@pytest.mark.parametrize("ckpt", [0, 1])
def test_loss_parity_with_cpu_oracle(family, ckpt):
    torch.manual_seed(0)
    tok = torch.randint(0, 1024, (4, 257))
    ref = run(make_args("fp32", family, ckpt), "cpu", tok)
    got = run(make_args("bf16", family, ckpt), "cuda", tok)
    _lib.assert_healthy()
    for (l0, n0), (l1, n1) in zip(ref, got):
        assert abs(l0 - l1) / l0 < 5e-3, (ref, got)
        assert abs(n0 - n1) / n0 < 5e-2, (ref, got)
    assert got[-1][0] < got[0][0]


def test_graft_smoke():
    import __graft_entry__ as g

    g.smoke()
