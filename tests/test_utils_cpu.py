"""Runtime helper functions (nested attributes, batch slicing, loss averaging, norm offsets)."""
import logging

import torch
import torch.nn as nn

from hetu_galvatron_b200 import utils as U
from hetu_galvatron_b200.models.modules import zigzag_positions


class Inner(nn.Module):
    def __init__(self):
        super().__init__()
        self.linear = nn.Linear(4, 4)
        self.value = 3


class Outer(nn.Module):
    def __init__(self):
        super().__init__()
        self.inner = Inner()
        self.norm = nn.LayerNorm(4)


def test_nested_attribute_helpers():
    m = Outer()
    assert U.rgetattr(m, "") is m
    assert U.rgetattr(m, "inner.linear") is m.inner.linear
    assert U.rgetattr(m, "inner.value") == 3
    U.rsetattr(m, "inner.value", 7)
    assert m.inner.value == 7
    U.rsetattr(m, "flag", True)
    assert m.flag is True
    assert U.rhasattr(m, "inner.linear.weight") and not U.rhasattr(m, "inner.missing.weight")


def test_nested_attribute_helpers_see_through_unit_wrappers():
    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs
    from hetu_galvatron_b200.runtime.engine import build_model

    args = GalvatronRuntimeArgs(
        parallel=dict(mixed_precision="fp32"),
        model=dict(model_size="llama-test", hidden_size=64, num_layers=1, num_attention_heads=4, ffn_hidden_size=96,
                   vocab_size=128, make_vocab_size_divisible_by=8, normalization="RMSNorm",
                   activation_func="torch.nn.functional.silu", gated_linear_unit=True),
        train=dict(seq_length=32, global_batch_size=2, chunks=1))
    m = build_model(args, device=torch.device("cpu"))
    layer = m.model.units[1]                                  # a wrapped decoder layer
    w = U.rgetattr(layer, "attn.attention.linear_qkv.weight")
    assert w is layer.inner.attn.attention.linear_qkv.weight
    assert U.rhasattr(layer, "ffn") and not U.rhasattr(layer, "nope")


def test_context_parallel_batch_slice_is_the_zigzag_split():
    B, S, cp = 2, 32, 4
    tokens = torch.arange(B * S).view(B, S)
    mask = torch.arange(B * 1 * S * S).view(B, 1, S, S)
    for r in range(cp):
        out = U.get_batch_on_this_cp_rank({"tokens": tokens, "labels": None, "attention_mask": mask}, cp, r)
        pos = zigzag_positions(S, cp, r, "cpu")
        assert torch.equal(out["tokens"], tokens[:, pos])
        assert out["labels"] is None
        assert torch.equal(out["attention_mask"], mask[:, :, pos])
    same = U.get_batch_on_this_cp_rank({"tokens": tokens}, 1, 0)
    assert same["tokens"] is tokens


def test_layernorm_offsets():
    m = Outer()
    offs, sizes = U.get_layernorm_offset([m], ["norm"])
    # named_modules order: "", inner, inner.linear (16 + 4 parameters), norm (4 + 4)
    assert offs == [[20, 24]] and sizes == [[4, 4]]
    assert U.get_layernorm_offset([m], []) == ([[]], [[]])


def test_rank_filtered_output_and_versions(capsys, caplog):
    U.print_rank_0("hello")
    assert "hello" in capsys.readouterr().out
    with caplog.at_level(logging.INFO):
        U.log_single_rank(logging.getLogger("hg-test"), logging.INFO, "only once")
    assert "only once" in caplog.text
    assert U.is_torch_min_version("1.0.0") and not U.is_torch_min_version("99.0.0")
    assert U.is_torch_min_version(str(U.get_torch_version())) and not U.is_torch_min_version(str(U.get_torch_version()), False)


def test_loss_average_without_process_group():
    out = U.average_losses_across_data_parallel_group([torch.tensor(1.0), torch.tensor([3.0])], group=None)
    assert torch.equal(out, torch.tensor([1.0, 3.0]))


def test_small_helpers():
    from hetu_galvatron_b200.runtime.datasets.utils import Split, normalize
    from hetu_galvatron_b200.utils.training_utils import VocabUtility, divide

    assert divide(12, 4) == 3
    assert VocabUtility.vocab_range_from_global_vocab_size(128, 1, 4) == (32, 64)
    assert [s.name for s in Split] == ["train", "valid", "test"] and normalize([1, 3]) == [0.25, 0.75]


def test_ensure_log_dir(tmp_path):
    from hetu_galvatron_b200.search.engine import ensure_log_dir

    d = ensure_log_dir(str(tmp_path / "a" / "b"))
    assert (tmp_path / "a" / "b").is_dir() and d.endswith("b")
