"""Cached generation, cross attention, multimodal RoPE and the S3 dataset reader (CPU, fp32 references)."""
import io
import math
import os

import numpy as np
import pytest
import torch

from hetu_galvatron_b200 import ops
from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs
from hetu_galvatron_b200.models.inference import StaticInferenceContext, forward_step, greedy_generate
from hetu_galvatron_b200.models.modules import CrossAttention
from hetu_galvatron_b200.models.spec import LayerCtx, ModelSpec
from hetu_galvatron_b200.runtime.datasets import s3 as s3mod
from hetu_galvatron_b200.runtime.datasets.indexed import IndexedDataset, IndexedDatasetBuilder, bin_path, idx_path
from hetu_galvatron_b200.runtime.engine import build_model


def small_model(pos="rope"):
    torch.manual_seed(0)
    args = GalvatronRuntimeArgs(
        parallel=dict(mixed_precision="fp32"),
        model=dict(model_size="llama-test", hidden_size=64, num_layers=2, num_attention_heads=4, num_query_groups=2,
                   ffn_hidden_size=96, vocab_size=128, make_vocab_size_divisible_by=8, normalization="RMSNorm",
                   activation_func="torch.nn.functional.silu", gated_linear_unit=True),
        train=dict(seq_length=32, global_batch_size=2, chunks=1))
    return build_model(args, device=torch.device("cpu"), full_init=True)


# ---- cached generation --------------------------------------------------------------------------------------
def test_cached_forward_equals_full_forward():
    m = small_model()
    tok = torch.randint(0, 128, (2, 24))
    with torch.no_grad():
        full = m.model(tok, None)                      # [S, B, V]
    ctx = StaticInferenceContext(2, 32)
    parts = [forward_step(m, tok[:, :16], ctx)]        # prefill
    for i in range(16, 24, 2):                         # then two tokens per call
        parts.append(forward_step(m, tok[:, i:i + 2], ctx))
    assert ctx.sequence_len_offset == 24
    assert torch.allclose(torch.cat(parts, 0), full, atol=1e-5, rtol=1e-5)
    ctx.reset()                                        # buffers are reused
    again = forward_step(m, tok[:, :24], ctx)
    assert torch.allclose(again, full, atol=1e-5, rtol=1e-5)


def test_greedy_generate_follows_the_argmax_of_the_full_model():
    m = small_model()
    prompt = torch.randint(0, 128, (2, 8))
    out = greedy_generate(m, prompt, 5)
    assert out.shape == (2, 13) and torch.equal(out[:, :8], prompt)
    with torch.no_grad():
        logits = m.model(out[:, :-1], None)            # [12, 2, V]
    for k in range(5):
        assert torch.equal(logits[7 + k].argmax(-1), out[:, 8 + k])


def test_cache_overflow_is_an_error():
    m = small_model()
    ctx = StaticInferenceContext(2, 8)
    with pytest.raises(ValueError):
        forward_step(m, torch.randint(0, 128, (2, 9)), ctx)


# ---- cross attention ---------------------------------------------------------------------------------------------
def test_cross_attention_matches_reference_math():
    torch.manual_seed(1)
    H, nh = 64, 4
    spec = ModelSpec(family="llama", hidden=H, heads=nh, kv_heads=nh, head_dim=H // nh, layers=1, ffn=96, vocab=128,
                     padded_vocab=128, seq_len=16, dtype=torch.float32)
    ca = CrossAttention(spec, LayerCtx(), torch.device("cpu"), "x")
    ca.reset_parameters(3, True)
    x = torch.randn(10, 2, H, requires_grad=True)
    mem = torch.randn(7, 2, H)
    out = ca(x, mem)
    hd = H // nh
    q = (x @ ca.linear_q.weight.t()).view(10, 2, nh, hd)
    kv = (mem @ ca.linear_kv.weight.t()).view(7, 2, nh, 2 * hd)
    k, v = kv[..., :hd], kv[..., hd:]
    att = torch.einsum("sbnd,tbnd->bnst", q, k) / math.sqrt(hd)
    ref = torch.einsum("bnst,tbnd->sbnd", att.softmax(-1), v).reshape(10, 2, H) @ ca.linear_proj.weight.t()
    assert torch.allclose(out, ref, atol=1e-5, rtol=1e-4)
    out.sum().backward()
    assert x.grad is not None and ca.linear_kv.weight.grad is not None


def test_qk_layernorm_matches_reference_math():
    """``qk_layernorm``: every query head and every key head is normalised over head_dim (one weight for all heads)
    before the rotary embedding; checked against the same attention written out with torch ops (no rotary embedding,
    LayerNorm, grouped-query heads)."""
    from hetu_galvatron_b200.models.modules import SelfAttention

    torch.manual_seed(2)
    H, nh, ng, S, B = 64, 4, 2, 12, 2
    hd = H // nh
    spec = ModelSpec(family="gpt", hidden=H, heads=nh, kv_heads=ng, head_dim=hd, layers=1, ffn=96, vocab=128,
                     padded_vocab=128, seq_len=S, dtype=torch.float32, norm="LayerNorm", pos="learned", qk_layernorm=True)
    att = SelfAttention(spec, LayerCtx(seq_len=S), torch.device("cpu"), "a")
    att.reset_parameters(5, True)
    with torch.no_grad():       # weights away from their initial 1 / 0 so that the test sees them
        for n in (att.q_layernorm, att.k_layernorm):
            n.weight.add_(0.3 * torch.randn(hd))
            n.bias.add_(0.1 * torch.randn(hd))
    x = torch.randn(S, B, H, requires_grad=True)
    out = att(x)
    qpg = nh // ng
    g = (x @ att.linear_qkv.weight.t()).view(S, B, ng, qpg + 2, hd)
    ln = torch.nn.functional.layer_norm
    q = ln(g[..., :qpg, :], (hd,), att.q_layernorm.weight, att.q_layernorm.bias, spec.eps).reshape(S, B, nh, hd)
    k = ln(g[..., qpg, :], (hd,), att.k_layernorm.weight, att.k_layernorm.bias, spec.eps)
    v = g[..., qpg + 1, :]
    k, v = k.repeat_interleave(qpg, dim=2), v.repeat_interleave(qpg, dim=2)
    sc = torch.einsum("sbnd,tbnd->bnst", q, k) / math.sqrt(hd)
    sc = sc.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
    ref = torch.einsum("bnst,tbnd->sbnd", sc.softmax(-1), v).reshape(S, B, H) @ att.linear_proj.weight.t()
    assert torch.allclose(out, ref, atol=1e-5, rtol=1e-4)
    out.sum().backward()
    assert att.q_layernorm.weight.grad is not None and att.k_layernorm.bias.grad is not None
    assert getattr(att.q_layernorm.weight, "tp_replicated", False)


def test_attention_dropout_takes_the_unfused_path_in_training_only():
    from hetu_galvatron_b200.models.modules import SelfAttention

    torch.manual_seed(4)
    H, nh, S, B = 64, 4, 16, 2
    kw = dict(family="gpt", hidden=H, heads=nh, kv_heads=nh, head_dim=H // nh, layers=1, ffn=96, vocab=128,
              padded_vocab=128, seq_len=S, dtype=torch.float32, pos="learned")
    plain = SelfAttention(ModelSpec(**kw), LayerCtx(seq_len=S), torch.device("cpu"), "a")
    drop = SelfAttention(ModelSpec(attention_dropout=0.5, **kw), LayerCtx(seq_len=S), torch.device("cpu"), "a")
    plain.reset_parameters(5, True)
    drop.reset_parameters(5, True)
    x = torch.randn(S, B, H)
    drop.eval()
    assert torch.allclose(drop(x), plain(x), atol=1e-6)            # no dropout outside training
    drop.train()
    with pytest.warns(UserWarning, match="unfused"):
        y1 = drop(x)
    y2 = drop(x)
    assert not torch.allclose(y1, y2) and not torch.allclose(y1, plain(x))      # a fresh mask per call
    # the first query sees one key only: its probability is 1, so the row is either dropped or doubled
    ys = torch.stack([drop(x) for _ in range(64)]).mean(0)
    assert (ys - plain(x)).abs().mean() < 0.25 * plain(x).abs().mean() + 0.05   # unbiased: the mean approaches the plain output


def test_cross_attention_rejects_grouped_query_heads():
    spec = ModelSpec(family="llama", hidden=64, heads=4, kv_heads=2, head_dim=16, layers=1, ffn=96, vocab=128,
                     padded_vocab=128, seq_len=16, dtype=torch.float32)
    with pytest.raises(ValueError):
        CrossAttention(spec, LayerCtx(), torch.device("cpu"), "x")


# ---- multimodal RoPE ---------------------------------------------------------------------------------------------
def test_mrope_matches_qwen2_vl():
    hf = pytest.importorskip("transformers.models.qwen2_vl.modeling_qwen2_vl")
    torch.manual_seed(2)
    B, S, nh, hd = 2, 12, 3, 32
    section = [4, 6, 6]
    pos = torch.stack([torch.randint(0, 50, (B, S)) for _ in range(3)])          # [3, B, S]
    q = torch.randn(S, B, nh, hd)
    k = torch.randn(S, B, nh, hd)
    ang = ops.mrope_angles(pos, section, hd, base=10000.0)                        # [S, B, hd/2]
    ours_q, ours_k = ops.apply_mrope(q, ang), ops.apply_mrope(k, ang)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    freqs = pos[..., None].float() * inv                                          # [3, B, S, hd/2]
    emb = torch.cat([freqs, freqs], -1)
    hq, hk = hf.apply_multimodal_rotary_pos_emb(q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3), emb.cos(), emb.sin(),
                                                section)                          # [B, nh, S, hd]
    assert torch.allclose(ours_q, hq.permute(2, 0, 1, 3), atol=1e-5)
    assert torch.allclose(ours_k, hk.permute(2, 0, 1, 3), atol=1e-5)


def test_mrope_with_equal_rows_is_plain_rope_and_partial_rotation_passes_through():
    S, B, nh, hd, rot = 9, 2, 2, 32, 16
    pos1 = torch.arange(S)[None].expand(B, S)
    ang = ops.mrope_angles(torch.stack([pos1] * 3), [2, 3, 3], rot)
    t = torch.randn(S, B, nh, hd)
    out = ops.apply_mrope(t, ang)
    cos, sin = ops.rope_tables(S, rot, 10000.0, "cpu")
    half = rot // 2
    a, b = t[..., :half], t[..., half:rot]
    c, s = cos[:, None, None, :], sin[:, None, None, :]
    assert torch.allclose(out[..., :half], a * c - b * s, atol=1e-5)
    assert torch.allclose(out[..., half:rot], b * c + a * s, atol=1e-5)
    assert torch.equal(out[..., rot:], t[..., rot:])
    with pytest.raises(ValueError):
        ops.mrope_angles(torch.zeros(3, 1, 4), [1, 2, 3], 16)


# ---- S3 reader ------------------------------------------------------------------------------------------------------
class FakeS3:
    """In-memory stand-in with boto3's method names."""

    def __init__(self):
        self.objects, self.ranges = {}, []

    def put(self, path, data):
        self.objects[s3mod.parse_s3_path(path)] = data

    def head_object(self, Bucket, Key):
        if (Bucket, Key) not in self.objects:
            raise KeyError(Key)
        return {"ContentLength": len(self.objects[(Bucket, Key)])}

    def download_file(self, Bucket, Key, Filename):
        with open(Filename, "wb") as f:
            f.write(self.objects[(Bucket, Key)])

    def get_object(self, Bucket, Key, Range):
        lo, hi = (int(v) for v in Range[len("bytes="):].split("-"))
        self.ranges.append((lo, hi))
        return {"Body": io.BytesIO(self.objects[(Bucket, Key)][lo:hi + 1])}


def test_s3_paths():
    assert s3mod.is_s3_path("s3://bucket/a/b") and not s3mod.is_s3_path("/data/a")
    assert s3mod.parse_s3_path("s3://bucket/a/b.bin") == ("bucket", "a/b.bin")
    assert s3mod.parse_s3_path("s3://bucket") == ("bucket", "")


def test_indexed_dataset_from_s3_reads_what_the_local_reader_reads(tmp_path):
    prefix = str(tmp_path / "corpus")
    b = IndexedDatasetBuilder(bin_path(prefix), dtype=np.int32)
    rng = np.random.default_rng(0)
    docs = [rng.integers(0, 1000, size=int(n)).astype(np.int32) for n in rng.integers(5, 400, size=40)]
    for d in docs:
        b.add_item(d)
        b.end_document()
    b.finalize(idx_path(prefix))
    fake = FakeS3()
    fake.put("s3://bkt/data/corpus.idx", open(idx_path(prefix), "rb").read())
    fake.put("s3://bkt/data/corpus.bin", open(bin_path(prefix), "rb").read())
    assert IndexedDataset.exists("s3://bkt/data/corpus", fake) and not IndexedDataset.exists("s3://bkt/data/nope", fake)
    cfg = s3mod.S3Config(path_to_idx_cache=str(tmp_path / "cache"), bin_chunk_nbytes=4096)
    remote = IndexedDataset("s3://bkt/data/corpus", s3_config=cfg, s3_client=fake)
    local = IndexedDataset(prefix)
    assert os.path.exists(tmp_path / "cache" / "corpus.idx")
    assert len(remote) == len(local) == 40
    for i in range(40):
        assert np.array_equal(remote[i], local[i])
    assert np.array_equal(remote.get(7, offset=2, length=3), local.get(7, offset=2, length=3))
    # sequential reads are served from the window: far fewer requests than sequences, all block aligned
    assert remote._s3.requests < 20 and all(lo % 4096 == 0 for lo, _ in fake.ranges)
    with pytest.raises(ValueError):
        IndexedDataset("s3://bkt/data/corpus")          # no S3Config


# ---- interleaved RoPE -------------------------------------------------------------------------------------------
def test_interleaved_rope_rotates_channel_pairs():
    torch.manual_seed(4)
    S, B, slots, hd = 6, 2, 3, 16
    qkv = torch.randn(S * B, slots * hd)
    cos, sin = ops.rope_tables(32, hd, 10000.0, "cpu")
    out = ops.rope_packed(qkv.clone(), torch.tensor([0, 2], dtype=torch.int32), hd, cos, sin, B, None, 3,
                          interleaved=True).view(S * B, slots, hd)
    x = qkv.view(S * B, slots, hd)
    pos = torch.arange(S * B) // B + 3
    # complex form: (x[2i] + j x[2i+1]) * exp(j * angle_i)
    ang = torch.outer(pos.float(), 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd)))
    rot = torch.polar(torch.ones_like(ang), ang)[:, None, :]
    for h in (0, 2):
        z = torch.view_as_complex(x[:, h].reshape(S * B, hd // 2, 2).contiguous()) * rot[:, 0]
        assert torch.allclose(out[:, h], torch.view_as_real(z).reshape(S * B, hd), atol=1e-5)
    assert torch.equal(out[:, 1], x[:, 1])                       # the slot that is not listed stays as it is


def test_rotary_interleaved_reaches_the_model_spec():
    from hetu_galvatron_b200.models.spec import spec_from_args

    args = GalvatronRuntimeArgs(
        parallel=dict(mixed_precision="fp32"),
        model=dict(model_size="llama-test", hidden_size=64, num_layers=1, num_attention_heads=4, ffn_hidden_size=96,
                   vocab_size=128, rotary_interleaved=True),
        train=dict(seq_length=32, global_batch_size=2, chunks=1))
    assert spec_from_args(args).rope_interleaved is True


def test_cached_forward_of_a_moe_model_and_beam_reorder():
    torch.manual_seed(0)
    args = GalvatronRuntimeArgs(
        parallel=dict(mixed_precision="fp32"),
        model=dict(model_size="mixtral-test", hidden_size=64, num_layers=2, num_attention_heads=4, num_query_groups=2,
                   vocab_size=128, make_vocab_size_divisible_by=8, normalization="RMSNorm",
                   activation_func="torch.nn.functional.silu", gated_linear_unit=True, is_moe_model=True,
                   num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=96),
        train=dict(seq_length=32, global_batch_size=2, chunks=1))
    m = build_model(args, device=torch.device("cpu"), full_init=True)
    tok = torch.randint(0, 128, (2, 20))
    with torch.no_grad():
        full = m.model(tok, None)
    ctx = StaticInferenceContext(2, 32)
    parts = [forward_step(m, tok[:, :12], ctx)] + [forward_step(m, tok[:, i:i + 1], ctx) for i in range(12, 20)]
    assert torch.allclose(torch.cat(parts, 0), full, atol=1e-5, rtol=1e-5)
    # swapping the two cached sequences and feeding the swapped next tokens gives the swapped logits
    nxt = torch.randint(0, 128, (2, 1))
    ref = StaticInferenceContext(2, 32)
    forward_step(m, tok, ref)
    a = forward_step(m, nxt, ref)
    ctx.swap_key_value_dict(torch.tensor([1, 0]))
    b = forward_step(m, nxt.flip(0), ctx)
    assert torch.allclose(b, a.flip(1), atol=1e-5, rtol=1e-5)
