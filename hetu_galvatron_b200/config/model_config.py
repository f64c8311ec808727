"""Resolution of the model architecture fields (``args.model.*`` / ``args.model_info.*``).

Priority, highest first: (1) fields given inline in the entry-point YAML or by overrides,
(2) the model YAML named by ``model_config_path`` (a file path, or a bare zoo name such as
``llama2-7b``), (3) a HuggingFace config named by ``hf_model_name_or_path``, (4) schema defaults.
Derived fields are filled last: ``kv_channels``, ``padded_vocab_size`` (vocabulary padded to a multiple
of ``make_vocab_size_divisible_by`` x the vocab tensor-parallel degree), ``ffn_hidden_size`` default.

Capability parity: galvatron/utils/hf_config_adapter.py:59-70 (attribute aliases), :212-278 (HF fill),
:285-326 (resolver), :333-365 (HF config reconstruction), :372-394 (name / layer metadata).
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional

import torch
import yaml

ZOO_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "model_zoo")

# canonical name -> spellings used by HuggingFace config classes
HF_ALIASES: Dict[str, List[str]] = {
    "hidden_size": ["hidden_size", "n_embd", "d_model"],
    "num_layers": ["num_hidden_layers", "n_layer", "num_layers"],
    "num_attention_heads": ["num_attention_heads", "n_head", "num_heads"],
    "ffn_hidden_size": ["intermediate_size", "n_inner", "ffn_dim", "d_ff"],
    "vocab_size": ["vocab_size"],
    "num_key_value_heads": ["num_key_value_heads"],
    "max_position_embeddings": ["max_position_embeddings", "n_positions", "max_seq_len", "max_sequence_length"],
    "norm_eps": ["rms_norm_eps", "layer_norm_epsilon", "layer_norm_eps", "norm_epsilon", "norm_eps"],
}

_ACTIVATIONS = {
    "silu": (torch.nn.functional.silu, True), "swiglu": (torch.nn.functional.silu, True),
    "gelu": (torch.nn.functional.gelu, False), "gelu_new": (torch.nn.functional.gelu, False),
    "gelu_pytorch_tanh": (torch.nn.functional.gelu, False),
}


def model_args_of(args):
    for name in ("model", "model_info"):
        if hasattr(args, name):
            return getattr(args, name)
    raise TypeError("no model section on %s" % type(args).__name__)


def train_args_of(args):
    for name in ("train", "common_train_info"):
        if hasattr(args, name):
            return getattr(args, name)
    return None


def hf_get(cfg, canonical: str, default=None):
    for alias in HF_ALIASES.get(canonical, [canonical]):
        val = getattr(cfg, alias, None)
        if val is not None:
            return val
    return default


def hf_set(cfg, canonical: str, value):
    names = HF_ALIASES.get(canonical, [canonical])
    for alias in names:
        if hasattr(cfg, alias):
            setattr(cfg, alias, value)
            return
    setattr(cfg, names[0], value)


def find_model_yaml(path_or_name: str) -> str:
    if os.path.exists(path_or_name):
        return path_or_name
    cand = os.path.join(ZOO_DIR, os.path.basename(path_or_name))
    if not cand.endswith(".yaml"):
        cand += ".yaml"
    if os.path.exists(cand):
        return cand
    raise FileNotFoundError("model config %r not found (looked in %s too)" % (path_or_name, ZOO_DIR))


def _from_hf(m, train, hf_cfg, keep: set):
    def put(field, value):
        if value is not None and field not in keep:
            setattr(m, field, value)

    put("hidden_size", hf_get(hf_cfg, "hidden_size"))
    put("num_layers", hf_get(hf_cfg, "num_layers"))
    put("num_attention_heads", hf_get(hf_cfg, "num_attention_heads"))
    put("ffn_hidden_size", hf_get(hf_cfg, "ffn_hidden_size"))
    put("vocab_size", hf_get(hf_cfg, "vocab_size"))
    kv = hf_get(hf_cfg, "num_key_value_heads")
    if kv is not None and kv != m.num_attention_heads:
        put("num_query_groups", kv)
    put("norm_epsilon", hf_get(hf_cfg, "norm_eps"))
    put("normalization", "RMSNorm" if hasattr(hf_cfg, "rms_norm_eps") else "LayerNorm")
    act = getattr(hf_cfg, "hidden_act", None) or getattr(hf_cfg, "activation_function", None) or "gelu"
    fn, gated = _ACTIVATIONS.get(act, (torch.nn.functional.gelu, False))
    put("activation_func", fn)
    put("gated_linear_unit", gated)
    learned = any(hasattr(hf_cfg, a) for a in ("n_positions",)) and not hasattr(hf_cfg, "rope_theta")
    put("position_embedding_type", "learned_absolute" if learned else "rope")
    theta = getattr(hf_cfg, "rope_theta", None)
    if theta is not None:
        put("rotary_base", int(theta))
    put("add_qkv_bias", getattr(hf_cfg, "attention_bias", None))
    put("add_bias_linear", getattr(hf_cfg, "mlp_bias", None))
    put("untie_embeddings_and_output_weights", not getattr(hf_cfg, "tie_word_embeddings", True))
    n_exp = getattr(hf_cfg, "num_local_experts", None)
    if n_exp:
        put("num_moe_experts", n_exp)
        put("moe_router_topk", getattr(hf_cfg, "num_experts_per_tok", 2))
        put("moe_ffn_hidden_size", hf_get(hf_cfg, "ffn_hidden_size"))
    if m.model_size is None and getattr(hf_cfg, "model_type", None):
        m.model_size = hf_cfg.model_type
    if train is not None and train.seq_length is None:
        seq = hf_get(hf_cfg, "max_position_embeddings")
        if seq is not None:
            train.seq_length = seq


def load_hf_config(name_or_path: str):
    """``AutoConfig`` from a hub name / directory, or a bare config class name such as ``LlamaConfig``."""
    import transformers

    if hasattr(transformers, name_or_path) and name_or_path.endswith("Config"):
        return getattr(transformers, name_or_path)()
    return transformers.AutoConfig.from_pretrained(name_or_path, trust_remote_code=False)


def resolve_model_config(args, vocab_tp: Optional[int] = None):
    """Fill ``args.model`` in place; returns the HF config when one was read, else ``None``."""
    m = model_args_of(args)
    train = train_args_of(args)
    inline = set(m.model_fields_set)
    yaml_data: Dict[str, Any] = {}
    if (m.model_config_path is None and m.hf_model_name_or_path is None and m.hidden_size is None and m.model_size
            and os.path.exists(os.path.join(ZOO_DIR, "%s.yaml" % m.model_size))):
        m.model_config_path = m.model_size  # a bare ``model_size`` that names a bundled configuration
    if m.model_config_path is not None:
        with open(find_model_yaml(m.model_config_path)) as f:
            yaml_data = {k: v for k, v in (yaml.safe_load(f) or {}).items() if v is not None}
        if m.hf_model_name_or_path is None and yaml_data.get("hf_model_name_or_path"):
            m.hf_model_name_or_path = yaml_data["hf_model_name_or_path"]
    hf_cfg = None
    if m.hf_model_name_or_path is not None:
        hf_cfg = load_hf_config(m.hf_model_name_or_path)
        _from_hf(m, train, hf_cfg, keep=inline | set(yaml_data))
    fields = type(m).model_fields
    for key, val in yaml_data.items():
        if key in fields and key not in inline:
            setattr(m, key, val)
    finalize_model_args(m, vocab_tp)
    return hf_cfg


def finalize_model_args(m, vocab_tp: Optional[int] = None):
    """Derived fields; idempotent."""
    if isinstance(m.activation_func, str):
        name = m.activation_func.rsplit(".", 1)[-1]
        m.activation_func = _ACTIVATIONS.get(name, (torch.nn.functional.gelu, False))[0]
    if m.kv_channels is None and m.hidden_size and m.num_attention_heads:
        m.kv_channels = m.hidden_size // m.num_attention_heads
    if m.num_moe_experts and not m.is_moe_model:
        m.is_moe_model = True
    if m.ffn_hidden_size is None and m.hidden_size:
        m.ffn_hidden_size = m.moe_ffn_hidden_size or 4 * m.hidden_size
    if m.model_size is None and m.hf_model_name_or_path:
        m.model_size = m.hf_model_name_or_path.split("/")[-1]
    if m.vocab_size is not None and (m.padded_vocab_size is None or vocab_tp is not None):
        m.padded_vocab_size = padded_vocab_size(m.vocab_size, m.make_vocab_size_divisible_by or 1, vocab_tp or 1)
    return m


def padded_vocab_size(vocab: int, divisible_by: int, tp: int) -> int:
    """Smallest multiple of ``divisible_by * tp`` that is >= ``vocab`` (padding rows are appended)."""
    mult = max(1, divisible_by) * max(1, tp)
    return ((vocab + mult - 1) // mult) * mult


def create_hf_config(args, hf_config_class=None):
    """An HF ``PretrainedConfig`` that mirrors ``args.model`` (used by the checkpoint converters and
    the optional HF-parity tests)."""
    m = model_args_of(args)
    if m.hf_model_name_or_path is not None:
        cfg = load_hf_config(m.hf_model_name_or_path)
    elif hf_config_class is not None:
        cfg = hf_config_class()
    else:
        raise ValueError("need hf_model_name_or_path or an HF config class")
    for canonical, field in (("hidden_size", "hidden_size"), ("num_layers", "num_layers"),
                             ("num_attention_heads", "num_attention_heads"), ("ffn_hidden_size", "ffn_hidden_size"),
                             ("vocab_size", "vocab_size")):
        if getattr(m, field) is not None:
            hf_set(cfg, canonical, getattr(m, field))
    if m.num_query_groups is not None:
        hf_set(cfg, "num_key_value_heads", m.num_query_groups)
    train = train_args_of(args)
    if train is not None and train.seq_length is not None:
        hf_set(cfg, "max_position_embeddings", train.seq_length)
    cfg.use_cache = False
    return cfg


def model_name(args) -> str:
    m = model_args_of(args)
    return str((m.model_size or m.hf_model_name_or_path or "unknown").split("/")[-1])


def model_layer_configs(args) -> List[Dict[str, Any]]:
    """Layer metadata the planner consumes: one entry per layer type."""
    m = model_args_of(args)
    train = train_args_of(args)
    return [{"hidden_size": m.hidden_size, "seq_len": train.seq_length if train else None, "layer_num": m.num_layers}]
