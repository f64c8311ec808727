"""Architecture description shared by every model family, and the per-layer execution context.

``ModelSpec`` is the resolved, immutable view of ``args.model`` (dense GPT / Llama / Qwen and the
Mixtral-style MoE).  ``LayerCtx`` carries what one layer needs from its searched strategy: its process
groups, whether its "tp" degree is a Megatron tensor-parallel degree or an Ulysses sequence-parallel
degree, context-parallel degree, checkpoint flag and ZeRO type.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass(frozen=True)
class ModelSpec:
    family: str                      # gpt | llama | qwen | mistral (MoE)
    hidden: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    padded_vocab: int
    seq_len: int
    norm: str = "RMSNorm"            # RMSNorm | LayerNorm
    eps: float = 1e-5
    activation: str = "swiglu"       # swiglu | geglu | gelu
    pos: str = "rope"                # rope | learned_absolute | none
    rope_base: float = 10000.0
    rope_pct: float = 1.0
    rope_interp: float = 1.0
    rope_scaling_factor: float = 0.0  # > 0: Llama-3.x frequency scaling with this factor
    rope_interleaved: bool = False   # rotate channel pairs (2i, 2i+1) instead of the two halves
    per_token_loss: bool = False     # `calculate_per_token_loss`: auxiliary losses scaled by the local token count
    attention_dropout: float = 0.0   # dropout on the attention probabilities (training only; unfused path)
    qk_layernorm: bool = False       # normalise every query and key head (over head_dim) before the rotary embedding
    test_mode: bool = False          # cross-check replicated parameters over the ranks while training
    bias: bool = False               # bias on every linear
    qkv_bias: bool = False
    tied: bool = False               # embedding and LM head share one weight
    init_std: float = 0.02
    hidden_dropout: float = 0.0      # applied to the attention and MLP block outputs before the residual add
    dtype: torch.dtype = torch.bfloat16
    # MoE
    experts: int = 0
    moe_ffn: int = 0
    shared_ffn: int = 0              # > 0: a dense MLP of this width runs on every token beside the routed experts
    topk: int = 2
    router_score: str = "softmax"
    router_pre_softmax: bool = False
    router_scaling: Optional[float] = None
    router_groups: Optional[int] = None
    router_group_topk: Optional[int] = None
    router_expert_bias: bool = False
    router_dtype: Optional[str] = None
    aux_loss_coeff: float = 0.0
    z_loss_coeff: Optional[float] = None
    load_balancing: str = "aux_loss"
    capacity_factor: Optional[float] = None
    pad_to_capacity: bool = False
    drop_policy: str = "probs"
    dispatcher: str = "alltoall"
    grouped_gemm: bool = True
    expert_buffer_factor: Optional[float] = None   # static expert buffers of the peer-memory dispatcher
    jitter_eps: Optional[float] = None

    @property
    def is_moe(self) -> bool:
        return self.experts > 0

    @property
    def gated(self) -> bool:
        return self.activation in ("swiglu", "geglu")

    @property
    def qkv_out(self) -> int:
        return (self.heads + 2 * self.kv_heads) * self.head_dim

    def layer_params(self) -> int:
        """Parameter count of one decoder layer (dense FFN or all experts)."""
        attn = self.hidden * self.qkv_out + self.heads * self.head_dim * self.hidden
        mult = 3 if self.gated else 2
        if self.is_moe:
            ffn = self.experts * mult * self.hidden * self.moe_ffn + self.experts * self.hidden
        else:
            ffn = mult * self.hidden * self.ffn
        return attn + ffn + 2 * self.hidden

    def total_params(self) -> int:
        emb = self.padded_vocab * self.hidden * (1 if self.tied else 2)
        return self.layers * self.layer_params() + emb + self.hidden

    def flops_per_token(self, seq_len: Optional[int] = None, causal: bool = True) -> float:
        """Training FLOPs per token (fwd + bwd = 3x fwd), dense GEMMs + attention, for MFU reporting."""
        s = seq_len or self.seq_len
        attn_proj = 2 * self.hidden * self.qkv_out + 2 * self.heads * self.head_dim * self.hidden
        mult = 3 if self.gated else 2
        if self.is_moe:
            ffn = 2 * mult * self.hidden * self.moe_ffn * self.topk + 2 * self.hidden * self.experts
        else:
            ffn = 2 * mult * self.hidden * self.ffn
        attn = 4 * s * self.heads * self.head_dim * (0.5 if causal else 1.0)
        head = 2 * self.hidden * self.padded_vocab
        return 3.0 * (self.layers * (attn_proj + ffn + attn) + head)


def spec_from_args(args) -> ModelSpec:
    """Build the spec from resolved runtime (or search) arguments."""
    from ..config.model_config import finalize_model_args, model_args_of, train_args_of

    m = finalize_model_args(model_args_of(args))
    tr = train_args_of(args)
    fam = m.model_type if m.model_size else ("mistral" if m.is_moe_model else "llama")
    act_name = getattr(m.activation_func, "__name__", str(m.activation_func))
    if m.gated_linear_unit:
        activation = "swiglu" if "silu" in act_name else "geglu"
    else:
        activation = "gelu"
    par = getattr(args, "parallel", None) or getattr(args, "parallelism_info", None)
    mp = getattr(par, "mixed_precision", "bf16") if par is not None else "bf16"
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[mp]
    return ModelSpec(
        family=fam, hidden=m.hidden_size, layers=m.num_layers, heads=m.num_attention_heads,
        kv_heads=m.num_query_groups or m.num_attention_heads,
        head_dim=m.kv_channels or m.hidden_size // m.num_attention_heads, ffn=m.ffn_hidden_size,
        vocab=m.vocab_size, padded_vocab=m.padded_vocab_size or m.vocab_size,
        seq_len=(tr.seq_length if tr is not None and tr.seq_length else 0),
        norm=m.normalization, eps=m.norm_epsilon if m.norm_epsilon is not None else 1e-5, activation=activation,
        pos=m.position_embedding_type, rope_base=float(m.rotary_base or 10000), rope_pct=m.rotary_percent or 1.0,
        rope_interp=float(m.rotary_seq_len_interpolation_factor or 1.0), bias=m.add_bias_linear,
        qkv_bias=m.add_qkv_bias or m.add_bias_linear, tied=not m.untie_embeddings_and_output_weights,
        init_std=(tr.init_method_std if tr is not None else 0.02), dtype=dtype,
        rope_scaling_factor=(float(getattr(m, "rope_scaling_factor", 8.0) or 8.0)
                             if getattr(m, "use_rope_scaling", False) else 0.0),
        hidden_dropout=float(getattr(m, "hidden_dropout", 0.0) or 0.0),
        rope_interleaved=bool(getattr(m, "rotary_interleaved", False)),
        qk_layernorm=bool(getattr(m, "qk_layernorm", False)),
        attention_dropout=float(getattr(m, "attention_dropout", 0.0) or 0.0),
        per_token_loss=bool(getattr(m, "calculate_per_token_loss", False)),
        test_mode=bool(getattr(tr, "test_mode", False)) if tr is not None else False,
        experts=m.num_moe_experts or 0, moe_ffn=m.moe_ffn_hidden_size or m.ffn_hidden_size or 0,
        topk=m.moe_router_topk, router_score=m.moe_router_score_function, router_pre_softmax=m.moe_router_pre_softmax,
        router_scaling=m.moe_router_topk_scaling_factor, router_groups=m.moe_router_num_groups,
        router_group_topk=m.moe_router_group_topk, router_expert_bias=m.moe_router_enable_expert_bias,
        router_dtype=m.moe_router_dtype, aux_loss_coeff=m.moe_aux_loss_coeff, z_loss_coeff=m.moe_z_loss_coeff,
        load_balancing=m.moe_router_load_balancing_type, capacity_factor=m.moe_expert_capacity_factor,
        pad_to_capacity=m.moe_pad_expert_input_to_capacity, drop_policy=m.moe_token_drop_policy,
        shared_ffn=int(getattr(m, "moe_shared_expert_intermediate_size", 0) or 0),
        dispatcher=m.moe_token_dispatcher_type, grouped_gemm=m.moe_grouped_gemm, expert_buffer_factor=getattr(m, "moe_expert_buffer_factor", None), jitter_eps=m.moe_input_jitter_eps,
    )


@dataclass
class LayerCtx:
    """Execution context of one layer (one row of the whole-model strategy table)."""

    tp: object = None         # CommGroup: Megatron tensor parallel (weights sharded)
    sp: object = None         # CommGroup: Ulysses sequence parallel (weights replicated, heads exchanged)
    cp: object = None         # CommGroup: ring context parallel
    dp: object = None
    sdp: object = None        # dp x sp x cp: parameter sharding / gradient reduction group
    tsp_cp: object = None
    ep: object = None
    tp_of_ep: object = None
    tp_and_ep: object = None
    dp_of_ep: object = None
    dp_type: str = "ddp"      # ddp | zero2 | zero3
    checkpoint: bool = False
    sequence_parallel: bool = True   # Megatron-SP whenever tp > 1
    seq_len: int = 0                 # full (global) sequence length
    fused_comm: bool = False         # use the fused compute+collective kernels over symmetric memory
    layer_index: int = 0

    @staticmethod
    def _n(g) -> int:
        return 1 if g is None else g.size

    @staticmethod
    def _r(g) -> int:
        return 0 if g is None else g.rank

    @property
    def tp_size(self) -> int:
        return self._n(self.tp)

    @property
    def tp_rank(self) -> int:
        return self._r(self.tp)

    @property
    def sp_size(self) -> int:
        return self._n(self.sp)

    @property
    def sp_rank(self) -> int:
        return self._r(self.sp)

    @property
    def cp_size(self) -> int:
        return self._n(self.cp)

    @property
    def cp_rank(self) -> int:
        return self._r(self.cp)

    @property
    def ep_size(self) -> int:
        return self._n(self.ep)

    @property
    def ep_rank(self) -> int:
        return self._r(self.ep)

    @property
    def etp_size(self) -> int:
        return self._n(self.tp_of_ep)

    @property
    def etp_rank(self) -> int:
        return self._r(self.tp_of_ep)

    @property
    def seq_shards(self) -> int:
        """Ways the sequence is split between layers: (tp | sp) * cp."""
        return max(self.tp_size, self.sp_size) * self.cp_size
