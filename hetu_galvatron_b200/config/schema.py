"""Argument schemas of the four entry points (train / search / model-profile / hardware-profile).

The public surface -- section names, field names, defaults and value constraints -- is the one of
the reference's Pydantic models (galvatron/core/runtime/args_schema.py:18-382,
core/search_engine/args_schema.py:12-74, core/profiler/args_schema.py:9-58, tools/args_schema.py:5-20,
core/args_schema.py:46-52), so its YAML files and ``a.b.c=v`` overrides validate unchanged.  The models
are generated from compact field tables: ``name: (type, default[, constraints])``.
"""
from __future__ import annotations

from typing import Any, Dict, List, Literal, Optional, Tuple

import torch
from pydantic import BaseModel, ConfigDict, Field, create_model, field_validator

O = Optional
_Spec = Dict[str, Tuple]


def _build(name: str, spec: _Spec, base=BaseModel, doc: str = ""):
    fields: Dict[str, Any] = {}
    for key, item in spec.items():
        typ, default = item[0], item[1]
        cons = item[2] if len(item) > 2 else {}
        if isinstance(default, (list, dict)):
            fields[key] = (typ, Field(default_factory=lambda d=default: type(d)(d), **cons))
        else:
            fields[key] = (typ, Field(default=default, **cons))
    model = create_model(name, __base__=base, **fields)
    model.__doc__ = doc
    return model


_DTYPES = {"fp32": torch.float32, "float32": torch.float32, "fp16": torch.float16, "float16": torch.float16,
           "bf16": torch.bfloat16, "bfloat16": torch.bfloat16}


class _ModelBase(BaseModel):
    model_config = ConfigDict(arbitrary_types_allowed=True, protected_namespaces=())

    @field_validator("params_dtype", mode="before", check_fields=False)
    @classmethod
    def _dtype(cls, v):
        if isinstance(v, str):
            return _DTYPES[v.replace("torch.", "")]
        return v

    @field_validator("activation_func", mode="before", check_fields=False)
    @classmethod
    def _act(cls, v):
        if isinstance(v, str):
            import importlib

            mod, _, fn = v.rpartition(".")
            return getattr(importlib.import_module(mod), fn)
        return v

    @property
    def model_type(self) -> str:
        """``"llama2-7b" -> "llama"``: family prefix of ``model_size`` without version digits."""
        return self.model_size.split("-")[0].rstrip("0123456789.")


GalvatronParallelArgs = _build("GalvatronParallelArgs", {
    "pp_deg": (int, 1, dict(ge=1)),
    "global_tp_deg": (int, 1, dict(ge=1)),
    "global_tp_consec": (Literal[0, 1], 1),
    "global_cp_deg": (int, 1, dict(ge=1)),
    "global_ep_deg": (int, 1, dict(ge=1)),
    "global_tp_of_ep_deg": (int, 1, dict(ge=1)),
    "global_checkpoint": (int, 0),
    "cp_mode": (Literal["ring", "zigzag"], "zigzag"),
    "sdp": (Literal[0, 1], 0),
    "default_dp_type": (Literal["ddp", "zero2", "zero3"], "ddp"),
    "pipeline_type": (Literal["gpipe", "pipedream_flush"], "gpipe"),
    "galvatron_config_path": (Any, None),  # path of a strategy JSON, or the parsed dict
    "vocab_sdp": (Literal[0, 1], 0),
    "vocab_tp": (int, 1, dict(ge=1)),
    "vocab_cp": (int, 1, dict(ge=1)),
    "vocab_sp": (int, 1),
    "async_grad_reduce": (bool, True),
    "mixed_precision": (Literal["fp32", "fp16", "bf16"], "bf16"),
    "use_ulysses": (bool, False),
    "reduce_in_fp32": (bool, False),
    "entropy_in_fp32": (bool, False),
    # this framework's own kernels over NVLink peer memory in place of NCCL (null = on wherever they apply):
    # fused_comm: all-gather->GEMM / GEMM->reduce-scatter, Ulysses and MoE all-to-all, resharding; fused_zero: ZeRO
    # gradient reduce-scatter and AdamW + parameter all-gather.  A strategy JSON may carry both keys.
    "fused_comm": (O[bool], None),
    "fused_zero": (O[bool], None),
}, doc="Parallelism and strategy (GLOBAL mode flags, or a searched strategy JSON).")

GalvatronModelArgs = _build("GalvatronModelArgs", {
    "hf_model_name_or_path": (O[str], None),
    "model_config_path": (O[str], None),
    "is_moe_model": (bool, False),
    "set_experts_manually": (int, 0),
    "set_model_config_manually": (int, 0),
    "set_layernum_manually": (int, 0),
    "set_seqlen_manually": (int, 0),
    "initialize_on_meta": (Literal[0, 1], 1),
    "shape_order": (Literal["SBH", "BSH"], "SBH"),
    "dropout_prob": (float, 0.0, dict(ge=0.0, le=1.0)),
    "print_loss": (int, 0),
    "model_size": (O[str], None),
    "vocab_size": (O[int], None),
    "padded_vocab_size": (O[int], None),
    "hidden_size": (O[int], None),
    "ffn_hidden_size": (O[int], None),
    "num_layers": (O[int], None),
    "num_attention_heads": (O[int], None),
    "num_query_groups": (O[int], None),
    "kv_channels": (O[int], None),
    "attention_dropout": (O[float], 0.0),
    "hidden_dropout": (O[float], 0.0),
    "add_qkv_bias": (bool, False),
    "layernorm_epsilon": (O[float], 1e-5),
    "qk_layernorm": (bool, False),
    "position_embedding_type": (Literal["learned_absolute", "rope", "mrope", "relative", "none"], "rope"),
    "rotary_base": (O[int], 10000),
    "rotary_percent": (O[float], 1.0),
    "rotary_interleaved": (bool, False),
    "use_rope_scaling": (bool, False),
    "rope_scaling_factor": (float, 8.0),
    "rotary_seq_len_interpolation_factor": (O[int], None),
    "mrope_section": (O[List[int]], None),
    "make_vocab_size_divisible_by": (O[int], 128),
    "normalization": (Literal["LayerNorm", "RMSNorm"], "RMSNorm"),
    "norm_epsilon": (O[float], 1e-5),
    "multi_latent_attention": (bool, False),
    "apply_rope_fusion": (bool, False),
    "add_bias_linear": (bool, False),
    "bias_activation_fusion": (bool, False),
    "activation_func_fp8_input_store": (bool, False),
    "gated_linear_unit": (bool, True),
    "activation_func": (Any, "torch.nn.functional.gelu"),
    "untie_embeddings_and_output_weights": (bool, True),
    "num_moe_experts": (O[int], None),
    "moe_ffn_hidden_size": (O[int], None),
    "moe_router_topk": (int, 2),
    "moe_router_load_balancing_type": (Literal["none", "aux_loss", "seq_aux_loss", "sinkhorn"], "aux_loss"),
    "moe_router_score_function": (Literal["softmax", "sigmoid"], "softmax"),
    "moe_router_pre_softmax": (bool, False),
    "moe_router_topk_scaling_factor": (O[float], None),
    "moe_router_num_groups": (O[int], None),
    "moe_router_group_topk": (O[int], None),
    "moe_router_enable_expert_bias": (bool, False),
    "moe_router_bias_update_rate": (float, 1.0e-3),
    "moe_router_dtype": (O[Literal["fp32", "fp64"]], None),
    "deterministic_mode": (bool, False),
    "moe_aux_loss_coeff": (float, 0.0),
    "moe_z_loss_coeff": (O[float], None),
    "moe_token_dispatcher_type": (Literal["allgather", "alltoall_seq", "alltoall", "flex"], "allgather"),
    "moe_expert_capacity_factor": (O[float], None),
    "moe_pad_expert_input_to_capacity": (bool, False),
    "moe_token_drop_policy": (Literal["probs", "position"], "probs"),
    "moe_input_jitter_eps": (O[float], None),
    "moe_permute_fusion": (bool, True),
    "moe_enable_deepep": (bool, False),
    "moe_shared_expert_intermediate_size": (O[int], None),
    "moe_shared_expert_overlap": (bool, False),
    "calculate_per_token_loss": (bool, False),
    "moe_grouped_gemm": (bool, False),
    # peer-memory dispatcher only: size every rank's expert buffer statically at this multiple of the balanced load
    # (the routing table is then built on the device with no host read; pairs beyond the buffer are dropped and
    # reported).  null = exact sizes, one host read per layer call.
    "moe_expert_buffer_factor": (O[float], None),
    "params_dtype": (Any, torch.float32),
    "gradient_accumulation_fusion": (bool, False),
    "defer_embedding_wgrad_compute": (bool, False),
    "wgrad_deferral_limit": (int, 0),
}, base=_ModelBase, doc="Model architecture (dense and MoE) and model-parallel numerics.")

GalvatronProfileArgs = _build("GalvatronProfileArgs", {
    "profile": (int, 0),
    "profile_mode": (Literal["static", "batch", "sequence"], "static"),
    "profile_unit": (Literal["attention", "mlp", "all"], "all"),
    "profile_forward": (Literal[0, 1], 0),
    "save_profiled_memory": (int, 0),
    "exit_after_profiling": (Literal[0, 1], 1),
    "save_profiled_iteration_time": (int, 0),   # write the whole-iteration time (fwd + bwd + optimizer) for the refit
}, doc="In-training profiling switches.")

CommonTrainArgs = _build("CommonTrainArgs", {
    "seed": (O[int], 42),
    "iteration": (O[int], 0, dict(ge=0)),
    "train_iters": (O[int], None),
    "train_samples": (O[int], None),
    "consumed_train_samples": (O[int], 0),
    "eval_iters": (O[int], 1),
    "eval_interval": (O[int], 1000),
    "consumed_valid_samples": (O[int], 0),
    "skip_train": (bool, False),
    "do_train": (bool, False),
    "do_valid": (bool, False),
    "do_test": (bool, False),
    "dataloader_type": (Literal["single", "cyclic", "external"], "single"),
    "num_workers": (int, 2),
    "data_sharding": (bool, False),
    "lr": (O[float], None),
    "min_lr": (O[float], None),
    "lr_decay_style": (Literal["constant", "linear", "cosine", "inverse-square-root", "WSD"], "cosine"),
    "lr_warmup_fraction": (O[float], None),
    "lr_warmup_iters": (O[int], 0),
    "lr_warmup_samples": (O[int], 0),
    "lr_warmup_init": (float, 0.0),
    "lr_decay_iters": (O[int], None),
    "lr_decay_samples": (O[int], None),
    "lr_wsd_decay_style": (Literal["exponential", "linear", "cosine"], "exponential"),
    "lr_wsd_decay_iters": (O[int], None),
    "lr_wsd_decay_samples": (O[int], None),
    "weight_decay": (float, 0.01),
    "start_weight_decay": (O[float], None),
    "end_weight_decay": (O[float], None),
    "weight_decay_incr_style": (Literal["constant", "linear", "cosine"], "constant"),
    "adam_beta1": (float, 0.9),
    "adam_beta2": (float, 0.999),
    "adam_eps": (float, 1e-8),
    "init_method_std": (float, 0.02),
    "use_checkpoint_opt_param_scheduler": (bool, False),
    "override_opt_param_scheduler": (bool, False),
    "sequence_parallel": (bool, True),
    "global_memory_buffer": (bool, True),
    "use_flash_attn": (bool, True),
    "global_batch_size": (O[int], None, dict(ge=1)),
    "micro_batch_size": (O[int], None),
    "chunks": (int, -1),
    "rampup_batch_size": (O[List[int]], None),
    "seq_length": (O[int], None),
    "clip_grad": (float, 1.0, dict(ge=0.0)),
    "flash_decode": (bool, True),
    "test_mode": (bool, False),
}, doc="Optimizer, schedule, batch geometry.")


class _DataBase(BaseModel):
    @field_validator("data_path", "train_data_path", "valid_data_path", "test_data_path", mode="before",
                     check_fields=False)
    @classmethod
    def _listify(cls, v):
        if v is None:
            return None
        return [v] if isinstance(v, str) else list(v)


CommonDataArgs = _build("CommonDataArgs", {
    "data_path": (O[List[str]], None),
    "split": (O[str], None),
    "train_data_path": (O[List[str]], None),
    "valid_data_path": (O[List[str]], None),
    "test_data_path": (O[List[str]], None),
    "data_args_path": (O[str], None),
    "per_split_data_args_path": (O[str], None),
    "tokenizer_type": (O[str], "HuggingFaceTokenizer"),
    "tokenizer_model": (O[str], None),
    "shared_storage": (bool, True),
    "num_dataset_builder_threads": (int, 1),
    "data_cache_path": (O[str], None),
    "mmap_bin_files": (bool, True),
    "s3_cache_path": (O[str], None),
    "reset_position_ids": (bool, False),
    "reset_attention_mask": (bool, False),
    "eod_mask_loss": (bool, False),
    "create_attention_mask_in_dataloader": (bool, False),
    "use_random_dataset": (bool, False),
}, base=_DataBase, doc="Datasets and tokenizer.")

CommonCkptArgs = _build("CommonCkptArgs", {
    "load": (O[str], None),
    "load_iteration": (int, 0, dict(ge=0)),
    "distributed_checkpoint": (bool, False),
    "save": (O[str], None),
    "save_interval": (O[int], None),
}, doc="Checkpoint load / save.")

LoggingConfig = _build("LoggingConfig", {
    "tensorboard_dir": (O[str], None),
    "tensorboard_queue_size": (int, 1000, dict(ge=1)),
    "wandb_project": (str, ""),
    "wandb_exp_name": (str, ""),
    "wandb_save_dir": (str, ""),
}, doc="Metric writers.")


def _sub(model):
    return (model, Field(default_factory=model))


GalvatronRuntimeArgs = create_model(
    "GalvatronRuntimeArgs",
    parallel=_sub(GalvatronParallelArgs), model=_sub(GalvatronModelArgs), profile=_sub(GalvatronProfileArgs),
    train=_sub(CommonTrainArgs), data=_sub(CommonDataArgs), ckpt=_sub(CommonCkptArgs), logging=_sub(LoggingConfig),
    rank=(int, Field(default=0, ge=0)), world_size=(int, Field(default=1, ge=1)),
    local_rank=(int, Field(default=0, ge=0)), distributed_backend=(str, "nccl"),
    distributed_timeout_minutes=(int, Field(default=10, ge=1)),
    __config__=ConfigDict(protected_namespaces=()),
)
GalvatronTrainingArgs = GalvatronRuntimeArgs

# ---- search engine ----------------------------------------------------------------------------
SearchEngineBatchSizeArgs = _build("SearchEngineBatchSizeArgs", {
    "min_bsz": (int, 8, dict(ge=1)), "max_bsz": (int, 8, dict(ge=1)), "recommend_min_bsz": (int, 0),
    "settle_bsz": (int, -1), "settle_chunk": (int, -1), "bsz_scale": (int, 8, dict(ge=1)),
})
SearchEngineHardwareInfoArgs = _build("SearchEngineHardwareInfoArgs", {
    "num_nodes": (int, 1, dict(ge=1)), "num_gpus_per_node": (int, 8, dict(ge=1)),
    "memory_constraint": (int, 24, dict(ge=1)),
})
SearchEngineSearchSpaceArgs = _build("SearchEngineSearchSpaceArgs", {
    "disable_dp": (int, 0), "disable_tp": (int, 0), "disable_cp": (int, 1), "disable_sp": (int, 0),
    "disable_embedding_lmhead_tp": (int, 0), "disable_embedding_lmhead_sp": (int, 0), "disable_pp": (int, 0),
    "disable_ckpt": (int, 0), "disable_fsdp": (int, 0),
    "max_tp_deg": (int, 8, dict(ge=1)), "max_pp_deg": (int, 8, dict(ge=1)), "max_sp_deg": (int, 8, dict(ge=1)),
    "max_cp_deg": (int, 8, dict(ge=1)),
})
_ProfileMode = Literal["static", "batch", "sequence", "hybrid"]
SearchEngineProfilingArgs = _build("SearchEngineProfilingArgs", {
    "memory_profiling_path": (O[str], None), "time_profiling_path": (O[str], None),
    "allreduce_bandwidth_config_path": (O[str], None), "p2p_bandwidth_config_path": (O[str], None),
    "overlap_coe_path": (O[str], None), "sp_time_path": (O[str], None),
    "time_profile_mode": (_ProfileMode, "static"), "memory_profile_mode": (_ProfileMode, "static"),
})
SearchEngineOptionsArgs = _build("SearchEngineOptionsArgs", {
    "parallel_search": (bool, False), "worker": (int, 0, dict(ge=0)), "log_dir": (str, "logs"),
    "output_config_path": (O[str], None), "fine_grained_mode": (int, 1),
})
SearchEngineDebugArgs = _build("SearchEngineDebugArgs", {"debug_costmodel_coe": (float, 1.0)})

GalvatronSearchArgs = create_model(
    "GalvatronSearchArgs",
    model_info=_sub(GalvatronModelArgs), parallelism_info=_sub(GalvatronParallelArgs),
    common_train_info=_sub(CommonTrainArgs), hardware_info=_sub(SearchEngineHardwareInfoArgs),
    batch_size_info=_sub(SearchEngineBatchSizeArgs), search_space_info=_sub(SearchEngineSearchSpaceArgs),
    profiling_info=_sub(SearchEngineProfilingArgs), options_info=_sub(SearchEngineOptionsArgs),
    debug_info=_sub(SearchEngineDebugArgs),
    __config__=ConfigDict(protected_namespaces=()),
)

# ---- profilers ----------------------------------------------------------------------------------
_GalvatronModelProfilerBase = _build("_GalvatronModelProfilerBase", {
    "profile_type": (Literal["memory", "computation"], "memory"),
    "profile_mode": (Literal["static", "batch", "sequence"], "static"),
    "profile_unit": (Literal["attention", "mlp", "all"], "all"),
    "profile_flow_control": (Literal["all", "scripts_only", "launch_only", "data_only"], "all"),
    "profile_mixed_precision": (Literal["fp32", "fp16", "bf16"], "bf16"),
    "profile_fixed_batch_size": (O[int], None), "profile_min_batch_size": (O[int], None),
    "profile_max_batch_size": (O[int], None), "profile_batch_size_step": (O[int], None),
    "profile_fixed_seq_length_list": (O[List[int]], None), "profile_min_seq_length": (O[int], None),
    "profile_max_seq_length": (O[int], None), "profile_seq_length_step": (O[int], None),
    "profile_layernum_min": (int, 1), "profile_layernum_max": (int, 2),
    "profile_max_tp_deg": (int, 8), "profile_dp_type": (Literal["zero3", "ddp"], "zero3"),
    "sequence_parallel": (bool, True),
    "runtime_yaml_template_path": (O[str], None),
})
GalvatronModelProfilerArgs = create_model(
    "GalvatronModelProfilerArgs", __base__=_GalvatronModelProfilerBase, model_info=_sub(GalvatronModelArgs))


class _HwBase(BaseModel):
    model_config = ConfigDict(extra="allow")


ProfilerHardwareArgs = _build("ProfilerHardwareArgs", {
    "num_nodes": (int, 1), "num_gpus_per_node": (int, 8),
    "master_addr": (str, "$MASTER_ADDR"), "master_port": (str, "$MASTER_PORT"), "node_rank": (str, "$RANK"),
    "max_tp_size": (int, 8), "envs": (List[str], []), "max_pp_deg": (int, 8), "overlap_time_multiply": (int, 4),
}, base=_HwBase, doc="NVLink / NCCL micro-benchmark sweep.")

# ---- tools ---------------------------------------------------------------------------------------
CheckpointConvertH2GArgs = _build("CheckpointConvertH2GArgs", {
    "model_type": (str, ...), "input_checkpoint": (str, ...), "output_dir": (str, ...)})
CheckpointConvertG2HArgs = create_model(
    "CheckpointConvertG2HArgs", load_iteration=(int, ...), input_checkpoint=(str, ...), output_dir=(str, ...),
    model_config=(str, ...), model_type=(str, ...), __config__=ConfigDict(protected_namespaces=()))

CoreArgs = create_model(
    "CoreArgs",
    runtime=(O[GalvatronRuntimeArgs], None), profiler_hardware=(O[ProfilerHardwareArgs], None),
    search_engine=(O[GalvatronSearchArgs], None), model_profiler=(O[GalvatronModelProfilerArgs], None),
)

MODE_TO_SECTION = {"train_dist": "runtime", "model_profiler": "model_profiler",
                   "profiler_hardware": "profiler_hardware", "search": "search_engine"}
