"""Checkpoints: HuggingFace -> per-module split files -> tensor/expert-parallel shards; distributed save / resume;
export back to HuggingFace names.

Formats (the reference's, galvatron/tools/checkpoint_convert_h2g.py:9-90 and core/runtime/checkpoint/*.py):

*HF split* (strategy independent, written by :func:`convert_hf_to_split`): one file per module, keys are the HF
names with the module prefix stripped --
``model_embed_tokens.pt {embed_tokens.weight}``, ``model_layers_{i}.pt {input_layernorm.weight,
self_attn.{q,k,v,o}_proj.weight, post_attention_layernorm.weight, mlp.{gate,up,down}_proj.weight}`` (Mixtral:
``block_sparse_moe.gate.weight``, ``block_sparse_moe.experts.{e}.{w1,w2,w3}.weight``), ``model_norm.pt {weight}``,
``lm_head.pt {weight}``; GPT-2: ``transformer_embedding.pt``, ``transformer_h_{i}.pt``, ``transformer_ln_f.pt``.

*Distributed checkpoint*::

    <save>/hybrid_parallel_configs.json
    <save>/iter_<N>/opt_param_scheduler.json
    <save>/iter_<N>/model_embed_tokens/<tp>.pt   model_layers_<i>/<tp>.pt   model_norm/<tp>.pt   lm_head/<tp>.pt
    <save>/iter_<N>/optimizer/<global_rank>.pt                       (sharded fp32 state: strategy locked)
    MoE: model_layers_<i>_attention/<tp>.pt  model_layers_<i>_router.pt  model_layers_<i>_mlp/<ep>_<tp>.pt

Each unit file is the unit's unsharded state dict for one tensor-parallel rank, written by the rank whose
index in the unit's sharding group is 0.  Differences from the reference, on purpose: vocabulary padding rows
are *appended* (it prepends them, llama_adapter.py:59), biases are restored too, and arguments are read from
their nested sections.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..models.spec import ModelSpec


# --------------------------------------------------------------------------------------------
# HF <-> split files
# --------------------------------------------------------------------------------------------
def convert_hf_to_split(state_dict: Dict[str, torch.Tensor], model_type: str, output_dir: str) -> List[str]:
    """Split an HF state dict into one file per module; returns the written file names."""
    os.makedirs(output_dir, exist_ok=True)
    groups: Dict[str, Dict[str, torch.Tensor]] = {}
    for key, val in state_dict.items():
        parts = key.split(".")
        if model_type in ("llama", "mixtral", "mistral", "qwen"):
            if parts[0] == "model" and parts[1] == "layers":
                fname, sub = "model_layers_%s" % parts[2], ".".join(parts[3:])
            elif parts[0] == "model":
                fname, sub = "model_%s" % parts[1], ".".join(parts[2:]) if parts[1] == "norm" else ".".join(parts[1:])
            else:
                fname, sub = parts[0], ".".join(parts[1:])
        elif model_type == "gpt":
            if parts[0] == "lm_head":
                continue  # tied to wte
            if parts[1] == "h":
                fname, sub = "transformer_h_%s" % parts[2], ".".join(parts[3:])
            elif parts[1] in ("wte", "wpe"):
                fname, sub = "transformer_embedding", ".".join(parts[1:])
            else:
                fname, sub = "transformer_%s" % parts[1], ".".join(parts[2:])
        elif model_type in ("bert", "bert-mlm"):
            # same grouping as the reference's convert_checkpoints_bert_mlm (tools/checkpoint_convert_h2g.py:93-138)
            if parts[0] == "bert" and parts[1] == "encoder":
                fname, sub = "bert_encoder_layer_%s" % parts[3], ".".join(parts[4:])
            elif parts[0] == "bert" and parts[1] in ("embeddings", "pooler"):
                fname, sub = "bert_%s" % parts[1], ".".join(parts[2:])
            elif parts[0] == "cls" and parts[1] == "predictions":
                fname, sub = "cls_predictions", ".".join(parts[2:])
            else:
                continue
        else:
            raise ValueError("unknown model type %r" % model_type)
        groups.setdefault(fname, {})[sub] = val.detach().clone()
    out = []
    for fname, sd in groups.items():
        torch.save(sd, os.path.join(output_dir, fname + ".pt"))
        out.append(fname + ".pt")
    return sorted(out)


def read_hf_checkpoint(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of an HF checkpoint directory (safetensors shards or torch ``.bin`` files)."""
    sd: Dict[str, torch.Tensor] = {}
    files = sorted(os.listdir(path))
    st = [f for f in files if f.endswith(".safetensors")]
    if st:
        from safetensors.torch import load_file

        for f in st:
            sd.update(load_file(os.path.join(path, f)))
        return sd
    for f in files:
        if f.endswith(".bin") or f.endswith(".pt"):
            sd.update(torch.load(os.path.join(path, f), map_location="cpu", weights_only=True))
    return sd


def _pad_vocab(w: torch.Tensor, padded: int) -> torch.Tensor:
    if w.shape[0] >= padded:
        return w[:padded]
    return torch.cat([w, w.new_zeros((padded - w.shape[0],) + tuple(w.shape[1:]))], dim=0)


def pack_qkv(q, k, v, nh: int, ng: int, hd: int) -> torch.Tensor:
    """HF q/k/v ``[n*hd, H]`` -> grouped rows ``[ng, (nh/ng + 2), hd, H]`` flattened (the fused QKV layout)."""
    H = q.shape[1]
    return torch.cat([q.reshape(ng, (nh // ng) * hd, H), k.reshape(ng, hd, H), v.reshape(ng, hd, H)], dim=1).reshape(-1, H)


def unpack_qkv(w, nh: int, ng: int, hd: int):
    H = w.shape[1]
    g = w.reshape(ng, (nh // ng + 2) * hd, H)
    qpg = nh // ng
    return (g[:, :qpg * hd].reshape(nh * hd, H), g[:, qpg * hd:(qpg + 1) * hd].reshape(ng * hd, H),
            g[:, (qpg + 1) * hd:].reshape(ng * hd, H))


def _rows(w, rank, world):
    return w.chunk(world, dim=0)[rank]


def _cols(w, rank, world):
    return w.chunk(world, dim=1)[rank]


def shard_from_hf(kind: str, hf: Dict[str, torch.Tensor], spec: ModelSpec, tp_rank: int, tp: int,
                  ep_rank: int = 0, ep: int = 1) -> Dict[str, torch.Tensor]:
    """Unit state dict (module-relative keys) of one tensor/expert-parallel rank from the HF tensors of that module."""
    nh, ng, hd = spec.heads, spec.kv_heads, spec.head_dim
    out: Dict[str, torch.Tensor] = {}
    if kind == "embedding":
        if "embed_tokens.weight" in hf:
            out["embed_tokens.weight"] = _rows(_pad_vocab(hf["embed_tokens.weight"], spec.padded_vocab), tp_rank, tp)
        else:  # GPT-2
            out["embed_tokens.weight"] = _rows(_pad_vocab(hf["wte.weight"], spec.padded_vocab), tp_rank, tp)
            out["embed_positions.weight"] = hf["wpe.weight"][: spec.seq_len]
    elif kind == "lm_head":
        out["lm_head.weight"] = _rows(_pad_vocab(hf["weight"], spec.padded_vocab), tp_rank, tp)
    elif kind == "prenorm":
        out["norm.weight"] = hf["weight"]
        if "bias" in hf:
            out["norm.bias"] = hf["bias"]
    elif kind in ("decoder", "moe_attention"):
        pre = "attn."   # GalvatronDecoderLayer.attn and GalvatronMoEAttention.attn are both a GalvatronAttention
        if "self_attn.q_proj.weight" in hf:  # llama-style names
            qkv = pack_qkv(hf["self_attn.q_proj.weight"], hf["self_attn.k_proj.weight"], hf["self_attn.v_proj.weight"],
                           nh, ng, hd)
            out[pre + "attention.linear_qkv.weight"] = _rows(qkv, tp_rank, tp)
            if "self_attn.q_proj.bias" in hf:
                b = pack_qkv(hf["self_attn.q_proj.bias"][:, None], hf["self_attn.k_proj.bias"][:, None],
                             hf["self_attn.v_proj.bias"][:, None], nh, ng, hd)[:, 0]
                out[pre + "attention.linear_qkv.bias"] = _rows(b, tp_rank, tp)
            out[pre + "attention.linear_proj.weight"] = _cols(hf["self_attn.o_proj.weight"], tp_rank, tp)
            out[pre + "input_layernorm.weight"] = hf["input_layernorm.weight"]
            post = hf["post_attention_layernorm.weight"]
            if kind == "decoder":
                out["ffn.post_attention_layernorm.weight"] = post
                gate, up = _rows(hf["mlp.gate_proj.weight"], tp_rank, tp), _rows(hf["mlp.up_proj.weight"], tp_rank, tp)
                out["ffn.mlp.linear_fc1.weight"] = torch.cat([gate, up], dim=0)
                out["ffn.mlp.linear_fc2.weight"] = _cols(hf["mlp.down_proj.weight"], tp_rank, tp)
            else:
                out["pre_router_norm.weight"] = post
        else:  # GPT-2 (Conv1D weights are [in, out])
            w = hf["attn.c_attn.weight"].t()
            q, k, v = w.chunk(3, dim=0)
            out[pre + "attention.linear_qkv.weight"] = _rows(pack_qkv(q, k, v, nh, ng, hd), tp_rank, tp)
            bq, bk, bv = hf["attn.c_attn.bias"].chunk(3)
            out[pre + "attention.linear_qkv.bias"] = _rows(pack_qkv(bq[:, None], bk[:, None], bv[:, None], nh, ng, hd)[:, 0],
                                                           tp_rank, tp)
            out[pre + "attention.linear_proj.weight"] = _cols(hf["attn.c_proj.weight"].t(), tp_rank, tp)
            out[pre + "attention.linear_proj.bias"] = hf["attn.c_proj.bias"]
            out[pre + "input_layernorm.weight"], out[pre + "input_layernorm.bias"] = hf["ln_1.weight"], hf["ln_1.bias"]
            out["ffn.post_attention_layernorm.weight"], out["ffn.post_attention_layernorm.bias"] = hf["ln_2.weight"], hf["ln_2.bias"]
            out["ffn.mlp.linear_fc1.weight"] = _rows(hf["mlp.c_fc.weight"].t(), tp_rank, tp)
            out["ffn.mlp.linear_fc1.bias"] = _rows(hf["mlp.c_fc.bias"], tp_rank, tp)
            out["ffn.mlp.linear_fc2.weight"] = _cols(hf["mlp.c_proj.weight"].t(), tp_rank, tp)
            out["ffn.mlp.linear_fc2.bias"] = hf["mlp.c_proj.bias"]
    elif kind == "moe_router":
        # classic Mixtral checkpoints name the gate block_sparse_moe.gate; newer transformers releases mlp.gate
        key = "block_sparse_moe.gate.weight" if "block_sparse_moe.gate.weight" in hf else "mlp.gate.weight"
        out["router.weight"] = hf[key].float()
    elif kind == "moe_mlp":
        e_loc = spec.experts // ep
        fc1, fc2 = [], []
        fused = "mlp.experts.gate_up_proj" in hf   # newer layout: [E, 2F, H] (gate rows, then up rows) and [E, H, F]
        for j in range(e_loc):
            e = ep_rank * e_loc + j
            if fused:
                gu = hf["mlp.experts.gate_up_proj"][e]
                F = gu.shape[0] // 2
                w1, w3, w2 = gu[:F], gu[F:], hf["mlp.experts.down_proj"][e]
            else:
                base = "block_sparse_moe.experts.%d." % e
                w1, w3, w2 = hf[base + "w1.weight"], hf[base + "w3.weight"], hf[base + "w2.weight"]
            gate, up = _rows(w1, tp_rank, tp), _rows(w3, tp_rank, tp)
            fc1.append(torch.cat([gate, up], dim=0))
            fc2.append(_cols(w2, tp_rank, tp))
        out["experts.linear_fc1.weight"] = torch.stack(fc1)
        out["experts.linear_fc2.weight"] = torch.stack(fc2)
    else:
        raise KeyError(kind)
    return out


def _split_file(load_dir: str, kind: str, layer_idx: int, gpt: bool) -> str:
    if kind == "embedding":
        return os.path.join(load_dir, "transformer_embedding.pt" if gpt else "model_embed_tokens.pt")
    if kind == "prenorm":
        return os.path.join(load_dir, "transformer_ln_f.pt" if gpt else "model_norm.pt")
    if kind == "lm_head":
        return os.path.join(load_dir, "transformer_embedding.pt" if gpt else "lm_head.pt")
    return os.path.join(load_dir, ("transformer_h_%d.pt" if gpt else "model_layers_%d.pt") % layer_idx)


def _copy_into(module: torch.nn.Module, sd: Dict[str, torch.Tensor], strict: bool = True):
    own = dict(module.named_parameters())
    own.update(dict(module.named_buffers()))
    for k, v in sd.items():
        if k not in own:
            if strict:
                raise KeyError("unexpected key %s (module has %s)" % (k, sorted(own)))
            continue
        with torch.no_grad():
            own[k].copy_(v.to(own[k].dtype).reshape(own[k].shape))


def _unit_modules(model):
    """Yields (layer plan, sub-kind, module, sharded unit, ctx) for every checkpoint unit of this stage."""
    for lp, wrapper in zip(model.model.plans, model.model.units):
        if lp.kind == "moe_decoder":
            ctx = wrapper.attention.inner.attn.attention.ctx
            yield lp, "moe_attention", wrapper.attention.inner, wrapper.attention.unit, ctx
            yield lp, "moe_router", wrapper.router.inner, wrapper.router.unit, ctx
            yield lp, "moe_mlp", wrapper.mlp.inner, wrapper.mlp.unit, ctx
        else:
            inner = wrapper.inner
            ctx = getattr(inner, "ctx", None)
            yield lp, lp.kind, inner, wrapper.unit, ctx


def load_hf_split(model, load_dir: str):
    """Initialise this rank's shards from HF split files."""
    spec = model.spec
    gpt = spec.family == "gpt"
    for lp, kind, module, unit, ctx in _unit_modules(model):
        if kind == "lm_head" and not getattr(module, "owns_weight", True):
            continue
        hf = torch.load(_split_file(load_dir, lp.kind, lp.index - 1, gpt), map_location="cpu", weights_only=True)
        if kind == "lm_head" and gpt:
            hf = {"weight": hf["wte.weight"]}
        if kind == "lm_head" and spec.tied and not gpt and "weight" not in hf:
            hf = {"weight": torch.load(_split_file(load_dir, "embedding", 0, gpt), map_location="cpu",
                                       weights_only=True)["embed_tokens.weight"]}
        tp_rank, tp = (ctx.tp_rank, ctx.tp_size) if ctx is not None else (0, 1)
        ep_rank, ep = (ctx.ep_rank, ctx.ep_size) if (ctx is not None and kind == "moe_mlp") else (0, 1)
        if kind == "moe_mlp":
            tp_rank, tp = ctx.etp_rank, ctx.etp_size
        sd = shard_from_hf(kind, hf, spec, tp_rank, tp, ep_rank, ep)
        unit.gather()
        _copy_into(module, sd, strict=True)   # a key the module does not have is a naming bug, not something to skip
        unit.reload_master()
        unit.release()


# --------------------------------------------------------------------------------------------
# distributed checkpoint
# --------------------------------------------------------------------------------------------
def _unit_dir(lp, kind: str) -> str:
    i = lp.index - 1
    return {"embedding": "model_embed_tokens", "prenorm": "model_norm", "lm_head": "lm_head",
            "decoder": "model_layers_%d" % i, "moe_attention": "model_layers_%d_attention" % i,
            "moe_router": "model_layers_%d_router" % i, "moe_mlp": "model_layers_%d_mlp" % i}[kind]


def _unit_file(root: str, lp, kind: str, ctx) -> str:
    d = _unit_dir(lp, kind)
    tp = ctx.tp_rank if ctx is not None else 0
    if kind == "moe_router":
        return os.path.join(root, d + ".pt")
    if kind == "moe_mlp":
        return os.path.join(root, d, "%d_%d.pt" % (ctx.ep_rank, ctx.etp_rank))
    return os.path.join(root, d, "%d.pt" % tp)


def save_distributed_checkpoint(model, optimizer, scheduler, iteration: int, save_dir: str, extra: Optional[Dict] = None):
    rank = dist.get_rank() if dist.is_initialized() else 0
    root = os.path.join(save_dir, "iter_%d" % iteration)
    if rank == 0:
        os.makedirs(root, exist_ok=True)
        with open(os.path.join(save_dir, "hybrid_parallel_configs.json"), "w") as f:
            json.dump(model.plan.as_config_dict(), f, indent=2)
        if scheduler is not None:
            with open(os.path.join(root, "opt_param_scheduler.json"), "w") as f:
                json.dump(scheduler.state_dict(), f)
        if extra:
            torch.save(extra, os.path.join(root, "extra_state.pt"))
    if dist.is_initialized():
        dist.barrier()
    for lp, kind, module, unit, ctx in _unit_modules(model):
        if not unit.params:
            continue
        sd = unit.full_state_dict()  # collective inside the unit's sharding group for ZeRO-3
        if unit.rank == 0 and (kind != "moe_router" or (ctx is None or ctx.tp_rank == 0)):
            path = _unit_file(root, lp, kind, ctx)
            os.makedirs(os.path.dirname(path), exist_ok=True)
            torch.save(sd, path)
    os.makedirs(os.path.join(root, "optimizer"), exist_ok=True)
    torch.save(optimizer.state_dict(), os.path.join(root, "optimizer", "%d.pt" % rank))
    if dist.is_initialized():
        dist.barrier()
    return root


def load_distributed_checkpoint(model, optimizer, scheduler, load_dir: str, iteration: int, load_optimizer: bool = True):
    from .plan import check_checkpoint_compatibility

    check_checkpoint_compatibility(model.plan, load_dir)
    rank = dist.get_rank() if dist.is_initialized() else 0
    root = os.path.join(load_dir, "iter_%d" % iteration)
    for lp, kind, module, unit, ctx in _unit_modules(model):
        if not unit.params:
            continue
        sd = torch.load(_unit_file(root, lp, kind, ctx), map_location="cpu", weights_only=True)
        unit.gather()
        _copy_into(module, sd)
        unit.reload_master()
        unit.release()
    if load_optimizer and optimizer is not None:
        p = os.path.join(root, "optimizer", "%d.pt" % rank)
        if os.path.exists(p):
            optimizer.load_state_dict(torch.load(p, map_location=model.device, weights_only=False))
    if scheduler is not None:
        p = os.path.join(root, "opt_param_scheduler.json")
        if os.path.exists(p):
            scheduler.load_state_dict(json.load(open(p)))
    extra = os.path.join(root, "extra_state.pt")
    return torch.load(extra, map_location="cpu", weights_only=False) if os.path.exists(extra) else None


# --------------------------------------------------------------------------------------------
# export
# --------------------------------------------------------------------------------------------
def export_to_hf(ckpt_dir: str, iteration: int, spec: ModelSpec, tp: int = None) -> Dict[str, torch.Tensor]:
    """Merge a dense (llama-family) distributed checkpoint back into HF parameter names."""
    root = os.path.join(ckpt_dir, "iter_%d" % iteration)

    def load_all(d):
        files = sorted(os.listdir(os.path.join(root, d)), key=lambda s: int(s.split(".")[0]))
        return [torch.load(os.path.join(root, d, f), map_location="cpu", weights_only=True) for f in files]

    nh, ng, hd = spec.heads, spec.kv_heads, spec.head_dim
    out: Dict[str, torch.Tensor] = {}
    emb = load_all("model_embed_tokens")
    out["model.embed_tokens.weight"] = torch.cat([s["embed_tokens.weight"] for s in emb], dim=0)[: spec.vocab]
    for i in range(spec.layers):
        shards = load_all("model_layers_%d" % i)
        t = len(shards)
        qs, ks, vs = zip(*[unpack_qkv(s["attn.attention.linear_qkv.weight"], nh // t, ng // t, hd) for s in shards])
        p = "model.layers.%d." % i
        out[p + "self_attn.q_proj.weight"], out[p + "self_attn.k_proj.weight"], out[p + "self_attn.v_proj.weight"] = \
            torch.cat(qs), torch.cat(ks), torch.cat(vs)
        out[p + "self_attn.o_proj.weight"] = torch.cat([s["attn.attention.linear_proj.weight"] for s in shards], dim=1)
        out[p + "input_layernorm.weight"] = shards[0]["attn.input_layernorm.weight"]
        out[p + "post_attention_layernorm.weight"] = shards[0]["ffn.post_attention_layernorm.weight"]
        gates, ups = zip(*[s["ffn.mlp.linear_fc1.weight"].chunk(2, dim=0) for s in shards])
        out[p + "mlp.gate_proj.weight"], out[p + "mlp.up_proj.weight"] = torch.cat(gates), torch.cat(ups)
        out[p + "mlp.down_proj.weight"] = torch.cat([s["ffn.mlp.linear_fc2.weight"] for s in shards], dim=1)
    out["model.norm.weight"] = load_all("model_norm")[0]["norm.weight"]
    if os.path.isdir(os.path.join(root, "lm_head")) and os.listdir(os.path.join(root, "lm_head")):
        out["lm_head.weight"] = torch.cat([s["lm_head.weight"] for s in load_all("lm_head")], dim=0)[: spec.vocab]
    else:
        out["lm_head.weight"] = out["model.embed_tokens.weight"]
    return out
