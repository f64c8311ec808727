"""Cached (incremental) forward for generation with a trained model.

The reference carries Megatron's inference hooks only as stubs: ``BaseInferenceContext`` with
"TODO: Support inference" (galvatron/core/runtime/transformer/inference.py:5-20) and the key / value cache branches of
its attention class (transformer/attention.py:253-389, 398-513), which none of its entry points reaches.  This module
is the working counterpart for the layouts where generation makes sense here: one pipeline stage, no Ulysses / context
parallelism, tensor parallelism only when the number of new tokens is divisible by the tp degree (the layers keep their
sequence-parallel activations).

    ctx = StaticInferenceContext(max_batch_size=B, max_sequence_length=S_max)
    logits = forward_step(model, prompt, ctx)          # prefill: [S_prompt, B, V / tp]
    logits = forward_step(model, next_tokens, ctx)     # one or more new tokens per call
    tokens = greedy_generate(model, prompt, 16)
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .modules import SelfAttention


class StaticInferenceContext:
    """Static batching: one key / value buffer ``[max_sequence_length, max_batch_size, kv_heads / tp, head_dim]`` per
    layer, allocated on first use, and the number of tokens already cached."""

    def __init__(self, max_batch_size: int, max_sequence_length: int):
        self.max_batch_size = int(max_batch_size)
        self.max_sequence_length = int(max_sequence_length)
        self.sequence_len_offset = 0
        self.batch_size_offset = 0
        self.key_value_memory_dict: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}

    def is_static_batching(self) -> bool:
        return True

    def is_dynamic_batching(self) -> bool:
        return False

    def reset(self):
        """Forget the cached tokens (the buffers are kept and overwritten)."""
        self.sequence_len_offset = 0
        self.batch_size_offset = 0

    def swap_key_value_dict(self, batch_idx: torch.Tensor):
        """Reorder the cached sequences along the batch dimension (beam search)."""
        for key, (k, v) in self.key_value_memory_dict.items():
            self.key_value_memory_dict[key] = (k.index_select(1, batch_idx), v.index_select(1, batch_idx))


def _stage(model):
    return model.model if hasattr(model, "model") and hasattr(model.model, "units") else model


@torch.no_grad()
def forward_step(model, tokens: torch.Tensor, ctx: StaticInferenceContext) -> torch.Tensor:
    """Run ``tokens [B, S_new]`` through the stage with the caches of ``ctx`` and advance it.  Returns the local
    logits ``[S_new, B, V / tp]`` (vocab-parallel: gather over the vocab tp group for the full distribution)."""
    stage = _stage(model)
    if not (stage.has_embedding and stage.has_head):
        raise NotImplementedError("cached generation runs on a single pipeline stage")
    attns = [m for m in stage.modules() if isinstance(m, SelfAttention)]
    for a in attns:
        a.inference_context = ctx
    try:
        logits = stage(tokens, None)
    finally:
        for a in attns:
            a.inference_context = None
    ctx.sequence_len_offset += tokens.shape[1]
    return logits


@torch.no_grad()
def greedy_generate(model, prompt: torch.Tensor, max_new_tokens: int, vocab_group=None,
                    new_tokens_per_step: int = 1) -> torch.Tensor:
    """Greedy continuation of ``prompt [B, S]``: prefill once, then one token per step.  With a vocab-parallel head
    pass its group (a ``parallel.groups.CommGroup``, e.g. ``model.vocab_ctx.tp``) so that the arg-max runs over the
    gathered vocabulary.

    Tensor-parallel layers keep sequence-parallel activations, so every call must feed a multiple of the tp degree:
    with ``new_tokens_per_step = t`` each step re-feeds the last ``t - 1`` cached tokens together with the new one
    (the cache offset is moved back accordingly), which costs ``t`` rows per step instead of one."""
    import torch.distributed as dist

    B, S = prompt.shape
    t = max(1, int(new_tokens_per_step))
    if S % t:
        raise ValueError("the prompt length (%d) must be divisible by new_tokens_per_step (%d)" % (S, t))
    ctx = StaticInferenceContext(B, S + max_new_tokens)
    seq = prompt
    feed = prompt
    for _ in range(max_new_tokens):
        logits = forward_step(model, feed, ctx)[-1]                   # [B, V / tp]
        if vocab_group is not None and vocab_group.size > 1:
            parts = [torch.empty_like(logits) for _ in range(vocab_group.size)]
            dist.all_gather(parts, logits.contiguous(), group=vocab_group.group)
            logits = torch.cat(parts, dim=-1)
        nxt = logits.float().argmax(dim=-1, keepdim=True).to(prompt.dtype)
        seq = torch.cat([seq, nxt], dim=1)
        feed = seq[:, -t:]                                            # the new token and the t - 1 before it
        ctx.sequence_len_offset = seq.shape[1] - t                    # their keys / values are simply rewritten
    return seq
