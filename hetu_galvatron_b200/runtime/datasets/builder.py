"""Train / valid / test dataset construction from ``args.data`` (weight-prefix lists, ``split`` proportions,
per-split paths), and the collate function of the GPT path.  Capability parity:
galvatron/core/runtime/datasets/megatron/blended_megatron_dataset_builder.py:39-589, blended_megatron_dataset_config.py:15-172,
core/runtime/dataloader.py:460-502."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .blended import BlendedDataset
from .gpt import GPTDataset, GPTDatasetConfig
from .indexed import IndexedDataset

SPLITS = ("train", "valid", "test")


def parse_weighted_paths(items: Optional[Sequence[str]]) -> Tuple[List[str], Optional[List[float]]]:
    """``[p]`` | ``[w1, p1, w2, p2, ...]`` | ``[p1, p2, ...]`` -> (prefixes, weights or None)."""
    if not items:
        return [], None
    items = list(items)
    if len(items) == 1:
        return items, None

    def is_num(s):
        try:
            float(s)
            return True
        except ValueError:
            return False

    if len(items) % 2 == 0 and all(is_num(items[i]) for i in range(0, len(items), 2)):
        return [items[i + 1] for i in range(0, len(items), 2)], [float(items[i]) for i in range(0, len(items), 2)]
    return items, None


def parse_split(split: Optional[str]) -> List[Optional[Tuple[float, float]]]:
    """``"949,50,1"`` -> cumulative fractions per split (``None`` for an empty split)."""
    if not split:
        return [(0.0, 1.0), None, None]
    w = [float(x) for x in split.replace("/", ",").split(",")]
    w = (w + [0.0, 0.0, 0.0])[:3]
    tot = sum(w)
    out, acc = [], 0.0
    for x in w:
        out.append((acc / tot, (acc + x) / tot) if x > 0 else None)
        acc += x
    return out


def _gpt_config(args) -> GPTDatasetConfig:
    d, t = args.data, args.train
    eod = None
    try:
        from ...parallel import state

        tok = state.get_tokenizer()
        eod = getattr(tok, "eos_token_id", None) if tok is not None else None
    except Exception:
        pass
    return GPTDatasetConfig(sequence_length=t.seq_length, random_seed=t.seed or 1234, reset_position_ids=d.reset_position_ids,
                            reset_attention_mask=d.reset_attention_mask, eod_mask_loss=d.eod_mask_loss,
                            create_attention_mask=d.create_attention_mask_in_dataloader, path_to_cache=d.data_cache_path,
                            eod_token=eod)


def _one_prefix(prefix: str, bounds, num_samples, cfg: GPTDatasetConfig, mmap: bool):
    indexed = IndexedDataset(prefix, mmap=mmap)
    n_docs = indexed.document_indices.shape[0] - 1
    out = []
    for name, b, ns in zip(SPLITS, bounds, num_samples):
        if b is None:
            out.append(None)
            continue
        lo, hi = int(round(b[0] * n_docs)), int(round(b[1] * n_docs))
        if hi <= lo:
            out.append(None)
            continue
        out.append(GPTDataset(indexed, prefix, np.arange(lo, hi, dtype=np.int32), ns, name, cfg))
    return out


def build_train_valid_test_datasets(args):
    t, d = args.train, args.data
    cfg = _gpt_config(args)
    from ..data import get_train_valid_test_num_samples

    train_n, eval_n, test_n = get_train_valid_test_num_samples(args)
    targets = [train_n or None, eval_n or None, test_n or None]
    per_split = [d.train_data_path, d.valid_data_path, d.test_data_path]
    results = []
    if any(per_split):
        for i, (paths, n) in enumerate(zip(per_split, targets)):
            prefixes, weights = parse_weighted_paths(paths)
            if not prefixes:
                results.append(None)
                continue
            bounds = [None, None, None]
            bounds[i] = (0.0, 1.0)
            parts = [_one_prefix(p, bounds, [n if j == i else None for j in range(3)], cfg, d.mmap_bin_files)[i] for p in prefixes]
            results.append(parts[0] if len(parts) == 1 else BlendedDataset(parts, weights, n))
        return tuple(results)
    prefixes, weights = parse_weighted_paths(d.data_path)
    bounds = parse_split(d.split)
    per_prefix = [_one_prefix(p, bounds, targets, cfg, d.mmap_bin_files) for p in prefixes]
    for i in range(3):
        parts = [pp[i] for pp in per_prefix if pp[i] is not None]
        if not parts:
            results.append(None)
        elif len(parts) == 1:
            results.append(parts[0])
        else:
            results.append(BlendedDataset(parts, weights, targets[i]))
    return tuple(results)


def gpt_collate_fn(batch):
    tokens = torch.stack([b["tokens"] for b in batch])
    labels = torch.stack([b["labels"] for b in batch])
    loss_mask = torch.stack([b["loss_mask"] for b in batch])
    kw = {"attention_mask": None, "labels": labels, "loss_mask": loss_mask, "rotary_embedding": None,
          "position_ids": torch.stack([b["position_ids"] for b in batch])}
    return tokens, kw, None
