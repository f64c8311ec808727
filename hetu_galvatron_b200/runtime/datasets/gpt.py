"""GPT dataset: packs the documents of an indexed dataset into ``seq_length + 1`` token samples.

Three cached index arrays (``.npy`` files named by an MD5 of the configuration) drive it: the *document index*
(document ids repeated per epoch and shuffled), the *sample index* (for sample ``i``: position in the document
index and token offset where it starts -- built by the native ``build_sample_idx``) and the *shuffle index*
(permutation of the samples).  ``__getitem__`` returns ``tokens, labels, loss_mask, position_ids`` (+
``attention_mask`` on request).  Capability parity: galvatron/core/runtime/datasets/megatron/gpt_dataset.py:65-232,
:304-523; helpers.py:11-64.
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np
import torch

from .indexed import IndexedDataset


def load_helpers():
    try:
        from ..._lib import hg_dataset_helpers  # type: ignore

        return hg_dataset_helpers
    except Exception:
        from ...csrc import build as _build

        _build.build_host()
        import importlib

        return importlib.import_module("hetu_galvatron_b200._lib.hg_dataset_helpers")


def build_sample_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch, drop_last=True, add_extra_token=1):
    """int32 table when every entry fits, else int64 (the native builders are typed)."""
    h = load_helpers()
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    doc_idx = np.ascontiguousarray(doc_idx, dtype=np.int32)
    fn = h.build_sample_idx_int32 if max(doc_idx.shape[0], int(sizes.max(initial=0))) < np.iinfo(np.int32).max \
        else h.build_sample_idx_int64
    return fn(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch, drop_last, add_extra_token)


def build_sample_idx_reference(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch, drop_last=True, extra=1):
    """Pure-Python oracle of the native builder (tests)."""
    total = num_epochs * tokens_per_epoch - extra
    n = total // seq_length if drop_last else -(-total // seq_length)
    out = np.zeros((n + 1, 2), dtype=np.int64)
    cur, off, s = 0, 0, 1
    while s <= n:
        remaining = seq_length + extra
        while remaining != 0:
            dl = int(sizes[doc_idx[cur]]) - off
            remaining -= dl
            if remaining <= 0:
                off += remaining + dl - extra
                remaining = 0
            else:
                if cur == len(doc_idx) - 1:
                    off = int(sizes[doc_idx[cur]]) - extra
                    break
                cur += 1
                off = 0
        out[s] = (cur, off)
        s += 1
    return out


@dataclass
class GPTDatasetConfig:
    sequence_length: int
    random_seed: int = 1234
    reset_position_ids: bool = False
    reset_attention_mask: bool = False
    eod_mask_loss: bool = False
    create_attention_mask: bool = False
    add_extra_token_to_sequence: bool = True
    drop_last_partial_validation_sequence: bool = True
    path_to_cache: Optional[str] = None
    eod_token: Optional[int] = None
    pad_token: Optional[int] = None


class GPTDataset(torch.utils.data.Dataset):
    def __init__(self, indexed: IndexedDataset, prefix: str, documents: np.ndarray, num_samples: Optional[int],
                 split_name: str, config: GPTDatasetConfig):
        self.indexed, self.prefix, self.documents, self.config, self.split = indexed, prefix, documents, config, split_name
        self.num_samples = num_samples
        self.doc_index, self.sample_index, self.shuffle_index = self._build_or_load()

    # ---- indices ------------------------------------------------------------------------------------------
    def _key(self) -> str:
        desc = {"prefix": os.path.basename(self.prefix), "split": self.split, "docs": [int(self.documents[0]), int(self.documents[-1]), len(self.documents)],
                "seq": self.config.sequence_length, "seed": self.config.random_seed, "samples": self.num_samples,
                "extra": self.config.add_extra_token_to_sequence}
        return hashlib.md5(json.dumps(desc, sort_keys=True).encode()).hexdigest()

    def _build_or_load(self):
        """The three index arrays of this split.  With ``torch.distributed`` initialised, global rank 0 builds and
        writes them (to temporary names, moved into place with ``os.replace`` so a reader never sees a partial file),
        all ranks meet at a barrier, and the others then memory-map the finished files (the reference builds on rank 0
        first as well: gpt_dataset.py:354, blended_megatron_dataset_builder.py:417)."""
        import torch.distributed as dist

        cache = self.config.path_to_cache or os.path.join(os.path.dirname(self.prefix) or ".", "cache", "GPTDataset_indices")
        base = os.path.join(cache, self._key())
        paths = [base + "-%s.npy" % n for n in ("document_index", "sample_index", "shuffle_index")]

        def load():
            return tuple(np.load(p, allow_pickle=False, mmap_mode="r") for p in paths)

        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
        builder = (not multi) or dist.get_rank() == 0
        built = None
        if builder and not all(os.path.exists(p) for p in paths):
            built = self._build_indices()
            os.makedirs(cache, exist_ok=True)
            for p, a in zip(paths, built):
                tmp = "%s.tmp.%d.npy" % (p[:-4], os.getpid())   # np.save appends ".npy" to other suffixes
                np.save(tmp, a, allow_pickle=False)
                os.replace(tmp, p)
        if multi:
            dist.barrier()
        return built if built is not None else load()

    def _build_indices(self):
        cfg = self.config
        extra = 1 if cfg.add_extra_token_to_sequence else 0
        sizes = self.indexed.sequence_lengths
        tokens_per_epoch = int(np.sum(sizes[self.documents]))
        epochs = 1
        if self.num_samples is not None:
            while (epochs * tokens_per_epoch - extra) // cfg.sequence_length < self.num_samples:
                epochs += 1
        rng = np.random.RandomState(cfg.random_seed)
        doc_index = np.tile(self.documents.astype(np.int32), epochs)
        rng.shuffle(doc_index)
        sample_index = build_sample_idx(sizes, doc_index, cfg.sequence_length, epochs, tokens_per_epoch,
                                        cfg.drop_last_partial_validation_sequence or self.split == "train", extra)
        n = sample_index.shape[0] - 1
        shuffle_index = np.arange(n, dtype=np.uint32 if n < 2 ** 32 - 1 else np.int64)
        rng.shuffle(shuffle_index)
        return doc_index, sample_index, shuffle_index

    # ---- samples -------------------------------------------------------------------------------------------
    def __len__(self):
        return self.sample_index.shape[0] - 1

    def _tokens(self, i: int) -> np.ndarray:
        i = int(self.shuffle_index[i])
        d0, o0 = (int(x) for x in self.sample_index[i])
        d1, o1 = (int(x) for x in self.sample_index[i + 1])
        extra = 1 if self.config.add_extra_token_to_sequence else 0
        if d0 == d1:
            return np.asarray(self.indexed.get(int(self.doc_index[d0]), o0, o1 - o0 + extra), dtype=np.int64)
        parts = [self.indexed.get(int(self.doc_index[d0]), o0)]
        for d in range(d0 + 1, d1):
            parts.append(self.indexed.get(int(self.doc_index[d])))
        parts.append(self.indexed.get(int(self.doc_index[d1]), 0, o1 + extra))
        return np.concatenate(parts).astype(np.int64)

    def __getitem__(self, i) -> Dict[str, torch.Tensor]:
        cfg = self.config
        text = torch.from_numpy(self._tokens(i % len(self)))
        L = cfg.sequence_length
        if text.numel() < L + 1:
            pad = cfg.pad_token if cfg.pad_token is not None else 0
            text = torch.cat([text, torch.full((L + 1 - text.numel(),), pad, dtype=torch.long)])
        tokens, labels = text[:L].contiguous(), text[1:L + 1].contiguous()
        loss_mask = torch.ones(L, dtype=torch.float)
        position_ids = torch.arange(L, dtype=torch.long)
        eod = cfg.eod_token
        if eod is not None:
            if cfg.eod_mask_loss:
                loss_mask[tokens == eod] = 0.0
            if cfg.reset_position_ids:
                prev = 0
                for j in (tokens == eod).nonzero().flatten().tolist():
                    position_ids[j + 1:] -= j + 1 - prev
                    prev = j + 1
        if cfg.pad_token is not None:
            loss_mask[labels == cfg.pad_token] = 0.0
        out = {"tokens": tokens, "labels": labels, "loss_mask": loss_mask, "position_ids": position_ids}
        if cfg.create_attention_mask:
            out["attention_mask"] = torch.tril(torch.ones(L, L, dtype=torch.bool)).unsqueeze(0).logical_not()
        return out
