"""Batches for training: synthetic token streams, samplers, the per-rank batch contract.

The engine consumes ``(tokens [B_local, S], {"labels": [B_local, S], "loss_mask": ...})`` where ``B_local`` is
this rank's share of the global batch over the *vocab layers'* data-parallel group.  Ranks that differ only in
their tensor / sequence / context-parallel coordinate must see the same samples: the sampler is indexed by the
data-parallel rank only (the reference instead reads on tensor-parallel rank 0 and broadcasts,
galvatron/core/runtime/dataloader.py:509-550, utils/utils.py:194-292 -- :func:`broadcast_batch` offers that too).

Datasets: :class:`RandomTokenDataset` / :class:`FakeCausalLMDataset` (uniform random ids, fixed seed;
datasets/random_dataset.py:11-46, dataloader.py:35-66), and the indexed GPT datasets of
``runtime/datasets`` through :func:`build_train_valid_test_datasets`.  Samplers follow Megatron's
``MegatronPretrainingSampler`` (sequential, resumable by ``consumed_samples``) and
``MegatronPretrainingRandomSampler`` (epoch-shuffled buckets) (dataloader.py:113-159, :184-251).
"""
from __future__ import annotations

from typing import Dict, Iterator, List, Optional, Tuple

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset


class RandomTokenDataset(Dataset):
    """``size`` sequences of ``seq_length + 1`` uniform random token ids, reproducible from ``seed``."""

    def __init__(self, vocab_size: int, seq_length: int, size: int = 4096, seed: int = 1234):
        g = torch.Generator().manual_seed(seed)
        self.data = torch.randint(0, vocab_size, (size, seq_length + 1), generator=g)
        self.vocab_size, self.seq_length = vocab_size, seq_length

    def __len__(self):
        return self.data.shape[0]

    def __getitem__(self, i):
        row = self.data[i % len(self)]
        return {"tokens": row[:-1], "labels": row[1:]}


class FakeCausalLMDataset(RandomTokenDataset):
    """Alias kept for the profiling paths (a fake dataset whose length covers the requested iterations)."""


def get_train_valid_test_num_samples(args):
    """Samples each split must provide: ``(train, valid, test)`` from the iteration counts and the global batch
    (dataloader.py:299-318)."""
    t = args.train
    gbsz = t.global_batch_size
    train_n = (t.train_iters or 0) * gbsz if t.train_iters else (t.train_samples or 0)
    eval_n = ((t.train_iters or 0) // max(1, t.eval_interval or 1) + 1) * (t.eval_iters or 0) * gbsz
    test_n = (t.eval_iters or 0) * gbsz
    return train_n, eval_n, test_n


def random_collate_fn(batch: List[Dict[str, torch.Tensor]]):
    tokens = torch.stack([b["tokens"] for b in batch])
    labels = torch.stack([b["labels"] for b in batch])
    return tokens, {"attention_mask": None, "labels": labels, "rotary_embedding": None}, None


class PretrainingSampler:
    """Sequential, resumable: batch ``k`` of data-parallel rank ``r`` is samples
    ``[consumed + k*gbsz + r*mbs, ... + (r+1)*mbs)``."""

    def __init__(self, total_samples: int, consumed_samples: int, local_batch_size: int, dp_rank: int, dp_size: int,
                 drop_last: bool = True):
        if total_samples <= 0 or local_batch_size <= 0 or not (0 <= dp_rank < dp_size):
            raise AssertionError("bad sampler arguments")
        self.total, self.consumed, self.lbs = total_samples, consumed_samples, local_batch_size
        self.rank, self.size, self.drop_last = dp_rank, dp_size, drop_last
        self.gbs = local_batch_size * dp_size

    def __len__(self):
        return self.total

    def __iter__(self) -> Iterator[List[int]]:
        batch = []
        for idx in range(self.consumed, self.total):
            batch.append(idx)
            if len(batch) == self.gbs:
                yield batch[self.rank * self.lbs:(self.rank + 1) * self.lbs]
                batch = []
        if batch and not self.drop_last:
            yield batch[self.rank * self.lbs:(self.rank + 1) * self.lbs]


class PretrainingRandomSampler:
    """Epoch-wise shuffled; every data-parallel rank draws from its own bucket (or from a shuffled global
    order when ``data_sharding`` is off)."""

    def __init__(self, dataset_len: int, total_samples: int, consumed_samples: int, local_batch_size: int,
                 dp_rank: int, dp_size: int, data_sharding: bool = True, seed: int = 1234):
        self.n, self.total, self.consumed, self.lbs = dataset_len, total_samples, consumed_samples, local_batch_size
        self.rank, self.size, self.sharding, self.seed = dp_rank, dp_size, data_sharding, seed
        self.gbs = local_batch_size * dp_size
        self.last_batch = self.total % self.gbs

    def __len__(self):
        return self.total

    def __iter__(self):
        active = self.total - self.last_batch
        epoch = self.consumed // active
        cur = self.consumed % active
        g = torch.Generator().manual_seed(self.seed + epoch)
        if self.sharding:
            bucket = (self.total // self.gbs) * self.lbs
            offset = cur // self.size
            start = self.rank * bucket
            order = [start + int(x) for x in torch.randperm(bucket, generator=g).tolist()[offset:]]
        else:
            full = (self.total // self.lbs) * self.lbs
            perm = torch.randperm(full, generator=g).tolist()
            order = perm[cur + self.rank::self.size]
        batch = []
        for idx in order:
            batch.append(idx % self.n)
            if len(batch) == self.lbs:
                self.consumed += self.gbs
                yield batch
                batch = []


def build_dataloader(dataset, consumed_samples: int, local_batch_size: int, dp_rank: int, dp_size: int,
                     dataloader_type: str = "single", num_workers: int = 0, seed: int = 1234, collate_fn=None,
                     data_sharding: bool = True):
    if dataset is None:
        return None
    if dataloader_type == "single":
        sampler = PretrainingSampler(len(dataset), consumed_samples, local_batch_size, dp_rank, dp_size)
    elif dataloader_type == "cyclic":
        sampler = PretrainingRandomSampler(len(dataset), len(dataset), consumed_samples, local_batch_size, dp_rank,
                                           dp_size, data_sharding, seed)
    elif dataloader_type == "external":
        return dataset
    else:
        raise ValueError(dataloader_type)
    return DataLoader(dataset, batch_sampler=sampler, num_workers=num_workers, pin_memory=torch.cuda.is_available(),
                      collate_fn=collate_fn, persistent_workers=num_workers > 0)


def cyclic_iter(loader):
    while True:
        for x in loader:
            yield x


def get_train_valid_test_data_iterators(args, model, collate_fn=None):
    """(train, valid, test) iterators for this rank; random tokens when ``data.use_random_dataset`` or no path."""
    t, d = args.train, args.data
    c = model.vocab_ctx
    dp_rank = c.dp.rank if c.dp is not None else 0
    dp_size = c.dp.size if c.dp is not None else 1
    lbs = model.local_batch_size()
    vocab = args.model.vocab_size
    if d.use_random_dataset or not (d.data_path or d.train_data_path):
        n = max(4096, (t.train_iters or 1) * t.global_batch_size)
        train = RandomTokenDataset(vocab, t.seq_length, min(n, 65536), seed=t.seed or 1234)
        valid = test = None
        coll = collate_fn or random_collate_fn
    else:
        from .datasets.builder import build_train_valid_test_datasets, gpt_collate_fn

        train, valid, test = build_train_valid_test_datasets(args)
        coll = collate_fn or gpt_collate_fn
    consumed = t.consumed_train_samples or (t.iteration or 0) * t.global_batch_size

    def it(ds, consumed_samples):
        if ds is None:
            return None
        loader = build_dataloader(ds, consumed_samples, lbs, dp_rank, dp_size, t.dataloader_type, 0, t.seed or 1234,
                                  coll, t.data_sharding)
        return iter(cyclic_iter(loader)) if t.dataloader_type == "cyclic" else iter(loader)

    out = it(train, consumed % max(1, len(train))), it(valid, 0), it(test, 0)
    # which phases have data and iterations to run (the reference sets the same flags: runtime/dataloader.py:363-384)
    if t.skip_train:
        t.do_train = False
    else:
        t.do_train = bool(t.do_train) or (out[0] is not None and (t.train_iters or 0) > 0)
    t.do_valid = bool(t.do_valid) or (out[1] is not None and (t.eval_iters or 0) > 0)
    t.do_test = bool(t.do_test) or (out[2] is not None and (t.eval_iters or 0) > 0)
    return out


def get_batch(data_iterator, device) -> Tuple[torch.Tensor, Dict, Optional[object]]:
    """Next batch on ``device``: ``(tokens, {"labels", "loss_mask", ...}, loss_func | None)``."""
    item = next(data_iterator)
    tokens, kw, loss_fn = item if isinstance(item, (tuple, list)) else (item["tokens"], {"labels": item["labels"]}, None)
    nb = device.type == "cuda"
    tokens = tokens.to(device, non_blocking=nb)
    kw = {k: (v.to(device, non_blocking=nb) if torch.is_tensor(v) else v) for k, v in kw.items()}
    return tokens, kw, loss_fn


def broadcast_batch(tokens: Optional[torch.Tensor], kwargs: Dict, group, device, shape, src_rank_in_group: int = 0):
    """The reference's loading scheme: only one rank of a tensor-parallel group reads, the others receive."""
    import torch.distributed as dist

    if group is None or group.size == 1:
        return tokens, kwargs
    src = group.ranks[src_rank_in_group]
    if group.rank != src_rank_in_group:
        tokens = torch.empty(shape, dtype=torch.long, device=device)
        kwargs = {"labels": torch.empty(shape, dtype=torch.long, device=device)}
    dist.broadcast(tokens, src=src, group=group.group)
    dist.broadcast(kwargs["labels"], src=src, group=group.group)
    return tokens, kwargs


def loss_func_with_mask(loss_mask: Optional[torch.Tensor]):
    """``sum(loss * mask) / sum(mask)`` (the reference's closure, dataloader.py:541-550)."""

    def fn(per_token_loss):
        if loss_mask is None:
            return per_token_loss.float().mean()
        m = loss_mask.reshape(per_token_loss.shape).float()
        return (per_token_loss.float() * m).sum() / m.sum().clamp(min=1)

    return fn
