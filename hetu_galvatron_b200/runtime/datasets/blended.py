"""Weighted mixture of datasets.  Sample ``i`` of the blend comes from dataset ``dataset_index[i]`` at position
``dataset_sample_index[i]``; both tables are produced by the native greedy builder so that after any prefix the
per-dataset counts track the target weights (galvatron/core/runtime/datasets/megatron/blended_dataset.py:24-201)."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .gpt import load_helpers


def normalize(weights: Sequence[float]) -> List[float]:
    w = np.asarray(weights, dtype=np.float64)
    return list(w / w.sum())


class BlendedDataset(torch.utils.data.Dataset):
    def __init__(self, datasets: List[torch.utils.data.Dataset], weights: Optional[Sequence[float]], size: Optional[int]):
        if not datasets:
            raise ValueError("no datasets to blend")
        self.datasets = datasets
        h = load_helpers()
        n = len(datasets)
        if weights is None or size is None:  # exhaustive: every dataset exactly once
            sizes = np.asarray([len(d) for d in datasets], dtype=np.int64)
            self.size = int(sizes.sum())
            self.dataset_index = np.zeros(self.size, dtype=np.int16)
            self.dataset_sample_index = np.zeros(self.size, dtype=np.int64)
            h.build_exhaustive_blending_indices(self.dataset_index, self.dataset_sample_index, sizes, n)
        else:
            self.size = int(size)
            self.weights = normalize(weights)
            self.dataset_index = np.zeros(self.size, dtype=np.int16)
            self.dataset_sample_index = np.zeros(self.size, dtype=np.int64)
            h.build_blending_indices(self.dataset_index, self.dataset_sample_index,
                                     np.asarray(self.weights, dtype=np.float64), n, self.size, False)

    def __len__(self):
        return self.size

    def __getitem__(self, i):
        d = int(self.dataset_index[i])
        ds = self.datasets[d]
        return dict(ds[int(self.dataset_sample_index[i]) % len(ds)], dataset_id=d)
