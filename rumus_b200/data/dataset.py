"""Dataset protocol (rumus/src/data/dataset.rs:7-31) and synthetic generators for the benchmark
configurations."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch


@dataclass
class DataItem:
    input: torch.Tensor
    target: torch.Tensor


class Dataset:
    def __len__(self) -> int:
        raise NotImplementedError

    def get(self, index: int) -> DataItem:
        raise NotImplementedError

    def __getitem__(self, index: int) -> DataItem:
        return self.get(index)


class TensorDataset(Dataset):
    def __init__(self, inputs: torch.Tensor, targets: torch.Tensor):
        assert inputs.shape[0] == targets.shape[0]
        self.inputs, self.targets = inputs, targets

    def __len__(self):
        return self.inputs.shape[0]

    def get(self, index):
        return DataItem(self.inputs[index], self.targets[index])


class SyntheticTokens(Dataset):
    """Token ids uniform in ``[0, vocab)`` from a seed; target = input shifted by one."""

    def __init__(self, n: int, seq_len: int, vocab: int, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.tokens = torch.randint(0, vocab, (n, seq_len + 1), generator=g)

    def __len__(self):
        return self.tokens.shape[0]

    def get(self, index):
        t = self.tokens[index]
        return DataItem(t[:-1], t[1:])


class SyntheticImages(Dataset):
    """N(0,1) images with labels uniform over ``num_classes`` (the ResNet-50 configuration)."""

    def __init__(self, n: int, shape: Sequence[int] = (3, 224, 224), num_classes: int = 1000, seed: int = 0):
        self.n, self.shape, self.num_classes, self.seed = n, tuple(shape), num_classes, seed

    def __len__(self):
        return self.n

    def get(self, index):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + index)
        return DataItem(torch.randn(self.shape, generator=g),
                        torch.randint(0, self.num_classes, (), generator=g))
