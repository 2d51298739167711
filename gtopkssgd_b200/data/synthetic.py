"""Synthetic datasets with the shapes of the supported workloads.

* images: fp32 ``N(0,1)`` tensors ``[3, S, S]`` with labels uniform in
  ``[0, classes)`` (CIFAR-style S=32, ImageNet-style S=224, MNIST 1x28x28);
* PTB: token ids uniform in ``[0, vocab)``, next-token targets;
* AN4: log-spectrogram-like ``[1, 161, T]`` inputs with random transcripts.

Samples come from a small pre-generated pool, so a data loader never becomes
the bottleneck of a throughput measurement, and a given (seed, index) always
yields the same sample on every rank.
"""
from __future__ import annotations

import torch
from torch.utils.data import Dataset


class SyntheticImages(Dataset):
    def __init__(self, length: int, shape=(3, 32, 32), num_classes: int = 10, pool: int = 256, seed: int = 1234):
        g = torch.Generator().manual_seed(seed)
        self.length = int(length)
        self.pool = min(pool, self.length)
        self.images = torch.randn((self.pool,) + tuple(shape), generator=g)
        self.labels = torch.randint(0, num_classes, (self.pool,), generator=g)

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        j = i % self.pool
        return self.images[j], self.labels[j]


class SyntheticPTB(Dataset):
    """Windows of ``num_steps`` tokens over a random corpus, target shifted by
    one (same indexing as the PTB reader)."""

    def __init__(self, num_tokens: int = 929589, vocab_size: int = 10000, batch_size: int = 20, num_steps: int = 35,
                 seed: int = 1234):
        g = torch.Generator().manual_seed(seed)
        self.raw = torch.randint(0, vocab_size, (num_tokens + 1,), generator=g)
        self.num_steps, self.batch_size = num_steps, batch_size
        n = num_tokens // num_steps
        self.length = n - n % batch_size

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        a = i * self.num_steps
        return self.raw[a:a + self.num_steps], self.raw[a + 1:a + 1 + self.num_steps]


class SyntheticAN4(Dataset):
    """(spectrogram [1, 161, T], transcript ids) with T in [min_t, max_t]."""

    def __init__(self, length: int = 948, n_labels: int = 29, min_t: int = 100, max_t: int = 400, seed: int = 1234):
        g = torch.Generator().manual_seed(seed)
        self.length = length
        self.frames = torch.randint(min_t, max_t + 1, (length,), generator=g)
        self.ntok = torch.randint(5, 30, (length,), generator=g)
        self.n_labels = n_labels
        self.seed = seed
        self.ids = list(range(length))

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed + 7919 * int(i))
        spect = torch.randn(161, int(self.frames[i]), generator=g)
        target = torch.randint(1, self.n_labels, (int(self.ntok[i]),), generator=g).tolist()
        return spect, target
