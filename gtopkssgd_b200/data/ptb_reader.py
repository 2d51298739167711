"""Penn Treebank reader (reference: ptb_reader.py:9-102): vocabulary by
descending frequency, ``<eos>`` at line ends, fixed windows of ``num_steps``
tokens with the target shifted by one."""
from __future__ import annotations

import collections
import os

import numpy as np
from torch.utils.data import Dataset


def _read_words(path):
    with open(path, "r") as fh:
        return fh.read().replace("\n", "<eos>").split()


def _build_vocab(path):
    counts = collections.Counter(_read_words(path))
    ordered = sorted(counts.items(), key=lambda kv: (-kv[1], kv[0]))
    word_to_id = {w: i for i, (w, _) in enumerate(ordered)}
    return word_to_id, {i: w for w, i in word_to_id.items()}


def _file_to_word_ids(path, word_to_id):
    return [word_to_id[w] for w in _read_words(path) if w in word_to_id]


def ptb_raw_data(data_path=None, prefix="ptb"):
    """(train ids, valid ids, test ids, word_to_id, id_to_word)."""
    paths = [os.path.join(data_path, "%s.%s.txt" % (prefix, part)) for part in ("train", "valid", "test")]
    word_to_id, id_to_word = _build_vocab(paths[0])
    train, valid, test = (_file_to_word_ids(p, word_to_id) for p in paths)
    return train, valid, test, word_to_id, id_to_word


class _WindowDataset(Dataset):
    def __init__(self, raw_data, batch_size, num_steps):
        self.raw_data = np.asarray(raw_data, dtype=np.int64)
        self.batch_size, self.num_steps = batch_size, num_steps
        self.data_len = len(self.raw_data)
        self.sample_len = self.data_len // num_steps

    def __getitem__(self, idx):
        a, b = self.num_steps * idx, self.num_steps * (idx + 1)
        return self.raw_data[a:b], self.raw_data[a + 1:b + 1]

    def __len__(self):
        return self.sample_len - self.sample_len % self.batch_size


class TrainDataset(_WindowDataset):
    pass


class TestDataset(_WindowDataset):
    __test__ = False  # not a pytest class
