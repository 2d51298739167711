"""Compressor registry with the reference's public surface
(compression.py:8-94): ``compressors = {'topk', 'topk2', 'gtopk', 'none'}``,
static ``compress / add_residuals / get_residuals / decompress`` and
class-level state keyed by the merged-group name.

``compress`` is the stand-alone form of the operation: it runs the fused K1
kernel (or the oracle on CPU) and then materialises the sparsified dense
vector in ``tensor`` as the reference does.  The training engine does not go
through this materialising form; it keeps the k pairs sparse end to end.
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch

from ..ops.oracle import num_selected
from ..ops.select import TopkSelector
from ..ops.sgd import scatter_dense


class NoneCompressor:
    name = "none"

    @staticmethod
    def compress(tensor, name=None, sigma_scale=2.5, ratio=1.0):
        return tensor, None

    @staticmethod
    def decompress(tensor, ctc, name=None):
        return tensor

    @staticmethod
    def get_residuals(name, like_tensor):
        return torch.zeros_like(like_tensor)

    @staticmethod
    def add_residuals(included_indexes, name):
        return None


class TopKCompressor:
    """Top-k sparsification with residual accumulation (Aji & Heafield 2017)."""
    residuals: Dict[str, torch.Tensor] = {}
    values: Dict[str, torch.Tensor] = {}
    indexes: Dict[str, torch.Tensor] = {}
    selectors: Dict[str, TopkSelector] = {}
    sparsities: list = []
    name = "topk"

    @classmethod
    def clear(cls) -> None:
        for d in (TopKCompressor.residuals, TopKCompressor.values, TopKCompressor.indexes, TopKCompressor.selectors):
            d.clear()

    @staticmethod
    def get_residuals(name, like_tensor):
        res = TopKCompressor.residuals
        if name not in res:
            res[name] = torch.zeros_like(like_tensor.data).view(-1)
        return res[name]

    @staticmethod
    def _selector(name: str, flat: torch.Tensor, k: int) -> TopkSelector:
        sel = TopKCompressor.selectors.get(name)
        if sel is None or sel.numel != flat.numel() or sel.max_k < k or sel.device != flat.device:
            sel = TopkSelector(flat.numel(), k, flat.device)
            TopKCompressor.selectors[name] = sel
        return sel

    @staticmethod
    def compress(tensor, name=None, sigma_scale=2.5, ratio=0.05):
        with torch.no_grad():
            flat = tensor.data.view(-1)
            k = num_selected(flat.numel(), ratio)
            residual = TopKCompressor.get_residuals(name, flat)
            sel = TopKCompressor._selector(name, flat, k)
            sel.select(flat, residual, k)
            counts = sel.n_sel_tensor
            scatter_dense(flat, sel.sel, counts, 1, sel.max_k, 1.0)
            idx, val = sel.pairs()
            TopKCompressor.values[name] = val.clone()
            TopKCompressor.indexes[name] = idx
            return tensor, idx

    @staticmethod
    def add_residuals(included_indexes, name):
        """``included_indexes`` are positions (into this rank's selection) of
        entries that made it into the global set; all others go back to the
        residual."""
        with torch.no_grad():
            residual = TopKCompressor.residuals[name]
            if isinstance(included_indexes, np.ndarray):
                included_indexes = torch.from_numpy(included_indexes)
            pos = torch.as_tensor(included_indexes, device=residual.device).long()
            values = TopKCompressor.values[name]
            values[pos] = 0.0
            residual.index_add_(0, TopKCompressor.indexes[name], values)

    @staticmethod
    def decompress(tensor, ctc, name=None):
        return tensor


class TopKCompressor2(TopKCompressor):
    name = "topk2"


class gTopKCompressor(TopKCompressor):  # noqa: N801 - public name of the reference
    name = "gtopk"


compressors = {
    "topk": TopKCompressor,
    "topk2": TopKCompressor2,
    "gtopk": gTopKCompressor,
    "none": NoneCompressor,
}
