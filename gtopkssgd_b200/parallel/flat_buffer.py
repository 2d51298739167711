"""Flat parameter / gradient / momentum / residual buffers with merged groups.

The reference copies every layer gradient into a merged buffer when its hook
fires and slices the reduced buffer back into per-layer tensors afterwards
(allreducer.py:235-322).  Here the copy never happens: at construction every
parameter's storage and every ``p.grad`` become permanent views into four flat
fp32 buffers, laid out group by group in backward order, so a merged group is
just a slice and the update kernels run over one contiguous range.

Grouping rule (allreducer.py:235-257): walk the parameters in reverse
registration order (the order in which backward produces their gradients) and
close a group once it holds at least ``threshold`` elements.  The default
threshold of 640 Mi elements puts any supported model into one group.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Sequence, Tuple

import torch

ALIGN = 64      # elements; every group starts on a 256-byte boundary
SLOT_ALIGN = 4  # elements; every parameter starts on a 16-byte boundary.  Library kernels (cuDNN, cuBLAS)
                # pick their vectorised and TMA-fed variants only for 16-byte aligned operands, and a
                # channels-last convolution faulted with "misaligned address" on an 8-byte aligned weight view
                # (VGG-16, whose 10-element classifier bias shifted every later parameter).


@dataclass
class ParamSlot:
    name: str
    param: torch.nn.Parameter
    group: int
    offset: int      # element offset inside the flat buffers
    numel: int
    channels_last: bool = False


@dataclass
class MergedGroup:
    index: int
    names: List[str]
    start: int       # element offset of the group inside the flat buffers
    numel: int       # span of the group in the flat buffers (parameters + alignment gaps, which stay zero)
    offsets: List[int] = field(default_factory=list)   # per-parameter offsets inside the group
    key: str = ""
    param_numel: int = 0   # elements that belong to parameters: the d that the density applies to


def generate_groups(names_in_order: Sequence[str], sizes: Dict[str, int], threshold: int) -> Tuple[List[List[str]], Dict[str, int]]:
    """Group parameter names by the threshold rule, last layer first."""
    groups: List[List[str]] = []
    key_group: Dict[str, int] = {}
    cur: List[str] = []
    acc = 0
    idx = 0
    for name in reversed(list(names_in_order)):
        acc += sizes[name]
        key_group[name] = idx
        cur.append(name)
        if acc >= threshold:
            groups.append(cur)
            cur, acc = [], 0
            idx += 1
    if cur:
        groups.append(cur)
    return groups, key_group


class FlatBuffers:
    """Owns the flat buffers and re-points the model's parameters into them."""

    def __init__(self, named_parameters: Iterable[Tuple[str, torch.nn.Parameter]], threshold: int,
                 with_residual: bool = True):
        named = [(n, p) for n, p in named_parameters if p.requires_grad]
        if not named:
            raise ValueError("no trainable parameters")
        dev, dtype = named[0][1].device, named[0][1].dtype
        if dtype != torch.float32:
            raise ValueError("flat buffers are fp32; got %s" % dtype)
        for n, p in named:
            if p.device != dev or p.dtype != dtype:
                raise ValueError("parameter %s is on %s/%s, expected %s/%s" % (n, p.device, p.dtype, dev, dtype))
        self.device = dev
        sizes = {n: p.numel() for n, p in named}
        by_name = dict(named)
        names = [n for n, _ in named]
        group_names, self.key_group = generate_groups(names, sizes, threshold)
        self.groups: List[MergedGroup] = []
        self.slots: Dict[str, ParamSlot] = {}
        cursor = 0
        for gi, gnames in enumerate(group_names):
            start = cursor
            offs = []
            end = cursor
            for n in gnames:
                offs.append(cursor - start)
                self.slots[n] = ParamSlot(n, by_name[n], gi, cursor, sizes[n])
                end = cursor + sizes[n]
                cursor = (end + SLOT_ALIGN - 1) // SLOT_ALIGN * SLOT_ALIGN
            self.groups.append(MergedGroup(gi, list(gnames), start, end - start, offs, ":".join(gnames),
                                           sum(sizes[n] for n in gnames)))
            cursor = (cursor + ALIGN - 1) // ALIGN * ALIGN
        self.total = cursor
        self.numel = sum(g.numel for g in self.groups)
        self.param_numel = sum(g.param_numel for g in self.groups)
        self.param = torch.zeros(self.total, dtype=dtype, device=dev)
        self.grad = torch.zeros(self.total, dtype=dtype, device=dev)
        self.momentum = torch.zeros(self.total, dtype=dtype, device=dev)
        self.residual = torch.zeros(self.total, dtype=dtype, device=dev) if with_residual else None
        with torch.no_grad():
            for slot in self.slots.values():
                p = slot.param
                slot.channels_last = (p.dim() == 4 and not p.is_contiguous()
                                      and p.is_contiguous(memory_format=torch.channels_last))
                view = self._view(self.param, slot)
                view.copy_(p.data)
                p.data = view
                p.grad = self._view(self.grad, slot)

    # -- views -----------------------------------------------------------------
    @staticmethod
    def _view(buf: torch.Tensor, slot: ParamSlot) -> torch.Tensor:
        """The parameter-shaped view of ``buf`` for this slot.  Channels-last
        4-D parameters keep their memory format (NHWC order inside the slot)."""
        flat = buf[slot.offset:slot.offset + slot.numel]
        shape = slot.param.shape
        if slot.channels_last:
            n, c, h, w = shape
            return flat.view(n, h, w, c).permute(0, 3, 1, 2)
        return flat.view(shape)

    def group_slice(self, buf: torch.Tensor, g: MergedGroup) -> torch.Tensor:
        return buf[g.start:g.start + g.numel]

    def grad_view(self, name: str) -> torch.Tensor:
        return self._view(self.grad, self.slots[name])

    def momentum_view(self, name: str) -> torch.Tensor:
        return self._view(self.momentum, self.slots[name])

    def residual_view(self, name: str) -> torch.Tensor:
        return self._view(self.residual, self.slots[name])

    def ensure_views(self) -> int:
        """Re-attach any parameter whose ``.data`` or ``.grad`` was replaced
        behind our back (``.cuda()``, ``zero_grad(set_to_none=True)``,
        ``flatten_parameters``).  Returns how many were repaired."""
        fixed = 0
        with torch.no_grad():
            for s in self.slots.values():
                p = s.param
                want = self._view(self.param, s)
                if p.data.data_ptr() != want.data_ptr():
                    want.copy_(p.data)
                    p.data = want
                    fixed += 1
                gwant = self._view(self.grad, s)
                if p.grad is None:
                    p.grad = gwant
                    fixed += 1
                elif p.grad.data_ptr() != gwant.data_ptr():
                    gwant.add_(p.grad)
                    p.grad = gwant
                    fixed += 1
        return fixed

    def zero_grad(self) -> None:
        self.grad.zero_()
