"""K3 wrapper: fused sparse scatter + averaging + weight decay + momentum SGD.

``sgd_dense`` applies the part of the update that does not depend on the
sparse exchange (weight decay, momentum decay, and the dense gradient in dense
mode); ``sgd_sparse`` applies the k global pairs on top.  Together they equal
the reference's scatter + ``/P`` + per-parameter SGD loop
(allreducer.py:458-475, distributed_optimizer.py:105-143).  CPU tensors go
through the PyTorch oracle.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import lib as _lib
from . import oracle
from .select import _ptr, current_stream_handle, pairs_to_tensors


@dataclass
class SgdHyper:
    lr: float
    momentum: float = 0.0
    dampening: float = 0.0
    weight_decay: float = 0.0
    nesterov: bool = False


def sgd_dense(p: torch.Tensor, buf: Optional[torch.Tensor], h: SgdHyper, first_step: bool,
              g: Optional[torch.Tensor] = None, scale: float = 1.0, coef: Optional[torch.Tensor] = None,
              lr_dev: Optional[torch.Tensor] = None) -> None:
    """Dense part of the step over a flat parameter buffer.  With ``g`` given
    (dense mode) the gradient is ``coef * scale * g``."""
    d = p.numel()
    if p.device.type != "cuda":
        if g is None and h.momentum == 0 and h.weight_decay == 0:
            return
        c = scale * (float(coef) if coef is not None else 1.0)
        grad = g * c if g is not None else torch.zeros_like(p)
        oracle.sgd_step(p, buf, grad, h.lr, h.momentum, h.dampening, h.weight_decay, h.nesterov, first_step)
        return
    L = _lib.lib()
    code = L.gtk_k3_dense(p.data_ptr(), _ptr(buf), _ptr(g), _ptr(coef), C.c_float(scale), d, C.c_float(h.lr),
                          _ptr(lr_dev), C.c_float(h.momentum), C.c_float(h.dampening), C.c_float(h.weight_decay),
                          int(h.nesterov), int(first_step), current_stream_handle(p.device))
    _lib.check(code, "gtk_k3_dense")


def sgd_sparse(p: torch.Tensor, buf: Optional[torch.Tensor], pairs: torch.Tensor, counts: torch.Tensor,
               nseg: int, seg_stride: int, h: SgdHyper, first_step: bool, scale: float,
               coef: Optional[torch.Tensor] = None, use_atomics: bool = False,
               bad_index_count: Optional[torch.Tensor] = None, lr_dev: Optional[torch.Tensor] = None,
               parity_word: Optional[torch.Tensor] = None, parity_stride: int = 0) -> None:
    """Sparse part of the step: for every pair (j, v) of every segment add
    ``coef * scale * v`` as gradient of element j.  ``counts`` is a device
    tensor with the live length of each segment.  ``lr_dev`` (a device scalar)
    overrides ``h.lr``; ``parity_word`` selects the half of a two-parity buffer
    on the device: base = pairs + ((word - 1) & 1) * parity_stride."""
    d = p.numel()
    if p.device.type != "cuda":
        if parity_word is not None:
            pairs = pairs[((int(parity_word) - 1) & 1) * parity_stride:]
        c = scale * (float(coef) if coef is not None else 1.0)
        f = 1.0 if first_step else 1.0 - h.dampening
        for s in range(nseg):
            n = int(counts[s])
            idx, val = pairs_to_tensors(pairs[s * seg_stride:(s + 1) * seg_stride], n)
            sv = val * c
            step = sv
            if h.momentum != 0 and buf is not None:
                sb = f * sv
                buf.index_add_(0, idx, sb)
                step = sv + h.momentum * sb if h.nesterov else sb
            p.index_add_(0, idx, step, alpha=-h.lr)
        return
    L = _lib.lib()
    if bad_index_count is None:
        bad_index_count = _scratch_word(p.device)
    code = L.gtk_k3_sparse(p.data_ptr(), _ptr(buf), pairs.data_ptr(), counts.data_ptr(), nseg, seg_stride,
                           _ptr(coef), C.c_float(scale), d, C.c_float(h.lr), _ptr(lr_dev), C.c_float(h.momentum),
                           C.c_float(h.dampening), C.c_float(h.weight_decay), int(h.nesterov), int(first_step),
                           int(use_atomics), bad_index_count.data_ptr(), _ptr(parity_word), int(parity_stride),
                           current_stream_handle(p.device))
    _lib.check(code, "gtk_k3_sparse")


def scatter_dense(g: torch.Tensor, pairs: torch.Tensor, counts: torch.Tensor, nseg: int, seg_stride: int,
                  scale: float, use_atomics: bool = False, parity_word: Optional[torch.Tensor] = None,
                  parity_stride: int = 0) -> None:
    """g <- 0, then g[j] (+)= scale * v for every pair: the dense averaged
    gradient, for callers that want to inspect ``p.grad``."""
    if g.device.type != "cuda":
        if parity_word is not None:
            pairs = pairs[((int(parity_word) - 1) & 1) * parity_stride:]
        g.zero_()
        for s in range(nseg):
            n = int(counts[s])
            idx, val = pairs_to_tensors(pairs[s * seg_stride:(s + 1) * seg_stride], n)
            g.index_add_(0, idx, val * scale)
        return
    L = _lib.lib()
    code = L.gtk_k3_scatter_dense(g.data_ptr(), pairs.data_ptr(), counts.data_ptr(), nseg, seg_stride,
                                  C.c_float(scale), g.numel(), int(use_atomics), _ptr(parity_word), int(parity_stride),
                                  current_stream_handle(g.device))
    _lib.check(code, "gtk_k3_scatter_dense")


_scratch = {}


def _scratch_word(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index)
    if key not in _scratch:
        _scratch[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _scratch[key]


def momentum_correct(v: torch.Tensor, g: torch.Tensor, momentum: float) -> None:
    """v = momentum * v + g; g = v, in place over flat buffers (one launch).
    The reference applies this per parameter in its gradient hook when
    ``momentum_correction`` is set (distributed_optimizer.py:81-88)."""
    if g.device.type != "cuda":
        v.mul_(momentum).add_(g)
        g.copy_(v)
        return
    L = _lib.lib()
    code = L.gtk_k3_momentum_correct(v.data_ptr(), g.data_ptr(), C.c_float(momentum), g.numel(),
                                     current_stream_handle(g.device))
    _lib.check(code, "gtk_k3_momentum_correct")
