"""Minimal dense data-parallel wrapper: flatten all gradients, one
``all_reduce``, unflatten, divide by the world size (the hand-rolled module in
the reference's audio_data/distributed.py:17-65, which none of its entry points
uses).  Kept as a dependency-free baseline for debugging; the training drivers
use DistributedOptimizer instead."""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch._utils import _flatten_dense_tensors, _unflatten_dense_tensors


def broadcast_module(module: torch.nn.Module, src: int = 0) -> None:
    if dist.is_initialized():
        for t in module.state_dict().values():
            if torch.is_tensor(t):
                dist.broadcast(t, src)


def allreduce_gradients(module: torch.nn.Module) -> None:
    """Average ``p.grad`` over all ranks with one flat all-reduce per dtype."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return
    buckets = {}
    for p in module.parameters():
        if p.requires_grad and p.grad is not None:
            buckets.setdefault(p.grad.dtype, []).append(p.grad)
    world = dist.get_world_size()
    for grads in buckets.values():
        flat = _flatten_dense_tensors(grads)
        dist.all_reduce(flat)
        flat /= world
        for g, synced in zip(grads, _unflatten_dense_tensors(flat, grads)):
            g.copy_(synced)


class DistributedDataParallel(torch.nn.Module):
    def __init__(self, module: torch.nn.Module):
        super().__init__()
        self.module = module
        broadcast_module(module)

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def sync_gradients(self):
        allreduce_gradients(self.module)
