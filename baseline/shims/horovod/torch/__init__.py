"""``horovod.torch`` on top of ``torch.distributed`` (NCCL for CUDA tensors).

Covers what the reference calls (``horovod_trainer.py:29-35,93``,
``gtopk_trainer.py:51,157``): ``init``, ``rank``, ``size``, ``local_rank``,
``broadcast``, ``broadcast_parameters``, ``allreduce`` and
``DistributedOptimizer``.  The optimizer wrapper follows Horovod's design: a
hook on every parameter's gradient accumulator queues the gradient; queued
gradients are packed into a fusion buffer (``HOROVOD_FUSION_THRESHOLD`` bytes,
64 MiB by default, as in Horovod), all-reduced with NCCL on a side stream while
backward continues, averaged and copied back; ``synchronize()`` flushes the
last buffer and makes the compute stream wait; ``step()`` = ``synchronize()`` +
the wrapped optimizer's ``step()``.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from mpi4py import MPI as _mpi  # the stand-in: owns the process group


def init():
    _mpi.ensure_process_group()


def shutdown():
    if dist.is_initialized():
        dist.destroy_process_group()


def rank():
    init()
    return dist.get_rank()


def size():
    init()
    return dist.get_world_size()


def local_rank():
    return int(os.environ.get("LOCAL_RANK", "0"))


def local_size():
    return int(os.environ.get("LOCAL_WORLD_SIZE", "1"))


def _group_for(tensor):
    return None if tensor.is_cuda else _mpi.ensure_process_group()


def broadcast_(tensor, root_rank, name=None):
    init()
    dist.broadcast(tensor, src=root_rank, group=_group_for(tensor))
    return tensor


def broadcast(tensor, root_rank, name=None):
    return broadcast_(tensor.clone(), root_rank, name)


def broadcast_parameters(params, root_rank):
    """In-place broadcast of a ``state_dict()`` or of ``named_parameters()``, in name order."""
    if isinstance(params, dict):
        items = sorted(params.items())
    else:
        items = sorted(list(params))
    for _, p in items:
        if torch.is_tensor(p):
            broadcast_(p.data if p.requires_grad else p, root_rank)


def allreduce_(tensor, average=True, name=None):
    init()
    dist.all_reduce(tensor, group=_group_for(tensor))
    if average:
        tensor.div_(size())
    return tensor


def allreduce(tensor, average=True, name=None):
    return allreduce_(tensor.clone(), average, name)


class _DistributedOptimizer(torch.optim.Optimizer):
    def __init__(self, params, named_parameters=None, compression=None, backward_passes_per_step=1):
        super(self.__class__, self).__init__(params)
        init()
        named_parameters = list(named_parameters) if named_parameters is not None else []
        self._parameter_names = {v: k for k, v in named_parameters}
        self._fusion_bytes = int(os.environ.get("HOROVOD_FUSION_THRESHOLD", 64 * 1024 * 1024))
        self._pending, self._pending_bytes, self._inflight = [], 0, []
        self._grad_accs = []
        self._comm_stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self._buffers = {}
        self._synchronized = False
        self.local = False
        if size() > 1:
            self._register_hooks()

    def _register_hooks(self):
        for group in self.param_groups:
            for p in group["params"]:
                if p.requires_grad:
                    acc = p.expand_as(p).grad_fn.next_functions[0][0]
                    acc.register_hook(self._make_hook(p))
                    self._grad_accs.append(acc)

    def _make_hook(self, p):
        def hook(*ignore):
            if self.local:
                return
            self._pending.append(p)
            self._pending_bytes += p.grad.numel() * p.grad.element_size()
            if self._pending_bytes >= self._fusion_bytes:
                self._flush()
        return hook

    def _flush(self):
        if not self._pending:
            return
        params, self._pending, self._pending_bytes = self._pending, [], 0
        grads = [p.grad for p in params]
        n = sum(g.numel() for g in grads)
        key = (grads[0].device, grads[0].dtype, len(self._inflight))
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            buf = self._buffers[key] = torch.empty(n, device=grads[0].device, dtype=grads[0].dtype)
        buf = buf[:n]
        views, off = [], 0
        for g in grads:
            views.append(buf[off:off + g.numel()].view_as(g))
            off += g.numel()
        torch._foreach_copy_(views, grads)          # pack (Horovod: memcpy into the fusion buffer)
        if self._comm_stream is not None and buf.is_cuda:
            self._comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._comm_stream):
                dist.all_reduce(buf)
                buf.div_(size())
        else:
            dist.all_reduce(buf, group=_group_for(buf))
            buf.div_(size())
        self._inflight.append((grads, views))

    def synchronize(self):
        self._flush()
        if self._inflight:
            if self._comm_stream is not None:
                torch.cuda.current_stream().wait_stream(self._comm_stream)
            for grads, views in self._inflight:
                torch._foreach_copy_(grads, views)  # unpack
            self._inflight = []
        self._synchronized = True

    def step(self, closure=None):
        if not self._synchronized and not self.local:
            self.synchronize()
        self._synchronized = False
        return super(self.__class__, self).step(closure)


def DistributedOptimizer(optimizer, named_parameters=None, compression=None, backward_passes_per_step=1):
    cls = type(optimizer.__class__.__name__, (optimizer.__class__,), dict(_DistributedOptimizer.__dict__))
    return cls(optimizer.param_groups, named_parameters, compression, backward_passes_per_step)
