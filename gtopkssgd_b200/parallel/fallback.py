"""Sparse all-reduce algorithms over ``torch.distributed`` point-to-point and
collective calls, on host tensors.

This is the path for CPU/gloo worlds (plumbing tests, machines without
NVLink) and the multi-process statement of the oracle: the message pattern is
the reference's (allreducer.py:29-64, 71-163) -- recursive-doubling send/recv
rounds, then a broadcast from rank 0 -- but the wire format is int64 indices +
fp32 values, there is no per-round barrier, and a shared index appears once in
a merged set.  Every blocking call takes a timeout so that a missing peer
raises ``PeerTimeout`` instead of hanging.
"""
from __future__ import annotations

import datetime
from typing import Tuple

import torch
import torch.distributed as dist

from ..ops import oracle


class PeerTimeout(RuntimeError):
    """A peer did not answer within the limit (or left the group)."""


def _wait(start, what: str, timeout_s: float) -> None:
    """Start a point-to-point operation (``start()`` returns the work handle)
    and wait for it with a limit.  gloo reports both an expired limit and a
    peer that closed its connection as RuntimeError."""
    try:
        ok = start().wait(datetime.timedelta(seconds=timeout_s))
    except RuntimeError as exc:
        raise PeerTimeout("%s: %s" % (what, str(exc).splitlines()[0])) from exc
    if ok is False:
        raise PeerTimeout(what + ": timed out")


def _send_pairs(idx: torch.Tensor, val: torch.Tensor, dst: int, group, timeout_s: float) -> None:
    head = torch.tensor([idx.numel()], dtype=torch.int64)
    for t, what in ((head, "send count"), (idx.contiguous(), "send indices"), (val.contiguous(), "send values")):
        _wait(lambda t=t: dist.isend(t, dst, group=group), "%s to rank %d" % (what, dst), timeout_s)


def _recv_pairs(src: int, group, timeout_s: float) -> Tuple[torch.Tensor, torch.Tensor]:
    head = torch.zeros(1, dtype=torch.int64)
    _wait(lambda: dist.irecv(head, src, group=group), "recv count from rank %d" % src, timeout_s)
    n = int(head.item())
    idx = torch.empty(n, dtype=torch.int64)
    val = torch.empty(n, dtype=torch.float32)
    _wait(lambda: dist.irecv(idx, src, group=group), "recv indices from rank %d" % src, timeout_s)
    _wait(lambda: dist.irecv(val, src, group=group), "recv values from rank %d" % src, timeout_s)
    return idx, val


def gtopk_allreduce(idx: torch.Tensor, val: torch.Tensor, k: int, group=None,
                    timeout_s: float = 60.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Global top-k set (indices, summed values) on every rank."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return idx, val
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    rounds = oracle.tree_rounds(world)
    cur = (idx.cpu().to(torch.int64), val.cpu().to(torch.float32))
    for r in range(rounds):
        bit = 1 << r
        low = rank & (2 * bit - 1)
        if low == bit:
            _send_pairs(cur[0], cur[1], dist.get_global_rank(group, rank - bit) if group else rank - bit, group,
                        timeout_s)
            break
        if low == 0:
            src = dist.get_global_rank(group, rank + bit) if group else rank + bit
            cur = oracle.merge_select(cur, _recv_pairs(src, group, timeout_s), k)
    # broadcast of the global set from rank 0
    root = dist.get_global_rank(group, 0) if group else 0
    head = torch.tensor([cur[0].numel() if rank == 0 else 0], dtype=torch.int64)
    _wait(lambda: dist.broadcast(head, root, group=group, async_op=True), "broadcast count", timeout_s)
    n = int(head.item())
    gi = cur[0].contiguous() if rank == 0 else torch.empty(n, dtype=torch.int64)
    gv = cur[1].contiguous() if rank == 0 else torch.empty(n, dtype=torch.float32)
    _wait(lambda: dist.broadcast(gi, root, group=group, async_op=True), "broadcast indices", timeout_s)
    _wait(lambda: dist.broadcast(gv, root, group=group, async_op=True), "broadcast values", timeout_s)
    return gi, gv


def topk_allgather(idx: torch.Tensor, val: torch.Tensor, group=None,
                   wire_dtype: torch.dtype = torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """All P selections concatenated in rank order: (P*k indices, P*k values).
    ``wire_dtype=torch.float16`` sends the values in half precision (two bytes per
    value on the wire; the reference registers such an MPI type, allreducer.py:19-24,
    and casts the gathered values to it, :52-53); every rank, the sender included,
    then sees the same rounded values, returned as fp32."""
    idx = idx.cpu().to(torch.int64).contiguous()
    val = val.cpu().to(torch.float32).to(wire_dtype).contiguous()
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return idx, val.to(torch.float32)
    world = dist.get_world_size(group)
    all_i = [torch.empty_like(idx) for _ in range(world)]
    all_v = [torch.empty_like(val) for _ in range(world)]
    dist.all_gather(all_i, idx, group=group)
    dist.all_gather(all_v, val, group=group)
    return torch.cat(all_i), torch.cat(all_v).to(torch.float32)


def dense_allreduce(tensor: torch.Tensor, group=None) -> torch.Tensor:
    """Sum over all ranks (in place); NCCL for CUDA tensors, gloo for CPU."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=group)
    return tensor
