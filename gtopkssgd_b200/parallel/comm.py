"""Process-group plumbing: one process per GPU over ``torch.distributed``.

NCCL (over NVLink/NVSwitch) when CUDA is present, gloo on CPU.  The reference
takes rank and size from ``MPI.COMM_WORLD`` (distributed_optimizer.py:207-211)
and broadcasts weights / epoch / iteration with Horovod and mpi4py
(gtopk_trainer.py:39-40,51); the helpers here give the same services on the
process group.  A single process without any launcher is a world of size 1.
"""
from __future__ import annotations

import datetime
import os
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

_cpu_group = None
_hosts: list = []  # host name of every rank of the group formed by init()


def env_rank() -> int:
    return int(os.environ.get("RANK", "0"))


def env_world_size() -> int:
    return int(os.environ.get("WORLD_SIZE", "1"))


def env_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))


def init(backend: Optional[str] = None, timeout_s: float = 1800.0, device: Optional[torch.device] = None) -> None:
    """Join the process group described by RANK / WORLD_SIZE / MASTER_* (the
    torchrun contract).  Does nothing for a single process or when the group
    already exists."""
    global _cpu_group, _hosts
    if env_world_size() <= 1 or dist.is_initialized():
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    kwargs: Dict[str, Any] = {}
    if backend == "nccl":
        dev = device or torch.device("cuda", env_local_rank() % max(torch.cuda.device_count(), 1))
        torch.cuda.set_device(dev)
        kwargs["device_id"] = dev
    dist.init_process_group(backend=backend, rank=env_rank(), world_size=env_world_size(),
                            timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    if backend == "nccl":
        _cpu_group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
    import socket
    _hosts = [None] * env_world_size()
    dist.all_gather_object(_hosts, socket.gethostname(), group=_cpu_group)


def cpu_group():
    """A gloo group for host-side object exchange (None = the default group)."""
    return _cpu_group


_generation = 0


def reform(survivors, timeout_s: float = 120.0):
    """Leave the current process group and form a new one of the surviving
    ranks (``survivors``: old rank numbers, the same list on every survivor).
    Called between two iterations, with no collective in flight and after the
    departing ranks have stopped taking part.  The new rank 0 (the lowest
    surviving old rank) hosts the new rendezvous store on MASTER_PORT + 17 +
    generation.  Returns (new_rank, new_world)."""
    global _cpu_group, _transport, _generation
    survivors = sorted(int(r) for r in survivors)
    old_rank = rank()
    if old_rank not in survivors:
        raise ValueError("rank %d is not among the survivors %s" % (old_rank, survivors))
    backend = dist.get_backend()
    new_rank, new_world = survivors.index(old_rank), len(survivors)
    master = os.environ.get("MASTER_ADDR", "127.0.0.1")
    if _hosts and len(set(_hosts)) > 1:
        master = _hosts[survivors[0]]
    _generation += 1
    port = int(os.environ.get("MASTER_PORT", "29500")) + 17 + _generation
    dist.destroy_process_group()
    _cpu_group, _transport = None, None
    if _hosts:
        _hosts[:] = [_hosts[r] for r in survivors]
    os.environ["RANK"], os.environ["WORLD_SIZE"] = str(new_rank), str(new_world)
    if new_world == 1:
        return 0, 1
    store = dist.TCPStore(master, port, new_world, is_master=(new_rank == 0),
                          timeout=datetime.timedelta(seconds=timeout_s))
    kwargs: Dict[str, Any] = {}
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group(backend=backend, store=store, rank=new_rank, world_size=new_world,
                            timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    if backend == "nccl":
        _cpu_group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
    return new_rank, new_world


def choose_transport(requested: str, hosts, peer_ok) -> str:
    """'p2p' or 'staged' for a CUDA world.  ``hosts``: host name of every rank;
    ``peer_ok``: per rank, whether it can map every other rank's GPU.  'auto'
    takes p2p only when one host holds all ranks and every rank has peer
    access; an explicit 'p2p' that cannot work is an error."""
    possible = len(set(hosts)) == 1 and all(peer_ok)
    if requested == "staged":
        return "staged"
    if requested == "p2p":
        if not possible:
            raise RuntimeError("GTOPK_TRANSPORT=p2p needs all ranks on one host with GPU peer access "
                               "(hosts: %s, peer access: %s)" % (sorted(set(hosts)), list(peer_ok)))
        return "p2p"
    if requested != "auto":
        raise ValueError("GTOPK_TRANSPORT must be auto, p2p or staged (got %r)" % requested)
    return "p2p" if possible else "staged"


_transport = None


def sparse_transport() -> str:
    """The transport of the sparse exchange for this CUDA world (decided once,
    collectively: every rank gets the same answer)."""
    global _transport
    if _transport is not None:
        return _transport
    import socket
    from .. import settings
    world = size()
    if world == 1:
        return "p2p"
    me = torch.cuda.current_device()
    mine = (socket.gethostname(), me)
    everyone = [None] * world
    dist.all_gather_object(everyone, mine, group=cpu_group())
    hosts = [h for h, _ in everyone]
    ok = True
    if len(set(hosts)) == 1:
        for _, other in everyone:
            if other != me and not torch.cuda.can_device_access_peer(me, other):
                ok = False
    oks = [None] * world
    dist.all_gather_object(oks, ok, group=cpu_group())
    _transport = choose_transport(settings.TRANSPORT, hosts, oks)
    return _transport


def shutdown() -> None:
    global _cpu_group, _transport
    if dist.is_initialized():
        dist.destroy_process_group()
    _cpu_group = None
    _transport = None


def rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def size() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def barrier() -> None:
    if dist.is_initialized():
        dist.barrier(group=_cpu_group) if _cpu_group is not None else dist.barrier()


def broadcast_object(obj: Any, root: int = 0) -> Any:
    """mpi4py-style ``comm.bcast`` of a small Python object."""
    if not dist.is_initialized():
        return obj
    box = [obj]
    dist.broadcast_object_list(box, src=root, group=_cpu_group)
    return box[0]


def broadcast_parameters(state: Dict[str, torch.Tensor], root_rank: int = 0) -> None:
    """In-place broadcast of every tensor of a ``state_dict`` (weights and BN
    buffers) from ``root_rank``; the equivalent of hvd.broadcast_parameters."""
    if not dist.is_initialized():
        return
    for _, t in sorted(state.items()):
        if not torch.is_tensor(t):
            continue
        if t.is_floating_point() or t.dtype in (torch.int64, torch.int32, torch.uint8, torch.bool):
            buf = t if t.is_contiguous() else t.contiguous()
            dist.broadcast(buf, src=root_rank)
            if buf is not t:
                t.copy_(buf)


def allreduce_max_float(value: float, device: Optional[torch.device] = None) -> float:
    if not dist.is_initialized():
        return value
    dev = device or (torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl"
                     else torch.device("cpu"))
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
