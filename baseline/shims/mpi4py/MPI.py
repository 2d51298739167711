"""``mpi4py.MPI`` on top of a ``torch.distributed`` gloo group.

The reference talks MPI on host numpy buffers
(``allreducer.py:62-63,118,139,143,153,169-170``, ``gtopk_trainer.py:13-14,39-40``).
This module gives those calls the same meaning over gloo, a CPU transport:
upper-case methods move the bytes of a contiguous numpy buffer in place,
lower-case ``bcast`` moves a pickled object.  A buffer argument may be an array
or the list form ``[array, datatype]`` / ``[array, count, datatype]``; as in MPI
with an inferred count, the whole array travels.

The process group is created on first use from the environment that
``torchrun`` sets (``RANK``, ``WORLD_SIZE``, ``MASTER_ADDR``, ``MASTER_PORT``);
without it a single-rank group is made on 127.0.0.1.
"""
from __future__ import annotations

import datetime
import os
import threading

import numpy as np
import torch
import torch.distributed as dist

ERRORS_RETURN = "ERRORS_RETURN"
ERRORS_ARE_FATAL = "ERRORS_ARE_FATAL"
SUM, MAX, MIN = "SUM", "MAX", "MIN"
_OPS = {SUM: dist.ReduceOp.SUM, MAX: dist.ReduceOp.MAX, MIN: dist.ReduceOp.MIN}
ANY_SOURCE, ANY_TAG = -1, -1
_lock = threading.Lock()
_group = None


class Datatype:
    """Carries an element size; the shim moves whole buffers, so nothing else is needed."""

    def __init__(self, name, size):
        self.name, self.size = name, size

    def Create_contiguous(self, count):
        return Datatype("%s[%d]" % (self.name, count), self.size * count)

    def Commit(self):
        return self

    def Free(self):
        return None

    def Get_size(self):
        return self.size


BYTE = Datatype("BYTE", 1)
CHAR = Datatype("CHAR", 1)
INT = Datatype("INT", 4)
UNSIGNED = Datatype("UNSIGNED", 4)
LONG = Datatype("LONG", 8)
FLOAT = Datatype("FLOAT", 4)
DOUBLE = Datatype("DOUBLE", 8)
_typedict = {"b": BYTE, "i": INT, "I": UNSIGNED, "l": LONG, "f": FLOAT, "d": DOUBLE}


def ensure_process_group():
    """Default group = ``cpu:gloo`` (+ ``cuda:nccl`` when a GPU is there); returns the gloo group used here."""
    global _group
    with _lock:
        if _group is not None:
            return _group
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29533")
            rank = int(os.environ.get("RANK", "0"))
            world = int(os.environ.get("WORLD_SIZE", "1"))
            backend = "cpu:gloo,cuda:nccl" if torch.cuda.is_available() else "gloo"
            kw = {}
            if torch.cuda.is_available():
                kw["device_id"] = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")) % torch.cuda.device_count())
            dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                    timeout=datetime.timedelta(seconds=600), **kw)
        # a group of its own: the reference calls MPI from its communication thread while the main thread
        # may use the default group (weight broadcast), and gloo matches operations by order within a group
        _group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=600))
        return _group


def _array(buf):
    if isinstance(buf, (list, tuple)):
        buf = buf[0]
    if not isinstance(buf, np.ndarray):
        raise TypeError("buffer must be a numpy array, got %r" % type(buf))
    if not buf.flags["C_CONTIGUOUS"]:
        raise ValueError("buffer must be C-contiguous")
    return buf


def _bytes_view(arr):
    """A uint8 torch tensor sharing the array's memory (gloo moves any dtype as bytes)."""
    return torch.from_numpy(arr.reshape(-1).view(np.uint8))


class Comm:
    def __init__(self):
        self._errhandler = ERRORS_ARE_FATAL

    # --- identity
    @property
    def rank(self):
        ensure_process_group()
        return dist.get_rank()

    @property
    def size(self):
        ensure_process_group()
        return dist.get_world_size()

    def Get_rank(self):
        return self.rank

    def Get_size(self):
        return self.size

    def Set_errhandler(self, handler):
        self._errhandler = handler

    def Get_errhandler(self):
        return self._errhandler

    # --- point to point
    def Send(self, buf, dest, tag=0):
        g = ensure_process_group()
        dist.send(_bytes_view(_array(buf)), dst=dest, group=g, tag=tag)

    def Recv(self, buf, source=ANY_SOURCE, tag=0, status=None):
        g = ensure_process_group()
        dist.recv(_bytes_view(_array(buf)), src=None if source == ANY_SOURCE else source, group=g, tag=max(tag, 0))

    # --- collectives on buffers
    def Barrier(self):
        dist.barrier(group=ensure_process_group())

    def Bcast(self, buf, root=0):
        g = ensure_process_group()
        dist.broadcast(_bytes_view(_array(buf)), src=root, group=g)

    def Allgather(self, sendbuf, recvbuf):
        g = ensure_process_group()
        s, r = _array(sendbuf), _array(recvbuf)
        sb, rb = _bytes_view(s), _bytes_view(r)
        n = self.size
        if rb.numel() != n * sb.numel():
            raise ValueError("Allgather: receive buffer has %d bytes, expected %d" % (rb.numel(), n * sb.numel()))
        dist.all_gather(list(rb.chunk(n)), sb, group=g)

    def Allreduce(self, sendbuf, recvbuf, op=SUM):
        g = ensure_process_group()
        s, r = _array(sendbuf), _array(recvbuf)
        if s.dtype != r.dtype or s.size != r.size:
            raise ValueError("Allreduce: buffers differ in type or size")
        np.copyto(r.reshape(-1), s.reshape(-1))
        dist.all_reduce(torch.from_numpy(r.reshape(-1)), op=_OPS[op], group=g)

    # --- pickled objects
    def bcast(self, obj=None, root=0):
        g = ensure_process_group()
        box = [obj]
        dist.broadcast_object_list(box, src=root, group=g)
        return box[0]

    def barrier(self):
        self.Barrier()


COMM_WORLD = Comm()


def Is_initialized():
    return dist.is_initialized()


def Finalize():
    if dist.is_initialized():
        dist.destroy_process_group()
