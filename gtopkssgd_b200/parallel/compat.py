"""Function-level API of the reference's allreducer.py on top of this
framework: ``gtopk_sparse_allreduce``, ``topk_sparse_allreduce``,
``dense_allreduce`` with the reference's argument lists and return values
(allreducer.py:29-64, 71-163, 166-171), numpy in / numpy out.

``comm`` is a ``torch.distributed`` process group or ``None`` for the default
group (the reference passes an mpi4py communicator).  These functions work on
host arrays through the gloo fallback; the training path uses the device
kernels instead.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from .. import settings
from ..settings import logger
from ..utils.misc import force_insert_item, topk  # noqa: F401
from . import fallback

THRESHOLD = settings.THRESHOLD
# value types that may travel (the reference's MPI_TYPES, allreducer.py:19-24: fp32, and a
# two-byte type registered for fp16)
WIRE_TYPES = {np.float32: torch.float32, np.float16: torch.float16, np.dtype("float32"): torch.float32,
              np.dtype("float16"): torch.float16}


def _as_numpy(x):
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().numpy()
    return np.asarray(x)


def gtopk_sparse_allreduce(comm, sparse_tensor, storage=None, indexes=None, dtype=np.float32):
    """Returns ``(values, indexes, included_indexes)``: the global top-k values
    and indices, and the positions (into this rank's input selection) of the
    entries whose index is in the global set."""
    tensor = _as_numpy(sparse_tensor)
    if indexes is None:
        k = max(int(tensor.size * 0.001), 1)
        indexes, values = topk(tensor, k)
    else:
        indexes = _as_numpy(indexes)
        values = tensor
    k = len(indexes)
    gi, gv = fallback.gtopk_allreduce(torch.from_numpy(indexes.astype(np.int64)),
                                      torch.from_numpy(values.astype(np.float32)), k, group=comm)
    gi, gv = gi.numpy(), gv.numpy()
    included = np.nonzero(np.isin(indexes, gi))[0]
    return gv.astype(dtype), gi.astype(np.uint32), included


def topk_sparse_allreduce(comm, sparse_tensor, storage, indexes=None, dtype=np.float32):
    """Returns ``(values_1d, indexes_1d, None)``: all P selections concatenated
    in rank order."""
    tensor = _as_numpy(sparse_tensor)
    if indexes is None:
        k = max(int(tensor.size * 0.01), 1)
        indexes, values = topk(tensor, k)
    else:
        indexes = _as_numpy(indexes)
        values = tensor
    ai, av = fallback.topk_allgather(torch.from_numpy(indexes.astype(np.int64)),
                                     torch.from_numpy(values.astype(np.float32)), group=comm,
                                     wire_dtype=WIRE_TYPES.get(dtype, torch.float32))
    return av.numpy().astype(dtype), ai.numpy().astype(np.uint32), None


def dense_allreduce(comm, tensor):
    """Element-wise sum over all ranks of a host array."""
    t = torch.from_numpy(np.array(_as_numpy(tensor), copy=True))
    if dist.is_initialized():
        dist.all_reduce(t, group=comm)
    return t.numpy()


def benchmark_gtopk_sparse_allreduce(size: int = 25 * 1024 * 1024, ratio: float = 0.001, iteration: int = 10):
    """The reference's built-in micro-benchmark (allreducer.py:603-631; its own
    version unpacks the 3-tuple wrongly and raises): 25 Mi random fp32 values,
    density 0.001, one warm-up and ten timed calls.  Uses the device kernels
    when CUDA is present, the host fallback otherwise."""
    from ..bench_allreduce import run_config
    row = run_config(size, ratio, iters=iteration, warmup=1, with_dense=False, with_rehost=False)
    if row is not None:
        logger.info("average time: %f", row["ours_ms"] / 1e3)
    return row
