"""Start N local ranks of a Python function (tests, small benchmarks).

Each child gets the torchrun environment (RANK, LOCAL_RANK, WORLD_SIZE,
MASTER_ADDR=127.0.0.1, a free MASTER_PORT) and runs ``fn(rank, world, *args)``;
the return values come back in rank order.  Children that are still alive when
the time limit expires are terminated by their own process handles.
"""
from __future__ import annotations

import io
import os
import socket
import traceback
from typing import Any, Callable, List, Sequence

import torch
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank: int, world: int, port: int, fn: Callable, args: Sequence[Any], queue, extra_env: dict) -> None:
    os.environ.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    os.environ.update(extra_env)
    try:
        buf = io.BytesIO()
        torch.save(fn(rank, world, *args), buf)  # by value: the child may exit before the parent reads
        queue.put((rank, "ok", buf.getvalue()))
    except BaseException as exc:  # report, then exit non-zero
        queue.put((rank, "error", "%s\n%s" % (exc, traceback.format_exc())))
        raise


class RankFailure(RuntimeError):
    pass


def spawn_ranks(fn: Callable, world: int, args: Sequence[Any] = (), timeout_s: float = 300.0,
                env: dict | None = None, allow_failures: bool = False) -> List[Any]:
    """Run ``fn(rank, world, *args)`` in ``world`` fresh processes."""
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, tuple(args), queue, dict(env or {})))
             for r in range(world)]
    for p in procs:
        p.start()
    results: List[Any] = [None] * world
    status = ["missing"] * world
    import queue as _q
    import time
    deadline = time.time() + timeout_s
    got = 0
    while got < world and time.time() < deadline:
        try:
            rank, st, val = queue.get(timeout=0.5)
        except _q.Empty:
            if all(not p.is_alive() for p in procs) and queue.empty():
                break
            continue
        if st == "ok":
            val = torch.load(io.BytesIO(val), weights_only=False)
        results[rank], status[rank] = val, st
        got += 1
    for p in procs:
        p.join(timeout=max(0.1, deadline - time.time()))
    for p in procs:
        if p.is_alive():
            p.terminate()
            p.join(timeout=5)
    if not allow_failures and any(s != "ok" for s in status):
        raise RankFailure("ranks failed: %s" % [(r, s, results[r] if s == "error" else None)
                                                for r, s in enumerate(status) if s != "ok"])
    return results if not allow_failures else list(zip(status, results))
