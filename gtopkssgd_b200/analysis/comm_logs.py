"""Readers for communication measurement logs, the alpha-beta fit and the
prediction of all-reduce times from it.

Covers what the reference's figure scripts read by hand:

* ``read_nccl_tests_log``  -- the table that the nccl-tests binaries print
  (12 whitespace-separated columns per message size; column 0 is the size in
  bytes, column 4 the out-of-place time in microseconds);
  scripts/icdcs2019/communication.py:235-254.
* ``read_allreduce_log``   -- "<size> ... <time>" lines of the MPI all-reduce and
  point-to-point probes, grouped by size into mean and standard deviation;
  communication.py:256-282.  ``read_node_allreduce_log`` is the variant whose
  first column is "<nodes>,<size>" (scripts/icdcs2019/plot_sth.py:117-136).
* ``read_layer_log`` / ``read_compute_log`` -- per-layer "[id, size, compute,
  comm, merged comm]" records and "...,size,compute" CSV records
  (scripts/icdcs2019/utils.py:4-53).
* ``fit_alpha_beta``, ``predict_allreduce`` -- least-squares line through
  (size, time) and the ring all-reduce model evaluated at measured sizes
  (communication.py:285-309, 557-564).

Nothing here needs matplotlib.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import cost_models as cm

SIZE_MIN = 16 * 1024          # window of message sizes the papers' fits use (communication.py:233-234)
SIZE_MAX = 4 * 1024 * 1024


def _fields(line: str) -> List[str]:
    return line.split()


def read_nccl_tests_log(path: str, size_min: int = SIZE_MIN, size_max: int = SIZE_MAX) -> Tuple[List[int], List[float]]:
    """(sizes in bytes, out-of-place times in microseconds) of one nccl-tests run."""
    sizes, times = [], []
    with open(path) as fh:
        for line in fh:
            f = _fields(line)
            if len(f) != 12 or f[0].startswith("#"):
                continue
            try:
                size, t = int(f[0]), float(f[4])
            except ValueError:
                continue
            if size == 8 or not (size_min <= size <= size_max):
                continue
            sizes.append(size)
            times.append(t)
    return sizes, times


def _group(pairs: Sequence[Tuple[int, float]]) -> Tuple[List[int], List[float], List[float]]:
    by: Dict[int, List[float]] = {}
    for s, t in pairs:
        by.setdefault(s, []).append(t)
    sizes = sorted(by)
    return sizes, [float(np.mean(by[s])) for s in sizes], [float(np.std(by[s])) for s in sizes]


def read_allreduce_log(path: str, size_min: int = SIZE_MIN, size_max: int = SIZE_MAX):
    """(sizes, mean time per size, std per size); lines that start with '#' or '[' and
    short lines are comments."""
    rows = []
    with open(path) as fh:
        for line in fh:
            if line[:1] in ("#", "[") or len(line) < 10:
                continue
            f = _fields(line)
            try:
                size, t = int(f[0]), float(f[-1])
            except (ValueError, IndexError):
                continue
            if size_min <= size <= size_max:
                rows.append((size, t))
    return _group(rows)


def read_node_allreduce_log(path: str):
    """Lines "<nodes>,<size> ... <time>": returns (nodes, sizes, times) in file order."""
    nodes, sizes, times = 0, [], []
    with open(path) as fh:
        for line in fh:
            if line[:1] == "#" or len(line) < 10:
                continue
            f = _fields(line)
            try:
                n, s = f[0].split(",")[:2]
                nodes, size, t = int(n), int(s), float(f[-1])
            except (ValueError, IndexError):
                continue
            sizes.append(size)
            times.append(t)
    return nodes, sizes, times


def read_layer_log(path: str):
    """Per-layer records "... [id, size, compute, comm, merged]" (one learnable layer per line,
    in backward order).  Layers whose compute or communication time truncates to zero are left
    out.  Returns (sizes, comms, computes, merged_comms)."""
    sizes, comms, computes, merged = [], [], [], []
    with open(path) as fh:
        for line in fh:
            lo, hi = line.find("["), line.rfind("]")
            if lo < 0 or hi <= lo:
                continue
            try:
                v = [float(x) for x in line[lo + 1:hi].split(",")]
            except ValueError:
                continue
            if len(v) < 5 or int(v[2]) == 0 or int(v[3]) == 0:
                continue
            sizes.append(v[1])
            computes.append(v[2])
            comms.append(v[4])
            merged.append(v[4])
    return sizes, comms, computes, merged


def read_compute_log(path: str):
    """CSV records whose last two fields are (size, compute time); consecutive records with the
    same compute time belong to one layer and are merged.  Returns (raw sizes, compute times per
    layer, sizes per layer)."""
    sizes, comps = [], []
    with open(path) as fh:
        for line in fh:
            f = line.strip().split(",")
            if len(f) < 2:
                continue
            try:
                sizes.append(float(f[-2]))
                comps.append(float(f[-1]))
            except ValueError:
                continue
    layer_sizes, layer_comps = [], []
    prev = None
    for s, c in zip(sizes, comps):
        if prev is None or c != prev:
            layer_sizes.append(s)
            layer_comps.append(c)
        else:
            layer_sizes[-1] += s
        prev = c
    return sizes, layer_comps, layer_sizes


def fit_alpha_beta(sizes: Sequence[float], times: Sequence[float]) -> Tuple[float, float]:
    """Least-squares line time = alpha + beta * size."""
    x, y = np.asarray(sizes, dtype=np.float64), np.asarray(times, dtype=np.float64)
    a = np.vstack([x, np.ones_like(x)]).T
    beta, alpha = np.linalg.lstsq(a, y, rcond=None)[0]
    return float(alpha), float(beta)


def predict_allreduce(sizes: Sequence[float], nworkers: int, bandwidth_bytes: Optional[float] = None) -> List[float]:
    """The papers' ring all-reduce model (microseconds) at the given message sizes, which are counts
    of fp32 elements as in the logs it is compared with."""
    if bandwidth_bytes is None:
        return [cm.ring_allreduce_us(nworkers, float(m)) for m in sizes]
    return [cm.ring_allreduce_us(nworkers, float(m), bandwidth_bytes) for m in sizes]


def relative_error(measured: Sequence[float], predicted: Sequence[float]) -> float:
    m, p = np.asarray(measured, dtype=np.float64), np.asarray(predicted, dtype=np.float64)
    return float(np.mean(np.abs(p - m) / np.maximum(np.abs(m), 1e-30)))


def gradient_size_statistics(sizes: Sequence[float]) -> "OrderedDict[str, float]":
    """What the papers quote about a network's per-layer message sizes (plot_sth.py:146-166)."""
    a = np.asarray(sizes, dtype=np.float64)
    return OrderedDict(layers=int(a.size), total=float(a.sum()), largest=float(a.max()) if a.size else 0.0,
                       smallest=float(a.min()) if a.size else 0.0, median=float(np.median(a)) if a.size else 0.0,
                       below_1m_fraction=float((a < 1e6).mean()) if a.size else 0.0)
