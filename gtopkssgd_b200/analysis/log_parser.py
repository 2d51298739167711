"""Parsers for the trainer's log lines (the informal interface the reference's
plot scripts rely on: scripts/icdcs2019/plot_loss.py:49-126,
scripts/ijcai2019/plot_loss.py:89-142)."""
from __future__ import annotations

import datetime
import re
from dataclasses import dataclass, field
from typing import List, Optional

_TS = re.compile(r"^(\d{4}-\d\d-\d\d \d\d:\d\d:\d\d)")
_TRAIN = re.compile(r"Epoch (\d+), avg train acc: ([-\w.]+), lr: ([\d.eE+-]+), avg loss: ([-\w.]+)")
_VAL = re.compile(r"Epoch (\d+), lr: ([\d.eE+-]+), val loss: ([-\w.]+), val acc: ([-\w.]+)")
_SPEED = re.compile(r"Time per iteration including communication: ([\d.eE+-]+)\. Speed: ([\d.eE+-]+) images/s"
                    r"(?:, current density: ([\d.eE+-]+))?")
_NBATCH = re.compile(r"num_batches_per_epoch: (\d+)")
_PROFILE = re.compile(r"\[rank:(\d+)\](\S+)\[(\d+)\]: ([\d.eE+,-]+)$")


@dataclass
class TrainingLog:
    epochs: List[int] = field(default_factory=list)
    train_loss: List[float] = field(default_factory=list)
    train_acc: List[float] = field(default_factory=list)
    lrs: List[float] = field(default_factory=list)
    val_epochs: List[int] = field(default_factory=list)
    val_loss: List[float] = field(default_factory=list)
    val_acc: List[float] = field(default_factory=list)
    times_s: List[int] = field(default_factory=list)        # seconds since the first epoch line
    iter_time_s: List[float] = field(default_factory=list)
    speeds: List[float] = field(default_factory=list)        # per-worker images/s
    densities: List[float] = field(default_factory=list)
    num_batches_per_epoch: Optional[int] = None
    profiling: List[dict] = field(default_factory=list)      # 7-column communication profile rows


def _timestamp(line: str):
    m = _TS.match(line)
    return datetime.datetime.strptime(m.group(1), "%Y-%m-%d %H:%M:%S") if m else None


def parse_log(path: str, max_epochs: Optional[int] = None) -> TrainingLog:
    log = TrainingLog()
    t0 = None
    with open(path) as fh:
        for line in fh:
            line = line.rstrip("\n")
            m = _NBATCH.search(line)
            if m:
                log.num_batches_per_epoch = int(m.group(1))
            m = _TRAIN.search(line)
            if m:
                if max_epochs is not None and len(log.epochs) >= max_epochs:
                    continue
                ts = _timestamp(line)
                t0 = t0 or ts
                log.epochs.append(int(m.group(1)))
                log.train_acc.append(float(m.group(2)))
                log.lrs.append(float(m.group(3)))
                log.train_loss.append(float(m.group(4)))
                if ts is not None and t0 is not None:
                    delta = ts - t0
                    log.times_s.append(delta.days * 86400 + delta.seconds)
                continue
            m = _VAL.search(line)
            if m:
                log.val_epochs.append(int(m.group(1)))
                log.val_loss.append(float(m.group(3)))
                log.val_acc.append(float(m.group(4)))
                continue
            m = _SPEED.search(line)
            if m:
                log.iter_time_s.append(float(m.group(1)))
                log.speeds.append(float(m.group(2)))
                if m.group(3):
                    log.densities.append(float(m.group(3)))
                continue
            m = _PROFILE.search(line)
            if m:
                cols = [float(x) for x in m.group(4).split(",")]
                if len(cols) == 7:
                    names = ("backward", "merge", "compression", "allreduce", "demerge", "d2h", "h2d")
                    row = dict(zip(names, cols))
                    row.update(rank=int(m.group(1)), name=m.group(2), size=int(m.group(3)))
                    log.profiling.append(row)
    return log


def mean_speed(log: TrainingLog, skip: int = 1) -> Optional[float]:
    vals = log.speeds[skip:] or log.speeds
    return sum(vals) / len(vals) if vals else None


def read_norm_from_log(path: str):
    """(means, stds) of the "gtopk-dense norm mean: m, std: s" lines that the error-norm diagnostic
    logs once per epoch (scripts/icdcs2019/plot_loss.py:128-141)."""
    means, stds = [], []
    pat = re.compile(r"gtopk-dense norm mean: ([-\w.+]+), std: ([-\w.+]+)")
    with open(path) as fh:
        for line in fh:
            m = pat.search(line)
            if m:
                means.append(float(m.group(1)))
                stds.append(float(m.group(2)))
    return means, stds


def value_histogram(values, bins: int = 100) -> dict:
    """Summary that the papers' ``plot_hist`` prints next to its histogram
    (scripts/icdcs2019/utils.py:55-69): mean, std, how many values are <= 0, and the normalised
    histogram itself."""
    import numpy as np
    flat = np.asarray(values, dtype=np.float64).ravel()
    density, edges = np.histogram(flat, bins=bins, density=True) if flat.size else (np.zeros(bins), np.zeros(bins + 1))
    return {"mean": float(flat.mean()) if flat.size else 0.0, "std": float(flat.std()) if flat.size else 0.0,
            "non_positive": int((flat <= 0).sum()), "total": int(flat.size), "density": density, "edges": edges}
