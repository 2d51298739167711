"""Figures of the papers, rendered head-less (Agg backend) to image files.
matplotlib is optional: without it every function raises a clear ImportError
and the numeric helpers in cost_models / log_parser remain usable.
(reference: scripts/icdcs2019/communication.py, plot_loss.py, plot_sth.py,
scripts/ijcai2019/plot_loss.py -- those need a display through TkAgg.)"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

from . import cost_models as cm
from .log_parser import parse_log


def _plt():
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        return plt
    except ImportError as exc:
        raise ImportError("plotting needs matplotlib, which is not installed") from exc


def plot_scaling_efficiency(model: str, out: str) -> str:
    plt = _plt()
    t = cm.PUBLISHED_THROUGHPUT[model]
    fig, ax = plt.subplots(figsize=(5, 4))
    for key, label, style in (("dense", "Dense S-SGD", "b-o"), ("topk", "Top-$k$ S-SGD", "r-x"),
                              ("gtopk", "gTop-$k$ S-SGD", "g-^")):
        ax.plot(cm.WORKERS[1:], cm.scaling_efficiency(t[key]), style, label=label)
    ax.set_xlabel("# of workers (GPU)")
    ax.set_ylabel("Scaling efficiency (Percentage)")
    ax.set_xticks(cm.WORKERS[1:])
    ax.set_title(model)
    ax.legend(loc=3)
    fig.savefig(out)
    plt.close(fig)
    return out


def plot_allreduce_models(out: str, m: int = 25 * 1024 * 1024, rho: float = 0.001,
                          workers: Sequence[int] = (4, 8, 16, 32, 64, 128)) -> str:
    plt = _plt()
    fig, ax = plt.subplots(figsize=(5, 3.8))
    ax.plot(workers, [cm.topk_allreduce_ms(p, m, rho) for p in workers], "r-x", label="TopKAllReduce")
    ax.plot(workers, [cm.gtopk_allreduce_ms(p, m, rho) for p in workers], "g-^", label="gTopKAllReduce")
    ax.set_xlabel("Number of workers")
    ax.set_ylabel("Communication time [ms]")
    ax.grid(linestyle=":")
    ax.legend(loc=2)
    fig.savefig(out)
    plt.close(fig)
    return out


def plot_breakdown(out: str) -> str:
    plt = _plt()
    models = list(cm.PUBLISHED_BREAKDOWN)
    ratios = np.array([cm.breakdown_ratios(m) for m in models])
    fig, ax = plt.subplots(figsize=(4.8, 3.4))
    bottom = np.zeros(len(models))
    for j, (name, hatch) in enumerate((("Compu.", "x"), ("Compr.", "-"), ("Commu.", ""))):
        ax.bar(np.arange(len(models)), ratios[:, j], 0.35, bottom=bottom, hatch=hatch, label=name)
        bottom += ratios[:, j]
    ax.set_xticks(np.arange(len(models)))
    ax.set_xticklabels(models)
    ax.set_ylabel("Percentage")
    ax.legend(ncol=3)
    fig.savefig(out)
    plt.close(fig)
    return out


def plot_loss_curves(logfiles: Sequence[str], labels: Sequence[str], out: str, accuracy: bool = False) -> str:
    plt = _plt()
    fig, ax = plt.subplots(figsize=(5, 4))
    for path, label in zip(logfiles, labels):
        log = parse_log(path)
        ys = log.val_acc if accuracy else log.train_loss
        ax.plot(np.arange(1, len(ys) + 1), ys, label=label)
    ax.set_xlabel("Epoch")
    ax.set_ylabel("Validation accuracy" if accuracy else "Training loss")
    ax.legend()
    fig.savefig(out)
    plt.close(fig)
    return out


def delta_from_norm_files(path: str, epochs: int, rank: int = 0) -> np.ndarray:
    """delta = ||x - gtopk(x)||^2 / ||x - randk(x)||^2 per epoch from the
    PROFILING_NORM dumps of the trainer."""
    out = []
    for e in range(epochs):
        g = np.load("%s/gtopknorm-rank%d-epoch%d.npy" % (path, rank, e))
        r = np.load("%s/randknorm-rank%d-epoch%d.npy" % (path, rank, e))
        out.append(float(np.mean(g ** 2) / np.mean(r ** 2)))
    return np.array(out)


def plot_delta(path: str, epochs: int, out: str, rank: int = 0) -> Optional[str]:
    plt = _plt()
    d = delta_from_norm_files(path, epochs, rank)
    fig, ax = plt.subplots(figsize=(5, 4))
    ax.plot(d, label=r"$\delta$")
    ax.plot(np.ones_like(d), ":", color="black", label="1 ref.")
    ax.set_xlabel("Epoch")
    ax.legend()
    fig.savefig(out)
    plt.close(fig)
    return out
