"""Figures of the papers, rendered head-less (Agg backend) to image files.
matplotlib is optional: without it every function raises a clear ImportError
and the numeric helpers in cost_models / log_parser remain usable.
(reference: scripts/icdcs2019/communication.py, plot_loss.py, plot_sth.py,
scripts/ijcai2019/plot_loss.py -- those need a display through TkAgg.)"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

from . import comm_logs as cl
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


# ---- communication measurements (scripts/icdcs2019/communication.py:285-331, 557-586) ---------------------
def plot_measured_allreduce(logfiles: dict, out: str, nccl: bool = False, with_model: bool = True) -> str:
    """Measured all-reduce time against message size, one curve per worker count
    (``logfiles``: {workers: path}), with the ring model's prediction dashed."""
    plt = _plt()
    fig, ax = plt.subplots(figsize=(5, 4.5))
    for n in sorted(logfiles):
        if nccl:
            sizes, times = cl.read_nccl_tests_log(logfiles[n])
            errs = None
            label = "%d GPUs" % n
        else:
            sizes, times, errs = cl.read_allreduce_log(logfiles[n])
            label = "%d nodes" % n
        if not sizes:
            continue
        ax.errorbar(sizes, times, errs, label=label, linewidth=1)
        if with_model:
            ax.plot(sizes, cl.predict_allreduce(sizes, n), "--", linewidth=1, color="gray")
    ax.set_xlabel("Size of parameters")
    ax.set_ylabel("Communication time [us]")
    ax.grid(linestyle=":")
    ax.legend(loc=2)
    fig.savefig(out)
    plt.close(fig)
    return out


def plot_p2p_latency(logfile: str, out: str) -> tuple:
    """Point-to-point probe with the fitted line time = alpha + beta * size (milliseconds).
    Returns (alpha, beta, path)."""
    plt = _plt()
    sizes, times, errs = cl.read_allreduce_log(logfile)
    times = [t / 1000.0 for t in times]
    errs = [e / 1000.0 for e in errs]
    alpha, beta = cl.fit_alpha_beta(sizes, times)
    fig, ax = plt.subplots(figsize=(5, 3.8))
    ax.errorbar(sizes, times, errs, fmt="o", linewidth=1, label="Measured point-to-point communication")
    ax.plot(sizes, alpha + np.asarray(sizes) * beta, linewidth=1,
            label=r"Predicted ($\alpha=%.3f, \beta=%f$)" % (alpha, beta))
    ax.set_xlabel("Size of parameters [bytes]")
    ax.set_ylabel("Communication time [ms]")
    ax.set_ylim(bottom=0)
    ax.grid(linestyle=":")
    ax.legend(loc=2, prop={"size": 9})
    fig.savefig(out)
    plt.close(fig)
    return alpha, beta, out


# ---- backward/communication timelines and per-layer sizes (scripts/icdcs2019/plot_sth.py:21-197) -----------
_LANES = {"compute": (0.40, "#2e75b6", "Comp."), "wfbp": (0.30, "#c00000", "Comm.(WF.)"),
          "single": (0.20, "#3F5EBA", "Comm.(S.E.)"), "merged": (0.08, "#c55a11", "Comm.(M.W.)")}


def plot_timeline(timelines: dict, out: str, title: str = "") -> str:
    """Gantt-style rendering of ``analysis.cost_models.Timeline`` objects: the compute lane of the
    first one on top, then one communication lane per entry of ``timelines`` (keys among
    'wfbp', 'single', 'merged').  Times in microseconds; the axis is labelled in milliseconds."""
    plt = _plt()
    from matplotlib.patches import Rectangle
    fig, ax = plt.subplots(figsize=(9, 3))
    span = max(max((s + d for s, d in tl.compute + tl.comm), default=1.0) for tl in timelines.values())
    first = next(iter(timelines.values()))
    height = 0.09

    def lane(tasks, key):
        y, color, label = _LANES[key]
        for i, (start, dur) in enumerate(tasks):
            if dur > 0:
                ax.add_patch(Rectangle((start / span, y), dur / span, height, color=color, ec="black", alpha=0.8))
                ax.annotate(str(i + 1), (start / span, y + 0.02), fontsize=7)
        ax.text(-0.01, y + height / 2, label, ha="right", va="center", fontsize=9)

    lane(first.compute, "compute")
    for key, tl in timelines.items():
        lane(tl.comm, key)
    ax.set_xlim(0, 1.05)
    ax.set_ylim(0, 0.55)
    ax.get_yaxis().set_ticks([])
    ax.set_xticks([i * 0.1 for i in range(11)])
    ax.set_xticklabels(["%.1f" % (span * i * 0.1 / 1000.0) for i in range(11)])
    ax.set_xlabel("t (ms)")
    for side in ("top", "right"):
        ax.spines[side].set_visible(False)
    if title:
        ax.set_title(title)
    fig.subplots_adjust(left=0.14, bottom=0.2)
    fig.savefig(out)
    plt.close(fig)
    return out


def plot_layer_log_timeline(logfile: str, out: str, num_of_nodes: int = 4) -> str:
    """Reads a per-layer log and renders its WFBP, single-all-reduce and merged timelines."""
    sizes, comms, computes, _ = cl.read_layer_log(logfile)
    sim = cm.Simulator(logfile, computes, sizes, num_of_nodes)
    return plot_timeline({"wfbp": sim.wfbp(comms), "single": sim.single_allreduce(), "merged": sim.mg_wfbp()}, out)


def plot_gradient_sizes(logfiles: dict, out: str) -> dict:
    """Number of parameters per learnable layer, one scatter series per network
    (``logfiles``: {label: per-layer log}).  Returns the size statistics per label."""
    plt = _plt()
    fig, ax = plt.subplots(figsize=(5, 4.5))
    stats = {}
    for (label, path), marker in zip(logfiles.items(), "+xdo^v"):
        sizes, _, _, _ = cl.read_layer_log(path)
        ax.scatter(range(1, len(sizes) + 1), sizes, label=label, marker=marker, s=40)
        stats[label] = cl.gradient_size_statistics(sizes)
    ax.set_xlim(left=0)
    ax.set_xlabel("Learnable layer ID")
    ax.set_ylabel("# of parameters")
    ax.set_yscale("log")
    ax.legend()
    fig.savefig(out)
    plt.close(fig)
    return stats


# ---- grouped figures of the convergence study (scripts/ijcai2019/plot_loss.py:237-252, 341-375) -------------
def _grid(plt, n, per_row=3):
    rows = (n + per_row - 1) // per_row
    fig, axs = plt.subplots(rows, per_row, figsize=(4.2 * per_row, 3.4 * rows), squeeze=False)
    return fig, [axs[i // per_row][i % per_row] for i in range(rows * per_row)]


def plot_group_norm_diff(runs: dict, out: str) -> str:
    """One panel per network: training loss of the dense and the gTop-k run (left axis)
    and delta = ||x - gtopk(x)||^2 / ||x - randk(x)||^2 per epoch (right axis, with the
    reference line at 1).  ``runs``: {network: {"dense_log": path or None,
    "gtopk_log": path or None, "norm_dir": dir with the PROFILING_NORM dumps, "epochs": n}}."""
    plt = _plt()
    fig, axes = _grid(plt, len(runs))
    for ax, (name, r) in zip(axes, runs.items()):
        for key, label, color in (("dense_log", "S-SGD loss", "C3"), ("gtopk_log", "gTop-$k$ S-SGD loss", "C2")):
            if r.get(key):
                log = parse_log(r[key])
                ax.plot(np.arange(1, len(log.train_loss) + 1), log.train_loss, label=label, color=color, linewidth=1)
        ax.set_xlabel("Epoch")
        ax.set_ylabel("Training loss")
        ax.set_title(name)
        twin = ax.twinx()
        d = delta_from_norm_files(r["norm_dir"], r["epochs"], r.get("rank", 0))
        twin.plot(d, label=r"$\delta$", color="C0", linewidth=1)
        twin.plot(np.ones_like(d), ":", color="black", linewidth=1, label="1 ref.")
        twin.set_ylabel(r"$\delta$")
    for ax in axes[len(runs):]:
        ax.axis("off")
    handles, labels = axes[0].get_legend_handles_labels()
    fig.legend(handles, labels, ncol=4, loc="upper center")
    fig.tight_layout(rect=(0, 0, 1, 0.93))
    fig.savefig(out)
    plt.close(fig)
    return out


def plot_group_sensitivity(runs: dict, out: str, accuracy: bool = False) -> str:
    """One panel per network, one curve per setting (the papers vary the density: c = 1/rho;
    the same layout serves a learning-rate sweep).  ``runs``: {network: {legend: logfile}}."""
    plt = _plt()
    fig, axes = _grid(plt, len(runs), per_row=2)
    for ax, (name, curves) in zip(axes, runs.items()):
        for legend, path in curves.items():
            log = parse_log(path)
            ys = log.val_acc if accuracy else log.train_loss
            ax.plot(np.arange(1, len(ys) + 1), ys, label=legend, linewidth=1)
        ax.set_xlabel("Epoch")
        ax.set_ylabel("Validation accuracy" if accuracy else "Training loss")
        ax.set_title(name)
        ax.legend(ncol=2, loc="upper right", fontsize=8)
    for ax in axes[len(runs):]:
        ax.axis("off")
    fig.tight_layout()
    fig.savefig(out)
    plt.close(fig)
    return out
