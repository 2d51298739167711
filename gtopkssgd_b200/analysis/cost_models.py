"""Analytical communication models and the numbers published with the papers
(reference: scripts/icdcs2019/communication.py).

* alpha-beta costs of dense ring all-reduce, Top-k all-gather and the gTop-k
  tree (communication.py:588-600, README.md:5-9), with the constants fitted on
  the papers' 1 GbE cluster, and an NVLink parameterisation for this hardware;
* the ring all-reduce lower-bound model used by the timeline simulator
  (communication.py:32-55);
* the wait-free back-propagation (WFBP) timeline simulator with greedy layer
  merging (MG-WFBP, communication.py:77-231), without any plotting inside;
* the measured per-worker throughputs and time breakdowns hard-coded in the
  paper scripts (communication.py:472-497, 674-678), as data.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

# ---- fitted point-to-point constants of the papers' cluster (milliseconds, fp32 elements) ----
ALPHA_MS = 0.436
BETA_MS_PER_ELEMENT = 4 * 9e-6


def dense_allreduce_ms(P, m, alpha=ALPHA_MS, beta=BETA_MS_PER_ELEMENT):
    """Ring all-reduce of m elements: 2(P-1)a + 2(P-1)/P m b."""
    return 2 * (P - 1) * alpha + 2.0 * (P - 1) / P * m * beta


def topk_allreduce_ms(P, m, rho=0.001, alpha=ALPHA_MS, beta=BETA_MS_PER_ELEMENT):
    """Top-k all-gather: log2(P) a + 2(P-1) rho m b."""
    return math.log2(P) * alpha + 2.0 * (P - 1) * rho * m * beta


def gtopk_allreduce_ms(P, m, rho=0.001, alpha=ALPHA_MS, beta=BETA_MS_PER_ELEMENT):
    """gTop-k tree + broadcast: 2 log2(P) a + 4 log2(P) rho m b."""
    return 2 * math.log2(P) * alpha + 4.0 * math.log2(P) * rho * m * beta


def nvlink_gtopk_roofline_ms(P, k, link_gbs=770.0):
    """Wire time of the 8-byte-pair exchange on one NVLink direction:
    2 k log2(P) 8 bytes / bandwidth."""
    return 2.0 * k * math.log2(P) * 8 / (link_gbs * 1e9) * 1e3


def ring_allreduce_us(n, M, bandwidth_bytes=9.0 * 1024 ** 3 / 8):
    """Lower-bound ring model (E. Chan et al. 2007) in microseconds for n nodes
    and M fp32 elements on a link of ``bandwidth_bytes`` per second."""
    alpha = 45.25e-6
    beta = 1.2 / bandwidth_bytes
    gamma = 160.0 / (16.0e9 * 4)
    nbytes = 4 * M
    return (2 * (n - 1) * alpha + 2 * (n - 1) * nbytes * beta / n + (n - 1) * nbytes * gamma / n) * 1e6


# ---- published measurements ----------------------------------------------------------------------
WORKERS = [1, 4, 8, 16, 32]
PUBLISHED_THROUGHPUT: Dict[str, Dict[str, List[float]]] = {
    "VGG-16": {"batch": [128], "dense": [1317.333, 104.200, 92.560, 39.480, 12.600],
               "topk": [1317.333, 110.576, 109.900, 97.865, 63.002],
               "gtopk": [1317.333, 131.060, 130.551, 126.434, 123.200]},
    "ResNet-20": {"batch": [32], "dense": [920.632, 821.700, 705.200, 520.400, 287.900],
                  "topk": [920.632, 908.837, 752.985, 737.594, 696.029],
                  "gtopk": [920.632, 916.260, 868.730, 808.500, 789.300]},
    "AlexNet": {"batch": [32], "dense": [173.469, 14.010, 12.118, 4.936, 1.234],
                "topk": [173.469, 14.238, 13.865, 13.352, 9.236],
                "gtopk": [173.469, 16.536, 16.446, 16.359, 15.777]},
    "ResNet-50": {"batch": [32], "dense": [52.873, 39.002, 36.989, 23.176, 10.721],
                  "topk": [52.873, 37.729, 35.703, 34.495, 30.583],
                  "gtopk": [52.873, 39.795, 39.713, 39.060, 39.119]},
    "LSTM-PTB": {"batch": [32], "dense": [392.0, 12.657, 8.7, 4.1, 2.1],
                 "topk": [392.0, 19.9, 18.6, 14.8, 5.4],
                 "gtopk": [392.0, 17.8, 17.6, 15.1, 10.8]},
}
# seconds per iteration at 32 workers: [compute, compression, communication]
PUBLISHED_BREAKDOWN = {
    "VGG-16": [0.139536, 0.091353, 0.811753],
    "ResNet-20": [0.146005, 0.001618, 0.024686],
    "AlexNet": [0.257205, 0.383776, 3.36298],
    "ResNet-50": [4.882041, 0.15405, 1.424253],
}


def scaling_efficiency(per_worker_throughput: Sequence[float]) -> List[float]:
    """Percent of the single-worker speed kept at each worker count (first
    entry is the single-worker speed itself)."""
    base = per_worker_throughput[0]
    return [100.0 * v / base for v in per_worker_throughput[1:]]


def speedup_over(a: Sequence[float], b: Sequence[float]) -> List[float]:
    return [x / y for x, y in zip(a[1:], b[1:])]


def breakdown_ratios(model: str) -> List[float]:
    vals = PUBLISHED_BREAKDOWN[model]
    total = sum(vals)
    return [v / total for v in vals]


# ---- WFBP / MG-WFBP timeline ---------------------------------------------------------------------
@dataclass
class Timeline:
    """Start time and duration (microseconds) of every compute and comm task."""
    compute: List[tuple] = field(default_factory=list)
    comm: List[tuple] = field(default_factory=list)
    total_ms: float = 0.0
    merged_layers: List[int] = field(default_factory=list)


class Simulator:
    """Backward pass of L layers (last layer first) with one all-reduce per
    layer.  ``computes[i]`` is the backward time of the i-th layer to finish,
    ``sizes[i]`` its gradient size in elements."""

    def __init__(self, name: str, computes: Sequence[float], sizes: Sequence[float], num_of_nodes: int,
                 comm_model=ring_allreduce_us):
        self.name, self.computes, self.sizes = name, list(computes), list(sizes)
        self.num_of_nodes, self.comm_model = num_of_nodes, comm_model

    def _comms(self, sizes):
        return [self.comm_model(self.num_of_nodes, s) for s in sizes]

    def wfbp(self, comms: Optional[Sequence[float]] = None) -> Timeline:
        """Each layer's all-reduce starts when its gradient exists and the
        previous all-reduce has finished."""
        comms = list(comms) if comms is not None else self._comms(self.sizes)
        tl = Timeline()
        t_comp, comm_start, comm = 0.0, 0.0, 0.0
        for comp, c in zip(self.computes, comms):
            tl.compute.append((t_comp, comp))
            comm_start = max(comm_start + comm, t_comp + comp)
            comm = c
            if c > 0:
                tl.comm.append((comm_start, c))
            t_comp += comp
        tl.total_ms = (comm_start + comm) / 1000.0
        return tl

    def single_allreduce(self) -> Timeline:
        """All gradients in one all-reduce after backward (no overlap)."""
        tl = Timeline()
        total_comp = sum(self.computes)
        comm = self.comm_model(self.num_of_nodes, sum(self.sizes))
        tl.compute = [(0.0, total_comp)]
        tl.comm = [(total_comp, comm)]
        tl.total_ms = (total_comp + comm) / 1000.0
        return tl

    @staticmethod
    def _comm_starts(comms, comps):
        starts = [0.0]
        done = 0.0
        for i in range(1, len(comms)):
            starts.append(max(starts[i - 1] + comms[i - 1], done + comps[i - 1]))
            done += comps[i - 1]
        return starts

    def mg_wfbp(self) -> Timeline:
        """Greedy merging: a layer whose all-reduce cannot be hidden behind the
        next layer's backward is merged into that next layer when this makes
        the pair finish earlier."""
        comms = self._comms(self.sizes)
        comps = self.computes[1:] + [0.0]
        opt_c, opt_s = list(comms), list(self.sizes)
        starts = self._comm_starts(opt_c, comps)
        merged: List[int] = []
        done = 0.0
        for i in range(len(comms) - 1):
            comp, comm = comps[i], opt_c[i]
            if starts[i] + comm > comp + done:
                size = opt_s[i] + opt_s[i + 1]
                together = self.comm_model(self.num_of_nodes, size)
                do_merge = (together < comm + opt_c[i + 1]) if starts[i] >= comp + done else \
                    (comp + done + together < starts[i] + comm + opt_c[i + 1])
                if do_merge:
                    opt_c[i], opt_c[i + 1], opt_s[i + 1] = 0.0, together, size
                    starts = self._comm_starts(opt_c, comps)
                    merged.append(i)
            done += comp
        tl = self.wfbp(opt_c)
        tl.merged_layers = merged
        return tl


# ---- speed-up studies built on the simulator (scripts/icdcs2019/communication.py:350-418, 420-470, 545-555) -------
def ssgd_speedup(r: float, n: int) -> float:
    """Speed-up of synchronous SGD on n workers when communication takes r times the compute time and
    nothing overlaps: n / (1 + r)."""
    return n / (1.0 + r)


def simulated_speedups(computes: Sequence[float], sizes: Sequence[float], batch: int,
                       nnodes: Sequence[int] = (4, 8, 16, 32, 64), comm_model=ring_allreduce_us) -> Dict[str, List[float]]:
    """Throughput on n nodes relative to one node for three schedules of the same per-layer
    backward times (microseconds) and gradient sizes: one all-reduce per layer as soon as its
    gradient exists (``wfbp``), the greedily merged version (``merged``), and a single all-reduce
    after backward (``single``).  Forward is taken as half of backward, as in the papers' script."""
    tb = float(sum(computes)) / 1000.0          # ms
    tf = 0.5 * tb
    single_node = batch / (tf + tb)
    out: Dict[str, List[float]] = {"nodes": list(nnodes), "linear": [float(n) for n in nnodes], "wfbp": [], "merged": [],
                                   "single": []}
    for n in nnodes:
        sim = Simulator("sim", computes, sizes, n, comm_model=comm_model)
        out["wfbp"].append(batch * n / (sim.wfbp().total_ms + tf) / single_node)
        out["merged"].append(batch * n / (sim.mg_wfbp().total_ms + tf) / single_node)
        out["single"].append(batch * n / (sim.single_allreduce().total_ms + tf) / single_node)
    return out


def real_comm_costs(per_gpu_pair_speeds: Sequence[float], batch: int):
    """From measured throughputs of 1, 2, 4, ... nodes with two GPUs each (samples/s of the whole job)
    to (compute seconds per iteration, [communication seconds at 2, 4, ... nodes]): the time per
    iteration of a worker is batch / (per-worker throughput); what exceeds the one-node time is
    communication (scripts/icdcs2019/communication.py:421-425)."""
    times = [batch / ((d / 2.0) / 2 ** (i - 1)) for i, d in enumerate(per_gpu_pair_speeds)]
    return times[0], [t - times[0] for t in times[1:]]
