"""Communication engine: merged gradient groups and their sparse / dense
all-reduce, driven by CUDA streams instead of a host thread.

Reference: allreducer.py:182-600 (``AllReducer``).  What it keeps: grouping by
threshold in backward order, the per-group residual store, the dynamic density
schedule ``[0.004, density]``, optional pre-compression norm clipping, the
three sparse modes plus dense, the ``err_callback(new_size, new_rank)`` hook,
the seven-column profiling line and the PROFILING_NORM diagnostic.

What changes: a group is a slice of the flat gradient buffer (no merge copy);
``reduce_group`` enqueues K1 (+K4) and the exchange kernel on a side stream as
soon as the group's last gradient has been produced, and nothing synchronises
the device.  The result of a sparse reduction stays sparse: ``SparseResult``
hands K3 the k global pairs.  On CUDA with more than one rank the exchange is
the persistent peer-store kernel (no MPI, no NCCL, no host staging) when all
ranks share a host and have GPU peer access, else the selection is staged
through the host and gloo; on CPU it is the gloo fallback, which is also the
oracle.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import numpy as np
import torch

from .. import settings
from ..ops import exchange as ex
from ..ops import oracle
from ..ops.clip import ClipNorm
from ..ops.select import TopkSelector, pairs_to_tensors, tensors_to_pairs
from ..settings import logger
from ..utils.timing import PhaseTimers
from . import comm, fallback
from .flat_buffer import FlatBuffers, MergedGroup


class MESSAGE:
    STOP = "STOP"
    RUNNING = "RUNNING"


class GTopkTimeout(RuntimeError):
    """A bounded device-side or host-side wait ran out: a peer is missing."""


def _default_err_callback(new_num_workers, new_rank):
    logger.error("Some process error accurs, number of workers changes to %d, my rank changes to %d",
                 new_num_workers, new_rank)


@dataclass
class SparseResult:
    """k global pairs of one group, ready for K3.

    ``pairs`` is an int32 [nseg * seg_stride, 2] tensor; segment s holds
    ``counts[s]`` live pairs.  ``use_atomics`` is set when indices can repeat
    across segments (Top-k all-gather).  ``scale`` is 1/P."""
    pairs: torch.Tensor
    counts: torch.Tensor
    nseg: int
    seg_stride: int
    use_atomics: bool
    scale: float
    # two-parity buffers of the exchange kernel: the live half is chosen on the device from the
    # exchange's call counter, base = pairs + ((word - 1) & 1) * parity_stride (None: single buffer)
    parity_word: Optional[torch.Tensor] = None
    parity_stride: int = 0

    def live_pairs(self) -> torch.Tensor:
        """The live half as a tensor (reads the counter: synchronises)."""
        if self.parity_word is None:
            return self.pairs
        off = ((int(self.parity_word.item()) - 1) & 1) * self.parity_stride
        return self.pairs[off:off + self.nseg * self.seg_stride]


class GroupEngine:
    """Everything one merged group needs to be reduced."""

    def __init__(self, owner: "AllReducer", g: MergedGroup):
        self.owner, self.g = owner, g
        fb = owner.flat
        self.grad = fb.group_slice(fb.grad, g)
        self.resid = fb.group_slice(fb.residual, g) if fb.residual is not None else None
        self.numel = g.numel                # span in the flat buffers: what the kernels run over
        self.param_numel = g.param_numel    # number of parameters: what the density applies to
        if self.numel >= 2 ** 31:
            raise ValueError("merged group %d holds %d elements; the sparse pairs carry int32 indices, so a group must "
                             "stay below 2^31 elements: lower the merge threshold" % (g.index, self.numel))
        self.last_k = 0
        self.select_done = None
        self.result: Optional[SparseResult] = None
        self.dense_ready = False
        dev = fb.device
        self.is_cuda = dev.type == "cuda"
        mode = owner.mode
        if mode == "none":
            return
        dens = max(owner.densities()) if owner.densities() else owner._density
        self.max_k = oracle.num_selected(self.param_numel, dens)
        self.selector = TopkSelector(self.numel, self.max_k, dev, limit_ms=owner.wait_limit_ms)
        self.rank_ctx = None
        world = owner.size()
        # CUDA ranks that cannot reach each other's memory (several hosts, no peer access) stage their
        # sets through the host and gloo, as CPU ranks do
        self.staged = world > 1 and self.is_cuda and comm.sparse_transport() == "staged"
        if world > 1 and self.is_cuda and not self.staged:
            with_ag = mode in ("topk", "topk2")
            nbytes = ex.region_bytes(self.max_k, with_ag)
            self.region = ex.SymmetricRegion.create_ipc(nbytes, group=comm.cpu_group())
            self.rank_ctx = ex.ExchangeRank(owner.rank(), world, self.numel, self.max_k, self.selector, self.resid,
                                            self.region, with_allgather=with_ag, reselect=(mode == "topk2"))
            self.gout = ex.pairs_view(self.rank_ctx.gout_ptr(0), 2 * self.max_k, dev)
            if with_ag:
                self.ag = ex.pairs_view(self.rank_ctx.ag_ptr(0), 2 * ex.MAX_PEERS * self.max_k, dev)
        elif world > 1:
            cap = self.max_k * (world if mode == "topk" else 1)
            self.host_pairs = torch.zeros((cap, 2), dtype=torch.int32, device=dev)
            self.host_counts = torch.zeros(ex.MAX_PEERS, dtype=torch.int32, device=dev)

    # ------------------------------------------------------------------
    def reduce(self, density: float, g_scale: Optional[torch.Tensor]) -> None:
        """Enqueue select + exchange for this group on the current stream."""
        o = self.owner
        world, mode = o.size(), o.mode
        k = oracle.num_selected(self.param_numel, density)
        k = min(k, self.max_k)
        self.last_k = k
        t = o.timers
        t.start(self.g.key, "compression")
        self.selector.select(self.grad, self.resid, k, g_scale=g_scale)
        if self.is_cuda:
            # the dense part of the update streams the same HBM as the select: it is ordered behind this
            # event, so the select has the bandwidth to itself and the dense part overlaps the exchange
            self.select_done = torch.cuda.Event()
            self.select_done.record()
        t.stop(self.g.key, "compression")
        t.start(self.g.key, "allreduce")
        if world == 1:
            self.result = SparseResult(self.selector.sel, self.selector.n_sel_tensor, 1, self.max_k, False, 1.0)
        elif self.is_cuda and not self.staged:
            rc = self.rank_ctx
            if mode == "gtopk":
                ex.launch_gtopk([rc], rc.desc, o.rank(), world, k, limit_ms=o.wait_limit_ms)
                self.result = SparseResult(self.gout, rc.n_global, 1, self.max_k, False, 1.0 / world,
                                           rc.epoch, rc.parity_stride)
            else:
                ex.launch_allgather([rc], rc.desc, rc.seg_counts, o.rank(), world, k,
                                    reselect=(mode == "topk2"), limit_ms=o.wait_limit_ms)
                if mode == "topk":
                    self.result = SparseResult(self.ag, rc.seg_counts, world, self.max_k, True, 1.0 / world,
                                               rc.epoch, rc.ag_parity_stride)
                else:
                    self.result = SparseResult(self.gout, rc.n_global, 1, self.max_k, False, 1.0 / world,
                                               rc.epoch, rc.parity_stride)
            rc.mirror_status()  # 16 bytes to pinned host memory, read by poll_failure() before the next iteration
        else:
            self._reduce_host(k, world, mode)
        t.stop(self.g.key, "allreduce")

    def _reduce_host(self, k: int, world: int, mode: str) -> None:
        """CPU tensors, or CUDA tensors in staged transport: the gloo fallback
        (also the multi-process oracle).  Synchronises the current stream."""
        o = self.owner
        idx, val = self.selector.pairs()
        grp = comm.cpu_group()
        dev = self.resid.device
        try:
            if mode == "gtopk":
                gi, gv = fallback.gtopk_allreduce(idx, val, k, group=grp, timeout_s=o.wait_limit_ms / 1e3)
                oracle.put_back(self.resid, (idx, val), gi.to(dev))
                n = tensors_to_pairs(gi, gv, self.host_pairs)
                self.host_counts[0] = n
                self.result = SparseResult(self.host_pairs, self.host_counts, 1, self.host_pairs.shape[0], False,
                                           1.0 / world)
            elif mode == "topk":
                ai, av = fallback.topk_allgather(idx, val, group=grp)
                n = tensors_to_pairs(ai, av, self.host_pairs)
                self.host_counts[0] = n
                self.result = SparseResult(self.host_pairs, self.host_counts, 1, self.host_pairs.shape[0], True,
                                           1.0 / world)
            else:  # topk2
                ai, av = fallback.topk_allgather(idx, val, group=grp)
                kk = idx.numel()
                sets = [(ai[q * kk:(q + 1) * kk], av[q * kk:(q + 1) * kk]) for q in range(world)]
                gi, gv = oracle.topk2_reselect(sets, k)
                oracle.put_back(self.resid, (idx, val), gi.to(dev))
                n = tensors_to_pairs(gi, gv, self.host_pairs)
                self.host_counts[0] = n
                self.result = SparseResult(self.host_pairs, self.host_counts, 1, self.host_pairs.shape[0], False,
                                           1.0 / world)
        except fallback.PeerTimeout as exc:
            o.report_failure(str(exc))
            raise GTopkTimeout(str(exc)) from exc

    def poll_failure(self) -> None:
        """Look at the host mirror of the exchange's result words (refreshed behind
        every exchange, at most an iteration old) without synchronising.  A failed
        exchange has applied nothing (its global set is empty) and every later one
        returns at once, so raising here, before the next iteration is launched,
        loses no more than the iterations in flight."""
        rc = getattr(self, "rank_ctx", None)
        if rc is None:
            return
        status, where = rc.failed_on_host_mirror()
        if status != 0:
            self._raise_status(status, where)

    def _raise_status(self, status: int, where: int) -> None:
        from ..ops.lib import STATUS_NAMES
        msg = "group %s: %s (code location %d)" % (self.g.key[:40], STATUS_NAMES.get(status, status), where)
        self.owner.report_failure(msg)
        raise GTopkTimeout(msg)

    def check_status(self) -> None:
        """Read the device status words of the last exchange (synchronises the
        stream it ran on).  Raises GTopkTimeout after telling err_callback."""
        if getattr(self, "rank_ctx", None) is None:
            return
        status, where = self.rank_ctx.status()
        if status != 0:
            self._raise_status(status, where)
        region = getattr(self, "region", None)
        if region is not None and not region.guards_intact():
            raise RuntimeError("group %s: a store landed outside the exchange slots (guard band of the "
                               "peer-visible region was overwritten)" % self.g.key[:40])


class AllReducer:
    def __init__(self, named_parameters, lock=None, key_lock=None, compression=None, sparse=False,
                 err_callback: Optional[Callable[[int, int], None]] = None, layerwise_times=None, sigma_scale=2.5,
                 density=0.001, train_epoch=0, norm_clip=None, msg_queue=None, msg_queue2=None, writer=None,
                 threshold: Optional[int] = None, flat: Optional[FlatBuffers] = None,
                 wait_limit_ms: Optional[float] = None):
        self._running = False
        self._msg_queue, self._msg_queue2 = msg_queue, msg_queue2
        self._writer = writer
        self._profiling = True
        self._sparse = bool(sparse)
        self._sigma_scale = sigma_scale
        self._density = density
        self.train_epoch = train_epoch
        self.train_iter = 0
        self._layerwise_times = layerwise_times
        self._lock, self._key_lock = lock, key_lock
        self._compression = compression
        self._err_callback = err_callback if err_callback else _default_err_callback
        self._norm_clip = norm_clip
        self.wait_limit_ms = float(wait_limit_ms if wait_limit_ms is not None else settings.WAIT_LIMIT_MS)
        cname = getattr(compression, "name", "none") if compression is not None else "none"
        self.mode = cname if self._sparse else "none"
        world = comm.size()
        if self.mode == "gtopk" and world & (world - 1):
            raise ValueError("gTop-k pairs ranks in a recursive-doubling tree and needs a power-of-two number of "
                             "workers (got %d); use the 'topk' or 'topk2' compressor otherwise" % world)
        logger.info("density: %f", self._density)
        named = list(named_parameters)
        self._named_parameters = dict(named)
        self._sequential_keys = [k for k, _ in named]
        self.flat = flat if flat is not None else FlatBuffers(
            named, settings.THRESHOLD if threshold is None else threshold, with_residual=True)
        self._groups = [g.names for g in self.flat.groups]
        self._key_groupidx_maps = dict(self.flat.key_group)
        self._merged_parameters = {g.key: self.flat.group_slice(self.flat.grad, g) for g in self.flat.groups}
        self._merged_parameter_offsets = {g.key: g.offsets for g in self.flat.groups}
        self._sizes = [self._named_parameters[k].numel() for k in self._sequential_keys][::-1]
        logger.info("groups: %d, sizes: %s", len(self._groups), [g.param_numel for g in self.flat.groups])
        # dynamic densities (allreducer.py:226-230): epoch 0 -> 0.004, then --density
        self._dynamic_densities = None if settings.PIN_DENSITY else [0.004, self._density]
        if self._dynamic_densities is not None:
            logger.info("dynamic densities = %s", self._dynamic_densities)
        self.timers = PhaseTimers(enabled=self._profiling)
        self._profiling_norms: List[tuple] = []
        self.allreduce_count = 0
        self._failed: Optional[str] = None
        self.clip = ClipNorm(self.flat.device) if norm_clip is not None else None
        self.engines = [GroupEngine(self, g) for g in self.flat.groups]
        self._entries: Dict[str, torch.Tensor] = {}
        self._outputs: Dict[str, torch.Tensor] = {}

    # -- topology ------------------------------------------------------------
    def rank(self) -> int:
        return comm.rank()

    def size(self) -> int:
        return comm.size()

    # -- density schedule ------------------------------------------------------
    def densities(self) -> List[float]:
        return list(self._dynamic_densities) if self._dynamic_densities is not None else [self._density]

    def get_current_density(self) -> float:
        d = self._dynamic_densities
        if d is None:
            return self._density
        return d[-1] if self.train_epoch >= len(d) else d[self.train_epoch]

    @staticmethod
    def get_approximate_sigma_scale(density: float) -> float:
        """Kept for log/API parity (allreducer.py:408-418); selection ignores it."""
        if density > 0.7:
            return 0.5
        if density > 0.05:
            return 1.5
        if density > 0.01:
            return 2.0
        return 3.0

    # -- reduction -----------------------------------------------------------
    def reduce_group(self, gi: int) -> None:
        """Enqueue the reduction of group ``gi`` on the current CUDA stream (or
        run it now on CPU)."""
        eng = self.engines[gi]
        key = eng.g.key
        if self.mode == "none":
            self.timers.start(key, "allreduce")
            if self.size() > 1:
                fallback.dense_allreduce(eng.grad)
            eng.dense_ready = True
            self.timers.stop(key, "allreduce")
            self.allreduce_count += 1
            return
        if settings.PROFILING_NORM:
            dense_ref = self._profiling_before(eng)
        g_scale = None
        if self._norm_clip is not None:
            self.clip.add_dense(eng.grad)
            g_scale = self.clip.finalize(float(np.sqrt(1.0 / self.size()) * self._norm_clip))
        eng.reduce(self.get_current_density(), g_scale)
        if settings.PROFILING_NORM:
            self._profiling_after(eng, dense_ref)
        self.allreduce_count += 1

    def results(self) -> List[Optional[SparseResult]]:
        return [e.result for e in self.engines]

    def check_status(self) -> None:
        for e in self.engines:
            e.check_status()

    def poll_failure(self) -> None:
        for e in self.engines:
            e.poll_failure()

    def report_failure(self, msg: str) -> None:
        """A peer is gone: tell the trainer (it may shrink the world and
        re-shard its data) once per failure."""
        if self._failed is None:
            self._failed = msg
            logger.error("communication failure: %s", msg)
            try:
                self._err_callback(max(self.size() - 1, 1), self.rank())
            except Exception:  # the callback must never mask the failure
                logger.exception("err_callback raised")

    # -- profiling -----------------------------------------------------------
    def maybe_print_profiling(self) -> None:
        """Every 100 samples rank 0 logs the per-group means in the reference's
        column order (allreducer.py:334-387)."""
        if not self._profiling or self.rank() != 0 or not self.engines:
            return
        if self.timers.samples(self.engines[0].g.key) < 100:
            return
        logger.info("[rank:%d]name[size]: backward, merge, compression, allreduce, demerge, d2h, h2d", self.rank())
        tot = np.zeros(7)
        total_sz = 0
        for e in self.engines:
            m = self.timers.means(e.g.key)
            row = [m[p] for p in PhaseTimers.PHASES]
            tot += np.array(row)
            total_sz += e.param_numel
            k = e.g.key
            logger.info("[rank:%d]%s[%d]: %f,%f,%f,%f,%f,%f,%f", self.rank(), k[0:3] + "..." + k[-3:], e.param_numel, *row)
        logger.info("[rank:%d]%s[%d]: %f,%f,%f,%f,%f,%f,%f", self.rank(), "total", total_sz, *tot.tolist())

    def _profiling_before(self, eng: GroupEngine):
        """PROFILING_NORM (allreducer.py:520-526): the dense all-reduce of
        g + r that the sparse result is compared with.  Diagnostic only."""
        with torch.no_grad():
            ref = eng.grad + eng.resid
            if self.size() > 1:
                fallback.dense_allreduce(ref)
            return ref / self.size()

    def _profiling_after(self, eng: GroupEngine, dense_ref: torch.Tensor) -> None:
        with torch.no_grad():
            res = eng.result
            sparse = torch.zeros_like(dense_ref)
            live = res.live_pairs()
            for s in range(res.nseg):
                n = int(res.counts[s])
                idx, val = pairs_to_tensors(live[s * res.seg_stride:(s + 1) * res.seg_stride], n)
                sparse.index_add_(0, idx.to(sparse.device), val.to(sparse.device) * res.scale)
            k = oracle.num_selected(eng.param_numel, self.get_current_density())
            perm = torch.randperm(dense_ref.numel(), device=dense_ref.device)[:k]
            randk = torch.zeros_like(dense_ref)
            randk[perm] = dense_ref[perm]
            xnorm = float(dense_ref.norm())
            self._profiling_norms.append((float((dense_ref - sparse).norm()), float((dense_ref - randk).norm()),
                                          1.0 * (dense_ref.numel() - k) / dense_ref.numel() * xnorm, xnorm,
                                          float(dense_ref.std())))

    # -- API kept from the reference's thread-based engine ---------------------
    def add_tensor(self, name, tensor):
        if name in self._entries:
            return None
        self._entries[name] = tensor
        return name

    def get_result(self, name):
        return self._outputs.get(name, self.flat.grad_view(name))

    def reset(self) -> None:
        self._entries.clear()
        self.maybe_print_profiling()

    def run(self) -> None:
        """Compatibility loop for callers that feed parameter names through
        ``msg_queue``: a group is reduced when its last name arrives."""
        if self._msg_queue is None:
            return
        self._running = True
        arrived = [0] * len(self.engines)
        reduced = 0  # groups completed in the current iteration
        while self._running:
            name = self._msg_queue.get()
            if name == MESSAGE.STOP:
                break
            gi = self._key_groupidx_maps[name]
            arrived[gi] += 1
            if arrived[gi] == len(self._groups[gi]):
                arrived[gi] = 0
                self.reduce_group(gi)
                reduced += 1
                # names arrive in backward order, so the last group completes first: "DONE" is due only
                # when all of them have been reduced (allreducer.py:594-597)
                if reduced == len(self.engines):
                    reduced = 0
                    if self._msg_queue2 is not None:
                        self.reset()
                        self._msg_queue2.put("DONE")

    def rebuild(self) -> None:
        """The process group changed (a smaller world after a planned
        departure): release what was tied to the old one and build the group
        engines again.  Gradients, residuals, parameters and momentum live in
        the flat buffers and are untouched; the selectors start again with an
        exact pass.  gTop-k needs a power-of-two world: on any other size the
        job continues with 'topk2' (all-gather, sum, global re-selection)."""
        self.stop()
        self._failed = None
        world = comm.size()
        if self.mode == "gtopk" and world & (world - 1):
            logger.warning("%d workers left: gTop-k needs a power of two, continuing with topk2", world)
            self.mode = "topk2"
        self.engines = [GroupEngine(self, g) for g in self.flat.groups]

    def stop(self) -> None:
        self._running = False
        for e in self.engines:
            region = getattr(e, "region", None)
            if region is not None:
                if torch.cuda.is_available():
                    torch.cuda.synchronize()
                region.close()
                e.region = None
