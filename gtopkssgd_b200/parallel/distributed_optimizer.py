"""DistributedOptimizer: wraps a torch optimizer, reduces gradients group by
group while backward is still running, and applies the update with the fused
K3 kernels.

Public surface of the reference (distributed_optimizer.py:21-212):
``DistributedOptimizer(optimizer, named_parameters, compression, is_sparse,
err_handler, layerwise_times, sigma_scale, density, norm_clip, writer)``
returns an instance of a dynamic subclass of the wrapped optimizer's class
with ``step() synchronize() stop() add_train_epoch() get_current_density()``,
the ``local`` switch for gradient accumulation and ``momentum_correction``;
module-level ``rank()`` and ``size()``.

Differences in mechanism, not in semantics:
* per-parameter hooks only count arrivals; when the last gradient of a merged
  group has been produced an event is recorded and the group's select +
  exchange kernels are enqueued on a side stream (no device synchronisation,
  no host thread, no queue);
* ``synchronize()`` makes the compute stream wait for that side stream;
* ``step()`` is two launches over the flat buffers (dense part + k sparse
  pairs) instead of three launches per tensor; weight decay is applied after
  sparsification and the first momentum step is ``buf = d_p`` as in the
  reference (distributed_optimizer.py:126-137).
"""
from __future__ import annotations

import threading
import time
from typing import Optional

import torch

from .. import settings
from ..ops.clip import ClipNorm
from ..ops.sgd import SgdHyper, momentum_correct, scatter_dense, sgd_dense, sgd_sparse
from ..settings import logger
from . import allreducer as ar
from . import comm
from .compression import NoneCompressor
from .elastic import Membership, PeerLeft, StreamWatchdog
from .flat_buffer import FlatBuffers


class _DistributedOptimizer(torch.optim.Optimizer):
    def __init__(self, params, named_parameters, compressor, is_sparse=True, err_handler=None, layerwise_times=None,
                 sigma_scale=2.5, density=0.01, norm_clip=None, writer=None, threshold=None, overlap=True,
                 wait_limit_ms=None, membership_check_every=50, elastic=False):
        super(self.__class__, self).__init__(params)
        self.elastic = bool(elastic)
        self.generation = 0        # bumped whenever the process group is re-formed (captured graphs are stale then)
        self.leave_at: Optional[int] = None
        self._membership_check_every = membership_check_every
        self._compressor = compressor
        self._sparse = is_sparse
        self._layerwise_times = layerwise_times
        named_parameters = list(named_parameters) if named_parameters is not None else []
        if any(not isinstance(p, tuple) for p in named_parameters):
            raise ValueError("named_parameters should be a sequence of tuples (name, parameter), "
                             "usually produced by model.named_parameters().")
        if not named_parameters:
            named_parameters = [("allreduce.noname.%s" % i, v) for pg in self.param_groups
                                for i, v in enumerate(pg["params"])]
        owned = {id(p) for pg in self.param_groups for p in pg["params"]}
        named_parameters = [(n, p) for n, p in named_parameters if id(p) in owned and p.requires_grad]
        self._parameter_names = {p: n for n, p in named_parameters}
        self._lock, self._key_lock = threading.Lock(), threading.Lock()
        self.momentum_correction = False
        self.local = False
        self._synced = False
        self._step_count = 0
        self._materialized = False
        thr = settings.THRESHOLD if threshold is None else threshold
        self._flat = FlatBuffers(named_parameters, thr, with_residual=True)
        self._allreducer = ar.AllReducer(named_parameters, self._lock, self._key_lock, compressor, sparse=is_sparse,
                                         err_callback=err_handler, layerwise_times=layerwise_times,
                                         sigma_scale=sigma_scale, density=density, norm_clip=norm_clip, writer=writer,
                                         flat=self._flat, wait_limit_ms=wait_limit_ms)
        dev = self._flat.device
        self._is_cuda = dev.type == "cuda"
        self._overlap = overlap and self._is_cuda
        self._comm_stream = torch.cuda.Stream(device=dev) if self._is_cuda else None
        self._arrived = [0] * len(self._flat.groups)
        self._launched = [False] * len(self._flat.groups)
        self._expected = [len(g.names) for g in self._flat.groups]
        # learning rate as the kernels see it: a device scalar, refreshed whenever the host value
        # changes, so that a captured CUDA graph follows the LR schedule
        self._lr_dev = torch.zeros(1, dtype=torch.float32, device=dev)
        self._lr_host = None
        self._capturing = False
        self._stalled: Optional[str] = None
        self._watchdog: Optional[StreamWatchdog] = None
        self._watchdog_armed_at = 0.0
        if self._is_cuda and comm.size() > 1 and settings.WATCHDOG_S >= 0:
            limit = settings.WATCHDOG_S or (2e-3 * self._allreducer.wait_limit_ms + 30.0)
            self._watchdog = StreamWatchdog(limit, self._on_stall)
        self._post_clip: Optional[ClipNorm] = None
        self._post_coef: Optional[torch.Tensor] = None
        self._hook_handles = []
        self._membership = Membership.for_default_group(check_every=membership_check_every) \
            if membership_check_every else None
        self._register_hooks()
        uniform = all(all(pg.get(k, 0) == self.param_groups[0].get(k, 0)
                          for k in ("lr", "momentum", "dampening", "weight_decay", "nesterov"))
                      for pg in self.param_groups)
        if not uniform:
            raise ValueError("the fused step needs the same hyper-parameters in every param group")

    # -- watchdog --------------------------------------------------------------
    @property
    def capturing(self) -> bool:
        return self._capturing

    @capturing.setter
    def capturing(self, value: bool) -> None:
        """Set around CUDA-graph capture of an iteration; the watchdog thread
        makes no CUDA call meanwhile."""
        self._capturing = bool(value)
        if self._watchdog is not None:
            (self._watchdog.pause if value else self._watchdog.resume)()

    def _on_stall(self, seconds: float) -> None:
        """Runs on the watchdog thread: only logs and leaves a note; err_handler
        (which may rebuild the trainer's data loaders) is called from the
        training thread, in pre_iteration()."""
        msg = "device work of iteration %d still running after %.0f s" % (self._allreducer.train_iter, seconds)
        logger.error("watchdog: %s", msg)
        self._stalled = msg

    def post_iteration(self) -> None:
        """Everything of an iteration has been enqueued: hand the watchdog an
        event behind it."""
        if self._watchdog is None or self._capturing:
            return
        # an event behind every iteration costs more than it is worth on short steps (measured: 0.15 ms of a
        # 1.8 ms ResNet-20 step on two GPUs); the limits it guards are tens of seconds, so two a second do
        now = time.monotonic()
        if now - self._watchdog_armed_at < 0.5:
            return
        self._watchdog_armed_at = now
        ev = torch.cuda.Event()
        ev.record()
        self._watchdog.arm(ev)

    # -- hooks -----------------------------------------------------------------
    def _register_hooks(self):
        for name, slot in self._flat.slots.items():
            self._hook_handles.append(slot.param.register_post_accumulate_grad_hook(self._make_hook(slot)))

    def _make_hook(self, slot):
        gi = slot.group

        def hook(p):
            if self.local:
                return
            if p.grad is None or p.grad.data_ptr() != self._flat.grad.data_ptr() + 4 * slot.offset:
                self._flat.ensure_views()
            self._arrived[gi] += 1
            if self._arrived[gi] == self._expected[gi] and not self._launched[gi]:
                self._launch_group(gi)
        return hook

    def _apply_momentum_correction(self, gi: int) -> None:
        """Optional (off by default, distributed_optimizer.py:81-88): the
        velocity, not the raw gradient, is what gets sparsified.  One launch
        over the merged group once its last gradient is there (the reference
        updates parameter by parameter inside the hook; the result is the same).
        The factor is the wrapped optimizer's momentum, 0.9 if it has none."""
        eng = self._allreducer.engines[gi]
        fb = self._flat
        m = float(self.param_groups[0].get("momentum", 0.0)) or 0.9
        momentum_correct(fb.group_slice(fb.momentum, eng.g), eng.grad, m)

    def _launch_group(self, gi: int) -> None:
        self._launched[gi] = True
        if self._comm_stream is not None and self._overlap:
            ev = torch.cuda.Event()
            ev.record()
            self._comm_stream.wait_event(ev)
            with torch.cuda.stream(self._comm_stream):
                if self.momentum_correction:
                    self._apply_momentum_correction(gi)
                self._allreducer.reduce_group(gi)
        else:
            if self.momentum_correction:
                self._apply_momentum_correction(gi)
            self._allreducer.reduce_group(gi)

    # -- public API ---------------------------------------------------------------
    def pre_iteration(self) -> None:
        """Host-side look at the job's membership before anything of the next
        iteration is launched.  If a peer has left, the trainer's ``err_handler``
        is told the new world size and GTopkTimeout is raised here, on the host,
        instead of a device-side wait running out later."""
        if self._stalled is not None and not self.capturing:
            msg, self._stalled = self._stalled, None
            self._allreducer.report_failure(msg)
            raise ar.GTopkTimeout(msg)
        if not self.capturing:
            self._allreducer.poll_failure()  # status of the exchanges already completed; no synchronisation
        m = self._membership
        if m is None or self.capturing:
            return
        try:
            m.check(self._allreducer.train_iter)
        except PeerLeft as exc:
            if self.elastic and exc.planned:
                self._shrink(exc.ranks)
                return
            a = self._allreducer
            a._failed = str(exc)
            logger.error("membership: %s", exc)
            try:
                a._err_callback(max(a.size() - len(exc.ranks), 1), a.rank())
            except Exception:
                logger.exception("err_callback raised")
            raise ar.GTopkTimeout(str(exc)) from exc

    def epoch_barrier(self) -> None:
        """Host-side meeting point at an epoch boundary.  Only rank 0 validates and
        saves there (dl_trainer.py:606-625 in the reference, where the others then
        block in MPI without a limit); here every device-side wait of the next
        exchange is bounded, so the other ranks must not launch it before rank 0 is
        back.  The barrier runs on the CPU group, whose time limit is that of the
        job set-up (half an hour by default), not the exchange's.  Heartbeats are
        renewed on both sides of a second barrier, so nobody looks stale for having
        waited."""
        if self._allreducer.size() < 2 or self.capturing:
            return
        comm.barrier()
        m = self._membership
        if m is not None and m.store is not None:
            m.beat(self._allreducer.train_iter)
            comm.barrier()

    # -- elastic: planned departures ------------------------------------------------
    def request_leave(self) -> Optional[int]:
        """This rank wants to leave (a pre-emption notice, a drained node).  It
        announces the iteration from which it no longer takes part and must
        keep training until ``should_exit()`` turns true.  Returns that
        iteration, or None when there is nobody to tell."""
        if self._membership is None:
            self.leave_at = self._allreducer.train_iter
            return self.leave_at
        if self.leave_at is None:
            self.leave_at = self._membership.announce_leave(self._allreducer.train_iter)
            logger.info("leaving the job before iteration %d", self.leave_at)
        return self.leave_at

    def should_exit(self) -> bool:
        return self.leave_at is not None and self._allreducer.train_iter >= self.leave_at

    def _shrink(self, gone) -> None:
        """Every survivor arrives here at the same iteration, before launching
        anything of it: re-form the process group without the departed ranks,
        rebuild the exchange for the new world and tell the trainer, which
        re-shards its data (err_handler(new_size, new_rank))."""
        a = self._allreducer
        old_world = a.size()
        survivors = [r for r in range(old_world) if r not in set(gone)]
        if self._is_cuda:
            torch.cuda.synchronize()
        if self._watchdog is not None:
            self._watchdog.disarm()
        for e in a.engines:  # peer mappings of the old world go first, while every mapped buffer still exists
            region = getattr(e, "region", None)
            if region is not None:
                region.close()
                e.region = None
        new_rank, new_world = comm.reform(survivors)
        if new_world == 1 and self._watchdog is not None:  # nobody left to wait for
            self._watchdog.stop()
            self._watchdog = None
        a.rebuild()
        self._membership = Membership.for_default_group(check_every=self._membership_check_every) \
            if self._membership_check_every else None
        self.generation += 1
        logger.warning("ranks %s left: continuing with %d workers as rank %d (%s)", list(gone), new_world, new_rank,
                       a.mode)
        try:
            a._err_callback(new_world, new_rank)
        except Exception:
            logger.exception("err_callback raised")

    def zero_grad(self, set_to_none: bool = False):
        """Clears the flat gradient buffer with one fill; ``p.grad`` stay views."""
        self.pre_iteration()
        self._flat.zero_grad()
        self._materialized = False

    def synchronize(self, materialize: bool = False):
        """Wait (on the stream, not on the host) until every group of this
        iteration has been reduced.  With ``materialize=True`` the dense
        averaged gradient is also written into ``p.grad`` for callers that
        want to look at it (the fused step does not need it)."""
        if not self._synced:
            for gi in range(len(self._launched)):
                if not self._launched[gi]:  # parameters that got no gradient this iteration
                    self._launch_group(gi)
            if self._comm_stream is not None and self._overlap:
                torch.cuda.current_stream().wait_stream(self._comm_stream)
            self._synced = True
        if materialize and not self._materialized and self._allreducer.mode != "none":
            for eng in self._allreducer.engines:
                r = eng.result
                scatter_dense(eng.grad, r.pairs, r.counts, r.nseg, r.seg_stride, r.scale, r.use_atomics,
                              r.parity_word, r.parity_stride)
            self._materialized = True

    def clip_grad_norm(self, max_norm: float) -> torch.Tensor:
        """Device-side ``clip_grad_norm_`` on the reduced gradient
        (gtopk_trainer.py:81-86): the coefficient is computed from the global
        pairs and applied inside the fused step.  Returns the device scalar."""
        self.synchronize()
        dev = self._flat.device
        if self._post_clip is None:
            self._post_clip = ClipNorm(dev)
        a = self._allreducer
        if a.mode == "none":
            for eng in a.engines:
                self._post_clip.add_dense(eng.grad)
            self._post_coef = self._post_clip.finalize(max_norm, scale=1.0 / a.size())
        elif any(e.result.use_atomics for e in a.engines):
            self.synchronize(materialize=True)
            for eng in a.engines:
                self._post_clip.add_dense(eng.grad)
            self._post_coef = self._post_clip.finalize(max_norm, scale=1.0)
        else:
            scale = 1.0
            for eng in a.engines:
                r = eng.result
                self._post_clip.add_pairs(r.pairs, r.counts, r.nseg, r.seg_stride, r.parity_word, r.parity_stride)
                scale = r.scale
            self._post_coef = self._post_clip.finalize(max_norm, scale=scale)
        return self._post_coef

    def sync_lr(self) -> None:
        """Copy the host learning rate to the device scalar if it changed
        (never called while a graph is being captured)."""
        lr = float(self.param_groups[0]["lr"])
        if lr != self._lr_host and not self.capturing:
            self._lr_dev.fill_(lr)
            self._lr_host = lr

    def _hyper(self) -> SgdHyper:
        g = self.param_groups[0]
        return SgdHyper(lr=float(g["lr"]), momentum=float(g.get("momentum", 0.0)),
                        dampening=float(g.get("dampening", 0.0)), weight_decay=float(g.get("weight_decay", 0.0)),
                        nesterov=bool(g.get("nesterov", False)))

    def _step(self, closure=None):
        """Fused update over the flat buffers.  In the sparse modes the dense
        part (weight decay + momentum decay) does not depend on the exchange, so
        it is enqueued before the compute stream waits for the side stream: it
        runs while the exchange kernel is still waiting on its peers."""
        loss = closure() if closure is not None else None
        self.sync_lr()
        h = self._hyper()
        lr_dev = self._lr_dev
        first = self._step_count == 0
        fb, a = self._flat, self._allreducer
        use_buf = h.momentum != 0 and not self.momentum_correction
        if self.momentum_correction:
            h = SgdHyper(h.lr, 0.0, 0.0, h.weight_decay, False)

        def bufs(eng):
            return (fb.group_slice(fb.param, eng.g), fb.group_slice(fb.momentum, eng.g) if use_buf else None)

        if self.local:
            # accumulation micro-step: plain local SGD on the raw gradient
            for eng in a.engines:
                p, buf = bufs(eng)
                sgd_dense(p, buf, h, first, g=eng.grad, scale=1.0, lr_dev=lr_dev)
        elif a.mode == "none" or self._materialized:
            self.synchronize()
            scale = 1.0 / a.size() if a.mode == "none" else 1.0
            for eng in a.engines:
                p, buf = bufs(eng)
                sgd_dense(p, buf, h, first, g=eng.grad, scale=scale, coef=self._post_coef, lr_dev=lr_dev)
        else:
            for eng in a.engines:
                if eng.select_done is not None and self._is_cuda:
                    torch.cuda.current_stream().wait_event(eng.select_done)  # select first, then dense || exchange
                p, buf = bufs(eng)
                sgd_dense(p, buf, h, first, lr_dev=lr_dev)
            self.synchronize()
            for eng in a.engines:
                p, buf = bufs(eng)
                r = eng.result
                sgd_sparse(p, buf, r.pairs, r.counts, r.nseg, r.seg_stride, h, first, r.scale, coef=self._post_coef,
                           use_atomics=r.use_atomics, lr_dev=lr_dev, parity_word=r.parity_word,
                           parity_stride=r.parity_stride)
        if use_buf and first:
            for name, slot in fb.slots.items():
                self.state[slot.param]["momentum_buffer"] = fb.momentum_view(name)
        self._step_count += 1
        self._post_coef = None
        return loss

    def step(self, closure=None):
        ret = self._step(closure)
        self._synced = False
        self._arrived = [0] * len(self._arrived)
        self._launched = [False] * len(self._launched)
        a = self._allreducer
        a.train_iter += 1
        a.maybe_print_profiling()
        self.post_iteration()
        return ret

    def check_status(self):
        """Raise GTopkTimeout if a device-side wait of the last exchange ran
        out (synchronises).  Cheap enough for every N-th iteration."""
        self._allreducer.check_status()

    def stop(self):
        if self._watchdog is not None:
            self._watchdog.stop()
            self._watchdog = None
        if self._membership is not None:
            self._membership.leave()
        self._allreducer.stop()
        for h in self._hook_handles:
            h.remove()
        self._hook_handles = []

    def add_train_epoch(self):
        self._allreducer.train_epoch += 1

    def get_current_density(self):
        return self._allreducer.get_current_density()

    # -- checkpoint helpers ------------------------------------------------------
    def residual_state(self):
        """Residuals by parameter name (the reference never saves them)."""
        return {n: self._flat.residual_view(n).clone() for n in self._flat.slots}

    def load_residual_state(self, state):
        for n, t in state.items():
            if n in self._flat.slots:
                self._flat.residual_view(n).copy_(t)

    def load_momentum_state(self, state):
        """Velocity by parameter name (resuming a run): fills the flat momentum
        buffer and marks the first step as done, so that the next step decays
        the loaded velocity instead of re-initialising it with the gradient."""
        hit = 0
        with torch.no_grad():
            for n, t in state.items():
                if n in self._flat.slots and t is not None:
                    self._flat.momentum_view(n).copy_(t)
                    hit += 1
        if hit:
            self._step_count = max(self._step_count, 1)
            for name, slot in self._flat.slots.items():
                self.state[slot.param]["momentum_buffer"] = self._flat.momentum_view(name)
        return hit


def DistributedOptimizer(optimizer, named_parameters=None, compression=NoneCompressor, is_sparse=False,
                         err_handler=None, layerwise_times=None, sigma_scale=2.5, density=0.1, norm_clip=None,
                         writer=None, threshold=None, overlap=True, wait_limit_ms=None, membership_check_every=50,
                         elastic=False):
    """Wrap ``optimizer``.  The returned object is an instance of a subclass of
    ``type(optimizer)`` that carries the methods above."""
    cls = type(optimizer.__class__.__name__, (optimizer.__class__,), dict(_DistributedOptimizer.__dict__))
    return cls(optimizer.param_groups, named_parameters, compression, is_sparse, err_handler, layerwise_times,
               sigma_scale=sigma_scale, density=density, norm_clip=norm_clip, writer=writer, threshold=threshold,
               overlap=overlap, wait_limit_ms=wait_limit_ms, membership_check_every=membership_check_every,
               elastic=elastic)


def rank():
    return comm.rank()


def size(*_ignored):
    return comm.size()
