"""Whole-iteration CUDA graph: zero_grad + forward + backward + fused select +
exchange + fused SGD step captured once and replayed, for models whose
iteration is bound by kernel-launch overhead (on B200: ResNet-20 2.4x,
ResNet-110 1.6x, VGG-16 1.1x for forward+backward alone).

Everything that varies between iterations is read from device memory, so the
captured launches stay valid: the batch is copied into static tensors, the
learning rate lives in a device scalar, the exchange kernels keep their call
counter (flag epoch, slot parity) in a device word, clip coefficients and
selection thresholds are device-resident already.  The graph is re-captured
when something structural changes (k after the density schedule moves, batch
shape).  The reference has no counterpart: it synchronises the device in every
parameter hook (distributed_optimizer.py:90).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..models.lstm import repackage_hidden
from ..ops import lib as _native


class GraphedStep:
    def __init__(self, trainer, clip_norm: Optional[float] = None, warmup: int = 3):
        self.t = trainer
        self.clip_norm = clip_norm
        self.warmup = warmup
        self.eager_done = 0
        self._generation = getattr(trainer.optimizer, "generation", 0)
        self.graphs: Dict[Tuple, torch.cuda.CUDAGraph] = {}
        self.static: Dict[Tuple, dict] = {}
        self.pool = None

    # -- one eager iteration (also what gets captured) --------------------------------------------
    def _iteration(self, x, y, hidden):
        t = self.t
        opt = t.optimizer
        opt.zero_grad()
        if t.dnn == "lstm":
            outputs, hidden = t.net(x, hidden)
            loss = t.criterion(outputs.view(-1, t.net.vocab_size), y.reshape(-1))
        else:
            outputs = t.net(x)
            loss = t.criterion(outputs, y)
        loss.backward()
        if self.clip_norm is not None and hasattr(opt, "clip_grad_norm"):
            opt.clip_grad_norm(self.clip_norm)
        opt.step()
        acc = None
        if t.dnn not in ("lstm", "lstman4"):
            acc = t.cal_accuracy(outputs.detach(), y, topk=(1,))[0]
        # nothing returned may keep the autograd graph alive: gradient accumulators that survive an
        # iteration remember the stream they were created on, which breaks a later capture
        if hidden is not None:
            hidden = repackage_hidden(hidden)
        return loss.detach(), acc, hidden

    def _signature(self, x, y) -> Tuple:
        opt = self.t.optimizer
        ks = ()
        a = getattr(opt, "_allreducer", None)
        if a is not None and a.mode != "none":
            from ..ops.oracle import num_selected
            ks = tuple(min(num_selected(e.param_numel, a.get_current_density()), e.max_k) for e in a.engines)
        return (tuple(x.shape), tuple(y.shape), ks, bool(getattr(opt, "_materialized", False)))

    def _capture(self, sig, x, y, hidden):
        t, opt = self.t, self.t.optimizer
        st = {"x": x.clone(), "y": y.clone(), "hidden": None}
        if hidden is not None:
            st["hidden"] = tuple(h.detach().clone() for h in hidden)
        a = getattr(opt, "_allreducer", None)
        if hasattr(opt, "sync_lr"):
            opt.sync_lr()
        if a is not None:
            a.timers.enabled = False  # timing events cannot be read back from inside a graph
        if hasattr(opt, "capturing"):
            opt.capturing = True
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        before = _native.launch_count()
        try:
            with torch.cuda.graph(g, pool=self.pool):
                loss, acc, new_hidden = self._iteration(st["x"], st["y"], st["hidden"])
                st["loss"], st["acc"] = loss, acc
                if new_hidden is not None:
                    for dst, src in zip(st["hidden"], new_hidden):
                        dst.copy_(src.detach())
        finally:
            if hasattr(opt, "capturing"):
                opt.capturing = False
        st["native_launches"] = _native.launch_count() - before  # kernels of the native library inside the graph
        _native.add_launches(-st["native_launches"])              # capture enqueued nothing yet
        if self.pool is None:
            self.pool = g.pool()
        self.graphs[sig], self.static[sig] = g, st
        return g, st

    def capturable(self) -> bool:
        """Dense multi-GPU training keeps NCCL collectives inside the iteration;
        capturing those needs the process group's asynchronous error handling
        switched off before it is created, so that case stays eager."""
        a = getattr(self.t.optimizer, "_allreducer", None)
        if a is None:
            return True
        if any(getattr(e, "staged", False) for e in a.engines):
            return False  # the staged transport reads the selection back on the host every iteration
        return not (a.mode == "none" and a.size() > 1)

    def run(self, x, y, hidden=None):
        """x, y: this iteration's batch on the device.  Returns (loss, acc, hidden)."""
        t, opt = self.t, self.t.optimizer
        if hasattr(opt, "pre_iteration"):
            opt.pre_iteration()  # a replay runs no Python of the iteration, so look at the membership here
        gen = getattr(opt, "generation", 0)
        if gen != self._generation:  # the process group was re-formed: captured graphs address the old exchange
            self.graphs.clear()
            self.static.clear()
            self.eager_done, self._generation = 0, gen
        if self.eager_done < self.warmup or not self.capturable():
            self.eager_done += 1
            if hidden is not None:
                hidden = repackage_hidden(hidden)
            return self._iteration(x, y, hidden)
        sig = self._signature(x, y)
        g, st = self.graphs.get(sig), self.static.get(sig)
        captured_now = False
        if g is None:
            g, st = self._capture(sig, x, y, hidden)
            captured_now = True  # capture does not execute: replay below does the work with the same inputs
        st["x"].copy_(x, non_blocking=True)
        st["y"].copy_(y, non_blocking=True)
        if hidden is not None and hidden is not st["hidden"] and not captured_now:
            for dst, src in zip(st["hidden"], hidden):
                if dst.data_ptr() != src.data_ptr():
                    dst.copy_(src.detach(), non_blocking=True)
        if hasattr(opt, "sync_lr"):
            opt.sync_lr()
        g.replay()
        if hasattr(opt, "post_iteration"):
            opt.post_iteration()
        _native.add_launches(st["native_launches"])
        a = getattr(opt, "_allreducer", None)
        if a is not None:
            a.train_iter += 1
        return st["loss"], st["acc"], st["hidden"]
