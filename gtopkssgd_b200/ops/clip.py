"""K4 wrapper: device-resident gradient-norm clipping coefficient.

``ClipNorm`` accumulates squared norms of dense vectors and/or sparse pair
lists on the device and turns them into ``coef = min(1, max_norm/(norm+1e-6))``
without a host round trip; K1 and K3 read ``coef`` from device memory.
Covers the reference's pre-compression clip (allreducer.py:531-538) and the
post-reduction ``clip_grad_norm_`` of the LSTM paths (gtopk_trainer.py:81-86).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import lib as _lib
from .select import current_stream_handle, pairs_to_tensors


class ClipNorm:
    def __init__(self, device: torch.device):
        self.device = torch.device(device)
        self.is_cuda = self.device.type == "cuda"
        # {double sumsq; float norm; float coef}
        self.state = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.coef = torch.ones(1, dtype=torch.float32, device=self.device)
        self._cpu_sumsq = 0.0
        if self.is_cuda:
            assert _lib.lib().gtk_clipstate_bytes() == 16

    def add_dense(self, x: torch.Tensor) -> None:
        if not self.is_cuda:
            self._cpu_sumsq += float(x.double().pow(2).sum())
            return
        code = _lib.lib().gtk_k4_sumsq_dense(x.data_ptr(), x.numel(), self.state.data_ptr(),
                                             current_stream_handle(self.device))
        _lib.check(code, "gtk_k4_sumsq_dense")

    def add_pairs(self, pairs: torch.Tensor, counts: torch.Tensor, nseg: int, seg_stride: int,
                  parity_word=None, parity_stride: int = 0) -> None:
        if not self.is_cuda:
            if parity_word is not None:
                pairs = pairs[((int(parity_word) - 1) & 1) * parity_stride:]
            for s in range(nseg):
                _, val = pairs_to_tensors(pairs[s * seg_stride:(s + 1) * seg_stride], int(counts[s]))
                self._cpu_sumsq += float(val.double().pow(2).sum())
            return
        code = _lib.lib().gtk_k4_sumsq_pairs(pairs.data_ptr(), counts.data_ptr(), nseg, seg_stride,
                                             self.state.data_ptr(),
                                             None if parity_word is None else parity_word.data_ptr(),
                                             int(parity_stride), current_stream_handle(self.device))
        _lib.check(code, "gtk_k4_sumsq_pairs")

    def finalize(self, max_norm: float, scale: float = 1.0) -> torch.Tensor:
        """coef <- min(1, max_norm / (scale*sqrt(sumsq) + 1e-6)); clears the
        accumulator.  Returns the device tensor holding coef."""
        if not self.is_cuda:
            norm = scale * self._cpu_sumsq ** 0.5
            c = max_norm / (norm + 1e-6)
            self.coef[0] = c if c < 1 else 1.0
            self.state.view(torch.float32)[2] = norm
            self._cpu_sumsq = 0.0
            return self.coef
        code = _lib.lib().gtk_k4_finalize(self.state.data_ptr(), C.c_float(scale), C.c_float(max_norm),
                                          self.coef.data_ptr(), current_stream_handle(self.device))
        _lib.check(code, "gtk_k4_finalize")
        return self.coef

    def last_norm(self) -> float:
        return float(self.state.view(torch.float32)[2].item())
