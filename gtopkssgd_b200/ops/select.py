"""K1 wrapper: fused residual add + top-k select + residual write-back.

``TopkSelector`` owns the device buffers of one merged gradient group (the
candidate list, the selected pairs, the persistent threshold state and the
control block) and enqueues the two K1 launches on the current stream.  On CPU
tensors it runs the PyTorch oracle instead, with the same outputs.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import torch

from . import lib as _lib
from . import oracle


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def current_stream_handle(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class TopkSelector:
    """Per-group selection state.

    Pairs are stored as an int32 tensor of shape [n, 2]: column 0 is the index,
    column 1 holds the fp32 value bits.
    """

    def __init__(self, numel: int, max_k: int, device: torch.device, target_ratio: float = 3.0,
                 cap_factor: int = 32, limit_ms: float = 2000.0):
        if numel >= 2 ** 31:
            raise ValueError("a merged group must have fewer than 2^31 elements")
        self.numel = int(numel)
        self.max_k = int(min(max_k, numel))
        self.device = torch.device(device)
        self.target_ratio = float(target_ratio)
        self.limit_ns = int(limit_ms * 1e6)
        self.cap = int(max(self.max_k, min(self.numel, max(cap_factor * self.max_k, 4096))))
        self.is_cuda = self.device.type == "cuda"
        self.sel = torch.zeros((self.max_k, 2), dtype=torch.int32, device=self.device)
        self.state = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.reset_threshold()
        if self.is_cuda:
            L = _lib.lib()
            assert L.gtk_k1state_bytes() == 32
            self.cand = torch.empty((self.cap, 2), dtype=torch.int32, device=self.device)
            # two control blocks: call i uses block i & 1 and clears the other one for call i + 1
            self.ctrl_words = int(L.gtk_ctrl_bytes()) // 4
            self.ctrl = torch.zeros(2 * self.ctrl_words, dtype=torch.int32, device=self.device)
        self.last_k = 0

    # -- state ---------------------------------------------------------------
    def reset_threshold(self) -> None:
        """Forget the predicted threshold: the next call takes the exact path."""
        self.state.view(torch.float32)[0] = math.inf

    @property
    def n_sel_tensor(self) -> torch.Tensor:
        """Device word holding the number of selected pairs of the last call."""
        return self.state[1:2]

    def stats(self) -> dict:
        """Host copy of the selection statistics (synchronises)."""
        s = self.state.cpu()
        f = s.view(torch.float32)
        return {"tau": float(f[0]), "n_sel": int(s[1]), "n_cand": int(s[2]), "fallback": int(s[3]),
                "n_fallbacks": int(s[4]), "n_calls": int(s[5]), "kth_mag": float(f[6])}

    def status(self) -> Tuple[int, int]:
        """(status, code location) of the last failure in either control block,
        (0, 0) if none.  Synchronises."""
        if not self.is_cuda:
            return (0, 0)
        for b in (0, 1):
            c = self.ctrl[b * self.ctrl_words:b * self.ctrl_words + 8].cpu()
            if int(c[_lib.CTRL_STATUS]):
                return int(c[_lib.CTRL_STATUS]), int(c[_lib.CTRL_WHERE])
        return (0, 0)

    def trace(self) -> dict:
        """Device-side phase stamps of the last select, in nanoseconds since its
        start: slot 1 = CTA 0 finished its share of the stream pass, 2 = every CTA
        did (grid barrier passed), 3 = k-th magnitude known, 4 = winners compacted
        (3 and 4 only on the predicted-threshold path).  Synchronises."""
        if not self.is_cuda:
            return {}
        calls = int(self.state[5].item())
        b = (calls - 1) & 1
        return _lib.read_trace(self.ctrl[b * self.ctrl_words:(b + 1) * self.ctrl_words])

    def reset(self) -> None:
        """Back to the initial state (after a reported failure)."""
        if self.is_cuda:
            self.ctrl.zero_()
        self.state.zero_()
        self.reset_threshold()

    # -- the op ----------------------------------------------------------------
    def select(self, g: torch.Tensor, r: torch.Tensor, k: int, g_scale: Optional[torch.Tensor] = None) -> None:
        """acc = g*scale + r; self.sel[:k] <- the k largest-magnitude (idx, acc)
        pairs; r <- acc off the selection, 0 on it.  g is not modified."""
        assert g.numel() == self.numel and r.numel() == self.numel
        assert g.dtype == torch.float32 and r.dtype == torch.float32
        k = int(min(k, self.max_k))
        self.last_k = k
        if not self.is_cuda:
            scale = float(g_scale) if g_scale is not None else 1.0
            idx, val = oracle.compress(g.view(-1), r.view(-1), k, scale)
            self.sel[:k, 0] = idx.to(torch.int32)
            self.sel[:k, 1] = val.view(torch.int32)
            self.state[1] = k
            return
        assert g.is_contiguous() and r.is_contiguous()
        L = _lib.lib()
        code = L.gtk_k1_select(g.data_ptr(), r.data_ptr(), _ptr(g_scale), self.numel, k, self.cand.data_ptr(),
                               self.cap, self.sel.data_ptr(), self.state.data_ptr(), self.ctrl.data_ptr(),
                               C.c_float(self.target_ratio), self.limit_ns, current_stream_handle(self.device))
        _lib.check(code, "gtk_k1_select")

    def pairs(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(int64 indices, fp32 values) of the last selection (synchronises)."""
        n = int(self.state[1].item())
        p = self.sel[:n]
        return p[:, 0].to(torch.int64), p[:, 1].contiguous().view(torch.float32)


def pairs_to_tensors(pairs: torch.Tensor, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
    p = pairs[:n]
    return p[:, 0].to(torch.int64), p[:, 1].contiguous().view(torch.float32)


def tensors_to_pairs(idx: torch.Tensor, val: torch.Tensor, out: torch.Tensor) -> int:
    n = idx.numel()
    out[:n, 0] = idx.to(torch.int32)
    out[:n, 1] = val.to(torch.float32).view(torch.int32)
    return n
