"""K2 / K2t wrappers: the sparse exchange over NVLink peer memory.

``SymmetricRegion``  a peer-visible device allocation per rank (receive slots,
                     all-gather slots, global-set buffer, flag words) plus the
                     addresses of every peer's copy.  Created either across
                     processes with CUDA IPC (one process per GPU) or inside
                     one process for P emulated ranks on one GPU (tests).
``ExchangeRank``     the per-rank work buffers and the device descriptor that
                     the exchange kernels read.
``launch_gtopk`` / ``launch_allgather``  enqueue one exchange on the current
                     stream for one rank (production) or for all emulated ranks
                     in a single cooperative launch.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch

from . import lib as _lib
from .select import TopkSelector, current_stream_handle

MAX_PEERS = 16
GUARD_BYTES = 256      # canary band before and after every symmetric region
GUARD_PATTERN = 0xA5


def symm_layout(kcap: int, with_allgather: bool) -> Tuple[int, int, int, int, int]:
    out = (C.c_ulonglong * 5)()
    _lib.lib().gtk_symm_layout(int(kcap), int(with_allgather), out)
    return tuple(int(v) for v in out)


class SymmetricRegion:
    """One rank's peer-visible buffer and the peers' mapped addresses."""

    def __init__(self, rank: int, world: int, nbytes: int, raw_ptr: int, raw_peer_ptrs: Sequence[int], device,
                 owner=None, ipc: bool = False):
        """``raw_ptr`` / ``raw_peer_ptrs`` address allocations of nbytes + 2 * GUARD_BYTES; the usable region
        starts GUARD_BYTES in.  Both guard bands of the local allocation are filled with a pattern that no
        kernel may touch; ``guards_intact()`` re-reads them (a peer or a local kernel that stored outside
        its slots shows up there instead of corrupting a neighbour silently)."""
        self.rank, self.world, self.nbytes = rank, world, nbytes
        self._raw_ptr = int(raw_ptr)
        self._raw_peers = [int(p) for p in raw_peer_ptrs]
        self.local_ptr = self._raw_ptr + GUARD_BYTES
        self.peer_ptrs = [p + GUARD_BYTES for p in self._raw_peers]
        self.device = torch.device(device)
        self._owner = owner  # keeps the torch tensor alive in the emulated case
        self._ipc = ipc
        self._closed = False
        for g in self._guard_views():
            g.fill_(GUARD_PATTERN)

    def _guard_views(self):
        return (bytes_view(self._raw_ptr, GUARD_BYTES, self.device),
                bytes_view(self.local_ptr + self.nbytes, GUARD_BYTES, self.device))

    def tensor(self) -> torch.Tensor:
        """uint8 view of the usable region (without the guard bands)."""
        return bytes_view(self.local_ptr, self.nbytes, self.device)

    def guards_intact(self) -> bool:
        """True when both canary bands still hold the pattern (synchronises)."""
        return all(bool((g == GUARD_PATTERN).all().item()) for g in self._guard_views())

    @classmethod
    def create_emulated(cls, world: int, nbytes: int, device: torch.device) -> List["SymmetricRegion"]:
        """P regions on one GPU; every 'peer' address is a local address."""
        bufs = [torch.zeros(nbytes + 2 * GUARD_BYTES, dtype=torch.uint8, device=device) for _ in range(world)]
        ptrs = [b.data_ptr() for b in bufs]
        return [cls(r, world, nbytes, ptrs[r], ptrs, device, owner=bufs[r]) for r in range(world)]

    @classmethod
    def create_ipc(cls, nbytes: int, group=None) -> "SymmetricRegion":
        """One region per process; handles are exchanged through the process
        group (set-up only) and every peer copy is mapped with CUDA IPC."""
        import torch.distributed as dist
        L = _lib.lib()
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        ptr = C.c_void_p()
        _lib.check(L.gtk_p2p_alloc(int(nbytes) + 2 * GUARD_BYTES, C.byref(ptr)), "gtk_p2p_alloc")
        hbytes = int(L.gtk_p2p_handle_bytes())
        hbuf = (C.c_char * hbytes)()
        _lib.check(L.gtk_p2p_export(ptr, hbuf), "gtk_p2p_export")
        handles: List[Optional[bytes]] = [None] * world
        dist.all_gather_object(handles, bytes(hbuf), group=group)
        peers = []
        for q in range(world):
            if q == rank:
                peers.append(ptr.value)
                continue
            out = C.c_void_p()
            src = (C.c_char * hbytes).from_buffer_copy(handles[q])
            _lib.check(L.gtk_p2p_import(src, C.byref(out)), "gtk_p2p_import")
            peers.append(out.value)
        dist.barrier(group=group)
        return cls(rank, world, nbytes, ptr.value, peers, torch.device("cuda", torch.cuda.current_device()), ipc=True)

    def close(self) -> None:
        if self._closed or not self._ipc:
            self._closed = True
            return
        L = _lib.lib()
        for q, p in enumerate(self._raw_peers):
            if q != self.rank:
                L.gtk_p2p_unmap(p)
        L.gtk_p2p_free(self._raw_ptr)
        self._closed = True


class ExchangeRank:
    """Work buffers + device descriptor of one rank for one gradient group."""

    def __init__(self, rank: int, world: int, numel: int, kcap: int, selector: TopkSelector, resid: torch.Tensor,
                 region: SymmetricRegion, with_allgather: bool = False, reselect: bool = False):
        L = _lib.lib()
        dev = resid.device
        self.rank, self.world, self.numel, self.kcap = rank, world, int(numel), int(kcap)
        self.selector, self.resid, self.region = selector, resid, region
        self.with_allgather = with_allgather
        self.work_cap = self.kcap * (world if reselect else 1)
        self.work0 = torch.empty((self.work_cap, 2), dtype=torch.int32, device=dev)
        self.work1 = torch.empty((self.kcap, 2), dtype=torch.int32, device=dev)
        self.map = torch.zeros(self.numel, dtype=torch.int32, device=dev)
        self.ctrl = torch.zeros(int(L.gtk_ctrl_bytes()) // 4, dtype=torch.int32, device=dev)
        self.n_global = torch.zeros(1, dtype=torch.int32, device=dev)
        self.seg_counts = torch.zeros(MAX_PEERS, dtype=torch.int32, device=dev)
        # call counter of this rank's exchanges: the kernel reads it at entry (flag epoch, slot parity)
        # and adds one at exit, so launches carry no per-call argument and can be replayed from a graph
        self.epoch = torch.ones(1, dtype=torch.int32, device=dev)
        lay = symm_layout(self.kcap, with_allgather)
        assert lay[4] <= region.nbytes, "symmetric region too small"
        self.layout = lay
        nb = int(L.gtk_k2rank_bytes())
        host = (C.c_char * nb)()
        peers = (C.c_void_p * MAX_PEERS)(*([C.c_void_p(p) for p in region.peer_ptrs] +
                                           [C.c_void_p(0)] * (MAX_PEERS - world)))
        _lib.check(L.gtk_k2rank_fill(host, selector.sel.data_ptr(), selector.state.data_ptr(), self.work0.data_ptr(),
                                     self.work1.data_ptr(), self.map.data_ptr(), resid.data_ptr(), region.local_ptr,
                                     self.ctrl.data_ptr(), self.n_global.data_ptr(), self.epoch.data_ptr(), self.kcap,
                                     int(with_allgather), world, peers), "gtk_k2rank_fill")
        self.desc_host = bytes(host)
        self.desc = torch.frombuffer(bytearray(self.desc_host), dtype=torch.uint8).to(dev)

    def gout_ptr(self, parity: int) -> int:
        return self.region.local_ptr + self.layout[2] + parity * self.kcap * 8

    def ag_ptr(self, parity: int) -> int:
        return self.region.local_ptr + self.layout[1] + parity * MAX_PEERS * self.kcap * 8

    def status(self) -> Tuple[int, int]:
        c = self.ctrl[:8].cpu()
        return int(c[_lib.CTRL_STATUS]), int(c[_lib.CTRL_WHERE])

    def last_parity(self) -> int:
        """Parity of the slot set the last completed exchange wrote (synchronises)."""
        return (int(self.epoch.item()) - 1) & 1

    @property
    def parity_stride(self) -> int:
        return self.kcap

    @property
    def ag_parity_stride(self) -> int:
        return MAX_PEERS * self.kcap


def _desc_array(ranks: Sequence[ExchangeRank]) -> torch.Tensor:
    if len(ranks) == 1:
        return ranks[0].desc
    return torch.cat([r.desc for r in ranks])


def default_nctas(k: int, nranks: int = 1, sms: int = 148) -> int:
    """CTAs per rank for the exchange kernels, from sweeps on B200 (in-kernel
    time of one tree round + broadcast + put-back):

    * up to 3 K union entries: one CTA (no inter-CTA barrier, histograms stay in
      shared memory; about 10 us per round);
    * up to 32 K union entries: a power-of-two cluster of 2..16 CTAs joined by
      the hardware cluster barrier, about 1024 entries per CTA (k = 4 000: 19 us
      against 25 us with the software barrier; k = 14 700: 23 us against 27 us);
    * above: one CTA per 768 entries (up to 128) with the software barrier
      (k = 25 600: 26 us with 64 CTAs against 33 us with a cluster of 16)."""
    n_u = 2 * k
    if n_u <= 3072:
        return 1
    if n_u <= 32768:
        n = 2
        while n < 16 and n * 1024 < n_u:
            n *= 2
        return n
    n = min(128, (n_u + 767) // 768)
    return max(1, min(n, sms // max(nranks, 1)))


def launch_gtopk(ranks: Sequence[ExchangeRank], desc: torch.Tensor, rank_base: int, world: int, k: int,
                 nctas: Optional[int] = None, limit_ms: float = 5000.0, use_cluster: bool = True) -> None:
    """Enqueue one gTop-k exchange.  ``ranks`` are the ranks served by this
    launch (one in production, all P when emulated); ``desc`` is their
    concatenated device descriptor array."""
    L = _lib.lib()
    r0 = ranks[0]
    if nctas is None:
        nctas = default_nctas(k, len(ranks))
    ctrls = (C.c_void_p * len(ranks))(*[C.c_void_p(r.ctrl.data_ptr()) for r in ranks])
    code = L.gtk_k2_exchange(desc.data_ptr(), ctrls, len(ranks), rank_base, world, k, r0.kcap, r0.numel,
                             nctas, int(limit_ms * 1e6), int(use_cluster), current_stream_handle(r0.resid.device))
    _lib.check(code, "gtk_k2_exchange")


def launch_allgather(ranks: Sequence[ExchangeRank], desc: torch.Tensor, seg_counts: torch.Tensor, rank_base: int,
                     world: int, k: int, reselect: bool, nctas: Optional[int] = None,
                     limit_ms: float = 5000.0) -> None:
    """Enqueue one Top-k all-gather ('topk'), optionally followed by the global
    re-selection ('topk2').  ``seg_counts`` is an int32 device tensor of
    len(ranks) * 16 words receiving the per-source counts."""
    L = _lib.lib()
    r0 = ranks[0]
    if nctas is None:
        nctas = default_nctas(k * (world if reselect else 1) // 2 + 1, len(ranks))
    ctrls = (C.c_void_p * len(ranks))(*[C.c_void_p(r.ctrl.data_ptr()) for r in ranks])
    code = L.gtk_k2t_allgather(desc.data_ptr(), ctrls, len(ranks), rank_base, world, k, r0.kcap, r0.work_cap,
                               r0.numel, int(reselect), seg_counts.data_ptr(), nctas,
                               int(limit_ms * 1e6), current_stream_handle(r0.resid.device))
    _lib.check(code, "gtk_k2t_allgather")


def region_bytes(kcap: int, with_allgather: bool) -> int:
    return symm_layout(kcap, with_allgather)[4]


def bytes_view(ptr: int, n: int, device: torch.device) -> torch.Tensor:
    """uint8 [n] tensor over raw device memory."""

    class _Holder:
        __cuda_array_interface__ = {"shape": (n,), "typestr": "|u1", "data": (int(ptr), False), "version": 3,
                                    "strides": None}

    return torch.as_tensor(_Holder(), device=device)


def pairs_view(ptr: int, n: int, device: torch.device) -> torch.Tensor:
    """int32 [n, 2] tensor over raw device memory (used for IPC regions, which
    are not torch allocations)."""

    class _Holder:
        __cuda_array_interface__ = {"shape": (n, 2), "typestr": "<i4", "data": (int(ptr), False), "version": 3,
                                    "strides": None}

    return torch.as_tensor(_Holder(), device=device)
