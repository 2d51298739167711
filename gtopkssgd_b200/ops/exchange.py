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
RES_COUNT, RES_STATUS, RES_WHERE, RES_EPOCH, RES_WORDS = 0, 1, 2, 3, 4   # K2Rank::n_global words (exchange_common.cuh)
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
        # two control blocks: the gTop-k kernel alternates between them and cleans the idle one itself
        self.ctrl_words = int(L.gtk_ctrl_bytes()) // 4
        self.ctrl = torch.zeros(2 * self.ctrl_words, dtype=torch.int32, device=dev)
        # result words of the last exchange: [count of global pairs, sticky status, where, failing call]
        self.result_words = torch.zeros(RES_WORDS, dtype=torch.int32, device=dev)
        self.n_global = self.result_words[0:1]
        # host mirror of the result words, refreshed by an asynchronous copy behind every exchange, so
        # that the host can look at the status before each iteration without synchronising
        self.result_host = torch.zeros(RES_WORDS, dtype=torch.int32)
        if dev.type == "cuda":
            self.result_host = self.result_host.pin_memory()
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
        """(status, code location) of the first failure, (0, 0) if none (synchronises)."""
        w = self.result_words.cpu()
        if int(w[RES_STATUS]) != 0:
            return int(w[RES_STATUS]), int(w[RES_WHERE])
        for b in range(2):
            c = self.ctrl[b * self.ctrl_words:b * self.ctrl_words + 8].cpu()
            if int(c[_lib.CTRL_STATUS]) != 0:
                return int(c[_lib.CTRL_STATUS]), int(c[_lib.CTRL_WHERE])
        return 0, 0

    def mirror_status(self) -> None:
        """Enqueue the copy of the result words to pinned host memory on the current stream."""
        self.result_host.copy_(self.result_words, non_blocking=True)

    def failed_on_host_mirror(self) -> Tuple[int, int]:
        """What the last completed mirror copy showed; never synchronises."""
        return int(self.result_host[RES_STATUS]), int(self.result_host[RES_WHERE])

    def clear_failure(self) -> None:
        """Forget a recorded failure so that the exchange runs again.  Every rank of
        the job has to do this at the same point, with nothing in flight (the call
        counter, which stamps the flags, was not advanced by the failed call)."""
        self.result_words.zero_()
        self.result_host.zero_()
        self.ctrl.zero_()

    def last_ctrl(self) -> torch.Tensor:
        """Control block that the last completed gTop-k call used (synchronises)."""
        b = (int(self.epoch.item()) - 1) & 1
        return self.ctrl[b * self.ctrl_words:(b + 1) * self.ctrl_words]

    def trace(self) -> dict:
        """Phase stamps of the last completed gTop-k call, decoded (``decode_k2_trace``)."""
        world = self.world
        return decode_k2_trace(_lib.read_trace(self.last_ctrl()), self.rank, world)

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
    code = L.gtk_k2_exchange(desc.data_ptr(), len(ranks), rank_base, world, k, r0.kcap, r0.numel,
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


def decode_k2_trace(tr: dict, rank: int, world: int) -> dict:
    """Turns the %globaltimer stamps that CTA 0 of a rank leaves in its control block
    (slot 0: start; 1 + 8r + j for tree round r: j = 0 before / 1 after the wait for the
    partner's flag, 2 table complete, 3 join done, 4 threshold known, 5 compaction done,
    6 pushed (round-0 sender), 7 flag raised; 40 global set here, 41 its table built,
    42 put-back done) into microseconds: ``total``, ``wait`` (time inside flag waits:
    partner or root not there yet), ``work`` = total - wait, and per-phase entries."""
    if 42 not in tr:
        return {"complete": False}
    us = lambda a, b: (tr[b] - tr[a]) / 1e3 if a in tr and b in tr else 0.0
    rounds = max(world.bit_length() - 1, 0)
    out = {"complete": True, "total": tr[42] / 1e3, "wait": 0.0, "rounds": []}
    last = 0
    for r in range(rounds):
        b = 1 + 8 * r
        row = {}
        if b + 1 in tr:  # receiver of round r
            row = {"role": "recv", "wait": us(b, b + 1), "table": us(b + 1, b + 2), "join": us(b + 2, b + 3),
                   "select": us(b + 3, b + 4), "compact": us(b + 4, b + 5)}
            out["wait"] += row["wait"]
            last = b + 5
        if b + 7 in tr:  # sent in round r (round 0: after a push; later: straight from the compaction)
            row = dict(row, sent=True) if row else {"role": "send", "push": us(last, b + 6) if b + 6 in tr else 0.0,
                                                     "flag": us(b + 6, b + 7) if b + 6 in tr else 0.0}
            last = b + 7
        out["rounds"].append(row)
    if rank != 0:
        w = us(last, 40)
        out["wait"] += w
        out["bcast_wait"] = w
    out["table_g"] = us(40, 41)
    out["put_back"] = us(41, 42)
    out["work"] = out["total"] - out["wait"]
    return out


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
