"""Single-GPU kernel micro-benchmark: achieved bandwidth of K1/K3/K4 and the
latency of the emulated K2 exchange, timed with CUDA events after warm-up.

    python -m gtopkssgd_b200.bench_kernels [--sizes 16 64 138] [--densities 0.001 0.01] [--json out.json]

Each timed iteration works on inputs larger than L2 (or L2 is flushed by
writing a 256 MiB buffer first when they are not).  A short bounded device-side
delay is queued in front of the first event, so that the host's launch work
(Python, ctypes, driver: about 10 us) overlaps it instead of being counted as
kernel time; in training these launches are queued behind backward in the same
way (``--no-prequeue`` times from an idle GPU instead).  Roofline bytes: K1 12*d,
K3 dense 16*d (8*d without momentum), K4 4*d.  Fractions are reported against
the measured copy bandwidth in MEASURED_PEAKS.json when that file is present.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch


def _peak_gbs() -> float:
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["hbm_gbs"])
    except Exception:
        return 6650.0


class _Timer:
    def __init__(self, flush: bool):
        self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None

    iters, warmup = 10, 3
    prequeue_cycles = 200_000  # about 100 us of bounded device-side spinning

    def time(self, fn, iters=None, warmup=None, setup=None):
        iters = iters or _Timer.iters
        warmup = _Timer.warmup if warmup is None else warmup
        for _ in range(warmup):
            if setup:
                setup()
            fn()
        torch.cuda.synchronize()
        out = []
        for _ in range(iters):
            if setup:
                setup()
            if self.flush_buf is not None:
                self.flush_buf.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if _Timer.prequeue_cycles:
                torch.cuda._sleep(_Timer.prequeue_cycles)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b) * 1e-3)
        return statistics.median(out), min(out)


def bench_k1(d: int, rho: float, peak: float, flush: bool):
    from .ops.select import TopkSelector
    dev = torch.device("cuda")
    k = max(int(d * rho), 1)
    sel = TopkSelector(d, k, dev)
    r = torch.zeros(d, device=dev)
    grads = [torch.randn(d, device=dev) * 0.1 for _ in range(2)]
    it = [0]

    def setup():
        r.zero_()

    def fn():
        sel.select(grads[it[0] & 1], r, k)
        it[0] += 1

    med, best = _Timer(flush).time(fn, setup=setup)
    st = sel.stats()
    gbs = 12.0 * d / med / 1e9
    # %globaltimer stamps of the last call (slot meanings: TopkSelector.trace)
    stamps = {str(s): v / 1e3 for s, v in sel.trace().items()}
    return {"kernel": "k1_select", "d": d, "rho": rho, "k": k, "ms": med * 1e3, "best_ms": best * 1e3,
            "GBps": gbs, "frac_of_measured_hbm": gbs / peak, "n_cand": st["n_cand"],
            "fallbacks": st["n_fallbacks"], "calls": st["n_calls"], "stamps_us": stamps}


def bench_k3(d: int, peak: float, flush: bool):
    from .ops.sgd import SgdHyper, sgd_dense, sgd_sparse
    dev = torch.device("cuda")
    p = torch.randn(d, device=dev)
    buf = torch.zeros(d, device=dev)
    h = SgdHyper(lr=0.1, momentum=0.9, weight_decay=1e-4)
    t = _Timer(flush)
    med, best = t.time(lambda: sgd_dense(p, buf, h, False))
    gbs = 16.0 * d / med / 1e9
    out = [{"kernel": "k3_dense", "d": d, "ms": med * 1e3, "best_ms": best * 1e3, "GBps": gbs,
            "frac_of_measured_hbm": gbs / peak}]
    k = max(int(d * 0.001), 1)
    pairs = torch.zeros((k, 2), dtype=torch.int32, device=dev)
    pairs[:, 0] = torch.randperm(d, device=dev)[:k].to(torch.int32)
    pairs[:, 1] = torch.randn(k, device=dev).view(torch.int32)
    counts = torch.tensor([k], dtype=torch.int32, device=dev)
    med, best = t.time(lambda: sgd_sparse(p, buf, pairs, counts, 1, k, h, False, 0.125))
    out.append({"kernel": "k3_sparse", "d": d, "k": k, "ms": med * 1e3, "best_ms": best * 1e3})
    return out


def bench_k4(d: int, peak: float, flush: bool):
    from .ops.clip import ClipNorm
    dev = torch.device("cuda")
    x = torch.randn(d, device=dev)
    c = ClipNorm(dev)

    def fn():
        c.add_dense(x)
        c.finalize(0.25)

    med, best = _Timer(flush).time(fn)
    gbs = 4.0 * d / med / 1e9
    return {"kernel": "k4_clip_norm", "d": d, "ms": med * 1e3, "best_ms": best * 1e3, "GBps": gbs,
            "frac_of_measured_hbm": gbs / peak}


def bench_k2_emulated(d: int, rho: float, world: int, nctas=None):
    """All P ranks on one GPU in one cooperative launch: measures the on-chip
    cost of the merge/re-select rounds without NVLink latency."""
    from .ops import exchange as ex
    from .ops.select import TopkSelector
    dev = torch.device("cuda")
    k = max(int(d * rho), 1)
    regions = ex.SymmetricRegion.create_emulated(world, ex.region_bytes(k, False), dev)
    ranks = []
    for r in range(world):
        sel = TopkSelector(d, k, dev)
        resid = torch.zeros(d, device=dev)
        ranks.append(ex.ExchangeRank(r, world, d, k, sel, resid, regions[r]))
    desc = torch.cat([r.desc for r in ranks])
    for r in ranks:
        g = torch.randn(d, device=dev) * 0.1
        r.selector.select(g, r.resid, k)
    def fn():
        ex.launch_gtopk(ranks, desc, 0, world, k, nctas=nctas)

    med, best = _Timer(False).time(fn, iters=2 * _Timer.iters)
    bad = [r.status() for r in ranks if r.status() != (0, 0)]
    # per-phase split of the last call from rank 0's and rank 1's %globaltimer stamps
    phases = {"rank%d" % r.rank: r.trace() for r in ranks[:2]}
    return {"kernel": "k2_gtopk_exchange(emulated)", "d": d, "rho": rho, "k": k, "P": world,
            "nctas": nctas or ex.default_nctas(k, world), "us": med * 1e6, "best_us": best * 1e6, "errors": bad,
            "phases_us": phases}


def bench_k2t_emulated(d: int, rho: float, world: int, reselect: bool):
    """The all-gather exchange ('topk', or 'topk2' with reselect) for P ranks
    emulated on one GPU in one cooperative launch."""
    from .ops import exchange as ex
    from .ops.select import TopkSelector
    dev = torch.device("cuda")
    k = max(int(d * rho), 1)
    regions = ex.SymmetricRegion.create_emulated(world, ex.region_bytes(k, True), dev)
    ranks = []
    for r in range(world):
        sel = TopkSelector(d, k, dev)
        resid = torch.zeros(d, device=dev)
        ranks.append(ex.ExchangeRank(r, world, d, k, sel, resid, regions[r], with_allgather=True, reselect=reselect))
        sel.select(torch.randn(d, device=dev) * 0.1, resid, k)
    desc = torch.cat([r.desc for r in ranks])
    seg_counts = torch.zeros(world * ex.MAX_PEERS, dtype=torch.int32, device=dev)

    def fn():
        ex.launch_allgather(ranks, desc, seg_counts, 0, world, k, reselect=reselect)

    med, best = _Timer(False).time(fn, iters=2 * _Timer.iters)
    bad = [r.status() for r in ranks if r.status() != (0, 0)]
    return {"kernel": "k2t_topk_allgather(emulated, %s)" % ("topk2" if reselect else "topk"), "d": d, "rho": rho,
            "k": k, "P": world, "us": med * 1e6, "best_us": best * 1e6, "errors": bad}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", type=float, nargs="*", default=[16, 64, 138], help="d in millions of elements")
    ap.add_argument("--densities", type=float, nargs="*", default=[0.001, 0.01])
    ap.add_argument("--k2-sizes", type=float, nargs="*", default=[0.27, 14.7, 25.6, 66])
    ap.add_argument("--worlds", type=int, nargs="*", default=[2, 4, 8])
    ap.add_argument("--json", type=str, default=None)
    ap.add_argument("--only", type=str, nargs="*", default=["k1", "k3", "k4", "k2"],
                    help="which kernels to run (a small selection keeps a profiler capture short)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-prequeue", action="store_true", help="time from an idle GPU (includes host launch latency)")
    args = ap.parse_args()
    _Timer.iters, _Timer.warmup = args.iters, args.warmup
    if args.no_prequeue:
        _Timer.prequeue_cycles = 0
    peak = _peak_gbs()
    rows = []
    for m in args.sizes:
        d = int(m * 1e6)
        flush = d * 4 < (160 << 20)
        if "k1" in args.only:
            for rho in args.densities:
                rows.append(bench_k1(d, rho, peak, flush))
                print(json.dumps(rows[-1]), flush=True)
        if "k3" in args.only:
            for row in bench_k3(d, peak, flush):
                rows.append(row)
                print(json.dumps(row), flush=True)
        if "k4" in args.only:
            rows.append(bench_k4(d, peak, flush))
            print(json.dumps(rows[-1]), flush=True)
        torch.cuda.empty_cache()
    for m in (args.k2_sizes if "k2" in args.only else []):
        d = int(m * 1e6)
        for world in args.worlds:
            rows.append(bench_k2_emulated(d, 0.001, world))
            print(json.dumps(rows[-1]), flush=True)
            torch.cuda.empty_cache()
    for m in (args.k2_sizes if "k2t" in args.only else []):
        d = int(m * 1e6)
        for world in args.worlds:
            for reselect in (False, True):
                rows.append(bench_k2t_emulated(d, 0.001, world, reselect))
                print(json.dumps(rows[-1]), flush=True)
                torch.cuda.empty_cache()
    if args.json:
        with open(args.json, "w") as fh:
            json.dump({"peak_hbm_gbs": peak, "rows": rows}, fh, indent=1)


if __name__ == "__main__":
    main()
