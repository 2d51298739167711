"""Sparse all-reduce micro-benchmark on P GPUs (one process per GPU).

    torchrun --nproc-per-node 8 -m gtopkssgd_b200.bench_allreduce \
        --sizes 1 4 16 64 138 --densities 0.001 0.01 --json out.json

For every (d, rho): fp32 vectors N(0, 1e-2) with a fresh seed per rank, zero
residual.  Timed per call on the device (CUDA events, max over ranks):
  ours_ms    K1 fused select + K2 persistent exchange (+ residual put-back)
  k1_ms/k2_ms the two parts separately
  *_chain_ms  K2 / the dense all-reduce per call over 20 calls back to back
             (steady state: no host barrier, hence no start skew, between calls);
             ours_steady_ms = k1_ms + k2_chain_ms
  k2_trace_us device-side phase stamps of one exchange on every rank
             (``ops.exchange.decode_k2_trace``): time in flag waits and in work
  dense_ms   NCCL all-reduce of the same d floats (the dense baseline)
  rehost_ms  the reference's algorithm re-hosted on today's PyTorch: torch.topk on the
             device, D2H of the k pairs, recursive-doubling tree over gloo
             send/recv with numpy merges on the host, H2D, scatter
             (the op sequence of allreducer.py:429-478 + 71-163; the unmodified
             reference cannot run here because mpi4py is absent)
Roofline of the exchange: 2*k*log2(P)*8 bytes over one NVLink direction.
With ``--prequeue`` a short bounded device-side delay is queued before the first
event of every timed call (all arms alike), so that host launch work overlaps
it, as it does in training where these launches sit behind backward.
"""
from __future__ import annotations

import argparse
import json
import math
import time

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0  # measured peer copy bandwidth per direction (NVLink 5 through NVSwitch, nominal 900)
PREQUEUE_CYCLES = 0  # set by --prequeue


def _timed(fn, iters, warmup, device, setup=None):
    from .parallel import comm
    for _ in range(warmup):
        if setup:
            setup()
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if setup:
            setup()
        comm.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if PREQUEUE_CYCLES:
            torch.cuda._sleep(PREQUEUE_CYCLES)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return comm.allreduce_max_float(total / iters, device)


def _timed_chain(fn, device, n=20, warmup=3, setup=None):
    """Steady-state time per call: n calls back to back on one stream between two events.  After the
    first call the ranks pace one another through the exchange itself, so the start skew that a host
    barrier leaves (tens of microseconds) is paid once, not once per call as in ``_timed``."""
    from .parallel import comm
    for _ in range(warmup):
        fn()
    if setup:
        setup()
    comm.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        fn()
    b.record()
    torch.cuda.synchronize()
    return comm.allreduce_max_float(a.elapsed_time(b) / n, device)


def _rehost_reference(g, resid, k, world, rank):
    """The reference's op sequence with today's PyTorch + gloo (host staged)."""
    from .ops import oracle
    from .parallel import comm, fallback
    acc = g + resid
    _, idx = torch.topk(acc.abs(), k)
    val = acc[idx]
    idx_h, val_h = idx.cpu(), val.cpu()                       # D2H (blocking)
    gi, gv = fallback.gtopk_allreduce(idx_h, val_h, k, group=comm.cpu_group())
    gi_d, gv_d = gi.to(g.device), gv.to(g.device)              # H2D
    out = torch.zeros_like(g)
    out[gi_d] = gv_d
    out /= world
    oracle.put_back(resid, (idx, val), gi_d)
    return out


def run_config(d, rho, iters=10, warmup=3, with_dense=True, with_rehost=True):
    from .ops import exchange as ex
    from .ops.select import TopkSelector
    from .parallel import comm
    if not torch.cuda.is_available():
        return None
    rank, world = comm.rank(), comm.size()
    dev = torch.device("cuda", torch.cuda.current_device())
    k = max(int(d * rho), 1)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    grads = [torch.randn(d, device=dev, generator=gen) * 0.1 for _ in range(2)]
    resid = torch.zeros(d, device=dev)
    sel = TopkSelector(d, k, dev)
    row = {"d": d, "rho": rho, "k": k, "P": world}
    it = [0]
    if world > 1:
        region = ex.SymmetricRegion.create_ipc(ex.region_bytes(k, False), group=comm.cpu_group())
        rc = ex.ExchangeRank(rank, world, d, k, sel, resid, region)
    def k1():
        sel.select(grads[it[0] & 1], resid, k)
        it[0] += 1

    def k2():
        ex.launch_gtopk([rc], rc.desc, rank, world, k, limit_ms=10000)

    def both():
        k1()
        if world > 1:
            k2()

    row["ours_ms"] = _timed(both, iters, warmup, dev, setup=resid.zero_)
    row["k1_ms"] = _timed(k1, iters, warmup, dev, setup=resid.zero_)
    if world > 1:
        row["k2_ms"] = _timed(k2, iters, warmup, dev)
        row["k2_chain_ms"] = _timed_chain(k2, dev)
        # K1 depends on no other rank, so its isolated time is its steady-state time; a chain of K1 + K2
        # calls would let the residual grow from call to call and time a different selection problem
        row["ours_steady_ms"] = row["k1_ms"] + row["k2_chain_ms"]
        # device-side phase stamps of one more call, from every rank
        k1()
        k2()
        torch.cuda.synchronize()
        traces = [None] * world
        dist.all_gather_object(traces, rc.trace(), group=comm.cpu_group())
        row["k2_trace_us"] = traces
        row["k2_in_kernel_us"] = max((t.get("total", 0.0) for t in traces), default=0.0)
        row["k2_work_us"] = max((t.get("work", 0.0) for t in traces), default=0.0)
        status = rc.status()
        row["status"] = list(status)
        rounds = int(math.log2(world))
        wire = 2.0 * k * rounds * 8
        row["nvlink_roofline_ms"] = wire / (NVLINK_GBS * 1e9) * 1e3
        row["k2_frac_of_nvlink_roofline"] = row["nvlink_roofline_ms"] / row["k2_chain_ms"]
    row["k1_hbm_roofline_ms"] = 12.0 * d / (6550.1e9) * 1e3
    st = sel.stats()
    row["k1_fallbacks"] = st["n_fallbacks"]
    if with_dense and world > 1:
        buf = grads[0].clone()
        row["dense_nccl_ms"] = _timed(lambda: dist.all_reduce(buf), iters, warmup, dev)
        row["dense_nccl_chain_ms"] = _timed_chain(lambda: dist.all_reduce(buf), dev)
    if with_rehost and world > 1 and (world & (world - 1)) == 0:
        r2 = torch.zeros(d, device=dev)
        row["rehost_ref_ms"] = _timed(lambda: _rehost_reference(grads[0], r2, k, world, rank), max(3, iters // 2), 1,
                                      dev, setup=r2.zero_)
    if world > 1:
        torch.cuda.synchronize()
        comm.barrier()
        region.close()
    return row


def main():
    from . import settings
    from .parallel import comm
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", type=float, nargs="*", default=[1, 4, 16, 64, 138], help="d in millions")
    ap.add_argument("--densities", type=float, nargs="*", default=[0.001, 0.01])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-rehost", action="store_true")
    ap.add_argument("--json", type=str, default=None)
    ap.add_argument("--prequeue", action="store_true",
                    help="queue a bounded ~100 us device-side delay before each timed call (hides host launch work)")
    args = ap.parse_args()
    global PREQUEUE_CYCLES
    PREQUEUE_CYCLES = 200_000 if args.prequeue else 0
    settings.logger.setLevel("WARNING")
    if torch.cuda.is_available():
        torch.cuda.set_device(comm.env_local_rank() % torch.cuda.device_count())
    comm.init()
    rows = []
    for m in args.sizes:
        for rho in args.densities:
            row = run_config(int(m * 1e6), rho, iters=args.iters, with_rehost=not args.no_rehost)
            rows.append(row)
            if comm.rank() == 0:
                print(json.dumps(row), flush=True)
            torch.cuda.empty_cache()
    if args.json and comm.rank() == 0:
        with open(args.json, "w") as fh:
            json.dump({"when": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), "rows": rows}, fh, indent=1)
    comm.shutdown()


if __name__ == "__main__":
    main()
