"""The reference's own sparse all-reduce, timed on the micro-benchmark grid.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        baseline/ref_allreduce_bench.py --sizes 1 4 16 64 138 --densities 0.001 0.01 --json out.json

Per (d, rho): an fp32 vector N(0, 1e-2) with a fresh seed per rank, zero residual.
One call is what the reference's communication thread does for a merged group
(``allreducer.py:541-570``), with the reference's own objects from
``baseline/_ref`` (unmodified; the stand-ins of ``baseline/shims`` carry its MPI
calls over gloo):

    TopKCompressor.compress(tensor, name, ratio=rho)        select_ms
    AllReducer._sparse_allreduce(...)  (D2H, gtopk_sparse_allreduce over host
        buffers, H2D, scatter, /P)  +  add_residuals(...)   exchange_ms

Host wall clock with a device synchronisation on both sides (the path blocks the
host anyway), mean over the timed calls, max over ranks.  Nothing of
``gtopkssgd_b200`` is imported.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import ref_arm  # noqa: E402  (import path set-up and the Python-2 dictionary only)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", type=float, nargs="*", default=[1, 4, 16, 64, 138], help="d in millions")
    ap.add_argument("--densities", type=float, nargs="*", default=[0.001, 0.01])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--json", type=str, default=None)
    args = ap.parse_args()
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    ref_arm._prepare_import_path()
    import numpy as np
    if not hasattr(np, "int"):
        np.int = int
    import torch
    import torch.distributed as dist
    from mpi4py import MPI
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")) % torch.cuda.device_count())
    MPI.ensure_process_group()
    rank, world = dist.get_rank(), dist.get_world_size()
    import settings as ref_settings
    ref_settings.logger.setLevel("WARNING")
    import allreducer as ref_ar
    from compression import compressors as ref_compressors
    assert os.path.abspath(ref_ar.__file__).startswith(ref_arm.REF)
    comp = ref_compressors["gtopk"]
    dev = torch.device("cuda", torch.cuda.current_device())

    def allmax(v):
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=MPI.ensure_process_group())
        return float(t.item())

    rows = []
    for m in args.sizes:
        d = int(m * 1e6)
        name = "w%d" % d
        param = torch.nn.Parameter(torch.zeros(d, device=dev), requires_grad=False)
        ar = ref_ar.AllReducer([(name, param)], None, None, comp, sparse=True, density=0.001)
        for attr in ("_allreduce_timers", "_compression_timers", "_merge_timers", "_demerge_timers", "_d2h_times",
                     "_h2d_times"):
            setattr(ar, attr, ref_arm.Py2Dict(getattr(ar, attr)))
        gen = torch.Generator(device=dev).manual_seed(1234 + rank)
        grad = torch.randn(d, device=dev, generator=gen) * 0.1
        for rho in args.densities:
            k = max(int(d * rho), 1)
            iters = args.iters if k < 500000 else 3
            sel_t, ex_t = [], []
            for it in range(iters + 1):           # call 0 is the warm-up (allocates the reference's caches)
                tensor = grad.clone()
                if name in comp.residuals:
                    comp.residuals[name].zero_()  # zero-initialised residual for every call, as the grid says
                MPI.COMM_WORLD.Barrier()
                torch.cuda.synchronize()
                t0 = time.time()
                new_tensor, ctx = comp.compress(tensor, name, sigma_scale=2.5, ratio=rho)
                selected = new_tensor[ctx]
                torch.cuda.synchronize()
                t1 = time.time()
                result, included, _ = ar._sparse_allreduce(name, new_tensor, selected, new_tensor.shape, topk_indexes=ctx)
                if included is not None:
                    comp.add_residuals(included, name)
                torch.cuda.synchronize()
                t2 = time.time()
                if it > 0:
                    sel_t.append(t1 - t0)
                    ex_t.append(t2 - t1)
            row = {"impl": "reference", "d": d, "rho": rho, "k": k, "P": world,
                   "select_ms": allmax(float(np.mean(sel_t)) * 1e3), "exchange_ms": allmax(float(np.mean(ex_t)) * 1e3)}
            row["total_ms"] = row["select_ms"] + row["exchange_ms"]
            rows.append(row)
            if rank == 0:
                os.write(real_stdout, (json.dumps(row) + "\n").encode())
        del ar, param, grad
        comp.residuals.pop(name, None)
        comp.zero_conditions.pop(name, None)
        comp.values.pop(name, None)
        comp.indexes.pop(name, None)
        torch.cuda.empty_cache()
    if args.json and rank == 0:
        with open(args.json, "w") as fh:
            json.dump({"when": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), "rows": rows}, fh, indent=1)
    MPI.COMM_WORLD.Barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    rc = main()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(rc)
