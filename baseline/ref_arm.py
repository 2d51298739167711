"""Reference arm of the headline benchmark: drives the UNMODIFIED reference
(hclhkbu/gtopkssgd, copied byte for byte into ``baseline/_ref/``) through its
own public API on the benchmark's configuration and prints one JSON line.

    python baseline/ref_arm.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29512 baseline/ref_arm.py --gpus 8 --steps 20 --warmup 5

What runs is the reference's code: ``dl_trainer.DLTrainer`` (its model zoo, its
``train()`` with the host-to-device copy and the ``loss.item()`` read), its
``distributed_optimizer.DistributedOptimizer`` with the per-parameter hooks and
the ``AllReducer`` thread, ``TopKCompressor.compress``,
``gtopk_sparse_allreduce`` and the hand-rolled SGD step
(``gtopk_trainer.py:26-127`` is the loop restated below, since that function
builds its own data loaders from files that do not exist here);
``--compressor none`` drives the dense path of ``horovod_trainer.py:22-68``.
Nothing of ``gtopkssgd_b200`` is imported in this process.

The reference is Python-2 era source.  It is not edited; three things of the
environment it was written for are put back before it is imported:

* ``numpy.int`` (removed in NumPy 1.24; ``allreducer.py:119``),
* Python 2's ``dict.keys()`` returning a list, for the three timer dictionaries
  that ``allreducer.py:335`` subscripts (set on the constructed object),
* the packages ``mpi4py``, ``horovod.torch``, ``tensorboardX`` and ``h5py``, as
  stand-ins under ``baseline/shims/`` over ``torch.distributed``.

Settings applied to the constructed objects, never to source: the density is
pinned (``_dynamic_densities``), the epoch length is set so that no epoch
boundary (validation pass over a test set that does not exist) falls into the
run, and TF32 is switched off as in the other arm.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SHIMS = os.path.join(HERE, "shims")
ROOT = os.path.dirname(HERE)

MODEL_DEFAULTS = {  # dataset, per-GPU batch, lr  (the named benchmark configurations)
    "resnet50": ("imagenet", 64, 0.1),
    "vgg16": ("cifar10", 128, 0.1),
    "resnet20": ("cifar10", 32, 0.1),
    "lstm": ("ptb", 20, 22.0),
    "alexnet": ("imagenet", 256, 0.01),
}


def _prepare_import_path():
    """The reference's flat modules (``settings``, ``utils``, ``allreducer`` ...) must win over any
    same-named module elsewhere: drop the repository root, put the reference and the stand-ins first."""
    drop = {ROOT, ""}
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or os.getcwd()) not in drop and p != ""]
    sys.path.insert(0, SHIMS)
    sys.path.insert(0, REF)


class Py2Dict(dict):
    """``keys()`` returns a list, as in the Python the reference was written for; entries removed with
    ``pop`` (the reference drops its timer lists after printing them) stay readable in ``archive``."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.archive = {}

    def keys(self):
        return list(super().keys())

    def pop(self, key, *default):
        if key in self:
            self.archive.setdefault(key, []).extend(self[key])
        return super().pop(key, *default)

    def all_values(self, key):
        return list(self.archive.get(key, [])) + list(self.get(key, []))


class ClockSampler:
    """SM clock and throttle reasons of one GPU, sampled by ``nvidia-smi`` in a child process."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0, period_ms=100):
        self.idx, self.period, self.proc = gpu_index, period_ms, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", str(self.period)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        if not out.strip():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q,
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=10).stdout
            except Exception:
                out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def _cpu_dry_run_patches(torch):
    """Plumbing check on a machine without a GPU: the reference hard-codes ``.cuda()`` and
    ``torch.cuda.synchronize()`` (``compression.py:70``, ``distributed_optimizer.py:90``), so both become
    no-ops.  Never used for a measurement."""
    torch.cuda.synchronize = lambda *a, **k: None
    torch.Tensor.cuda = lambda self, *a, **k: self
    torch.nn.Module.cuda = lambda self, *a, **k: self
    torch.cuda.manual_seed_all = lambda *a, **k: None
    torch.cuda.set_device = lambda *a, **k: None
    torch.cuda.empty_cache = lambda *a, **k: None
    for n in ("memory_allocated", "max_memory_allocated", "memory_cached", "max_memory_cached"):
        setattr(torch.cuda, n, lambda *a, **k: 0)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--model", type=str, default="resnet50", choices=sorted(MODEL_DEFAULTS))
    ap.add_argument("--batch-size", type=int, default=None)
    ap.add_argument("--density", type=float, default=0.001)
    ap.add_argument("--compressor", type=str, default="gtopk", choices=["gtopk", "topk", "topk2", "none"])
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--cpu-dry-run", action="store_true", help="plumbing check without a GPU; prints no measurement")
    args, _unknown = ap.parse_known_args(argv)   # flags that only the other arm knows are ignored
    if args.warmup < 3:
        args.warmup = 3
    if not os.path.isfile(os.path.join(REF, "allreducer.py")):
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is missing: run baseline/setup_ref.py "
                              "where the reference tree is mounted"}), flush=True)
        return 0

    # keep stdout for the one JSON line (the reference logs to stderr, NCCL banners may not)
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    sys.path.insert(0, HERE)
    import setup_ref
    source_ok = setup_ref.verify(REF)
    sys.path.pop(0)
    _prepare_import_path()
    import numpy as np
    if not hasattr(np, "int"):
        np.int = int
    import torch
    dry = args.cpu_dry_run
    if dry:
        _cpu_dry_run_patches(torch)
    elif not torch.cuda.is_available():
        os.write(real_stdout, (json.dumps({"impl": "reference", "error": "needs a CUDA device"}) + "\n").encode())
        return 1
    import torch.distributed as dist
    from mpi4py import MPI
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not dry:
        torch.cuda.set_device(local_rank % torch.cuda.device_count())
    MPI.ensure_process_group()
    rank, world = dist.get_rank(), dist.get_world_size()
    if world != args.gpus:
        if rank == 0:
            os.write(real_stdout, (json.dumps({"impl": "reference", "error": "--gpus %d but world size is %d"
                                               % (args.gpus, world)}) + "\n").encode())
        return 1

    # ---- the reference's own modules
    import settings as ref_settings
    ref_settings.logger.setLevel("WARNING")
    import dl_trainer as ref_dl
    import distributed_optimizer as ref_dopt
    from compression import compressors as ref_compressors
    import horovod.torch as hvd
    assert os.path.abspath(ref_dl.__file__).startswith(REF), ref_dl.__file__
    assert os.path.abspath(ref_dopt.__file__).startswith(REF), ref_dopt.__file__
    torch.backends.cudnn.allow_tf32 = False          # strict fp32 in both arms
    torch.backends.cuda.matmul.allow_tf32 = False
    hvd.init()

    dataset, bs, lr = MODEL_DEFAULTS[args.model]
    bs = args.batch_size or bs
    is_lstm = args.model == "lstm"
    ngpus = 0 if dry else 1
    if is_lstm:
        # DLTrainer takes a constructed network too (dl_trainer.py:131-134); the PTB vocabulary size would
        # otherwise come from the corpus files
        import models.lstm as ref_lstm
        net = ref_lstm.lstm(vocab_size=10000, batch_size=bs)
        net.name = "lstm"
        dnn = net
    else:
        dnn = args.model
    trainer = ref_dl.DLTrainer(rank, world, dist=False, batch_size=bs, is_weak_scaling=True, ngpus=ngpus,
                               data_dir=None, dataset=dataset, dnn=dnn, lr=lr, nworkers=world,
                               prefix="bench-ds%s" % str(args.density), pretrain=None, tb_writer=None)
    trainer.num_batches_per_epoch = 1 << 40      # no epoch boundary inside the run
    trainer.train_sampler = None
    hvd.broadcast_parameters(trainer.net.state_dict(), root_rank=0)
    sparse = args.compressor != "none"
    if sparse:   # gtopk_trainer.py:46-57
        optimizer = ref_dopt.DistributedOptimizer(trainer.optimizer, trainer.net.named_parameters(),
                                                  compression=ref_compressors[args.compressor], is_sparse=True,
                                                  err_handler=None, layerwise_times=None, sigma_scale=2.5,
                                                  density=args.density, norm_clip=None, writer=None)
        ar = optimizer._allreducer
        ar._dynamic_densities = [args.density]                  # pinned from the first step
        for name in ("_allreduce_timers", "_compression_timers", "_merge_timers", "_demerge_timers",
                     "_d2h_times", "_h2d_times"):
            setattr(ar, name, Py2Dict(getattr(ar, name)))
    else:        # horovod_trainer.py:34-35
        optimizer = hvd.DistributedOptimizer(trainer.optimizer, named_parameters=trainer.net.named_parameters())
        ar = None
    trainer.update_optimizer(optimizer)

    # ---- synthetic batches of the named shape, in pinned host memory and on the device
    g = torch.Generator().manual_seed(1234 + rank)
    def make_batch():
        if is_lstm:
            x = torch.randint(0, 10000, (bs, 35), generator=g)
            y = torch.randint(0, 10000, (bs, 35), generator=g)
        elif dataset == "imagenet":
            x = torch.randn(bs, 3, 224, 224, generator=g)
            y = torch.randint(0, 1000, (bs,), generator=g)
        else:
            x = torch.randn(bs, 3, 32, 32, generator=g)
            y = torch.randint(0, 10, (bs,), generator=g)
        return (x, y) if dry else (x.pin_memory(), y.pin_memory())
    host_batches = [make_batch() for _ in range(4)]
    h2d_bytes = sum(t.numel() * t.element_size() for t in host_batches[0])
    dev_batch = host_batches[0] if dry else tuple(t.cuda(non_blocking=True) for t in host_batches[0])
    state = {"hidden": trainer.net.init_hidden() if is_lstm else None, "i": 0}

    def iteration(data):
        # gtopk_trainer.py:69-88 / horovod_trainer.py:44-63 with nsteps_update = 1
        optimizer.zero_grad()
        optimizer.local = False
        if is_lstm:
            _, state["hidden"] = trainer.train(1, data=data, hidden=state["hidden"])
            optimizer.synchronize()
            torch.nn.utils.clip_grad_norm_(trainer.net.parameters(), 0.25)
        else:
            trainer.train(1, data=data)
        trainer.update_model()

    def device_step():
        iteration(dev_batch)

    def e2e_step():
        i = state["i"]
        state["i"] += 1
        iteration(host_batches[i % len(host_batches)])   # train() copies the batch to the GPU and reads loss.item()

    def sync():
        if not dry:
            torch.cuda.synchronize()

    def allmax(v):
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=MPI.ensure_process_group())
        return float(t.item())

    def timed(fn, steps):
        MPI.COMM_WORLD.Barrier()
        sync()
        t0 = time.time()
        if not dry:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        for _ in range(steps):
            fn()
        if not dry:
            b.record()
        sync()
        wall = time.time() - t0
        MPI.COMM_WORLD.Barrier()
        dev_s = a.elapsed_time(b) * 1e-3 if not dry else wall
        return allmax(dev_s), allmax(wall)

    def timer_means(skip):
        if ar is None:
            return {}
        out = {}
        for label, d in (("exchange_ms", ar._allreduce_timers), ("select_ms", ar._compression_timers),
                         ("d2h_ms", ar._d2h_times), ("h2d_scatter_ms", ar._h2d_times)):
            tot = 0.0
            for key in set(list(d.archive) + list(d.keys())):   # one key per merged group
                v = d.all_values(key)[skip:]
                if v:
                    tot += float(np.mean(v))
            out[label] = allmax(tot * 1e3)
        return out

    for _ in range(args.warmup):
        device_step()
    sync()
    n_before = args.warmup
    sampler = ClockSampler(gpu_index=local_rank, period_ms=100)
    if rank == 0 and not dry:
        sampler.start()
    dev_s, wall_s = timed(device_step, args.steps)
    clocks = sampler.stop() if (rank == 0 and not dry) else {}
    comm_ms = timer_means(n_before)
    if comm_ms:
        comm_ms["ranks"] = "max over %d" % world
        comm_ms["mode"] = "the reference's own host timers: exchange = _allreduce_timers (D2H + tree over the host " \
                          "transport + H2D + scatter + residual put-back), select = _compression_timers"

    e2e = None
    if not args.skip_e2e:
        for _ in range(3):
            e2e_step()
        e2e_dev_s, e2e_wall = timed(e2e_step, args.steps)
        e2e = {"value": bs * world * args.steps / e2e_dev_s, "unit": "samples/s", "h2d_bytes_per_step": h2d_bytes,
               "d2h_bytes_per_step": 4, "ms_per_step": e2e_dev_s / args.steps * 1e3,
               "wall_ms_per_step": e2e_wall / args.steps * 1e3,
               "timing": "CUDA events around K iterations of the reference's loop; DLTrainer.train() copies each "
                         "batch from pinned host memory and reads loss.item(); max over ranks"}

    value = bs * world * args.steps / dev_s
    out = {
        "impl": "reference",
        "metric": "samples/sec at density %g (gTop-k S-SGD training throughput)" % args.density,
        "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dev_s / args.steps * 1e3, "wall_ms_per_step": wall_s / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"model": args.model, "global_batch": bs * world, "per_gpu_batch": bs,
                   "seq_len": 35 if is_lstm else None, "parallelism": "dp%d" % world,
                   "compressor": args.compressor, "density": args.density, "lr": lr,
                   "optimizer": "the reference's DistributedOptimizer._step" if sparse else "horovod-style wrapper + SGD.step",
                   "l2": "inputs larger than L2 (activations and gradients exceed 126 MB per step); no flush",
                   "tf32": False, "cudnn": "benchmark off, deterministic on (dl_trainer.py:20-21)",
                   "transport": "gloo (host buffers) for the MPI calls, NCCL for the Horovod calls",
                   "source": "baseline/_ref", "source_matches_manifest": bool(source_ok)},
        "comm_ms_per_iter": comm_ms,
        "clocks": clocks,
        "e2e": e2e,
        "gpu_launches": 0,
    }
    if dry:
        out["dry_run"] = "no GPU: plumbing check, not a measurement"
    if rank == 0:
        os.write(real_stdout, (json.dumps(out) + "\n").encode())
    if sparse:
        optimizer.stop()
        optimizer.allreducer_thread.join(timeout=10)
    MPI.COMM_WORLD.Barrier()
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    rc = main()
    sys.stdout.flush()
    sys.stderr.flush()
    # the reference's communication thread is not a daemon; leave without waiting for stragglers
    os._exit(rc)
