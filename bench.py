"""Headline benchmark: training throughput (samples/s) of gTop-k S-SGD at
density 0.001 on N GPUs of one node, ResNet-50 / batch 64 per GPU / fp32 /
synthetic ImageNet-shaped data, plus the per-iteration communication time.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 20 --warmup 5

Prints one JSON line on rank 0.  ``value`` is the whole-job samples/s timed on
the device (CUDA events, barrier + synchronize on both sides, max over ranks)
with the batch already resident on the GPU; ``e2e`` is the same loop through
the public trainer API (``DLTrainer.prefetch`` + ``DLTrainer.train_step``): every
step issues one copy of a batch from pinned host memory (the next step's
inputs, on a copy stream) and ends with the loss read back to the host.
``comm_ms_per_iter`` is the per-iteration communication time in the benchmarked
(graph) mode from the kernels' own device-side stamps, max over ranks: select
(K1), exchange (K2 incl. residual put-back), split into time inside flag waits
and work.  At N > 1 one more, checked exchange follows the timed region:
``exchange_check`` compares the global set on the real NVLink transport, every
rank's selection and every rank's residual with the CPU oracle's tree.
``--impl reference`` is the reference arm: the process is replaced by
``baseline/ref_arm.py``, which runs the unmodified reference on the same
configuration and prints the same JSON shape.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Per-worker images/s of the reference's gTop-k runs (scripts/icdcs2019/communication.py:492 for
# ResNet-50, :477 VGG-16, :482 ResNet-20, :497 LSTM-PTB), P = 1, 4, 8 workers.
PUBLISHED_PER_WORKER = {
    "resnet50": {1: 52.873, 4: 39.795, 8: 39.713},
    "vgg16": {1: 1317.333, 4: 131.060, 8: 130.551},
    "resnet20": {1: 920.632, 4: 916.260, 8: 868.730},
    "lstm": {1: 392.0, 4: 17.8, 8: 17.6},
    "alexnet": {1: 173.469, 4: 16.536, 8: 16.446},  # :487, batch 32 per worker
}
MODEL_DEFAULTS = {  # dataset, per-GPU batch, lr
    "resnet50": ("imagenet", 64, 0.1),
    "vgg16": ("cifar10", 128, 0.1),
    "resnet20": ("cifar10", 32, 0.1),
    "lstm": ("ptb", 20, 22.0),
    "alexnet": ("imagenet", 256, 0.01),
}


def _claim_stdout() -> int:
    """Keep stdout for the one JSON line: everything else that writes to file
    descriptor 1 during the run (library banners such as NCCL's version line)
    goes to stderr.  Returns a descriptor of the original stdout."""
    sys.stdout.flush()
    real = os.dup(1)
    os.dup2(2, 1)
    return real


def _emit(real_stdout: int, obj) -> None:
    sys.stdout.flush()
    os.write(real_stdout, (json.dumps(obj) + "\n").encode())


def reference_arm(args):
    """Hands the process over to ``baseline/ref_arm.py``, which drives the unmodified reference under
    ``baseline/_ref`` (none of this package is imported there).  Same launch, same flags, same JSON shape."""
    script = os.path.join(ROOT, "baseline", "ref_arm.py")
    if not os.path.isfile(os.path.join(ROOT, "baseline", "_ref", "allreducer.py")):
        if int(os.environ.get("RANK", "0")) == 0:  # one line per job, also under torchrun
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref (the copy of the reference tree made "
                              "by baseline/setup_ref.py) is missing"}), flush=True)
        return 0
    argv = [sys.executable, script, "--gpus", str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup),
            "--model", args.model, "--density", str(args.density), "--compressor", args.compressor]
    if args.batch_size:
        argv += ["--batch-size", str(args.batch_size)]
    if args.skip_e2e:
        argv.append("--skip-e2e")
    sys.stdout.flush()
    os.execv(sys.executable, argv)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", type=str, default="resnet50", choices=sorted(MODEL_DEFAULTS))
    ap.add_argument("--batch-size", type=int, default=None, help="per-GPU batch (default: the named config's)")
    ap.add_argument("--density", type=float, default=0.001)
    ap.add_argument("--compressor", type=str, default="gtopk", choices=["gtopk", "topk", "topk2", "none"])
    ap.add_argument("--threshold", type=int, default=None, help="merge threshold in elements (default: one group)")
    ap.add_argument("--channels-last", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--cudnn-benchmark-limit", type=int, default=None,
                    help="how many algorithms cuDNN's autotuner tries per convolution (0 = all; default: PyTorch's 10)")
    ap.add_argument("--no-cuda-graph", action="store_true",
                    help="run every iteration eagerly instead of replaying the captured whole-iteration graph")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3
    real_stdout = _claim_stdout()

    import torch
    from gtopkssgd_b200 import settings
    from gtopkssgd_b200.ops import lib as native
    from gtopkssgd_b200.parallel import comm
    from gtopkssgd_b200.parallel import distributed_optimizer as dopt
    from gtopkssgd_b200.parallel.compression import compressors
    from gtopkssgd_b200.trainer.dl_trainer import DLTrainer
    from gtopkssgd_b200.utils.timing import ClockSampler

    settings.PIN_DENSITY = True  # the named configs fix the density at 0.001 from the first step
    settings.logger.setLevel("WARNING")
    if not torch.cuda.is_available():
        _emit(real_stdout, {"error": "bench.py needs a CUDA device"})
        return 1
    torch.backends.cudnn.benchmark = True
    if args.cudnn_benchmark_limit is not None:
        torch.backends.cudnn.benchmark_limit = args.cudnn_benchmark_limit
    torch.backends.cudnn.allow_tf32 = False          # strict fp32, as the reference trains
    torch.backends.cuda.matmul.allow_tf32 = False
    local_rank = comm.env_local_rank()
    device = torch.device("cuda", local_rank % torch.cuda.device_count())
    torch.cuda.set_device(device)
    comm.init()
    rank, world = comm.rank(), comm.size()
    if world != args.gpus:
        if rank == 0:
            _emit(real_stdout, {"error": "--gpus %d but world size is %d" % (args.gpus, world)})
        return 1

    dataset, bs, lr = MODEL_DEFAULTS[args.model]
    bs = args.batch_size or bs
    sparse = args.compressor != "none"
    trainer = DLTrainer(rank, world, dist=False, batch_size=bs, is_weak_scaling=True, ngpus=1, data_dir="synthetic",
                        dataset=dataset, dnn=args.model, lr=lr, nworkers=world, device=device,
                        synthetic_train_size=max(4096, bs * world * 64), cuda_graph=not args.no_cuda_graph)
    if args.channels_last and args.model not in ("lstm",):
        trainer.net.to(memory_format=torch.channels_last)
    comm.broadcast_parameters(trainer.net.state_dict(), root_rank=0)
    optimizer = dopt.DistributedOptimizer(trainer.optimizer, trainer.net.named_parameters(),
                                          compression=compressors[args.compressor], is_sparse=sparse,
                                          density=args.density, threshold=args.threshold)
    trainer.update_optimizer(optimizer)
    net, crit = trainer.net, trainer.criterion
    is_lstm = args.model == "lstm"

    # ---- a few batches in pinned host memory (e2e) and one resident on the device (kernel-only)
    host_batches = []
    for _ in range(4):
        x, y = trainer.data_iter()
        host_batches.append((x.pin_memory(), y.pin_memory()))
    h2d_bytes = sum(t.numel() * t.element_size() for t in host_batches[0])
    dev_x, dev_y, _, _ = trainer._to_device(host_batches[0])
    if args.channels_last and dev_x.dim() == 4:
        dev_x = dev_x.contiguous(memory_format=torch.channels_last)
    hidden = net.init_hidden() if is_lstm else None

    from gtopkssgd_b200.trainer.graphed_step import GraphedStep
    clip = 0.25 if is_lstm else None
    stepper = GraphedStep(trainer, clip_norm=clip, warmup=3 if not args.no_cuda_graph else 1 << 60)

    def device_step():
        # kernel-only arm: same iteration as DLTrainer.train_step, batch already on the device
        nonlocal hidden
        loss, _, hidden = stepper.run(dev_x, dev_y, hidden)
        return loss

    e2e_state = {"hidden": net.init_hidden() if is_lstm else None, "i": 0, "next": None}

    def e2e_step():
        # one host-to-device copy per step: the batch of the NEXT step leaves pinned memory on the trainer's copy
        # stream while this step computes (DLTrainer.prefetch); the very first step copies its own batch up front
        i = e2e_state["i"]
        e2e_state["i"] += 1
        cur = e2e_state["next"]
        if cur is None:
            cur = trainer.prefetch(host_batches[i % len(host_batches)])
        e2e_state["hidden"] = trainer.train_step(data=cur, hidden=e2e_state["hidden"], clip_norm=clip)
        # issued after this step has been enqueued, so the host side of the copy hides behind the GPU's work
        e2e_state["next"] = trainer.prefetch(host_batches[(i + 1) % len(host_batches)])
        return trainer.loss  # device -> host read of this step's loss

    def timed(fn, steps):
        comm.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        wall = time.time() - t0
        comm.barrier()
        dev_s = a.elapsed_time(b) * 1e-3
        return comm.allreduce_max_float(dev_s, device), comm.allreduce_max_float(wall, device)

    # the CUDA-graph step runs its first 3 calls eagerly and captures on the 4th: keep the capture (and one
    # replay) out of the timed region whatever --warmup says
    for _ in range(max(args.warmup, 5 if not args.no_cuda_graph else 0)):
        device_step()
    torch.cuda.synchronize()
    optimizer.check_status()
    sampler = ClockSampler(gpu_index=device.index or 0, period_ms=100)
    if rank == 0:
        sampler.start()
    native.reset_launch_count()
    dev_s, _ = timed(device_step, args.steps)
    launches = native.launch_count()
    clocks = sampler.stop() if rank == 0 else {}
    optimizer.check_status()

    e2e = None
    if not args.skip_e2e:
        for _ in range(max(6, args.warmup)):  # covers the eager warm-up and the graph capture of this arm
            e2e_step()
        e2e_dev_s, e2e_wall = timed(e2e_step, args.steps)
        e2e = {"value": bs * world * args.steps / e2e_dev_s, "unit": "samples/s", "h2d_bytes_per_step": h2d_bytes,
               "d2h_bytes_per_step": 4, "ms_per_step": e2e_dev_s / args.steps * 1e3,
               "wall_ms_per_step": e2e_wall / args.steps * 1e3,
               "timing": "CUDA events around K steps through DLTrainer.prefetch + DLTrainer.train_step; every step "
                         "issues one copy of a batch from pinned host memory (the next step's inputs, on a copy "
                         "stream, overlapping this step's compute) and ends in a blocking loss read; max over ranks"}

    # ---- per-iteration communication time in the benchmarked mode: the kernels stamp %globaltimer at
    # their phase boundaries into their control blocks, and those stamps survive a graph replay (CUDA-event
    # timers do not).  Three bursts of four more steps of the timed kind; the last step of each burst is
    # read back; mean per rank, max over ranks.
    comm_ms = {}
    a = optimizer._allreducer
    if sparse:
        acc = {"select_ms": 0.0, "exchange_ms": 0.0, "exchange_wait_ms": 0.0, "exchange_work_ms": 0.0}
        n_samples = 3
        for _ in range(n_samples):
            for _ in range(4):  # back to back, as in the timed region; the stamps of the last one are read
                device_step()
            torch.cuda.synchronize()
            for e in a.engines:
                tr = e.selector.trace()
                acc["select_ms"] += max(tr.values()) / 1e6 if tr else 0.0
                rc = getattr(e, "rank_ctx", None)
                if rc is not None and args.compressor == "gtopk":
                    t = rc.trace()
                    if t.get("complete"):
                        acc["exchange_ms"] += t["total"] / 1e3
                        acc["exchange_wait_ms"] += t["wait"] / 1e3
                        acc["exchange_work_ms"] += t["work"] / 1e3
        mine = {k_: v / n_samples for k_, v in acc.items()}
        comm_ms = {k_: comm.allreduce_max_float(v, device) for k_, v in mine.items()}
        if world > 1:  # which rank waits and which one is waited for
            import torch.distributed as dist
            per_rank = [None] * world
            dist.all_gather_object(per_rank, {k_: round(v, 4) for k_, v in mine.items()}, group=comm.cpu_group())
            comm_ms["per_rank"] = per_rank
        comm_ms.update({"ranks": "max over %d" % world, "mode": "graph" if not args.no_cuda_graph else "eager",
                        "how": "device %globaltimer stamps of K1 and K2, last step of 3 bursts of 4 further steps; exchange "
                               "= K2 from its first instruction to the end of the residual put-back, wait = time "
                               "inside its flag waits (partner or root not there yet), work = exchange - wait"})
    # ---- one checked exchange on the real transport against the oracle's tree (off the timed path)
    exchange_check = None
    if sparse and world > 1:
        from gtopkssgd_b200.parallel.selfcheck import exchange_selfcheck
        chk = exchange_selfcheck(optimizer)
        exchange_check = {"ok": chk["ok"], "k": chk.get("k"), "max_rel_err": chk.get("max_rel_err"),
                          "groups": chk["groups"]}
    sel_stats = a.engines[0].selector.stats() if sparse else {}

    value = bs * world * args.steps / dev_s
    pub = PUBLISHED_PER_WORKER.get(args.model, {}).get(world)
    out = {
        "metric": "samples/sec at density %g (gTop-k S-SGD training throughput)" % args.density,
        "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dev_s / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (value / (pub * world)) if pub else None, "dtype": "fp32", "data": "synthetic",
        "impl": "ours",
        "config": {"model": args.model, "global_batch": bs * world, "per_gpu_batch": bs,
                   "seq_len": 35 if is_lstm else None, "parallelism": "dp%d" % world,
                   "compressor": args.compressor, "density": args.density, "lr": lr,
                   "optimizer": "momentum SGD (fused flat-buffer step)",
                   "l2": "inputs larger than L2 (activations and gradients exceed 126 MB per step); no flush",
                   "merge_groups": len(a.engines), "channels_last": bool(args.channels_last),
                   "cuda_graph": not args.no_cuda_graph,
                   "tf32": False},
        "comm_ms_per_iter": comm_ms,
        "exchange_check": exchange_check,
        "published_baseline": {"per_worker_samples_per_s": pub, "workers": world,
                               "source": "scripts/icdcs2019/communication.py:472-497 of the reference (its own "
                                         "cluster, other GPUs and network); vs_baseline divides by this x N"},
        "select_stats": sel_stats,
        "clocks": clocks,
        "e2e": e2e,
        "gpu_launches": int(launches),
    }
    if rank == 0:
        _emit(real_stdout, out)
    optimizer.stop()
    comm.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
