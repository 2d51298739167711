"""gTop-k S-SGD training driver and command line
(reference: gtopk_trainer.py:26-168, launched there with ``mpirun``; here one
process per GPU under ``torchrun``).

    torchrun --nproc-per-node 8 gtopk_trainer.py --dnn resnet20 --dataset cifar10 \
        --data-dir synthetic --batch-size 32 --lr 0.1 --nworkers 8 \
        --compression --compressor gtopk --density 0.001

Same flags, same log-directory naming and the same throughput log line as the
reference.  Extra flags: ``--max-iters`` (stop early), ``--threshold`` (merge
threshold in elements), ``--pin-density`` (skip the 0.004 warm-up density of
epoch 0), ``--save-checkpoints``.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import numpy as np
import torch

from .. import settings
from ..parallel import comm
from ..parallel import distributed_optimizer as dopt
from ..parallel.allreducer import GTopkTimeout
from ..parallel.compression import compressors
from ..settings import logger
from ..utils import create_path
from .dl_trainer import DLTrainer, _support_datasets, _support_dnns

writer = None
relative_path = None


def _dump_profiling_norms(optimizer, rank, epoch):
    """PROFILING_NORM files of the reference (gtopk_trainer.py:94-126)."""
    norms = optimizer._allreducer._profiling_norms
    cols = list(zip(*norms)) if norms else [[], [], [], [], []]
    names = ["gtopknorm", "randknorm", "upbound", "xnorm", "densestd"]
    labels = ["gtopk norm", "randk norm", "upbound norm", "x norm", "dense std"]
    for name, label, col in zip(names, labels, cols):
        arr = np.array(col)
        if arr.size:
            logger.info("[rank:%d][%d] %s mean: %f, std: %f", rank, epoch, label, np.mean(arr), np.std(arr))
        if name != "xnorm" and relative_path:
            np.save(os.path.join(relative_path, "%s-rank%d-epoch%d.npy" % (name, rank, epoch)), arr)
    optimizer._allreducer._profiling_norms = []


def robust_ssgd(dnn, dataset, data_dir, nworkers, lr, batch_size, nsteps_update, max_epochs, compression=False,
                compressor="topk", nwpernode=1, sigma_scale=2.5, pretrain=None, density=0.01, prefix=None,
                max_iters=None, threshold=None, save_checkpoints=None, check_every=50, cuda_graph=None,
                prefetch=None, membership_check_every=50, elastic=False, leave_requested=None,
                synthetic_train_size=None):
    """``elastic``: a rank that gets a departure request (``leave_requested()``
    turns true, e.g. from a SIGTERM handler) announces it, keeps training up
    to the agreed iteration and returns; the others re-form a smaller job at
    that iteration and continue."""
    use_cuda = torch.cuda.is_available()
    rank = dopt.rank()
    if use_cuda:
        torch.cuda.set_device(comm.env_local_rank() % max(torch.cuda.device_count(), 1))
    if rank != 0 and pretrain:
        # weights come from rank 0's broadcast; a rank still reads its own file of the same checkpoint, if
        # there is one, for what differs between ranks (the residuals)
        own = pretrain.replace("-rank0-", "-rank%d-" % rank)
        pretrain = own if own != pretrain and os.path.isfile(own) else None
    prefix = (prefix or settings.PREFIX) + "-ds%s" % str(density)
    trainer = DLTrainer(rank, nworkers, dist=False, batch_size=batch_size, is_weak_scaling=True,
                        ngpus=1 if use_cuda else 0, data_dir=data_dir, dataset=dataset, dnn=dnn, lr=lr,
                        nworkers=nworkers, prefix=prefix, pretrain=pretrain, tb_writer=writer,
                        save_checkpoints=save_checkpoints, cuda_graph=cuda_graph,
                        synthetic_train_size=synthetic_train_size)
    if prefetch is not None:
        trainer.prefetch_batches = bool(prefetch)
    trainer.set_train_epoch(comm.broadcast_object(trainer.get_train_epoch()))
    trainer.set_train_iter(comm.broadcast_object(trainer.get_train_iter()))

    def _error_handler(new_num_workers, new_rank):
        logger.info("Error info catched by trainer")
        trainer.update_nworker(new_num_workers, new_rank)

    comp = compressors[compressor if compression else "none"]
    logger.info("Broadcast parameters....")
    comm.broadcast_parameters(trainer.net.state_dict(), root_rank=0)
    logger.info("Broadcast parameters finished....")
    optimizer = dopt.DistributedOptimizer(trainer.optimizer, trainer.net.named_parameters(), compression=comp,
                                          is_sparse=compression, err_handler=_error_handler, layerwise_times=None,
                                          sigma_scale=sigma_scale, density=density, norm_clip=None, writer=writer,
                                          threshold=threshold, membership_check_every=membership_check_every,
                                          elastic=elastic)
    trainer.update_optimizer(optimizer)
    iters_per_epoch = trainer.get_num_of_training_samples() // (nworkers * batch_size * nsteps_update)
    times, done = [], 0
    display = 100 if iters_per_epoch > 100 else max(iters_per_epoch - 1, 1)
    logger.info("Start training ....")
    try:
        for epoch in range(max_epochs):
            hidden = trainer.net.init_hidden() if dnn == "lstm" else None
            for i in range(iters_per_epoch):
                s = time.time()
                clip = 0.25 if dnn == "lstm" else 400 if dnn == "lstman4" else None
                if nsteps_update == 1:
                    hidden = trainer.train_step(hidden=hidden, clip_norm=clip)
                else:
                    optimizer.zero_grad()
                    for j in range(nsteps_update):
                        optimizer.local = j < nsteps_update - 1
                        if dnn == "lstm":
                            _, hidden = trainer.train(1, hidden=hidden)
                        else:
                            trainer.train(1)
                    if clip is not None:
                        optimizer.clip_grad_norm(clip)
                    trainer.update_model()
                if i % display == 0 or (check_every and done % check_every == 0):
                    if use_cuda:
                        torch.cuda.synchronize()
                    optimizer.check_status()
                times.append(time.time() - s)
                if i % display == 0 and i > 0:
                    t = float(np.mean(times))
                    logger.info("Time per iteration including communication: %f. Speed: %f images/s, "
                                "current density: %f", t, batch_size * nsteps_update / t,
                                optimizer.get_current_density())
                    times = []
                done += 1
                if max_iters and done >= max_iters:
                    return trainer
                if elastic:
                    if leave_requested is not None and leave_requested():
                        optimizer.request_leave()
                    if optimizer.should_exit():
                        logger.info("leaving the job after iteration %d as announced", done)
                        return trainer
            optimizer.add_train_epoch()
            if settings.PROFILING_NORM:
                _dump_profiling_norms(optimizer, rank, epoch)
    except GTopkTimeout as exc:
        logger.error("training stopped: %s", exc)
        _save_interrupted(trainer, exc)
        raise
    finally:
        optimizer.stop()
    return trainer


def _save_interrupted(trainer, exc):
    """A departure noticed on the host BEFORE an iteration was launched leaves
    every surviving rank with the state of the last completed iteration:
    write it out (weights, optimizer state, residuals) so that the job can be
    restarted with ``--pretrain``.  After a device-side wait ran out in the
    middle of an exchange the update may be partial, so nothing is saved."""
    from ..parallel.elastic import PeerLeft
    if not isinstance(exc.__cause__, PeerLeft):
        return None
    fn = os.path.join(trainer.checkpoint_dir(), "%s-rank%d-interrupted.pth" % (trainer.dnn, trainer.rank))
    try:
        trainer.save_checkpoint(trainer.make_checkpoint(full=True), fn)
        logger.info("state of iteration %d saved to %s (restart with --pretrain)", trainer.train_iter, fn)
        return fn
    except Exception:  # never mask the communication failure
        logger.exception("could not save the interrupted state")
        return None


def build_parser():
    p = argparse.ArgumentParser(description="AllReduce trainer")
    p.add_argument("--batch-size", type=int, default=32)
    p.add_argument("--nsteps-update", type=int, default=1)
    p.add_argument("--nworkers", type=int, default=1, help="Just for experiments, and it cannot be used in production")
    p.add_argument("--nwpernode", type=int, default=1, help="Number of workers per node")
    p.add_argument("--compression", dest="compression", action="store_true")
    p.add_argument("--compressor", type=str, default="topk", choices=list(compressors.keys()),
                   help="Specify the compressors if 'compression' is open")
    p.add_argument("--sigma-scale", type=float, default=2.5, help="Maximum sigma scaler for sparsification")
    p.add_argument("--density", type=float, default=0.01, help="Density for sparsification")
    p.add_argument("--dataset", type=str, default="imagenet", choices=_support_datasets)
    p.add_argument("--dnn", type=str, default="resnet50", choices=_support_dnns)
    p.add_argument("--data-dir", type=str, default="./data", help="Specify the data root path, or 'synthetic'")
    p.add_argument("--lr", type=float, default=0.1, help="Default learning rate")
    p.add_argument("--max-epochs", type=int, default=90, help="Default maximum epochs to train")
    p.add_argument("--pretrain", type=str, default=None, help="Specify the pretrain path")
    p.add_argument("--max-iters", type=int, default=None, help="Stop after this many iterations")
    p.add_argument("--threshold", type=int, default=None, help="Merge threshold in elements")
    p.add_argument("--pin-density", action="store_true", help="Use --density from epoch 0 on")
    p.add_argument("--save-checkpoints", action="store_true", help="Write a checkpoint at every epoch end")
    p.add_argument("--cuda-graph", action="store_true",
                   help="Capture the whole iteration as a CUDA graph (pays off for launch-bound models)")
    p.add_argument("--elastic", action="store_true",
                   help="On SIGTERM a rank announces its departure and leaves at an agreed iteration; "
                        "the other ranks continue as a smaller job")
    p.add_argument("--prefetch", action="store_true",
                   help="Copy the next batch to the device on a side stream while the current iteration runs")
    p.set_defaults(compression=False)
    return p


def main(argv=None):
    global writer, relative_path
    args = build_parser().parse_args(argv)
    if args.pin_density:
        settings.PIN_DENSITY = True
    comm.init()
    if comm.size() > 1 and args.nworkers != comm.size():
        logger.warning("--nworkers %d differs from the launched world size %d; using %d", args.nworkers, comm.size(),
                       comm.size())
        args.nworkers = comm.size()
    batch_size = args.batch_size * args.nsteps_update
    prefix = settings.PREFIX
    if args.compression:
        prefix = "comp-" + args.compressor + "-" + prefix
    logdir = "allreduce-%s/%s-n%d-bs%d-lr%.4f-ns%d-sg%.2f-ds%s" % (prefix, args.dnn, args.nworkers, batch_size,
                                                                     args.lr, args.nsteps_update, args.sigma_scale,
                                                                     str(args.density))
    relative_path = create_path("./logs/%s" % logdir)
    rank = dopt.rank()
    if rank == 0 and settings.TENSORBOARD:
        try:
            from torch.utils.tensorboard import SummaryWriter
            writer = SummaryWriter("./runs/%s" % logdir)
        except Exception:  # tensorboard is optional
            writer = None
    settings.add_file_handler(os.path.join(relative_path, settings.hostname + "-" + str(rank) + ".log"))
    logger.info("Configurations: %s", args)
    logger.info("Interpreter: %s", sys.version)
    leave = None
    if args.elastic:
        import signal
        import threading
        asked = threading.Event()
        signal.signal(signal.SIGTERM, lambda *_: asked.set())
        leave = asked.is_set
    try:
        robust_ssgd(args.dnn, args.dataset, args.data_dir, args.nworkers, args.lr, args.batch_size,
                    args.nsteps_update, args.max_epochs, args.compression, args.compressor, args.nwpernode,
                    args.sigma_scale, args.pretrain, args.density, prefix, max_iters=args.max_iters,
                    threshold=args.threshold, save_checkpoints=args.save_checkpoints or None,
                    cuda_graph=args.cuda_graph or None, prefetch=args.prefetch or None, elastic=args.elastic,
                    leave_requested=leave)
    finally:
        if writer is not None:
            writer.close()
        comm.shutdown()


if __name__ == "__main__":
    main()
