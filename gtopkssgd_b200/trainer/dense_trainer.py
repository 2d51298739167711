"""Dense S-SGD driver on NCCL: the baseline that the sparse modes are compared
with (reference: horovod_trainer.py:22-103, where Horovod issues the NCCL ring
all-reduce).  Gradients of a merged group are summed with one
``torch.distributed.all_reduce`` on the flat buffer, launched on a side stream
while backward continues, and the fused K3 step applies ``/P``, weight decay
and momentum.

    torchrun --nproc-per-node 8 dense_trainer.py --dnn resnet50 --dataset imagenet \
        --data-dir synthetic --batch-size 64 --lr 0.1 --nworkers 8
"""
from __future__ import annotations

import argparse
import os
import time

import numpy as np
import torch

from .. import settings
from ..parallel import comm
from ..parallel import distributed_optimizer as dopt
from ..parallel.compression import NoneCompressor
from ..settings import logger
from ..utils import create_path
from .dl_trainer import DLTrainer, _support_datasets, _support_dnns

writer = None


def ssgd_dense(dnn, dataset, data_dir, nworkers, lr, batch_size, nsteps_update, max_epochs, nwpernode, pretrain,
               num_steps=1, max_iters=None, threshold=None, cuda_graph=None, prefetch=None):
    use_cuda = torch.cuda.is_available()
    rank = comm.rank()
    if use_cuda:
        torch.cuda.set_device(comm.env_local_rank() % max(torch.cuda.device_count(), 1))
    if rank != 0:
        pretrain = None
    trainer = DLTrainer(rank, nworkers, dist=False, batch_size=batch_size, is_weak_scaling=True,
                        ngpus=1 if use_cuda else 0, data_dir=data_dir, dataset=dataset, dnn=dnn, lr=lr,
                        nworkers=nworkers, prefix="allreduce", pretrain=pretrain, num_steps=num_steps,
                        tb_writer=writer, cuda_graph=cuda_graph)
    if prefetch is not None:
        trainer.prefetch_batches = bool(prefetch)
    trainer.set_train_epoch(int(comm.broadcast_object(trainer.get_train_epoch())))
    trainer.set_train_iter(int(comm.broadcast_object(trainer.get_train_iter())))
    comm.broadcast_parameters(trainer.net.state_dict(), root_rank=0)
    optimizer = dopt.DistributedOptimizer(trainer.optimizer, trainer.net.named_parameters(),
                                          compression=NoneCompressor, is_sparse=False, threshold=threshold)
    trainer.update_optimizer(optimizer)
    iters_per_epoch = trainer.get_num_of_training_samples() // (nworkers * batch_size * nsteps_update)
    times, done = [], 0
    display = 20 if iters_per_epoch > 20 else max(iters_per_epoch - 1, 1)
    try:
        for _epoch in range(max_epochs):
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
                if i % display == 0 and use_cuda:
                    torch.cuda.synchronize()
                times.append(time.time() - s)
                if i % display == 0 and i > 0:
                    t = float(np.mean(times))
                    logger.info("Time per iteration including communication: %f. Speed: %f images/s", t,
                                batch_size * nsteps_update / t)
                    times = []
                done += 1
                if max_iters and done >= max_iters:
                    return trainer
    finally:
        optimizer.stop()
    return trainer


# name used by the reference's entry point
ssgd_with_horovod = ssgd_dense


def main(argv=None):
    global writer
    p = argparse.ArgumentParser(description="AllReduce trainer")
    p.add_argument("--batch-size", type=int, default=32)
    p.add_argument("--nsteps-update", type=int, default=1)
    p.add_argument("--nworkers", type=int, default=1, help="Just for experiments, and it cannot be used in production")
    p.add_argument("--nwpernode", type=int, default=1, help="Number of workers per node")
    p.add_argument("--dataset", type=str, default="imagenet", choices=_support_datasets)
    p.add_argument("--dnn", type=str, default="resnet50", choices=_support_dnns)
    p.add_argument("--data-dir", type=str, default="./data", help="Specify the data root path, or 'synthetic'")
    p.add_argument("--lr", type=float, default=0.1)
    p.add_argument("--max-epochs", type=int, default=90)
    p.add_argument("--pretrain", type=str, default=None)
    p.add_argument("--num-steps", type=int, default=35)
    p.add_argument("--max-iters", type=int, default=None)
    p.add_argument("--threshold", type=int, default=None)
    p.add_argument("--cuda-graph", action="store_true")
    p.add_argument("--prefetch", action="store_true")
    args = p.parse_args(argv)
    comm.init()
    if comm.size() > 1:
        args.nworkers = comm.size()
    batch_size = args.batch_size * args.nsteps_update
    logdir = "allreduce-%s/%s-n%d-bs%d-lr%.4f-ns%d" % (settings.PREFIX, args.dnn, args.nworkers, batch_size, args.lr,
                                                        args.nsteps_update)
    rel = create_path("./logs/%s" % logdir)
    rank = comm.rank()
    if rank == 0 and settings.TENSORBOARD:
        try:
            from torch.utils.tensorboard import SummaryWriter
            writer = SummaryWriter("./runs/%s" % logdir)
        except Exception:
            writer = None
    settings.add_file_handler(os.path.join(rel, settings.hostname + "-" + str(rank) + ".log"))
    logger.info("Configurations: %s", args)
    try:
        ssgd_dense(args.dnn, args.dataset, args.data_dir, args.nworkers, args.lr, args.batch_size, args.nsteps_update,
                   args.max_epochs, args.nwpernode, args.pretrain, args.num_steps, args.max_iters, args.threshold,
                   args.cuda_graph or None, args.prefetch or None)
    finally:
        if writer is not None:
            writer.close()
        comm.shutdown()


if __name__ == "__main__":
    main()
