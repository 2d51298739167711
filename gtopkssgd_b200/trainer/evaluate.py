"""Evaluate saved checkpoints epoch by epoch (reference: evaluate.py:20-74).

``--model-path`` is a checkpoint directory named ``<dnn>-n<N>-bs<B>-lr<lr>``;
files inside are ``<dnn>-rank0-epoch<e>.pth`` with keys ``state/epoch/iter``.
Tracks the best accuracy (CNNs) or the lowest perplexity / WER (LSTMs).
"""
from __future__ import annotations

import argparse
import os

import torch

from .. import settings
from ..settings import logger
from .dl_trainer import DLTrainer


def model_average(trainers):
    """Average the weights of several trainers into the first one."""
    first = trainers[0]
    state = {k: v.clone().float() for k, v in first.net.state_dict().items()}
    for t in trainers[1:]:
        for k, v in t.net.state_dict().items():
            state[k] += v.float()
    for k in state:
        state[k] /= len(trainers)
    first.net.load_state_dict({k: v.to(first.net.state_dict()[k].dtype) for k, v in state.items()})


def parse_model_dir(model_path):
    """('resnet20', batch size, lr) from '<dnn>-n<N>-bs<B>-lr<lr>'."""
    items = os.path.basename(os.path.normpath(model_path)).split("-")
    return items[0], int(items[2][2:]), float(items[-1][2:])


def evaluate(model_path, dnn, dataset, data_dir, nepochs, allreduce=False, start_epoch=1):
    dnn, batch_size, lr = parse_model_dir(model_path)
    ngpus = 1 if torch.cuda.is_available() else 0
    trainer = DLTrainer(0, 1, dist=False, ngpus=ngpus, batch_size=batch_size, is_weak_scaling=True, dataset=dataset,
                        dnn=dnn, data_dir=data_dir, lr=lr, nworkers=1)
    lower_is_better = dnn in ("lstm", "lstman4")
    best = None
    for i in range(start_epoch, nepochs + 1):
        fn = os.path.join(model_path, "%s-rank%d-epoch%d.pth" % (dnn, 0, i))
        if not os.path.isfile(fn):
            logger.warning("missing checkpoint %s", fn)
            continue
        trainer.load_model_from_file(fn)
        acc = trainer.test(i)
        if best is None or (acc < best if lower_is_better else acc > best):
            best = acc
        logger.info("Best validation accuracy or perprexity: %f", best)
    return best


def main(argv=None):
    p = argparse.ArgumentParser(description="p2pdl model evaluater")
    p.add_argument("--model-path", type=str, help="Saved model path")
    p.add_argument("--dnn", type=str, default="resnet20")
    p.add_argument("--dataset", type=str, default="cifar10")
    p.add_argument("--data-dir", type=str, default="./data", help="Specify the data root path")
    p.add_argument("--nepochs", type=int, default=90, help="Number of epochs to evaluate")
    args = p.parse_args(argv)
    settings.add_file_handler("%s/evaluate.log" % args.model_path)
    evaluate(args.model_path, args.dnn, args.dataset, args.data_dir, args.nepochs)


if __name__ == "__main__":
    main()
