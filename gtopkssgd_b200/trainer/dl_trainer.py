"""Trainer core: model + data + loss + SGD + LR schedule + checkpoints for one
worker.  Same constructor, methods and log lines as the reference's
``DLTrainer`` (dl_trainer.py:104-835); ``python -m gtopkssgd_b200.trainer.dl_trainer``
(or the top-level ``dl_trainer.py``) is the single-GPU command line.

Additions: ``--data-dir synthetic`` (or ``synthetic=True``) generates data of
the named shapes on the fly; checkpoints are actually written when
``save_checkpoints`` is on (the reference builds the dict and the path but its
save call is commented out, dl_trainer.py:613-625); the loss stays on the
device until somebody reads ``trainer.loss``.
"""
from __future__ import annotations

import argparse
import os
import time
from typing import Optional

import numpy as np
import torch
import torch.nn as nn
import torch.optim as optim
import torch.utils.data
import torch.utils.data.distributed

from .. import models, settings
from ..data import ptb_reader
from ..data.synthetic import SyntheticAN4, SyntheticImages, SyntheticPTB
from ..models.lstm import repackage_hidden
from ..settings import logger
from ..utils import create_path

_support_datasets = ["imagenet", "cifar10", "an4", "ptb", "mnist"]
_support_dnns = ["resnet50", "resnet20", "resnet56", "resnet110", "vgg19", "vgg16", "alexnet", "lstman4", "lstm",
                 "mnistnet"]
NUM_CPU_THREADS = 1
SYNTHETIC_SIZES = {"cifar10": (50000, 10000), "mnist": (60000, 10000), "imagenet": (1281167, 50000),
                   "ptb": (929589, 73760), "an4": (948, 130)}


def is_synthetic(data_dir: Optional[str]) -> bool:
    return data_dir is not None and str(data_dir).lower().startswith("synthetic")


def create_net(num_classes, dnn="resnet20", **kwargs):
    return models.create_net(num_classes, dnn, **kwargs)


class _CTC(nn.Module):
    """warp-ctc calling convention (activations TxNxH, flat CPU labels, sizes;
    summed over the batch) on top of ``torch.nn.functional.ctc_loss``."""

    def forward(self, acts, labels, act_lens, label_lens):
        logp = torch.log_softmax(acts.float(), dim=-1)
        return torch.nn.functional.ctc_loss(logp, labels.to(torch.long), act_lens.to(torch.long),
                                            label_lens.to(torch.long), blank=0, reduction="sum", zero_infinity=True)


class PrefetchedBatch:
    """A batch whose device copy is in flight on the copy stream (see ``DLTrainer.prefetch``)."""
    __slots__ = ("tensors", "event")

    def __init__(self, tensors, event):
        self.tensors, self.event = tensors, event


class DLTrainer:
    def __init__(self, rank, size, master="gpu10", dist=True, ngpus=1, batch_size=32, is_weak_scaling=True,
                 data_dir="./data", dataset="cifar10", dnn="resnet20", lr=0.04, nworkers=1, prefix=None,
                 sparsity=0.95, pretrain=None, num_steps=35, tb_writer=None, device=None, save_checkpoints=None,
                 synthetic_train_size=None, cuda_graph=None):
        self.size, self.rank = size, rank
        self.pretrain, self.dataset, self.prefix = pretrain, dataset, prefix
        self.num_steps, self.ngpus, self.writer = num_steps, ngpus, tb_writer
        self.batch_size = batch_size * ngpus if (ngpus > 0 and is_weak_scaling) else batch_size
        self.num_batches_per_epoch = -1
        self.num_classes = {"cifar10": 10, "mnist": 10, "imagenet": 1000, "an4": 29, "ptb": 10}[dataset]
        self.nworkers = nworkers
        self.data_dir = data_dir
        self.synthetic = is_synthetic(data_dir)
        self.synthetic_train_size = synthetic_train_size
        self.save_checkpoints = (os.environ.get("GTOPK_SAVE_CHECKPOINTS", "0") == "1"
                                 if save_checkpoints is None else bool(save_checkpoints))
        self.train_sampler = None
        self.ext = None
        self.use_cuda_graph = os.environ.get("GTOPK_CUDA_GRAPH", "0") == "1" if cuda_graph is None else bool(cuda_graph)
        self._copy_stream = None
        self._pending_residuals = None
        self.prefetch_batches = os.environ.get("GTOPK_PREFETCH", "0") == "1"
        self._inflight = None
        self._graphed = None
        if not isinstance(dnn, str):
            self.net, self.dnn = dnn, dnn.name
        else:
            self.dnn = dnn
            if dnn == "lstm":
                if data_dir is not None:
                    self.data_prepare()
                else:
                    self.vocab_size = 10000
                self.net, self.ext = create_net(self.num_classes, dnn, vocab_size=self.vocab_size,
                                                batch_size=self.batch_size, num_steps=self.num_steps)
            elif dnn == "lstman4":
                self.net, self.ext = create_net(self.num_classes, dnn,
                                                datapath=None if self.synthetic else self.data_dir)
                if data_dir is not None:
                    self.data_prepare()
            else:
                if data_dir is not None:
                    self.data_prepare()
                self.net, self.ext = create_net(self.num_classes, dnn)
        self.lr = self.base_lr = lr
        self.is_cuda = ngpus > 0 and torch.cuda.is_available()
        if device is not None:
            self.device = torch.device(device)
            self.is_cuda = self.device.type == "cuda"
        else:
            self.device = torch.device("cuda", torch.cuda.current_device()) if self.is_cuda else torch.device("cpu")
        if self.is_cuda:
            torch.cuda.manual_seed_all(3000)
            if ngpus > 1:
                self.net = torch.nn.DataParallel(self.net, device_ids=list(range(ngpus))).to(self.device)
            else:
                self.net.to(self.device)
        self.accuracy = 0
        self._loss_t: Optional[torch.Tensor] = None
        self.train_iter = 0
        self.master = master
        if dist:
            from ..parallel import comm
            comm.init()
        self.criterion = _CTC() if dataset == "an4" else nn.CrossEntropyLoss().to(self.device)
        weight_decay, self.m, nesterov = 1e-4, 0.9, False
        if dataset == "an4":
            self.lstman4_lr_epoch_tag = 0
        elif dataset == "ptb":
            self.m, weight_decay = 0.0, 0.0
        elif dataset == "imagenet":
            weight_decay = 5e-4
        self.optimizer = optim.SGD(self.net.parameters(), lr=self.lr, momentum=self.m, weight_decay=weight_decay,
                                   nesterov=nesterov)
        self.train_epoch = 0
        if self.pretrain is not None and os.path.isfile(self.pretrain):
            self.load_model_from_file(self.pretrain)
        self.sparsities, self.compression_ratios, self.communication_sizes = [], [], []
        self.sparsity = sparsity
        self._avg_loss_t: Optional[torch.Tensor] = None
        self.timer = 0.0
        self.iotime = 0.0
        self.epochs_info = []
        self.train_acc_top1 = []
        self.num_of_updates_during_comm = 0
        self.data_iterator = None
        logger.info("num_batches_per_epoch: %d" % self.num_batches_per_epoch)

    # -- small accessors ---------------------------------------------------------
    @property
    def loss(self) -> float:
        """Mean loss of the last ``train`` call (reading it synchronises)."""
        return float(self._loss_t) if self._loss_t is not None else 0.0

    @property
    def avg_loss_per_epoch(self) -> float:
        return float(self._avg_loss_t) if self._avg_loss_t is not None else 0.0

    def get_acc(self):
        return self.accuracy

    def get_loss(self):
        return self.loss

    def get_model_state(self):
        return self.net.state_dict()

    def get_data_shape(self):
        return self._input_shape, self._output_shape

    def get_train_epoch(self):
        return self.train_epoch

    def get_train_iter(self):
        return self.train_iter

    def set_train_epoch(self, epoch):
        self.train_epoch = epoch

    def set_train_iter(self, iteration):
        self.train_iter = iteration

    def get_num_of_training_samples(self):
        return len(self.trainset)

    def update_optimizer(self, optimizer):
        """Swap in the (wrapped) optimizer.  State that a checkpoint loaded
        before the wrapping existed -- the velocity held by the plain optimizer
        and the residuals, which only the wrapper can take -- moves over."""
        old, self.optimizer = self.optimizer, optimizer
        if old is not optimizer and hasattr(optimizer, "load_momentum_state"):
            names = {p: n for n, p in self.net.named_parameters()}
            bufs = {names[p]: st["momentum_buffer"] for p, st in old.state.items()
                    if p in names and st.get("momentum_buffer") is not None}
            if bufs:
                optimizer.load_momentum_state(bufs)
        if self._pending_residuals is not None and hasattr(optimizer, "load_residual_state"):
            optimizer.load_residual_state(self._pending_residuals)
            self._pending_residuals = None

    def update_model(self):
        self.optimizer.step()

    def zero_grad(self):
        self.optimizer.zero_grad()

    def finish(self):
        if self.writer is not None:
            self.writer.close()

    # -- checkpoints ---------------------------------------------------------------
    def load_model_from_file(self, filename):
        """Reads ``{'state', 'epoch', 'iter'}`` (dl_trainer.py:250-255); extra
        keys written by this framework are optional."""
        ckpt = torch.load(filename, map_location="cpu", weights_only=False)
        with torch.no_grad():
            own = self.net.state_dict()
            for k, v in ckpt["state"].items():
                own[k].copy_(v)
        self.train_epoch, self.train_iter = ckpt["epoch"], ckpt["iter"]
        opt = ckpt.get("optimizer")
        if opt is not None:
            try:
                self.optimizer.load_state_dict(opt)
            except (ValueError, KeyError):
                logger.warning("optimizer state in %s does not fit; ignored", filename)
        if ckpt.get("residuals") is not None:
            if hasattr(self.optimizer, "load_residual_state"):
                self.optimizer.load_residual_state(ckpt["residuals"])
            else:
                self._pending_residuals = ckpt["residuals"]  # handed to the wrapper in update_optimizer
        logger.info("Load pretrain model: %s, start from epoch %d and iter: %d", filename, self.train_epoch,
                    self.train_iter)

    def checkpoint_dir(self) -> str:
        if self.prefix:
            rel = "./weights/%s/%s-n%d-bs%d-lr%.4f" % (self.prefix, self.dnn, self.nworkers, self.batch_size,
                                                        self.base_lr)
        else:
            rel = "./weights/%s-n%d-bs%d-lr%.4f" % (self.dnn, self.nworkers, self.batch_size, self.base_lr)
        if settings.SPARSE:
            rel += "-s%.5f" % self.sparsity
        return rel

    def checkpoint_path(self, epoch: Optional[int] = None) -> str:
        e = self.train_epoch if epoch is None else epoch
        return os.path.join(self.checkpoint_dir(), "%s-rank%d-epoch%d.pth" % (self.dnn, self.rank, e))

    def save_checkpoint(self, state, filename):
        create_path(os.path.dirname(filename))
        torch.save(state, filename)

    def make_checkpoint(self, full: bool = False) -> dict:
        state = {"iter": self.train_iter, "epoch": self.train_epoch,
                 "state": {k: v.detach().cpu().clone() for k, v in self.get_model_state().items()}}
        if full:
            state["optimizer"] = self.optimizer.state_dict()
            if hasattr(self.optimizer, "residual_state"):
                state["residuals"] = {k: v.cpu() for k, v in self.optimizer.residual_state().items()}
        return state

    def remove_dict(self, dictionary):
        dictionary.clear()

    # -- data --------------------------------------------------------------------------
    def _loaders(self, trainset, testset, collate=None, pin=False):
        self.trainset, self.testset = trainset, testset
        sampler, shuffle = None, True
        if self.nworkers > 1:
            sampler = torch.utils.data.distributed.DistributedSampler(trainset, num_replicas=self.nworkers,
                                                                      rank=self.rank)
            sampler.set_epoch(0)
            shuffle = False
        self.train_sampler = sampler
        workers = 0 if self.synthetic else NUM_CPU_THREADS
        self.trainloader = torch.utils.data.DataLoader(trainset, batch_size=self.batch_size, shuffle=shuffle,
                                                       num_workers=workers, sampler=sampler, pin_memory=pin,
                                                       collate_fn=collate)
        self.testloader = torch.utils.data.DataLoader(testset, batch_size=self.batch_size, shuffle=False,
                                                      num_workers=0 if self.synthetic else 1, pin_memory=pin,
                                                      collate_fn=collate)

    def _synthetic_sizes(self):
        ntrain, ntest = SYNTHETIC_SIZES[self.dataset]
        if self.synthetic_train_size:
            ntrain = int(self.synthetic_train_size)  # in samples
            ntest = max(self.batch_size, min(ntest, ntrain // 5))
            if self.dataset == "ptb":  # the PTB generator is sized in tokens
                ntrain, ntest = ntrain * self.num_steps, max(ntest, 2 * self.batch_size) * self.num_steps
        return ntrain, ntest

    def imagenet_prepare(self):
        size = 224
        self._input_shape, self._output_shape = (self.batch_size, 3, size, size), (self.batch_size, 1000)
        if self.synthetic:
            ntrain, ntest = self._synthetic_sizes()
            self._loaders(SyntheticImages(ntrain, (3, size, size), 1000, pool=max(64, self.batch_size)),
                          SyntheticImages(ntest, (3, size, size), 1000, pool=max(64, self.batch_size), seed=99),
                          pin=True)
            return
        import torchvision.transforms as T
        from ..data.datasets import DatasetHDF5
        norm = T.Normalize(mean=[0.485, 0.456, 0.406], std=[0.229, 0.224, 0.225])
        fn = os.path.join(self.data_dir, "imagenet-shuffled.hdf5")
        train = DatasetHDF5(fn, "train", T.Compose([T.ToPILImage(), T.RandomResizedCrop(size),
                                                    T.RandomHorizontalFlip(), T.ToTensor(), norm]))
        test = DatasetHDF5(fn, "val", T.Compose([T.ToPILImage(), T.CenterCrop(size), T.ToTensor(), norm]))
        self._loaders(train, test, pin=True)

    def cifar10_prepare(self):
        size = 32
        self._input_shape, self._output_shape = (self.batch_size, 3, size, size), (self.batch_size, 10)
        self.classes = ("plane", "car", "bird", "cat", "deer", "dog", "frog", "horse", "ship", "truck")
        if self.synthetic:
            ntrain, ntest = self._synthetic_sizes()
            self._loaders(SyntheticImages(ntrain, (3, size, size), 10, pool=4096),
                          SyntheticImages(ntest, (3, size, size), 10, pool=1024, seed=99))
            return
        import torchvision
        import torchvision.transforms as T
        norm = T.Normalize(mean=[0.491, 0.482, 0.447], std=[0.247, 0.243, 0.262])
        tr = T.Compose([T.RandomCrop(size, padding=4), T.RandomHorizontalFlip(), T.ToTensor(), norm])
        te = T.Compose([T.ToTensor(), norm])
        have = os.path.isdir(os.path.join(self.data_dir, "cifar-10-batches-py"))
        self._loaders(torchvision.datasets.CIFAR10(self.data_dir, train=True, download=not have, transform=tr),
                      torchvision.datasets.CIFAR10(self.data_dir, train=False, download=not have, transform=te))

    def mnist_prepare(self):
        size = 28
        self._input_shape, self._output_shape = (self.batch_size, 1, size, size), (self.batch_size, 10)
        if self.synthetic:
            ntrain, ntest = self._synthetic_sizes()
            self._loaders(SyntheticImages(ntrain, (1, size, size), 10, pool=4096),
                          SyntheticImages(ntest, (1, size, size), 10, pool=1024, seed=99))
            return
        import torchvision
        import torchvision.transforms as T
        tf = T.Compose([T.ToTensor(), T.Normalize((0.1307,), (0.3081,))])
        have = os.path.isdir(os.path.join(self.data_dir, "MNIST"))
        self._loaders(torchvision.datasets.MNIST(self.data_dir, train=True, download=not have, transform=tf),
                      torchvision.datasets.MNIST(self.data_dir, train=False, download=not have, transform=tf))

    def ptb_prepare(self):
        self._input_shape = self._output_shape = (self.batch_size, self.num_steps)
        if self.synthetic:
            self.vocab_size = 10000
            ntrain, ntest = self._synthetic_sizes()
            self._loaders(SyntheticPTB(ntrain, self.vocab_size, self.batch_size, self.num_steps),
                          SyntheticPTB(ntest, self.vocab_size, self.batch_size, self.num_steps, seed=99), pin=True)
        else:
            train, valid, _test, word_to_id, _ = ptb_reader.ptb_raw_data(data_path=self.data_dir)
            self.vocab_size = len(word_to_id)
            self._loaders(ptb_reader.TrainDataset(train, self.batch_size, self.num_steps),
                          ptb_reader.TestDataset(valid, self.batch_size, self.num_steps), pin=True)
        logger.info("Vocabluary size: {}".format(self.vocab_size))
        logger.info("=========****** finish getting ptb data===========")

    def an4_prepare(self):
        from ..data.audio import (AudioDataLoader, BucketingSampler, DistributedBucketingSampler, SpectrogramDataset,
                                  collate_spectrograms)
        from ..data.decoder import GreedyDecoder
        labels = self.ext["labels"]
        if self.synthetic:
            ntrain, ntest = self._synthetic_sizes()
            trainset, testset = SyntheticAN4(ntrain, len(labels)), SyntheticAN4(ntest, len(labels), seed=99)
        else:
            conf = self.ext["audio_conf"]
            trainset = SpectrogramDataset(conf, os.path.join(self.data_dir, "an4_train_manifest.csv"), labels,
                                          normalize=True, augment=True)
            testset = SpectrogramDataset(conf, os.path.join(self.data_dir, "an4_val_manifest.csv"), labels,
                                         normalize=True, augment=False)
        self.trainset, self.testset = trainset, testset
        if self.nworkers > 1:
            sampler = DistributedBucketingSampler(trainset, batch_size=self.batch_size, num_replicas=self.nworkers,
                                                  rank=self.rank)
        else:
            sampler = BucketingSampler(trainset, batch_size=self.batch_size)
        self.train_sampler = sampler
        self.trainloader = AudioDataLoader(trainset, num_workers=0 if self.synthetic else 4, batch_sampler=sampler)
        self.testloader = AudioDataLoader(testset, batch_size=self.batch_size, num_workers=0 if self.synthetic else 4)
        self.decoder = GreedyDecoder(labels)
        self._input_shape, self._output_shape = (self.batch_size, 1, 161, -1), (self.batch_size, -1)
        del collate_spectrograms

    def data_prepare(self):
        prep = {"imagenet": self.imagenet_prepare, "cifar10": self.cifar10_prepare, "mnist": self.mnist_prepare,
                "an4": self.an4_prepare, "ptb": self.ptb_prepare}.get(self.dataset)
        if prep is None:
            raise ValueError("Unsupport dataset: %s" % self.dataset)
        prep()
        self.data_iterator = None
        n = self.get_num_of_training_samples()
        self.num_batches_per_epoch = (n + self.batch_size * self.nworkers - 1) // (self.batch_size * self.nworkers)

    def update_nworker(self, nworkers, new_rank=-1):
        """Elastic hook (dl_trainer.py:465-486): re-shard the data for a new
        world size / rank."""
        if new_rank >= 0:
            rank = new_rank
        else:
            lost = self.nworkers - nworkers
            rank = self.rank - lost if (lost > 0 and self.rank >= lost) else self.rank
        self.rank = rank
        self.nworkers = nworkers
        if self.dnn != "lstman4":
            sampler = torch.utils.data.distributed.DistributedSampler(self.trainset, num_replicas=nworkers, rank=rank)
            sampler.set_epoch(self.train_epoch)
            self.train_sampler = sampler
            workers = 0 if self.synthetic else NUM_CPU_THREADS
            self.trainloader = torch.utils.data.DataLoader(self.trainset, batch_size=self.batch_size, shuffle=False,
                                                           num_workers=workers, sampler=sampler)
            self.testloader = torch.utils.data.DataLoader(self.testset, batch_size=self.batch_size, shuffle=False,
                                                          num_workers=0 if self.synthetic else 1)
        self.data_iterator = None
        self._inflight = None
        n = self.get_num_of_training_samples()
        self.num_batches_per_epoch = (n + self.batch_size * nworkers - 1) // (self.batch_size * nworkers)

    def data_iter(self):
        """Endless batch iterator; short last batches are skipped.  With
        ``prefetch_batches`` on a GPU the batch after the returned one is
        already on its way to the device (see ``prefetch``)."""
        if not (self.prefetch_batches and self.is_cuda):
            return self._next_host_batch()
        cur = self._inflight if self._inflight is not None else self.prefetch(self._next_host_batch())
        self._inflight = self.prefetch(self._next_host_batch())
        return cur

    def _next_host_batch(self):
        while True:
            if self.data_iterator is None:
                self.data_iterator = iter(self.trainloader)
            try:
                d = next(self.data_iterator)
            except StopIteration:
                self.data_iterator = iter(self.trainloader)
                d = next(self.data_iterator)
            if d[0].size(0) == self.batch_size:
                return d

    # -- learning-rate schedules (dl_trainer.py:499-562) ------------------------------------
    def _set_lr(self, optimizer, lr):
        self.lr = lr
        for pg in optimizer.param_groups:
            pg["lr"] = lr
        return lr

    def _adjust_learning_rate_lstman4(self, progress, optimizer):
        if self.lstman4_lr_epoch_tag != progress:
            self.lstman4_lr_epoch_tag = progress
            self._set_lr(optimizer, self.lr / 1.01)

    def _adjust_learning_rate_lstmptb(self, progress, optimizer):
        first, second, third = 23 + 40, 60, 80
        if progress < first:
            scale = 1.0
        elif progress < second:  # unreachable band, kept so that the numbers match
            scale = 0.1
        elif progress < third:
            scale = 0.01
        else:
            scale = 0.001
        return self._set_lr(optimizer, self.base_lr * scale)

    def _adjust_learning_rate_general(self, progress, optimizer):
        warmup = 10
        if settings.WARMUP and progress < warmup:
            total = self.num_batches_per_epoch * warmup
            min_lr = self.base_lr / self.nworkers
            return self._set_lr(optimizer, min_lr + (self.base_lr - min_lr) / total * self.train_iter)
        first, second, third = 81, 122, 155
        if self.dataset == "imagenet":
            first, second, third = 30, 60, 80
        elif self.dataset == "ptb":
            first, second, third = 24, 60, 80
        scale = 1.0 if progress < first else 0.1 if progress < second else 0.01 if progress < third else 0.001
        return self._set_lr(optimizer, self.base_lr * scale)

    def adjust_learning_rate(self, progress, optimizer):
        if self.dnn == "lstman4":
            return self._adjust_learning_rate_lstman4(self.train_iter // self.num_batches_per_epoch, optimizer)
        if self.dnn == "lstm":
            return self._adjust_learning_rate_lstmptb(progress, optimizer)
        return self._adjust_learning_rate_general(progress, optimizer)

    def print_weight_gradient_ratio(self):
        if self.rank == 0 and self.writer is not None:
            for name, param in self.net.named_parameters():
                self.writer.add_histogram(name, param.detach().cpu().numpy(), self.train_epoch)

    @staticmethod
    def cal_accuracy(output, target, topk=(1,)):
        with torch.no_grad():
            maxk = max(topk)
            _, pred = output.topk(maxk, 1, True, True)
            correct = pred.t().eq(target.view(1, -1))
            return [correct[:k].reshape(-1).float().sum(0, keepdim=True).mul_(100.0 / target.size(0)) for k in topk]

    # -- one or more training iterations ------------------------------------------------------
    def _epoch_boundary(self):
        nb = self.num_batches_per_epoch
        logger.info("train iter: %d, num_batches_per_epoch: %d", self.train_iter, nb)
        acc = float(torch.stack([a.reshape(()) for a in self.train_acc_top1]).mean()) if self.train_acc_top1 else float("nan")
        avg_loss = self.avg_loss_per_epoch / nb
        logger.info("Epoch %d, avg train acc: %f, lr: %f, avg loss: %f" % (self.train_iter // nb, acc, self.lr, avg_loss))
        logger.info("Average Sparsity: %f, compression ratio: %f, communication size: %f",
                    np.mean(self.sparsities) if self.sparsities else float("nan"),
                    np.mean(self.compression_ratios) if self.compression_ratios else float("nan"),
                    np.mean(self.communication_sizes) if self.communication_sizes else float("nan"))
        if self.rank == 0 and self.writer is not None:
            self.writer.add_scalar("cross_entropy", avg_loss, self.train_epoch)
            self.writer.add_scalar("top-1 acc", acc, self.train_epoch)
        if self.rank == 0:
            self.test(self.train_epoch)
        self.sparsities, self.compression_ratios, self.communication_sizes = [], [], []
        self.train_acc_top1 = []
        self.epochs_info.append(avg_loss)
        self._avg_loss_t = None
        if self.rank == 0 and self.save_checkpoints:
            self.save_checkpoint(self.make_checkpoint(), self.checkpoint_path())
        # rank 0 alone validated and saved: the others wait for it on the host, not in a bounded device wait
        meet = getattr(self.optimizer, "epoch_barrier", None)
        if meet is not None and self.nworkers > 1:
            meet()
        self.train_epoch += 1
        if self.train_sampler is not None and self.nworkers > 1 and hasattr(self.train_sampler, "set_epoch"):
            self.train_sampler.set_epoch(self.train_epoch)

    def prefetch(self, data):
        """Start the host-to-device copy of a batch (pinned memory makes it
        asynchronous) on the trainer's copy stream and return a handle that
        ``train`` / ``train_step`` accept as ``data``.  The copy runs while the
        compute stream works on the previous iteration; the consumer waits for
        it on the device (a stream wait, no host synchronisation).  Without a
        GPU the batch is returned unchanged."""
        if not self.is_cuda or isinstance(data, PrefetchedBatch):
            return data
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
        with torch.cuda.stream(self._copy_stream):
            tensors = self._to_device(data)
            ev = torch.cuda.Event()
            ev.record()
        return PrefetchedBatch(tensors, ev)

    def _to_device(self, data):
        if isinstance(data, PrefetchedBatch):
            cur = torch.cuda.current_stream(self.device)
            cur.wait_event(data.event)
            for t in data.tensors:
                if torch.is_tensor(t) and t.is_cuda:
                    t.record_stream(cur)  # allocated on the copy stream, consumed here
            return data.tensors
        if self.dataset == "an4":
            inputs, labels_cpu, pct, target_sizes = data
            input_sizes = pct.mul(int(inputs.size(3))).int()
            return inputs.to(self.device, non_blocking=True), labels_cpu, input_sizes, target_sizes
        inputs, labels = data
        if self.dnn == "lstm":
            inputs, labels = inputs.t().contiguous(), labels.t().contiguous()
        return inputs.to(self.device, non_blocking=True), labels.to(self.device, non_blocking=True), None, None

    def train(self, num_of_iters=1, data=None, hidden=None):
        loss_acc = None
        s = time.time()
        for _ in range(num_of_iters):
            self.adjust_learning_rate(self.train_epoch, self.optimizer)
            if self.train_iter % self.num_batches_per_epoch == 0 and self.train_iter > 0:
                self._epoch_boundary()
            ss = time.time()
            batch = self.data_iter() if data is None else data
            inputs, labels, input_sizes, target_sizes = self._to_device(batch)
            self.iotime += time.time() - ss
            if self.dnn == "lstman4":
                out, output_sizes = self.net(inputs, input_sizes)
                loss = self.criterion(out.transpose(0, 1), labels, output_sizes, target_sizes) / inputs.size(0)
            elif self.dnn == "lstm":
                hidden = repackage_hidden(hidden)
                outputs, hidden = self.net(inputs, hidden)
                loss = self.criterion(outputs.view(-1, self.net.vocab_size), labels.reshape(-1))
            else:
                outputs = self.net(inputs)
                loss = self.criterion(outputs, labels)
            loss.backward()
            ld = loss.detach()
            loss_acc = ld if loss_acc is None else loss_acc + ld
            self._avg_loss_t = ld if self._avg_loss_t is None else self._avg_loss_t + ld
            if self.dnn not in ("lstm", "lstman4"):
                self.train_acc_top1.append(self.cal_accuracy(outputs.detach(), labels, topk=(1,))[0])
            self.train_iter += 1
        self.num_of_updates_during_comm += 1
        self._loss_t = loss_acc / num_of_iters
        self.timer += time.time() - s
        display = 100
        if self.train_iter % display == 0:
            logger.info("[%3d][%5d/%5d][rank:%d] loss: %.3f, average forward and backward time: %f, iotime: %f " %
                        (self.train_epoch, self.train_iter, self.num_batches_per_epoch, self.rank, self.loss,
                         self.timer / display, self.iotime / display))
            if self.is_cuda:
                mb = 1024.0 * 1024
                try:
                    import psutil
                    rss = psutil.Process(os.getpid()).memory_info().rss / mb
                except ImportError:
                    rss = 0
                logger.info("GPU memory usage memory_allocated: %d MBytes, max_memory_allocated: %d MBytes, "
                            "memory_cached: %d MBytes, max_memory_cached: %d MBytes, CPU memory usage: %d MBytes",
                            torch.cuda.memory_allocated() / mb, torch.cuda.max_memory_allocated() / mb,
                            torch.cuda.memory_reserved() / mb, torch.cuda.max_memory_reserved() / mb, rss)
            self.timer = 0.0
            self.iotime = 0.0
        if self.dnn == "lstm":
            return num_of_iters, hidden
        return num_of_iters

    def train_step(self, data=None, hidden=None, clip_norm=None, cuda_graph=None):
        """One complete iteration: zero_grad, forward, backward, optional
        gradient-norm clip, optimizer step.  With ``cuda_graph`` (default: the
        trainer's ``use_cuda_graph``) the whole iteration is captured once as a
        CUDA graph and replayed.  Returns the carried hidden state for the LSTM
        model, else None."""
        from ..utils.timing import nvtx_range
        with nvtx_range("gtopk/train_step"):
            return self._train_step(data, hidden, clip_norm, cuda_graph)

    def _train_step(self, data, hidden, clip_norm, cuda_graph):
        use_graph = self.use_cuda_graph if cuda_graph is None else cuda_graph
        if not (use_graph and self.is_cuda and self.dnn != "lstman4"):
            self.optimizer.zero_grad()
            if self.dnn == "lstm":
                _, hidden = self.train(1, data=data, hidden=hidden)
            else:
                self.train(1, data=data)
            if clip_norm is not None:
                if hasattr(self.optimizer, "clip_grad_norm"):
                    self.optimizer.clip_grad_norm(clip_norm)
                else:
                    torch.nn.utils.clip_grad_norm_(self.net.parameters(), clip_norm)
            self.update_model()
            return hidden
        from .graphed_step import GraphedStep
        if self._graphed is None or self._graphed.clip_norm != clip_norm:
            self._graphed = GraphedStep(self, clip_norm=clip_norm)
        s = time.time()
        self.adjust_learning_rate(self.train_epoch, self.optimizer)
        if self.train_iter % self.num_batches_per_epoch == 0 and self.train_iter > 0:
            self._epoch_boundary()
        batch = self.data_iter() if data is None else data
        x, y, _, _ = self._to_device(batch)
        loss, acc, hidden = self._graphed.run(x, y, hidden)
        self._loss_t = loss
        self._avg_loss_t = loss.clone() if self._avg_loss_t is None else self._avg_loss_t + loss
        if acc is not None:
            self.train_acc_top1.append(acc.clone())
        self.train_iter += 1
        self.timer += time.time() - s
        return hidden

    def test(self, epoch):
        """Validation: accuracy (CNNs), perplexity (LSTM LM), WER (AN4)."""
        self.net.eval()
        test_loss, correct, total, total_iters = 0.0, 0, 0, 0
        costs, total_steps, total_wer = 0.0, 0, 0.0
        with torch.no_grad():
            for data in self.testloader:
                if data[0].size(0) != self.batch_size and self.dnn == "lstm":
                    continue
                inputs, labels, input_sizes, target_sizes = self._to_device(data)
                if self.dnn == "lstm":
                    hidden = repackage_hidden(self.net.init_hidden())
                    outputs, hidden = self.net(inputs, hidden)
                    loss = float(self.criterion(outputs.view(-1, self.net.vocab_size), labels.reshape(-1)))
                    test_loss += loss
                    costs += loss * self.net.num_steps
                    total_steps += self.net.num_steps
                elif self.dnn == "lstman4":
                    out, output_sizes = self.net(inputs, input_sizes)
                    decoded, _ = self.decoder.decode(out, output_sizes)
                    off, wer = 0, 0.0
                    for x, size in enumerate(target_sizes.tolist()):
                        ref = self.decoder.convert_to_strings([labels[off:off + size]])[0][0]
                        off += size
                        wer += self.decoder.wer(decoded[x][0], ref) / float(max(len(ref.split()), 1))
                    total_wer += wer
                else:
                    outputs = self.net(inputs)
                    test_loss += float(self.criterion(outputs, labels))
                    correct += int(outputs.argmax(1).eq(labels).sum())
                total += inputs.size(0) if self.dnn == "lstman4" else labels.size(0)
                total_iters += 1
        test_loss /= max(total_iters, 1)
        if self.dnn == "lstm":
            acc = float(np.exp(costs / max(total_steps, 1)))
        elif self.dnn == "lstman4":
            acc = total_wer / max(len(self.testloader.dataset), 1)
        else:
            acc = float(correct) / max(total, 1)
        logger.info("Epoch %d, lr: %f, val loss: %f, val acc: %f" % (epoch, self.lr, test_loss, acc))
        self.net.train()
        self.accuracy = acc
        return acc


def train_with_single(dnn, dataset, data_dir, nworkers, lr, batch_size, nsteps_update, max_epochs, num_steps=1,
                      max_iters=None):
    """Single-GPU loop (dl_trainer.py:787-812) with the same throughput line."""
    if torch.cuda.is_available():
        torch.cuda.set_device(0)
    trainer = DLTrainer(0, nworkers, dist=False, batch_size=batch_size, is_weak_scaling=True,
                        ngpus=1 if torch.cuda.is_available() else 0, data_dir=data_dir, dataset=dataset, dnn=dnn,
                        lr=lr, nworkers=nworkers, prefix="singlegpu", num_steps=num_steps)
    iters_per_epoch = trainer.get_num_of_training_samples() // (nworkers * batch_size * nsteps_update)
    times, done = [], 0
    display = 100 if iters_per_epoch > 100 else max(iters_per_epoch - 1, 1)
    for _epoch in range(max_epochs):
        hidden = trainer.net.init_hidden() if dnn == "lstm" else None
        for i in range(iters_per_epoch):
            s = time.time()
            trainer.optimizer.zero_grad()
            for _ in range(nsteps_update):
                if dnn == "lstm":
                    _, hidden = trainer.train(1, hidden=hidden)
                else:
                    trainer.train(1)
            trainer.update_model()
            if trainer.is_cuda:
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
    return trainer


def main(argv=None):
    parser = argparse.ArgumentParser(description="Single trainer")
    parser.add_argument("--batch-size", type=int, default=32)
    parser.add_argument("--nsteps-update", type=int, default=1)
    parser.add_argument("--dataset", type=str, default="imagenet", choices=_support_datasets)
    parser.add_argument("--dnn", type=str, default="resnet50", choices=_support_dnns)
    parser.add_argument("--data-dir", type=str, default="./data", help="data root, or 'synthetic'")
    parser.add_argument("--lr", type=float, default=0.1)
    parser.add_argument("--max-epochs", type=int, default=90)
    parser.add_argument("--num-steps", type=int, default=35)
    parser.add_argument("--max-iters", type=int, default=None, help="stop after this many iterations")
    args = parser.parse_args(argv)
    batch_size = args.batch_size * args.nsteps_update
    rel = "./logs/singlegpu-%s/%s-n%d-bs%d-lr%.4f-ns%d" % (settings.PREFIX, args.dnn, 1, batch_size, args.lr,
                                                            args.nsteps_update)
    create_path(rel)
    settings.add_file_handler(os.path.join(rel, settings.hostname + ".log"))
    logger.info("Configurations: %s", args)
    train_with_single(args.dnn, args.dataset, args.data_dir, 1, args.lr, args.batch_size, args.nsteps_update,
                      args.max_epochs, args.num_steps, args.max_iters)


if __name__ == "__main__":
    main()
