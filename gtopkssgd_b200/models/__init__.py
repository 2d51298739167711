"""Model zoo: every architecture reachable from the reference's trainers
(dl_trainer.py:38-39,80-101) plus its extra CIFAR nets, with random
initialisation and reference-compatible ``state_dict`` keys."""
from __future__ import annotations

from .alexnet import AlexNet
from .cifar_extras import (caffe_cifar, densenet100_12, preresnet20, preresnet32, preresnet44, preresnet56,
                           preresnet110, resnet_mod20, resnet_mod32, resnet_mod44, resnet_mod56, resnet_mod110,
                           resnext29_8_64, resnext29_16_64)
from .imagenet_resnet import resnet18, resnet34, resnet50, resnet101, resnet152
from .lstm import lstm, repackage_hidden
from .lstman4 import create_net as LSTMAN4
from .mnistnet import MnistNet
from .resnet import resnet20, resnet32, resnet44, resnet56, resnet110
from .vgg import VGG

SUPPORTED_DNNS = ["resnet50", "resnet20", "resnet56", "resnet110", "vgg19", "vgg16", "alexnet", "lstman4", "lstm",
                  "mnistnet"]


def create_net(num_classes: int, dnn: str = "resnet20", **kwargs):
    """Build a network by its ``--dnn`` name.  Returns ``(net, ext)`` where
    ``ext`` carries model-specific extras (the AN4 audio configuration)."""
    ext = None
    if dnn in ("resnet20", "resnet32", "resnet44", "resnet56", "resnet110"):
        net = globals()[dnn](num_classes=num_classes)
    elif dnn in ("resnet18", "resnet34", "resnet50", "resnet101", "resnet152"):
        net = globals()[dnn](num_classes=num_classes)
    elif dnn in ("preresnet20", "preresnet32", "preresnet44", "preresnet56", "preresnet110", "resnet_mod20",
                 "resnet_mod32", "resnet_mod44", "resnet_mod56", "resnet_mod110", "resnext29_8_64",
                 "resnext29_16_64", "densenet100_12", "caffe_cifar"):
        net = globals()[dnn](num_classes=num_classes)
    elif dnn == "mnistnet":
        net = MnistNet()
    elif dnn in ("vgg11", "vgg13", "vgg16", "vgg19"):
        net = VGG(dnn.upper())
    elif dnn == "alexnet":
        import torchvision
        net = torchvision.models.alexnet(num_classes=num_classes)
        net.name = "alexnet"
    elif dnn == "alexnet_lrn":
        net = AlexNet(num_classes=num_classes)
    elif dnn == "lstman4":
        net, ext = LSTMAN4(datapath=kwargs.get("datapath"))
    elif dnn == "lstm":
        net = lstm(vocab_size=kwargs["vocab_size"], batch_size=kwargs["batch_size"],
                   num_steps=kwargs.get("num_steps", 35))
    else:
        raise ValueError("Unsupport neural network %s" % dnn)
    if not hasattr(net, "name"):
        net.name = dnn
    return net, ext
