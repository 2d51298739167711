"""The reference's additional CIFAR networks, none of which its trainers can
reach from the command line but all of which its ``models`` package exports:

* pre-activation ResNets (models/preresnet.py:9-151),
* the feature-returning ResNet variant (models/resnet_mod.py:9-167),
* ResNeXt-29 8x64d / 16x64d (models/resnext.py:6-126),
* DenseNet-100 (k = 12) (models/densenet.py:6-101),
* the small Caffe-style CIFAR net (models/caffe_cifar.py:8-59).

They share one initialiser and one stage builder here; parameter names match
the reference so that its checkpoints load.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .resnet import BasicBlock, CifarResNet, ZeroPadShortcut


def init_cifar(model: nn.Module, linear_kaiming: bool = True) -> None:
    for m in model.modules():
        if isinstance(m, nn.Conv2d):
            fan = m.kernel_size[0] * m.kernel_size[1] * m.out_channels
            nn.init.normal_(m.weight, 0.0, math.sqrt(2.0 / fan))
        elif isinstance(m, nn.BatchNorm2d):
            nn.init.ones_(m.weight)
            nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Linear):
            if linear_kaiming:
                nn.init.kaiming_normal_(m.weight)
            nn.init.zeros_(m.bias)


# ---- pre-activation ResNet ---------------------------------------------------------------
class PreActBlock(nn.Module):
    expansion = 1

    def __init__(self, cin, cout, stride, downsample, kind):
        super().__init__()
        if kind not in ("both_preact", "normal"):
            raise ValueError("Unknow type : {}".format(kind))
        self.Type = kind
        self.bn_a = nn.BatchNorm2d(cin)
        self.conv_a = nn.Conv2d(cin, cout, 3, stride, 1, bias=False)
        self.bn_b = nn.BatchNorm2d(cout)
        self.conv_b = nn.Conv2d(cout, cout, 3, 1, 1, bias=False)
        self.relu = nn.ReLU(inplace=True)
        self.downsample = downsample

    def forward(self, x):
        pre = self.relu(self.bn_a(x))
        skip = pre if self.Type == "both_preact" else x
        y = self.conv_b(self.relu(self.bn_b(self.conv_a(pre))))
        if self.downsample is not None:
            skip = self.downsample(skip)
        return skip + y


class CifarPreResNet(nn.Module):
    def __init__(self, depth, num_classes=10):
        super().__init__()
        if (depth - 2) % 6:
            raise ValueError("depth should be one of 20, 32, 44, 56, 110")
        n = (depth - 2) // 6
        self.name = "preresnet%d" % depth
        self.num_classes = num_classes
        self.conv_3x3 = nn.Conv2d(3, 16, 3, 1, 1, bias=False)
        cin = 16
        for s, (w, st) in enumerate(zip((16, 32, 64), (1, 2, 2)), start=1):
            blocks = []
            for i in range(n):
                stride = st if i == 0 else 1
                short = ZeroPadShortcut(stride) if (i == 0 and (stride != 1 or cin != w)) else None
                blocks.append(PreActBlock(cin, w, stride, short, "both_preact" if i == 0 else "normal"))
                cin = w
            setattr(self, "stage_%d" % s, nn.Sequential(*blocks))
        self.lastact = nn.Sequential(nn.BatchNorm2d(64), nn.ReLU(inplace=True))
        self.avgpool = nn.AvgPool2d(8)
        self.classifier = nn.Linear(64, num_classes)
        init_cifar(self)

    def forward(self, x):
        x = self.stage_3(self.stage_2(self.stage_1(self.conv_3x3(x))))
        return self.classifier(torch.flatten(self.avgpool(self.lastact(x)), 1))


# ---- ResNet that can also return the per-block batch-norm outputs --------------------------
class FeatureBlock(BasicBlock):
    """Basic block; given a list ``[x, f1, f2, ...]`` it appends its two BN outputs."""

    def forward(self, x):
        feats = None
        if isinstance(x, list):
            x, feats = x[0], x[1:]
        bn_a = self.bn_a(self.conv_a(x))
        bn_b = self.bn_b(self.conv_b(F.relu(bn_a, inplace=False)))
        skip = x if self.downsample is None else self.downsample(x)
        out = F.relu(skip + bn_b, inplace=False)
        return out if feats is None else [out] + feats + [bn_a, bn_b]


class CifarResNetMod(CifarResNet):
    def __init__(self, depth, num_classes=10):
        super().__init__(depth, num_classes, block=FeatureBlock)
        self.name = "resnet_mod%d" % depth

    def forward(self, x):
        as_list = isinstance(x, list)
        if as_list:
            if len(x) != 1:
                raise ValueError("The length of inputs must be one vs {}".format(len(x)))
            x = x[0]
        x = F.relu(self.bn_1(self.conv_1_3x3(x)), inplace=True)
        x = self.stage_3(self.stage_2(self.stage_1([x] if as_list else x)))
        feats = None
        if as_list:
            x, feats = x[0], x[1:]
        cls = self.classifier(torch.flatten(self.avgpool(x), 1))
        return (cls, feats) if as_list else cls


# ---- ResNeXt ---------------------------------------------------------------------------------
class ResNeXtBottleneck(nn.Module):
    expansion = 4

    def __init__(self, cin, planes, cardinality, base_width, stride=1, downsample=None):
        super().__init__()
        width = int(math.floor(planes * (base_width / 64.0))) * cardinality
        self.conv_reduce = nn.Conv2d(cin, width, 1, bias=False)
        self.bn_reduce = nn.BatchNorm2d(width)
        self.conv_conv = nn.Conv2d(width, width, 3, stride, 1, groups=cardinality, bias=False)
        self.bn = nn.BatchNorm2d(width)
        self.conv_expand = nn.Conv2d(width, planes * 4, 1, bias=False)
        self.bn_expand = nn.BatchNorm2d(planes * 4)
        self.downsample = downsample

    def forward(self, x):
        y = F.relu(self.bn_reduce(self.conv_reduce(x)), inplace=True)
        y = F.relu(self.bn(self.conv_conv(y)), inplace=True)
        y = self.bn_expand(self.conv_expand(y))
        skip = x if self.downsample is None else self.downsample(x)
        return F.relu(skip + y, inplace=True)


class CifarResNeXt(nn.Module):
    def __init__(self, depth, cardinality, base_width, num_classes=10):
        super().__init__()
        if (depth - 2) % 9:
            raise ValueError("depth should be one of 29, 38, 47, 56, 101")
        n = (depth - 2) // 9
        self.name = "resnext%d_%d_%d" % (depth, cardinality, base_width)
        self.cardinality, self.base_width, self.num_classes = cardinality, base_width, num_classes
        self.conv_1_3x3 = nn.Conv2d(3, 64, 3, 1, 1, bias=False)
        self.bn_1 = nn.BatchNorm2d(64)
        cin = 64
        for s, (planes, st) in enumerate(zip((64, 128, 256), (1, 2, 2)), start=1):
            blocks = []
            for i in range(n):
                stride = st if i == 0 else 1
                down = None
                if i == 0 and (stride != 1 or cin != planes * 4):
                    down = nn.Sequential(nn.Conv2d(cin, planes * 4, 1, stride, bias=False),
                                         nn.BatchNorm2d(planes * 4))
                blocks.append(ResNeXtBottleneck(cin, planes, cardinality, base_width, stride, down))
                cin = planes * 4
            setattr(self, "stage_%d" % s, nn.Sequential(*blocks))
        self.avgpool = nn.AvgPool2d(8)
        self.classifier = nn.Linear(1024, num_classes)
        init_cifar(self)

    def forward(self, x):
        x = F.relu(self.bn_1(self.conv_1_3x3(x)), inplace=True)
        x = self.stage_3(self.stage_2(self.stage_1(x)))
        return self.classifier(torch.flatten(self.avgpool(x), 1))


# ---- DenseNet --------------------------------------------------------------------------------
class DenseBottleneck(nn.Module):
    def __init__(self, cin, growth):
        super().__init__()
        self.bn1 = nn.BatchNorm2d(cin)
        self.conv1 = nn.Conv2d(cin, 4 * growth, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(4 * growth)
        self.conv2 = nn.Conv2d(4 * growth, growth, 3, padding=1, bias=False)

    def forward(self, x):
        y = self.conv1(F.relu(self.bn1(x)))
        return torch.cat((x, self.conv2(F.relu(self.bn2(y)))), 1)


class DenseSingle(nn.Module):
    def __init__(self, cin, growth):
        super().__init__()
        self.bn1 = nn.BatchNorm2d(cin)
        self.conv1 = nn.Conv2d(cin, growth, 3, padding=1, bias=False)

    def forward(self, x):
        return torch.cat((x, self.conv1(F.relu(self.bn1(x)))), 1)


class Transition(nn.Module):
    def __init__(self, cin, cout):
        super().__init__()
        self.bn1 = nn.BatchNorm2d(cin)
        self.conv1 = nn.Conv2d(cin, cout, 1, bias=False)

    def forward(self, x):
        return F.avg_pool2d(self.conv1(F.relu(self.bn1(x))), 2)


class DenseNet(nn.Module):
    def __init__(self, growthRate, depth, reduction, nClasses, bottleneck):
        super().__init__()
        self.name = "densenet%d_%d" % (depth, growthRate)
        n = (depth - 4) // (6 if bottleneck else 3)
        layer = DenseBottleneck if bottleneck else DenseSingle
        ch = 2 * growthRate
        self.conv1 = nn.Conv2d(3, ch, 3, padding=1, bias=False)
        for stage in (1, 2, 3):
            blocks = []
            for _ in range(n):
                blocks.append(layer(ch, growthRate))
                ch += growthRate
            setattr(self, "dense%d" % stage, nn.Sequential(*blocks))
            if stage < 3:
                out = int(math.floor(ch * reduction))
                setattr(self, "trans%d" % stage, Transition(ch, out))
                ch = out
        self.bn1 = nn.BatchNorm2d(ch)
        self.fc = nn.Linear(ch, nClasses)
        init_cifar(self, linear_kaiming=False)

    def forward(self, x):
        x = self.trans1(self.dense1(self.conv1(x)))
        x = self.dense3(self.trans2(self.dense2(x)))
        x = torch.flatten(F.avg_pool2d(F.relu(self.bn1(x)), 8), 1)
        return F.log_softmax(self.fc(x), dim=1)


# ---- Caffe-style CIFAR net -----------------------------------------------------------------
class CifarCaffeNet(nn.Module):
    def __init__(self, num_classes=10):
        super().__init__()
        self.name = "caffe_cifar"
        self.num_classes = num_classes
        self.block_1 = nn.Sequential(nn.Conv2d(3, 32, 3, 1, 1), nn.MaxPool2d(3, 2), nn.ReLU(), nn.BatchNorm2d(32))
        self.block_2 = nn.Sequential(nn.Conv2d(32, 32, 3, 1, 1), nn.Conv2d(32, 64, 3, 1, 1), nn.ReLU(),
                                     nn.AvgPool2d(3, 2), nn.BatchNorm2d(64))
        self.block_3 = nn.Sequential(nn.Conv2d(64, 64, 3, 1, 1), nn.Conv2d(64, 128, 3, 1, 1), nn.ReLU(),
                                     nn.AvgPool2d(3, 2), nn.BatchNorm2d(128))
        self.classifier = nn.Linear(128 * 9, num_classes)
        init_cifar(self)

    def forward(self, x):
        return self.classifier(torch.flatten(self.block_3(self.block_2(self.block_1(x))), 1))


def _depths(cls, prefix):
    def make(depth):
        def f(num_classes=10):
            return cls(depth, num_classes)
        f.__name__ = "%s%d" % (prefix, depth)
        return f
    return [make(d) for d in (20, 32, 44, 56, 110)]


preresnet20, preresnet32, preresnet44, preresnet56, preresnet110 = _depths(CifarPreResNet, "preresnet")
resnet_mod20, resnet_mod32, resnet_mod44, resnet_mod56, resnet_mod110 = _depths(CifarResNetMod, "resnet_mod")


def resnext29_16_64(num_classes=10):
    return CifarResNeXt(29, 16, 64, num_classes)


def resnext29_8_64(num_classes=10):
    return CifarResNeXt(29, 8, 64, num_classes)


def densenet100_12(num_classes=10):
    return DenseNet(12, 100, 0.5, num_classes, False)


def caffe_cifar(num_classes=10):
    return CifarCaffeNet(num_classes)
