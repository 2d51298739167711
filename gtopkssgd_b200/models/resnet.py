"""CIFAR ResNet-20/32/44/56/110 (three stages of basic blocks, 16/32/64
channels, parameter-free zero-padding shortcut).

Same architecture, initialisation and state_dict keys as the reference's
models/resnet.py:12-145 (``conv_1_3x3``, ``bn_1``, ``stage_k.i.conv_a`` ...,
``classifier``), so checkpoints are interchangeable.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class ZeroPadShortcut(nn.Module):
    """Option-A shortcut: stride-2 subsampling, new channels filled with zeros."""

    def __init__(self, stride: int):
        super().__init__()
        if stride != 2:
            raise ValueError("the zero-padding shortcut is only defined for stride 2")
        self.stride = stride

    def forward(self, x):
        x = x[:, :, ::self.stride, ::self.stride]
        return torch.cat((x, torch.zeros_like(x)), dim=1)


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, cin: int, cout: int, stride: int = 1, downsample: nn.Module | None = None):
        super().__init__()
        self.conv_a = nn.Conv2d(cin, cout, 3, stride, 1, bias=False)
        self.bn_a = nn.BatchNorm2d(cout)
        self.conv_b = nn.Conv2d(cout, cout, 3, 1, 1, bias=False)
        self.bn_b = nn.BatchNorm2d(cout)
        self.downsample = downsample

    def forward(self, x):
        y = F.relu(self.bn_a(self.conv_a(x)), inplace=True)
        y = self.bn_b(self.conv_b(y))
        skip = x if self.downsample is None else self.downsample(x)
        return F.relu(skip + y, inplace=True)


class CifarResNet(nn.Module):
    def __init__(self, depth: int, num_classes: int = 10, block=BasicBlock):
        super().__init__()
        if (depth - 2) % 6:
            raise ValueError("depth must be 6n+2 (20, 32, 44, 56, 110)")
        n = (depth - 2) // 6
        self.name = "resnet%d" % depth
        self.num_classes = num_classes
        self.conv_1_3x3 = nn.Conv2d(3, 16, 3, 1, 1, bias=False)
        self.bn_1 = nn.BatchNorm2d(16)
        widths, strides = (16, 32, 64), (1, 2, 2)
        cin = 16
        for s, (w, st) in enumerate(zip(widths, strides), start=1):
            blocks = []
            for i in range(n):
                stride = st if i == 0 else 1
                short = ZeroPadShortcut(stride) if (stride != 1 or cin != w * block.expansion) else None
                blocks.append(block(cin, w, stride, short))
                cin = w * block.expansion
            setattr(self, "stage_%d" % s, nn.Sequential(*blocks))
        self.avgpool = nn.AvgPool2d(8)
        self.classifier = nn.Linear(64 * block.expansion, num_classes)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                fan = m.kernel_size[0] * m.kernel_size[1] * m.out_channels
                nn.init.normal_(m.weight, 0.0, math.sqrt(2.0 / fan))
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.ones_(m.weight)
                nn.init.zeros_(m.bias)
            elif isinstance(m, nn.Linear):
                nn.init.kaiming_normal_(m.weight)
                nn.init.zeros_(m.bias)

    def forward(self, x):
        x = F.relu(self.bn_1(self.conv_1_3x3(x)), inplace=True)
        x = self.stage_3(self.stage_2(self.stage_1(x)))
        return self.classifier(torch.flatten(self.avgpool(x), 1))


def _factory(depth):
    def make(num_classes: int = 10):
        return CifarResNet(depth, num_classes)
    make.__name__ = "resnet%d" % depth
    make.__doc__ = "CIFAR ResNet-%d." % depth
    return make


resnet20, resnet32, resnet44, resnet56, resnet110 = (_factory(d) for d in (20, 32, 44, 56, 110))
