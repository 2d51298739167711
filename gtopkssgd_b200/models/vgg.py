"""VGG-11/13/16/19 with batch norm for 32x32 inputs and a single
``Linear(512, 10)`` classifier (reference: models/vgg.py:6-38, same
``features.N`` / ``fc`` state_dict keys)."""
from __future__ import annotations

import torch
import torch.nn as nn

cfg = {
    "VGG11": [64, "M", 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
    "VGG13": [64, 64, "M", 128, 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
    "VGG16": [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"],
    "VGG19": [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512, "M"],
}


class VGG(nn.Module):
    def __init__(self, vgg_name: str = "VGG16", num_classes: int = 10):
        super().__init__()
        self.name = vgg_name.lower()
        layers, cin = [], 3
        for v in cfg[vgg_name.upper()]:
            if v == "M":
                layers.append(nn.MaxPool2d(2, 2))
            else:
                layers += [nn.Conv2d(cin, v, 3, padding=1), nn.BatchNorm2d(v), nn.ReLU(inplace=True)]
                cin = v
        layers.append(nn.AvgPool2d(1, 1))
        self.features = nn.Sequential(*layers)
        self.fc = nn.Linear(512, num_classes)

    def forward(self, x):
        return self.fc(torch.flatten(self.features(x), 1))
