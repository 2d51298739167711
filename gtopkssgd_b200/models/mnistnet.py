"""Small MNIST CNN (reference: dl_trainer.py:58-75 / model_builder.py:4-21)."""
import torch.nn as nn
import torch.nn.functional as F


class MnistNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.name = "mnistnet"
        self.conv1 = nn.Conv2d(1, 10, 5)
        self.conv2 = nn.Conv2d(10, 20, 5)
        self.conv2_drop = nn.Dropout2d()
        self.fc1 = nn.Linear(320, 50)
        self.fc2 = nn.Linear(50, 10)

    def forward(self, x):
        x = F.relu(F.max_pool2d(self.conv1(x), 2))
        x = F.relu(F.max_pool2d(self.conv2_drop(self.conv2(x)), 2))
        x = F.dropout(F.relu(self.fc1(x.view(-1, 320))), training=self.training)
        return self.fc2(x)  # logits, as the reference returns them (dl_trainer.py:68-75)
