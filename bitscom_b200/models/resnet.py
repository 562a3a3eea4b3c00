"""ResNet-18 for 32x32 inputs (CIFAR shape): 3x3 stem, no max-pool, 10 classes; and a
standard ResNet-50 (bottleneck blocks, 7x7 stem, max-pool) for the multi-model
convergence benchmark (the reference takes it from torchvision,
``benchmarks/multimodel_stochastic_e2e_curve.py:42-45``).
Convolutions and batch-norm are torch / cuDNN (not a hot path this library owns); what
the workload exercises is the gradient all-reduce through the DDP communication hook.
The reference's single-GPU integration test uses a similar small ResNet
(``tests/test_single_gpu_train_e2e.py:79-126``)."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class BasicBlock(nn.Module):
    def __init__(self, cin: int, cout: int, stride: int):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, cout, 3, stride, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(cout)
        self.conv2 = nn.Conv2d(cout, cout, 3, 1, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(cout)
        self.short = None
        if stride != 1 or cin != cout:
            self.short = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False),
                                       nn.BatchNorm2d(cout))

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = self.bn2(self.conv2(y))
        return F.relu(y + (x if self.short is None else self.short(x)))


class ResNet18(nn.Module):
    def __init__(self, num_classes: int = 10):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, 64, 3, 1, 1, bias=False), nn.BatchNorm2d(64),
                                  nn.ReLU(inplace=True))
        cfg = [(64, 1), (64, 1), (128, 2), (128, 1), (256, 2), (256, 1), (512, 2), (512, 1)]
        blocks, cin = [], 64
        for cout, stride in cfg:
            blocks.append(BasicBlock(cin, cout, stride))
            cin = cout
        self.blocks = nn.Sequential(*blocks)
        self.fc = nn.Linear(512, num_classes)

    def forward(self, x):
        x = self.blocks(self.stem(x))
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, cin: int, width: int, stride: int):
        super().__init__()
        cout = width * self.expansion
        self.conv1 = nn.Conv2d(cin, width, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        self.conv2 = nn.Conv2d(width, width, 3, stride, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(width)
        self.conv3 = nn.Conv2d(width, cout, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(cout)
        self.short = None
        if stride != 1 or cin != cout:
            self.short = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False),
                                       nn.BatchNorm2d(cout))

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = F.relu(self.bn2(self.conv2(y)))
        y = self.bn3(self.conv3(y))
        return F.relu(y + (x if self.short is None else self.short(x)))


class ResNet50(nn.Module):
    """Bottleneck ResNet with stage depths (3, 4, 6, 3); ``depths`` shrinks it for tests."""

    def __init__(self, num_classes: int = 1000, depths=(3, 4, 6, 3), base_width: int = 64):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, base_width, 7, 2, 3, bias=False),
                                  nn.BatchNorm2d(base_width), nn.ReLU(inplace=True),
                                  nn.MaxPool2d(3, 2, 1))
        blocks, cin = [], base_width
        for stage, depth in enumerate(depths):
            width = base_width << stage
            for i in range(depth):
                blocks.append(Bottleneck(cin, width, 2 if (i == 0 and stage > 0) else 1))
                cin = width * Bottleneck.expansion
        self.blocks = nn.Sequential(*blocks)
        self.fc = nn.Linear(cin, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def forward(self, x):
        x = self.blocks(self.stem(x))
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))
