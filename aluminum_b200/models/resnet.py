"""ResNet-50 (v1.5: stride on the 3x3 convolution of each bottleneck), 25.6 M parameters.

This is the data-parallel training workload of the end-to-end benchmark: the
communication library is what is being measured, the network is the standard
consumer (the reference itself ships no model; LBANN drives it with ResNet-50,
see README.md:9-17 of the reference).  Random initialisation, no pretrained
weights.
"""
from __future__ import annotations

import torch
from torch import nn


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, c_in: int, width: int, stride: int = 1, downsample: nn.Module | None = None):
        super().__init__()
        self.conv1 = nn.Conv2d(c_in, width, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        self.conv2 = nn.Conv2d(width, width, 3, stride=stride, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(width)
        self.conv3 = nn.Conv2d(width, width * self.expansion, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(width * self.expansion)
        self.relu = nn.ReLU(inplace=True)
        self.downsample = downsample

    def forward(self, x):
        identity = x if self.downsample is None else self.downsample(x)
        out = self.relu(self.bn1(self.conv1(x)))
        out = self.relu(self.bn2(self.conv2(out)))
        out = self.bn3(self.conv3(out))
        return self.relu(out + identity)


class ResNet(nn.Module):
    def __init__(self, layers=(3, 4, 6, 3), num_classes: int = 1000, width: int = 64):
        super().__init__()
        self.c = width
        self.conv1 = nn.Conv2d(3, width, 7, stride=2, padding=3, bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        self.relu = nn.ReLU(inplace=True)
        self.maxpool = nn.MaxPool2d(3, stride=2, padding=1)
        self.layer1 = self._stage(width, layers[0], 1)
        self.layer2 = self._stage(width * 2, layers[1], 2)
        self.layer3 = self._stage(width * 4, layers[2], 2)
        self.layer4 = self._stage(width * 8, layers[3], 2)
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.fc = nn.Linear(width * 8 * Bottleneck.expansion, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.ones_(m.weight)
                nn.init.zeros_(m.bias)
        for m in self.modules():
            if isinstance(m, Bottleneck):
                nn.init.zeros_(m.bn3.weight)  # residual branches start as identity

    def _stage(self, width: int, blocks: int, stride: int) -> nn.Sequential:
        down = None
        if stride != 1 or self.c != width * Bottleneck.expansion:
            down = nn.Sequential(nn.Conv2d(self.c, width * Bottleneck.expansion, 1, stride=stride, bias=False),
                                 nn.BatchNorm2d(width * Bottleneck.expansion))
        mods = [Bottleneck(self.c, width, stride, down)]
        self.c = width * Bottleneck.expansion
        mods += [Bottleneck(self.c, width) for _ in range(1, blocks)]
        return nn.Sequential(*mods)

    def forward(self, x):
        x = self.maxpool(self.relu(self.bn1(self.conv1(x))))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.fc(torch.flatten(self.avgpool(x), 1))


def resnet50(num_classes: int = 1000) -> ResNet:
    return ResNet((3, 4, 6, 3), num_classes)
