"""Bottleneck ResNets with a channel-width multiplier (ResNet-50/101/152 and their "wide" variants).

``wide_resnet152(width_mult=8)`` is the enlarged model of the benchmark definition: ResNet-152 block
counts (3, 8, 36, 3) with every convolution's channel count multiplied by 8.  Plain ``torch.nn`` code;
BatchNorm running statistics are ordinary buffers (per replica, as in the reference: no sync-BN)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, inplanes: int, planes: int, stride: int = 1, downsample=None):
        super().__init__()
        self.conv1 = nn.Conv2d(inplanes, planes, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(planes)
        self.conv2 = nn.Conv2d(planes, planes, 3, stride=stride, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.conv3 = nn.Conv2d(planes, planes * self.expansion, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(planes * self.expansion)
        self.downsample = downsample

    def forward(self, x):
        idt = x if self.downsample is None else self.downsample(x)
        out = F.relu(self.bn1(self.conv1(x)))
        out = F.relu(self.bn2(self.conv2(out)))
        out = self.bn3(self.conv3(out))
        return F.relu(out + idt)


class ResNet(nn.Module):
    def __init__(self, blocks=(3, 4, 6, 3), width_mult: float = 1.0, num_classes: int = 1000, base: int = 64):
        super().__init__()
        w = lambda c: max(8, int(c * width_mult))  # noqa: E731
        self.inplanes = w(base)
        self.conv1 = nn.Conv2d(3, self.inplanes, 7, stride=2, padding=3, bias=False)
        self.bn1 = nn.BatchNorm2d(self.inplanes)
        self.layer1 = self._make(w(base), blocks[0], 1)
        self.layer2 = self._make(w(base * 2), blocks[1], 2)
        self.layer3 = self._make(w(base * 4), blocks[2], 2)
        self.layer4 = self._make(w(base * 8), blocks[3], 2)
        self.fc = nn.Linear(w(base * 8) * Bottleneck.expansion, num_classes)

    def _make(self, planes: int, n: int, stride: int):
        down = None
        if stride != 1 or self.inplanes != planes * Bottleneck.expansion:
            down = nn.Sequential(nn.Conv2d(self.inplanes, planes * Bottleneck.expansion, 1, stride=stride, bias=False),
                                 nn.BatchNorm2d(planes * Bottleneck.expansion))
        layers = [Bottleneck(self.inplanes, planes, stride, down)]
        self.inplanes = planes * Bottleneck.expansion
        layers += [Bottleneck(self.inplanes, planes) for _ in range(1, n)]
        return nn.Sequential(*layers)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.bn1(self.conv1(x))), 3, 2, 1)
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


class ResNetWithLoss(nn.Module):
    """Returns the cross-entropy loss, like the training scripts the middleware is meant to wrap."""

    def __init__(self, net: ResNet):
        super().__init__()
        self.net = net

    def forward(self, x, y):
        return F.cross_entropy(self.net(x).float(), y)


def resnet50(**kw) -> ResNet:
    return ResNet((3, 4, 6, 3), **kw)


def resnet152(**kw) -> ResNet:
    return ResNet((3, 8, 36, 3), **kw)


def wide_resnet152(width_mult: float = 8.0, **kw) -> ResNet:
    return ResNet((3, 8, 36, 3), width_mult=width_mult, **kw)


def tiny_resnet(**kw) -> ResNet:
    return ResNet((1, 1, 1, 1), width_mult=0.125, num_classes=10, **kw)
