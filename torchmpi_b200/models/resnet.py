"""ResNet (bottleneck) for the data-parallel benchmark: ResNet-50 = layers [3, 4, 6, 3], 25.6 M parameters.

The reference ships no model beyond a logistic regressor
(examples/mnist/mnist_allreduce.lua:31); this is the standard architecture
(He et al. 2015, stride on the 3x3 convolution) written for channels_last bf16
training.  With ``fused_bn=True`` batch-norm + ReLU (+ residual add) run as the fused kernels of
``ops.bn_relu``, the max-pool as ``ops.pool`` and the stem convolution as im2col + tcgen05 GEMM
(``ops.stem_conv``); the other convolutions run in cuDNN.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn


def _bn(ch: int, fused: bool, relu: bool, zero_init: bool = False) -> nn.Module:
    if fused:
        from ..ops.bn_relu import FusedBatchNormReLU
        m = FusedBatchNormReLU(ch, relu=relu)
    else:
        m = nn.BatchNorm2d(ch)
    if zero_init:
        nn.init.zeros_(m.weight)
    return m


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, inplanes: int, planes: int, stride: int = 1, downsample: Optional[nn.Module] = None,
                 fused_bn: bool = False):
        super().__init__()
        self.fused = fused_bn
        self.conv1 = nn.Conv2d(inplanes, planes, 1, bias=False)
        self.bn1 = _bn(planes, fused_bn, relu=True)
        self.conv2 = nn.Conv2d(planes, planes, 3, stride=stride, padding=1, bias=False)
        self.bn2 = _bn(planes, fused_bn, relu=True)
        self.conv3 = nn.Conv2d(planes, planes * 4, 1, bias=False)
        self.bn3 = _bn(planes * 4, fused_bn, relu=True, zero_init=True)   # relu after the residual add
        self.downsample = downsample

    def forward(self, x):
        identity = x if (self.downsample is None or self.fused) else self.downsample(x)
        if self.fused:
            from ..ops.conv import conv_bn
            from ..parallel.flat_buckets import GradFork
            # x has two consumers (the first convolution and the identity branch): their gradients are summed
            # inside the kernel of whichever runs last in backward instead of by a separate add
            from .. import config
            fork = GradFork(2) if (torch.is_grad_enabled() and x.requires_grad and config.get("grad_fork")) else None
            res_fork = None
            if self.downsample is not None:
                identity = conv_bn(self.downsample[0], self.downsample[1], x, fork=fork)
            else:
                res_fork = fork
            out = conv_bn(self.conv1, self.bn1, x, fork=fork)
            out = conv_bn(self.conv2, self.bn2, out)
            return conv_bn(self.conv3, self.bn3, out, residual=identity, res_fork=res_fork)
        out = torch.relu(self.bn1(self.conv1(x)))
        out = torch.relu(self.bn2(self.conv2(out)))
        out = self.bn3(self.conv3(out))
        return torch.relu(out + identity)


class ResNet(nn.Module):
    def __init__(self, layers: List[int], num_classes: int = 1000, fused_bn: bool = False, width: int = 64):
        super().__init__()
        self.fused = fused_bn
        self.inplanes = width
        if fused_bn:
            from ..ops.stem_conv import StemConv7x7
            self.conv1 = StemConv7x7(width)           # im2col + tensor-core GEMM; same parameter as the Conv2d
        else:
            self.conv1 = nn.Conv2d(3, width, 7, stride=2, padding=3, bias=False)
        if fused_bn:
            from ..ops.bn_relu import FusedBatchNormReLUMaxPool
            self.bn1 = FusedBatchNormReLUMaxPool(width)     # batch-norm + ReLU + max-pool in one stage
            self.maxpool = nn.Identity()
        else:
            self.bn1 = _bn(width, fused_bn, relu=True)
            self.maxpool = nn.MaxPool2d(3, stride=2, padding=1)
        self.layer1 = self._make_layer(width, layers[0], 1)
        self.layer2 = self._make_layer(width * 2, layers[1], 2)
        self.layer3 = self._make_layer(width * 4, layers[2], 2)
        self.layer4 = self._make_layer(width * 8, layers[3], 2)
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        if fused_bn:
            from ..ops.gemm import Linear
            self.fc = Linear(width * 8 * 4, num_classes)     # same parameters as nn.Linear; tcgen05 GEMMs where the shape allows
        else:
            self.fc = nn.Linear(width * 8 * 4, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def _make_layer(self, planes: int, blocks: int, stride: int) -> nn.Sequential:
        down = None
        if stride != 1 or self.inplanes != planes * 4:
            down = nn.Sequential(nn.Conv2d(self.inplanes, planes * 4, 1, stride=stride, bias=False),
                                 _bn(planes * 4, self.fused, relu=False))
        layers = [Bottleneck(self.inplanes, planes, stride, down, self.fused)]
        self.inplanes = planes * 4
        layers += [Bottleneck(self.inplanes, planes, fused_bn=self.fused) for _ in range(1, blocks)]
        return nn.Sequential(*layers)

    def forward(self, x):
        x = self.bn1(self.conv1(x))
        if not self.fused:
            x = torch.relu(x)
        x = self.maxpool(x)
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        x = torch.flatten(self.avgpool(x), 1)
        return self.fc(x)


def resnet50(num_classes: int = 1000, fused_bn: bool = False) -> ResNet:
    return ResNet([3, 4, 6, 3], num_classes, fused_bn)


def resnet_tiny(num_classes: int = 10, fused_bn: bool = False) -> ResNet:
    """A two-stage miniature for tests and smoke runs."""
    return ResNet([1, 1, 1, 1], num_classes, fused_bn, width=16)


def resnet_small(num_classes: int = 10, fused_bn: bool = False) -> ResNet:
    """One bottleneck block per stage at the real widths (64 .. 2048 channels): small enough for a smoke run,
    wide enough that every convolution takes the same kernels as ResNet-50."""
    return ResNet([1, 1, 1, 1], num_classes, fused_bn, width=64)
