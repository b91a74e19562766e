"""ResNet-50 (v1.5: stride on the 3x3 convolution of each bottleneck), the data-parallel
workload of the training benchmark.  Convolutions, normalisation and the classifier run on
cuDNN / cuBLAS through PyTorch - the reference is a collective library and has no compute
kernels; what this repository contributes to the step is the gradient path (daemon
all-reduce with fused scale / cast, fused optimizer over flat buckets)."""
from __future__ import annotations

import torch
import torch.nn as nn


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, cin: int, width: int, stride: int = 1, downsample: nn.Module | None = None):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, width, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        self.conv2 = nn.Conv2d(width, width, 3, stride=stride, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(width)
        self.conv3 = nn.Conv2d(width, width * self.expansion, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(width * self.expansion)
        self.relu = nn.ReLU(inplace=True)
        self.downsample = downsample

    def forward(self, x):
        idt = x if self.downsample is None else self.downsample(x)
        out = self.relu(self.bn1(self.conv1(x)))
        out = self.relu(self.bn2(self.conv2(out)))
        out = self.bn3(self.conv3(out))
        return self.relu(out + idt)


class ResNet(nn.Module):
    def __init__(self, layers=(3, 4, 6, 3), num_classes: int = 1000, width: int = 64):
        super().__init__()
        self.cin = width
        self.conv1 = nn.Conv2d(3, width, 7, stride=2, padding=3, bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        self.relu = nn.ReLU(inplace=True)
        self.maxpool = nn.MaxPool2d(3, stride=2, padding=1)
        self.layer1 = self._make(width, layers[0], 1)
        self.layer2 = self._make(width * 2, layers[1], 2)
        self.layer3 = self._make(width * 4, layers[2], 2)
        self.layer4 = self._make(width * 8, layers[3], 2)
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.fc = nn.Linear(width * 8 * Bottleneck.expansion, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.ones_(m.weight)
                nn.init.zeros_(m.bias)
        for m in self.modules():                      # zero-init the last norm of each block
            if isinstance(m, Bottleneck):
                nn.init.zeros_(m.bn3.weight)

    def _make(self, width: int, blocks: int, stride: int) -> nn.Sequential:
        down = None
        if stride != 1 or self.cin != width * Bottleneck.expansion:
            down = nn.Sequential(nn.Conv2d(self.cin, width * Bottleneck.expansion, 1, stride=stride, bias=False),
                                 nn.BatchNorm2d(width * Bottleneck.expansion))
        seq = [Bottleneck(self.cin, width, stride, down)]
        self.cin = width * Bottleneck.expansion
        seq += [Bottleneck(self.cin, width) for _ in range(1, blocks)]
        return nn.Sequential(*seq)

    def forward(self, x):
        x = self.maxpool(self.relu(self.bn1(self.conv1(x))))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.fc(torch.flatten(self.avgpool(x), 1))


def resnet50(num_classes: int = 1000) -> ResNet:
    return ResNet((3, 4, 6, 3), num_classes)


def resnet_tiny(num_classes: int = 10) -> ResNet:
    """Two-stage miniature with the same block structure (tests, smoke)."""
    return ResNet((1, 1, 1, 1), num_classes, width=8)


def to_bf16_channels_last(model: nn.Module) -> nn.Module:
    """bf16 weights in channels-last layout; normalisation parameters and statistics stay fp32
    (the mixed mode cuDNN's NHWC batch-norm kernels take)."""
    model = model.to(memory_format=torch.channels_last).to(torch.bfloat16)
    for m in model.modules():
        if isinstance(m, nn.modules.batchnorm._BatchNorm):
            m.float()
    return model
