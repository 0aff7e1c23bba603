"""ResNet v1.5 image classifiers from ``torch.nn`` alone (the second DDP benchmark model).

Same architecture as the reference's benchmark model (scripts/gpu/train_bench.py:191-221):
a 7x7 stride-2 stem, a 3x3 max-pool, stages of bottleneck blocks whose stride sits on the
3x3 convolution (the "v1.5" variant), global average pooling and one linear classifier.
``resnet50``: stages of 3, 4, 6 and 3 blocks from 64 channels, 1000 classes, 224x224 images
(25.6 M parameters).  ``resnet-tiny``: two stages of one block from 8 channels, 10 classes,
32x32 images, for CPU tests.

On a GPU the benchmark runs it in ``channels_last`` under bf16 autocast: cuDNN's
tensor-core convolutions want NHWC, and BatchNorm keeps fp32 statistics either way.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass(frozen=True)
class ResNetConfig:
    stages: tuple[int, ...] = (3, 4, 6, 3)
    stem: int = 64
    classes: int = 1000
    image: int = 224


CONFIGS = {
    "resnet50": ResNetConfig(),
    "resnet-tiny": ResNetConfig(stages=(1, 1), stem=8, classes=10, image=32),
}


def _conv_bn(cin: int, cout: int, kernel: int, stride: int = 1) -> nn.Sequential:
    return nn.Sequential(nn.Conv2d(cin, cout, kernel, stride, kernel // 2, bias=False),
                         nn.BatchNorm2d(cout))


class Bottleneck(nn.Module):
    """1x1 reduce, 3x3 (strided), 1x1 expand to four times the width, plus the shortcut."""

    expansion = 4

    def __init__(self, cin: int, width: int, stride: int) -> None:
        super().__init__()
        cout = width * self.expansion
        self.reduce = _conv_bn(cin, width, 1)
        self.spatial = _conv_bn(width, width, 3, stride)
        self.expand = _conv_bn(width, cout, 1)
        self.shortcut = _conv_bn(cin, cout, 1, stride) if (stride != 1 or cin != cout) else nn.Identity()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = F.relu(self.reduce(x), inplace=True)
        y = F.relu(self.spatial(y), inplace=True)
        return F.relu(self.expand(y) + self.shortcut(x), inplace=True)


class ResNet(nn.Module):
    def __init__(self, c: ResNetConfig) -> None:
        super().__init__()
        self.config = c
        self.stem = _conv_bn(3, c.stem, 7, 2)
        blocks, cin = [], c.stem
        for index, count in enumerate(c.stages):
            width = c.stem << index
            for b in range(count):
                blocks.append(Bottleneck(cin, width, 2 if (b == 0 and index > 0) else 1))
                cin = width * Bottleneck.expansion
        self.blocks = nn.Sequential(*blocks)
        self.classifier = nn.Linear(cin, c.classes)

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        x = F.max_pool2d(F.relu(self.stem(images), inplace=True), 3, 2, 1)
        x = self.blocks(x)
        return self.classifier(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))

    def loss(self, images: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        return F.cross_entropy(self(images).float(), labels)


def build(name: str = "resnet50") -> ResNet:
    return ResNet(CONFIGS[name])


def synthetic_images(config: ResNetConfig, batch: int, seed: int = 0,
                     count: int = 1) -> list[tuple[torch.Tensor, torch.Tensor]]:
    """``count`` (images, labels) pairs of normal noise and uniform labels, on the host."""
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(batch, 3, config.image, config.image, generator=g),
             torch.randint(config.classes, (batch,), generator=g)) for _ in range(count)]
