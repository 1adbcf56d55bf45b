"""CIFAR-10 ResNets (3x3 stem, no max-pool) with module ReLUs, so that every activation is visible
to the FX-based converters.  Parity: ``spikingjelly/activation_based/ann2snn/sample_models/cifar10_resnet.py:1-155``."""
import torch
import torch.nn as nn

__all__ = ["ResNet", "ResNet18", "ResNet34", "ResNet50", "ResNet101", "ResNet152"]


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, in_planes, planes, stride=1):
        super().__init__()
        self.conv1 = nn.Conv2d(in_planes, planes, 3, stride, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(planes)
        self.relu1 = nn.ReLU()
        self.conv2 = nn.Conv2d(planes, planes, 3, 1, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.relu2 = nn.ReLU()
        self.shortcut = nn.Sequential()
        if stride != 1 or in_planes != planes * self.expansion:
            self.shortcut = nn.Sequential(nn.Conv2d(in_planes, planes * self.expansion, 1, stride, bias=False),
                                          nn.BatchNorm2d(planes * self.expansion))

    def forward(self, x):
        out = self.relu1(self.bn1(self.conv1(x)))
        return self.relu2(self.bn2(self.conv2(out)) + self.shortcut(x))


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, in_planes, planes, stride=1):
        super().__init__()
        self.conv1, self.bn1, self.relu1 = nn.Conv2d(in_planes, planes, 1, bias=False), nn.BatchNorm2d(planes), nn.ReLU()
        self.conv2, self.bn2, self.relu2 = nn.Conv2d(planes, planes, 3, stride, 1, bias=False), nn.BatchNorm2d(planes), nn.ReLU()
        self.conv3, self.bn3, self.relu3 = nn.Conv2d(planes, planes * 4, 1, bias=False), nn.BatchNorm2d(planes * 4), nn.ReLU()
        self.shortcut = nn.Sequential()
        if stride != 1 or in_planes != planes * 4:
            self.shortcut = nn.Sequential(nn.Conv2d(in_planes, planes * 4, 1, stride, bias=False), nn.BatchNorm2d(planes * 4))

    def forward(self, x):
        out = self.relu1(self.bn1(self.conv1(x)))
        out = self.relu2(self.bn2(self.conv2(out)))
        return self.relu3(self.bn3(self.conv3(out)) + self.shortcut(x))


class ResNet(nn.Module):
    def __init__(self, block, num_blocks, num_classes=10):
        super().__init__()
        self.in_planes = 64
        self.conv1, self.bn1, self.relu = nn.Conv2d(3, 64, 3, 1, 1, bias=False), nn.BatchNorm2d(64), nn.ReLU()
        self.layer1 = self._make_layer(block, 64, num_blocks[0], 1)
        self.layer2 = self._make_layer(block, 128, num_blocks[1], 2)
        self.layer3 = self._make_layer(block, 256, num_blocks[2], 2)
        self.layer4 = self._make_layer(block, 512, num_blocks[3], 2)
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.flatten = nn.Flatten()
        self.linear = nn.Linear(512 * block.expansion, num_classes)

    def _make_layer(self, block, planes, n, stride):
        blocks = []
        for s in [stride] + [1] * (n - 1):
            blocks.append(block(self.in_planes, planes, s))
            self.in_planes = planes * block.expansion
        return nn.Sequential(*blocks)

    def forward(self, x):
        x = self.relu(self.bn1(self.conv1(x)))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.linear(self.flatten(self.avgpool(x)))


def ResNet18(**kw):
    return ResNet(BasicBlock, [2, 2, 2, 2], **kw)


def ResNet34(**kw):
    return ResNet(BasicBlock, [3, 4, 6, 3], **kw)


def ResNet50(**kw):
    return ResNet(Bottleneck, [3, 4, 6, 3], **kw)


def ResNet101(**kw):
    return ResNet(Bottleneck, [3, 4, 23, 3], **kw)


def ResNet152(**kw):
    return ResNet(Bottleneck, [3, 8, 36, 3], **kw)


def test():
    """Shape check of ``ResNet18`` on one CIFAR-sized image; returns the output shape."""
    shape = tuple(ResNet18()(torch.randn(1, 3, 32, 32)).shape)
    assert shape == (1, 10), shape
    return shape
