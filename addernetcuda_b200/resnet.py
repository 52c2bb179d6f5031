"""ResNet-20 (CIFAR) and ResNet-50 (ImageNet) adder networks: the callers that fix the layer shapes.

Same architectures, module names and state-dict keys as the reference's resnet20.py:12-97 and
resnet50.py:19-121, so a checkpoint written by either loads into the other.  The reference files
themselves also run unchanged on top of this package (they only do `import adder`); these builders
exist because a training harness needs the networks where the reference sources are not installed.

The layer class is a parameter (`conv=`), so the same builder yields the CUDA network
(`addernetcuda_b200.adder.adder2d`, the default) or, in tests, a CPU checker network.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn as nn


def _default_conv():
    from .adder import adder2d
    return adder2d


def _norm_class(fused: bool):
    if fused:
        from .batchnorm import FusedBatchNorm2d
        return FusedBatchNorm2d
    return nn.BatchNorm2d


def _bn_act(bn, y, residual=None, relu=False):
    """relu?(bn(y) + residual?) - one fused pass when `bn` is a FusedBatchNorm2d (training) or a
    FoldedBatchNorm2d (evaluation, `inference.fold_batchnorm`)."""
    if bn.__class__.__name__ in ("FusedBatchNorm2d", "FoldedBatchNorm2d"):
        return bn(y, residual=residual, relu=relu)
    out = bn(y)
    if residual is not None:
        out = out + residual
    return torch.relu(out) if relu else out


def _conv_bn_act(conv, bn, x, residual=None, relu=False):
    """relu?(bn(conv(x)) + residual?).  An adder layer followed by a FusedBatchNorm2d in training mode hands
    the batch statistics over from its own epilogue, so the normalisation reads the layer's output once."""
    if (bn.__class__.__name__ == "FusedBatchNorm2d" and bn.training and x.is_cuda and x.dtype == torch.float32
            and hasattr(conv, "forward_with_stats")):
        y, st = conv.forward_with_stats(x)
        return bn(y, residual=residual, relu=relu, stats=st)
    return _bn_act(bn, conv(x), residual=residual, relu=relu)


def _shortcut(downsample, x):
    if isinstance(downsample, nn.Sequential) and len(downsample) == 2:
        return _conv_bn_act(downsample[0], downsample[1], x)
    return downsample(x)


class BasicBlock(nn.Module):
    """conv3x3-BN-ReLU-conv3x3-BN + shortcut, ReLU (resnet20.py:12-41)."""
    expansion = 1

    def __init__(self, conv, inplanes, planes, stride=1, downsample=None, norm=nn.BatchNorm2d):
        super().__init__()
        self.conv1 = conv(inplanes, planes, kernel_size=3, stride=stride, padding=1, bias=False)
        self.bn1 = norm(planes)
        self.relu = nn.ReLU(inplace=True)
        self.conv2 = conv(planes, planes, kernel_size=3, stride=1, padding=1, bias=False)
        self.bn2 = norm(planes)
        self.downsample = downsample
        self.stride = stride

    def forward(self, x):
        out = _conv_bn_act(self.conv1, self.bn1, x, relu=True)
        res = x if self.downsample is None else _shortcut(self.downsample, x)
        return _conv_bn_act(self.conv2, self.bn2, out, residual=res, relu=True)


class Bottleneck(nn.Module):
    """1x1-3x3(stride)-1x1(x4) bottleneck (resnet50.py:19-55)."""
    expansion = 4

    def __init__(self, conv, inplanes, planes, stride=1, downsample=None, norm=nn.BatchNorm2d):
        super().__init__()
        self.conv1 = conv(inplanes, planes, kernel_size=1, stride=1, bias=False)
        self.bn1 = norm(planes)
        self.conv2 = conv(planes, planes, kernel_size=3, stride=stride, padding=1, bias=False)
        self.bn2 = norm(planes)
        self.conv3 = conv(planes, planes * 4, kernel_size=1, stride=1, bias=False)
        self.bn3 = norm(planes * 4)
        self.relu = nn.ReLU(inplace=True)
        self.downsample = downsample
        self.stride = stride

    def forward(self, x):
        out = _conv_bn_act(self.conv1, self.bn1, x, relu=True)
        out = _conv_bn_act(self.conv2, self.bn2, out, relu=True)
        res = x if self.downsample is None else _shortcut(self.downsample, x)
        return _conv_bn_act(self.conv3, self.bn3, out, residual=res, relu=True)


class _ResNet(nn.Module):
    def _make_layer(self, conv, block, planes, blocks, stride=1):
        norm = self.norm
        downsample = None
        if stride != 1 or self.inplanes != planes * block.expansion:
            downsample = nn.Sequential(
                conv(self.inplanes, planes * block.expansion, kernel_size=1, stride=stride, bias=False),
                norm(planes * block.expansion))
        layers = [block(conv, self.inplanes, planes, stride, downsample, norm)]
        self.inplanes = planes * block.expansion
        layers += [block(conv, self.inplanes, planes, norm=norm) for _ in range(1, blocks)]
        return nn.Sequential(*layers)


class ResNet20(_ResNet):
    """Stem Conv2d(3,16,3) and the 1x1 `fc` + BatchNorm head stay multiply-based; the 18 3x3 layers
    and the two stride-2 1x1 shortcuts are adder layers (resnet20.py:44-93)."""

    def __init__(self, conv=None, num_classes=10, fused_bn=None):
        super().__init__()
        self.norm = _norm_class(conv is None if fused_bn is None else fused_bn)
        conv = conv or _default_conv()
        self.inplanes = 16
        self.conv1 = nn.Conv2d(3, 16, kernel_size=3, stride=1, padding=1, bias=False)
        self.bn1 = self.norm(16)
        self.relu = nn.ReLU(inplace=True)
        self.layer1 = self._make_layer(conv, BasicBlock, 16, 3)
        self.layer2 = self._make_layer(conv, BasicBlock, 32, 3, stride=2)
        self.layer3 = self._make_layer(conv, BasicBlock, 64, 3, stride=2)
        self.avgpool = nn.AvgPool2d(8, stride=1)
        self.fc = nn.Conv2d(64, num_classes, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(num_classes)

    def forward(self, x):
        x = _bn_act(self.bn1, self.conv1(x), relu=True)
        x = self.layer3(self.layer2(self.layer1(x)))
        x = self.bn2(self.fc(self.avgpool(x)))
        return x.view(x.size(0), -1)


class ResNet50(_ResNet):
    """Stem Conv2d(3,64,7,s2) + maxpool and the 1x1 `fc` (with bias) + BatchNorm head stay
    multiply-based; all 52 other convolutions are adder layers (resnet50.py:58-115)."""

    def __init__(self, conv=None, num_classes=1000, fused_bn=None):
        super().__init__()
        self.norm = _norm_class(conv is None if fused_bn is None else fused_bn)
        conv = conv or _default_conv()
        self.inplanes = 64
        self.conv1 = nn.Conv2d(3, 64, kernel_size=7, stride=2, padding=3, bias=False)
        self.bn1 = self.norm(64)
        self.relu = nn.ReLU(inplace=True)
        self.maxpool = nn.MaxPool2d(kernel_size=3, stride=2, padding=1)
        self.layer1 = self._make_layer(conv, Bottleneck, 64, 3)
        self.layer2 = self._make_layer(conv, Bottleneck, 128, 4, stride=2)
        self.layer3 = self._make_layer(conv, Bottleneck, 256, 6, stride=2)
        self.layer4 = self._make_layer(conv, Bottleneck, 512, 3, stride=2)
        self.avgpool = nn.AdaptiveAvgPool2d((1, 1))
        self.fc = nn.Conv2d(2048, num_classes, 1)
        self.bn2 = nn.BatchNorm2d(num_classes)

    def forward(self, x):
        x = self.maxpool(_bn_act(self.bn1, self.conv1(x), relu=True))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        x = self.bn2(self.fc(self.avgpool(x)))
        return x.view(x.size(0), -1)


def resnet20(**kw):
    return ResNet20(**kw)


def resnet50(**kw):
    return ResNet50(**kw)


def init_seeded(model: nn.Module, seed: int) -> None:
    """Deterministic, platform-independent initialisation for parity runs and benchmarks.

    Every parameter is drawn from a NumPy PCG64 stream in state-dict order: adder and convolution
    weights Kaiming-normal with std sqrt(2 / fan_in); BatchNorm weight 1, bias 0 (as the reference
    constructors set them, resnet20.py:59-62); other biases 0.  The same call on a reference-built
    network with the same key order gives bit-identical weights.
    """
    rng = np.random.default_rng(seed)
    with torch.no_grad():
        for name, p in model.state_dict().items():
            if not torch.is_floating_point(p):
                continue
            leaf = name.rsplit(".", 1)[-1]
            if p.dim() == 4:
                fan_in = p.shape[1] * p.shape[2] * p.shape[3]
                v = rng.standard_normal(tuple(p.shape)).astype(np.float32) * np.float32(math.sqrt(2.0 / fan_in))
                p.copy_(torch.from_numpy(v))
            elif p.dim() == 2:     # nn.Linear (the classifier of vgg.py:27-40): Kaiming-normal as well
                v = rng.standard_normal(tuple(p.shape)).astype(np.float32) * np.float32(math.sqrt(2.0 / p.shape[1]))
                p.copy_(torch.from_numpy(v))
            elif leaf == "running_var" or (leaf == "weight" and p.dim() == 1):
                p.fill_(1.0)
            else:
                p.zero_()
