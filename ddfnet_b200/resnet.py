"""DDF-ResNet measurement harness: bottleneck ResNets whose 3x3 convolution
(``conv2`` of every block) is a DDFPack, as the reference builds them on top of
timm (ddf_resnet.py:34-63: ``DDFPack(width, kernel_size=3, stride=stride,
dilation=first_dilation, se_ratio=0.2, kernel_combine=...)``; layer lists at
ddf_resnet.py:66-111).  timm is not a dependency here: the surrounding network
is the standard ImageNet bottleneck layout (7x7/2 stem, 3x3/2 max-pool, stride
on conv2, 1x1-conv + BN projection shortcuts, global pool + FC), written out in
plain PyTorch.  Parameter counts match the reference's model table
(README.md:21-24): 16.8 M for the 50-layer and 28.1 M for the 101-layer net.

Only the ``ddf`` call inside DDFPack reaches the CUDA kernels; this file exists
to measure whole-network inference throughput with the op in place.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .layout import to_channels_last
from .modules import DDFPack, _derived


class DDFBottleneck(nn.Module):
    expansion = 4

    def __init__(self, inplanes, planes, stride=1, downsample=None, kernel_combine='mul',
                 se_ratio=0.2):
        super().__init__()
        width = planes
        self.conv1 = nn.Conv2d(inplanes, width, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        self.act1 = nn.ReLU(inplace=True)
        self.conv2 = DDFPack(width, kernel_size=3, stride=stride, dilation=1,
                             se_ratio=se_ratio, kernel_combine=kernel_combine)
        self.bn2 = nn.BatchNorm2d(width)
        self.act2 = nn.ReLU(inplace=True)
        self.conv3 = nn.Conv2d(width, planes * self.expansion, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(planes * self.expansion)
        self.act3 = nn.ReLU(inplace=True)
        self.downsample = downsample
        self.fused_inference = False  # set by fold_batchnorm(..., fuse_activations=True)

    def forward(self, x):
        if self.fused_inference:
            return self._forward_fused(x)
        shortcut = x
        x = self.act1(self.bn1(self.conv1(x)))
        x = self.act2(self.bn2(self.conv2(x)))
        x = self.bn3(self.conv3(x))
        if self.downsample is not None:
            shortcut = self.downsample(shortcut)
        return self.act3(x + shortcut)

    def _bn2_scale_shift(self, device):
        # The eval-mode BatchNorm after the DDFPack as a float32 per-channel affine map; kept
        # outside the module's buffers so that .half() / .to(dtype) leave it in float32.
        bn = self.bn2
        key = tuple((t.data_ptr(), t._version) for t in (bn.weight, bn.bias, bn.running_mean, bn.running_var))
        cache = _derived(self).get("bn2_affine")
        if cache is None or cache[0] != key or cache[1].device != device:
            scale = bn.weight.detach().float() / torch.sqrt(bn.running_var.float() + bn.eps)
            shift = bn.bias.detach().float() - bn.running_mean.float() * scale
            cache = (key, scale.contiguous().to(device), shift.contiguous().to(device))
            _derived(self)["bn2_affine"] = cache
        return cache[1], cache[2]

    def _forward_fused(self, x):
        # After fold_batchnorm: conv1 + bias + ReLU and conv3 + bias + shortcut + ReLU each as
        # one cuDNN call instead of conv, BatchNorm, (add,) ReLU kernels.
        shortcut = x if self.downsample is None else self.downsample(x)
        c1, c3 = self.conv1, self.conv3
        x = torch.cudnn_convolution_relu(x, c1.weight, c1.bias, c1.stride, c1.padding, c1.dilation, 1)
        if x.is_contiguous(memory_format=torch.channels_last) and not x.is_contiguous():
            # channels_last network: the channels-innermost DDF kernel takes the tensor as it is and
            # applies BatchNorm + ReLU on its store
            y = self.conv2.forward_channels_last(x, *self._bn2_scale_shift(x.device), relu=True)
            if y is not None:
                return torch.cudnn_convolution_add_relu(y, c3.weight, shortcut, 1.0, c3.bias, c3.stride,
                                                        c3.padding, c3.dilation, 1)
        x = self.conv2(x)  # DDFPack: contiguous NCHW out (or channels_last from its own NHWC path)
        if x.is_contiguous(memory_format=torch.channels_last) and not x.is_contiguous():
            x = self.act2(self.bn2(x))
        elif shortcut.is_contiguous(memory_format=torch.channels_last) and not shortcut.is_contiguous():
            # channels_last network: BatchNorm + ReLU ride on the conversion back to NHWC
            x = to_channels_last(x, *self._bn2_scale_shift(x.device), relu=True)
        else:
            x = self.act2(self.bn2(x))
        return torch.cudnn_convolution_add_relu(x, c3.weight, shortcut, 1.0, c3.bias, c3.stride,
                                                c3.padding, c3.dilation, 1)


class DDFResNet(nn.Module):
    def __init__(self, layers, kernel_combine='mul', num_classes=1000, se_ratio=0.2):
        super().__init__()
        self.inplanes = 64
        self.conv1 = nn.Conv2d(3, 64, 7, stride=2, padding=3, bias=False)
        self.bn1 = nn.BatchNorm2d(64)
        self.act1 = nn.ReLU(inplace=True)
        self.maxpool = nn.MaxPool2d(3, stride=2, padding=1)
        self.layer1 = self._make_layer(64, layers[0], 1, kernel_combine, se_ratio)
        self.layer2 = self._make_layer(128, layers[1], 2, kernel_combine, se_ratio)
        self.layer3 = self._make_layer(256, layers[2], 2, kernel_combine, se_ratio)
        self.layer4 = self._make_layer(512, layers[3], 2, kernel_combine, se_ratio)
        self.global_pool = nn.AdaptiveAvgPool2d(1)
        self.fc = nn.Linear(512 * DDFBottleneck.expansion, num_classes)
        self.fused_inference = False
        self.init_weights()

    def _make_layer(self, planes, blocks, stride, kernel_combine, se_ratio):
        downsample = None
        if stride != 1 or self.inplanes != planes * DDFBottleneck.expansion:
            downsample = nn.Sequential(
                nn.Conv2d(self.inplanes, planes * DDFBottleneck.expansion, 1, stride=stride, bias=False),
                nn.BatchNorm2d(planes * DDFBottleneck.expansion))
        layers = [DDFBottleneck(self.inplanes, planes, stride, downsample, kernel_combine, se_ratio)]
        self.inplanes = planes * DDFBottleneck.expansion
        for _ in range(1, blocks):
            layers.append(DDFBottleneck(self.inplanes, planes, 1, None, kernel_combine, se_ratio))
        return nn.Sequential(*layers)

    def init_weights(self):
        """Kaiming-normal (fan_out, relu) convolutions, BN gamma = 1 / beta = 0."""
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode='fan_out', nonlinearity='relu')
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.ones_(m.weight)
                nn.init.zeros_(m.bias)

    def forward(self, x):
        if self.fused_inference:
            c = self.conv1
            x = self.maxpool(torch.cudnn_convolution_relu(x, c.weight, c.bias, c.stride, c.padding,
                                                          c.dilation, 1))
            x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
            return self.fc(torch.flatten(self.global_pool(x), 1))
        x = self.maxpool(self.act1(self.bn1(self.conv1(x))))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.fc(torch.flatten(self.global_pool(x), 1))

    def ddf_layers(self):
        """The DDFPack modules in network order."""
        return [m for m in self.modules() if isinstance(m, DDFPack)]


def _fold(conv: nn.Conv2d, bn: nn.BatchNorm2d) -> nn.Conv2d:
    """conv followed by an eval-mode BatchNorm as one convolution with a bias."""
    scale = bn.weight / torch.sqrt(bn.running_var + bn.eps)
    out = nn.Conv2d(conv.in_channels, conv.out_channels, conv.kernel_size, conv.stride, conv.padding,
                    conv.dilation, conv.groups, bias=True).to(conv.weight.device, conv.weight.dtype)
    with torch.no_grad():
        out.weight.copy_(conv.weight * scale.reshape(-1, 1, 1, 1).to(conv.weight.dtype))
        bias = conv.bias if conv.bias is not None else torch.zeros_like(bn.running_mean)
        out.bias.copy_(((bias - bn.running_mean) * scale + bn.bias).to(conv.weight.dtype))
    return out


def fold_batchnorm(model: "DDFResNet", fuse_activations: bool = False) -> "DDFResNet":
    """Inference-only rewrite, in place: every BatchNorm that directly follows a convolution
    (stem, conv1 / conv3 of each block, projection shortcuts) is folded into that
    convolution's weights and bias.  The BatchNorm after each DDFPack stays: the DDF output
    is not linear in any stored weight.  The model must be in eval mode.

    fuse_activations=True (CUDA only) additionally routes conv + bias + ReLU and
    conv + bias + shortcut + ReLU through cuDNN's fused convolution calls."""
    assert not model.training, "fold_batchnorm is for eval-mode models"
    model.fused_inference = fuse_activations
    for m in model.modules():
        if isinstance(m, DDFBottleneck):
            m.fused_inference = fuse_activations
    model.conv1, model.bn1 = _fold(model.conv1, model.bn1), nn.Identity()
    for m in model.modules():
        if isinstance(m, DDFBottleneck):
            m.conv1, m.bn1 = _fold(m.conv1, m.bn1), nn.Identity()
            m.conv3, m.bn3 = _fold(m.conv3, m.bn3), nn.Identity()
            if m.downsample is not None:
                m.downsample = nn.Sequential(_fold(m.downsample[0], m.downsample[1]))
                if fuse_activations:
                    # relu(conv3(x) + b3 + (conv_d(s) + b_d)): one bias instead of two, and no
                    # separate bias-add kernel over the widest tensor of the block
                    with torch.no_grad():
                        m.conv3.bias.add_(m.downsample[0].bias)
                    m.downsample[0].bias = None
    return model


_LAYERS = {50: [3, 4, 6, 3], 101: [3, 4, 23, 3], 152: [3, 8, 36, 3]}


def ddf_mul_resnet50(**kw):
    return DDFResNet(_LAYERS[50], 'mul', **kw)


def ddf_mul_resnet101(**kw):
    return DDFResNet(_LAYERS[101], 'mul', **kw)


def ddf_mul_resnet152(**kw):
    return DDFResNet(_LAYERS[152], 'mul', **kw)


def ddf_add_resnet50(**kw):
    return DDFResNet(_LAYERS[50], 'add', **kw)


def ddf_add_resnet101(**kw):
    return DDFResNet(_LAYERS[101], 'add', **kw)


def ddf_add_resnet152(**kw):
    return DDFResNet(_LAYERS[152], 'add', **kw)


MODELS = {f.__name__: f for f in (ddf_mul_resnet50, ddf_mul_resnet101, ddf_mul_resnet152,
                                  ddf_add_resnet50, ddf_add_resnet101, ddf_add_resnet152)}
