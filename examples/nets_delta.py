"""The "ops" factory that builds the networks of ``nets`` out of the DC* modules of deltacnn_b200 (the delta
twin of ``nets.DenseOps``): folded delta convolutions with fused activation, DCAdd, delta pooling, and the
device-side heads."""
from deltacnn_b200 import (DCAdaptiveAveragePooling, DCAdd, DCCenterNetDecode, DCConv2d, DCConvTranspose2d, DCDensify, DCFusedHeads,
                           DCFusedInvertedResidual,
                           DCHeatmapArgmax, DCLinear, DCMaxPooling, DCModule, DCSparsify, DCUpsamplingNearest2d)


class DeltaConv(DCModule):
    """Folded delta convolution with fused activation; parameter names match DenseConv."""

    def __init__(self, cin, cout, k, stride=1, padding=0, groups=1, act=None, transposed=False):
        super().__init__()
        if transposed:
            self.conv = DCConvTranspose2d(cin, cout, k, stride, padding, bias=True, activation=act)
        else:
            self.conv = DCConv2d(cin, cout, k, stride, padding, groups=groups, bias=True, activation=act)

    def forward(self, x):
        return self.conv(x)


class DeltaOps:
    delta = True
    base = DCModule
    conv = DeltaConv

    @staticmethod
    def add(act=None):
        return DCAdd(activation=act)

    @staticmethod
    def deconv(cin, cout, k, stride, padding, act=None):
        return DeltaConv(cin, cout, k, stride, padding, act=act, transposed=True)

    @staticmethod
    def maxpool(k, stride, padding):
        return DCMaxPooling(k, stride, padding)

    @staticmethod
    def avgpool():
        return DCAdaptiveAveragePooling((1, 1))

    @staticmethod
    def upsample(scale):
        return DCUpsamplingNearest2d(scale_factor=scale)

    sparsify = DCSparsify
    densify = DCDensify
    linear = DCLinear
    keypoints = DCHeatmapArgmax

    @staticmethod
    def boxes(topk=100, min_score=0.0, stride=4.0):
        return DCCenterNetDecode(topk=topk, min_score=min_score, stride=stride, apply_sigmoid=True)

    @staticmethod
    def fused_block(expand, depthwise, project):
        """One-kernel form of an inverted-residual block built from its three DeltaConv layers."""
        return DCFusedInvertedResidual(expand.conv, depthwise.conv, project.conv)

    @staticmethod
    def fused_heads(convs):
        """One-kernel form of the 3x3 first layers of several heads that read the same feature map."""
        return DCFusedHeads([c.conv for c in convs])

