"""The networks of the benchmark configurations, each written once against a small "ops"
factory so that the dense PyTorch model (the equivalence anchor) and the delta model (DC*
modules) share structure, parameter names and weights:

  MobileNetV2 (width 1.0)          -- the reference's example network (example/mobilenet_deltacnn.py)
  ResNet-50                        -- bottlenecks, DCAdd residuals + ReLU, 3x3/2 max pool, global average pool
  HRNet-W32 style pose network     -- four resolution branches, nearest upsampling fusion, 17 heat maps
  CenterNet style detector         -- ResNet-18, three 4x4/2 transposed convolutions, three heads

Convolutions are built as conv + BatchNorm + activation; ``calibrate_and_fold`` sets the BatchNorm
statistics from frames of the synthetic video (so that randomly initialised networks keep
unit-scale activations at every depth) and folds them into the convolution weights and a bias.
The delta network is then built with folded convolutions (bias=True, fused activation) and loads
the folded state dict.

This module itself never imports the CUDA library: the delta factory lives in ``nets_delta`` and is imported
by ``build_pair`` only when a delta model is asked for, so dense baselines can be built without loading it.
"""
import torch
import torch.nn as nn

_ACTS = {None: nn.Identity, "relu": nn.ReLU, "relu6": nn.ReLU6}
DELTA_HEADS = True      # delta networks end in DCLinear on the pooled delta instead of DCDensify + a dense linear layer


class DenseConv(nn.Module):
    """conv (+BatchNorm until folded) + activation on dense tensors."""

    def __init__(self, cin, cout, k, stride=1, padding=0, groups=1, act=None, transposed=False):
        super().__init__()
        if transposed:
            self.conv = nn.ConvTranspose2d(cin, cout, k, stride, padding, bias=False)
        else:
            self.conv = nn.Conv2d(cin, cout, k, stride, padding, groups=groups, bias=False)
        self.bn = nn.BatchNorm2d(cout, momentum=None)
        self.act = _ACTS[act]()
        self.transposed = transposed

    def forward(self, x):
        x = self.conv(x)
        if self.bn is not None:
            x = self.bn(x)
        return self.act(x)

    def fold(self):
        if self.bn is None:
            return
        scale = self.bn.weight * torch.rsqrt(self.bn.running_var + self.bn.eps)
        shape = (1, -1, 1, 1) if self.transposed else (-1, 1, 1, 1)
        self.conv.weight.data = self.conv.weight.data * scale.view(shape)
        self.conv.bias = nn.Parameter(self.bn.bias.data - self.bn.running_mean * scale)
        self.bn = None


class _DenseAdd(nn.Module):
    def __init__(self, act=None):
        super().__init__()
        self.act = _ACTS[act]()

    def forward(self, a, b):
        return self.act(a + b)


class DenseOps:
    delta = False
    base = nn.Module
    conv = DenseConv
    add = _DenseAdd

    @staticmethod
    def deconv(cin, cout, k, stride, padding, act=None):
        return DenseConv(cin, cout, k, stride, padding, act=act, transposed=True)

    @staticmethod
    def maxpool(k, stride, padding):
        return nn.MaxPool2d(k, stride, padding)

    @staticmethod
    def avgpool():
        return nn.AdaptiveAvgPool2d((1, 1))

    @staticmethod
    def upsample(scale):
        return nn.UpsamplingNearest2d(scale_factor=scale)

    sparsify = nn.Identity
    densify = nn.Identity
    linear = nn.Linear

    class keypoints(nn.Module):
        """(x, y, value) of the largest element of every heat map: the dense anchor of DCHeatmapArgmax."""

        def forward(self, heat):
            n, j, h, w = heat.shape
            val, idx = heat.float().reshape(n, j, h * w).max(dim=2)
            return torch.stack(((idx % w).float(), (idx // w).float(), val), dim=2)

    class boxes(nn.Module):
        """CenterNet decode with torch operators: the dense anchor of DCCenterNetDecode (same tie order)."""

        def __init__(self, topk=100, min_score=0.0, stride=4.0):
            super().__init__()
            self.topk, self.min_score, self.stride = topk, min_score, stride

        def forward(self, heat, wh, off):
            n, c, h, w = heat.shape
            hf = heat.float()
            peak = (torch.nn.functional.max_pool2d(hf, 3, 1, 1) == hf) & (hf > self.min_score)
            score = torch.where(peak, hf, torch.full_like(hf, float("-inf"))).permute(0, 2, 3, 1).reshape(n, -1)
            val, idx = torch.sort(score, dim=1, descending=True, stable=True)
            val, idx = val[:, :self.topk], idx[:, :self.topk]
            ok = torch.isfinite(val)
            cls, pix = idx % c, idx // c
            x, y = (pix % w).float(), (pix // w).float()
            g = lambda t, ch: t.float()[:, ch].reshape(n, -1).gather(1, pix)
            cx, cy, bw, bh = x + g(off, 0), y + g(off, 1), g(wh, 0), g(wh, 1)
            okf = ok.float()
            det = torch.stack(((cx - bw / 2) * self.stride * okf, (cy - bh / 2) * self.stride * okf, (cx + bw / 2) * self.stride * okf,
                               (cy + bh / 2) * self.stride * okf, torch.sigmoid(val) * okf, cls.float() * okf - (1.0 - okf)), dim=2)
            return det, ok.sum(dim=1).to(torch.int32)


def _conv_then_add(ops, conv, h, idt, add):
    """add(conv(h), idt). In the delta network the convolution adds the residual (and applies the add layer's
    activation) in its own epilogue where it has a kernel for that: one launch instead of two."""
    if ops.delta:
        inner = conv.conv
        if inner.can_fuse_residual(h, add):
            return inner(h, residual=idt, add_layer=add)
    return add(conv(h), idt)


def _base(ops):
    return ops.base


def depth_stages_of(front, blocks, tail, cuts):
    """A network ``tail(blocks[-1](... blocks[0](front(frame))))`` as consecutive stages for a frame pipeline
    (deltacnn_b200/stepping.py, DepthPipeline): ``cuts`` are the indices into ``blocks`` where a new stage starts. Returns one
    callable per stage; the first takes the frame batch, the others the previous stage's output, the last returns what
    the network returns. Called in order on one frame they are the network's forward pass."""
    blocks = list(blocks)
    edges = [0] + [int(c) for c in cuts] + [len(blocks)]
    assert all(a < b for a, b in zip(edges, edges[1:])), "cuts must be increasing indices inside the block list"

    def make(si):
        lo, hi = edges[si], edges[si + 1]
        first, last = si == 0, si == len(edges) - 2

        def stage(x):
            if first:
                x = front(x)
            for b in blocks[lo:hi]:
                x = b(x)
            return tail(x) if last else x
        return stage
    return [make(si) for si in range(len(edges) - 1)]


# ------------------------------------------------------------------------------------------------
# MobileNetV2
# ------------------------------------------------------------------------------------------------
def make_mobilenet_v2(ops, num_classes=1000):
    Base = _base(ops)

    class InvertedResidual(Base):
        def __init__(self, inp, oup, stride, expand):
            super().__init__()
            hidden = int(round(inp * expand))
            self.use_res = stride == 1 and inp == oup
            layers = []
            if expand != 1:
                layers.append(ops.conv(inp, hidden, 1, act="relu6"))
            layers.append(ops.conv(hidden, hidden, 3, stride, 1, groups=hidden, act="relu6"))
            layers.append(ops.conv(hidden, oup, 1))
            self.conv = nn.Sequential(*layers)
            if self.use_res:
                self.add = ops.add()
                layers[-1].residual_last = True
            # delta networks: the whole block as one kernel where the library has one (small maps, steady-state frames)
            self.fused = ops.fused_block(*layers) if (ops.delta and expand != 1) else None

        def forward(self, x):
            if self.fused is not None and self.fused.ready(x, self.use_res):
                return self.fused(x, self.use_res)
            if not self.use_res:
                return self.conv(x)
            if ops.delta:
                # the projection convolution adds the residual itself where it has a kernel for it (one launch less)
                h = x
                for layer in list(self.conv)[:-1]:
                    h = layer(h)
                proj = self.conv[-1].conv
                if proj.can_fuse_residual(h):
                    return proj(h, residual=x)
                return self.add(x, proj(h))
            return self.add(x, self.conv(x))

    class MobileNetV2(Base):
        def __init__(self):
            super().__init__()
            setting = [[1, 16, 1, 1], [6, 24, 2, 2], [6, 32, 3, 2], [6, 64, 4, 2], [6, 96, 3, 1], [6, 160, 3, 2], [6, 320, 1, 1]]
            feats = [ops.conv(3, 32, 3, 2, 1, act="relu6")]
            cin = 32
            for t, c, n, s in setting:
                for i in range(n):
                    feats.append(InvertedResidual(cin, c, s if i == 0 else 1, t))
                    cin = c
            feats.append(ops.conv(cin, 1280, 1, act="relu6"))
            self.features = nn.Sequential(*feats)
            self.sparsify = ops.sparsify()
            self.pool = ops.avgpool()
            self.densify = ops.densify()
            self.classifier = ops.linear(1280, num_classes)

        def tail(self, x):
            x = self.pool(x)
            if ops.delta and DELTA_HEADS:
                return self.classifier(x)           # the classifier consumes the pooled delta: no dense feature vector
            x = self.densify(x)
            return self.classifier(x.reshape(x.shape[0], -1))

        def forward(self, x):
            return self.tail(self.features(self.sparsify(x)))

        def depth_stages(self, cuts):
            """Stages for a frame pipeline; ``cuts`` are indices into ``features`` where a new stage starts."""
            return depth_stages_of(self.sparsify, self.features, self.tail, cuts)

    return MobileNetV2()


# ------------------------------------------------------------------------------------------------
# ResNet-50 / ResNet-18 trunks
# ------------------------------------------------------------------------------------------------
def _make_resnet_parts(ops):
    Base = _base(ops)

    class Bottleneck(Base):
        def __init__(self, cin, width, stride):
            super().__init__()
            cout = width * 4
            self.c1 = ops.conv(cin, width, 1, act="relu")
            self.c2 = ops.conv(width, width, 3, stride, 1, act="relu")
            self.c3 = ops.conv(width, cout, 1)
            self.down = ops.conv(cin, cout, 1, stride) if (stride != 1 or cin != cout) else None
            self.add = ops.add("relu")
            self.c3.residual_last = True

        def forward(self, x):
            idt = x if self.down is None else self.down(x)
            return _conv_then_add(ops, self.c3, self.c2(self.c1(x)), idt, self.add)

    class Basic(Base):
        def __init__(self, cin, cout, stride):
            super().__init__()
            self.c1 = ops.conv(cin, cout, 3, stride, 1, act="relu")
            self.c2 = ops.conv(cout, cout, 3, 1, 1)
            self.down = ops.conv(cin, cout, 1, stride) if (stride != 1 or cin != cout) else None
            self.add = ops.add("relu")
            self.c2.residual_last = True

        def forward(self, x):
            idt = x if self.down is None else self.down(x)
            return _conv_then_add(ops, self.c2, self.c1(x), idt, self.add)

    return Base, Bottleneck, Basic


def make_resnet50(ops, num_classes=1000, widths=(64, 128, 256, 512), blocks=(3, 4, 6, 3)):
    Base, Bottleneck, _ = _make_resnet_parts(ops)

    class ResNet50(Base):
        def __init__(self):
            super().__init__()
            self.sparsify = ops.sparsify()
            self.stem = ops.conv(3, 64, 7, 2, 3, act="relu")
            self.maxpool = ops.maxpool(3, 2, 1)
            layers, cin = [], 64
            for i, (w, n) in enumerate(zip(widths, blocks)):
                for j in range(n):
                    layers.append(Bottleneck(cin, w, (2 if i > 0 else 1) if j == 0 else 1))
                    cin = w * 4
            self.layers = nn.Sequential(*layers)
            self.pool = ops.avgpool()
            self.densify = ops.densify()
            self.fc = ops.linear(cin, num_classes)

        def front(self, x):
            return self.maxpool(self.stem(self.sparsify(x)))

        def tail(self, x):
            x = self.pool(x)
            if ops.delta and DELTA_HEADS:
                return self.fc(x)
            x = self.densify(x)
            return self.fc(x.reshape(x.shape[0], -1))

        def forward(self, x):
            return self.tail(self.layers(self.front(x)))

        def depth_stages(self, cuts):
            """Stages for a frame pipeline; ``cuts`` are indices into ``layers`` (16 blocks) where a new stage starts."""
            return depth_stages_of(self.front, self.layers, self.tail, cuts)

    return ResNet50()


def make_centernet(ops, head_channels=64, decode=False):
    """ResNet-18 trunk, three 4x4 stride-2 transposed convolutions (256 channels, BN, ReLU) and
    three heads (3x3 conv + ReLU + 1x1 conv): heat map (1), size (2), offset (2). With ``decode`` the network
    returns boxes (det (N, 100, 6), count) instead of the three dense maps."""
    Base, _, Basic = _make_resnet_parts(ops)

    class Head(Base):
        def __init__(self, cin, cout):
            super().__init__()
            self.c1 = ops.conv(cin, head_channels, 3, 1, 1, act="relu")
            self.c2 = ops.conv(head_channels, cout, 1)
            self.densify = ops.densify()

        def forward(self, x, dense=True):
            return self.tail(self.c1(x), dense)

        def tail(self, x, dense=True):            # everything behind the 3x3 layer
            x = self.c2(x)
            return self.densify(x) if dense else x

    class CenterNet(Base):
        def __init__(self):
            super().__init__()
            self.sparsify = ops.sparsify()
            self.stem = ops.conv(3, 64, 7, 2, 3, act="relu")
            self.maxpool = ops.maxpool(3, 2, 1)
            layers, cin = [], 64
            for i, w in enumerate((64, 128, 256, 512)):
                for j in range(2):
                    layers.append(Basic(cin, w, 2 if (i > 0 and j == 0) else 1))
                    cin = w
            self.layers = nn.Sequential(*layers)
            ups = []
            for _ in range(3):
                ups.append(ops.deconv(cin, 256, 4, 2, 1, act="relu"))
                cin = 256
            self.ups = nn.Sequential(*ups)
            self.hm, self.wh, self.off = Head(256, 1), Head(256, 2), Head(256, 2)
            self.boxes = ops.boxes() if decode else None
            # the three heads' 3x3 layers read the same map: one kernel on steady-state frames of the delta network
            self.fused_heads = ops.fused_heads([self.hm.c1, self.wh.c1, self.off.c1]) if ops.delta else None

        def front(self, x):
            return self.maxpool(self.stem(self.sparsify(x)))

        def tail(self, x):
            dense = self.boxes is None or not ops.delta     # the delta decode accumulates the three head deltas itself
            heads = (self.hm, self.wh, self.off)
            if self.fused_heads is not None and self.fused_heads.ready(x):
                outs = [h.tail(t, dense) for h, t in zip(heads, self.fused_heads(x))]
            else:
                outs = [h(x, dense) for h in heads]
            return tuple(outs) if self.boxes is None else self.boxes(*outs)

        def forward(self, x):
            return self.tail(self.ups(self.layers(self.front(x))))

        def depth_stages(self, cuts):
            """Stages for a frame pipeline; ``cuts`` are indices into the eight trunk blocks followed by the three
            transposed convolutions (0..10) where a new stage starts."""
            return depth_stages_of(self.front, list(self.layers) + list(self.ups), self.tail, cuts)

    return CenterNet()


# ------------------------------------------------------------------------------------------------
# HRNet-W32 style pose network
# ------------------------------------------------------------------------------------------------
def make_hrnet_w32(ops, n_joints=17, width=32, blocks_per_branch=4, modules=(1, 4, 3), decode=False):
    """Stem of two 3x3 stride-2 convolutions to 1/4 resolution; stage 1 of four bottlenecks;
    stages 2-4 with 2/3/4 parallel branches (widths w, 2w, 4w, 8w at 1/4 ... 1/32 resolution) of
    basic 3x3 blocks; every module ends with a full fusion (1x1 conv + nearest upsampling toward
    higher resolution, chains of 3x3 stride-2 convolutions toward lower); a final 1x1 convolution
    gives ``n_joints`` heat maps at 1/4 resolution."""
    Base, Bottleneck, Basic = _make_resnet_parts(ops)

    class Fuse(Base):
        def __init__(self, chans, n_out):
            super().__init__()
            self.n_in, self.n_out = len(chans), n_out
            self.paths = nn.ModuleList()
            self.adds = nn.ModuleList()
            for i in range(n_out):
                row = nn.ModuleList()
                for j in range(self.n_in):
                    if j == i:
                        row.append(nn.Identity())
                    elif j > i:
                        row.append(nn.Sequential(ops.conv(chans[j], chans[i], 1), ops.upsample(2 ** (j - i))))
                    else:
                        seq, c = [], chans[j]
                        for k in range(i - j):
                            last = k == i - j - 1
                            seq.append(ops.conv(c, chans[i] if last else c, 3, 2, 1, act=None if last else "relu"))
                            c = chans[i] if last else c
                        row.append(nn.Sequential(*seq))
                self.paths.append(row)
                self.adds.append(nn.ModuleList([ops.add("relu" if j == self.n_in - 1 else None) for j in range(1, self.n_in)]))

        def forward(self, xs):
            outs = []
            for i in range(self.n_out):
                y = self.paths[i][0](xs[0])
                for j in range(1, self.n_in):
                    y = self.adds[i][j - 1](y, self.paths[i][j](xs[j]))
                outs.append(y)
            return outs

    class HRModule(Base):
        def __init__(self, chans, n_out):
            super().__init__()
            self.branches = nn.ModuleList([nn.Sequential(*[Basic(c, c, 1) for _ in range(blocks_per_branch)]) for c in chans])
            self.fuse = Fuse(chans, n_out)

        def forward(self, xs):
            return self.fuse([b(x) for b, x in zip(self.branches, xs)])

    class HRNet(Base):
        def __init__(self):
            super().__init__()
            self.sparsify = ops.sparsify()
            self.stem = nn.Sequential(ops.conv(3, 64, 3, 2, 1, act="relu"), ops.conv(64, 64, 3, 2, 1, act="relu"))
            self.stage1 = nn.Sequential(Bottleneck(64, 64, 1), *[Bottleneck(256, 64, 1) for _ in range(3)])
            chans = [width, width * 2, width * 4, width * 8]
            self.trans = nn.ModuleList([ops.conv(256, chans[0], 3, 1, 1, act="relu"), ops.conv(256, chans[1], 3, 2, 1, act="relu"),
                                        ops.conv(chans[1], chans[2], 3, 2, 1, act="relu"), ops.conv(chans[2], chans[3], 3, 2, 1, act="relu")])
            self.stage2 = nn.ModuleList([HRModule(chans[:2], 2) for _ in range(modules[0])])
            self.stage3 = nn.ModuleList([HRModule(chans[:3], 3) for _ in range(modules[1])])
            self.stage4 = nn.ModuleList([HRModule(chans[:4], 4 if m < modules[2] - 1 else 1) for m in range(modules[2])])
            self.final = ops.conv(chans[0], n_joints, 1)
            self.densify = ops.densify()
            self.keypoints = ops.keypoints() if decode else None     # (x, y, value) per joint instead of the heat maps

        def front(self, x):
            return self.stage1(self.stem(self.sparsify(x)))

        def blocks(self):
            """The network between ``front`` and ``tail`` as a chain of callables on the list of branch tensors."""
            split = lambda x: [self.trans[0](x), self.trans[1](x)]
            grow = lambda k: (lambda xs: list(xs) + [self.trans[k](xs[-1])])
            return [split, *self.stage2, grow(2), *self.stage3, grow(3), *self.stage4]

        def tail(self, xs):
            x = self.final(xs[0])
            if self.keypoints is not None:
                return self.keypoints(x)
            return self.densify(x)

        def forward(self, x):
            xs = self.front(x)
            for b in self.blocks():
                xs = b(xs)
            return self.tail(xs)

        def depth_stages(self, cuts):
            """Stages for a frame pipeline; ``cuts`` are indices into ``blocks()`` (branch split, the modules of stage 2,
            new branch, the modules of stage 3, new branch, the modules of stage 4) where a new stage starts."""
            return depth_stages_of(self.front, self.blocks(), self.tail, cuts)

    return HRNet()


BUILDERS = {"mobilenet": make_mobilenet_v2, "resnet50": make_resnet50, "hrnet": make_hrnet_w32, "centernet": make_centernet}


def init_weights(model, seed=0, residual_gain=1.0):
    """Kaiming-normal (fan_out) convolutions, unit BatchNorm, N(0, 0.01) classifier -- the
    initialisation of the reference's example constructors (example/mobilenet_original.py:190-200).
    ``residual_gain`` < 1 sets the BatchNorm scale of the last convolution of every residual branch (the usual
    "small last gamma" initialisation): the blocks stay close to the identity, which keeps a randomly initialised
    network from amplifying rounding errors layer by layer."""
    torch.manual_seed(seed)
    for m in model.modules():
        if isinstance(m, (nn.Conv2d, nn.ConvTranspose2d)):
            nn.init.kaiming_normal_(m.weight, mode="fan_out")
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.BatchNorm2d):
            nn.init.ones_(m.weight)
            nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, 0, 0.01)
            nn.init.zeros_(m.bias)
    if residual_gain != 1.0:
        for m in model.modules():
            if getattr(m, "residual_last", False) and getattr(m, "bn", None) is not None:
                nn.init.constant_(m.bn.weight, residual_gain)


@torch.no_grad()
def calibrate_and_fold(dense_model, frames):
    """One training-mode forward over ``frames`` sets every BatchNorm's running statistics to the
    batch statistics (momentum=None: cumulative average), then every BatchNorm is folded."""
    # one host thread: the batch statistics are sums whose order would otherwise follow the thread count. (A process
    # whose thread pool has size one from the start, OMP_NUM_THREADS=1, still takes other kernels of the CPU libraries and
    # folds weights that differ in the last bits: callers that compare runs keep the pool larger than one.)
    threads = torch.get_num_threads()
    torch.set_num_threads(1)
    try:
        dense_model.train()
        dense_model(frames)
        dense_model.eval()
    finally:
        torch.set_num_threads(threads)
    for m in dense_model.modules():
        if isinstance(m, DenseConv):
            m.fold()
    return dense_model


def build_pair(name, calib_frames, seed=0, device="cpu", dtype=torch.float32, residual_gain=1.0, **kwargs):
    """(dense folded model, delta model) with identical weights on ``device``/``dtype``; the delta
    model is ready to run (``process_filters()`` done). ``device`` must be a CUDA device for the
    delta model; with device='cpu' only the dense model is returned (delta is None)."""
    dense = BUILDERS[name](DenseOps, **kwargs)
    init_weights(dense, seed, residual_gain)
    calibrate_and_fold(dense, calib_frames)
    state = dense.state_dict()
    delta = None
    if torch.device(device).type == "cuda":
        from .nets_delta import DeltaOps        # the only place this module touches the CUDA library
        delta = BUILDERS[name](DeltaOps, **kwargs)
        delta.load_state_dict(state)
        delta.eval()
        delta = delta.to(device, memory_format=torch.channels_last)
        if dtype == torch.float16:
            delta = delta.half()
        delta.process_filters()
    dense = dense.to(device, memory_format=torch.channels_last)
    if dtype == torch.float16 and torch.device(device).type == "cuda":
        dense = dense.half()
    return dense, delta
