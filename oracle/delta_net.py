"""Network-level CPU oracle (TEST INFRASTRUCTURE): the stateful layer lifecycle of the reference's
module API (src/deltacnn/sparse_layers.py) restated over the CPU operator oracle
(oracle/delta_ops.py), so that whole networks can be stepped frame by frame on a CPU and compared
with the CUDA path, and timed as the CPU baseline. Never imported by the product.

The networks themselves come from ``examples.nets`` through its ops-factory: ``OracleOps`` supplies
CPU layers that keep the same parameter names as the dense and the delta networks.
Parity status: unpinned by the reference (it has no tests); pinned by threshold-0 equivalence with
the dense network (tests/test_oracle_cpu.py) and by the recorded reference-kernel fixtures that
pin the operator oracle underneath.
"""
import torch
import torch.nn as nn

from . import delta_ops as O

_ACT_CODE = {None: 0, "relu": 1, "relu6": 2}


class Thresholds:
    """Per-layer thresholds in frame-0 registration order (DCThreshold, sparse_layers.py:122-208)."""
    default = 0.0
    table = {}

    @classmethod
    def reset(cls):
        cls.table = {}
        cls.default = 0.0

    @classmethod
    def register(cls, key):
        cls.table.setdefault(key, cls.default)

    @classmethod
    def get(cls, key):
        return cls.table.get(key, 0.0)

    @classmethod
    def set_depth_table(cls, input_threshold, first, last):
        keys = list(cls.table.keys())
        acts = [k for k in keys if not isinstance(k, OracleSparsify)]
        for k in keys:
            if isinstance(k, OracleSparsify):
                cls.table[k] = input_threshold
            else:
                cls.table[k] = first + (last - first) * (acts.index(k) / max(len(acts) - 1, 1))


class OracleActivation(nn.Module):
    """DCActivation lifecycle (sparse_layers.py:1378-1417)."""

    def __init__(self, act):
        super().__init__()
        self.code = _ACT_CODE[act]
        self.prev_out = None
        self.truncated = None

    def forward(self, xm):
        x, m = xm
        if self.prev_out is None:
            Thresholds.register(self)
            self.prev_out = x.clone()
            self.truncated = torch.zeros_like(x)
            return O.activation_fn(x.float(), self.code).to(x.dtype), m
        x, m = x.clone(), m.clone()
        O.activate_truncate(x, self.prev_out, self.truncated, m, Thresholds.get(self), self.code, O.TRUNC_MAX)
        return x, m


class OracleConv(nn.Module):
    """DCConv2d / DCConvTranspose2d lifecycle: bias only on the first frame (sparse_layers.py:616),
    optional activation layer (:636-638)."""

    def __init__(self, cin, cout, k, stride=1, padding=0, groups=1, act=None, transposed=False):
        super().__init__()
        if transposed:
            self.conv = nn.ConvTranspose2d(cin, cout, k, stride, padding, bias=True)
        else:
            self.conv = nn.Conv2d(cin, cout, k, stride, padding, groups=groups, bias=True)
        self.transposed = transposed
        self.act = OracleActivation(act) if act is not None else None
        self.frame = -1

    def forward(self, xm):
        x, m = xm
        self.frame += 1
        c = self.conv
        bias = c.bias if self.frame == 0 else None
        if self.transposed:
            out = O.deconv(x, m, c.weight, bias, c.stride, c.padding)
        else:
            out = O.conv(x, m, c.weight, bias, c.stride, c.padding, c.dilation, c.groups)
        return self.act(out) if self.act is not None else out


class OracleAdd(nn.Module):
    """DCAdd lifecycle (sparse_layers.py:1101-1174)."""

    def __init__(self, act=None):
        super().__init__()
        self.code = _ACT_CODE[act]
        self.prev_out = None

    def forward(self, a, b):
        if self.prev_out is None and self.code > 0:
            self.prev_out = torch.zeros_like(a[0])
        return O.add(a[0], a[1], b[0], b[1], self.prev_out, 1.0, 1.0, self.code, False)


class OracleMaxPool(nn.Module):
    """DCMaxPooling lifecycle (sparse_layers.py:1441-1469)."""

    def __init__(self, k, stride, padding):
        super().__init__()
        self.k, self.s, self.p = (k, k), (stride, stride), (padding, padding)
        self.prev_in = None

    def forward(self, xm):
        x, m = xm
        if self.prev_in is None:
            self.prev_in = torch.zeros_like(x)
        out = O.max_pool(x, m, self.prev_in, self.k, self.s, self.p)
        O.add_to_dense(x, self.prev_in, m)
        return out


class OracleAvgPool(nn.Module):
    def forward(self, xm):
        return O.global_avg_pool(xm[0], xm[1])


class OracleUpsample(nn.Module):
    def __init__(self, scale):
        super().__init__()
        self.scale = scale

    def forward(self, xm):
        return O.upsample(xm[0], xm[1], self.scale)


class OracleSparsify(nn.Module):
    """DCSparsify lifecycle (sparse_layers.py:1210-1264)."""

    def __init__(self):
        super().__init__()
        self.prev_in = None

    def forward(self, x):
        if self.prev_in is None:
            Thresholds.register(self)
            self.prev_in = x.clone()
            return x, torch.ones_like(x[:, :1], dtype=torch.int32)
        delta = torch.zeros_like(x)
        mask = torch.zeros_like(x[:, :1], dtype=torch.int32)
        O.sparsify(x, self.prev_in, delta, mask, Thresholds.get(self))
        return delta, mask


class OracleDensify(nn.Module):
    """DCDensify lifecycle (sparse_layers.py:1287-1329)."""

    def __init__(self):
        super().__init__()
        self.prev_out = None

    def forward(self, xm):
        x, m = xm
        if self.prev_out is None:
            self.prev_out = torch.zeros_like(x)
        return O.densify(x, m, self.prev_out, 0)


class OracleOps:
    delta = False          # plain nn.Module containers
    base = nn.Module
    linear = nn.Linear     # the reference's tail: densify, then a dense linear layer (example/mobilenet_deltacnn.py:216-227)
    conv = OracleConv
    add = OracleAdd
    sparsify = OracleSparsify
    densify = OracleDensify

    @staticmethod
    def deconv(cin, cout, k, stride, padding, act=None):
        return OracleConv(cin, cout, k, stride, padding, act=act, transposed=True)

    @staticmethod
    def maxpool(k, stride, padding):
        return OracleMaxPool(k, stride, padding)

    @staticmethod
    def avgpool():
        return OracleAvgPool()

    @staticmethod
    def upsample(scale):
        return OracleUpsample(scale)

    @staticmethod
    def keypoints():
        from examples.nets import DenseOps
        return nn.Sequential(OracleDensify(), DenseOps.keypoints())

    @staticmethod
    def boxes(**kw):
        from examples.nets import DenseOps
        return DenseOps.boxes(**kw)


def build_oracle_net(name, folded_state_dict, **kwargs):
    """CPU delta network of configuration ``name`` carrying the weights of a folded dense network."""
    from examples.nets import BUILDERS
    Thresholds.reset()
    net = BUILDERS[name](OracleOps, **kwargs)
    net.load_state_dict(folded_state_dict)
    return net.eval()
