"""Stateful module API of the delta-update path (drop-in for the reference's
src/deltacnn/sparse_layers.py): the same class names, constructor signatures, tuple
convention ``(delta, mask)`` between layers, first-frame behaviour, threshold registry and
``process_filters()`` / ``reset_layers()`` protocol, driving the sm_100a kernels of this
package through ``cuda_kernels``.

Not carried over (no multi-backend dispatch): the ``delta_cudnn`` soft-threshold training
emulation (reference :37-82, :467-533) and the TensorBoard logging forward (:535-601);
selecting them raises. ``DCBackend.cudnn`` keeps working by delegating to torch, as in the
reference (:449-465).

Per-layer output buffers are allocated once and reused every frame (the reference calls
``torch.empty`` per layer per frame, cuda_kernels.py:34-37), which also makes a whole frame
step capturable in a CUDA graph.
"""
from collections import OrderedDict
from enum import Enum

import torch
import torch.nn as nn
from torch import Tensor

from . import cuda_kernels as K
from .filter_conversion import convert_filter_out_channels_last, convert_half_filter


def convert_activation_string(name, **kwargs):
    """Activation name -> (torch callable, kernel code). Codes as reference :20-34; the kernels'
    leaky slope is 0.1 (src/cuda/other_nn_layers.cu:33) and the torch module uses the same."""
    if name is None or name == "" or name.lower() == "linear":
        return None, -1
    key = name.lower()
    if key == "relu":
        return torch.nn.ReLU(), 1
    if key == "relu6":
        return torch.nn.ReLU6(), 2
    if key == "leaky":
        return torch.nn.LeakyReLU(kwargs.get("leaky_relu_negative_slope", 0.1)), 3
    if key == "sigmoid":
        return torch.nn.Sigmoid(), 4
    if key == "swish":
        return (lambda x: torch.sigmoid(x).mul_(x)), 5
    raise Exception(f"Activation {name} not implemented")


class DCBackend(Enum):
    cudnn = 0
    deltacnn = 1
    delta_cudnn = 2

    @classmethod
    def parse_string(cls, x):
        try:
            return cls[x.lower()]
        except KeyError:
            raise Exception(f"invalid backend {x}") from None


class DCTruncation(Enum):
    none = -1
    max = 0
    norm = 1
    rms = 2

    @classmethod
    def parse_string(cls, x):
        try:
            return cls[x.lower()]
        except KeyError:
            raise Exception(f"invalid truncation mode {x}") from None


class DCThreshold:
    """Registry of per-layer thresholds keyed by module, in frame-0 forward order
    (reference :122-208). JSON files map the stringified position to the value."""
    t_default = 0.0
    t = OrderedDict()
    path = None
    initialized = False
    scale = 1.0

    @classmethod
    def get(cls, key, default=0.0):
        return cls.t.get(key, default)

    @classmethod
    def set(cls, key, val):
        if key not in cls.t:
            cls.t[key] = val

    @classmethod
    def load_thresholds(cls):
        if cls.initialized:
            return
        cls.initialized = True
        if cls.path is None:
            return
        import json
        with open(cls.path) as f:
            thresholds = json.load(f)
        if len(thresholds) != len(cls.t):
            print(f"WARNING: thresholds file contains different number of thresholds. file: {len(thresholds)} expected {len(cls.t)}")
        # a shorter file addresses the LAST len(file) layers
        skip = len(cls.t) - len(thresholds)
        for i, key in enumerate(list(cls.t.keys())):
            if i >= skip:
                cls.t[key] = thresholds[str(i - skip)] * cls.scale

    @classmethod
    def save_thresholds(cls, name):
        import json
        with open(f"thresholds_{name}.json", "w+") as f:
            json.dump({i: v for i, v in enumerate(cls.t.values())}, f)

    @classmethod
    def reset(cls):
        cls.t.clear()
        cls.initialized = False
        cls.path = None

    @classmethod
    def create_trainable_parameters(cls, device):
        raise NotImplementedError("trainable thresholds belong to the delta_cudnn training emulation, which this package does not provide")


class DCModule(nn.Module):
    temp_buffers = []

    def __init__(self):
        super().__init__()

    @classmethod
    def get_temp_buffer_numel(cls):
        return sum(x.numel() for x in cls.temp_buffers)

    def reset(self):
        DCModule.temp_buffers = []

    def process_filters(self):
        """Re-layout the filters of every delta convolution below this module (once, after
        ``.to(device, memory_format=channels_last)`` and the optional ``.half()``)."""
        for mod in self.modules():
            if type(mod) in (DCConv2d, DCConvTranspose2d):
                mod.process_filters()

    def reset_layers(self):
        """Drop every cache below this module; the next forward is a first frame again."""
        for mod in self.modules():
            if mod is not self and isinstance(mod, DCModule):
                mod.reset()
        DCModule.temp_buffers.clear()


def to_tuple(*args):
    result = []
    for x in args:
        if type(x) == int:
            result.append((x, x))
        elif len(x) == 1:
            result.append((x[0], x[0]))
        else:
            result.append(tuple(x))
    return result[0] if len(result) == 1 else result


def _unsupported_backend(backend):
    raise NotImplementedError(
        f"backend {backend} is not provided: deltacnn_b200 implements DCBackend.deltacnn (sm_100a kernels) and "
        "delegates DCBackend.cudnn to torch; the delta_cudnn soft-threshold emulation is training-side code")


class _DeltaConvMixin:
    """State and forward logic shared by DCConv2d and DCConvTranspose2d."""
    _transposed = False

    def _init_delta_state(self, delta_threshold, name, activation, dense_out, backend, use_logging, kwargs):
        self.prev_in = None
        self.prev_out = None
        self.delta_threshold = delta_threshold if delta_threshold is not None else DCThreshold.t_default
        self.name = name
        self.backend = backend if backend is not None else DCConv2d.backend
        self.activation, self.activation_int = convert_activation_string(activation, **kwargs)
        self.dense_out = dense_out
        self.use_logging = use_logging
        if self.logging_enabled():
            raise NotImplementedError("the TensorBoard logging forward of the reference is not provided")
        self.densify_layer = None
        self.activation_layer = None
        if self.dense_out:
            self.densify_layer = DCDensify(activation=activation, name=self.name)
        elif self.activation is not None:
            self.activation_layer = DCActivation(self.name, delta_threshold=delta_threshold, activation=activation)
        self.conv_idx = -1
        self.dense_in = False
        self.mask = None
        self.frame_idx = -1
        self.out_truncated = None
        self.out_mask = None
        self.out_shape = []
        self.kwargs = kwargs
        self.in_shape = None
        self.orig_weights = None
        self.weight_umma = None
        self._out = None
        self._desc = None
        self._epilogue = None
        self._workspace = None
        self.fuse_activation = True
        assert kwargs.get("leaky_relu_negative_slope", 0.1) == 0.1, "Leaky ReLU implementation uses hard coded negative slope of 0.1"

    def logging_enabled(self):
        return self.use_logging if self.use_logging is not None else DCConv2d.use_logging

    def init_first_iter(self, input):
        self.conv_idx = DCConv2d.conv_idx
        self.dense_in = type(input) == Tensor
        self.in_shape = input.shape if self.dense_in else input[0].shape
        registers = self.activation is not None or self.dense_in or (self._transposed and self.dense_out)
        if registers and self.backend != DCBackend.cudnn:
            DCThreshold.set(self, self.delta_threshold)
        if self.dense_in:
            DCConv2d.n_dense_inputs += 1
        else:
            DCConv2d.n_sparse_inputs += 1
        if self.dense_out:
            DCConv2d.n_dense_output += 1
        else:
            DCConv2d.n_sparse_output += 1

    def __repr__(self):
        return f"MyConv2d{self.conv_idx} cin={self.in_channels} cout={self.out_channels}"

    def can_fuse_residual(self, input, add_layer=None):
        """True when forward(input, residual=(delta, mask), add_layer=...) adds the residual inside the convolution
        kernel: a linear fp16 stride-1 convolution on the tensor-core path, 1x1 without padding or KxK on patch tiles
        (no reference counterpart; it replaces the DCAdd that follows the convolution, reference sparse_layers.py
        DCAdd.forward). ``add_layer`` is that DCAdd when it has an activation."""
        if not (DCConv2d.fuse_residual and not self._transposed and self.backend == DCBackend.deltacnn and type(input) != Tensor
                and input[0].dtype == torch.float16 and tuple(self.stride) == (1, 1) and self.groups == 1
                and self.weight_umma is not None and self.activation is None and not self.dense_out):
            return False
        if tuple(self.kernel_size) == (1, 1):
            if not all(int(v) == 0 for v in self.padding):
                return False
        elif not DCConv2d.patch_tiles or max(self.kernel_size) > 5:
            return False
        if add_layer is not None and (add_layer.dense_out or add_layer.weight_a != 1.0 or add_layer.weight_b != 1.0):
            return False
        if add_layer is not None and add_layer.activation is not None and not DCConv2d.fuse_residual_activation:
            return False
        return True

    def _delta_forward_common(self, input, residual=None, add_layer=None):
        DCConv2d.conv_idx += 1
        self.frame_idx += 1
        first_iter = self.conv_idx == -1
        if first_iter:
            self.init_first_iter(input)
        if self.backend == DCBackend.cudnn:
            assert len(self.padding) == 2
            out = self._forward_cudnn(input, first_iter)
            return out if residual is None else out + residual
        if self.backend != DCBackend.deltacnn:
            _unsupported_backend(self.backend)
        if residual is not None and not self.can_fuse_residual(input, add_layer):
            raise RuntimeError("this convolution cannot add a residual itself (see can_fuse_residual); use DCAdd")
        return self._forward_delta_conv(input, first_iter, residual, add_layer)

    def _forward_cudnn(self, input, first_iter):
        out = super(_DeltaConvMixin, self).forward(input)
        if self.activation is not None:
            out = self.activation(out)
        if DCConv2d.measure_flops:
            n_updated = (input if self._transposed else out)[:, :1].numel()
            DCConv2d.flops_sum += n_updated * self.weight.numel()
        return out

    def _forward_delta_conv(self, input, first_iter, residual=None, add_layer=None):
        if type(input) == Tensor:
            raise RuntimeError("delta convolutions take a (delta, mask) tuple; put a DCSparsify in front of the first layer")
        if self.orig_weights is None:
            raise RuntimeError("process_filters() must be called on the model before the first forward")
        x, mask = input
        if x.shape[-1] != self.in_shape[-1] or x.shape[-2] != self.in_shape[-2] or x.shape[0] != self.in_shape[0]:
            # resolution or batch change: forget the cached geometry and buffers
            self.in_shape = x.shape
            self.out_shape = []
            self._out = self.out_mask = self._desc = self._workspace = None

        if self._desc is None:
            size_fn = K.deconv_out_hw if self._transposed else K.conv_out_hw
            hw = size_fn(x.shape[2], x.shape[3], self.kernel_size, self.stride, self.padding, self.dilation)
            self.out_shape = list(hw)
            self._desc = K.make_conv_desc(tuple(x.shape), self.out_channels, hw, tuple(self.kernel_size), self.stride,
                                          self.padding, self.dilation, self.groups, K._dtype(x))
        out_dims = (x.shape[0], self.out_channels, self.out_shape[0], self.out_shape[1])

        def check_cache(t, what):
            # caches go to the kernel as raw pointers: a stale one must fail here, not on the device
            if t is not None and (tuple(t.shape) != out_dims or t.dtype != x.dtype or t.device != x.device):
                raise RuntimeError(f"deltacnn_b200: {what} of {self!r} has shape {tuple(t.shape)}, the output is {out_dims} "
                                   "(call reset_layers() after a batch or resolution change)")

        epilogue = None
        act = self.activation_layer
        fuse = act is not None and self.fuse_activation and not act.first_iter and act.inplace and \
            act.truncation_mode == DCTruncation.max and self.frame_idx > 0
        if K.DCPerformanceMetricsManager.enabled:
            # work accounting: the truncation layer runs (and counts) on its own; same results as the fused epilogue
            fuse = False
            K.DCPerformanceMetricsManager.add_conv(mask, self.in_channels, self.out_channels, tuple(self.kernel_size), tuple(self.stride),
                                                   self.padding, tuple(self.dilation), self.groups, tuple(self.out_shape),
                                                   transposed=self._transposed)
        if fuse:
            check_cache(act.prev_out, "the activation cache")
            check_cache(act.out_truncated, "the truncation cache")
            epilogue = K.make_epilogue(act.prev_out, act.out_truncated, DCThreshold.get(act), act.activation_int,
                                       act.truncation_mode.value)
        if residual is not None:
            res_delta, res_mask = residual
            check_cache(res_delta, "the residual")
            if add_layer is not None and add_layer.activation is not None:
                if add_layer.first_iter:              # what DCAdd.forward does on its first call
                    add_layer.first_iter = False
                    DCAdd.idx += 1
                    add_layer.idx = DCAdd.idx
                    add_layer.prev_out = torch.zeros_like(res_delta)
                    DCModule.temp_buffers.append(add_layer.prev_out)
                check_cache(add_layer.prev_out, "the add layer's cache")
                epilogue = K.make_residual_epilogue(res_delta, res_mask, add_layer.prev_out, add_layer.activation_int)
            else:
                epilogue = K.make_residual_epilogue(res_delta, res_mask)
        op = K.sparse_deconv if self._transposed else K.sparse_conv
        extra = {}
        if self._transposed:
            if DCConv2d.use_worklist and self._workspace is None and self.weight_umma is not None:
                self._workspace = torch.empty(K.deconv_workspace_bytes(self._desc), dtype=torch.uint8, device=x.device)
            # stride-2 layers: per-phase work lists in scratch memory (measured faster than the patch tiles the library
            # uses for a call without scratch)
            extra = {"filter_umma": self.weight_umma, "workspace": self._workspace}
        else:
            if DCConv2d.use_worklist and self._workspace is None:
                self._workspace = torch.empty(K.conv_workspace_bytes(self._desc), dtype=torch.uint8, device=x.device)
            # with scratch memory KxK layers use a work list (best on sparse maps), without it patch tiles (best on
            # mostly active maps); calls the tensor-core path cannot take fall back to the CUDA-core kernels
            ws = self._workspace
            if DCConv2d.patch_tiles and tuple(self.stride) == (1, 1) and tuple(self.kernel_size) != (1, 1):
                ws = None
            extra = {"filter_umma": self.weight_umma, "workspace": ws}
        out, out_mask = op(
            x=x, filter=self.weight, mask=mask, bias=self.bias if self.frame_idx <= 0 else None, stride=self.stride,
            padding=self.padding, dilation=self.dilation, groups=self.groups, c_out=self.out_channels, create_out_mask=True,
            out_mask=self.out_mask, out_shape=self.out_shape, out=self._out, epilogue=epilogue, desc=self._desc, **extra)
        if DCModule_reuse_buffers():
            self._out, self.out_mask = out, out_mask

        if self.dense_out:
            return self.densify_layer((out, out_mask))
        if act is not None:
            if fuse:
                return out, out_mask
            return act((out, out_mask))
        return out, out_mask

    def reset(self):
        DCModule.reset(self)
        self.frame_idx = -1
        self.conv_idx = -1
        self.prev_out = None
        self.prev_in = None
        self.out_truncated = None
        self.out_mask = None
        self.out_shape = []
        self._out = None
        self._desc = None
        self._workspace = None
        DCConv2d.conv_idx = -1
        DCConv2d.n_dense_output, DCConv2d.n_sparse_output = 0, 0
        DCConv2d.n_dense_inputs, DCConv2d.n_sparse_inputs = 0, 0

    def process_filters(self):
        """Keep the torch-layout weights in ``orig_weights`` and replace ``weight.data`` by the
        kernel layout (reference :655-675)."""
        if self.orig_weights is not None:
            return
        self.orig_weights = self.weight.data.clone()
        if self.backend != DCBackend.deltacnn:
            return
        if self.weight.data.dtype == torch.float16:
            self.weight.data = convert_half_filter(self.weight.data, transposed=self._transposed)
        else:
            self.weight.data = convert_filter_out_channels_last(self.weight.data, transposed=self._transposed)
        self._pack_umma()

    def _pack_umma(self):
        """Build the tensor-core image of the filter when the shape has a tcgen05 kernel."""
        self.weight_umma = None
        if self.weight.dtype != torch.float16 or not self.weight.is_cuda:
            return
        from ._lib import lib, check
        kh, kw = self.kernel_size
        desc = K.make_conv_desc((1, self.in_channels, 8, 8), self.out_channels, (8, 8), (kh, kw), self.stride,
                                self.padding, self.dilation, self.groups, 1)
        tr = 1 if self._transposed else 0
        nbytes = lib.dc_filter_umma_bytes(desc, tr)
        if nbytes == 0:
            return
        packed = torch.empty(nbytes, dtype=torch.uint8, device=self.weight.device)
        check(lib.dc_pack_filter_umma(desc, tr, self.weight.data_ptr(), packed.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream), "pack_filter_umma")
        self.weight_umma = packed


def DCModule_reuse_buffers():
    return DCConv2d.reuse_buffers


class DCConv2d(_DeltaConvMixin, nn.Conv2d, DCModule):
    """Delta convolution module (reference :261-675)."""
    backend = DCBackend.deltacnn
    conv_idx = -1
    out_masks = []
    use_logging = False
    n_sparse_inputs = 0
    n_dense_inputs = 0
    n_sparse_output = 0
    n_dense_output = 0
    store_out_masks = False
    flops_sum = 0
    measure_flops = False
    reuse_buffers = True      # keep per-layer output buffers across frames
    use_worklist = True       # steady-state frames: active-pixel work lists in per-layer scratch memory
    fuse_residual = True      # forward(input, residual=...) adds the residual inside the convolution kernel where it can
    fuse_residual_activation = False   # ... also when the add layer has an activation (its accumulated sum is updated by the convolution)
    patch_tiles = False       # stride-1 KxK layers: patch tiles loaded by tiled TMA (mostly active maps) instead of work lists
    fuse_blocks = False       # DCFusedInvertedResidual: whole inverted-residual blocks of small maps in one kernel (opt-in)
    fuse_heads = True         # DCFusedHeads: the 3x3 layers of several heads on the same input in one kernel

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1, groups: int = 1,
                 bias: bool = True, padding_mode: str = "zeros", delta_threshold: float = None, name: str = None,
                 activation: str = None, dense_out=False, backend=None, use_logging=None, **kwargs):
        kernel_size, stride, padding, dilation = to_tuple(kernel_size, stride, padding, dilation)
        nn.Conv2d.__init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias, padding_mode)
        self._init_delta_state(delta_threshold, name, activation, dense_out, backend, use_logging, kwargs)

    def forward(self, input, residual=None, add_layer=None):
        return self._delta_forward_common(input, residual, add_layer)


class DCConvTranspose2d(_DeltaConvMixin, nn.ConvTranspose2d, DCModule):
    """Delta transposed convolution module (reference :678-1083). output_padding is ignored by the
    delta path, as in the reference (cuda_kernels.py:55-57)."""
    _transposed = True

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, output_padding=0,
                 groups: int = 1, bias: bool = True, dilation=1, padding_mode: str = "zeros", delta_threshold: float = None,
                 name: str = None, activation: str = None, store_prev_in=False, dense_out=False, backend=None,
                 use_logging=None, **kwargs):
        kernel_size, stride, padding, dilation = to_tuple(kernel_size, stride, padding, dilation)
        nn.ConvTranspose2d.__init__(self, in_channels, out_channels, kernel_size, stride, padding, output_padding, groups,
                                    bias, dilation, padding_mode)
        self.stores_prev_in = store_prev_in
        self._init_delta_state(delta_threshold, name, activation, dense_out, backend, use_logging, kwargs)

    def forward(self, input):
        assert self.backend == DCBackend.cudnn or self.backend == DCBackend.deltacnn
        return self._delta_forward_common(input)


class DCAdd(DCModule):
    """Residual add of two delta tensors (reference :1086-1182)."""
    idx = -1

    def __init__(self, activation: str = None, dense_out=False, weight_a=None, weight_b=None, name=""):
        super().__init__()
        self.name = name
        self.dense_out = dense_out
        self.activation, self.activation_int = convert_activation_string(activation)
        self.idx = -1
        self.prev_out = None
        self.mask_out = None
        self.weight_a = 1.0 if weight_a is None else weight_a
        self.weight_b = 1.0 if weight_b is None else weight_b
        self.first_iter = True
        self._out = None

    def forward(self, a, b, weight_a=None, weight_b=None):
        w_a = self.weight_a if weight_a is None else weight_a
        w_b = self.weight_b if weight_b is None else weight_b
        if type(a) == torch.Tensor:
            if DCConv2d.backend == DCBackend.delta_cudnn:
                _unsupported_backend(DCConv2d.backend)
            c = w_a * a + w_b * b
            return self.activation(c) if self.activation is not None else c

        val_a, mask_a = a
        val_b, mask_b = b
        if self.first_iter:
            self.first_iter = False
            DCAdd.idx += 1
            self.idx = DCAdd.idx
            if self.dense_out or self.activation is not None:
                self.prev_out = torch.zeros_like(val_a)
                DCModule.temp_buffers.append(self.prev_out)
        if self.mask_out is None or self.mask_out.shape != mask_a.shape:
            self.mask_out = torch.empty_like(mask_a)
        if self._out is None or self._out.shape != val_a.shape or not DCConv2d.reuse_buffers or self.dense_out:
            self._out = torch.empty_like(val_a)
        out, mask_out = self._out, self.mask_out
        K.sparse_add_tensors(val_a, val_b, self.prev_out, out, mask_a, mask_b, mask_out, w_a, w_b, self.activation_int,
                             self.dense_out)
        if self.dense_out:
            return out
        return out, mask_out

    def reset(self):
        super().reset()
        self.idx = -1
        self.mask_out = None
        self.prev_out = None
        self._out = None
        self.first_iter = True
        DCAdd.idx = -1


class DCConcatenate(DCModule):
    """Channel concatenation (reference :1185-1194)."""

    def __init__(self, name=""):
        super().__init__()
        self.name = name

    def forward(self, a, b):
        if type(a) == torch.Tensor:
            return torch.cat((a, b), dim=1)
        return K.sparse_concatenate(a, b)


class DCSparsify(DCModule):
    """Dense frame -> (delta, mask) against the cached previous frame (reference :1197-1273)."""
    idx = -1

    def __init__(self, name="", delta_threshold=None, dilation=-1):
        super().__init__()
        self.name = name
        self.prev_in = None
        self.idx = -1
        self.delta_threshold = delta_threshold if delta_threshold is not None else DCThreshold.t_default
        self.dilation = dilation
        self.frame_idx = -1
        self.mask = None
        self._delta = None
        self._hit = None
        self._u8 = None

    def set_u8_input(self, scale=1.0 / 255.0, offset=0.0, dtype=torch.float16, channels=3):
        """Accept 8-bit frames: ``forward`` then takes a contiguous uint8 tensor of shape (N, H, W, C) and
        the value compared and cached is ``frame * scale[c] + offset[c]`` in ``dtype``; normalisation, delta
        and mask are one kernel. ``scale`` / ``offset`` are numbers or per-channel sequences."""
        def vec(v):
            t = torch.as_tensor(v, dtype=torch.float32).flatten()
            return t.expand(channels).contiguous() if t.numel() == 1 else t.contiguous()
        self._u8 = (vec(scale), vec(offset), dtype)
        return self

    def _u8_to_float(self, frame):
        scale, offset, dtype = self._u8
        if scale.device != frame.device:
            scale, offset = scale.to(frame.device), offset.to(frame.device)
            self._u8 = (scale, offset, dtype)
        x = (frame.float() * scale + offset).to(dtype)                 # N,H,W,C contiguous
        return x.permute(0, 3, 1, 2)                                   # logical NCHW, channels-last memory

    def forward(self, input):
        if input.dtype == torch.uint8:
            if self._u8 is None:
                raise RuntimeError("DCSparsify got a uint8 frame: call set_u8_input() first")
            if DCConv2d.backend != DCBackend.deltacnn or self.idx == -1 or self.dilation > 1:
                return self.forward(self._u8_to_float(input))
            self.frame_idx += 1
            n, h, w, c = input.shape
            if self.mask is None or tuple(self.mask.shape) != (n, 1, h, w):
                self.mask = torch.empty((n, 1, h, w), dtype=torch.int, device=input.device)
            if self._delta is None or self._delta.shape != self.prev_in.shape or not DCConv2d.reuse_buffers:
                self._delta = torch.empty_like(self.prev_in)
            scale, offset, dtype = self._u8
            if scale.device != input.device:              # the tables go to the kernel as device pointers
                scale, offset = scale.to(input.device), offset.to(input.device)
                self._u8 = (scale, offset, dtype)
            K.sparsify_u8(input, scale, offset, self.prev_in, self._delta, self.mask, DCThreshold.get(self))
            return self._delta, self.mask
        if DCConv2d.backend == DCBackend.cudnn:
            return input
        if DCConv2d.backend != DCBackend.deltacnn:
            _unsupported_backend(DCConv2d.backend)
        first_iter = self.idx == -1
        self.frame_idx += 1
        if first_iter:
            if self not in DCThreshold.t:
                DCThreshold.set(self, self.delta_threshold)
            DCSparsify.idx += 1
            self.idx = DCSparsify.idx
            self.prev_in = input.clone()
            DCModule.temp_buffers.append(self.prev_in)
            mask = torch.ones_like(input[:, :1], dtype=torch.int)
            return input, mask

        threshold = DCThreshold.get(self)
        if self.mask is not None and (self.mask.shape[0] != input.shape[0] or self.mask.shape[2:] != input.shape[2:]):
            self.mask = None
        if self.dilation > 1:
            # noise-robust variant: the mask is the max-pooled |delta| > threshold (reference :1233-1248), two kernels here
            if self.mask is None:
                self.mask = torch.empty_like(input[:, :1], dtype=torch.int)
            if self._delta is None or self._delta.shape != input.shape or not DCConv2d.reuse_buffers:
                self._delta = torch.empty_like(input)
            if self._hit is None or self._hit.numel() != self.mask.numel():
                self._hit = torch.empty(self.mask.numel(), dtype=torch.uint8, device=input.device)
            K.sparsify_dilated(input, self.prev_in, self._delta, self.mask, self._hit, threshold, self.dilation)
            return self._delta, self.mask

        if self.mask is None or self.mask.shape[0] != input.shape[0] or self.mask.shape[2:] != input.shape[2:]:
            self.mask = torch.empty_like(input[:, :1], dtype=torch.int)
        if self._delta is None or self._delta.shape != input.shape or not DCConv2d.reuse_buffers:
            self._delta = torch.empty_like(input)
        K.sparsify(input, self.prev_in, self._delta, self.mask, threshold)
        return self._delta, self.mask

    def reset(self):
        super().reset()
        self.idx = -1
        self.frame_idx = -1
        self.prev_in = None
        self.prev_out = None
        self.mask = None
        self._delta = None
        self._hit = None
        DCSparsify.idx = -1


class DCDensify(DCModule):
    """(delta, mask) -> dense accumulated tensor (reference :1276-1333), one kernel."""
    idx = -1

    def __init__(self, activation: str = None, name="", clone_out=True):
        super().__init__()
        self.name = name
        self.activation, self.activation_int = convert_activation_string(activation)
        self.prev_out = None
        self.idx = -1
        self.clone_out = clone_out

    def forward(self, input):
        if type(input) == torch.Tensor:
            if DCConv2d.backend == DCBackend.delta_cudnn:
                _unsupported_backend(DCConv2d.backend)
            return input
        input, mask = input
        if self.prev_out is None:
            DCDensify.idx += 1
            self.idx = DCDensify.idx
            self.prev_out = torch.zeros_like(input)
            DCModule.temp_buffers.append(self.prev_out)
        if not self.clone_out and self.activation is None:
            K.sparse_activation(input, self.prev_out, None, mask, -1, -1, DCTruncation.none.value)
            return self.prev_out
        return K.sparse_densify(input, mask, self.prev_out, None, self.activation_int)

    def reset(self):
        super().reset()
        self.prev_out = None


class DCUpsamplingNearest2d(DCModule):
    """Nearest-neighbour upsampling of a (delta, mask) pair (reference :1336-1359)."""
    idx = -1

    def __init__(self, scale_factor=2, name=""):
        super().__init__()
        self.name = name
        self.scale_factor = int(scale_factor)
        self.idx = -1
        self.out = None
        self.torch_upsample = nn.UpsamplingNearest2d(scale_factor=scale_factor)

    def forward(self, input):
        if type(input) == torch.Tensor:
            return self.torch_upsample(input)
        val, mask = input
        if self.out is not None and (self.out[0].shape[0] != val.shape[0] or self.out[0].shape[2] != val.shape[2] * self.scale_factor
                                     or self.out[0].shape[3] != val.shape[3] * self.scale_factor):
            self.out = None
        self.out = K.sparse_upsample(val, mask, self.scale_factor, self.out)
        return self.out

    def reset(self):
        super().reset()
        self.out = None


class DCActivation(DCModule):
    """Accumulate + activation delta + truncation (reference :1362-1425)."""
    idx = -1
    truncation_default = DCTruncation.max

    def __init__(self, name="", inplace=True, delta_threshold=None, activation="relu", truncation_mode: DCTruncation = None):
        super().__init__()
        self.name = name
        self.idx = -1
        self.prev_out = None
        self.inplace = inplace
        self.out_truncated = None
        self.activation, self.activation_int = convert_activation_string(activation)
        self.delta_threshold = delta_threshold if delta_threshold is not None else DCThreshold.t_default
        self.first_iter = True
        self.truncation_mode = truncation_mode if truncation_mode is not None else DCActivation.truncation_default

    def forward(self, input):
        if type(input) == torch.Tensor:
            if DCConv2d.backend == DCBackend.delta_cudnn:
                _unsupported_backend(DCConv2d.backend)
            return self.activation(input) if self.activation is not None else input
        val, mask = input
        if self.first_iter:
            self.first_iter = False
            if self not in DCThreshold.t:
                DCThreshold.set(self, self.delta_threshold)
            if self.idx < 0:
                DCActivation.idx += 1
                self.idx = DCActivation.idx
            self.prev_out = val.clone()
            self.out_truncated = torch.zeros_like(val)
            DCModule.temp_buffers.append(self.prev_out)
            DCModule.temp_buffers.append(self.out_truncated)
            if self.activation is not None:
                val = self.activation(val)
            return val, mask

        threshold = DCThreshold.get(self)
        if not self.inplace:
            val = val.clone()
            mask = mask.clone()
        mask_before = mask.clone() if K.DCPerformanceMetricsManager.enabled else None
        K.sparse_activation(val, self.prev_out, self.out_truncated, mask, threshold, self.activation_int, self.truncation_mode.value)
        if mask_before is not None:
            K.DCPerformanceMetricsManager.add_activation(mask_before, val.shape[1], self.truncation_mode.value, mask)
        return val, mask

    def reset(self):
        super().reset()
        self.idx = -1
        self.prev_out = None
        self.out_truncated = None
        self.first_iter = True
        DCActivation.idx = -1


class DCMaxPooling(nn.MaxPool2d, DCModule):
    """Delta max pooling with an accumulated-input cache (reference :1428-1474); the cache
    update is part of the same library call."""

    def __init__(self, kernel_size, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
        kernel_size, stride, padding, dilation = to_tuple(kernel_size, stride, padding, dilation)
        super().__init__(kernel_size, stride=stride, padding=padding, dilation=dilation)
        self.first_iter = True
        self.out_shape = []
        self.prev_in = None
        self._out = None

    def forward(self, input):
        if type(input) == Tensor:
            if DCConv2d.backend == DCBackend.delta_cudnn:
                _unsupported_backend(DCConv2d.backend)
            if len(self.padding) == 4:
                pt, pb, pl, pr = self.padding
                input = torch.nn.functional.pad(input, (pl, pr, pt, pb))
                return torch.nn.functional.max_pool2d(input, self.kernel_size, self.stride, 0, self.dilation)
            return super().forward(input)
        x, mask = input
        if self.first_iter:
            self.first_iter = False
            self.prev_in = torch.zeros_like(x)
            DCModule.temp_buffers.append(self.prev_in)
        if self._out is not None and self._out[0].shape[0] != x.shape[0]:
            self._out = None
        buf, mbuf = self._out if self._out is not None else (None, None)
        out = K.sparse_pooling(x, self.prev_in, self.kernel_size, mask, self.stride, self.padding, self.dilation,
                               create_out_mask=True, pooling_mode_int=0, out_shape=self.out_shape, out=buf, out_mask=mbuf,
                               update_prev=True)
        if DCConv2d.reuse_buffers:
            self._out = out
        return out

    def reset(self):
        DCModule.reset(self)
        self.first_iter = True
        self.prev_in = None
        self.out_shape = []
        self._out = None


class DCAdaptiveAveragePooling(nn.AdaptiveAvgPool2d, DCModule):
    """Delta global average pooling, output 1x1 only (reference :1477-1513)."""

    def __init__(self, output_size=None):
        output_size = to_tuple(output_size)
        super().__init__(output_size=output_size)
        self.first_iter = True
        self.out_shape = output_size
        self.prev_in = None

    def get_target_size(self, input):
        assert self.output_size[0] == 1 and self.output_size[1] == 1
        return tuple(input.shape[2:]), (1, 1), (0, 0), (1, 1)

    def forward(self, input):
        if type(input) == Tensor:
            return super().forward(input)
        x, mask = input
        self.first_iter = False
        kernel_size, stride, padding, dilation = self.get_target_size(x)
        return K.sparse_pooling(x, None, kernel_size, mask, stride, padding, dilation, create_out_mask=True,
                                pooling_mode_int=1, out_shape=list(self.out_shape))

    def reset(self):
        DCModule.reset(self)
        self.first_iter = True
        self.prev_in = None


class DCBatchNorm2d(nn.BatchNorm2d, DCModule):
    """Inference BatchNorm on delta tensors: scale every frame, offset on the first only
    (reference :1516-1585). Folding it into the preceding convolution is cheaper."""

    def __init__(self, num_features, eps=1e-5, momentum=0.1, affine=True, track_running_stats=True, inplace=True):
        super().__init__(num_features, eps, momentum, affine, track_running_stats)
        self.first_iter = True
        self.scale = None
        self.offset = None
        self.inplace = inplace

    def convert_to_scale_offset(self, input):
        bn_scale = self.weight * torch.rsqrt(self.running_var + self.eps)
        self.scale = bn_scale[None, :, None, None]
        self.offset = (-self.running_mean * bn_scale + self.bias)[None, :, None, None]

    def forward(self, input):
        mask = None
        dense = type(input) != tuple
        if not dense:
            input, mask = input
        use_offset = dense
        if self.first_iter:
            self.first_iter = False
            use_offset = True
            self.convert_to_scale_offset(input)
        if dense:
            out = input.mul_(self.scale) if self.inplace else input * self.scale
            out.add_(self.offset)
            return out
        bias = self.offset if use_offset else None
        if self.inplace:
            K.sparse_mul_add(input, mask, input, mask, self.scale, bias)
            return input, mask
        out = torch.empty_like(input)
        out_mask = torch.empty_like(mask)
        K.sparse_mul_add(input, mask, out, out_mask, self.scale, bias)
        return out, out_mask

    def reset(self):
        DCModule.reset(self)
        self.first_iter = True


class DCLinear(nn.Linear, DCModule):
    """Fully connected head that consumes the (delta, mask) of a pooled 1x1 feature directly: the logits are a
    running fp32 sum updated by ``weight @ delta`` for the streams whose mask is set, so the dense feature vector
    is never formed. No reference counterpart: it replaces ``DCDensify`` + ``nn.Linear`` at the end of the
    reference's example network (example/mobilenet_deltacnn.py:216-227), which is valid because a linear layer
    commutes with the accumulation over frames. A dense tensor input goes through ``nn.Linear`` unchanged."""

    def __init__(self, in_features, out_features, bias=True):
        super().__init__(in_features, out_features, bias)
        self.acc = None
        self._out = None

    def forward(self, input):
        if type(input) == Tensor:
            return super().forward(input.reshape(input.shape[0], -1))
        delta, mask = input
        n = delta.shape[0]
        if delta.shape[2] != 1 or delta.shape[3] != 1:
            raise RuntimeError("DCLinear takes the (delta, mask) of a 1x1 feature (put it behind DCAdaptiveAveragePooling)")
        first = self.acc is None
        if first:
            self.acc = torch.zeros((n, self.out_features), dtype=torch.float32, device=delta.device)
            DCModule.temp_buffers.append(self.acc)
        elif self.acc.shape[0] != n:
            raise RuntimeError("DCLinear: the batch size changed (call reset_layers())")
        if self._out is None or self._out.shape[0] != n or self._out.dtype != delta.dtype or not DCConv2d.reuse_buffers:
            self._out = torch.empty((n, self.out_features), dtype=delta.dtype, device=delta.device)
        return K.linear_delta(delta, mask, self.weight, self.bias, self.acc, self._out, first)

    def reset(self):
        DCModule.reset(self)
        self.acc = None
        self._out = None


class DCHeatmapArgmax(DCModule):
    """Pose head tail on the device: accumulates the heat-map delta (as ``DCDensify``) and returns, per stream and
    joint, (x, y, value) of the largest heat-map element as a float32 (N, J, 3) tensor; streams without an updated
    pixel keep their previous result. ``heatmaps`` holds the dense accumulated maps. No reference counterpart (the
    reference returns the densified maps to torch code, src/deltacnn/sparse_layers.py:1322-1329)."""

    def __init__(self, activation=None, name=""):
        super().__init__()
        self.name = name
        self.densify = DCDensify(activation=activation)
        self.heatmaps = None
        self._out = None

    def forward(self, input):
        if type(input) == Tensor:
            self.heatmaps = input
            return K.heatmap_argmax(input.contiguous(memory_format=torch.channels_last), None)
        _, mask = input
        first = self._out is None
        self.heatmaps = self.densify(input)
        self._out = K.heatmap_argmax(self.heatmaps, None if first else mask, self._out)
        return self._out

    def reset(self):
        super().reset()
        self.heatmaps = None
        self._out = None


class DCCenterNetDecode(DCModule):
    """Detector tail on the device: accumulates the three head deltas (heat map, size, offset; as ``DCDensify``)
    and decodes boxes there: a peak is an element equal to the maximum of its 3x3 neighbourhood, the ``topk`` best
    peaks above ``min_score`` become rows (x1, y1, x2, y2, score, class). Only pixels next to an updated pixel of any
    head are re-examined; streams without an update keep their boxes. Returns (det (N, topk, 6) float32,
    count (N,) int32). No reference counterpart (src/deltacnn/sparse_layers.py:1322-1329 returns dense maps)."""

    def __init__(self, topk=100, min_score=0.0, stride=4.0, apply_sigmoid=True, name=""):
        super().__init__()
        self.name = name
        self.topk, self.min_score, self.stride, self.apply_sigmoid = topk, min_score, stride, apply_sigmoid
        self.densify = nn.ModuleList([DCDensify(), DCDensify(), DCDensify()])
        self.dense = None
        self._state = None
        self._union = None

    def forward(self, heat, wh, offset):
        ins = (heat, wh, offset)
        if type(heat) == Tensor:
            self.dense = tuple(t.contiguous(memory_format=torch.channels_last) for t in ins)
            det, count, _ = K.centernet_decode(*self.dense, None, None, self.topk, self.min_score, self.stride, self.apply_sigmoid)
            return det, count
        first = self._state is None
        masks = [m for _, m in ins]
        self.dense = tuple(d(x) for d, x in zip(self.densify, ins))
        mask = None
        if not first:
            if self._union is None or self._union.shape != masks[0].shape:
                self._union = torch.empty_like(masks[0])
            torch.bitwise_or(masks[0], masks[1], out=self._union)
            torch.bitwise_or(self._union, masks[2], out=self._union)
            mask = self._union
        det, count, self._state = K.centernet_decode(*self.dense, mask, self._state, self.topk, self.min_score, self.stride,
                                                     self.apply_sigmoid)
        return det, count

    def reset(self):
        super().reset()
        self.dense = None
        self._state = None
        self._union = None


class DCFusedHeads:
    """Runs the first layers of several heads that read the SAME input -- stride-1 3x3 ``DCConv2d`` layers with a fused
    activation, equal in shape -- as ONE kernel on steady-state frames (``cuda_kernels.conv3x3_heads``): the input tile
    is loaded once for all heads, every head keeps its own output, out-mask, caches and threshold. It owns no state (the
    caches are those of the layers' activation layers), so a stream may switch between this call and the layers' own
    forwards from frame to frame. No reference counterpart (the reference runs every head's convolution and truncation
    kernels on their own)."""

    def __init__(self, convs):
        self.convs = list(convs)
        self._key = None
        self._desc = None
        self._packed = None

    def ready(self, input):
        """True when this frame can take the fused kernel."""
        if not DCConv2d.fuse_heads or K.DCPerformanceMetricsManager.enabled or type(input) == Tensor or len(self.convs) < 2:
            return False
        x = input[0]
        c0 = self.convs[0]
        if x.dtype != torch.float16 or not x.is_cuda:
            return False
        for c in self.convs:
            a = c.activation_layer
            if c.backend != DCBackend.deltacnn or c._transposed or tuple(c.kernel_size) != (3, 3) or tuple(c.stride) != (1, 1) or \
                    tuple(c.dilation) != (1, 1) or c.groups != 1 or tuple(c.padding) != tuple(c0.padding) or \
                    c.in_channels != c0.in_channels or c.out_channels != c0.out_channels or c.orig_weights is None or c.dense_out:
                return False
            if a is None or a.first_iter or not a.inplace or a.truncation_mode != DCTruncation.max or not c.fuse_activation or c.frame_idx <= 0:
                return False
        key = tuple(x.shape)
        if self._key != key:
            self._key, self._desc = key, None
            hw = K.conv_out_hw(x.shape[2], x.shape[3], c0.kernel_size, c0.stride, c0.padding, c0.dilation)
            total = c0.out_channels * len(self.convs)
            desc = K.make_conv_desc(key, total, hw, (3, 3), c0.stride, c0.padding, c0.dilation, 1, K._dtype(x))
            if K.conv3x3_heads_supported(desc, len(self.convs)):
                from ._lib import lib, check
                w_cat = torch.cat([c.weight.data for c in self.convs], dim=3).contiguous()      # HWIO, concatenated outputs
                nbytes = lib.dc_filter_umma_bytes(desc, 0)
                if nbytes > 0:
                    self._packed = torch.zeros(nbytes, dtype=torch.uint8, device=x.device)
                    check(lib.dc_pack_filter_umma(desc, 0, w_cat.data_ptr(), self._packed.data_ptr(),
                                                  torch.cuda.current_stream(x.device).cuda_stream), "pack_filter_umma")
                    self._desc = desc
        return self._desc is not None

    def __call__(self, input):
        x, mask = input
        desc = self._desc
        n = x.shape[0]
        outs, masks, eps = [], [], []
        for c in self.convs:
            dims = (n, c.out_channels, desc.h_out, desc.w_out)
            if c._out is None or tuple(c._out.shape) != dims or not DCModule_reuse_buffers():
                c._out = torch.empty(dims, dtype=x.dtype, device=x.device).contiguous(memory_format=torch.channels_last)
                c.out_mask = torch.empty((n, 1, desc.h_out, desc.w_out), dtype=torch.int32, device=x.device)
            a = c.activation_layer
            for t, what in ((a.prev_out, "the activation cache"), (a.out_truncated, "the truncation cache")):
                if t is None or tuple(t.shape) != dims or t.dtype != x.dtype or t.device != x.device:
                    raise RuntimeError(f"deltacnn_b200: {what} of {c!r} does not match the output {dims} "
                                       "(call reset_layers() after a batch or resolution change)")
            outs.append(c._out)
            masks.append(c.out_mask)
            eps.append(K.make_epilogue(a.prev_out, a.out_truncated, DCThreshold.get(a), a.activation_int, a.truncation_mode.value))
            DCConv2d.conv_idx += 1                    # what the layer's own forward would have counted
            c.frame_idx += 1
        K.conv3x3_heads(x, mask, self._packed, None, outs, masks, desc, epilogues=eps)
        return [(o, m) for o, m in zip(outs, masks)]


class DCFusedInvertedResidual:
    """Runs an inverted-residual block -- expansion ``DCConv2d`` 1x1 with activation, depthwise ``DCConv2d`` 3x3 with
    activation, projection ``DCConv2d`` 1x1, optionally followed by the residual ``DCAdd`` of the block input -- as ONE
    kernel on steady-state frames of small feature maps (``cuda_kernels.fused_inverted_residual``). It owns no state:
    the caches and thresholds are those of the three layers' activation layers, so a stream may switch between this
    call and the layers' own forwards from frame to frame, with identical results. No reference counterpart (the
    reference runs six kernels per block, example/mobilenet_deltacnn.py:87-128)."""

    def __init__(self, expand, depthwise, project):
        self.expand, self.depthwise, self.project = expand, depthwise, project
        self._desc = None
        self._key = None
        self._out = None
        self._mask_out = None

    def ready(self, input, residual=False):
        """True when this frame of this block can take the fused kernel."""
        e, d, p = self.expand, self.depthwise, self.project
        if not DCConv2d.fuse_blocks or K.DCPerformanceMetricsManager.enabled or type(input) == Tensor:
            return False
        x = input[0]
        if x.dtype != torch.float16 or any(c.backend != DCBackend.deltacnn for c in (e, d, p)):
            return False
        if e.weight_umma is None or p.weight_umma is None or d.orig_weights is None or tuple(d.kernel_size) != (3, 3) or \
                tuple(d.padding) != (1, 1) or d.groups != d.in_channels or tuple(e.kernel_size) != (1, 1) or tuple(p.kernel_size) != (1, 1) or \
                tuple(e.stride) != (1, 1) or tuple(p.stride) != (1, 1) or d.stride[0] != d.stride[1] or tuple(d.dilation) != (1, 1):
            return False
        if p.activation_layer is not None or p.dense_out or e.dense_out or d.dense_out:
            return False
        for c in (e, d):
            a = c.activation_layer
            if a is None or a.first_iter or not a.inplace or a.truncation_mode != DCTruncation.max or c.frame_idx < 0 or not c.fuse_activation:
                return False
        if p.frame_idx < 0:
            return False
        key = (tuple(x.shape), bool(residual))
        if self._key != key:
            ae, ad = e.activation_layer, d.activation_layer
            desc = K.make_irb_desc(tuple(x.shape), e.out_channels, p.out_channels, d.stride[0], residual, ae.activation_int,
                                   ad.activation_int, 0.0, 0.0)
            self._key, self._desc = key, (desc if K.irb_supported(desc) else None)
            self._out = self._mask_out = None
        return self._desc is not None

    def __call__(self, input, residual=False):
        x, mask = input
        e, d, p = self.expand, self.depthwise, self.project
        ae, ad = e.activation_layer, d.activation_layer
        desc = self._desc
        desc.thr_expand, desc.thr_dw = float(DCThreshold.get(ae)), float(DCThreshold.get(ad))
        n, _, h, w = x.shape
        ho, wo = (h - 1) // desc.stride + 1, (w - 1) // desc.stride + 1
        if self._out is None or not DCConv2d.reuse_buffers:
            self._out = torch.empty((n, p.out_channels, ho, wo), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
            self._mask_out = torch.empty((n, 1, ho, wo), dtype=torch.int32, device=x.device)
        for c in (e, d, p):                       # what the three forwards would have counted
            DCConv2d.conv_idx += 1
            c.frame_idx += 1
        return K.fused_inverted_residual(x, mask, e.weight_umma, d.weight, p.weight_umma, ae.prev_out, ae.out_truncated, ad.prev_out,
                                         ad.out_truncated, self._out, self._mask_out, desc)
