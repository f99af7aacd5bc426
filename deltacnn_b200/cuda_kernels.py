"""Functional operator API: output-shape arithmetic, buffer allocation, and the call into
the C-ABI library. Mirrors the names and argument meaning of the reference's
src/deltacnn/cuda_kernels.py:13-185; the tensors stay owned by torch.

Differences a caller can see: launches go to torch's current stream (the reference uses
the legacy default stream); unsupported configurations, wrong devices, dtypes or memory
formats raise RuntimeError instead of printing or computing garbage; ``filter`` is in this
package's layout ([kh, kw, c_in/groups, c_out], see filter_conversion.py).
"""
import torch

from . import _lib
from ._lib import lib, check, ConvDesc, Epilogue

_DTYPES = {torch.float32: _lib.DC_F32, torch.float16: _lib.DC_F16}


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _dtype(x):
    try:
        return _DTYPES[x.dtype]
    except KeyError:
        raise RuntimeError(f"deltacnn_b200: unsupported dtype {x.dtype} (float32 and float16 only)") from None


def _check_feature(x, name):
    if not x.is_cuda:
        raise RuntimeError(f"deltacnn_b200: {name} must be a CUDA tensor (there is no CPU path)")
    if x.dim() != 4 or not x.is_contiguous(memory_format=torch.channels_last):
        raise RuntimeError(f"deltacnn_b200: {name} must be a 4-D channels_last contiguous tensor")


def _check_mask(m, x, name):
    if m is None:
        return
    if not m.is_cuda or m.dtype != torch.int32:
        raise RuntimeError(f"deltacnn_b200: {name} must be a CUDA int32 tensor")
    if m.numel() != x.shape[0] * x.shape[2] * x.shape[3]:
        raise RuntimeError(f"deltacnn_b200: {name} has {m.numel()} elements, expected one per pixel")


def _check_like(t, x, name):
    """A cache or output tensor handed over as a raw pointer must match ``x`` in shape, dtype, device and memory
    format: the kernels index it with x's geometry. A stale cache (batch or resolution changed without
    ``reset_layers()``) is an error here instead of an out-of-bounds access on the device."""
    if t is None:
        return
    if t.shape != x.shape or t.dtype != x.dtype or t.device != x.device:
        raise RuntimeError(f"deltacnn_b200: {name} is {tuple(t.shape)} {t.dtype} on {t.device}, expected {tuple(x.shape)} {x.dtype} on "
                           f"{x.device} (call reset_layers() after a batch or resolution change)")
    if not t.is_contiguous(memory_format=torch.channels_last):
        raise RuntimeError(f"deltacnn_b200: {name} must be channels_last contiguous")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _pad4(padding):
    if len(padding) == 2:
        return padding[0], padding[0], padding[1], padding[1]
    if len(padding) == 4:
        return padding[0], padding[1], padding[2], padding[3]   # (top, bottom, left, right), cuda_kernels.py:24-26
    raise RuntimeError("Padding must be iterable of size 2 or 4")


def make_conv_desc(x_shape, c_out, out_hw, kernel, stride, padding, dilation, groups, dtype_code):
    pt, pb, pl, pr = _pad4(padding)
    d = ConvDesc()
    d.n, d.c_in, d.h_in, d.w_in = x_shape
    d.h_out, d.w_out = out_hw
    d.c_out = c_out
    d.kh, d.kw = kernel
    d.stride_h, d.stride_w = stride
    d.pad_top, d.pad_left, d.pad_bottom, d.pad_right = pt, pl, pb, pr
    d.dil_h, d.dil_w = dilation
    d.groups = groups
    d.dtype = dtype_code
    return d


def conv_out_hw(h, w, kernel, stride, padding, dilation):
    pt, pb, pl, pr = _pad4(padding)
    out_h = int((h + pt + pb - dilation[0] * (kernel[0] - 1) - 1) // stride[0] + 1)
    out_w = int((w + pl + pr - dilation[1] * (kernel[1] - 1) - 1) // stride[1] + 1)
    return out_h, out_w


def conv_workspace_bytes(desc):
    """Scratch bytes the work-list kernels want for this geometry."""
    return int(lib.dc_conv_workspace_bytes(desc))


def make_epilogue(prev_out, truncated, threshold, activation, truncation_mode):
    e = Epilogue()
    e.prev_out = _ptr(prev_out)
    e.truncated = _ptr(truncated)
    e.threshold = float(threshold)
    e.activation = max(int(activation), 0)
    e.truncation = int(truncation_mode)
    return e


def make_residual_epilogue(residual, residual_mask, prev_out=None, activation=0):
    """Epilogue of a linear convolution that adds a residual (delta, mask) to its result, the out-mask becoming the
    union of both masks (the DCAdd behind the convolution, in the same launch). With ``activation`` > 0 the add
    layer's activation is applied too, ``prev_out`` being that layer's accumulated sum."""
    e = Epilogue()
    e.prev_out = _ptr(prev_out) if int(activation) > 0 else None
    e.truncated = None
    e.threshold = 0.0
    e.activation = max(int(activation), 0)
    e.truncation = -1
    e.residual = _ptr(residual)
    e.residual_mask = _ptr(residual_mask)
    return e


def sparse_conv(x, filter, mask=None, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, c_out: int = None,
                create_out_mask=False, sub_tile_sparsity=True, out_mask=None, out_shape=None, out=None,
                filter_umma=None, epilogue=None, desc=None, workspace=None):
    """Delta convolution (reference: cuda_kernels.py:13-45). Returns ``out`` or ``(out, out_mask)``.

    ``out`` / ``out_mask`` may be passed to reuse buffers; ``filter_umma`` is the packed
    tensor-core image of the same filter (optional); ``epilogue`` a ``make_epilogue`` result
    fusing activation + truncation; ``desc`` a cached ``make_conv_desc`` result; ``workspace`` a uint8
    scratch tensor of at least ``conv_workspace_bytes(desc)`` bytes enabling the work-list kernels.
    """
    _check_feature(x, "x")
    _check_mask(mask, x, "mask")
    kernel = (filter.shape[0], filter.shape[1])
    if out_shape is not None and len(out_shape) == 2:
        out_h, out_w = out_shape[0], out_shape[1]
    else:
        out_h, out_w = conv_out_hw(x.shape[2], x.shape[3], kernel, stride, padding, dilation)
        if type(out_shape) == list:
            out_shape.extend([out_h, out_w])
    out_c = filter.shape[3] if c_out is None else c_out
    if out is None:
        out = torch.empty((x.shape[0], out_c, out_h, out_w), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
    if mask is not None and out_mask is None and create_out_mask:
        out_mask = torch.empty((x.shape[0], 1, out_h, out_w), dtype=torch.int32, device=x.device)
    if desc is None:
        desc = make_conv_desc(tuple(x.shape), out_c, (out_h, out_w), kernel, stride, padding, dilation, groups, _dtype(x))
    if filter_umma is not None and mask is not None and out_mask is not None:
        filt, layout = filter_umma, _lib.DC_FILTER_UMMA
    else:
        filt, layout = filter, _lib.DC_FILTER_HWIO
        if filter.dtype != x.dtype:
            raise RuntimeError("deltacnn_b200.sparse_conv: filter dtype differs from input dtype")
    ws_ptr, ws_len = (workspace.data_ptr(), workspace.numel()) if (workspace is not None and mask is not None and out_mask is not None) else (None, 0)
    status = lib.dc_conv2d_ws(desc, x.data_ptr(), _ptr(mask), filt.data_ptr(), layout, _ptr(bias), out.data_ptr(), _ptr(out_mask),
                              epilogue, ws_ptr, ws_len, _stream())
    if status == 2 and layout == _lib.DC_FILTER_UMMA:
        # no tensor-core kernel for this call (e.g. a KxK filter without scratch): CUDA-core kernel, same result
        if filter.dtype != x.dtype:
            raise RuntimeError("deltacnn_b200.sparse_conv: filter dtype differs from input dtype")
        status = lib.dc_conv2d_ws(desc, x.data_ptr(), _ptr(mask), filter.data_ptr(), _lib.DC_FILTER_HWIO, _ptr(bias), out.data_ptr(),
                                  _ptr(out_mask), epilogue, ws_ptr, ws_len, _stream())
    check(status, "sparse_conv")
    if create_out_mask and mask is not None:
        return out, out_mask
    return out


def deconv_out_hw(h, w, kernel, stride, padding, dilation):
    out_h = int((h - 1) * stride[0] - 2 * padding[0] + dilation[0] * (kernel[0] - 1) + 1)
    out_w = int((w - 1) * stride[1] - 2 * padding[1] + dilation[1] * (kernel[1] - 1) + 1)
    return out_h, out_w


def sparse_deconv(x, filter, mask=None, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, c_out: int = None,
                  create_out_mask=False, sub_tile_sparsity=True, out_mask=None, out_shape=None, out=None, epilogue=None,
                  desc=None, filter_umma=None, workspace=None):
    """Delta transposed convolution (reference: cuda_kernels.py:47-78); output_padding is not applied."""
    _check_feature(x, "x")
    _check_mask(mask, x, "mask")
    kernel = (filter.shape[0], filter.shape[1])
    if out_shape is not None and len(out_shape) == 2:
        out_h, out_w = out_shape[0], out_shape[1]
    else:
        if len(padding) != 2:
            raise RuntimeError("Padding must be iterable of size 2")
        out_h, out_w = deconv_out_hw(x.shape[2], x.shape[3], kernel, stride, padding, dilation)
        if type(out_shape) == list:
            out_shape.extend([out_h, out_w])
    out_c = filter.shape[3] if c_out is None else c_out
    if out is None:
        out = torch.empty((x.shape[0], out_c, out_h, out_w), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
    if mask is not None and out_mask is None and create_out_mask:
        out_mask = torch.empty((x.shape[0], 1, out_h, out_w), dtype=torch.int32, device=x.device)
    if desc is None:
        desc = make_conv_desc(tuple(x.shape), out_c, (out_h, out_w), kernel, stride, padding, dilation, groups, _dtype(x))
    if filter.dtype != x.dtype:
        raise RuntimeError("deltacnn_b200.sparse_deconv: filter dtype differs from input dtype")
    ws_ptr, ws_len = (workspace.data_ptr(), workspace.numel()) if (workspace is not None and mask is not None and out_mask is not None) else (None, 0)
    status = 2
    if filter_umma is not None and mask is not None and out_mask is not None:     # with scratch: work lists; without: patch tiles
        status = lib.dc_deconv2d_ws(desc, x.data_ptr(), _ptr(mask), filter_umma.data_ptr(), _lib.DC_FILTER_UMMA, _ptr(bias),
                                    out.data_ptr(), _ptr(out_mask), epilogue, ws_ptr, ws_len, _stream())
    if status == 2:     # no tensor-core kernel for this call: CUDA-core kernel, same result
        status = lib.dc_deconv2d(desc, x.data_ptr(), _ptr(mask), filter.data_ptr(), _lib.DC_FILTER_HWIO, _ptr(bias), out.data_ptr(),
                                 _ptr(out_mask), epilogue, _stream())
    check(status, "sparse_deconv")
    if create_out_mask and mask is not None:
        return out, out_mask
    return out


def deconv_workspace_bytes(desc):
    """Scratch bytes the work-list transposed convolution wants for this geometry."""
    return int(lib.dc_deconv_workspace_bytes(desc))


def sparse_pooling(x, prev_x, kernel_size, mask=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), create_out_mask=True,
                   sub_tile_sparsity=True, out_mask=None, pooling_mode_int=0, out_shape=None, out=None, update_prev=False):
    """Delta max (mode 0) / average (mode 1) pooling (reference: cuda_kernels.py:80-129).

    ``update_prev`` additionally applies ``prev_x += x`` on masked pixels in the same call.
    The global average pool reduces in fp32 inside the kernel and stores the input dtype, so
    no fp32 staging buffer or cast is needed.
    """
    _check_feature(x, "x")
    _check_mask(mask, x, "mask")
    if out_shape is not None and len(out_shape) == 2:
        out_h, out_w = out_shape[0], out_shape[1]
    else:
        out_h, out_w = conv_out_hw(x.shape[2], x.shape[3], kernel_size, stride, padding, dilation)
        if type(out_shape) == list:
            out_shape.extend([out_h, out_w])
    c = x.shape[1]
    _check_like(prev_x, x, "prev_x")
    if out is None:
        out = torch.empty((x.shape[0], c, out_h, out_w), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
    elif tuple(out.shape) != (x.shape[0], c, out_h, out_w) or out.dtype != x.dtype:
        raise RuntimeError("deltacnn_b200.sparse_pooling: out has the wrong shape or dtype")
    if mask is not None and out_mask is None and create_out_mask:
        out_mask = torch.empty((x.shape[0], 1, out_h, out_w), dtype=torch.int32, device=x.device)
    desc = make_conv_desc(tuple(x.shape), c, (out_h, out_w), tuple(kernel_size), stride, padding, dilation, 1, _dtype(x))
    check(lib.dc_pool(desc, x.data_ptr(), _ptr(prev_x), _ptr(mask), out.data_ptr(), _ptr(out_mask), int(pooling_mode_int),
                      1 if update_prev else 0, _stream()), "sparse_pooling")
    if create_out_mask and mask is not None:
        return out, out_mask
    return out


def _npix(x):
    return x.shape[0] * x.shape[2] * x.shape[3]


def sparse_activation(x, prev_x, truncated, mask, threshold, activation, truncation_mode):
    """In-place accumulate + activation delta + truncation (reference: cuda_kernels.py:132-133)."""
    _check_feature(x, "x")
    _check_mask(mask, x, "mask")
    _check_like(prev_x, x, "prev_x")
    _check_like(truncated, x, "truncated")
    check(lib.dc_activate_truncate(x.data_ptr(), prev_x.data_ptr(), _ptr(truncated), mask.data_ptr(), _npix(x), x.shape[1],
                                   _dtype(x), float(threshold), max(int(activation), 0), int(truncation_mode), _stream()),
          "sparse_activation")


def sparsify(input, prev_in, delta, mask, threshold):
    """Input delta + update mask (reference: cuda_kernels.py:136-137)."""
    _check_feature(input, "input")
    _check_mask(mask, input, "mask")
    _check_like(prev_in, input, "prev_in")
    _check_like(delta, input, "delta")
    check(lib.dc_sparsify(input.data_ptr(), prev_in.data_ptr(), delta.data_ptr(), mask.data_ptr(), _npix(input),
                          input.shape[1], _dtype(input), float(threshold), _stream()), "sparsify")


def sparsify_u8(frame_u8, scale, offset, prev_in, delta, mask, threshold):
    """``sparsify`` on an 8-bit N,H,W,C frame normalised per channel by ``scale``/``offset`` (float32)."""
    _check_feature(delta, "delta")
    _check_like(prev_in, delta, "prev_in")
    _check_mask(mask, delta, "mask")
    if frame_u8.dtype != torch.uint8 or not frame_u8.is_contiguous() or \
            tuple(frame_u8.shape) != (delta.shape[0], delta.shape[2], delta.shape[3], delta.shape[1]):
        raise RuntimeError("deltacnn_b200.sparsify_u8: the frame must be a contiguous uint8 tensor of shape (N, H, W, C) matching delta")
    check(lib.dc_sparsify_u8(frame_u8.data_ptr(), scale.data_ptr(), offset.data_ptr(), prev_in.data_ptr(), delta.data_ptr(),
                             mask.data_ptr(), _npix(delta), delta.shape[1], _dtype(delta), float(threshold), _stream()),
          "sparsify_u8")


def sparse_add_tensors(a, b, prev_out, out, mask_a, mask_b, mask_out, weight_a, weight_b, activation, dense_out):
    """Weighted add of two delta tensors (reference: cuda_kernels.py:140-141)."""
    _check_feature(a, "a")
    _check_feature(b, "b")
    if a.shape != b.shape:
        raise RuntimeError("deltacnn_b200.sparse_add_tensors: shapes differ")
    _check_like(prev_out, a, "prev_out")
    _check_like(out, a, "out")
    _check_mask(mask_a, a, "mask_a")
    _check_mask(mask_b, a, "mask_b")
    _check_mask(mask_out, a, "mask_out")
    check(lib.dc_add(a.data_ptr(), b.data_ptr(), _ptr(prev_out), out.data_ptr(), mask_a.data_ptr(), mask_b.data_ptr(),
                     _ptr(mask_out), float(weight_a), float(weight_b), _npix(a), a.shape[1], _dtype(a),
                     max(int(activation), 0), 1 if dense_out else 0, _stream()), "sparse_add_tensors")


def sparse_add_to_dense_tensor(a, b, mask_a, activation=0):
    """b += a on the masked pixels of a (reference: cuda_kernels.py:144-145; the activation argument is unused there too)."""
    _check_feature(a, "a")
    _check_like(b, a, "b")
    _check_mask(mask_a, a, "mask_a")
    check(lib.dc_add_to_dense(a.data_ptr(), b.data_ptr(), mask_a.data_ptr(), _npix(a), a.shape[1], _dtype(a), _stream()),
          "sparse_add_to_dense_tensor")


def sparse_mul_add(x, x_mask, out, out_mask, scale, bias):
    """Per-channel scale (+bias) on masked pixels (reference: cuda_kernels.py:148-149)."""
    _check_feature(x, "x")
    scale = scale.reshape(-1).to(x.dtype).contiguous()
    bias = None if bias is None else bias.reshape(-1).to(x.dtype).contiguous()
    check(lib.dc_scale_bias(x.data_ptr(), _ptr(x_mask), out.data_ptr(), _ptr(out_mask), scale.data_ptr(), _ptr(bias),
                            _npix(x), x.shape[1], _dtype(x), _stream()), "sparse_mul_add")


def sparse_upsample(input, mask_in, scale, out=None):
    """Nearest-neighbour upsampling of values and mask (reference: cuda_kernels.py:152-166)."""
    _check_feature(input, "input")
    if out is None:
        n, c, h, w = input.shape
        o = torch.empty((n, c, h * scale, w * scale), device=input.device, dtype=input.dtype, memory_format=torch.channels_last)
        mask_out = torch.empty((n, 1, h * scale, w * scale), device=input.device, dtype=torch.int)
    else:
        o, mask_out = out
    n, c, h, w = input.shape
    check(lib.dc_upsample(input.data_ptr(), mask_in.data_ptr(), o.data_ptr(), mask_out.data_ptr(), n, h, w, c, int(scale),
                          _dtype(input), _stream()), "sparse_upsample")
    return o, mask_out


def sparse_concatenate(a, b, out=None):
    """Channel concatenation of two (delta, mask) pairs (reference: cuda_kernels.py:169-185)."""
    a, mask_a = a
    b, mask_b = b
    _check_feature(a, "a")
    _check_feature(b, "b")
    if out is None:
        o = torch.empty((a.shape[0], a.shape[1] + b.shape[1], a.shape[2], a.shape[3]), device=a.device, dtype=a.dtype,
                        memory_format=torch.channels_last)
        mask_out = torch.empty((a.shape[0], 1, a.shape[2], a.shape[3]), device=a.device, dtype=torch.int)
    else:
        o, mask_out = out
    check(lib.dc_concat(a.data_ptr(), b.data_ptr(), o.data_ptr(), mask_a.data_ptr(), mask_b.data_ptr(), mask_out.data_ptr(),
                        _npix(a), a.shape[1], b.shape[1], _dtype(a), _stream()), "sparse_concatenate")
    return o, mask_out


def sparse_densify(delta, mask, prev_out, out=None, activation=0):
    """prev_out += delta on masked pixels; ``out`` (new tensor when None) = f(prev_out).
    One launch for the reference's accumulate + clone + activation (sparse_layers.py:1322-1329)."""
    _check_feature(delta, "delta")
    _check_like(prev_out, delta, "prev_out")
    _check_mask(mask, delta, "mask")
    if out is None:
        out = torch.empty_like(prev_out)
    _check_like(out, delta, "out")
    check(lib.dc_densify(delta.data_ptr(), mask.data_ptr(), prev_out.data_ptr(), out.data_ptr(), _npix(delta), delta.shape[1],
                         _dtype(delta), max(int(activation), 0), _stream()), "sparse_densify")
    return out


def compact_mask(mask, indices=None, count=None):
    """Indices of the active pixels of ``mask`` (order unspecified) and their number, on the device."""
    n = mask.numel()
    if indices is None:
        indices = torch.empty(n, dtype=torch.int32, device=mask.device)
    if count is None:
        count = torch.empty(1, dtype=torch.int32, device=mask.device)
    check(lib.dc_compact_mask(mask.data_ptr(), n, indices.data_ptr(), count.data_ptr(), _stream()), "compact_mask")
    return indices, count


class DCPerformanceMetrics:
    """Host-side accounting of one frame (reference: cuda_kernels.py:188-245 reads device counters
    that are compiled out by default, src/cuda/common.cuh:37). Filled by ``DCPerformanceMetricsManager``
    from the masks the layers produced."""

    def __init__(self, tiles, inputs, flops, memtransfer, n_frames=1):
        n_frames = max(n_frames, 1)
        self.tiles_active, self.tiles_total = tiles[0] // n_frames, tiles[1] // n_frames
        self.tiles_ratio = self.tiles_active / max(self.tiles_total, 1)
        self.inputs_active, self.inputs_total = inputs[0] // n_frames, inputs[1] // n_frames
        self.inputs_ratio = self.inputs_active / max(self.inputs_total, 1)
        self.flops_actual, self.flops_theoretical, self.flops_dense = (f // n_frames for f in flops)
        self.flops_ratio_actual = self.flops_actual / max(self.flops_dense, 1)
        self.flops_ratio_theoretical = self.flops_theoretical / max(self.flops_dense, 1)
        self.mem_read_actual, self.mem_read_dense, self.mem_write_actual, self.mem_write_dense = (m // n_frames for m in memtransfer)
        self.mem_read_ratio = self.mem_read_actual / max(self.mem_read_dense, 1)
        self.mem_write_ratio = self.mem_write_actual / max(self.mem_write_dense, 1)

    def to_dict(self):
        return dict(self.__dict__)

    def save_json(self, path):
        import json
        with open(path, "w+") as f:
            json.dump(self.to_dict(), f)


class DCPerformanceMetricsManager:
    """Collects per-layer work records appended by the layers while ``enabled`` is True."""
    enabled = False
    records = []

    @classmethod
    def init(cls):
        return True

    @classmethod
    def reset(cls):
        cls.records = []

    @classmethod
    def add(cls, record):
        cls.records.append(record)

    @classmethod
    def get_metrics(cls, n_frames=1):
        tiles, inputs, flops, mem = [0, 0], [0, 0], [0, 0, 0], [0, 0, 0, 0]
        for r in cls.records:
            for acc, key in ((tiles, "tiles"), (inputs, "inputs"), (flops, "flops"), (mem, "mem")):
                for i, v in enumerate(r.get(key, ())):
                    acc[i] += int(v)
        return DCPerformanceMetrics(tiles, inputs, flops, mem, n_frames=n_frames)
