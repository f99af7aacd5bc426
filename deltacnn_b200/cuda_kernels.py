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
    for t, name in ((frame_u8, "frame"), (scale, "scale"), (offset, "offset"), (prev_in, "prev_in"), (mask, "mask")):
        if t.device != delta.device:
            raise RuntimeError(f"deltacnn_b200.sparsify_u8: {name} is on {t.device}, the delta tensor on {delta.device}")
    if scale.dtype != torch.float32 or offset.dtype != torch.float32 or scale.numel() != delta.shape[1] or offset.numel() != delta.shape[1]:
        raise RuntimeError("deltacnn_b200.sparsify_u8: scale and offset must be float32 with one entry per channel")
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


def sparsify_dilated(input, prev_in, delta, mask, hit_scratch, threshold, dilation):
    """``DCSparsify(dilation=k)``: dense difference, k x k window OR of the per-pixel threshold test, cache update
    where the mask is set (reference: sparse_layers.py:1233-1248, torch ops there). ``hit_scratch``: uint8, one
    byte per pixel."""
    _check_feature(input, "input")
    _check_mask(mask, input, "mask")
    _check_like(prev_in, input, "prev_in")
    _check_like(delta, input, "delta")
    if hit_scratch.dtype != torch.uint8 or hit_scratch.numel() < _npix(input) or hit_scratch.device != input.device:
        raise RuntimeError("deltacnn_b200.sparsify_dilated: hit_scratch must hold one byte per pixel on the input's device")
    n, c, h, w = input.shape
    check(lib.dc_sparsify_dilated(input.data_ptr(), prev_in.data_ptr(), delta.data_ptr(), mask.data_ptr(), hit_scratch.data_ptr(),
                                  n, h, w, c, _dtype(input), float(threshold), int(dilation), _stream()), "sparsify_dilated")


def linear_delta(delta, mask, weight, bias, acc, out, first_frame):
    """Fully connected layer in delta form: ``acc += delta @ weight.T`` (+ bias on the first frame) for the streams
    whose mask is set, ``out = acc`` in the feature dtype. ``delta``: (N, C) or (N, C, 1, 1); ``mask``: one int32 per
    stream; ``acc``: (N, out) float32 state. No reference counterpart (it replaces densify + nn.Linear,
    example/mobilenet_deltacnn.py:216-227)."""
    if not delta.is_cuda:
        raise RuntimeError("deltacnn_b200: delta must be a CUDA tensor (there is no CPU path)")
    n, c_in = delta.shape[0], delta.shape[1]
    c_out = weight.shape[0]
    if delta.numel() != n * c_in or tuple(weight.shape) != (c_out, c_in) or not weight.is_contiguous() or weight.dtype != delta.dtype:
        raise RuntimeError("deltacnn_b200.linear_delta: delta must be (N, C[, 1, 1]) and weight a contiguous (out, C) tensor of the same dtype")
    if acc.dtype != torch.float32 or tuple(acc.shape) != (n, c_out) or tuple(out.shape) != (n, c_out) or out.dtype != delta.dtype:
        raise RuntimeError("deltacnn_b200.linear_delta: acc must be float32 (N, out) and out (N, out) in the feature dtype")
    if mask is not None and (mask.dtype != torch.int32 or mask.numel() != n):
        raise RuntimeError("deltacnn_b200.linear_delta: mask must hold one int32 per stream")
    check(lib.dc_linear_delta(delta.data_ptr(), _ptr(mask), weight.data_ptr(), _ptr(bias), acc.data_ptr(), out.data_ptr(),
                              n, c_in, c_out, _dtype(delta), 1 if first_frame else 0, _stream()), "linear_delta")
    return out


def heatmap_argmax(heat, mask, out=None):
    """(x, y, value) of the largest element of every heat map of a dense (N, J, H, W) channels-last tensor; streams
    whose mask is empty keep their rows of ``out``. Returns a float32 (N, J, 3) tensor."""
    _check_feature(heat, "heat")
    _check_mask(mask, heat, "mask")
    n, j, h, w = heat.shape
    if out is None:
        if mask is not None:
            raise RuntimeError("deltacnn_b200.heatmap_argmax: the first call (no previous result) must not pass a mask")
        out = torch.empty((n, j, 3), dtype=torch.float32, device=heat.device)
    check(lib.dc_heatmap_argmax(heat.data_ptr(), _ptr(mask), out.data_ptr(), n, h, w, j, _dtype(heat), _stream()), "heatmap_argmax")
    return out


def centernet_decode(heat, wh, offset, mask, state=None, topk=100, min_score=0.0, stride=4.0, apply_sigmoid=False):
    """CenterNet decode of dense head outputs on the device: 3x3 peak test, top-k, boxes. ``state`` is the tuple
    (peaks, det, count) returned by the previous call (None on the first frame, where ``mask`` must be None);
    returns (det (N, topk, 6) float32, count (N,) int32, state)."""
    _check_feature(heat, "heat")
    _check_feature(wh, "wh")
    _check_feature(offset, "offset")
    _check_mask(mask, heat, "mask")
    n, classes, h, w = heat.shape
    if tuple(wh.shape) != (n, 2, h, w) or tuple(offset.shape) != (n, 2, h, w) or wh.dtype != heat.dtype or offset.dtype != heat.dtype:
        raise RuntimeError("deltacnn_b200.centernet_decode: wh and offset must be (N, 2, H, W) tensors of the heat map's dtype")
    if state is None:
        if mask is not None:
            raise RuntimeError("deltacnn_b200.centernet_decode: the first call (no state) must not pass a mask")
        state = (torch.empty((n, h, w, classes), dtype=torch.float32, device=heat.device),
                 torch.empty((n, topk, 6), dtype=torch.float32, device=heat.device),
                 torch.empty((n,), dtype=torch.int32, device=heat.device))
    peaks, det, count = state
    if tuple(det.shape) != (n, topk, 6) or peaks.numel() != n * h * w * classes:
        raise RuntimeError("deltacnn_b200.centernet_decode: state does not match the input (call reset_layers())")
    check(lib.dc_centernet_decode(heat.data_ptr(), wh.data_ptr(), offset.data_ptr(), _ptr(mask), peaks.data_ptr(), det.data_ptr(),
                                  count.data_ptr(), n, h, w, classes, int(topk), float(min_score), float(stride),
                                  1 if apply_sigmoid else 0, _dtype(heat), _stream()), "centernet_decode")
    return det, count, state


def make_irb_desc(x_shape, c_hidden, c_out, stride, residual, act_expand, act_dw, thr_expand, thr_dw):
    d = _lib.IrbDesc()
    d.n, d.c_in, d.h, d.w = x_shape
    d.c_hidden, d.c_out, d.stride, d.residual = int(c_hidden), int(c_out), int(stride), 1 if residual else 0
    d.act_expand, d.act_dw, d.dtype = max(int(act_expand), 0), max(int(act_dw), 0), _lib.DC_F16
    d.thr_expand, d.thr_dw = float(thr_expand), float(thr_dw)
    return d


def irb_supported(desc):
    """True when ``fused_inverted_residual`` has a kernel for this block shape (small maps, fp16)."""
    return bool(lib.dc_irb_supported(desc))


def fused_inverted_residual(x, mask, w_expand_umma, w_dw, w_project_umma, prev_expand, trunc_expand, prev_dw, trunc_dw, out, mask_out, desc):
    """One launch for a whole inverted-residual block on a steady-state frame: expansion 1x1 + activation/truncation,
    depthwise 3x3 + activation/truncation, projection 1x1 and the residual add, with the results and cache updates of
    the separate calls bit for bit. No reference counterpart (the reference issues six launches per block,
    example/mobilenet_deltacnn.py:87-128). ``desc`` from ``make_irb_desc``; returns (out, mask_out)."""
    _check_feature(x, "x")
    _check_mask(mask, x, "mask")
    n, _, h, w = x.shape
    ho, wo = (h - 1) // desc.stride + 1, (w - 1) // desc.stride + 1
    for t, shape, name in ((prev_expand, (n, desc.c_hidden, h, w), "prev_expand"), (trunc_expand, (n, desc.c_hidden, h, w), "trunc_expand"),
                           (prev_dw, (n, desc.c_hidden, ho, wo), "prev_dw"), (trunc_dw, (n, desc.c_hidden, ho, wo), "trunc_dw"),
                           (out, (n, desc.c_out, ho, wo), "out")):
        if tuple(t.shape) != shape or t.dtype != x.dtype or t.device != x.device or not t.is_contiguous(memory_format=torch.channels_last):
            raise RuntimeError(f"deltacnn_b200.fused_inverted_residual: {name} must be a channels_last {shape} tensor like x "
                               "(call reset_layers() after a batch or resolution change)")
    if mask_out.dtype != torch.int32 or mask_out.numel() != n * ho * wo:
        raise RuntimeError("deltacnn_b200.fused_inverted_residual: mask_out must hold one int32 per output pixel")
    check(lib.dc_irb_fused(desc, x.data_ptr(), mask.data_ptr(), w_expand_umma.data_ptr(), w_dw.data_ptr(), w_project_umma.data_ptr(),
                           prev_expand.data_ptr(), trunc_expand.data_ptr(), prev_dw.data_ptr(), trunc_dw.data_ptr(), out.data_ptr(),
                           mask_out.data_ptr(), _stream()), "fused_inverted_residual")
    return out, mask_out


def conv3x3_heads_supported(desc, n_heads):
    """Whether ``conv3x3_heads`` has a kernel for the concatenated layer ``desc`` (c_out = all heads' output channels)."""
    return bool(lib.dc_conv3x3_heads_supported(desc, int(n_heads)))


def conv3x3_heads(x, mask, filter_umma, bias, outs, masks_out, desc, epilogues=None):
    """Several stride-1 3x3 convolutions on the same input (delta, mask) in one launch; head h writes ``outs[h]`` /
    ``masks_out[h]`` and, with ``epilogues`` (one ``make_epilogue`` per head), runs that head's activation/truncation
    step in the same launch. ``desc`` is the descriptor of the concatenated layer, ``filter_umma`` / ``bias`` the packed
    filter / bias of the filters concatenated along the output channels. Same results per head as ``sparse_conv`` with a
    fused epilogue. No reference counterpart (the reference runs every head's convolution and truncation on its own,
    src/cuda/conv_torch_wrapper.cpp:62-134, 295-344)."""
    import ctypes
    _check_feature(x, "x")
    _check_mask(mask, x, "mask")
    nh = len(outs)
    if len(masks_out) != nh or (epilogues is not None and len(epilogues) != nh):
        raise RuntimeError("deltacnn_b200.conv3x3_heads: outs, masks_out and epilogues must have one entry per head")
    n = x.shape[0]
    seg = desc.c_out // max(nh, 1)
    for h, (o, m) in enumerate(zip(outs, masks_out)):
        if tuple(o.shape) != (n, seg, desc.h_out, desc.w_out) or o.dtype != x.dtype or o.device != x.device or \
                not o.is_contiguous(memory_format=torch.channels_last):
            raise RuntimeError(f"deltacnn_b200.conv3x3_heads: outs[{h}] must be a channels_last {(n, seg, desc.h_out, desc.w_out)} tensor like x")
        if m.dtype != torch.int32 or m.device != x.device or m.numel() != n * desc.h_out * desc.w_out:
            raise RuntimeError(f"deltacnn_b200.conv3x3_heads: masks_out[{h}] must hold one int32 per output pixel")
    out_ptrs = (ctypes.c_void_p * nh)(*[o.data_ptr() for o in outs])
    mask_ptrs = (ctypes.c_void_p * nh)(*[m.data_ptr() for m in masks_out])
    eps = None
    if epilogues is not None:
        eps = (Epilogue * nh)(*epilogues)
    check(lib.dc_conv3x3_heads(desc, x.data_ptr(), mask.data_ptr(), filter_umma.data_ptr(), _ptr(bias), nh, out_ptrs, mask_ptrs, eps,
                               _stream()), "conv3x3_heads")
    return outs, masks_out


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
    """Work accounting of the delta path over one or more frames, with the fields and ratios of the reference's
    class (src/deltacnn/cuda_kernels.py:188-245). The reference fills it from device counters that its kernels
    increment with atomics when built with ENABLE_METRICS (src/cuda/common.cuh:37-65, off by default); here the
    same quantities are computed from the layers' masks by ``DCPerformanceMetricsManager`` (no atomics in the
    kernels). Counts are per frame (totals divided by ``n_frames``); "flops" count multiply-accumulates, "mem" counts
    tensor elements, as in the reference."""

    def __init__(self, tiles, inputs, mode, flops, memtransfer, histogram, n_frames=1):
        n_frames = max(n_frames, 1)
        val = lambda v: int(v) // n_frames
        self.tiles_active, self.tiles_total = val(tiles[0]), val(tiles[1])
        self.tiles_ratio = self.tiles_active / max(self.tiles_total, 1)
        self.inputs_active, self.inputs_total = val(inputs[0]), val(inputs[1])
        self.inputs_ratio = self.inputs_active / max(self.inputs_total, 1)
        self.mode_sparse, self.mode_dense = val(mode[0]), val(mode[1])
        self.mode_ratio = self.mode_sparse / max(self.mode_sparse + self.mode_dense, 1)
        self.flops_actual, self.flops_theoretical, self.flops_dense = (val(f) for f in flops)
        self.flops_ratio_actual = self.flops_actual / max(self.flops_dense, 1)
        self.flops_ratio_theoretical = self.flops_theoretical / max(self.flops_dense, 1)
        self.mem_read_actual, self.mem_read_dense, self.mem_write_actual, self.mem_write_dense = (val(m) for m in memtransfer)
        self.mem_read_ratio = self.mem_read_actual / max(self.mem_read_dense, 1)
        self.mem_write_ratio = self.mem_write_actual / max(self.mem_write_dense, 1)
        self.histogram = [int(h) // n_frames for h in histogram]
        active = max(sum(int(h) for h in histogram[1:]), 1)
        self.histogram_ratio = [int(h) / active for h in histogram]

    def to_dict(self):
        return dict(self.__dict__)

    def save_json(self, path):
        import json
        with open(path, "w+") as f:
            json.dump(self.to_dict(), f)


class DCPerformanceMetricsManager:
    """Collects the counters of ``DCPerformanceMetrics`` while ``enabled`` is True (the reference's switch is the
    compile-time ENABLE_METRICS). Every delta convolution and every truncation layer adds its frame's work through
    ``add_conv`` / ``add_activation``; the sums stay on the device as int64 until ``get_metrics()`` reads them, so
    collecting does not synchronise the stream.

    Definitions, restated from the reference's counters (src/cuda/conv_kernel.cu:90-107, 196-217, 319-332;
    src/cuda/other_nn_layers.cu:808-813), with an 8x8 output tile for every layer (the reference's tile size varies
    with its kernel heuristics):
      tiles     every tile / tiles with an active input pixel in their receptive field
      inputs    receptive-field pixels of every tile / the active ones among them
      histogram tiles by number of active input pixels (128 bins, the last holds 127 and more)
      flops     actual: kernel MACs of every output pixel of an active tile (depthwise: of its active taps);
                theoretical: active taps x Cin x Cout / groups of every updated output pixel; dense: all pixels
      mem       read: active inputs x Cin + the filter, per active tile; written: Cout per updated output pixel;
                dense: all inputs / outputs; truncation layers add 2 C read and 2 C written per masked pixel
      mode      tiles handled with / without sub-tile sparsity (the reference's 3x3 kernel switches per tile; every
                tile of this library's kernels gathers only active pixels, so all active tiles count as sparse)."""
    enabled = False
    tile = 8
    _acc = None            # int64 device tensor: 13 counters followed by the 128 histogram bins
    N_BINS = 128

    @classmethod
    def init(cls):
        return True

    @classmethod
    def reset(cls):
        cls._acc = None

    @classmethod
    def _accumulate(cls, device, scalars, hist=None):
        if cls._acc is None or cls._acc.device != device:
            cls._acc = torch.zeros(13 + cls.N_BINS, dtype=torch.int64, device=device)
        cls._acc[:13] += torch.stack([torch.as_tensor(v, dtype=torch.int64, device=device) for v in scalars])
        if hist is not None:
            cls._acc[13:] += hist

    @classmethod
    def add_conv(cls, mask_in, c_in, c_out, kernel, stride, padding, dilation, groups, out_hw, transposed=False):
        """Account one delta convolution call from its in-mask (N,1,H,W int32) and geometry."""
        if not cls.enabled or transposed:
            return
        import torch.nn.functional as F
        t = cls.tile
        n, _, h, w = mask_in.shape
        ho, wo = out_hw
        kh, kw = kernel
        pt, pb, pl, pr = _pad4(padding)
        m = (mask_in != 0).float()
        # receptive field of a t x t tile of outputs; pad so that every (also partial) tile has a full window
        rh, rw = (t - 1) * stride[0] + (kh - 1) * dilation[0] + 1, (t - 1) * stride[1] + (kw - 1) * dilation[1] + 1
        ty, tx = -(-ho // t), -(-wo // t)
        need_h, need_w = (ty - 1) * t * stride[0] + rh, (tx - 1) * t * stride[1] + rw
        mp = F.pad(m, (pl, max(need_w - w - pl, 0), pt, max(need_h - h - pt, 0)))[:, :, :need_h, :need_w]
        dens = F.avg_pool2d(mp, (rh, rw), stride=(t * stride[0], t * stride[1]), divisor_override=1)
        dens = dens.round().long()                                   # (N,1,ty,tx) active inputs per tile
        active_tile = dens > 0
        # per output pixel: number of active taps (in-bounds) and the updated flag
        ones = torch.ones(1, 1, kh, kw, device=m.device)
        taps = F.conv2d(F.pad(m, (pl, pr, pt, pb)), ones, None, stride, 0, dilation).round().long()[:, :, :ho, :wo]
        updated = taps > 0
        tile_of = active_tile.repeat_interleave(t, 2).repeat_interleave(t, 3)[:, :, :ho, :wo]
        per_px = kh * kw * c_in * c_out // groups
        cig = c_in * c_out // groups                                 # MACs per active tap
        n_tiles = n * ty * tx
        if groups == 1:
            flops_actual = tile_of.sum() * per_px
        else:
            flops_actual = (taps * tile_of).sum() * cig
        filt = kh * kw * c_in * c_out // groups
        scalars = [
            active_tile.sum(), n_tiles, dens.sum(), n_tiles * rh * rw,
            active_tile.sum(), 0,
            flops_actual, taps.sum() * cig, n * ho * wo * per_px,
            dens.sum() * c_in + active_tile.sum() * filt, n_tiles * (rh * rw * c_in + filt),
            updated.sum() * c_out, n * ho * wo * c_out,
        ]
        hist = torch.bincount(dens.clamp(max=cls.N_BINS - 1).flatten(), minlength=cls.N_BINS)
        cls._accumulate(mask_in.device, scalars, hist)

    @classmethod
    def add_activation(cls, mask_in, channels, truncation_mode=0, mask_kept=None):
        """Account one truncation layer call: 2 C (3 C for norm/rms) elements read per masked pixel; 2 C written
        (3 C where a norm/rms pixel stays active)."""
        if not cls.enabled:
            return
        m_in = (mask_in != 0).sum()
        read = (2 if truncation_mode == 0 else 3) * channels * m_in
        if truncation_mode == 0 or mask_kept is None:
            written = 2 * channels * m_in
        else:
            written = channels * (2 * m_in + (mask_kept != 0).sum())
        zero = 0
        cls._accumulate(mask_in.device, [zero, zero, zero, zero, zero, zero, zero, zero, zero, read, read, written, written])

    @classmethod
    def get_metrics(cls, n_frames=1):
        if cls._acc is None:
            vals = [0] * (13 + cls.N_BINS)
        else:
            vals = cls._acc.cpu().tolist()
        return DCPerformanceMetrics(vals[0:2], vals[2:4], vals[4:6], vals[6:9], vals[9:13], vals[13:], n_frames=n_frames)
