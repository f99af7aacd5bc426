"""ctypes access to the reference project's own CUDA kernels (TEST INFRASTRUCTURE).

oracle/_ref/libdeltacnn_ref.so is built by oracle/Makefile from the reference sources plus the shim
oracle/ref_shim.cu. This module feeds it torch CUDA tensors, so GPU tests can compare this library's
kernels with the reference's on the same inputs, and so fixtures can be recorded from the reference.
The reference launches on the legacy default stream; every call here synchronises.
"""
import ctypes
import os

import torch

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libdeltacnn_ref.so")
_lib = None


def available():
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIB_PATH)
    return _lib


def _p(t):
    return ctypes.c_void_p(None if t is None else t.data_ptr())


def _ints(*v):
    return (ctypes.c_int * len(v))(*[int(x) for x in v])


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"reference kernel {what} failed with code {rc}")


def _f16(x):
    return 1 if x.dtype == torch.float16 else 0


def ref_filter(weight, transposed=False):
    """torch-layout filter -> the layout the reference kernels read: [c_in, kh, kw, c_out]
    (src/deltacnn/filter_conversion.py:8-11); for fp16 non-depthwise filters additionally the pair
    swizzle of :13-38 (odd output channels take their input-channel pairs swapped, channel counts
    padded to even)."""
    w = weight.transpose(0, 1) if transposed else weight          # -> [c_out, c_in, kh, kw]
    x = w.permute(1, 2, 3, 0).contiguous()                        # [c_in, kh, kw, c_out]
    if weight.dtype != torch.float16:
        return x.clone()
    cin, kh, kw, cout = x.shape
    depthwise = (not transposed) and weight.shape[1] == 1 and cout > 1
    if depthwise:
        return x.clone()
    res = torch.zeros((cin + cin % 2, kh, kw, cout + cout % 2), dtype=torch.float16, device=x.device)

    def put(dst, src):
        dst[:src.shape[0], :, :, :src.shape[-1]] += src

    put(res[::2, :, :, ::2], x[::2, :, :, ::2])
    put(res[::2, :, :, 1::2], x[1::2, :, :, 1::2])
    put(res[1::2, :, :, ::2], x[1::2, :, :, ::2])
    put(res[1::2, :, :, 1::2], x[::2, :, :, 1::2])
    return res


def _conv_like(fn, x, mask, filt, bias, out_hw, cout, kernel, stride, padding4, dilation, groups):
    n, cin, h, w = x.shape
    out = torch.zeros((n, cout, out_hw[0], out_hw[1]), dtype=x.dtype, device=x.device).contiguous(memory_format=torch.channels_last)
    om = torch.zeros((n, 1, out_hw[0], out_hw[1]), dtype=torch.int32, device=x.device)
    shape = _ints(n, h, w, cin, out_hw[0], out_hw[1], cout)
    pt, pb, pl, pr = padding4
    geom = _ints(kernel[0], kernel[1], stride[0], stride[1], pt, pl, pb, pr, dilation[0], dilation[1], groups)
    torch.cuda.synchronize()
    _check(fn(_f16(x), _p(x), _p(out), _p(filt), _p(bias), _p(mask), _p(om), shape, geom, 1), "conv")
    return out, om


def conv(x, mask, weight, bias, stride, padding, dilation=(1, 1), groups=1):
    from .delta_ops import conv_out_size, _pad4
    k = tuple(weight.shape[2:])
    hw = conv_out_size(x.shape[2], x.shape[3], k, stride, padding, dilation)
    return _conv_like(lib().ref_conv, x, mask, ref_filter(weight), bias, hw, weight.shape[0], k, stride, _pad4(padding), dilation, groups)


def deconv(x, mask, weight, bias, stride, padding):
    from .delta_ops import deconv_out_size
    k = tuple(weight.shape[2:])
    hw = deconv_out_size(x.shape[2], x.shape[3], k, stride, padding, (1, 1))
    return _conv_like(lib().ref_deconv, x, mask, ref_filter(weight, transposed=True), bias, hw, weight.shape[1], k, stride,
                      (padding[0], padding[0], padding[1], padding[1]), (1, 1), 1)


def sparsify(x, prev_in, threshold):
    """Returns (delta, mask); prev_in is updated in place."""
    n, c, h, w = x.shape
    delta = torch.zeros_like(x)
    mask = torch.zeros((n, 1, h, w), dtype=torch.int32, device=x.device)
    torch.cuda.synchronize()
    _check(lib().ref_sparsify(_f16(x), _p(x), _p(prev_in), _p(delta), _p(mask), ctypes.c_float(threshold), n, h, w, c, 1), "sparsify")
    return delta, mask


def activate_truncate(delta, prev_out, truncated, mask, threshold, activation, truncation_mode):
    n, c, h, w = delta.shape
    torch.cuda.synchronize()
    _check(lib().ref_activate_truncate(_f16(delta), _p(delta), _p(prev_out), _p(truncated), _p(mask), ctypes.c_float(threshold),
                                       n, h, w, c, activation, truncation_mode, 1), "activate_truncate")


def add(a, ma, b, mb, prev_out, wa, wb, activation, dense_out):
    n, c, h, w = a.shape
    out = torch.zeros_like(a)
    mo = torch.zeros((n, 1, h, w), dtype=torch.int32, device=a.device)
    torch.cuda.synchronize()
    _check(lib().ref_add(_f16(a), _p(a), _p(b), _p(prev_out), _p(out), _p(ma), _p(mb), _p(mo), ctypes.c_float(wa), ctypes.c_float(wb),
                         n, h, w, c, activation, 1 if dense_out else 0, 1), "add")
    return out, mo


def max_pool(x, mask, prev_in, kernel, stride, padding):
    """``padding``: (h, w) or (top, bottom, left, right) as in the Python API; the kernel config takes
    (top, left, bottom, right) (src/deltacnn/cuda_kernels.py:43-47)."""
    from .delta_ops import conv_out_size, _pad4
    n, c, h, w = x.shape
    ho, wo = conv_out_size(h, w, kernel, stride, padding, (1, 1))
    pt, pb, pl, pr = _pad4(padding)
    out = torch.zeros((n, c, ho, wo), dtype=x.dtype, device=x.device).contiguous(memory_format=torch.channels_last)
    om = torch.zeros((n, 1, ho, wo), dtype=torch.int32, device=x.device)
    shape = _ints(n, h, w, c, ho, wo, c)
    geom = _ints(kernel[0], kernel[1], stride[0], stride[1], pt, pl, pb, pr, 1, 1, 1)
    torch.cuda.synchronize()
    _check(lib().ref_pool(_f16(x), _p(x), _p(prev_in), _p(out), _p(mask), _p(om), shape, geom, 0, 1), "pool")
    return out, om


def global_avg_pool(x, mask):
    """Average pool to 1x1 as the reference's Python wrapper sets it up (src/deltacnn/cuda_kernels.py:101-124):
    a pre-zeroed float32 output (the fp16 kernel accumulates into fp32 with atomics), a pre-zeroed out-mask, window =
    the whole image; the result is cast back to the input dtype."""
    n, c, h, w = x.shape
    out = torch.zeros((n, c, 1, 1), dtype=torch.float32, device=x.device).contiguous(memory_format=torch.channels_last)
    om = torch.zeros((n, 1, 1, 1), dtype=torch.int32, device=x.device)
    shape = _ints(n, h, w, c, 1, 1, c)
    geom = _ints(h, w, 1, 1, 0, 0, 0, 0, 1, 1, 1)
    torch.cuda.synchronize()
    _check(lib().ref_pool(_f16(x), _p(x), _p(None), _p(out), _p(mask), _p(om), shape, geom, 1, 1), "global_avg_pool")
    return out.to(x.dtype), om


def add_to_dense(a, b, mask_a):
    n, c, h, w = a.shape
    torch.cuda.synchronize()
    _check(lib().ref_add_to_dense(_f16(a), _p(a), _p(b), _p(mask_a), n, h, w, c, 0, 1), "add_to_dense")
    return b


def concatenate(a, ma, b, mb):
    n, ca, h, w = a.shape
    cb = b.shape[1]
    out = torch.zeros((n, ca + cb, h, w), dtype=a.dtype, device=a.device).contiguous(memory_format=torch.channels_last)
    mo = torch.zeros((n, 1, h, w), dtype=torch.int32, device=a.device)
    torch.cuda.synchronize()
    _check(lib().ref_concat(_f16(a), _p(a), _p(b), _p(out), _p(ma), _p(mb), _p(mo), n, h, w, ca, cb, 1), "concat")
    return out, mo


def mul_add(x, mask, scale, bias):
    n, c, h, w = x.shape
    out = torch.zeros_like(x)
    mo = torch.zeros((n, 1, h, w), dtype=torch.int32, device=x.device)
    torch.cuda.synchronize()
    _check(lib().ref_mul_add(_f16(x), _p(x), _p(mask), _p(out), _p(mo), _p(scale), _p(bias), n, h, w, c, 1), "mul_add")
    return out, mo


def upsample(x, mask, scale):
    n, c, h, w = x.shape
    out = torch.zeros((n, c, h * scale, w * scale), dtype=x.dtype, device=x.device).contiguous(memory_format=torch.channels_last)
    om = torch.zeros((n, 1, h * scale, w * scale), dtype=torch.int32, device=x.device)
    torch.cuda.synchronize()
    _check(lib().ref_upsample(_f16(x), _p(x), _p(out), _p(mask), _p(om), n, h, w, c, scale, 1), "upsample")
    return out, om
