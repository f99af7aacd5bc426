"""ctypes binding of libdeltacnn_b200.so (the C-ABI declared in include/deltacnn_b200.h).

There is no fallback: if the shared library is missing or fails to load, importing this
module raises, and every operator of the package is unusable.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdeltacnn_b200.so")

DC_F32, DC_F16 = 0, 1
DC_FILTER_HWIO, DC_FILTER_UMMA = 0, 1

c_int, c_i64, c_float, c_void_p, c_size_t = ctypes.c_int32, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t


class ConvDesc(ctypes.Structure):
    """dc_conv_desc."""
    _fields_ = [(n, c_int) for n in (
        "n", "h_in", "w_in", "c_in", "h_out", "w_out", "c_out", "kh", "kw", "stride_h", "stride_w",
        "pad_top", "pad_left", "pad_bottom", "pad_right", "dil_h", "dil_w", "groups", "dtype")]


class IrbDesc(ctypes.Structure):
    """dc_irb_desc."""
    _fields_ = [(n, c_int) for n in ("n", "h", "w", "c_in", "c_hidden", "c_out", "stride", "residual", "act_expand", "act_dw", "dtype")] + \
               [("thr_expand", c_float), ("thr_dw", c_float)]


class Epilogue(ctypes.Structure):
    """dc_epilogue."""
    _fields_ = [("prev_out", c_void_p), ("truncated", c_void_p), ("threshold", c_float),
                ("activation", c_int), ("truncation", c_int),
                ("residual", c_void_p), ("residual_mask", c_void_p)]


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} not found: the CUDA extension is not built. Run `python deltacnn_b200/build.py` "
        "(needs nvcc with sm_100a support). deltacnn_b200 has no CPU or PyTorch fallback.")

lib = ctypes.CDLL(LIB_PATH)

_P = c_void_p
_SIGNATURES = {
    "dc_version": (c_int, []),
    "dc_status_string": (ctypes.c_char_p, [c_int]),
    "dc_last_cuda_error": (c_int, []),
    "dc_umma_error": (c_int, []),
    "dc_sparsify": (c_int, [_P, _P, _P, _P, c_i64, c_int, c_int, c_float, _P]),
    "dc_sparsify_u8": (c_int, [_P, _P, _P, _P, _P, _P, c_i64, c_int, c_int, c_float, _P]),
    "dc_conv2d": (c_int, [ctypes.POINTER(ConvDesc), _P, _P, _P, c_int, _P, _P, _P, ctypes.POINTER(Epilogue), _P]),
    "dc_conv2d_ws": (c_int, [ctypes.POINTER(ConvDesc), _P, _P, _P, c_int, _P, _P, _P, ctypes.POINTER(Epilogue), _P, c_size_t, _P]),
    "dc_conv_workspace_bytes": (c_size_t, [ctypes.POINTER(ConvDesc)]),
    "dc_conv2d_static": (c_int, [ctypes.POINTER(ConvDesc), _P, _P, _P, c_int, _P, _P, _P, ctypes.POINTER(Epilogue), _P]),
    "dc_static_workspace_max_pixels": (c_size_t, []),
    "dc_deconv2d": (c_int, [ctypes.POINTER(ConvDesc), _P, _P, _P, c_int, _P, _P, _P, ctypes.POINTER(Epilogue), _P]),
    "dc_deconv2d_ws": (c_int, [ctypes.POINTER(ConvDesc), _P, _P, _P, c_int, _P, _P, _P, ctypes.POINTER(Epilogue), _P, c_size_t, _P]),
    "dc_deconv_workspace_bytes": (c_size_t, [ctypes.POINTER(ConvDesc)]),
    "dc_filter_umma_bytes": (c_size_t, [ctypes.POINTER(ConvDesc), c_int]),
    "dc_pack_filter_umma": (c_int, [ctypes.POINTER(ConvDesc), c_int, _P, _P, _P]),
    "dc_activate_truncate": (c_int, [_P, _P, _P, _P, c_i64, c_int, c_int, c_float, c_int, c_int, _P]),
    "dc_add": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_float, c_float, c_i64, c_int, c_int, c_int, c_int, _P]),
    "dc_add_to_dense": (c_int, [_P, _P, _P, c_i64, c_int, c_int, _P]),
    "dc_scale_bias": (c_int, [_P, _P, _P, _P, _P, _P, c_i64, c_int, c_int, _P]),
    "dc_pool": (c_int, [ctypes.POINTER(ConvDesc), _P, _P, _P, _P, _P, c_int, c_int, _P]),
    "dc_upsample": (c_int, [_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P]),
    "dc_concat": (c_int, [_P, _P, _P, _P, _P, _P, c_i64, c_int, c_int, c_int, _P]),
    "dc_densify": (c_int, [_P, _P, _P, _P, c_i64, c_int, c_int, c_int, _P]),
    "dc_compact_mask": (c_int, [_P, c_i64, _P, _P, _P]),
    "dc_conv3x3_heads_supported": (c_int, [ctypes.POINTER(ConvDesc), c_int]),
    "dc_conv3x3_heads": (c_int, [ctypes.POINTER(ConvDesc), _P, _P, _P, _P, c_int, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p),
                                 ctypes.POINTER(Epilogue), _P]),
    "dc_irb_supported": (c_int, [ctypes.POINTER(IrbDesc)]),
    "dc_irb_fused": (c_int, [ctypes.POINTER(IrbDesc), _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "dc_sparsify_dilated": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_float, c_int, _P]),
    "dc_linear_delta": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "dc_heatmap_argmax": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "dc_centernet_decode": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, _P]),
}
EXPORTED_SYMBOLS = tuple(_SIGNATURES)

for _name, (_res, _args) in _SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError here = header and library disagree
    _fn.restype = _res
    _fn.argtypes = _args


def check(status, what):
    """Raise RuntimeError for a non-zero dc_status."""
    if status != 0:
        msg = lib.dc_status_string(status).decode()
        extra = f" (cudaError {lib.dc_last_cuda_error()})" if status == 6 else ""
        raise RuntimeError(f"deltacnn_b200.{what}: {msg}{extra}")
