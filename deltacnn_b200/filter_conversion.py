"""Weight re-layout for the delta convolution kernels.

The reference converts torch filters to [c_in, kh, kw, c_out] (src/deltacnn/filter_conversion.py:8-11)
and, for fp16, to a pair-swizzled variant (:13-38). This package uses [kh, kw, c_in/groups, c_out]
("HWIO") for the CUDA-core kernels in both precisions, plus a packed tensor-core image made on the
device by dc_pack_filter_umma for the layers that have a tcgen05 kernel.
"""
import torch


def convert_filter_out_channels_last(filter, transposed=False):
    """torch Conv2d weight [c_out, c_in/g, kh, kw] (or ConvTranspose2d weight [c_in, c_out, kh, kw]
    with ``transposed``) -> [kh, kw, c_in/g, c_out], contiguous copy."""
    if transposed:
        return filter.permute(2, 3, 0, 1).contiguous().clone()
    return filter.permute(2, 3, 1, 0).contiguous().clone()


def convert_half_filter(x, pixel_wise=False, transposed=False):
    """fp16 filters use the same HWIO layout (no pair swizzle, no channel padding)."""
    return convert_filter_out_channels_last(x.half(), transposed=transposed)
