"""CPU restatement of the reference DeltaCNN operator semantics (TEST INFRASTRUCTURE).

This file is the parity checker for the CUDA kernels of ``deltacnn_b200``. It is
never imported by the product; only tests, the smoke check and the CPU-baseline leg
of the benchmark use it.

Parity status: the reference project ships no tests, golden vectors or fixtures for
this path, and its delta kernels are CUDA-only, so nothing in the reference pins
these functions on a CPU. They are pinned instead against (1) fixtures recorded from
the reference's own kernels (``tests/golden/ref_*.npz``, produced by
``tests/golden/make_golden.py`` on a GPU through ``oracle/_ref``) and (2) the
mathematical identity that at threshold 0 the delta network equals the dense one.

Conventions: tensors are torch CPU tensors, logical NCHW; ``mask`` is int32
(N,1,H,W) with values 0/1. Arithmetic is carried out in float32 and rounded to the
tensor dtype on every store ("fp16 emulation" when the tensors are float16). State
tensors (``prev_in``, ``prev_out``, ``truncated``) are updated in place, as in the
reference operator API (src/deltacnn/cuda_kernels.py:132-150).

Each function cites the reference lines it follows.
"""
import torch
import torch.nn.functional as F

ACT_NONE, ACT_RELU, ACT_RELU6, ACT_LEAKY, ACT_SIGMOID, ACT_SWISH = 0, 1, 2, 3, 4, 5
TRUNC_NONE, TRUNC_MAX, TRUNC_NORM, TRUNC_RMS = -1, 0, 1, 2


def activation_fn(x, code):
    """Activation codes of src/cuda/other_nn_layers.cu:106-121 (leaky slope 0.1, :33)."""
    if code <= 0:
        return x
    if code == ACT_RELU:
        return torch.clamp_min(x, 0.0)
    if code == ACT_RELU6:
        return torch.clamp(x, 0.0, 6.0)
    if code == ACT_LEAKY:
        return torch.where(x < 0, x * 0.1, x)
    if code == ACT_SIGMOID:
        return 1.0 / (1.0 + torch.exp(-x))
    if code == ACT_SWISH:
        return x / (1.0 + torch.exp(-x))
    raise ValueError(f"activation code {code}")


def _round_threshold(threshold, dtype):
    """Half kernels compare against __float2half(threshold) (other_nn_layers.cu:1343)."""
    if dtype == torch.float16:
        return float(torch.tensor(threshold, dtype=torch.float32).to(torch.float16).float())
    return float(threshold)


def sparsify(x, prev_in, delta, mask, threshold):
    """Input delta and update mask. src/cuda/other_nn_layers.cu:821-881 (fp32), :1261-1376 (fp16).

    d = x - prev_in; a pixel is active when any channel has |d| > threshold (strict).
    Active pixels write d to ``delta`` and x to ``prev_in``; inactive pixels leave
    ``prev_in`` (and ``delta``) untouched, so sub-threshold drift keeps accumulating.
    """
    d = (x.float() - prev_in.float()).to(x.dtype)          # one rounding, as __hsub
    thr = _round_threshold(threshold, x.dtype)
    active = (d.float().abs() > thr).any(dim=1, keepdim=True)
    mask.copy_(active.to(torch.int32))
    sel = active.expand_as(x)
    delta[sel] = d[sel]
    prev_in[sel] = x[sel]
    return delta, mask


def _pad4(padding):
    """Python-level padding: 2-tuple (h, w) or 4-tuple (top, bottom, left, right)
    (src/deltacnn/cuda_kernels.py:21-26). Returns (top, bottom, left, right)."""
    if len(padding) == 2:
        return padding[0], padding[0], padding[1], padding[1]
    return padding[0], padding[1], padding[2], padding[3]


def conv_out_size(h, w, kernel, stride, padding, dilation):
    """src/deltacnn/cuda_kernels.py:20-26."""
    pt, pb, pl, pr = _pad4(padding)
    ho = (h + pt + pb - dilation[0] * (kernel[0] - 1) - 1) // stride[0] + 1
    wo = (w + pl + pr - dilation[1] * (kernel[1] - 1) - 1) // stride[1] + 1
    return ho, wo


def dilate_mask(mask, kernel, stride, padding, dilation):
    """Out-mask of a convolution / pooling: OR of the in-mask over each output pixel's
    in-bounds taps. src/cuda/conv_kernel.cu:156-219 (write_mask), :46-61 (load_mask)."""
    pt, pb, pl, pr = _pad4(padding)
    m = F.pad(mask.float(), (pl, pr, pt, pb), value=0.0)
    out = F.max_pool2d(m, kernel_size=tuple(kernel), stride=tuple(stride), padding=0, dilation=tuple(dilation))
    return (out > 0).to(torch.int32)


def conv(x, mask, weight, bias, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1):
    """Masked delta convolution. src/cuda/conv_kernel.cu:505-630 (dense-tile branch),
    mask handling :46-219; host semantics src/deltacnn/sparse_layers.py:603-640.

    ``weight`` is in torch layout [Cout, Cin/groups, kh, kw]. Returns (out, out_mask);
    ``out`` holds conv(x*mask) (+bias) at every pixel -- the reference defines it only
    where out_mask == 1 or inside tiles that saw an active input, so comparisons use
    out_mask == 1 pixels only.
    """
    pt, pb, pl, pr = _pad4(padding)
    xm = x.float() * (mask != 0).float()
    xm = F.pad(xm, (pl, pr, pt, pb))
    out = F.conv2d(xm, weight.float(), None if bias is None else bias.float(),
                   stride=tuple(stride), padding=0, dilation=tuple(dilation), groups=groups)
    kernel = weight.shape[2:]
    out_mask = dilate_mask(mask, kernel, stride, padding, dilation)
    return out.to(x.dtype).contiguous(memory_format=torch.channels_last), out_mask


def deconv_out_size(h, w, kernel, stride, padding, dilation):
    """src/deltacnn/cuda_kernels.py:55-57 (output_padding is ignored by the reference)."""
    ho = (h - 1) * stride[0] - 2 * padding[0] + dilation[0] * (kernel[0] - 1) + 1
    wo = (w - 1) * stride[1] - 2 * padding[1] + dilation[1] * (kernel[1] - 1) + 1
    return ho, wo


def deconv(x, mask, weight, bias, stride=(2, 2), padding=(1, 1)):
    """Masked transposed convolution, groups 1, dilation 1. src/cuda/deconv_kernel.cu:447-499
    (scatter with un-flipped taps), out-mask :280-346. ``weight`` in torch layout
    [Cin, Cout, kh, kw]."""
    xm = x.float() * (mask != 0).float()
    out = F.conv_transpose2d(xm, weight.float(), None if bias is None else bias.float(),
                             stride=tuple(stride), padding=tuple(padding))
    ones = torch.ones(1, 1, weight.shape[2], weight.shape[3])
    om = F.conv_transpose2d((mask != 0).float(), ones, None, stride=tuple(stride), padding=tuple(padding))
    return out.to(x.dtype).contiguous(memory_format=torch.channels_last), (om > 0).to(torch.int32)


def activate_truncate(delta, prev_out, truncated, mask, threshold, activation, truncation_mode):
    """Accumulate + activation delta + truncation, in place on delta, mask and the
    two state tensors. src/cuda/other_nn_layers.cu:397-463 (max), :664-719 (norm/rms),
    :378-394 (no truncation); host src/deltacnn/sparse_layers.py:1403-1417.

    Identity activation emits e = delta + truncated (the reference leaves the incoming
    delta in some branches; that quirk is not reproduced).
    """
    dt = delta.dtype
    m = mask != 0
    d32, y32 = delta.float(), prev_out.float()
    if truncation_mode < 0:
        u = (y32 + d32).to(dt)
        e = (activation_fn(u.float(), activation) - activation_fn(y32, activation)).to(dt) if activation > 0 else delta
        sel = m.expand_as(delta)
        prev_out[sel] = u[sel]
        if activation > 0:
            delta[sel] = e[sel]
        return delta, mask
    r = (truncated.float() + d32).to(dt)
    u = (y32 + r.float()).to(dt)
    e = (activation_fn(u.float(), activation) - activation_fn(y32, activation)).to(dt)
    thr = _round_threshold(threshold, dt)
    ef = e.float()
    if truncation_mode == TRUNC_MAX:
        active = (ef.abs() > thr).any(dim=1, keepdim=True)
    elif truncation_mode == TRUNC_NORM:
        active = torch.sqrt((ef * ef).sum(dim=1, keepdim=True)) > thr
    else:
        active = torch.sqrt((ef * ef).sum(dim=1, keepdim=True) / delta.shape[1]) > thr
    keep = (m & active).expand_as(delta)
    drop = (m & ~active).expand_as(delta)
    prev_out[keep] = u[keep]
    truncated[keep] = 0
    delta[keep] = e[keep]
    truncated[drop] = r[drop]
    mask[m & ~active] = 0
    return delta, mask


def add(a, mask_a, b, mask_b, prev_out, weight_a=1.0, weight_b=1.0, activation=0, dense_out=False):
    """Weighted add of two delta tensors. src/cuda/other_nn_layers.cu:1380-1559;
    host src/deltacnn/sparse_layers.py:1101-1174. Returns (out, mask_out); with
    ``dense_out`` the output is f(prev_out) at every pixel and mask_out is None."""
    dt = a.dtype
    ma, mb = (mask_a != 0), (mask_b != 0)
    mo = ma | mb
    s = (a.float() * ma.float() * weight_a + b.float() * mb.float() * weight_b)
    if not dense_out and activation <= 0:
        return s.to(dt), mo.to(torch.int32)
    y_old = prev_out.float()
    y_new = (y_old + s).to(dt)
    sel = mo.expand_as(a)
    if dense_out:
        prev_out[sel] = y_new[sel]
        return activation_fn(prev_out.float(), activation).to(dt), None
    e = (activation_fn(y_new.float(), activation) - activation_fn(y_old, activation)).to(dt)
    prev_out[sel] = y_new[sel]
    return e, mo.to(torch.int32)


def add_to_dense(a, b, mask_a, activation=0):
    """b += a on masked pixels. src/cuda/other_nn_layers.cu:1732-1847."""
    sel = (mask_a != 0).expand_as(a)
    s = (b.float() + a.float()).to(b.dtype)
    b[sel] = s[sel]
    return b


def max_pool(x, mask, prev_in, kernel, stride, padding, dilation=(1, 1)):
    """Delta max-pool: out = max(prev + x*mask) - max(prev) over in-bounds window
    elements, fp32 math; out-mask = OR over the window. Does NOT update prev_in (the
    module does that with add_to_dense afterwards, sparse_layers.py:1466-1468).
    src/cuda/other_nn_layers.cu:2390-2459.

    Padding is a 2-tuple or (top, bottom, left, right). Out-of-bounds window elements are
    ignored, with the reference's one exception (:2402-2422, "same behaviour as when first
    applying padding and then pooling"): a literal 0 joins the window for rows inside the
    bottom padding when top != bottom padding, and for columns inside the right padding
    (of rows inside the image) when left != right padding."""
    pt, pb, pl, pr = _pad4(padding)
    xm = x.float() * (mask != 0).float()
    p = prev_in.float()
    neg = -1e30
    h, w = x.shape[2], x.shape[3]

    def padded(t):
        t = F.pad(t, (pl, pr, pt, pb), value=neg)
        if pl != pr and pr > 0:
            t[:, :, pt:pt + h, pl + w:] = 0.0
        if pt != pb and pb > 0:
            t[:, :, pt + h:, :] = 0.0
        return t

    o = F.max_pool2d(padded(p + xm), tuple(kernel), tuple(stride), 0, tuple(dilation)) - \
        F.max_pool2d(padded(p), tuple(kernel), tuple(stride), 0, tuple(dilation))
    om = dilate_mask(mask, kernel, stride, padding, dilation)
    return o.to(x.dtype).contiguous(memory_format=torch.channels_last), om


def global_avg_pool(x, mask):
    """Delta global average pool to 1x1: mean over H*W of masked deltas, fp32
    accumulate, cast to the input dtype; mask_out = any(mask) per image.
    src/cuda/other_nn_layers.cu:3139-3288, 2915-3135; cuda_kernels.py:101-124."""
    n, c, h, w = x.shape
    xm = x.float() * (mask != 0).float()
    o = xm.sum(dim=(2, 3), keepdim=True) / float(h * w)
    om = (mask != 0).flatten(1).any(dim=1).to(torch.int32).view(n, 1, 1, 1)
    return o.to(x.dtype), om


def upsample(x, mask, scale):
    """Nearest-neighbour x``scale`` of values and mask. other_nn_layers.cu:3483-3522."""
    o = x.repeat_interleave(scale, dim=2).repeat_interleave(scale, dim=3)
    om = mask.repeat_interleave(scale, dim=2).repeat_interleave(scale, dim=3)
    return o.contiguous(memory_format=torch.channels_last), om.contiguous()


def concatenate(a, mask_a, b, mask_b):
    """Channel concat, mask union, inactive side zero-filled. other_nn_layers.cu:3625-3671."""
    ma, mb = (mask_a != 0), (mask_b != 0)
    o = torch.cat((a * ma.to(a.dtype), b * mb.to(b.dtype)), dim=1)
    return o.contiguous(memory_format=torch.channels_last), (ma | mb).to(torch.int32)


def scale_bias(x, mask, scale, bias):
    """x*scale (+bias) on masked pixels (un-folded BatchNorm). other_nn_layers.cu:3774-3818;
    sparse_layers.py:1532-1581. ``scale``/``bias`` are per-channel 1-D tensors."""
    o = x.float() * scale.float().view(1, -1, 1, 1)
    if bias is not None:
        o = o + bias.float().view(1, -1, 1, 1)
    return o.to(x.dtype), mask.clone()


def densify(delta, mask, prev_out, activation=0):
    """prev_out += delta on masked pixels; returns f(prev_out) as a new dense tensor.
    src/deltacnn/sparse_layers.py:1287-1329 (kernel: no-truncation branch of
    other_nn_layers.cu:378-394)."""
    sel = (mask != 0).expand_as(delta)
    s = (prev_out.float() + delta.float()).to(prev_out.dtype)
    prev_out[sel] = s[sel]
    return activation_fn(prev_out.float(), activation).to(prev_out.dtype)


def sparsify_dilated(x, prev_in, threshold, dilation):
    """DCSparsify(dilation=k): src/deltacnn/sparse_layers.py:1233-1248. Returns (delta, mask); the delta is dense
    (x - prev_in everywhere), the mask is the k x k max-pool (stride 1, padding (k-1)//2) of max_c |delta| compared
    with the threshold, and prev_in takes x where the mask is set."""
    d = (x.float() - prev_in.float()).to(x.dtype)
    thr = _round_threshold(threshold, x.dtype)
    a = d.float().abs().amax(dim=1, keepdim=True)
    k = int(dilation)
    m = F.max_pool2d(a, (k, k), stride=(1, 1), padding=((k - 1) // 2, (k - 1) // 2)) > thr
    sel = m.expand_as(x)
    prev_in[sel] = x[sel]
    return d, m.to(torch.int32)


def linear_delta(delta, mask, weight, bias, acc, first_frame):
    """Classifier on the pooled delta. The reference's tail is DCDensify (prev_out += delta, sparse_layers.py:1322-1329)
    followed by nn.Linear on the dense vector (example/mobilenet_deltacnn.py:216-227); a linear layer commutes with
    that accumulation, so acc (float32, N x out) += delta @ W^T on masked streams (+ bias on the first frame) holds the
    same logits. Returns acc rounded to the feature dtype."""
    n = delta.shape[0]
    d = delta.reshape(n, -1).float()
    on = torch.ones(n, dtype=torch.bool) if (first_frame or mask is None) else (mask.reshape(n) != 0)
    upd = d @ weight.float().t()
    if first_frame:
        acc.zero_()
        if bias is not None:
            upd = upd + bias.float()
    acc[on] += upd[on]
    return acc.to(delta.dtype)


def heatmap_argmax(heat):
    """(x, y, value) of the first maximum of every map of a dense (N, J, H, W) tensor (torch.argmax semantics)."""
    n, j, h, w = heat.shape
    flat = heat.float().reshape(n, j, h * w)
    val, idx = flat.max(dim=2)
    idx = torch.argmax(flat, dim=2)
    return torch.stack(((idx % w).float(), (idx // w).float(), val), dim=2)


def centernet_decode(heat, wh, offset, topk=100, min_score=0.0, stride=4.0, apply_sigmoid=False):
    """CenterNet-style decode of dense head outputs (N,C,H,W / N,2,H,W): peaks = elements equal to the 3x3 max-pool
    of the heat map, the topk best above min_score (ties by ascending (pixel, class) index), boxes from centre
    (x + off_x, y + off_y) and size wh, times stride. Returns (det (N, topk, 6), count (N,))."""
    n, c, h, w = heat.shape
    hf = heat.float()
    peak = F.max_pool2d(hf, 3, 1, 1) == hf
    score = torch.where(peak & (hf > min_score), hf, torch.full_like(hf, float("-inf")))
    det = torch.zeros(n, topk, 6)
    det[:, :, 5] = -1
    count = torch.zeros(n, dtype=torch.int32)
    for b in range(n):
        s = score[b].permute(1, 2, 0).reshape(-1)                      # index = pixel * classes + class
        order = torch.sort(s, descending=True, stable=True)[1]
        order = order[torch.isfinite(s[order])][:topk]
        count[b] = len(order)
        for k, i in enumerate(order.tolist()):
            cl, p = i % c, i // c
            y, x = p // w, p % w
            cx, cy = x + float(offset[b, 0, y, x]), y + float(offset[b, 1, y, x])
            bw, bh = float(wh[b, 0, y, x]), float(wh[b, 1, y, x])
            sc = float(s[i])
            if apply_sigmoid:
                sc = 1.0 / (1.0 + float(torch.exp(torch.tensor(-sc))))
            det[b, k] = torch.tensor([(cx - bw / 2) * stride, (cy - bh / 2) * stride, (cx + bw / 2) * stride, (cy + bh / 2) * stride, sc, cl])
    return det, count
