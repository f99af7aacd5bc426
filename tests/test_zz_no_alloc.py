"""dc_conv2d_static: the convolution entry point for callers that may not allocate device memory
(a plugin inside another application's fixed memory allotment, a loop that must not touch the allocator
once it runs). It keeps its work-list scratch in a fixed array inside the library, so nothing is
allocated by the caller or by the call.

Every case here is one whose kernel really runs from the work list in that array (a KxK tensor-core
layer, a strided 1x1 layer and a wide depthwise layer with at least 40 000 output pixels), so the scan
pass writes the array and the convolution kernel reads it. Each case is called twice in a row with
different data and masks (the array keeps the first call's list) and checked through the C-ABI against
dc_conv2d on the same inputs, bit for bit at every pixel the operator defines, and against the CPU
oracle within the half-precision tolerance of the other operator tests. One case has exactly the
largest number of output pixels the array holds; one more pixel must be refused.

Collected last on purpose: a run that stops at the first failure has then run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

# name: (n, cin, cout, h, w, kernel, stride, padding, depthwise)
CASES = {
    "3x3_tensor_core_list": (2, 64, 64, 40, 40, 3, 1, 1, False),
    "1x1_stride2_list": (2, 32, 64, 290, 290, 1, 2, 0, False),
    "depthwise_wide_list": (1, 288, 288, 208, 200, 3, 1, 1, True),
    "largest_size_524288_pixels": (2, 16, 16, 1024, 1024, 1, 2, 0, False),
}


def _case(seed, density, n, cin, cout, h, w, ksz, stride, pad, depthwise):
    import deltacnn_b200.cuda_kernels as k
    from deltacnn_b200 import _lib
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    g = torch.Generator().manual_seed(seed)
    cl = lambda t: t.contiguous(memory_format=torch.channels_last)
    x = cl((torch.randn(n, cin, h, w, generator=g) * 0.3).half())
    mask = (torch.rand(n, 1, h, w, generator=g) < density).to(torch.int32)
    if depthwise:
        wt = (torch.randn(cin, 1, ksz, ksz, generator=g) * 0.4).half()
        groups = cin
    else:
        wt = (torch.randn(cout, cin, ksz, ksz, generator=g) * (cin * ksz * ksz) ** -0.5).half()
        groups = 1
    ho, wo = k.conv_out_hw(h, w, (ksz, ksz), (stride, stride), (pad, pad), (1, 1))
    f = convert_filter_out_channels_last(wt).cuda()
    desc = k.make_conv_desc(tuple(x.shape), cout, (ho, wo), (ksz, ksz), (stride, stride), (pad, pad), (1, 1), groups, 1)
    filt, layout = f, _lib.DC_FILTER_HWIO
    if not depthwise:
        pd = k.make_conv_desc((1, cin, 8, 8), cout, (8, 8), (ksz, ksz), (stride, stride), (pad, pad), (1, 1), 1, 1)
        packed = torch.zeros(_lib.lib.dc_filter_umma_bytes(pd, 0), dtype=torch.uint8, device="cuda")
        _lib.check(_lib.lib.dc_pack_filter_umma(pd, 0, f.data_ptr(), packed.data_ptr(), torch.cuda.current_stream().cuda_stream), "pack")
        filt, layout = packed, _lib.DC_FILTER_UMMA
    prev = cl(torch.randn(n, cout, ho, wo, generator=g).half())
    trunc = cl((torch.randn(n, cout, ho, wo, generator=g) * 0.02).half())
    return dict(k=k, lib=_lib, x=x, mask=mask, wt=wt, groups=groups, filt=filt, layout=layout, desc=desc, prev=prev, trunc=trunc,
                geom=(n, cout, ho, wo), conv=((stride, stride), (pad, pad)), keep=f)


THRESHOLD, ACTIVATION = 0.3, 2


def _run(entry, c):
    n, cout, ho, wo = c["geom"]
    p, t = c["prev"].cuda(), c["trunc"].cuda()
    x, mask = c["x"].cuda(), c["mask"].cuda()
    ep = c["k"].make_epilogue(p, t, THRESHOLD, ACTIVATION, 0)
    out = torch.full((n, cout, ho, wo), float("nan"), dtype=torch.float16, device="cuda").contiguous(memory_format=torch.channels_last)
    om = torch.full((n, 1, ho, wo), -5, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    rc = entry(c["desc"], x.data_ptr(), mask.data_ptr(), c["filt"].data_ptr(), c["layout"], None, out.data_ptr(), om.data_ptr(),
               ctypes.byref(ep), st)
    assert rc == 0, c["lib"].lib.dc_status_string(rc)
    torch.cuda.synchronize()
    return out, om, p, t


def _oracle(c):
    from oracle import delta_ops as O
    stride, pad = c["conv"]
    o, om = O.conv(c["x"], c["mask"], c["wt"], None, stride, pad, (1, 1), c["groups"])
    p, t = c["prev"].clone(), c["trunc"].clone()
    O.activate_truncate(o, p, t, om, THRESHOLD, ACTIVATION, 0)
    return o, om, p, t


@pytest.mark.parametrize("name", list(CASES))
def test_static_scratch_entry_point_runs_from_its_work_list_twice(name):
    geom = CASES[name]
    assert geom[0] * ((geom[3] + 2 * geom[7] - geom[5]) // geom[6] + 1) * ((geom[4] + 2 * geom[7] - geom[5]) // geom[6] + 1) <= 524288
    for call, (seed, density) in enumerate(((7, 0.2), (8, 0.05))):     # the second call finds the first call's list in the array
        c = _case(seed, density, *geom)
        o1, m1, p1, t1 = _run(c["lib"].lib.dc_conv2d, c)
        o2, m2, p2, t2 = _run(c["lib"].lib.dc_conv2d_static, c)
        assert torch.equal(m1, m2), f"call {call}: out-mask differs from dc_conv2d"
        assert torch.equal(p1, p2) and torch.equal(t1, t2), f"call {call}: caches differ from dc_conv2d"
        sel = (m1 != 0).expand_as(o1)
        assert torch.equal(o1[sel], o2[sel]), f"call {call}: values differ from dc_conv2d"
        assert 0 < int(m1.sum()) < m1.numel()
        # against the CPU oracle: fp32 accumulation order differs, so a few pixels next to the threshold may flip
        o_ref, m_ref, p_ref, t_ref = _oracle(c)
        agree = (m2.cpu() == m_ref).float().mean().item()
        assert agree > 0.99, f"call {call}: mask agreement with the oracle {agree}"
        both = ((m2.cpu() != 0) & (m_ref != 0)).expand_as(o_ref)
        err = (o2.cpu().float()[both] - o_ref.float()[both]).abs().max().item()
        assert err < 2e-2, f"call {call}: values differ from the oracle by {err}"
        same = (m2.cpu() == m_ref).expand_as(p_ref)
        assert (p2.cpu().float()[same] - p_ref.float()[same]).abs().max().item() < 2e-2, f"call {call}: cache differs from the oracle"
    assert c["lib"].lib.dc_umma_error() == 0


def test_static_scratch_entry_point_refuses_oversized_calls():
    import deltacnn_b200.cuda_kernels as k
    from deltacnn_b200 import _lib
    limit = _lib.lib.dc_static_workspace_max_pixels()
    assert limit == 524288
    dummy = torch.zeros(16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    # one pixel more than the array holds, and a much larger call: rejected before any pointer is touched
    for n, h, w in ((1, 524289, 1), (3, 512, 512)):
        desc = k.make_conv_desc((n, 16, h, w), 16, (h, w), (1, 1), (1, 1), (0, 0), (1, 1), 1, 1)
        rc = _lib.lib.dc_conv2d_static(desc, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 0, None, dummy.data_ptr(),
                                       dummy.data_ptr(), None, st)
        assert rc == 7 and b"workspace" in _lib.lib.dc_status_string(rc)
