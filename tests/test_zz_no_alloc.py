"""dc_conv2d_static: the convolution entry point for callers that may not allocate device memory
(a plugin inside another application's fixed memory allotment, a loop that must not touch the allocator
once it runs). It keeps its work-list scratch in a fixed array inside the library, so nothing is
allocated by the caller or by the call. Checked through the C-ABI against dc_conv2d on the same
inputs, twice in a row (the scratch array keeps the first call's contents), bit for bit at every
pixel the operator defines; sizes beyond the built-in scratch must be refused.

Collected last on purpose: a run that stops at the first failure has then run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, n, cin, cout, h, w, depthwise):
    import deltacnn_b200.cuda_kernels as k
    from deltacnn_b200 import _lib
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    g = torch.Generator().manual_seed(seed)
    cl = lambda t: t.contiguous(memory_format=torch.channels_last)
    x = cl((torch.randn(n, cin, h, w, generator=g) * 0.3).half()).cuda()
    mask = (torch.rand(n, 1, h, w, generator=g) < 0.2).to(torch.int32).cuda()
    if depthwise:
        wt = (torch.randn(cin, 1, 3, 3, generator=g) * 0.4).half()
        ksz, pad, groups = 3, 1, cin
    else:
        wt = (torch.randn(cout, cin, 1, 1, generator=g) * cin ** -0.5).half()
        ksz, pad, groups = 1, 0, 1
    f = convert_filter_out_channels_last(wt).cuda()
    desc = k.make_conv_desc(tuple(x.shape), cout, (h, w), (ksz, ksz), (1, 1), (pad, pad), (1, 1), groups, 1)
    filt, layout = f, _lib.DC_FILTER_HWIO
    if not depthwise:
        pd = k.make_conv_desc((1, cin, 8, 8), cout, (8, 8), (1, 1), (1, 1), (0, 0), (1, 1), 1, 1)
        packed = torch.zeros(_lib.lib.dc_filter_umma_bytes(pd, 0), dtype=torch.uint8, device="cuda")
        _lib.check(_lib.lib.dc_pack_filter_umma(pd, 0, f.data_ptr(), packed.data_ptr(), torch.cuda.current_stream().cuda_stream), "pack")
        filt, layout = packed, _lib.DC_FILTER_UMMA
    prev = cl(torch.randn(n, cout, h, w, generator=g).half())
    trunc = cl((torch.randn(n, cout, h, w, generator=g) * 0.02).half())
    return k, _lib, x, mask, filt, layout, desc, prev, trunc


def _run(entry, k, _lib, x, mask, filt, layout, desc, prev, trunc, cout, h, w):
    n = x.shape[0]
    p, t = prev.cuda(), trunc.cuda()
    ep = k.make_epilogue(p, t, 0.7, 2, 0)
    out = torch.full((n, cout, h, w), float("nan"), dtype=torch.float16, device="cuda").contiguous(memory_format=torch.channels_last)
    om = torch.full((n, 1, h, w), -5, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    rc = entry(desc, x.data_ptr(), mask.data_ptr(), filt.data_ptr(), layout, None, out.data_ptr(), om.data_ptr(), ctypes.byref(ep), st)
    assert rc == 0, _lib.lib.dc_status_string(rc)
    torch.cuda.synchronize()
    return out, om, p, t


@pytest.mark.parametrize("depthwise", [False, True])
def test_static_scratch_entry_point_matches_dc_conv2d_twice(depthwise):
    cin = cout = 96 if depthwise else 0
    if not depthwise:
        cin, cout = 32, 192
    n, h, w = 3, 28, 28
    for call, seed in enumerate((7, 8)):            # second call reuses the scratch array with other data
        k, _lib, x, mask, filt, layout, desc, prev, trunc = _case(seed, n, cin, cout, h, w, depthwise)
        ref = _run(_lib.lib.dc_conv2d, k, _lib, x, mask, filt, layout, desc, prev, trunc, cout, h, w)
        got = _run(_lib.lib.dc_conv2d_static, k, _lib, x, mask, filt, layout, desc, prev, trunc, cout, h, w)
        o1, m1, p1, t1 = ref
        o2, m2, p2, t2 = got
        assert torch.equal(m1, m2), f"call {call}: out-mask differs"
        assert torch.equal(p1, p2) and torch.equal(t1, t2), f"call {call}: caches differ"
        sel = (m1 != 0).expand_as(o1)
        assert torch.equal(o1[sel], o2[sel]), f"call {call}: values differ"
        assert 0 < int(m1.sum()) < m1.numel()
    assert _lib.lib.dc_umma_error() == 0


def test_static_scratch_entry_point_refuses_oversized_calls():
    import deltacnn_b200.cuda_kernels as k
    from deltacnn_b200 import _lib
    limit = _lib.lib.dc_static_workspace_max_pixels()
    assert limit == 524288
    n, h, w = 3, 512, 512                       # 786432 output pixels > limit; rejected before any pointer is touched
    desc = k.make_conv_desc((n, 16, h, w), 16, (h, w), (1, 1), (1, 1), (0, 0), (1, 1), 1, 1)
    dummy = torch.zeros(16, device="cuda")
    rc = _lib.lib.dc_conv2d_static(desc, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 0, None, dummy.data_ptr(),
                                   dummy.data_ptr(), None, torch.cuda.current_stream().cuda_stream)
    assert rc == 7 and b"workspace" in _lib.lib.dc_status_string(rc)
