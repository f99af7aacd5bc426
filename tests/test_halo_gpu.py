"""Stride-1 3x3 convolutions on halo tiles (dc_conv_halo.cu: one tiled TMA load of a patch's halo per channel block,
nine shifted views of it for the nine taps, two accumulators in tensor memory, warp-specialised roles) against the
CPU oracle: out-masks exact, values within the half-precision tolerance, nothing written outside the out-mask,
inactive inputs (NaN here) never used; the fused truncation epilogue against convolution + stand-alone truncation."""
import pytest
import torch

from oracle import delta_ops as O

pytestmark = pytest.mark.gpu


def cl(t):
    return t.contiguous(memory_format=torch.channels_last)


def _packed(kk, f, cin, cout, pad):
    from deltacnn_b200 import _lib
    desc = kk.make_conv_desc((1, cin, 8, 8), cout, (8 + 2 * pad - 2, 8 + 2 * pad - 2), (3, 3), (1, 1), (pad, pad), (1, 1), 1, 1)
    packed = torch.zeros(_lib.lib.dc_filter_umma_bytes(desc, 0), dtype=torch.uint8, device="cuda")
    _lib.check(_lib.lib.dc_pack_filter_umma(desc, 0, f.data_ptr(), packed.data_ptr(), torch.cuda.current_stream().cuda_stream), "pack")
    return packed


def _masks(g, n, h, w, kind):
    if kind == "full":
        return torch.ones(n, 1, h, w, dtype=torch.int32)
    if kind == "half":
        return (torch.rand(n, 1, h, w, generator=g) < 0.5).to(torch.int32)
    if kind == "sparse":
        return (torch.rand(n, 1, h, w, generator=g) < 0.02).to(torch.int32)
    m = torch.zeros(n, 1, h, w, dtype=torch.int32)
    if kind == "corners":                        # single pixels at the image border and at patch borders (patches are 16 x 8)
        for (y, x) in ((0, 0), (h - 1, w - 1), (0, w - 1), (min(15, h - 1), min(7, w - 1)), (min(16, h - 1), min(8, w - 1))):
            m[:, 0, y, x] = 1
        m[n - 1] = 0                             # and an image without any update
    return m


# cin, cout, n, h, w, pad
CASES = [
    (32, 32, 2, 64, 64, 1),        # filter resident, one channel block half filled
    (64, 64, 3, 33, 21, 1),        # odd sizes: patches overhang the image
    (64, 32, 2, 16, 8, 1),         # exactly one patch per image
    (128, 128, 2, 20, 24, 1),      # two channel blocks, filter streamed through the ring
    (256, 128, 1, 17, 30, 1),      # four channel blocks, streamed
    (48, 80, 2, 24, 40, 1),        # channel counts that are no multiple of 64 / 16
    (64, 64, 2, 26, 19, 0),        # no padding: the output is smaller than the input
    (32, 32, 24, 96, 80, 1),       # ~10 tiles per CTA: the rings of tile records, stages and accumulators wrap around
    (256, 64, 2, 33, 40, 1),       # narrow N with a filter too large to stay: the patch-tile kernel takes these
    (128, 32, 3, 48, 24, 1),
    (128, 64, 16, 64, 64, 1),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(str(v) for v in c))
@pytest.mark.parametrize("kind", ["full", "half", "sparse", "corners"])
@pytest.mark.parametrize("fused", [False, True])
def test_halo_tiles_match_oracle(case, kind, fused):
    import deltacnn_b200.cuda_kernels as kk
    from deltacnn_b200 import _lib
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    cin, cout, n, h, w, pad = case
    g = torch.Generator().manual_seed(97)
    x = cl((torch.randn(n, cin, h, w, generator=g) * 0.5).half())
    mask = _masks(g, n, h, w, kind)
    wt = (torch.randn(cout, cin, 3, 3, generator=g) / (3 * cin ** 0.5)).half()
    bias = torch.randn(cout, generator=g).half()
    ref, m_ref = O.conv(x, mask, wt, bias, (1, 1), (pad, pad), (1, 1), 1)
    f = convert_filter_out_channels_last(wt).cuda()
    packed = _packed(kk, f, cin, cout, pad)
    xd, md = x.cuda(), mask.cuda()
    xd[(mask == 0).expand_as(x)] = float("nan")              # the delta tensor is undefined at inactive pixels
    if not fused:
        out = cl(torch.full(ref.shape, float("nan"), dtype=torch.float16)).cuda()
        out, om = kk.sparse_conv(xd, f, md, bias.cuda(), (1, 1), (pad, pad), (1, 1), 1, create_out_mask=True, out=out, filter_umma=packed)
        torch.cuda.synchronize()
        assert _lib.lib.dc_umma_error() == 0
        assert torch.equal(om.cpu(), m_ref)
        sel = (m_ref != 0).expand_as(ref)
        if sel.any():
            scale = max(ref.float()[sel].abs().max().item(), 1e-6)
            assert (out.cpu().float()[sel] - ref.float()[sel]).abs().max().item() / scale <= 1e-2
        assert torch.isnan(out.cpu()[~sel]).all(), "pixels outside the out-mask must not be written"
        return
    ho, wo = ref.shape[2:]
    prev = cl(torch.randn(n, cout, ho, wo, generator=g).half())
    trunc = cl((torch.randn(n, cout, ho, wo, generator=g) * 0.02).half())
    for act in (1, 3):                                        # ReLU (packed-half form) and leaky ReLU (fp32 form)
        o1, m1 = kk.sparse_conv(xd, f, md, None, (1, 1), (pad, pad), (1, 1), 1, create_out_mask=True, filter_umma=packed)
        p1, t1 = prev.cuda(), trunc.cuda()
        kk.sparse_activation(o1, p1, t1, m1, 0.8, act, 0)
        p2, t2 = prev.cuda(), trunc.cuda()
        o2, m2 = kk.sparse_conv(xd, f, md, None, (1, 1), (pad, pad), (1, 1), 1, create_out_mask=True, filter_umma=packed,
                                epilogue=kk.make_epilogue(p2, t2, 0.8, act, 0))
        torch.cuda.synchronize()
        assert _lib.lib.dc_umma_error() == 0
        assert torch.equal(m1, m2) and torch.equal(p1, p2) and torch.equal(t1, t2)
        sel = (m1 != 0).expand_as(o1)
        assert torch.equal(o1[sel], o2[sel])
        if kind == "full":
            assert 0 < int(m2.sum()) < m2.numel(), "the case must exercise kept and dropped pixels"


def test_halo_tiles_repeat_calls_give_identical_results():
    """The same call twice (persistent CTAs, rings re-initialised per launch): identical bits."""
    import deltacnn_b200.cuda_kernels as kk
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    g = torch.Generator().manual_seed(5)
    cin, cout, n, h, w = 64, 64, 4, 40, 56
    x = cl((torch.randn(n, cin, h, w, generator=g) * 0.5).half()).cuda()
    mask = (torch.rand(n, 1, h, w, generator=g) < 0.7).to(torch.int32).cuda()
    f = convert_filter_out_channels_last((torch.randn(cout, cin, 3, 3, generator=g) * 0.05).half()).cuda()
    packed = _packed(kk, f, cin, cout, 1)
    outs = []
    for _ in range(2):
        out = cl(torch.zeros(n, cout, h, w, dtype=torch.float16)).cuda()
        o, m = kk.sparse_conv(x, f, mask, None, (1, 1), (1, 1), (1, 1), 1, create_out_mask=True, out=out, filter_umma=packed)
        outs.append((o.clone(), m.clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("cin,seg,nh,n,h,w", [(256, 64, 3, 2, 33, 40), (64, 32, 2, 3, 24, 16), (64, 32, 4, 1, 40, 24), (128, 64, 3, 1, 20, 17)])
@pytest.mark.parametrize("kind", ["full", "half", "sparse"])
def test_several_heads_in_one_launch(cin, seg, nh, n, h, w, kind):
    """dc_conv3x3_heads: the 3x3 convolutions of several heads on the same input in one launch. Plain form against the
    oracle per head; fused form (each head's own caches, threshold and activation) against the plain form followed by the
    stand-alone truncation kernel per head: identical masks, caches and values."""
    import deltacnn_b200.cuda_kernels as kk
    from deltacnn_b200 import _lib
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    g = torch.Generator().manual_seed(3)
    x = cl((torch.randn(n, cin, h, w, generator=g) * 0.5).half())
    mask = _masks(g, n, h, w, kind)
    wts = [(torch.randn(seg, cin, 3, 3, generator=g) / (3 * cin ** 0.5)).half() for _ in range(nh)]
    biases = [torch.randn(seg, generator=g).half() for _ in range(nh)]
    wcat, bcat = torch.cat(wts, dim=0), torch.cat(biases, dim=0)
    f = convert_filter_out_channels_last(wcat).cuda()
    packed = _packed(kk, f, cin, seg * nh, 1)
    desc = kk.make_conv_desc((n, cin, h, w), seg * nh, (h, w), (3, 3), (1, 1), (1, 1), (1, 1), 1, 1)
    assert kk.conv3x3_heads_supported(desc, nh)
    xd, md = x.cuda(), mask.cuda()
    xd[(mask == 0).expand_as(x)] = float("nan")
    outs = [cl(torch.full((n, seg, h, w), float("nan"), dtype=torch.float16)).cuda() for _ in range(nh)]
    mos = [torch.full((n, 1, h, w), -7, dtype=torch.int32, device="cuda") for _ in range(nh)]
    kk.conv3x3_heads(xd, md, packed, bcat.cuda(), outs, mos, desc)
    torch.cuda.synchronize()
    assert _lib.lib.dc_umma_error() == 0
    for hd in range(nh):
        ref, m_ref = O.conv(x, mask, wts[hd], biases[hd], (1, 1), (1, 1), (1, 1), 1)
        assert torch.equal(mos[hd].cpu(), m_ref), f"head {hd}: out-mask"
        sel = (m_ref != 0).expand_as(ref)
        if sel.any():
            scale = max(ref.float()[sel].abs().max().item(), 1e-6)
            assert (outs[hd].cpu().float()[sel] - ref.float()[sel]).abs().max().item() / scale <= 1e-2, f"head {hd}: values"
        assert torch.isnan(outs[hd].cpu()[~sel]).all(), "pixels outside the out-mask must not be written"
    # fused truncation, every head with its own threshold and activation
    prevs = [cl(torch.randn(n, seg, h, w, generator=g).half()) for _ in range(nh)]
    truncs = [cl((torch.randn(n, seg, h, w, generator=g) * 0.02).half()) for _ in range(nh)]
    thr = [0.6 + 0.15 * hd for hd in range(nh)]
    acts = [1, 2, 1, 0][:nh]
    p1, t1 = [p.cuda() for p in prevs], [t.cuda() for t in truncs]
    o1 = [cl(torch.zeros(n, seg, h, w, dtype=torch.float16)).cuda() for _ in range(nh)]
    m1 = [torch.empty(n, 1, h, w, dtype=torch.int32, device="cuda") for _ in range(nh)]
    kk.conv3x3_heads(xd, md, packed, None, o1, m1, desc)
    for hd in range(nh):
        kk.sparse_activation(o1[hd], p1[hd], t1[hd], m1[hd], thr[hd], acts[hd], 0)
    p2, t2 = [p.cuda() for p in prevs], [t.cuda() for t in truncs]
    o2 = [cl(torch.zeros(n, seg, h, w, dtype=torch.float16)).cuda() for _ in range(nh)]
    m2 = [torch.empty(n, 1, h, w, dtype=torch.int32, device="cuda") for _ in range(nh)]
    kk.conv3x3_heads(xd, md, packed, None, o2, m2, desc,
                     epilogues=[kk.make_epilogue(p2[hd], t2[hd], thr[hd], acts[hd], 0) for hd in range(nh)])
    torch.cuda.synchronize()
    assert _lib.lib.dc_umma_error() == 0
    for hd in range(nh):
        assert torch.equal(m1[hd], m2[hd]) and torch.equal(p1[hd], p2[hd]) and torch.equal(t1[hd], t2[hd]), f"head {hd}"
        sel = (m1[hd] != 0).expand_as(o1[hd])
        assert torch.equal(o1[hd][sel], o2[hd][sel]), f"head {hd}"
