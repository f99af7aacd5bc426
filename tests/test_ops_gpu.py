"""Parity of every C-ABI operator (through the Python operator API) with the CPU oracle on
seeded inputs. Integer results (masks) must be bit-exact; floating point within the stated
tolerance of the oracle at the pixels the operator defines (out-mask == 1)."""
import pytest
import torch

from oracle import delta_ops as O

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16]
TOL = {torch.float32: 1e-4, torch.float16: 1e-2}   # relative to max |reference|


def K():
    import deltacnn_b200.cuda_kernels as k
    return k


def cl(t):
    return t.contiguous(memory_format=torch.channels_last)


def rand_feat(g, n, c, h, w, dtype, scale=1.0):
    return cl((torch.randn(n, c, h, w, generator=g) * scale).to(dtype))


def rand_mask(g, n, h, w, density):
    if density >= 1.0:
        return torch.ones(n, 1, h, w, dtype=torch.int32)
    if density <= 0.0:
        return torch.zeros(n, 1, h, w, dtype=torch.int32)
    return (torch.rand(n, 1, h, w, generator=g) < density).to(torch.int32)


def assert_close_masked(got, ref, mask, dtype, what=""):
    sel = (mask != 0).expand_as(ref)
    if sel.sum() == 0:
        return
    r = ref.float()[sel]
    g_ = got.float().cpu()[sel]
    scale = max(r.abs().max().item(), 1e-6)
    err = (g_ - r).abs().max().item() / scale
    assert err <= TOL[dtype], f"{what}: relative error {err:.3e} > {TOL[dtype]}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("c", [3, 8, 17, 64])
@pytest.mark.parametrize("thr", [0.0, 0.05])
def test_sparsify(dtype, c, thr):
    g = torch.Generator().manual_seed(1)
    n, h, w = 2, 13, 19
    prev = rand_feat(g, n, c, h, w, dtype)
    x = prev.clone()
    upd = torch.rand(n, 1, h, w, generator=g) < 0.3
    x = cl(torch.where(upd.expand_as(x), rand_feat(g, n, c, h, w, dtype), x + (0.01 * torch.randn(n, c, h, w, generator=g)).to(dtype)))
    d_ref, m_ref, p_ref = torch.zeros_like(x), torch.zeros(n, 1, h, w, dtype=torch.int32), prev.clone()
    O.sparsify(x, p_ref, d_ref, m_ref, thr)
    xd, pd = x.cuda(), prev.cuda()
    dd = torch.full_like(xd, float("nan"))
    md = torch.full((n, 1, h, w), -7, dtype=torch.int32, device="cuda")
    K().sparsify(xd, pd, dd, md, thr)
    assert torch.equal(md.cpu(), m_ref)
    assert torch.equal(pd.cpu(), p_ref)
    sel = (m_ref != 0).expand_as(x)
    assert torch.equal(dd.cpu()[sel], d_ref[sel])
    # inactive pixels of delta are either untouched or (RGB vector kernel: a run of pixels with an active member is
    # written whole) hold their own sub-threshold difference -- never anything else
    rest = dd.cpu()[~sel].float()
    sub = (x.float() - prev.float()).to(dtype).float()[~sel]
    assert (torch.isnan(rest) | (rest == sub)).all(), "inactive pixels of delta hold foreign values"
    if c != 3:
        assert torch.isnan(rest).all(), "inactive pixels of delta must not be written"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("c", [3, 32, 96, 200, 1280])
@pytest.mark.parametrize("act,mode", [(1, 0), (2, 0), (0, 0), (3, 0), (2, 1), (2, 2), (1, -1), (0, -1)])
def test_activate_truncate(dtype, c, act, mode):
    if c == 1280 and dtype == torch.float32 and mode > 0:
        pytest.skip("covered by the other widths")
    g = torch.Generator().manual_seed(2)
    n, h, w = 2, 9, 11
    delta = rand_feat(g, n, c, h, w, dtype, 0.05)
    prev = rand_feat(g, n, c, h, w, dtype, 2.0)
    trunc = rand_feat(g, n, c, h, w, dtype, 0.01)
    mask = rand_mask(g, n, h, w, 0.5)
    thr = 0.12 if mode == 0 else (0.5 if mode == 1 else 0.04)
    d_ref, p_ref, t_ref, m_ref = delta.clone(), prev.clone(), trunc.clone(), mask.clone()
    O.activate_truncate(d_ref, p_ref, t_ref, m_ref, thr, act, mode)
    dd, pd, td, md = delta.cuda(), prev.cuda(), trunc.cuda(), mask.cuda()
    K().sparse_activation(dd, pd, td if mode >= 0 else None, md, thr, act, mode)
    if mode <= 0:
        assert torch.equal(md.cpu(), m_ref)
        assert torch.equal(pd.cpu(), p_ref)
        if mode == 0:
            assert torch.equal(td.cpu(), t_ref)
        sel = (m_ref != 0).expand_as(delta)
        assert torch.equal(dd.cpu()[sel], d_ref[sel])
    else:
        # the norm is a floating-point reduction: allow decisions to differ only where it ties the threshold
        agree = (md.cpu() == m_ref).float().mean().item()
        assert agree > 0.99
    # pixels outside the incoming mask are untouched
    off = (mask == 0).expand_as(delta)
    assert torch.equal(dd.cpu()[off], delta[off]) and torch.equal(pd.cpu()[off], prev[off])


CONV_CASES = [
    # cin, cout, k, stride, pad, dil, groups, h, w
    (3, 32, 3, 2, 1, 1, 1, 18, 22),
    (16, 24, 1, 1, 0, 1, 1, 9, 13),
    (24, 144, 1, 1, 0, 1, 1, 8, 8),
    (32, 64, 1, 2, 0, 1, 1, 10, 12),
    (20, 36, 3, 1, 1, 1, 1, 11, 9),
    (64, 64, 3, 2, 1, 1, 1, 12, 12),
    (8, 8, 3, 1, 2, 2, 1, 12, 12),
    (3, 16, 7, 2, 3, 1, 1, 20, 20),
    (6, 10, 5, 1, 2, 1, 1, 9, 9),
    (32, 32, 3, 1, 1, 1, 32, 9, 10),
    (96, 96, 3, 2, 1, 1, 96, 12, 12),
    (12, 12, 5, 1, 2, 1, 12, 8, 8),
    (7, 7, 3, 1, 1, 1, 7, 8, 8),
    # maps large enough for the persistent kernels that compact the active pixels per CTA
    (3, 32, 3, 2, 1, 1, 1, 320, 330), (3, 16, 7, 2, 3, 1, 1, 300, 300), (32, 32, 3, 1, 1, 1, 32, 150, 151), (96, 96, 3, 2, 1, 1, 96, 300, 302),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CONV_CASES)
@pytest.mark.parametrize("density", [0.0, 0.1, 1.0])
def test_conv(dtype, case, density):
    cin, cout, k, s, p, d, groups, h, w = case
    g = torch.Generator().manual_seed(3)
    n = 2
    x = rand_feat(g, n, cin, h, w, dtype)
    mask = rand_mask(g, n, h, w, density)
    wt = (torch.randn(cout, cin // groups, k, k, generator=g) * (1.0 / (k * (cin // groups) ** 0.5))).to(dtype)
    bias = torch.randn(cout, generator=g).to(dtype)
    ref, m_ref = O.conv(x, mask, wt, bias, (s, s), (p, p), (d, d), groups)
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    f = convert_filter_out_channels_last(wt).cuda()
    xd = x.cuda()
    xd[(mask == 0).expand_as(x)] = float("nan")       # inactive inputs must never be read
    out, om = K().sparse_conv(xd, f, mask.cuda(), bias.cuda(), (s, s), (p, p), (d, d), groups, create_out_mask=True)
    assert torch.equal(om.cpu(), m_ref)
    assert_close_masked(out, ref, m_ref, dtype, "conv")
    # dense-output mode (no out-mask): every pixel defined, zeros + bias where nothing is active
    out2 = K().sparse_conv(xd, f, mask.cuda(), bias.cuda(), (s, s), (p, p), (d, d), groups, create_out_mask=False)
    assert_close_masked(out2, ref, torch.ones_like(m_ref), dtype, "conv dense-out")


def test_conv_asymmetric_padding():
    g = torch.Generator().manual_seed(4)
    x = rand_feat(g, 1, 8, 9, 9, torch.float32)
    mask = rand_mask(g, 1, 9, 9, 0.4)
    wt = torch.randn(8, 8, 3, 3, generator=g) * 0.1
    ref, m_ref = O.conv(x, mask, wt, None, (2, 2), (0, 1, 0, 1), (1, 1), 1)
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    out, om = K().sparse_conv(x.cuda(), convert_filter_out_channels_last(wt).cuda(), mask.cuda(), None, (2, 2), (0, 1, 0, 1),
                              (1, 1), 1, create_out_mask=True)
    assert torch.equal(om.cpu(), m_ref)
    assert_close_masked(out, ref, m_ref, torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("k,s,p", [(4, 2, 1), (6, 4, 1), (2, 2, 0)])
@pytest.mark.parametrize("density", [0.0, 0.15, 1.0])
def test_deconv(dtype, k, s, p, density):
    g = torch.Generator().manual_seed(5)
    n, cin, cout, h, w = 2, 24, 20, 7, 9
    x = rand_feat(g, n, cin, h, w, dtype)
    mask = rand_mask(g, n, h, w, density)
    wt = (torch.randn(cin, cout, k, k, generator=g) * 0.1).to(dtype)
    bias = torch.randn(cout, generator=g).to(dtype)
    ref, m_ref = O.deconv(x, mask, wt, bias, (s, s), (p, p))
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    f = convert_filter_out_channels_last(wt, transposed=True).cuda()
    out, om = K().sparse_deconv(x.cuda(), f, mask.cuda(), bias.cuda(), (s, s), (p, p), (1, 1), 1, create_out_mask=True)
    assert out.shape == ref.shape
    assert torch.equal(om.cpu(), m_ref)
    assert_close_masked(out, ref, m_ref, dtype, "deconv")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("c", [5, 64])
@pytest.mark.parametrize("act,dense_out", [(0, False), (1, False), (1, True), (0, True)])
def test_add(dtype, c, act, dense_out):
    g = torch.Generator().manual_seed(6)
    n, h, w = 2, 7, 9
    a, b = rand_feat(g, n, c, h, w, dtype), rand_feat(g, n, c, h, w, dtype)
    ma, mb = rand_mask(g, n, h, w, 0.3), rand_mask(g, n, h, w, 0.3)
    prev = rand_feat(g, n, c, h, w, dtype)
    p_ref = prev.clone()
    ref, m_ref = O.add(a, ma, b, mb, p_ref, 0.5, 2.0, act, dense_out)
    pd = prev.cuda()
    out = torch.full_like(a, float("nan")).cuda()
    mo = torch.full((n, 1, h, w), -3, dtype=torch.int32, device="cuda")
    K().sparse_add_tensors(a.cuda(), b.cuda(), pd if (act > 0 or dense_out) else None, out, ma.cuda(), mb.cuda(), mo, 0.5, 2.0, act, dense_out)
    if dense_out:
        assert_close_masked(out, ref, torch.ones(n, 1, h, w, dtype=torch.int32), dtype, "add dense")
    else:
        assert torch.equal(mo.cpu(), m_ref)
        assert_close_masked(out, ref, m_ref, dtype, "add")
    if act > 0 or dense_out:
        assert_close_masked(pd, p_ref, torch.ones(n, 1, h, w, dtype=torch.int32), dtype, "add prev")


@pytest.mark.parametrize("dtype", DTYPES)
def test_add_to_dense_and_densify(dtype):
    g = torch.Generator().manual_seed(7)
    n, c, h, w = 2, 24, 6, 5
    a, b = rand_feat(g, n, c, h, w, dtype), rand_feat(g, n, c, h, w, dtype)
    m = rand_mask(g, n, h, w, 0.4)
    b_ref = b.clone()
    O.add_to_dense(a, b_ref, m)
    bd = b.cuda()
    K().sparse_add_to_dense_tensor(a.cuda(), bd, m.cuda())
    assert torch.equal(bd.cpu(), b_ref)
    p_ref = b.clone()
    ref = O.densify(a, m, p_ref, 2)
    pd = b.cuda()
    out = K().sparse_densify(a.cuda(), m.cuda(), pd, None, 2)
    assert torch.equal(pd.cpu(), p_ref)
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("k,s,p,c", [(3, 2, 1, 64), (2, 2, 0, 12), (3, 1, 1, 5)])
def test_max_pool(dtype, k, s, p, c):
    g = torch.Generator().manual_seed(8)
    n, h, w = 2, 12, 14
    x = rand_feat(g, n, c, h, w, dtype)
    prev = rand_feat(g, n, c, h, w, dtype)
    m = rand_mask(g, n, h, w, 0.2)
    ref, m_ref = O.max_pool(x, m, prev, (k, k), (s, s), (p, p))
    p_ref = prev.clone()
    O.add_to_dense(x, p_ref, m)
    pd = prev.cuda()
    out, om = K().sparse_pooling(x.cuda(), pd, (k, k), m.cuda(), (s, s), (p, p), (1, 1), update_prev=True)
    assert torch.equal(om.cpu(), m_ref)
    assert_close_masked(out, ref, m_ref, dtype, "maxpool")
    assert torch.equal(pd.cpu(), p_ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("c,h,w", [(1280, 7, 7), (40, 16, 16), (6, 40, 40)])
@pytest.mark.parametrize("density", [0.0, 0.3, 1.0])
def test_global_avg_pool(dtype, c, h, w, density):
    g = torch.Generator().manual_seed(9)
    n = 3
    x = rand_feat(g, n, c, h, w, dtype)
    m = rand_mask(g, n, h, w, density)
    m[1] = 0
    ref, m_ref = O.global_avg_pool(x, m)
    out, om = K().sparse_pooling(x.cuda(), None, (h, w), m.cuda(), (1, 1), (0, 0), (1, 1), pooling_mode_int=1)
    assert torch.equal(om.cpu(), m_ref)
    assert_close_masked(out, ref, torch.ones_like(m_ref), dtype, "avgpool")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("scale,c", [(2, 32), (4, 5), (8, 64)])
def test_upsample(dtype, scale, c):
    g = torch.Generator().manual_seed(10)
    x = rand_feat(g, 2, c, 5, 6, dtype)
    m = rand_mask(g, 2, 5, 6, 0.4)
    ref, m_ref = O.upsample(x, m, scale)
    out, om = K().sparse_upsample(x.cuda(), m.cuda(), scale)
    assert torch.equal(om.cpu().view_as(m_ref), m_ref)
    sel = (m_ref != 0).expand_as(ref)
    assert torch.equal(out.cpu()[sel], ref[sel])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("ca,cb", [(8, 16), (3, 5)])
def test_concat_and_scale_bias(dtype, ca, cb):
    g = torch.Generator().manual_seed(11)
    n, h, w = 2, 6, 7
    a, b = rand_feat(g, n, ca, h, w, dtype), rand_feat(g, n, cb, h, w, dtype)
    ma, mb = rand_mask(g, n, h, w, 0.4), rand_mask(g, n, h, w, 0.4)
    ref, m_ref = O.concatenate(a, ma, b, mb)
    out, om = K().sparse_concatenate((a.cuda(), ma.cuda()), (b.cuda(), mb.cuda()))
    assert torch.equal(om.cpu().view_as(m_ref), m_ref)
    sel = (m_ref != 0).expand_as(ref)
    assert torch.equal(out.cpu()[sel], ref[sel])
    scale, bias = torch.randn(ca, generator=g).to(dtype), torch.randn(ca, generator=g).to(dtype)
    ref2, _ = O.scale_bias(a, ma, scale, bias)
    ad = a.cuda()
    K().sparse_mul_add(ad, ma.cuda(), ad, ma.cuda(), scale.cuda(), bias.cuda())
    assert_close_masked(ad, ref2, ma, dtype, "scale_bias")


def test_compact_mask():
    g = torch.Generator().manual_seed(12)
    m = rand_mask(g, 3, 37, 41, 0.13)
    idx, cnt = K().compact_mask(m.cuda())
    k = int(cnt.item())
    want = torch.nonzero(m.flatten()).flatten()
    assert k == want.numel()
    assert torch.equal(torch.sort(idx[:k].cpu().long())[0], want)


def test_empty_batch_and_errors():
    k = K()
    x = torch.zeros(0, 8, 4, 4, device="cuda").contiguous(memory_format=torch.channels_last)
    k.sparsify(x, x.clone(), x.clone(), torch.zeros(0, 1, 4, 4, dtype=torch.int32, device="cuda"), 0.1)
    with pytest.raises(RuntimeError):
        k.sparsify(torch.zeros(1, 8, 4, 4), torch.zeros(1, 8, 4, 4), torch.zeros(1, 8, 4, 4), torch.zeros(1, 1, 4, 4, dtype=torch.int32), 0.1)
    with pytest.raises(RuntimeError):      # NCHW-contiguous input is rejected, not silently misread
        k.sparse_activation(torch.zeros(1, 8, 4, 4, device="cuda"), torch.zeros(1, 8, 4, 4, device="cuda"), None,
                            torch.zeros(1, 1, 4, 4, dtype=torch.int32, device="cuda"), 0.0, 1, -1)
    with pytest.raises(RuntimeError):      # grouped convolution that is neither dense nor depthwise
        xx = torch.zeros(1, 8, 4, 4, device="cuda").contiguous(memory_format=torch.channels_last)
        k.sparse_conv(xx, torch.zeros(3, 3, 4, 8, device="cuda"), torch.ones(1, 1, 4, 4, dtype=torch.int32, device="cuda"), None,
                      (1, 1), (1, 1), (1, 1), 2, create_out_mask=True)
    with pytest.raises(RuntimeError):
        k.sparsify(x.double(), x.double(), x.double(), torch.zeros(0, 1, 4, 4, dtype=torch.int32, device="cuda"), 0.1)


# ---------------------------------------------------------------------------------------------
# tensor-core pointwise convolution (tcgen05 gather-GEMM), fp16
# ---------------------------------------------------------------------------------------------
PW_CASES = [
    # cin, cout, stride, n, h, w
    (32, 16, 1, 2, 20, 24), (16, 96, 1, 2, 24, 20), (96, 24, 1, 2, 16, 16), (24, 144, 1, 2, 16, 12), (144, 32, 1, 3, 9, 9),
    (192, 64, 1, 2, 14, 14), (64, 384, 1, 2, 14, 14), (576, 160, 1, 2, 7, 7), (960, 320, 1, 2, 7, 7), (320, 1280, 1, 3, 7, 7),
    (256, 512, 2, 2, 16, 16), (64, 256, 1, 1, 40, 40), (1024, 2048, 2, 1, 8, 8),
    # large maps: persistent CTAs over strided spans, one and several rounds
    (16, 96, 1, 3, 120, 121), (96, 24, 1, 4, 112, 112), (16, 32, 1, 10, 224, 224),
]


def _pack_umma(wt_hwio, cin, cout, stride):
    from deltacnn_b200 import _lib
    import deltacnn_b200.cuda_kernels as k
    desc = k.make_conv_desc((1, cin, 8, 8), cout, (8, 8), (1, 1), (stride, stride), (0, 0), (1, 1), 1, 1)
    nbytes = _lib.lib.dc_filter_umma_bytes(desc, 0)
    assert nbytes > 0
    packed = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    _lib.check(_lib.lib.dc_pack_filter_umma(desc, 0, wt_hwio.data_ptr(), packed.data_ptr(), torch.cuda.current_stream().cuda_stream), "pack")
    return packed


@pytest.mark.parametrize("case", PW_CASES)
@pytest.mark.parametrize("density", [0.0, 0.08, 0.6, 1.0])
def test_pointwise_umma_matches_oracle(case, density):
    from deltacnn_b200 import _lib
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    cin, cout, s, n, h, w = case
    dtype = torch.float16
    g = torch.Generator().manual_seed(21)
    x = rand_feat(g, n, cin, h, w, dtype)
    mask = rand_mask(g, n, h, w, density)
    wt = (torch.randn(cout, cin, 1, 1, generator=g) / cin ** 0.5).to(dtype)
    bias = torch.randn(cout, generator=g).to(dtype)
    ref, m_ref = O.conv(x, mask, wt, bias, (s, s), (0, 0), (1, 1), 1)
    f = convert_filter_out_channels_last(wt).cuda()
    packed = _pack_umma(f, cin, cout, s)
    xd = x.cuda()
    xd[(mask == 0).expand_as(x)] = float("nan")
    out = torch.full(ref.shape, float("nan"), dtype=dtype, device="cuda").contiguous(memory_format=torch.channels_last)
    out, om = K().sparse_conv(xd, f, mask.cuda(), bias.cuda(), (s, s), (0, 0), (1, 1), 1, create_out_mask=True, out=out, filter_umma=packed)
    assert _lib.lib.dc_umma_error() == 0
    assert torch.equal(om.cpu(), m_ref)
    assert_close_masked(out, ref, m_ref, dtype, "pointwise umma")
    off = (m_ref == 0).expand_as(ref)
    assert torch.isnan(out.cpu()[off]).all(), "pixels outside the out-mask must not be written"
    # the CUDA-core kernel computes the same thing
    out2, om2 = K().sparse_conv(xd, f, mask.cuda(), bias.cuda(), (s, s), (0, 0), (1, 1), 1, create_out_mask=True)
    assert torch.equal(om2, om)
    assert_close_masked(out2, out.cpu(), m_ref, dtype, "umma vs simt")


@pytest.mark.parametrize("case", PW_CASES + [(64, 384, 1, 2, 14, 14), (96, 576, 1, 3, 14, 14), (160, 960, 1, 2, 7, 7), (320, 1280, 1, 2, 7, 7),
                                             (256, 2048, 1, 1, 9, 9), (32, 272, 1, 3, 30, 30)])
@pytest.mark.parametrize("act", [2, 0])
def test_pointwise_umma_fused_epilogue_equals_two_kernels(case, act):
    from deltacnn_b200 import _lib
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    import deltacnn_b200.cuda_kernels as k
    cin, cout, s, n, h, w = case
    dtype = torch.float16
    g = torch.Generator().manual_seed(22)
    x = rand_feat(g, n, cin, h, w, dtype, 0.2).cuda()
    mask = rand_mask(g, n, h, w, 0.3).cuda()
    wt = (torch.randn(cout, cin, 1, 1, generator=g) / cin ** 0.5).to(dtype)
    f = convert_filter_out_channels_last(wt).cuda()
    packed = _pack_umma(f, cin, cout, s)
    ho, wo = k.conv_out_hw(h, w, (1, 1), (s, s), (0, 0), (1, 1))
    prev = rand_feat(g, n, cout, ho, wo, dtype, 1.0).cuda()
    trunc = rand_feat(g, n, cout, ho, wo, dtype, 0.02).cuda()
    thr = 0.6 if cout <= 64 else 0.9 if cout <= 300 else 0.75       # drops some pixels and keeps others
    # two kernels: convolution, then activation/truncation
    o1, m1 = k.sparse_conv(x, f, mask, None, (s, s), (0, 0), (1, 1), 1, create_out_mask=True, filter_umma=packed)
    p1, t1 = prev.clone(), trunc.clone()
    k.sparse_activation(o1, p1, t1, m1, thr, act, 0)
    # fused
    p2, t2 = prev.clone(), trunc.clone()
    ep = k.make_epilogue(p2, t2, thr, act, 0)
    o2, m2 = k.sparse_conv(x, f, mask, None, (s, s), (0, 0), (1, 1), 1, create_out_mask=True, filter_umma=packed, epilogue=ep)
    assert _lib.lib.dc_umma_error() == 0
    assert torch.equal(m1, m2)
    assert int(m2.sum()) <= int(mask[:, :, ::s, ::s].sum())
    if cout > 300:
        assert 0 < int(m2.sum()) < int(mask[:, :, ::s, ::s].sum()), "the threshold must keep some active pixels and drop others"
    assert torch.equal(p1, p2) and torch.equal(t1, t2)
    sel = (m1 != 0).expand_as(o1)
    assert torch.equal(o1[sel], o2[sel])


@pytest.mark.parametrize("c,h,w,s", [(32, 40, 36, 1), (96, 30, 30, 2), (144, 17, 19, 1), (576, 14, 14, 1), (960, 7, 7, 1), (192, 28, 28, 2)])
@pytest.mark.parametrize("density", [0.05, 0.7])
def test_depthwise_fused_epilogue_equals_two_kernels(c, h, w, s, density):
    """fp16 depthwise 3x3 tile kernel with the fused activation/truncation epilogue against the same
    convolution followed by the stand-alone activation kernel (bit-exact), and against the oracle."""
    import deltacnn_b200.cuda_kernels as k
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    dtype = torch.float16
    g = torch.Generator().manual_seed(31)
    n = 2
    x = rand_feat(g, n, c, h, w, dtype, 0.3)
    mask = rand_mask(g, n, h, w, density)
    mask[:, :, : h // 3, : w // 2] = 0            # some tiles without any active input
    wt = (torch.randn(c, 1, 3, 3, generator=g) * 0.4).to(dtype)
    f = convert_filter_out_channels_last(wt).cuda()
    ho, wo = k.conv_out_hw(h, w, (3, 3), (s, s), (1, 1), (1, 1))
    prev = rand_feat(g, n, c, ho, wo, dtype, 1.0)
    trunc = rand_feat(g, n, c, ho, wo, dtype, 0.02)
    thr = 0.8
    xd, md = x.cuda(), mask.cuda()
    xd[(mask == 0).expand_as(x)] = float("nan")
    o1, m1 = k.sparse_conv(xd, f, md, None, (s, s), (1, 1), (1, 1), c, create_out_mask=True)
    ref, m_ref = O.conv(x, mask, wt, None, (s, s), (1, 1), (1, 1), c)
    assert torch.equal(m1.cpu(), m_ref)
    assert_close_masked(o1, ref, m_ref, dtype, "depthwise tile")
    p1, t1 = prev.cuda(), trunc.cuda()
    k.sparse_activation(o1, p1, t1, m1, thr, 2, 0)
    p2, t2 = prev.cuda(), trunc.cuda()
    o2, m2 = k.sparse_conv(xd, f, md, None, (s, s), (1, 1), (1, 1), c, create_out_mask=True,
                           epilogue=k.make_epilogue(p2, t2, thr, 2, 0))
    assert torch.equal(m1, m2) and torch.equal(p1, p2) and torch.equal(t1, t2)
    sel = (m1 != 0).expand_as(o1)
    assert torch.equal(o1[sel], o2[sel])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cout,k,s,p", [(32, 3, 2, 1), (64, 7, 2, 3), (24, 3, 1, 1)])
@pytest.mark.parametrize("h,w", [(37, 41), (150, 161)])      # the larger map takes the tensor-core stem kernel in fp16
def test_stem_conv_fused_epilogue_equals_two_kernels(dtype, cout, k, s, p, h, w):
    import deltacnn_b200.cuda_kernels as kk
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    g = torch.Generator().manual_seed(41)
    n = 2
    x = rand_feat(g, n, 3, h, w, dtype, 0.5).cuda()
    mask = rand_mask(g, n, h, w, 0.15).cuda()
    wt = (torch.randn(cout, 3, k, k, generator=g) * 0.3).to(dtype)
    f = convert_filter_out_channels_last(wt).cuda()
    ho, wo = kk.conv_out_hw(h, w, (k, k), (s, s), (p, p), (1, 1))
    prev = rand_feat(g, n, cout, ho, wo, dtype, 1.0)
    trunc = rand_feat(g, n, cout, ho, wo, dtype, 0.02)
    o1, m1 = kk.sparse_conv(x, f, mask, None, (s, s), (p, p), (1, 1), 1, create_out_mask=True)
    p1, t1 = prev.cuda(), trunc.cuda()
    kk.sparse_activation(o1, p1, t1, m1, 0.9, 2, 0)
    p2, t2 = prev.cuda(), trunc.cuda()
    o2, m2 = kk.sparse_conv(x, f, mask, None, (s, s), (p, p), (1, 1), 1, create_out_mask=True, epilogue=kk.make_epilogue(p2, t2, 0.9, 2, 0))
    assert torch.equal(m1, m2) and torch.equal(p1, p2) and torch.equal(t1, t2)
    assert 0 < int(m2.sum())
    sel = (m1 != 0).expand_as(o1)
    assert torch.equal(o1[sel], o2[sel])


@pytest.mark.parametrize("kind,cin,cout,h,w,s", [("pw", 16, 96, 40, 44, 1), ("pw", 144, 24, 28, 28, 1), ("pw", 960, 320, 7, 7, 1), ("pw", 64, 384, 14, 14, 1),
                                                  ("pw", 256, 512, 16, 16, 2), ("dw", 96, 96, 40, 44, 2), ("dw", 32, 32, 50, 50, 1), ("dw", 960, 960, 7, 7, 1),
                                                  # maps large enough for the list-driven kernels to be chosen
                                                  ("pw", 16, 96, 120, 121, 1), ("pw", 96, 24, 120, 121, 1), ("dw", 32, 32, 120, 121, 1),
                                                  ("dw", 96, 96, 240, 236, 2), ("stem", 3, 32, 240, 236, 2), ("stem", 3, 32, 45, 47, 2)])
@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("density", [0.0, 0.1, 1.0])
def test_worklist_kernels_equal_the_plain_ones(kind, cin, cout, h, w, s, fused, density):
    """dc_conv2d_ws (active-pixel work list in caller scratch) must give exactly what dc_conv2d gives."""
    import deltacnn_b200.cuda_kernels as k
    from deltacnn_b200 import _lib
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    dtype = torch.float16
    g = torch.Generator().manual_seed(51)
    n = 3
    x = rand_feat(g, n, cin, h, w, dtype, 0.3).cuda()
    mask = rand_mask(g, n, h, w, density)
    mask[0, :, : h // 2] = 0
    mask = mask.cuda()
    groups = cin if kind == "dw" else 1
    ksz, pad = (1, 0) if kind == "pw" else (3, 1)
    wt = (torch.randn(cout, cin // groups, ksz, ksz, generator=g) * (0.4 if kind == "dw" else cin ** -0.5)).to(dtype)
    f = convert_filter_out_channels_last(wt).cuda()
    packed = _pack_umma(f, cin, cout, s) if kind == "pw" else None
    ho, wo = k.conv_out_hw(h, w, (ksz, ksz), (s, s), (pad, pad), (1, 1))
    prev = rand_feat(g, n, cout, ho, wo, dtype, 1.0)
    trunc = rand_feat(g, n, cout, ho, wo, dtype, 0.02)
    desc = k.make_conv_desc(tuple(x.shape), cout, (ho, wo), (ksz, ksz), (s, s), (pad, pad), (1, 1), groups, 1)
    ws = torch.full((k.conv_workspace_bytes(desc) + 64,), 0xAB, dtype=torch.uint8, device="cuda")
    res = []
    for workspace in (None, ws):
        p_, t_ = prev.cuda(), trunc.cuda()
        ep = k.make_epilogue(p_, t_, 0.7, 2, 0) if fused else None
        out = torch.full((n, cout, ho, wo), float("nan"), dtype=dtype, device="cuda").contiguous(memory_format=torch.channels_last)
        o, m = k.sparse_conv(x, f, mask, None, (s, s), (pad, pad), (1, 1), groups, create_out_mask=True, out=out,
                             filter_umma=packed, epilogue=ep, workspace=workspace)
        res.append((o.clone(), m.clone(), p_, t_))
    assert _lib.lib.dc_umma_error() == 0
    (o1, m1, p1, t1), (o2, m2, p2, t2) = res
    assert torch.equal(m1, m2) and torch.equal(p1, p2) and torch.equal(t1, t2)
    sel = (m1 != 0).expand_as(o1)
    assert torch.equal(o1[sel], o2[sel])
    if not fused:
        assert torch.isnan(o2[~sel]).all(), "pixels outside the out-mask must not be written"


KXK_CASES = [
    # cin, cout, k, stride, pad, dil, n, h, w
    (64, 64, 3, 1, 1, 1, 2, 20, 24), (64, 128, 3, 2, 1, 1, 2, 21, 19), (128, 128, 3, 1, 1, 1, 2, 16, 16), (32, 32, 3, 1, 2, 2, 2, 15, 15),
    (256, 256, 3, 1, 1, 1, 1, 12, 12), (512, 512, 3, 1, 1, 1, 1, 8, 8), (24, 40, 5, 1, 2, 1, 2, 13, 13), (256, 64, 3, 1, 1, 1, 2, 17, 30),
]


def _pack_umma_kxk(wt_hwio, cin, cout, k, stride, pad, dil):
    from deltacnn_b200 import _lib
    import deltacnn_b200.cuda_kernels as kk
    desc = kk.make_conv_desc((1, cin, 8, 8), cout, (8, 8), (k, k), (stride, stride), (pad, pad), (dil, dil), 1, 1)
    nbytes = _lib.lib.dc_filter_umma_bytes(desc, 0)
    assert nbytes > 0
    packed = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    _lib.check(_lib.lib.dc_pack_filter_umma(desc, 0, wt_hwio.data_ptr(), packed.data_ptr(), torch.cuda.current_stream().cuda_stream), "pack")
    return packed


@pytest.mark.parametrize("case", KXK_CASES + [(64, 64, 3, 1, 1, 1, 2, 40, 48), (32, 64, 3, 1, 1, 1, 1, 70, 33), (128, 128, 3, 1, 1, 1, 3, 17, 136)])
@pytest.mark.parametrize("density", [0.0, 0.1, 0.97, 1.0])
@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("scratch", [True, False])
def test_kxk_conv_umma_matches_oracle_and_cuda_core_kernel(case, density, fused, scratch):
    """3x3 / 5x5 convolutions as implicit GEMM on tcgen05 against the oracle, and the fused epilogue against
    convolution + stand-alone activation kernel. With scratch memory: work-list mode. Without: stride-1 layers run
    on patch tiles (rows of a fully active patch loaded by 4-D tiled TMA, other patches gathered), strided layers
    fall back to the CUDA-core kernel."""
    import deltacnn_b200.cuda_kernels as kk
    from deltacnn_b200 import _lib
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    cin, cout, k, s, p, d, n, h, w = case
    dtype = torch.float16
    g = torch.Generator().manual_seed(61)
    x = rand_feat(g, n, cin, h, w, dtype, 0.5)
    mask = rand_mask(g, n, h, w, density)
    if density == 0.97:
        mask[0] = 1                      # one fully active image: its patches take the TMA path, the others gather
    wt = (torch.randn(cout, cin, k, k, generator=g) / (k * cin ** 0.5)).to(dtype)
    bias = torch.randn(cout, generator=g).to(dtype)
    ref, m_ref = O.conv(x, mask, wt, bias, (s, s), (p, p), (d, d), 1)
    f = convert_filter_out_channels_last(wt).cuda()
    packed = _pack_umma_kxk(f, cin, cout, k, s, p, d)
    xd, md = x.cuda(), mask.cuda()
    xd[(mask == 0).expand_as(x)] = float("nan")
    ho, wo = ref.shape[2:]
    desc = kk.make_conv_desc(tuple(x.shape), cout, (ho, wo), (k, k), (s, s), (p, p), (d, d), 1, 1)
    ws = torch.empty(kk.conv_workspace_bytes(desc), dtype=torch.uint8, device="cuda") if scratch else None
    if not fused:
        out = torch.full(ref.shape, float("nan"), dtype=dtype, device="cuda").contiguous(memory_format=torch.channels_last)
        out, om = kk.sparse_conv(xd, f, md, bias.cuda(), (s, s), (p, p), (d, d), 1, create_out_mask=True, out=out, filter_umma=packed, workspace=ws)
        assert _lib.lib.dc_umma_error() == 0
        assert torch.equal(om.cpu(), m_ref)
        assert_close_masked(out, ref, m_ref, dtype, "kxk umma")
        assert torch.isnan(out.cpu()[(m_ref == 0).expand_as(ref)]).all()
        return
    prev = rand_feat(g, n, cout, ho, wo, dtype, 1.0)
    trunc = rand_feat(g, n, cout, ho, wo, dtype, 0.02)
    o1, m1 = kk.sparse_conv(xd, f, md, None, (s, s), (p, p), (d, d), 1, create_out_mask=True, filter_umma=packed, workspace=ws)
    p1, t1 = prev.cuda(), trunc.cuda()
    kk.sparse_activation(o1, p1, t1, m1, 0.8, 1, 0)
    p2, t2 = prev.cuda(), trunc.cuda()
    o2, m2 = kk.sparse_conv(xd, f, md, None, (s, s), (p, p), (d, d), 1, create_out_mask=True, filter_umma=packed, workspace=ws,
                            epilogue=kk.make_epilogue(p2, t2, 0.8, 1, 0))
    assert _lib.lib.dc_umma_error() == 0
    assert torch.equal(m1, m2) and torch.equal(p1, p2) and torch.equal(t1, t2)
    sel = (m1 != 0).expand_as(o1)
    assert torch.equal(o1[sel], o2[sel])


@pytest.mark.parametrize("cin,cout,k,p,n,h,w", [(64, 64, 4, 1, 2, 9, 11), (512, 256, 4, 1, 1, 6, 7), (256, 256, 4, 1, 2, 12, 10), (32, 48, 2, 0, 2, 8, 8),
                                                (64, 32, 4, 1, 2, 33, 70), (128, 64, 4, 1, 1, 17, 40)])
@pytest.mark.parametrize("density", [0.0, 0.15, 0.97, 1.0])
@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("scratch", [True, False])
def test_deconv_umma_matches_oracle(cin, cout, k, p, n, h, w, density, fused, scratch):
    """Transposed convolution (stride 2) as four per-phase implicit GEMMs on tcgen05: per-phase work lists with
    scratch memory, patch tiles over the input lattice without."""
    import deltacnn_b200.cuda_kernels as kk
    from deltacnn_b200 import _lib
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    dtype = torch.float16
    g = torch.Generator().manual_seed(71)
    x = rand_feat(g, n, cin, h, w, dtype, 0.5)
    mask = rand_mask(g, n, h, w, density)
    wt = (torch.randn(cin, cout, k, k, generator=g) / cin ** 0.5).to(dtype)
    bias = torch.randn(cout, generator=g).to(dtype)
    ref, m_ref = O.deconv(x, mask, wt, bias, (2, 2), (p, p))
    f = convert_filter_out_channels_last(wt, transposed=True).cuda()
    ho, wo = ref.shape[2:]
    desc = kk.make_conv_desc(tuple(x.shape), cout, (ho, wo), (k, k), (2, 2), (p, p), (1, 1), 1, 1)
    nbytes = _lib.lib.dc_filter_umma_bytes(desc, 1)
    assert nbytes > 0
    packed = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    _lib.check(_lib.lib.dc_pack_filter_umma(desc, 1, f.data_ptr(), packed.data_ptr(), torch.cuda.current_stream().cuda_stream), "pack")
    ws = torch.empty(kk.deconv_workspace_bytes(desc), dtype=torch.uint8, device="cuda") if scratch else None
    xd, md = x.cuda(), mask.cuda()
    xd[(mask == 0).expand_as(x)] = float("nan")
    if not fused:
        out = torch.full(ref.shape, float("nan"), dtype=dtype, device="cuda").contiguous(memory_format=torch.channels_last)
        out, om = kk.sparse_deconv(xd, f, md, bias.cuda(), (2, 2), (p, p), (1, 1), 1, create_out_mask=True, out=out, filter_umma=packed, workspace=ws)
        assert _lib.lib.dc_umma_error() == 0
        assert torch.equal(om.cpu(), m_ref)
        assert_close_masked(out, ref, m_ref, dtype, "deconv umma")
        assert torch.isnan(out.cpu()[(m_ref == 0).expand_as(ref)]).all()
        return
    prev = rand_feat(g, n, cout, ho, wo, dtype, 1.0)
    trunc = rand_feat(g, n, cout, ho, wo, dtype, 0.02)
    o1, m1 = kk.sparse_deconv(xd, f, md, None, (2, 2), (p, p), (1, 1), 1, create_out_mask=True, filter_umma=packed, workspace=ws)
    p1, t1 = prev.cuda(), trunc.cuda()
    kk.sparse_activation(o1, p1, t1, m1, 0.8, 1, 0)
    p2, t2 = prev.cuda(), trunc.cuda()
    o2, m2 = kk.sparse_deconv(xd, f, md, None, (2, 2), (p, p), (1, 1), 1, create_out_mask=True, filter_umma=packed, workspace=ws,
                              epilogue=kk.make_epilogue(p2, t2, 0.8, 1, 0))
    assert torch.equal(m1, m2) and torch.equal(p1, p2) and torch.equal(t1, t2)
    sel = (m1 != 0).expand_as(o1)
    assert torch.equal(o1[sel], o2[sel])


@pytest.mark.parametrize("dtype", DTYPES)
def test_sparsify_u8_ingest_matches_float_path(dtype):
    """8-bit frames through DCSparsify.set_u8_input(): same masks, deltas and cache as normalising with
    torch first and feeding the float frame."""
    from deltacnn_b200 import DCSparsify, DCThreshold
    g = torch.Generator().manual_seed(81)
    n, h, w = 3, 30, 34
    frames = torch.randint(0, 256, (4, n, h, w, 3), generator=g, dtype=torch.uint8)
    frames[1:] = frames[0]
    frames[1, :, 5:12, 7:20] += 40
    frames[2] = frames[1]
    frames[2, :, 15:18, :] -= 9
    frames[3] = frames[2]
    frames = frames.cuda()
    a, b = DCSparsify(delta_threshold=0.05).set_u8_input(1.0 / 255.0, 0.0, dtype), DCSparsify(delta_threshold=0.05)
    for t in range(4):
        xf = (frames[t].float() * (1.0 / 255.0)).to(dtype).permute(0, 3, 1, 2)
        d1, m1 = a(frames[t])
        d2, m2 = b(xf)
        assert torch.equal(m1, m2), t
        sel = (m2 != 0).expand_as(d2)
        assert torch.equal(d1[sel], d2[sel])
        assert torch.equal(a.prev_in, b.prev_in)
        if t > 0:
            assert 0 < int(m1.sum()) < m1.numel() or t == 3
    assert len(DCThreshold.t) == 2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cin,cout", [(64, 1), (64, 2), (32, 17), (256, 5), (20, 3)])
@pytest.mark.parametrize("density", [0.0, 0.2, 1.0])
def test_thin_pointwise_conv(dtype, cin, cout, density):
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    g = torch.Generator().manual_seed(91)
    n, h, w = 2, 17, 23
    x = rand_feat(g, n, cin, h, w, dtype)
    mask = rand_mask(g, n, h, w, density)
    wt = (torch.randn(cout, cin, 1, 1, generator=g) / cin ** 0.5).to(dtype)
    bias = torch.randn(cout, generator=g).to(dtype)
    ref, m_ref = O.conv(x, mask, wt, bias, (1, 1), (0, 0), (1, 1), 1)
    xd = x.cuda()
    xd[(mask == 0).expand_as(x)] = float("nan")
    out, om = K().sparse_conv(xd, convert_filter_out_channels_last(wt).cuda(), mask.cuda(), bias.cuda(), (1, 1), (0, 0), (1, 1), 1,
                              create_out_mask=True)
    assert torch.equal(om.cpu(), m_ref)
    assert_close_masked(out, ref, m_ref, dtype, "thin conv")


@pytest.mark.parametrize("cin,cout,n,h,w", [(144, 24, 2, 28, 28), (384, 64, 3, 14, 14), (960, 160, 2, 7, 7), (96, 24, 4, 112, 112), (192, 32, 1, 19, 23)])
@pytest.mark.parametrize("density,res_density", [(0.1, 0.1), (0.7, 0.3), (1.0, 1.0), (0.0, 0.2), (0.3, 0.0)])
def test_pointwise_conv_with_fused_residual_equals_conv_then_add(cin, cout, n, h, w, density, res_density):
    """A linear 1x1 convolution that adds a residual (delta, mask) in its epilogue must give exactly what the
    convolution followed by dc_add gives: values on the union mask, and the union mask itself."""
    import deltacnn_b200.cuda_kernels as k
    from deltacnn_b200 import _lib
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    dtype = torch.float16
    g = torch.Generator().manual_seed(61)
    x = rand_feat(g, n, cin, h, w, dtype, 0.3).cuda()
    mask = rand_mask(g, n, h, w, density).cuda()
    xn = x.clone()
    xn[(mask == 0).expand_as(x)] = float("nan")              # inactive inputs must never reach the result
    res = rand_feat(g, n, cout, h, w, dtype, 0.5).cuda()
    rmask = rand_mask(g, n, h, w, res_density).cuda()
    resn = res.clone()
    resn[(rmask == 0).expand_as(res)] = float("nan")
    wt = (torch.randn(cout, cin, 1, 1, generator=g) / cin ** 0.5).to(dtype)
    f = convert_filter_out_channels_last(wt).cuda()
    packed = _pack_umma(f, cin, cout, 1)
    # reference: two calls
    o1, m1 = k.sparse_conv(xn, f, mask, None, (1, 1), (0, 0), (1, 1), 1, create_out_mask=True, filter_umma=packed)
    ref = torch.full_like(o1, float("nan"))
    mref = torch.empty_like(m1)
    k.sparse_add_tensors(resn, o1, None, ref, rmask, m1, mref, 1.0, 1.0, 0, False)
    # fused
    out = torch.full_like(o1, float("nan"))
    o2, m2 = k.sparse_conv(xn, f, mask, None, (1, 1), (0, 0), (1, 1), 1, create_out_mask=True, out=out, filter_umma=packed,
                           epilogue=k.make_residual_epilogue(resn, rmask))
    assert _lib.lib.dc_umma_error() == 0
    assert torch.equal(m2, mref)
    assert torch.equal(m2, ((mask != 0) | (rmask != 0)).to(torch.int32))
    sel = (mref != 0).expand_as(ref)
    assert not torch.isnan(o2[sel]).any()
    assert torch.equal(o2[sel], ref[sel])
    assert torch.isnan(o2[~sel]).all(), "pixels outside the union mask must not be written"


def test_fused_residual_on_a_large_pointwise_layer_with_scratch():
    """The residual form of a 1x1 layer whose map is large enough for the work-list front (more than eight 128-pixel
    spans per persistent CTA) and whose caller passes scratch memory, as DCConv2d always does: the call must not be
    refused, the scratch stays unused, and the result equals convolution + dc_add."""
    import deltacnn_b200.cuda_kernels as k
    from deltacnn_b200 import _lib
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    cin, cout, n, h, w = 32, 16, 8, 256, 256                 # 524 288 output pixels
    g = torch.Generator().manual_seed(7)
    x = rand_feat(g, n, cin, h, w, torch.float16, 0.3).cuda()
    mask = rand_mask(g, n, h, w, 0.3).cuda()
    res = rand_feat(g, n, cout, h, w, torch.float16, 0.5).cuda()
    rmask = rand_mask(g, n, h, w, 0.2).cuda()
    f = convert_filter_out_channels_last((torch.randn(cout, cin, 1, 1, generator=g) / cin ** 0.5).half()).cuda()
    packed = _pack_umma(f, cin, cout, 1)
    desc = k.make_conv_desc(tuple(x.shape), cout, (h, w), (1, 1), (1, 1), (0, 0), (1, 1), 1, 1)
    ws = torch.full((k.conv_workspace_bytes(desc),), 0x5A, dtype=torch.uint8, device="cuda")
    o1, m1 = k.sparse_conv(x, f, mask, None, (1, 1), (0, 0), (1, 1), 1, create_out_mask=True, filter_umma=packed)
    ref, mref = torch.zeros_like(o1), torch.empty_like(m1)
    k.sparse_add_tensors(res, o1, None, ref, rmask, m1, mref, 1.0, 1.0, 0, False)
    out = torch.zeros_like(o1)
    o2, m2 = k.sparse_conv(x, f, mask, None, (1, 1), (0, 0), (1, 1), 1, create_out_mask=True, out=out, filter_umma=packed,
                           epilogue=k.make_residual_epilogue(res, rmask), workspace=ws)
    assert _lib.lib.dc_umma_error() == 0
    assert torch.equal(m2, mref)
    sel = (mref != 0).expand_as(ref)
    assert torch.equal(o2[sel], ref[sel])
    assert bool((ws == 0x5A).all()), "the residual form finds its own rows: the scratch must stay untouched"


@pytest.mark.parametrize("cin,cout,k,n,h,w", [(64, 64, 3, 2, 40, 48), (32, 32, 3, 2, 64, 64), (128, 256, 1, 2, 20, 20), (256, 64, 3, 1, 17, 33)])
@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("density,res_density", [(0.1, 0.1), (1.0, 1.0), (0.97, 0.5), (0.0, 0.3)])
def test_conv_with_fused_residual_and_add_activation(cin, cout, k, n, h, w, act, density, res_density):
    """A linear stride-1 convolution (1x1, or 3x3 on patch tiles) that adds a residual and applies the add layer's
    activation in its epilogue against convolution followed by dc_add: same union mask, same values, same
    accumulated sum."""
    import deltacnn_b200.cuda_kernels as kk
    from deltacnn_b200 import _lib
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    dtype = torch.float16
    g = torch.Generator().manual_seed(81)
    pad = k // 2
    x = rand_feat(g, n, cin, h, w, dtype, 0.3).cuda()
    mask = rand_mask(g, n, h, w, density)
    if density == 0.97:
        mask[0] = 1
    mask = mask.cuda()
    xn = x.clone()
    xn[(mask == 0).expand_as(x)] = float("nan")
    res = rand_feat(g, n, cout, h, w, dtype, 0.5).cuda()
    rmask = rand_mask(g, n, h, w, res_density).cuda()
    resn = res.clone()
    resn[(rmask == 0).expand_as(res)] = float("nan")
    wt = (torch.randn(cout, cin, k, k, generator=g) / (k * cin ** 0.5)).to(dtype)
    f = convert_filter_out_channels_last(wt).cuda()
    packed = _pack_umma_kxk(f, cin, cout, k, 1, pad, 1)
    prev = rand_feat(g, n, cout, h, w, dtype, 1.0)
    # reference: convolution, then dc_add
    o1, m1 = kk.sparse_conv(xn, f, mask, None, (1, 1), (pad, pad), (1, 1), 1, create_out_mask=True, filter_umma=packed)
    ref = torch.full_like(o1, float("nan"))
    mref = torch.empty_like(m1)
    p1 = prev.cuda()
    kk.sparse_add_tensors(o1, resn, p1 if act > 0 else None, ref, m1, rmask, mref, 1.0, 1.0, act, False)
    # fused
    p2 = prev.cuda()
    out = torch.full_like(o1, float("nan"))
    o2, m2 = kk.sparse_conv(xn, f, mask, None, (1, 1), (pad, pad), (1, 1), 1, create_out_mask=True, out=out, filter_umma=packed,
                            epilogue=kk.make_residual_epilogue(resn, rmask, p2 if act > 0 else None, act))
    assert _lib.lib.dc_umma_error() == 0
    assert torch.equal(m2, mref)
    sel = (mref != 0).expand_as(ref)
    assert not torch.isnan(o2[sel]).any()
    assert torch.equal(o2[sel], ref[sel])
    assert torch.isnan(o2[~sel]).all(), "pixels outside the union mask must not be written"
    if act > 0:
        assert torch.equal(p1, p2), "accumulated sum of the add layer differs"
