"""Parity of the device-side task heads and the input-side kernels with the CPU oracle: the classifier in delta
form, heat-map arg-max, CenterNet decode, DCSparsify(dilation=k) and the 8-bit ingest. Integer results (positions,
classes, counts, masks) must be exact; floating point within the tolerance stated in each test."""
import pytest
import torch

from oracle import delta_ops as O

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16]


def K():
    import deltacnn_b200.cuda_kernels as k
    return k


def cl(t):
    return t.contiguous(memory_format=torch.channels_last)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,cin,cout", [(5, 1280, 1000), (1, 64, 10), (7, 100, 33), (64, 2048, 1000)])
def test_linear_delta_accumulates_like_the_oracle(dtype, n, cin, cout):
    """Three frames: all streams on the first, a subset afterwards. fp32 accumulator: 1e-5 relative (fp32), and the
    rounded output within one half ulp of it (1e-3 relative, fp16)."""
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(cout, cin, generator=g) * cin ** -0.5).to(dtype)
    b = torch.randn(cout, generator=g).to(dtype)
    acc_ref = torch.zeros(n, cout)
    acc = torch.full((n, cout), float("nan"), device="cuda")
    out = torch.empty(n, cout, dtype=dtype, device="cuda")
    wd, bd = w.cuda(), b.cuda()
    for t in range(3):
        delta = cl((torch.randn(n, cin, 1, 1, generator=g) * (1.0 if t == 0 else 0.1)).to(dtype))
        mask = torch.ones(n, 1, 1, 1, dtype=torch.int32) if t == 0 else (torch.rand(n, 1, 1, 1, generator=g) < 0.5).to(torch.int32)
        ref = O.linear_delta(delta, mask, w, b, acc_ref, t == 0)
        before = acc.clone()
        got = K().linear_delta(delta.cuda(), mask.cuda(), wd, bd, acc, out, t == 0)
        scale = acc_ref.abs().max().item()
        assert (acc.cpu() - acc_ref).abs().max().item() <= 1e-5 * scale + 1e-6
        assert (got.float().cpu() - ref.float()).abs().max().item() <= (1e-5 if dtype == torch.float32 else 1e-3) * scale
        if t > 0:       # streams without an update are not touched
            off = (mask.reshape(n) == 0)
            assert torch.equal(acc.cpu()[off], before.cpu()[off])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,j,h,w", [(3, 17, 64, 64), (2, 1, 5, 7), (2, 40, 16, 12)])
def test_heatmap_argmax_matches_torch_argmax(dtype, n, j, h, w):
    g = torch.Generator().manual_seed(9)
    heat = cl(torch.randn(n, j, h, w, generator=g).to(dtype))
    heat[0, 0, 2, 3] = heat[0, 0, 4, 1] = 9.0            # a tie: the first in row-major order wins
    ref = O.heatmap_argmax(heat)
    out = K().heatmap_argmax(heat.cuda(), None)
    assert torch.equal(out.cpu(), ref)
    assert out[0, 0, 0].item() == 3 and out[0, 0, 1].item() == 2
    # second frame: only stream 1 changes; stream 0 keeps its previous row although its map is overwritten
    heat2 = heat.clone()
    heat2[1] = cl(torch.randn(1, j, h, w, generator=g).to(dtype))[0]
    heat2[0] = 0
    mask = torch.zeros(n, 1, h, w, dtype=torch.int32)
    mask[1, 0, h // 2, w // 2] = 1
    out2 = K().heatmap_argmax(heat2.cuda(), mask.cuda(), out.clone())
    ref2 = O.heatmap_argmax(heat2)
    assert torch.equal(out2.cpu()[1], ref2[1])
    assert torch.equal(out2.cpu()[0], ref[0])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,c,h,w,topk", [(2, 1, 34, 60, 100), (3, 3, 9, 11, 5), (1, 1, 136, 240, 100), (1, 2, 64, 64, 1024)])
def test_centernet_decode_matches_the_oracle(dtype, n, c, h, w, topk):
    g = torch.Generator().manual_seed(13)
    heat = cl((torch.randn(n, c, h, w, generator=g) * 2).to(dtype))
    wh = cl((torch.rand(n, 2, h, w, generator=g) * 8 + 1).to(dtype))
    off = cl(torch.rand(n, 2, h, w, generator=g).to(dtype))
    det_ref, cnt_ref = O.centernet_decode(heat, wh, off, topk, -1.0, 4.0, True)
    det, cnt, state = K().centernet_decode(heat.cuda(), wh.cuda(), off.cuda(), None, None, topk, -1.0, 4.0, True)
    assert torch.equal(cnt.cpu(), cnt_ref)
    assert torch.equal(det.cpu()[..., 5], det_ref[..., 5]), "classes / order differ"
    assert (det.cpu() - det_ref).abs().max().item() < 1e-3
    # second frame: a new peak in stream 0 near the corner, everything else unchanged; only stream 0 is re-decoded
    heat2 = heat.clone()
    heat2[0, 0, 1, 1] = 30.0
    mask = torch.zeros(n, 1, h, w, dtype=torch.int32)
    mask[0, 0, 1, 1] = 1
    poisoned = state[1].clone()
    if n > 1:
        poisoned[1:] = -123.0                            # rows of untouched streams must stay as they are
    det2, cnt2, _ = K().centernet_decode(heat2.cuda(), wh.cuda(), off.cuda(), mask.cuda(), (state[0], poisoned, state[2]), topk, -1.0, 4.0, True)
    ref2, cref2 = O.centernet_decode(heat2, wh, off, topk, -1.0, 4.0, True)
    assert torch.equal(cnt2.cpu()[:1], cref2[:1])
    assert (det2.cpu()[0] - ref2[0]).abs().max().item() < 1e-3
    assert det2[0, 0, 4].item() == pytest.approx(1.0, abs=1e-4)
    if n > 1:
        assert (det2[1:] == -123.0).all()


def test_centernet_decode_many_peaks_is_exact():
    """A checkerboard has more peaks than one sorting batch holds: the batches must merge to the exact top-k."""
    h, w = 128, 192
    yy, xx = torch.meshgrid(torch.arange(h), torch.arange(w), indexing="ij")
    g = torch.Generator().manual_seed(3)
    heat = torch.where(((yy % 2 == 0) & (xx % 2 == 0)), torch.rand(h, w, generator=g) + 1.0, torch.zeros(h, w))[None, None]
    heat = cl(heat.float())
    assert int((heat > 1).sum()) > 2048
    wh, off = cl(torch.ones(1, 2, h, w)), cl(torch.zeros(1, 2, h, w))
    det_ref, cnt_ref = O.centernet_decode(heat, wh, off, 100, 0.5, 1.0, False)
    det, cnt, _ = K().centernet_decode(heat.cuda(), wh.cuda(), off.cuda(), None, None, 100, 0.5, 1.0, False)
    assert torch.equal(cnt.cpu(), cnt_ref)
    assert torch.allclose(det.cpu(), det_ref, atol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("k", [3, 7, 15, 33])
@pytest.mark.parametrize("c", [3, 8])
def test_sparsify_dilated_matches_the_oracle(dtype, k, c):
    """Mask, cache and (dense) delta bit-exact against the reference's torch formulation, two frames in a row."""
    g = torch.Generator().manual_seed(21)
    n, h, w = 2, 45, 70
    prev = cl(torch.rand(n, c, h, w, generator=g).to(dtype))
    p_ref, pd = prev.clone(), prev.cuda()
    delta = torch.empty_like(pd)
    mask = torch.full((n, 1, h, w), -3, dtype=torch.int32, device="cuda")
    hit = torch.empty(n * h * w, dtype=torch.uint8, device="cuda")
    for t in range(2):
        x = prev + (0.004 * torch.randn(n, c, h, w, generator=g)).to(dtype)
        x[:, :, 10 + 5 * t:14 + 5 * t, 20:26] += 0.5
        x[0, :, 0, 0] += 0.5                              # a corner: the window is clipped
        x = cl(x)
        d_ref, m_ref = O.sparsify_dilated(x, p_ref, 0.1, k)
        K().sparsify_dilated(x.cuda(), pd, delta, mask, hit, 0.1, k)
        assert torch.equal(mask.cpu(), m_ref)
        assert torch.equal(pd.cpu(), p_ref)
        assert torch.equal(delta.cpu(), d_ref)
        assert 0 < int(m_ref.sum()) < m_ref.numel()
        prev = x


def test_dcsparsify_dilation_module_uses_the_kernel():
    from deltacnn_b200 import DCSparsify
    g = torch.Generator().manual_seed(2)
    layer = DCSparsify(delta_threshold=0.2, dilation=5)
    x0 = cl(torch.rand(2, 3, 20, 24, generator=g)).cuda()
    d0, m0 = layer(x0)
    assert bool((m0 == 1).all())
    x1 = x0.clone()
    x1[:, :, 9, 11] += 0.6
    d1, m1 = layer(x1)
    expect = torch.zeros(2, 1, 20, 24, dtype=torch.int32)
    expect[:, :, 7:12, 9:14] = 1
    assert torch.equal(m1.cpu(), expect)
    assert torch.equal(layer.prev_in[:, :, 9, 11], x1[:, :, 9, 11])
    assert layer._hit is not None


@pytest.mark.parametrize("dtype", DTYPES)
def test_sparsify_u8_matches_the_oracle(dtype):
    """8-bit ingest against the oracle directly: the oracle sparsifies the normalised frame."""
    g = torch.Generator().manual_seed(31)
    n, h, w = 2, 33, 40
    f0 = torch.randint(0, 256, (n, h, w, 3), generator=g, dtype=torch.uint8)
    f1 = f0.clone()
    f1[:, 4:9, 10:30] = torch.randint(0, 256, (n, 5, 20, 3), generator=g, dtype=torch.uint8)
    scale = torch.tensor([1 / 255.0, 1 / 200.0, 1 / 255.0])
    offset = torch.tensor([0.0, -0.1, 0.2])
    norm = lambda f: cl((f.float() * scale + offset).to(dtype).permute(0, 3, 1, 2))
    p_ref = norm(f0).clone()
    d_ref, m_ref = torch.zeros_like(p_ref), torch.zeros(n, 1, h, w, dtype=torch.int32)
    O.sparsify(norm(f1), p_ref, d_ref, m_ref, 0.03)
    pd = norm(f0).cuda()
    dd = torch.full_like(pd, float("nan"))
    md = torch.full((n, 1, h, w), -7, dtype=torch.int32, device="cuda")
    K().sparsify_u8(f1.cuda(), scale.cuda(), offset.cuda(), pd, dd, md, 0.03)
    assert torch.equal(md.cpu(), m_ref)
    assert torch.equal(pd.cpu(), p_ref)
    sel = (m_ref != 0).expand_as(d_ref)
    assert torch.equal(dd.cpu()[sel], d_ref[sel])
    assert 0 < int(m_ref.sum()) < m_ref.numel()
