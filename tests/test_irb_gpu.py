"""The fused inverted-residual block kernel (dc_irb_fused) against the chain of separate operator calls it replaces
(expansion with fused truncation, depthwise with fused truncation, projection with the residual add): outputs at the
out-mask, the out-mask and all four truncation caches must be identical bit for bit, frame after frame; and against
the CPU oracle within the half-precision tolerance of the operator tests. Network level: MobileNetV2 with and without
the fused blocks gives identical logits at the benchmark's thresholds."""
import pytest
import torch

from oracle import delta_ops as O

pytestmark = pytest.mark.gpu

# (c_in, c_hidden, c_out, h, w, stride, residual)
BLOCKS = [
    (64, 384, 64, 14, 14, 1, True),
    (64, 384, 96, 14, 14, 1, False),
    (96, 576, 96, 14, 14, 1, True),
    (96, 576, 160, 14, 14, 2, False),
    (160, 960, 160, 7, 7, 1, True),
    (160, 960, 320, 7, 7, 1, False),
    (32, 64, 32, 10, 12, 1, True),           # two uneven bands, one K block, narrow N
    (24, 128, 48, 9, 5, 2, False),           # odd sizes, stride 2
]


def cl(t):
    return t.contiguous(memory_format=torch.channels_last)


def _packed(kk, lib, w_hwio, cin, cout):
    desc = kk.make_conv_desc((1, cin, 8, 8), cout, (8, 8), (1, 1), (1, 1), (0, 0), (1, 1), 1, 1)
    packed = torch.zeros(lib.lib.dc_filter_umma_bytes(desc, 0), dtype=torch.uint8, device="cuda")
    lib.check(lib.lib.dc_pack_filter_umma(desc, 0, w_hwio.data_ptr(), packed.data_ptr(), torch.cuda.current_stream().cuda_stream), "pack")
    return packed


class _Block:
    """Weights, caches and both execution forms of one block."""

    def __init__(self, g, n, cin, chid, cout, h, w, stride, residual):
        import deltacnn_b200.cuda_kernels as kk
        from deltacnn_b200 import _lib
        from deltacnn_b200.filter_conversion import convert_filter_out_channels_last as hwio
        self.kk, self.geom = kk, (n, cin, chid, cout, h, w, stride, residual)
        self.ho, self.wo = (h - 1) // stride + 1, (w - 1) // stride + 1
        self.w1 = (torch.randn(chid, cin, 1, 1, generator=g) * cin ** -0.5).half()
        self.wd = (torch.randn(chid, 1, 3, 3, generator=g) * 0.4).half()
        self.w2 = (torch.randn(cout, chid, 1, 1, generator=g) * chid ** -0.5).half()
        self.f1, self.fd, self.f2 = hwio(self.w1).cuda(), hwio(self.wd).cuda(), hwio(self.w2).cuda()
        self.p1, self.p2 = _packed(kk, _lib, self.f1, cin, chid), _packed(kk, _lib, self.f2, chid, cout)
        self.caches0 = [cl(torch.randn(n, chid, h, w, generator=g).half()), cl((torch.randn(n, chid, h, w, generator=g) * 0.01).half()),
                        cl(torch.randn(n, chid, self.ho, self.wo, generator=g).half()), cl((torch.randn(n, chid, self.ho, self.wo, generator=g) * 0.01).half())]
        # a few cache residuals exactly zero, as after a frame in which the pixel was active
        self.caches0[1][:, :, ::2] = 0
        self.caches0[3][:, :, ::2] = 0
        self.thr = (0.35, 0.3)
        self.inner = None          # (mask after the expansion's truncation, after the depthwise truncation) of the last separate() call

    def fresh(self):
        return [c.clone().cuda() for c in self.caches0]

    def separate(self, x, m, caches):
        kk = self.kk
        n, cin, chid, cout, h, w, s, res = self.geom
        pe, te, pd, td = caches
        a, ma = kk.sparse_conv(x, self.f1, m, None, (1, 1), (0, 0), (1, 1), 1, create_out_mask=True, filter_umma=self.p1,
                               epilogue=kk.make_epilogue(pe, te, self.thr[0], 2, 0))
        b, mb = kk.sparse_conv(a, self.fd, ma, None, (s, s), (1, 1), (1, 1), chid, create_out_mask=True,
                               epilogue=kk.make_epilogue(pd, td, self.thr[1], 2, 0))
        self.inner = (ma.clone(), mb.clone())
        ep = kk.make_residual_epilogue(x, m) if res else None
        return kk.sparse_conv(b, self.f2, mb, None, (1, 1), (0, 0), (1, 1), 1, create_out_mask=True, filter_umma=self.p2, epilogue=ep)

    def fused(self, x, m, caches):
        kk = self.kk
        n, cin, chid, cout, h, w, s, res = self.geom
        desc = kk.make_irb_desc(tuple(x.shape), chid, cout, s, res, 2, 2, self.thr[0], self.thr[1])
        assert kk.irb_supported(desc)
        out = torch.full((n, cout, self.ho, self.wo), float("nan"), dtype=torch.float16, device="cuda").contiguous(memory_format=torch.channels_last)
        mo = torch.full((n, 1, self.ho, self.wo), -9, dtype=torch.int32, device="cuda")
        return kk.fused_inverted_residual(x, m, self.p1, self.fd, self.p2, *caches, out, mo, desc)

    def oracle(self, x, m, caches):
        n, cin, chid, cout, h, w, s, res = self.geom
        pe, te, pd, td = caches
        a, ma = O.conv(x, m, self.w1, None, (1, 1), (0, 0), (1, 1), 1)
        O.activate_truncate(a, pe, te, ma, self.thr[0], 2, 0)
        b, mb = O.conv(a, ma, self.wd, None, (s, s), (1, 1), (1, 1), chid)
        O.activate_truncate(b, pd, td, mb, self.thr[1], 2, 0)
        c, mc = O.conv(b, mb, self.w2, None, (1, 1), (0, 0), (1, 1), 1)
        if res:
            c, mc = O.add(c, mc, x, m, None)
        return c, mc


@pytest.mark.parametrize("geom", BLOCKS, ids=lambda g: "x".join(str(v) for v in g))
@pytest.mark.parametrize("density", [1.0, 0.5])
def test_fused_block_equals_separate_calls_and_oracle(geom, density):
    from deltacnn_b200 import _lib
    cin, chid, cout, h, w, s, res = geom
    g = torch.Generator().manual_seed(11)
    n = 3
    blk = _Block(g, n, cin, chid, cout, h, w, s, res)
    c_sep, c_fus, c_ref = blk.fresh(), blk.fresh(), [c.clone() for c in blk.caches0]
    kept, dropped = 0, 0
    for frame in range(3):
        blk.thr = ((0.35, 0.3), (0.85, 0.5), (0.95, 0.7))[frame]      # from "nearly every pixel passes" to a mix of kept and dropped pixels
        x = cl((torch.randn(n, cin, h, w, generator=g) * (0.6 if frame == 0 else 0.3)).half())
        m = (torch.rand(n, 1, h, w, generator=g) < density).to(torch.int32)
        if density < 1.0:
            m[2] = 0                                              # a stream without any update
            m[1, :, :2] = 0
        xs = torch.where((m != 0).expand_as(x), x, torch.full_like(x, float("nan")))       # inactive pixels must never be read
        o1, m1 = blk.separate(xs.cuda(), m.cuda(), c_sep)
        o2, m2 = blk.fused(xs.cuda(), m.cuda(), c_fus)
        torch.cuda.synchronize()
        assert _lib.lib.dc_umma_error() == 0
        for inner, full in zip(blk.inner, (m, None)):
            kept += int(inner.sum())
            dropped += int((full.cuda() != 0).sum() - inner.sum()) if full is not None else 0
        assert torch.equal(m1, m2), f"frame {frame}: out-mask differs"
        for name, a, b in zip(("prev_expand", "trunc_expand", "prev_dw", "trunc_dw"), c_sep, c_fus):
            assert torch.equal(a, b), f"frame {frame}: {name} differs ({int((a != b).sum())} elements)"
        sel = (m1 != 0).expand_as(o1)
        assert torch.equal(o1[sel], o2[sel]), f"frame {frame}: values differ"
        assert torch.isnan(o2[~sel]).all(), "pixels outside the out-mask must not be written"
        if density == 1.0:
            assert int(m1.sum()) > 0
        # CPU oracle: fp32 accumulation order differs, so pixels next to a threshold flip (the thresholds of frames 1 and 2
        # sit in the middle of the distribution on purpose) and a flipped pixel changes its neighbours' inputs downstream
        o_ref, m_ref = blk.oracle(x * (m != 0), m, c_ref)
        agree = (m2.cpu() == m_ref).float().mean().item()
        assert agree >= 0.9, f"frame {frame}: out-mask agreement with the oracle {agree}"
        both = ((m2.cpu() != 0) & (m_ref != 0)).expand_as(o_ref)
        if both.any():
            err = (o2.cpu().float()[both] - o_ref.float()[both]).abs()
            assert err.median().item() < 5e-3 and (err > 0.1).float().mean().item() < 0.05, f"frame {frame}: values differ from the oracle"
    assert kept > 0 and dropped > 0, "the case must exercise both outcomes of the truncation decision"


def test_unsupported_shapes_are_refused_not_run():
    import deltacnn_b200.cuda_kernels as kk
    for shape, chid, cout, s, res in (((2, 32, 28, 28), 192, 32, 1, True),      # too many bands
                                      ((2, 64, 14, 14), 384, 64, 2, True),      # residual with stride 2
                                      ((2, 64, 14, 14), 100, 64, 1, False),     # hidden channels not a multiple of 64
                                      ((2, 64, 14, 14), 2048, 64, 1, False)):   # too wide
        assert not kk.irb_supported(kk.make_irb_desc(shape, chid, cout, s, res, 2, 2, 0.1, 0.1))


def test_mobilenet_with_fused_blocks_equals_unfused():
    """MobileNetV2 fp16, two streams, benchmark thresholds: the network with its ten small-map blocks in the fused
    kernel and the network with separate layer kernels give identical logits on every frame."""
    from deltacnn_b200 import DCConv2d, DCThreshold
    from examples.nets import build_pair
    from deltacnn_b200.stepping import set_depth_thresholds
    from examples.synthetic_video import make_video
    frames = make_video("mobilenet", 4).frames(7)
    xs = [frames[t:t + 1].cuda().half().repeat(2, 1, 1, 1).contiguous(memory_format=torch.channels_last) for t in range(7)]
    xs[3][1] = xs[2][1]                                           # stream 1 stands still for a frame
    outs, used = {}, {}
    try:
        for fused in (True, False):
            DCConv2d.fuse_blocks = fused
            DCThreshold.reset()
            _, delta = build_pair("mobilenet", frames[:4], device="cuda", dtype=torch.float16)
            with torch.no_grad():
                delta(xs[0])
                set_depth_thresholds(0.05, 0.01, 0.05)
                outs[fused] = [delta(x).clone() for x in xs[1:]]
            used[fused] = sum(1 for b in delta.features if getattr(b, "fused", None) is not None and b.fused._desc is not None)
    finally:
        DCConv2d.fuse_blocks = False
    assert used[True] == 10 and used[False] == 0
    for t, (a, b) in enumerate(zip(outs[True], outs[False])):
        assert torch.equal(a, b), f"frame {t + 1}"
