"""Operator modes and module paths beyond the five benchmark networks: 5x5 pooling windows, x16 upsampling,
pooling with (top, bottom, left, right) padding, un-folded BatchNorm (the layout of the reference's own example
network), a resolution change in the middle of a stream, and the telescoping of the max-pool cache over many
frames. Oracle comparisons follow tests/test_ops_gpu.py: masks exact, values within 1e-4 (fp32) / 1e-2 (fp16)
of max |reference|."""
import pytest
import torch
import torch.nn as nn

from oracle import delta_ops as O

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16]
TOL = {torch.float32: 1e-4, torch.float16: 1e-2}


def K():
    import deltacnn_b200.cuda_kernels as k
    return k


def cl(t):
    return t.contiguous(memory_format=torch.channels_last)


def _close(got, ref, mask, dtype, what):
    sel = (mask != 0).expand_as(ref)
    if sel.sum() == 0:
        return
    r, g_ = ref.float()[sel], got.float().cpu()[sel]
    err = (g_ - r).abs().max().item() / max(r.abs().max().item(), 1e-6)
    assert err <= TOL[dtype], f"{what}: relative error {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("k,s,p,c", [(5, 1, 2, 16), (5, 2, 2, 24), (5, 5, 0, 7), (3, 3, 0, 8)])
def test_max_pool_larger_windows(dtype, k, s, p, c):
    g = torch.Generator().manual_seed(41)
    n, h, w = 2, 20, 25
    x = cl(torch.randn(n, c, h, w, generator=g).to(dtype))
    prev = cl(torch.randn(n, c, h, w, generator=g).to(dtype))
    m = (torch.rand(n, 1, h, w, generator=g) < 0.15).to(torch.int32)
    ref, m_ref = O.max_pool(x, m, prev, (k, k), (s, s), (p, p))
    p_ref = prev.clone()
    O.add_to_dense(x, p_ref, m)
    pd = prev.cuda()
    out, om = K().sparse_pooling(x.cuda(), pd, (k, k), m.cuda(), (s, s), (p, p), (1, 1), update_prev=True)
    assert torch.equal(om.cpu(), m_ref)
    _close(out, ref, m_ref, dtype, "maxpool")
    assert torch.equal(pd.cpu(), p_ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pad", [(0, 1, 0, 1), (1, 0, 1, 0), (0, 2, 1, 1), (1, 1, 0, 1)])
def test_max_pool_with_four_sided_padding(dtype, pad):
    """(top, bottom, left, right) padding: the reference lets a literal 0 join windows that reach into the bottom /
    right padding when it differs from the top / left padding (src/cuda/other_nn_layers.cu:2402-2422). With
    negative inputs that zero decides the result, so the case is not vacuous."""
    g = torch.Generator().manual_seed(43)
    n, c, h, w = 2, 8, 11, 13
    x = cl((torch.randn(n, c, h, w, generator=g) * 0.3).to(dtype))
    prev = cl((torch.randn(n, c, h, w, generator=g) - 1.5).to(dtype))         # mostly negative: the padded zero wins at the border
    m = (torch.rand(n, 1, h, w, generator=g) < 0.3).to(torch.int32)
    ref, m_ref = O.max_pool(x, m, prev, (3, 3), (2, 2), pad)
    out, om = K().sparse_pooling(x.cuda(), prev.cuda(), (3, 3), m.cuda(), (2, 2), pad, (1, 1), update_prev=False)
    assert tuple(out.shape) == tuple(ref.shape)
    assert torch.equal(om.cpu(), m_ref)
    _close(out, ref, m_ref, dtype, f"maxpool pad {pad}")
    # the oracle itself against torch: pad with zeros where the reference does, then pool the accumulated input
    pt, pb, pl, pr = pad
    acc = prev.float() + x.float() * (m != 0).float()
    full = lambda t: torch.nn.functional.max_pool2d(torch.nn.functional.pad(t, (pl, pr, pt, pb), value=0.0), 3, 2)
    if pt == 0 and pl == 0:      # only bottom/right padding: identical to zero padding followed by pooling
        want = (full(acc) - full(prev.float()))
        sel = (m_ref != 0).expand_as(ref)
        assert (ref.float()[sel] - want[sel]).abs().max().item() <= TOL[dtype] * max(want.abs().max().item(), 1.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_upsample_x16(dtype):
    g = torch.Generator().manual_seed(45)
    x = cl(torch.randn(2, 24, 3, 4, generator=g).to(dtype))
    m = (torch.rand(2, 1, 3, 4, generator=g) < 0.5).to(torch.int32)
    ref, m_ref = O.upsample(x, m, 16)
    out, om = K().sparse_upsample(x.cuda(), m.cuda(), 16)
    assert tuple(out.shape) == (2, 24, 48, 64)
    assert torch.equal(om.cpu().view_as(m_ref), m_ref)
    sel = (m_ref != 0).expand_as(ref)
    assert torch.equal(out.cpu()[sel], ref[sel])


def test_max_pool_cache_telescopes_in_fp16():
    """fp16, 40 frames: the sum of the delta max-pool's outputs (summed in fp32 here) equals the dense max-pool of the
    accumulated input cache up to the rounding of each output delta. The kernel pools the value the cache will
    hold after the frame (rounded to half), so consecutive frames' terms cancel exactly; pooling the unrounded sum
    would leave half an ulp of the cache value (about 1e-3 here) behind on every frame."""
    from deltacnn_b200 import DCMaxPooling
    g = torch.Generator().manual_seed(47)
    n, c, h, w = 2, 16, 24, 24
    pool = DCMaxPooling(3, 2, 1)
    acc = None
    for t in range(40):
        d = cl((torch.randn(n, c, h, w, generator=g) * (2.0 if t == 0 else 0.05)).half())
        m = torch.ones(n, 1, h, w, dtype=torch.int32) if t == 0 else (torch.rand(n, 1, h, w, generator=g) < 0.3).to(torch.int32)
        out, om = pool((d.cuda(), m.cuda()))
        step = out.float() * (om != 0).float()
        acc = step if acc is None else acc + step
    want = torch.nn.functional.max_pool2d(pool.prev_in.float(), 3, 2, 1)
    err = (acc - want).abs().max().item()
    assert err <= 1.5e-3, err


class _BNBlockDense(nn.Module):
    """conv -> BatchNorm -> ReLU6 blocks with BatchNorm left un-folded, as example/mobilenet_deltacnn.py:98,155."""

    def __init__(self):
        super().__init__()
        self.c1, self.b1 = nn.Conv2d(3, 16, 3, 2, 1, bias=False), nn.BatchNorm2d(16)
        self.c2, self.b2 = nn.Conv2d(16, 16, 3, 1, 1, groups=16, bias=False), nn.BatchNorm2d(16)
        self.c3, self.b3 = nn.Conv2d(16, 24, 1, bias=False), nn.BatchNorm2d(24)
        self.act = nn.ReLU6()

    def forward(self, x):
        x = self.act(self.b1(self.c1(x)))
        x = self.act(self.b2(self.c2(x)))
        return self.b3(self.c3(x))


def _bn_block_delta():
    from deltacnn_b200 import DCActivation, DCBatchNorm2d, DCConv2d, DCDensify, DCModule, DCSparsify

    class Net(DCModule):
        def __init__(self):
            super().__init__()
            self.sparsify = DCSparsify()
            self.c1, self.b1, self.a1 = DCConv2d(3, 16, 3, 2, 1, bias=False), DCBatchNorm2d(16), DCActivation(activation="relu6")
            self.c2, self.b2, self.a2 = DCConv2d(16, 16, 3, 1, 1, groups=16, bias=False), DCBatchNorm2d(16), DCActivation(activation="relu6")
            self.c3, self.b3 = DCConv2d(16, 24, 1, bias=False), DCBatchNorm2d(24)
            self.densify = DCDensify()

        def forward(self, x):
            x = self.sparsify(x)
            x = self.a1(self.b1(self.c1(x)))
            x = self.a2(self.b2(self.c2(x)))
            return self.densify(self.b3(self.c3(x)))

    return Net()


@pytest.mark.parametrize("dtype", DTYPES)
def test_unfolded_batchnorm_network_matches_dense(dtype):
    """DCBatchNorm2d on (delta, mask) tuples: scale on every frame, offset on the first only. Threshold 0 against
    the dense torch network with the same statistics, eight frames."""
    torch.manual_seed(3)
    dense = _BNBlockDense().eval()
    for bn in (dense.b1, dense.b2, dense.b3):
        bn.running_mean.normal_(0, 0.3)
        bn.running_var.uniform_(0.5, 2.0)
        bn.weight.data.uniform_(0.5, 1.5)
        bn.bias.data.normal_(0, 0.2)
    delta = _bn_block_delta()
    delta.load_state_dict(dense.state_dict())
    delta = delta.eval().to("cuda", memory_format=torch.channels_last)
    dense = dense.cuda()
    if dtype == torch.float16:
        delta = delta.half()
    delta.process_filters()
    g = torch.Generator().manual_seed(4)
    base = torch.rand(2, 3, 40, 48, generator=g)
    with torch.no_grad():
        for t in range(8):
            x = base.clone()
            x[:, :, 5 + 2 * t:15 + 2 * t, 10:30] = torch.rand(2, 3, 10, 20, generator=g)
            x = cl(x).cuda()
            ref = dense(x)
            got = delta(x.to(dtype))
            err = (got.float() - ref).abs().max().item() / ref.abs().max().item()
            assert err <= TOL[dtype], f"frame {t}: {err:.3e}"
    assert not delta.b1.first_iter and delta.b1.scale is not None


def test_resolution_change_needs_reset_and_then_matches_dense():
    """A stream that changes resolution: after reset_layers() the next frame is a first frame at the new size and the
    network matches the dense one again; without the reset the stale caches are refused instead of being indexed with
    the new geometry."""
    from examples.nets import build_pair
    from examples.synthetic_video import make_video
    frames = make_video("mobilenet", 5).frames(6)
    dense, delta = build_pair("mobilenet", frames[:4], device="cuda")
    small = lambda t: cl(frames[t:t + 1, :, :160, :192]).cuda()
    large = lambda t: cl(frames[t:t + 1]).cuda()
    rel = lambda a, b: (a - b).abs().max().item() / b.abs().max().item()
    with torch.no_grad():
        for t in range(3):
            assert rel(delta(small(t)), dense(small(t))) <= 1e-4
        with pytest.raises(RuntimeError, match="reset_layers"):
            delta(large(3))
        delta.reset_layers()
        for t in range(3, 6):
            assert rel(delta(large(t)), dense(large(t))) <= 1e-4
