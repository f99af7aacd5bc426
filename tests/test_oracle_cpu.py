"""CPU checks of the oracle: at threshold 0 the CPU delta network equals the dense network on every
frame (the identity that pins the layer lifecycle), and thresholds make it sparse but bounded."""
import torch

from examples.nets import build_pair
from examples.synthetic_video import make_video
from oracle import delta_ops as O
from oracle.delta_net import Thresholds, build_oracle_net


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(b.float().abs().max().item(), 1e-12)


def test_mobilenet_oracle_threshold0_equals_dense():
    frames = make_video("mobilenet", 0).frames(5)
    dense, _ = build_pair("mobilenet", frames[:4], device="cpu")
    net = build_oracle_net("mobilenet", dense.state_dict())
    with torch.no_grad():
        for t in range(5):
            assert _rel(net(frames[t:t + 1]), dense(frames[t:t + 1])) < 1e-4


def test_small_networks_oracle_threshold0_equals_dense():
    torch.manual_seed(0)
    for name, size, kw in (("resnet50", (64, 64), dict(blocks=(1, 1, 1, 1))), ("centernet", (64, 96), {}),
                           ("hrnet", (64, 64), dict(blocks_per_branch=1, modules=(1, 1, 2)))):
        frames = make_video("mobilenet", 1).frames(3)[:, :, :size[0], :size[1]].contiguous()
        dense, _ = build_pair(name, frames, device="cpu", **kw)
        net = build_oracle_net(name, dense.state_dict(), **kw)
        with torch.no_grad():
            for t in range(3):
                ref, got = dense(frames[t:t + 1]), net(frames[t:t + 1])
                ref = ref if isinstance(ref, tuple) else (ref,)
                got = got if isinstance(got, tuple) else (got,)
                for r, g in zip(ref, got):
                    assert _rel(g, r) < 1e-4, name


def test_thresholds_give_sparse_masks_and_bounded_error():
    frames = make_video("mobilenet", 2).frames(6)
    dense, _ = build_pair("mobilenet", frames[:4], device="cpu")
    net = build_oracle_net("mobilenet", dense.state_dict())
    with torch.no_grad():
        net(frames[0:1])
        Thresholds.set_depth_table(0.05, 0.01, 0.05)
        assert len(Thresholds.table) == 36          # 1 sparsify + 35 activation sites
        for t in range(1, 6):
            out = net(frames[t:t + 1])
            ref = dense(frames[t:t + 1])
        density = net.sparsify.prev_in is not None
        assert density
        assert _rel(out, ref) < 0.5


def test_sparsify_semantics_small_case():
    x = torch.tensor([[[[1.0, 2.0]], [[0.0, 0.0]], [[0.0, 0.5]]]])        # N=1,C=3,H=1,W=2
    prev = torch.zeros_like(x)
    prev[0, :, 0, 1] = torch.tensor([1.95, 0.0, 0.48])
    delta = torch.full_like(x, -9.0)
    mask = torch.zeros(1, 1, 1, 2, dtype=torch.int32)
    O.sparsify(x, prev, delta, mask, 0.05)
    assert mask.flatten().tolist() == [1, 0]         # |2-1.95| = 0.05 is not > 0.05 (strict compare)
    assert delta[0, :, 0, 0].tolist() == [1.0, 0.0, 0.0] and delta[0, :, 0, 1].tolist() == [-9.0] * 3
    assert prev[0, :, 0, 0].tolist() == [1.0, 0.0, 0.0] and abs(prev[0, 0, 0, 1].item() - 1.95) < 1e-6


def test_truncation_carries_residual_forward():
    d = torch.full((1, 2, 1, 1), 0.03)
    y = torch.ones(1, 2, 1, 1)
    r = torch.zeros(1, 2, 1, 1)
    for step in range(3):
        delta, mask = d.clone(), torch.ones(1, 1, 1, 1, dtype=torch.int32)
        O.activate_truncate(delta, y, r, mask, 0.05, O.ACT_RELU, O.TRUNC_MAX)
        if step == 0:
            assert mask.item() == 0 and abs(r[0, 0, 0, 0].item() - 0.03) < 1e-7 and y[0, 0, 0, 0].item() == 1.0
        if step == 1:     # 0.06 > 0.05: emitted, residual cleared, cache advanced
            assert mask.item() == 1 and r.abs().max().item() == 0 and abs(y[0, 0, 0, 0].item() - 1.06) < 1e-6
            assert abs(delta[0, 0, 0, 0].item() - 0.06) < 1e-6


def test_mask_dilation_property():
    g = torch.Generator().manual_seed(0)
    for k, s, p, d in ((3, 1, 1, 1), (3, 2, 1, 1), (1, 2, 0, 1), (5, 1, 2, 1), (7, 2, 3, 1), (3, 1, 2, 2)):
        m = (torch.rand(2, 1, 11, 13, generator=g) < 0.1).to(torch.int32)
        om = O.dilate_mask(m, (k, k), (s, s), (p, p), (d, d))
        # brute force
        ho, wo = O.conv_out_size(11, 13, (k, k), (s, s), (p, p), (d, d))
        want = torch.zeros(2, 1, ho, wo, dtype=torch.int32)
        for b in range(2):
            for oy in range(ho):
                for ox in range(wo):
                    for ky in range(k):
                        for kx in range(k):
                            iy, ix = oy * s - p + ky * d, ox * s - p + kx * d
                            if 0 <= iy < 11 and 0 <= ix < 13 and m[b, 0, iy, ix]:
                                want[b, 0, oy, ox] = 1
        assert torch.equal(om, want)


def _tmap(f, x):
    """``f`` applied to every tensor of a nested list / tuple structure."""
    return f(x) if torch.is_tensor(x) else type(x)(_tmap(f, v) for v in x)


def _tlist(x):
    return [x] if torch.is_tensor(x) else [t for v in x for t in _tlist(v)]


def _pipeline_cases():
    pool2 = lambda f: torch.nn.functional.avg_pool2d(f, 2)
    return [("mobilenet", pool2(make_video("mobilenet", 3).frames(9)), {}, [5, 9, 13]),
            ("hrnet", make_video("hrnet", 3).frames(7)[:, :, 96:160, 96:160].contiguous(), dict(blocks_per_branch=1, modules=(1, 1, 2)), [2, 4, 6]),
            ("centernet", pool2(pool2(make_video("mobilenet", 4).frames(7)))[:, :, :32, :32].contiguous() * 1.0, {}, [3, 7, 9])]


def test_frame_pipeline_over_the_depth_is_exact_on_the_oracle():
    """The frame pipeline of deltacnn_b200/stepping.py rests on two properties of the delta algorithm, checked here on
    the CPU restatement: a layer that receives an all-zero mask changes nothing and emits an all-zero mask, and a stage
    that sees the deltas of its predecessor one step late produces the same sequence of states. Stage s of a step
    works on what stage s-1 produced in the step before; the outputs of frame t leave the last stage len(cuts) steps
    later, bit for bit (MobileNetV2; HRNet, whose stages hand lists of branch tensors on; CenterNet with its three heads)."""
    import copy
    for name, frames, kw, cuts in _pipeline_cases():
        n = frames.shape[0]
        dense, _ = build_pair(name, frames[:4], device="cpu", **kw)
        net = build_oracle_net(name, dense.state_dict(), **kw)
        with torch.no_grad():
            net(frames[0:1])
            Thresholds.set_depth_table(0.05, 0.01, 0.05)
            net(frames[1:2])
            twin = copy.deepcopy(net)                               # same weights, caches and thresholds
            for a, b in zip(net.modules(), twin.modules()):
                if a in Thresholds.table:
                    Thresholds.table[b] = Thresholds.table[a]
            clone = lambda y: _tmap(torch.clone, y)
            same = lambda p, q: all(torch.equal(u, v) for u, v in zip(_tlist(p), _tlist(q)))
            want = [clone(net(frames[t:t + 1])) for t in range(1, n)]        # frame 1 again (zero delta), then frames 2..
            assert not same(want[0], want[-1]), f"{name}: the frames must change the output for this test to mean anything"
            stages = twin.depth_stages(cuts)
            # what lies between the stages: learnt from a pass over the frame seen last (zero delta), then all zeros
            x, between = frames[1:2], []
            for stage in stages[:-1]:
                x = stage(x)
                between.append(_tmap(torch.zeros_like, x))
            assert same(stages[-1](x), want[0]), f"{name}: a zero delta must change nothing"
            got = []
            for x in [frames[t:t + 1] for t in range(2, n)] + [frames[n - 1:n]] * len(cuts):
                new = list(between)
                for s, stage in enumerate(stages):
                    y = stage(x if s == 0 else between[s - 1])
                    if s < len(stages) - 1:
                        new[s] = clone(y)
                    else:
                        got.append(clone(y))
                between = new
        for k in range(len(cuts)):                                   # the pipeline fills: the outputs of frame 1 stay
            assert same(got[k], want[0]), name
        for t in range(2, n):                                        # frame t leaves len(cuts) steps after it entered
            assert same(got[t - 2 + len(cuts)], want[t - 1]), (name, t)
