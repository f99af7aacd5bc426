"""The CPU oracle against fixtures recorded from the reference's own CUDA kernels
(tests/golden/ref_ops.npz, written by tests/golden/make_golden.py on a B200). Masks and every
state tensor of the element-wise operators must be bit-exact; convolution values are compared at
out-mask pixels within a tolerance (the reference accumulates fp16 convolutions in fp16)."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from golden.make_golden import cases  # noqa: E402
from oracle import delta_ops as O  # noqa: E402

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_ops.npz"))
CASES = cases()


def gold(name, key, like=None):
    a = torch.from_numpy(GOLD[f"{name}/{key}"].astype(np.float32) if GOLD[f"{name}/{key}"].dtype != np.int32 else GOLD[f"{name}/{key}"])
    return a


def close_at(got, ref, mask, tol):
    sel = (mask != 0).expand_as(ref)
    if sel.sum() == 0:
        return
    r, g = ref.float()[sel], got.float()[sel]
    err = (g - r).abs().max().item() / max(r.abs().max().item(), 1e-6)
    assert err <= tol, f"relative error {err:.3e} > {tol}"


def test_every_recorded_case_is_checked():
    recorded = {k.split("/")[0] for k in GOLD.files}
    assert recorded == set(CASES), "fixture file and case list are out of step: re-run tests/golden/make_golden.py"


@pytest.mark.parametrize("name", [n for n in CASES if CASES[n]["op"] == "sparsify"])
def test_sparsify_bit_exact(name):
    c = CASES[name]
    prev, delta, mask = c["prev"].clone(), torch.zeros_like(c["x"]), torch.zeros(c["x"].shape[0], 1, *c["x"].shape[2:], dtype=torch.int32)
    O.sparsify(c["x"], prev, delta, mask, c["thr"])
    m_ref = gold(name, "mask")
    assert torch.equal(mask, m_ref)
    assert torch.equal(prev.float(), gold(name, "prev"))
    sel = (m_ref != 0).expand_as(delta)
    assert torch.equal(delta.float()[sel], gold(name, "delta")[sel])


def _exact_act(c):
    """Cases whose arithmetic has one correctly rounded result: max-truncation (or none) with identity, ReLU, ReLU6 or
    fp32 leaky ReLU. Sigmoid / swish go through exp (the reference uses the fast and the half intrinsics), the half
    leaky ReLU multiplies by 0.1 rounded to half (src/cuda/other_nn_layers.cu:57-60) and norm / rms sum the channels in
    another order, so those are compared with a tolerance."""
    half = c["delta"].dtype == torch.float16
    return c["mode"] <= 0 and (c["act"] <= 2 or (c["act"] == 3 and not half))


@pytest.mark.parametrize("name", [n for n in CASES if CASES[n]["op"] == "act" and _exact_act(CASES[n])])
def test_activation_truncation_bit_exact(name):
    c = CASES[name]
    d, p, m = c["delta"].clone(), c["prev"].clone(), c["mask"].clone()
    t = None if c["trunc"] is None else c["trunc"].clone()
    O.activate_truncate(d, p, t, m, c["thr"], max(c["act"], 0), c["mode"])
    m_ref = gold(name, "mask")
    assert torch.equal(m, m_ref)
    assert torch.equal(p.float(), gold(name, "prev"))
    if t is not None:
        assert torch.equal(t.float(), gold(name, "trunc"))
    if c["act"] > 0 or c["mode"] >= 0:          # identity without truncation leaves the delta as it came
        sel = (m_ref != 0).expand_as(d)
        assert torch.equal(d.float()[sel], gold(name, "delta")[sel])


@pytest.mark.parametrize("name", [n for n in CASES if CASES[n]["op"] == "act" and not _exact_act(CASES[n])])
def test_activation_truncation_transcendental_and_norm_modes(name):
    c = CASES[name]
    half = name.endswith("f16")
    d, p, t, m = c["delta"].clone(), c["prev"].clone(), c["trunc"].clone(), c["mask"].clone()
    O.activate_truncate(d, p, t, m, c["thr"], c["act"], c["mode"])
    m_ref = gold(name, "mask")
    agree = (m == m_ref).float().mean().item()
    assert agree >= 0.99, f"mask agreement {agree}"
    assert 0 < int(m_ref.sum()) <= int(c["mask"].sum()), "the case must keep some pixels"
    same = (m == m_ref)
    both = ((m != 0) & (m_ref != 0)).expand_as(d)
    tol = 1e-2 if half else 1e-5          # half: both activations are evaluated in half arithmetic by the reference (one ulp of values up to 8)
    assert (d.float()[both] - gold(name, "delta")[both]).abs().max().item() <= tol
    sel = same.expand_as(p)
    assert (p.float()[sel] - gold(name, "prev")[sel]).abs().max().item() <= tol
    assert (t.float()[sel] - gold(name, "trunc")[sel]).abs().max().item() <= tol


@pytest.mark.parametrize("name", [n for n in CASES if CASES[n]["op"] in ("conv", "deconv")])
def test_convolutions(name):
    c = CASES[name]
    if c["op"] == "conv":
        out, om = O.conv(c["x"], c["mask"], c["w"], c["b"], c["s"], c["p"], (1, 1), c["groups"])
    else:
        out, om = O.deconv(c["x"], c["mask"], c["w"], c["b"], c["s"], c["p"])
    m_ref = gold(name, "mask")
    assert torch.equal(om, m_ref), "out-mask differs from the reference kernels"
    close_at(out, gold(name, "out"), m_ref, 1e-4 if name.endswith("f32") else 3e-2)


@pytest.mark.parametrize("name", [n for n in CASES if CASES[n]["op"] in ("add", "maxpool", "upsample")])
def test_other_ops(name):
    c = CASES[name]
    half = name.endswith("f16")
    if c["op"] == "add":
        prev = c["prev"].clone() if "prev" in c else None
        out, om = O.add(c["a"], c["ma"], c["b"], c["mb"], prev, c["wa"], c["wb"], c["act"], c.get("dense", False))
        if prev is not None:
            assert (prev.float() - gold(name, "prev")).abs().max().item() <= 1e-6
        if c.get("dense", False):               # dense output: f(prev_out) at every pixel, no out-mask
            assert (out.float() - gold(name, "out")).abs().max().item() <= 1e-6
            return
    elif c["op"] == "maxpool":
        out, om = O.max_pool(c["x"], c["mask"], c["prev"], c["k"], c["s"], c["p"])
    else:
        out, om = O.upsample(c["x"], c["mask"], c["scale"])
    m_ref = gold(name, "mask")
    assert torch.equal(om.view_as(m_ref), m_ref)
    close_at(out, gold(name, "out"), m_ref, 2e-3 if half else 1e-6)


@pytest.mark.parametrize("name", [n for n in CASES if CASES[n]["op"] in ("gap", "add_to_dense", "concat", "mul_add")])
def test_remaining_ops(name):
    c = CASES[name]
    half = name.endswith("f16")
    if c["op"] == "gap":
        out, om = O.global_avg_pool(c["x"], c["mask"])
        assert torch.equal(om.view(-1), gold(name, "mask").view(-1))
        # the reference sums with float atomics (any order) and rounds once at the end
        ref = gold(name, "out").view_as(out)
        assert (out.float() - ref).abs().max().item() <= (2e-3 if half else 1e-6) * max(ref.abs().max().item(), 1e-6)
    elif c["op"] == "add_to_dense":
        b = c["b"].clone()
        O.add_to_dense(c["a"], b, c["ma"])
        assert torch.equal(b.float(), gold(name, "b"))
    elif c["op"] == "concat":
        out, om = O.concatenate(c["a"], c["ma"], c["b"], c["mb"])
        m_ref = gold(name, "mask")
        assert torch.equal(om, m_ref)
        sel = (m_ref != 0).expand_as(out)
        assert torch.equal(out.float()[sel], gold(name, "out")[sel])
    else:
        # the reference kernel never writes its mask_out argument (src/cuda/other_nn_layers.cu:3774-3818: the module passes
        # the in-mask for both), so only the values at masked pixels are pinned
        out, om = O.scale_bias(c["x"], c["mask"], c["scale"], c["bias"])
        assert torch.equal(om, c["mask"]) and int(gold(name, "mask").sum()) == 0
        close_at(out, gold(name, "out"), c["mask"], 2e-3 if half else 1e-6)
