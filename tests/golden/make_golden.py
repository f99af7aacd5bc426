"""Records fixtures from the REFERENCE's own CUDA kernels (through oracle/_ref) for seeded inputs.

Run on a machine with a GPU after `make -C oracle`:   python tests/golden/make_golden.py
It writes tests/golden/ref_ops.npz: per case only the reference OUTPUTS (inputs are regenerated
from the seeds by `cases()` below, which the CPU test imports). The CPU test
tests/test_golden_cpu.py then checks the CPU oracle against these recordings.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_ops.npz")


def cl(t):
    return t.contiguous(memory_format=torch.channels_last)


def feat(g, n, c, h, w, dtype, scale=1.0):
    return cl((torch.randn(n, c, h, w, generator=g) * scale).to(dtype))


def mask(g, n, h, w, density):
    return (torch.rand(n, 1, h, w, generator=g) < density).to(torch.int32)


def cases():
    """name -> dict of CPU input tensors and parameters (deterministic)."""
    out = {}
    for dt_name, dtype in (("f32", torch.float32), ("f16", torch.float16)):
        g = torch.Generator().manual_seed(100)
        n, h, w = 2, 16, 20
        prev = feat(g, n, 3, h, w, dtype)
        x = prev.clone()
        upd = torch.rand(n, 1, h, w, generator=g) < 0.25
        x = cl(torch.where(upd.expand_as(x), feat(g, n, 3, h, w, dtype), x + (0.02 * torch.randn(n, 3, h, w, generator=g)).to(dtype)))
        out[f"sparsify_{dt_name}"] = dict(op="sparsify", x=x, prev=prev, thr=0.05)
        for act in (1, 2):
            c = 32
            out[f"act{act}_{dt_name}"] = dict(op="act", delta=feat(g, n, c, h, w, dtype, 0.05), prev=feat(g, n, c, h, w, dtype, 2.0),
                                              trunc=feat(g, n, c, h, w, dtype, 0.01), mask=mask(g, n, h, w, 0.5), thr=0.12, act=act, mode=0)
        out[f"add_{dt_name}"] = dict(op="add", a=feat(g, n, 24, h, w, dtype), b=feat(g, n, 24, h, w, dtype), ma=mask(g, n, h, w, 0.3),
                                     mb=mask(g, n, h, w, 0.3), wa=1.0, wb=1.0, act=0)
        out[f"maxpool_{dt_name}"] = dict(op="maxpool", x=feat(g, n, 16, h, w, dtype), prev=feat(g, n, 16, h, w, dtype),
                                         mask=mask(g, n, h, w, 0.2), k=(3, 3), s=(2, 2), p=(1, 1))
        out[f"upsample_{dt_name}"] = dict(op="upsample", x=feat(g, n, 8, 6, 7, dtype), mask=mask(g, n, 6, 7, 0.4), scale=2)
        convs = {"stem3x3s2": (3, 32, 3, 2, 1, 1), "pw": (32, 64, 1, 1, 0, 1), "pw_s2": (32, 64, 1, 2, 0, 1), "c3x3": (32, 32, 3, 1, 1, 1),
                 "dw3x3": (32, 32, 3, 1, 1, 32), "dw3x3s2": (32, 32, 3, 2, 1, 32), "c7x7s2": (3, 16, 7, 2, 3, 1)}
        for name, (cin, cout, k, s, p, groups) in convs.items():
            if name == "c7x7s2" and dtype == torch.float16:
                continue
            wt = (torch.randn(cout, cin // groups, k, k, generator=g) / (k * (cin // groups) ** 0.5)).to(dtype)
            out[f"conv_{name}_{dt_name}"] = dict(op="conv", x=feat(g, n, cin, h, w, dtype), mask=mask(g, n, h, w, 0.12), w=wt,
                                                 b=torch.randn(cout, generator=g).to(dtype), s=(s, s), p=(p, p), groups=groups)
        wt = (torch.randn(32, 24, 4, 4, generator=g) * 0.1).to(dtype)
        out[f"deconv4x4s2_{dt_name}"] = dict(op="deconv", x=feat(g, n, 32, 8, 9, dtype), mask=mask(g, n, 8, 9, 0.15), w=wt,
                                             b=torch.randn(24, generator=g).to(dtype), s=(2, 2), p=(1, 1))
    return out


def run_reference(case):
    """Runs one case on the reference kernels; returns dict of numpy arrays."""
    from oracle import ref_kernels as R
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in case.items()}
    op = c["op"]
    f = lambda t: t.float().cpu().numpy() if t.dtype != torch.int32 else t.cpu().numpy()
    if op == "sparsify":
        prev = c["prev"].clone()
        d, m = R.sparsify(c["x"], prev, c["thr"])
        return dict(delta=f(d), mask=f(m), prev=f(prev))
    if op == "act":
        d, p, t, m = c["delta"].clone(), c["prev"].clone(), c["trunc"].clone(), c["mask"].clone()
        R.activate_truncate(d, p, t, m, c["thr"], c["act"], c["mode"])
        return dict(delta=f(d), prev=f(p), trunc=f(t), mask=f(m))
    if op == "add":
        o, m = R.add(c["a"], c["ma"], c["b"], c["mb"], None, c["wa"], c["wb"], c["act"], False)
        return dict(out=f(o), mask=f(m))
    if op == "maxpool":
        o, m = R.max_pool(c["x"], c["mask"], c["prev"], c["k"], c["s"], c["p"])
        return dict(out=f(o), mask=f(m))
    if op == "upsample":
        o, m = R.upsample(c["x"], c["mask"], c["scale"])
        return dict(out=f(o), mask=f(m))
    if op == "conv":
        o, m = R.conv(c["x"], c["mask"], c["w"], c["b"], c["s"], c["p"], (1, 1), c["groups"])
        return dict(out=f(o), mask=f(m))
    if op == "deconv":
        o, m = R.deconv(c["x"], c["mask"], c["w"], c["b"], c["s"], c["p"])
        return dict(out=f(o), mask=f(m))
    raise ValueError(op)


def main():
    blob = {}
    for name, case in cases().items():
        for k, v in run_reference(case).items():
            blob[f"{name}/{k}"] = v.astype(np.float16) if (v.dtype == np.float32 and name.endswith("f16")) else v
    np.savez_compressed(OUT, **blob)
    print(f"wrote {OUT}: {len(blob)} arrays, {os.path.getsize(OUT)} bytes")


if __name__ == "__main__":
    main()
