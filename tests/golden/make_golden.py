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
    out.update(more_cases())
    return out


def more_cases():
    """Second batch of cases (own generators, so the first batch keeps its inputs): the operators and modes the
    first batch left unpinned. Configurations the reference cannot run are left out: its fp16 add with an
    activation or dense output dereferences a null cache pointer (src/cuda/conv_torch_wrapper.cpp:426-434) and its
    fp16 norm/rms truncation updates the caches of dropped pixels (src/cuda/other_nn_layers.cu:1018-1030)."""
    out = {}
    for dt_name, dtype in (("f32", torch.float32), ("f16", torch.float16)):
        g = torch.Generator().manual_seed(200)
        n, h, w = 2, 16, 20
        gm = mask(g, 3, 7, 7, 0.4)
        gm[1] = 0
        out[f"gap_{dt_name}"] = dict(op="gap", x=feat(g, 3, 40, 7, 7, dtype), mask=gm)
        out[f"add_to_dense_{dt_name}"] = dict(op="add_to_dense", a=feat(g, n, 24, h, w, dtype), b=feat(g, n, 24, h, w, dtype), ma=mask(g, n, h, w, 0.3))
        out[f"concat_{dt_name}"] = dict(op="concat", a=feat(g, n, 8, h, w, dtype), b=feat(g, n, 16, h, w, dtype), ma=mask(g, n, h, w, 0.3),
                                        mb=mask(g, n, h, w, 0.3))
        out[f"mul_add_{dt_name}"] = dict(op="mul_add", x=feat(g, n, 24, h, w, dtype), mask=mask(g, n, h, w, 0.4),
                                         scale=torch.randn(24, generator=g).to(dtype), bias=torch.randn(24, generator=g).to(dtype))
        for act in (3, 4, 5):
            out[f"act{act}_{dt_name}"] = dict(op="act", delta=feat(g, n, 32, h, w, dtype, 0.05), prev=feat(g, n, 32, h, w, dtype, 2.0),
                                              trunc=feat(g, n, 32, h, w, dtype, 0.01), mask=mask(g, n, h, w, 0.5), thr=0.02, act=act, mode=0)
        out[f"accumulate_{dt_name}"] = dict(op="act", delta=feat(g, n, 32, h, w, dtype, 0.05), prev=feat(g, n, 32, h, w, dtype, 2.0),
                                            trunc=None, mask=mask(g, n, h, w, 0.5), thr=-1.0, act=-1, mode=-1)
        out[f"maxpool5x5s2_{dt_name}"] = dict(op="maxpool", x=feat(g, n, 16, h, w, dtype), prev=feat(g, n, 16, h, w, dtype),
                                              mask=mask(g, n, h, w, 0.2), k=(5, 5), s=(2, 2), p=(2, 2))
        out[f"maxpool_pad0101_{dt_name}"] = dict(op="maxpool", x=feat(g, n, 16, 15, 17, dtype, 0.3), prev=feat(g, n, 16, 15, 17, dtype) - 1.5,
                                                 mask=mask(g, n, 15, 17, 0.3), k=(3, 3), s=(2, 2), p=(0, 1, 0, 1))
        out[f"upsample16_{dt_name}"] = dict(op="upsample", x=feat(g, n, 8, 3, 4, dtype), mask=mask(g, n, 3, 4, 0.5), scale=16)
        wt = (torch.randn(16, 16, 5, 5, generator=g) / 20.0).to(dtype)
        out[f"conv_c5x5_{dt_name}"] = dict(op="conv", x=feat(g, n, 16, h, w, dtype), mask=mask(g, n, h, w, 0.12), w=wt,
                                           b=torch.randn(16, generator=g).to(dtype), s=(1, 1), p=(2, 2), groups=1)
    g = torch.Generator().manual_seed(300)
    n, h, w, dtype = 2, 16, 20, torch.float32
    for mode, name in ((1, "norm"), (2, "rms")):
        out[f"act_{name}_f32"] = dict(op="act", delta=feat(g, n, 32, h, w, dtype, 0.05), prev=feat(g, n, 32, h, w, dtype, 2.0),
                                      trunc=feat(g, n, 32, h, w, dtype, 0.01), mask=mask(g, n, h, w, 0.5), thr=0.2 if mode == 1 else 0.035, act=1, mode=mode)
    out["add_relu_f32"] = dict(op="add", a=feat(g, n, 24, h, w, dtype), b=feat(g, n, 24, h, w, dtype), ma=mask(g, n, h, w, 0.3),
                               mb=mask(g, n, h, w, 0.3), wa=1.0, wb=0.5, act=1, prev=feat(g, n, 24, h, w, dtype), dense=False)
    out["add_dense_f32"] = dict(op="add", a=feat(g, n, 24, h, w, dtype), b=feat(g, n, 24, h, w, dtype), ma=mask(g, n, h, w, 0.3),
                                mb=mask(g, n, h, w, 0.3), wa=1.0, wb=1.0, act=1, prev=feat(g, n, 24, h, w, dtype), dense=True)
    wt = (torch.randn(16, 8, 6, 6, generator=g) * 0.1).to(dtype)
    out["deconv6x6s4_f32"] = dict(op="deconv", x=feat(g, n, 16, 5, 6, dtype), mask=mask(g, n, 5, 6, 0.2), w=wt,
                                  b=torch.randn(8, generator=g).to(dtype), s=(4, 4), p=(1, 1))
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
        d, p, m = c["delta"].clone(), c["prev"].clone(), c["mask"].clone()
        t = None if c["trunc"] is None else c["trunc"].clone()
        R.activate_truncate(d, p, t, m, c["thr"], c["act"], c["mode"])
        res = dict(delta=f(d), prev=f(p), mask=f(m))
        if t is not None:
            res["trunc"] = f(t)
        return res
    if op == "add":
        prev = c["prev"].clone() if "prev" in c else None
        o, m = R.add(c["a"], c["ma"], c["b"], c["mb"], prev, c["wa"], c["wb"], c["act"], c.get("dense", False))
        res = dict(out=f(o), mask=f(m))
        if prev is not None:
            res["prev"] = f(prev)
        return res
    if op == "gap":
        o, m = R.global_avg_pool(c["x"], c["mask"])
        return dict(out=f(o), mask=f(m))
    if op == "add_to_dense":
        b = c["b"].clone()
        R.add_to_dense(c["a"], b, c["ma"])
        return dict(b=f(b))
    if op == "concat":
        o, m = R.concatenate(c["a"], c["ma"], c["b"], c["mb"])
        return dict(out=f(o), mask=f(m))
    if op == "mul_add":
        o, m = R.mul_add(c["x"], c["mask"], c["scale"], c["bias"])
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
