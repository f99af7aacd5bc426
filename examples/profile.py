"""Per-kernel timing and algorithmic-byte accounting of one delta frame step.

The operator functions of ``deltacnn_b200.cuda_kernels`` are wrapped for a few eager frames: before
every call a buffer larger than L2 is overwritten (cold cache, and the GPU stays busy so that the
event pair brackets only the kernel), a CUDA-event pair on the launching stream times the call, and
afterwards the algorithmic bytes of the call are computed on the host from the masks. The byte
formulas mirror the reference's own counters (DCMetrics, src/cuda/common.cuh:41-65; increments at
src/cuda/conv_kernel.cu:90-107,196-209 and src/cuda/other_nn_layers.cu:810-813):

  conv / deconv  esize*(A_in*Cin + U_out*Cout + kh*kw*Cin*Cout/groups) + 4*(HW_in + HW_out)
  activation     esize*C*(3*M_in + 3*M_kept) + 8*HW           (also added to a conv with fused epilogue)
  conv + add     conv bytes + esize*Cout*(2*U_union - U_conv) + 4*HW   (residual added in the convolution's epilogue;
                 an upper bound on the residual reads: every pixel of the union is counted once)
  sparsify       esize*C*(2*HW + 2*M) + 4*HW
  add            esize*C*(n_a + n_b + n_ab [+ 2*n_ab with activation]) + 12*HW
  pool           esize*C*(A_in [*2 for max: prev] + U_out) + 4*(HW_in + HW_out) [+ 2*esize*C*A_in cache update]
  densify        esize*C*(2*M + 2*HW) + 4*HW ; upsample esize*C*(M_in + M_out) + 4*(HW_in + HW_out)

with A_in = active input pixels, U_out = output pixels whose out-mask is 1, M = masked pixels.
"""
import collections

import torch

import deltacnn_b200.cuda_kernels as K

L2_FLUSH_BYTES = 256 << 20


def _esize(t):
    return t.element_size()


def _count(m):
    return int((m != 0).sum().item())


class OpProfiler:
    OPS = ("sparse_conv", "sparse_deconv", "sparse_activation", "sparsify", "sparse_add_tensors", "sparse_pooling",
           "sparse_densify", "sparse_upsample", "sparse_add_to_dense_tensor", "sparse_mul_add", "sparse_concatenate")

    def __init__(self, stream):
        self.stream = stream
        self.records = []          # (class key, site description, ms, algorithmic bytes, flops)
        self.flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")
        self._orig = {}

    # ---- accounting -------------------------------------------------------------------------
    def _act_bytes(self, c, es, m_in, m_kept, hw):
        return es * c * (3 * m_in + 3 * m_kept) + 8 * hw

    def _account(self, name, args, kwargs, result, pre):
        if name in ("sparse_conv", "sparse_deconv"):
            x, filt = kwargs.get("x", args[0] if args else None), kwargs.get("filter")
            mask = kwargs.get("mask")
            out, om = result
            kh, kw, cig, co = filt.shape
            es = _esize(x)
            n, ci, hi, wi = x.shape
            a_in = _count(mask)
            u_out = pre["u_out"]
            groups = kwargs.get("groups", 1)
            b = es * (a_in * ci + u_out * co + kh * kw * cig * co) + 4 * (n * hi * wi + om.numel())
            taps = kh * kw / (kwargs["stride"][0] * kwargs["stride"][1]) if name == "sparse_deconv" else kh * kw
            flops = 2.0 * u_out * taps * cig * co
            kind = "dwconv" if groups > 1 else ("deconv" if name == "sparse_deconv" else "conv")
            key = f"{kind}{kh}x{kw}"
            ep = kwargs.get("epilogue")
            if ep is not None and getattr(ep, "residual", None):
                # linear convolution with the residual add in its epilogue: the union mask is written, the residual
                # is read where it is active (as many pixels as the union minus those only the convolution touches)
                u_union = _count(om)
                b += es * co * (u_union - u_out) + es * co * u_union + 4 * om.numel()
                key += "+add"
            elif ep is not None:
                b += self._act_bytes(co, es, u_out, _count(om), om.numel())
                key += "+act"
            return key, f"{ci}->{co} @{hi}x{wi} s{kwargs['stride'][0]}", b, flops
        if name == "sparse_activation":
            x, mask = args[0], args[3]
            return "act_trunc", f"{x.shape[1]} @{x.shape[2]}x{x.shape[3]}", \
                self._act_bytes(x.shape[1], _esize(x), pre["m_in"], _count(mask), mask.numel()), 0.0
        if name == "sparsify":
            x, mask = args[0], args[3]
            return "sparsify", f"{x.shape[1]} @{x.shape[2]}x{x.shape[3]}", \
                _esize(x) * x.shape[1] * (2 * mask.numel() + 2 * _count(mask)) + 4 * mask.numel(), 0.0
        if name == "sparse_add_tensors":
            a, ma, mb, act = args[0], args[4], args[5], args[9]
            na, nb, nab = _count(ma), _count(mb), _count((ma != 0) | (mb != 0))
            return "add", f"{a.shape[1]} @{a.shape[2]}x{a.shape[3]}", \
                _esize(a) * a.shape[1] * (na + nb + nab + (2 * nab if act > 0 else 0)) + 12 * ma.numel(), 0.0
        if name == "sparse_pooling":
            x, mask = args[0], args[3] if len(args) > 3 else kwargs.get("mask")
            out, om = result
            mode = kwargs.get("pooling_mode_int", 0)
            a_in, u_out = _count(mask), _count(om)
            b = _esize(x) * x.shape[1] * (a_in * (2 if mode == 0 else 1) + u_out) + 4 * (mask.numel() + om.numel())
            if kwargs.get("update_prev"):
                b += 2 * _esize(x) * x.shape[1] * a_in
            return ("maxpool" if mode == 0 else "avgpool"), f"{x.shape[1]} @{x.shape[2]}x{x.shape[3]}", b, 0.0
        if name == "sparse_densify":
            x, mask = args[0], args[1]
            return "densify", f"{x.shape[1]} @{x.shape[2]}x{x.shape[3]}", \
                _esize(x) * x.shape[1] * (2 * _count(mask) + 2 * mask.numel()) + 4 * mask.numel(), 0.0
        if name == "sparse_upsample":
            x, mask = args[0], args[1]
            o, om = result
            return "upsample", f"{x.shape[1]} @{x.shape[2]}x{x.shape[3]}", \
                _esize(x) * x.shape[1] * (_count(mask) + _count(om)) + 4 * (mask.numel() + om.numel()), 0.0
        x = args[0] if torch.is_tensor(args[0]) else args[0][0]
        return name, f"{x.shape[1]} @{x.shape[2]}x{x.shape[3]}", 0, 0.0

    def _pre(self, name, args, kwargs):
        """Quantities that must be read before the call mutates its arguments."""
        if name == "sparse_activation":
            return {"m_in": _count(args[3])}
        if name in ("sparse_conv", "sparse_deconv"):
            mask, filt = kwargs["mask"], kwargs["filter"]
            m = (mask != 0).float()
            kh, kw = filt.shape[0], filt.shape[1]
            if name == "sparse_conv":
                pt, pb, pl, pr = K._pad4(kwargs["padding"])
                m = torch.nn.functional.pad(m, (pl, pr, pt, pb))
                u = torch.nn.functional.max_pool2d(m, (kh, kw), kwargs["stride"], 0, kwargs["dilation"])
            else:
                u = torch.nn.functional.conv_transpose2d(m, torch.ones(1, 1, kh, kw, device=m.device), None,
                                                         kwargs["stride"], kwargs["padding"])
            return {"u_out": int((u > 0).sum().item())}
        return {}

    # ---- wrapping ---------------------------------------------------------------------------
    def _wrap(self, name, fn):
        def inner(*args, **kwargs):
            pre = self._pre(name, args, kwargs)
            self.flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            res = fn(*args, **kwargs)
            e1.record(self.stream)
            e1.synchronize()
            ms = e0.elapsed_time(e1)
            key, site, nbytes, flops = self._account(name, args, kwargs, res, pre)
            self.records.append((key, site, ms, nbytes, flops))
            return res
        return inner

    def __enter__(self):
        for n in self.OPS:
            self._orig[n] = getattr(K, n)
            setattr(K, n, self._wrap(n, self._orig[n]))
        return self

    def __exit__(self, *exc):
        for n, f in self._orig.items():
            setattr(K, n, f)

    def summary(self):
        agg = collections.OrderedDict()
        for key, _site, ms, nbytes, flops in self.records:
            a = agg.setdefault(key, {"launches": 0, "ms": 0.0, "bytes": 0, "flops": 0.0})
            a["launches"] += 1
            a["ms"] += ms
            a["bytes"] += nbytes
            a["flops"] += flops
        return agg


def profile_frames(delta, frames, stream):
    """Run ``frames`` (steady-state inputs) eagerly under the profiler; returns per-class totals."""
    with OpProfiler(stream) as prof, torch.no_grad():
        for f in frames:
            delta(f)
    return prof.summary(), prof.records


def roofline_of_dominant_kernel(delta, frames_dev, stream, peak):
    """The kernel class with the largest share of a frame step, its algorithmic bytes per launch over
    its measured (cold-L2) launch time, against the HBM copy bandwidth."""
    peak_gbs, peak_kind = peak
    n = frames_dev.shape[0]
    summary, _ = profile_frames(delta, [frames_dev[i % n] for i in range(3, 7)], stream)
    total_ms = sum(a["ms"] for a in summary.values())
    key, top = max(summary.items(), key=lambda kv: kv[1]["ms"])
    per_launch_bytes = top["bytes"] / top["launches"]
    per_launch_ms = top["ms"] / top["launches"]
    achieved = per_launch_bytes / (per_launch_ms * 1e-3) / 1e9
    table = {k: {"launches": a["launches"], "ms": round(a["ms"], 4), "share": round(a["ms"] / total_ms, 4),
                 "GBps": round(a["bytes"] / max(a["ms"], 1e-9) / 1e6, 1)} for k, a in summary.items()}
    # DRAM traffic of the class's kernel from a profiler capture of one of its layers (16->96 @112x112, 32 streams:
    # 20.8 MB read + written for 47.1 MB of algorithmic bytes: the writes and part of the caches stay in L2), scaled to
    # this launch's algorithmic bytes; None for classes without such a capture.
    traffic = per_launch_bytes * (20.8 / 47.1) if key == "conv1x1+act" else None
    return {"bound": "hbm", "kernel": key, "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
            "frac": achieved / peak_gbs, "peak_kind": f"of {peak_kind}", "traffic": traffic,
            "traffic_how": "scaled from an ncu capture of one layer of the class (profiles/k_pw_umma_16to96_112x112_32streams.md)",
            "bytes_per_launch": per_launch_bytes, "ms_per_launch": per_launch_ms, "launches_timed": top["launches"],
            "share_of_step": top["ms"] / total_ms, "kernels": table}
