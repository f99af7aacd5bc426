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

Roofline of a whole frame step: per layer t = max(flops_tile / P, bytes / BW) with flops_tile =
2 * T_active * 64 * kh*kw*Cin*Cout/groups (T_active = 8x8 output tiles holding an updated pixel; transposed
convolutions count kh*kw / stride^2 taps per output pixel), P the tensor-core peak for layers on the tcgen05 path
and the fp32 CUDA-core peak for depthwise / thin / RGB layers, BW the HBM copy bandwidth; the layers of a step
depend on each other, so the step's roofline time is the sum.
"""
import collections
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import deltacnn_b200.cuda_kernels as K  # noqa: E402

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
        self.details = []          # per record: mask densities (in, dilated out, kept out) and whether it runs on tensor cores
        self.last_density, self.last_tensor = None, False
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
            flops = 2.0 * pre["tiles_active"] * 64 * taps * cig * co          # active 8x8 tiles, every pixel and tap of them
            self.last_density = (a_in / max(mask.numel(), 1), u_out / max(om.numel(), 1), _count(om) / max(om.numel(), 1))
            self.last_tensor = groups == 1 and ci >= 16 and co >= 16 and x.dtype == torch.float16
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
            tiles = torch.nn.functional.max_pool2d((u > 0).float(), 8, 8, ceil_mode=True)
            return {"u_out": int((u > 0).sum().item()), "tiles_active": int(tiles.sum().item())}
        return {}

    # ---- wrapping ---------------------------------------------------------------------------
    def _wrap(self, name, fn):
        def inner(*args, **kwargs):
            pre = self._pre(name, args, kwargs)
            self.flush.fill_(1)
            # keep the device busy while the host prepares the call (argument checks, descriptors): the interval between
            # the two events must hold the kernels of the call and no idle time
            torch.cuda._sleep(600000)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            res = fn(*args, **kwargs)
            e1.record(self.stream)
            e1.synchronize()
            ms = e0.elapsed_time(e1)
            self.last_density, self.last_tensor = None, False
            key, site, nbytes, flops = self._account(name, args, kwargs, res, pre)
            self.records.append((key, site, ms, nbytes, flops))
            self.details.append({"density": self.last_density, "tensor": self.last_tensor})
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
    """Run ``frames`` (steady-state inputs) eagerly under the profiler; returns per-class totals, the records
    and the per-record details."""
    with OpProfiler(stream) as prof, torch.no_grad():
        for f in frames:
            delta(f)
    return prof.summary(), prof.records, prof.details


# DRAM bytes (read + written) of one profiler capture of a kernel class beside the algorithmic bytes of the captured
# launch (profiles/*.md): traffic of a bench launch = its algorithmic bytes times this ratio. Classes without a
# capture report no traffic.
NCU_TRAFFIC_RATIO = {"conv1x1+act": 20.8 / 47.1}
CUDA_CORE_PEAK_TFLOPS = 74.4      # fp32 FMA peak of the CUDA cores: 148 SMs x 128 lanes x 2 flops x 1.965 GHz


def roofline_report(delta, frames_dev, stream, peak, tensor_peak_tflops, ms_per_step, group_fraction):
    """Per-class table, the dominant class (algorithmic bytes per launch over its cold-L2 launch time against the HBM
    copy bandwidth), the roofline of the whole step and of its convolution layers, and the per-layer mask
    densities. ``group_fraction`` = streams profiled / streams of a step (the profile runs one stream group)."""
    peak_gbs, peak_kind = peak
    n = frames_dev.shape[0]
    n_frames = 4
    summary, records, details = profile_frames(delta, [frames_dev[i % n] for i in range(3, 3 + n_frames)], stream)
    total_ms = sum(a["ms"] for a in summary.values())
    key, top = max(summary.items(), key=lambda kv: kv[1]["ms"])
    per_launch_bytes = top["bytes"] / top["launches"]
    per_launch_ms = top["ms"] / top["launches"]
    achieved = per_launch_bytes / (per_launch_ms * 1e-3) / 1e9
    table = {k: {"launches": a["launches"], "ms": round(a["ms"], 4), "share": round(a["ms"] / total_ms, 4),
                 "GBps": round(a["bytes"] / max(a["ms"], 1e-9) / 1e6, 1)} for k, a in summary.items()}
    ratio = NCU_TRAFFIC_RATIO.get(key)
    # whole-step roofline: every layer at the slower of its two bounds, summed (layers depend on each other)
    scale = 1.0 / (n_frames * group_fraction)             # profiled totals -> one step of all streams
    t_all = t_conv = ms_conv = bytes_all = flops_all = 0.0
    for (k, _site, ms, nbytes, flops), det in zip(records, details):
        p_flops = (tensor_peak_tflops if det["tensor"] else CUDA_CORE_PEAK_TFLOPS) * 1e12
        t = max(flops / p_flops, nbytes / (peak_gbs * 1e9))
        t_all += t
        bytes_all += nbytes
        flops_all += flops
        if "conv" in k:
            t_conv += t
            ms_conv += ms
    per_layer = len(records) // n_frames
    density = [{"layer": f"{k} {site}", "in": round(d["density"][0], 4), "out_dilated": round(d["density"][1], 4),
                "out_kept": round(d["density"][2], 4)}
               for (k, site, *_), d in list(zip(records, details))[-per_layer:] if d["density"] is not None]
    frame = {"algorithmic_bytes_per_step": bytes_all * scale, "flops_tile_per_step": flops_all * scale,
             "t_roofline_ms": t_all * scale * 1e3, "achieved": t_all * scale * 1e3 / ms_per_step,
             "how": "sum over layers of max(flops_tile / peak flops, bytes / HBM bandwidth) over the measured step time (CUDA graph)",
             "conv_layers": {"t_roofline_ms": t_conv * scale * 1e3, "cold_serialised_ms": ms_conv * scale,
                             "achieved": t_conv * 1e3 / max(ms_conv, 1e-9),
                             "how": "convolution layers only, against the sum of their per-launch times (cold L2, launches serialised)"},
             "peaks": {"hbm_gbs": peak_gbs, "tensor_tflops": tensor_peak_tflops, "cuda_core_tflops": CUDA_CORE_PEAK_TFLOPS}}
    return {"bound": "hbm", "kernel": key, "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
            "frac": achieved / peak_gbs, "peak_kind": f"of {peak_kind}",
            "traffic": per_launch_bytes * ratio if ratio is not None else None,
            "traffic_how": "algorithmic bytes of the launch times the DRAM/algorithmic ratio of an ncu capture of one layer of the class (profiles/)" if ratio is not None else "no ncu capture of this class",
            "timing": "per-launch CUDA events with L2 flushed before every launch, launches serialised (not the in-graph time)",
            "bytes_per_launch": per_launch_bytes, "ms_per_launch": per_launch_ms, "launches_timed": top["launches"],
            "share_of_step": top["ms"] / total_ms, "kernels": table, "frame": frame}, density


def main():
    """``python examples/profile.py [config] [streams]``: every layer call of one steady-state frame step (eager, cold
    L2, CUDA events; the best of three frames per layer) with its algorithmic bytes and the time those bytes take at
    the measured copy bandwidth of the GPU."""
    from examples.nets import build_pair
    from examples.synthetic_video import make_video
    from deltacnn_b200.stepping import set_depth_thresholds
    # the copy bandwidth measured on this kind of GPU, if the file with it is there (else an earlier measurement)
    peaks_file = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    hbm_gbs, kind = 6650.0, "fallback"
    if os.path.exists(peaks_file):
        import json
        with open(peaks_file) as f:
            hbm_gbs, kind = float(json.load(f)["hbm_gbs"]), "measured"
    name = sys.argv[1] if len(sys.argv) > 1 else "mobilenet"
    streams = int(sys.argv[2]) if len(sys.argv) > 2 else 32
    vids = torch.stack([make_video(name, s).frames(6) for s in range(streams)], dim=1)
    dev = torch.device("cuda")
    _, delta = build_pair(name, vids[:4, 0], device=dev, dtype=torch.float16)
    fd = [vids[i].to(dev, torch.float16).contiguous(memory_format=torch.channels_last) for i in range(6)]
    stream = torch.cuda.current_stream()
    runs = []
    with torch.no_grad():
        delta(fd[0])
        set_depth_thresholds(0.03 if name != "mobilenet" else 0.05, 0.01, 0.05)
        delta(fd[1])
        delta(fd[2])
        for f in (3, 4, 5):
            with OpProfiler(stream) as prof:
                delta(fd[f])
            runs.append(prof.records)
    total = roof = 0.0
    print(f"{name}, {streams} streams: layer call, best of three frames (cold L2) | algorithmic MB | time of the bytes at {hbm_gbs:.0f} GB/s ({kind})")
    for i in range(min(len(r) for r in runs)):
        key, site, _, nbytes, _ = runs[-1][i]
        ms = min(r[i][2] for r in runs)
        total += ms
        roof += nbytes / (hbm_gbs * 1e6)
        print(f"{i:3d} {key:16s} {site:30s} {ms * 1000:7.1f} us {nbytes / 1e6:8.2f} MB {nbytes / (hbm_gbs * 1e3):6.1f} us")
    print(f"sum {total:.3f} ms, bytes at bandwidth {roof:.3f} ms")


if __name__ == "__main__":
    main()
