"""One kernel of the delta path on a fixed, seeded, benchmark-shaped input, a few launches: the
small case that profiler captures are taken on (inputs larger than L2, well under 1 GB on the device).

    python examples/kernel_case.py pw     # tcgen05 pointwise 16->96 @112x112, fused ReLU6 + truncation, 32 streams (persistent CTAs over strided spans)
    python examples/kernel_case.py dw     # depthwise 3x3 96 ch @112x112 stride 2, fused ReLU6 + truncation, 32 streams
    python examples/kernel_case.py act    # stand-alone activation/truncation, 96 ch @112x112, 32 streams
    python examples/kernel_case.py c3x3   # tcgen05 3x3 256->256 @64x64, fused ReLU + truncation, 32 streams, work list
    python examples/kernel_case.py c3x3p  # the same layer on patch tiles (tiled TMA loads), no scratch
    python examples/kernel_case.py h32    # 3x3 32->32 @64x64 fully active, 32 streams (halo tiles; DC_HALO=0: patch tiles); also h64, h128, h256to64
    python examples/kernel_case.py heads3 [reps] [streams]   # three 3x3 256->64 head layers @136x240 in one segmented halo-tile launch, 16 streams
    python examples/kernel_case.py stem   # tcgen05 RGB stem 3x3/2 3->32 @224x224, fused ReLU6 + truncation, 32 streams
    python examples/kernel_case.py deconv # tcgen05 transposed 4x4/2 256->256 @34x60, fused ReLU + truncation, 16 streams, per-phase work lists
    python examples/kernel_case.py dw576  # depthwise 3x3 576 ch @14x14 (a warp per channel slice), fully active, 64 streams
    python examples/kernel_case.py sparsify  # RGB input delta + mask @224x224, 64 streams
    python examples/kernel_case.py linear [reps] [streams]   # classifier on the pooled delta, 1280 -> 1000 ("linear_dense": densify + torch linear)
    python examples/kernel_case.py irb576 [reps] [streams]   # fused inverted-residual block 96->576->96 @14x14 with residual, fully active
    python examples/kernel_case.py irb960 [reps] [streams]   # fused block 160->960->160 @7x7; "sep576" / "sep960": the same blocks as three calls
Prints the CUDA-event time per launch (L2 flushed between launches) and the algorithmic GB/s.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import deltacnn_b200.cuda_kernels as K  # noqa: E402
from deltacnn_b200 import _lib  # noqa: E402
from deltacnn_b200.filter_conversion import convert_filter_out_channels_last  # noqa: E402


def blob_mask(g, n, h, w, density):
    """Update mask made of three rectangles per image covering about ``density`` of the pixels."""
    m = torch.zeros(n, 1, h, w, dtype=torch.int32)
    side = max(int((density * h * w / 3) ** 0.5), 1)
    for b in range(n):
        for _ in range(3):
            y = int(torch.randint(0, h - side + 1, (1,), generator=g))
            x = int(torch.randint(0, w - side + 1, (1,), generator=g))
            m[b, 0, y:y + side, x:x + side] = 1
    return m


def main():
    which = sys.argv[1] if len(sys.argv) > 1 else "pw"
    reps = int(sys.argv[2]) if len(sys.argv) > 2 else 5
    n, dtype = 32, torch.float16
    g = torch.Generator().manual_seed(0)
    cl = lambda t: t.contiguous(memory_format=torch.channels_last)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    if which == "pw":
        cin, cout, h, w = 16, 96, 112, 112
        x = cl((torch.randn(n, cin, h, w, generator=g) * 0.3).to(dtype)).cuda()
        mask = blob_mask(g, n, h, w, 0.12).cuda()
        wt = (torch.randn(cout, cin, 1, 1, generator=g) * 0.25).to(dtype)
        f = convert_filter_out_channels_last(wt).cuda()
        desc = K.make_conv_desc((1, cin, 8, 8), cout, (8, 8), (1, 1), (1, 1), (0, 0), (1, 1), 1, 1)
        packed = torch.zeros(_lib.lib.dc_filter_umma_bytes(desc, 0), dtype=torch.uint8, device="cuda")
        _lib.check(_lib.lib.dc_pack_filter_umma(desc, 0, f.data_ptr(), packed.data_ptr(), torch.cuda.current_stream().cuda_stream), "pack")
        prev = cl(torch.randn(n, cout, h, w, generator=g).to(dtype)).cuda()
        trunc = torch.zeros_like(prev)
        out = torch.empty_like(prev)
        om = torch.empty(n, 1, h, w, dtype=torch.int32, device="cuda")
        ep = K.make_epilogue(prev, trunc, 0.02, 2, 0)
        d2 = K.make_conv_desc(tuple(x.shape), cout, (h, w), (1, 1), (1, 1), (0, 0), (1, 1), 1, 1)
        ws = torch.zeros(K.conv_workspace_bytes(d2), dtype=torch.uint8, device="cuda")
        run = lambda: K.sparse_conv(x, f, mask, None, (1, 1), (0, 0), (1, 1), 1, create_out_mask=True, out=out, out_mask=om,
                                    filter_umma=packed, epilogue=ep, workspace=ws)
        act_px = int(mask.sum())
        nbytes = 2 * (act_px * cin + cin * cout) + 2 * cout * 5 * act_px + 8 * mask.numel()
    elif which == "dw":
        c, h, w, s = 96, 112, 112, 2
        x = cl((torch.randn(n, c, h, w, generator=g) * 0.3).to(dtype)).cuda()
        mask = blob_mask(g, n, h, w, 0.12).cuda()
        wt = (torch.randn(c, 1, 3, 3, generator=g) * 0.3).to(dtype)
        f = convert_filter_out_channels_last(wt).cuda()
        ho = h // s
        prev = cl(torch.randn(n, c, ho, ho, generator=g).to(dtype)).cuda()
        trunc = torch.zeros_like(prev)
        out = torch.empty_like(prev)
        om = torch.empty(n, 1, ho, ho, dtype=torch.int32, device="cuda")
        ep = K.make_epilogue(prev, trunc, 0.02, 2, 0)
        d2 = K.make_conv_desc(tuple(x.shape), c, (ho, ho), (3, 3), (s, s), (1, 1), (1, 1), c, 1)
        ws = torch.zeros(K.conv_workspace_bytes(d2), dtype=torch.uint8, device="cuda")
        run = lambda: K.sparse_conv(x, f, mask, None, (s, s), (1, 1), (1, 1), c, create_out_mask=True, out=out, out_mask=om, epilogue=ep,
                                    workspace=ws)
        run()
        nbytes = 2 * c * (int(mask.sum()) + 5 * int((torch.nn.functional.max_pool2d(mask.float(), 3, s, 1) > 0).sum())) + 4 * (mask.numel() + om.numel())
    elif which in ("c3x3", "c3x3p", "h32", "h64", "h128", "h256to64", "h32n", "h64n", "stem", "deconv", "dw576"):
        geo = {"c3x3": (32, 256, 256, 64, 64, 3, 1, 1, 1, 0.12, 1), "c3x3p": (32, 256, 256, 64, 64, 3, 1, 1, 1, 0.6, 1),
               "h32": (32, 32, 32, 64, 64, 3, 1, 1, 1, 1.0, 1), "h64": (32, 64, 64, 136, 240, 3, 1, 1, 1, 0.9, 1),
               "h32n": (32, 32, 32, 64, 64, 3, 1, 1, 1, 1.0, 1), "h64n": (32, 64, 64, 136, 240, 3, 1, 1, 1, 0.9, 1),
               "h128": (32, 128, 128, 68, 120, 3, 1, 1, 1, 0.9, 1), "h256to64": (32, 256, 64, 136, 240, 3, 1, 1, 1, 0.9, 1),
               "stem": (32, 3, 32, 224, 224, 3, 2, 1, 1, 0.12, 2), "deconv": (16, 256, 256, 34, 60, 4, 2, 1, 1, 0.3, 1),
               "dw576": (64, 576, 576, 14, 14, 3, 1, 1, 576, 1.0, 2)}[which]
        n, cin, cout, h, w, k, s, pad, groups, density, act = geo
        transposed = which == "deconv"
        x = cl((torch.randn(n, cin, h, w, generator=g) * 0.3).to(dtype)).cuda()
        mask = (torch.ones(n, 1, h, w, dtype=torch.int32) if density >= 1.0 else blob_mask(g, n, h, w, density)).cuda()
        if transposed:
            wt = (torch.randn(cin, cout, k, k, generator=g) * 0.05).to(dtype)
            ho, wo = K.deconv_out_hw(h, w, (k, k), (s, s), (pad, pad), (1, 1))
        else:
            wt = (torch.randn(cout, cin // groups, k, k, generator=g) * (k * k * cin // groups) ** -0.5).to(dtype)
            ho, wo = K.conv_out_hw(h, w, (k, k), (s, s), (pad, pad), (1, 1))
        f = convert_filter_out_channels_last(wt, transposed=transposed).cuda()
        desc = K.make_conv_desc(tuple(x.shape), cout, (ho, wo), (k, k), (s, s), (pad, pad), (1, 1), groups, 1)
        packed = None
        nb = _lib.lib.dc_filter_umma_bytes(desc, 1 if transposed else 0)
        if nb > 0:
            packed = torch.zeros(nb, dtype=torch.uint8, device="cuda")
            _lib.check(_lib.lib.dc_pack_filter_umma(desc, 1 if transposed else 0, f.data_ptr(), packed.data_ptr(), torch.cuda.current_stream().cuda_stream), "pack")
        prev = cl(torch.randn(n, cout, ho, wo, generator=g).to(dtype)).cuda()
        trunc = torch.zeros_like(prev)
        out = torch.empty_like(prev)
        om = torch.empty(n, 1, ho, wo, dtype=torch.int32, device="cuda")
        ep = None if which in ("h32n", "h64n") else K.make_epilogue(prev, trunc, 0.02, act, 0)      # ...n: plain store, no truncation
        if transposed:
            ws = torch.zeros(K.deconv_workspace_bytes(desc), dtype=torch.uint8, device="cuda")
            run = lambda: K.sparse_deconv(x, f, mask, None, (s, s), (pad, pad), (1, 1), 1, create_out_mask=True, out=out, out_mask=om,
                                          epilogue=ep, desc=desc, filter_umma=packed, workspace=ws)
            u = torch.nn.functional.conv_transpose2d(mask.float(), torch.ones(1, 1, k, k, device="cuda"), None, s, pad) > 0
            taps = (k // s) ** 2
        else:
            ws = None if which == "c3x3p" or which[0] == "h" else torch.zeros(K.conv_workspace_bytes(desc), dtype=torch.uint8, device="cuda")
            run = lambda: K.sparse_conv(x, f, mask, None, (s, s), (pad, pad), (1, 1), groups, create_out_mask=True, out=out, out_mask=om,
                                        filter_umma=packed, epilogue=ep, desc=desc, workspace=ws)
            u = torch.nn.functional.max_pool2d(mask.float(), k, s, pad) > 0
            taps = k * k
        u_out = int(u.sum())
        nbytes = 2 * (int(mask.sum()) * cin + taps * (cin // groups) * cout) + 2 * cout * 5 * u_out + 4 * (mask.numel() + om.numel())
        print(f"{which}: {int(mask.sum())} active input pixels, {u_out} updated output pixels, {2.0 * u_out * taps * (cin // groups) * cout / 1e9:.2f} GFLOP")
    elif which in ("irb576", "irb960", "sep576", "sep960", "irb384", "sep384"):
        n = int(sys.argv[3]) if len(sys.argv) > 3 else 64
        cin, chid, cout, h, w = {"576": (96, 576, 96, 14, 14), "960": (160, 960, 160, 7, 7), "384": (64, 384, 64, 14, 14)}[which[3:]]
        x = cl((torch.randn(n, cin, h, w, generator=g) * 0.3).to(dtype)).cuda()
        mask = torch.ones(n, 1, h, w, dtype=torch.int32, device="cuda")
        hw = lambda wt: convert_filter_out_channels_last(wt).cuda()
        f1 = hw((torch.randn(chid, cin, 1, 1, generator=g) * cin ** -0.5).to(dtype))
        fd = hw((torch.randn(chid, 1, 3, 3, generator=g) * 0.4).to(dtype))
        f2 = hw((torch.randn(cout, chid, 1, 1, generator=g) * chid ** -0.5).to(dtype))

        def pack(f, ci, co):
            d_ = K.make_conv_desc((1, ci, 8, 8), co, (8, 8), (1, 1), (1, 1), (0, 0), (1, 1), 1, 1)
            pk = torch.zeros(_lib.lib.dc_filter_umma_bytes(d_, 0), dtype=torch.uint8, device="cuda")
            _lib.check(_lib.lib.dc_pack_filter_umma(d_, 0, f.data_ptr(), pk.data_ptr(), torch.cuda.current_stream().cuda_stream), "pack")
            return pk
        p1, p2 = pack(f1, cin, chid), pack(f2, chid, cout)
        caches = [cl(torch.randn(n, chid, h, w, generator=g).to(dtype)).cuda(), torch.zeros(n, chid, h, w, dtype=dtype, device="cuda").contiguous(memory_format=torch.channels_last),
                  cl(torch.randn(n, chid, h, w, generator=g).to(dtype)).cuda(), torch.zeros(n, chid, h, w, dtype=dtype, device="cuda").contiguous(memory_format=torch.channels_last)]
        out = torch.empty(n, cout, h, w, dtype=dtype, device="cuda").contiguous(memory_format=torch.channels_last)
        om = torch.empty(n, 1, h, w, dtype=torch.int32, device="cuda")
        if which.startswith("irb"):
            desc = K.make_irb_desc(tuple(x.shape), chid, cout, 1, True, 2, 2, 0.02, 0.02)
            run = lambda: K.fused_inverted_residual(x, mask, p1, fd, p2, *caches, out, om, desc)
        else:
            a, ma = torch.empty_like(caches[0]), torch.empty_like(om)
            b_, mb = torch.empty_like(caches[0]), torch.empty_like(om)

            def run():
                K.sparse_conv(x, f1, mask, None, (1, 1), (0, 0), (1, 1), 1, create_out_mask=True, out=a, out_mask=ma, filter_umma=p1,
                              epilogue=K.make_epilogue(caches[0], caches[1], 0.02, 2, 0))
                K.sparse_conv(a, fd, ma, None, (1, 1), (1, 1), (1, 1), chid, create_out_mask=True, out=b_, out_mask=mb,
                              epilogue=K.make_epilogue(caches[2], caches[3], 0.02, 2, 0))
                K.sparse_conv(b_, f2, mb, None, (1, 1), (0, 0), (1, 1), 1, create_out_mask=True, out=out, out_mask=om, filter_umma=p2,
                              epilogue=K.make_residual_epilogue(x, mask))
        npx = n * h * w
        nbytes = 2 * npx * (2 * cin + cout + 8 * chid) + 8 * npx          # block input (twice: residual), output, four caches read and written
    elif which in ("linear", "linear_dense"):
        n = int(sys.argv[3]) if len(sys.argv) > 3 else 32
        cin, cout = 1280, 1000
        wt = (torch.randn(cout, cin, generator=g) * 0.01).to(dtype).cuda()
        bias = torch.zeros(cout, dtype=dtype, device="cuda")
        delta = cl(torch.randn(n, cin, 1, 1, generator=g).to(dtype)).cuda()
        mask = torch.ones(n, 1, 1, 1, dtype=torch.int32, device="cuda")
        acc = torch.zeros(n, cout, device="cuda")
        out = torch.empty(n, cout, dtype=dtype, device="cuda")
        prev = torch.zeros_like(delta)
        if which == "linear":
            run = lambda: K.linear_delta(delta, mask, wt, bias, acc, out, False)
        else:
            run = lambda: torch.nn.functional.linear(K.sparse_densify(delta, mask, prev).reshape(n, -1), wt, bias)
        nbytes = 2 * (n * cin + cin * cout + n * cout) + 8 * n * cout
    elif which == "heads3":
        # three 3x3 256 -> 64 head layers on the same 136x240 map (90 % active) as ONE launch, each with its own fused
        # ReLU + truncation, caches, output and out-mask
        n = int(sys.argv[3]) if len(sys.argv) > 3 else 16
        cin, seg, nh, h, w = 256, 64, 3, 136, 240
        x = cl((torch.randn(n, cin, h, w, generator=g) * 0.3).to(dtype)).cuda()
        mask = blob_mask(g, n, h, w, 0.9).cuda()
        wt = (torch.randn(nh * seg, cin, 3, 3, generator=g) * (9 * cin) ** -0.5).to(dtype)
        f = convert_filter_out_channels_last(wt).cuda()
        desc = K.make_conv_desc(tuple(x.shape), nh * seg, (h, w), (3, 3), (1, 1), (1, 1), (1, 1), 1, 1)
        assert K.conv3x3_heads_supported(desc, nh)
        packed = torch.zeros(_lib.lib.dc_filter_umma_bytes(desc, 0), dtype=torch.uint8, device="cuda")
        _lib.check(_lib.lib.dc_pack_filter_umma(desc, 0, f.data_ptr(), packed.data_ptr(), torch.cuda.current_stream().cuda_stream), "pack")
        outs = [torch.empty(n, seg, h, w, dtype=dtype, device="cuda").contiguous(memory_format=torch.channels_last) for _ in range(nh)]
        oms = [torch.empty(n, 1, h, w, dtype=torch.int32, device="cuda") for _ in range(nh)]
        prevs = [cl(torch.randn(n, seg, h, w, generator=g).to(dtype)).cuda() for _ in range(nh)]
        truncs = [torch.zeros_like(p_) for p_ in prevs]
        eps = [K.make_epilogue(prevs[i], truncs[i], 0.02, 1, 0) for i in range(nh)]
        run = lambda: K.conv3x3_heads(x, mask, packed, None, outs, oms, desc, eps)
        u_out = int((torch.nn.functional.max_pool2d(mask.float(), 3, 1, 1) > 0).sum())
        nbytes = 2 * (int(mask.sum()) * cin + 9 * cin * nh * seg) + 2 * nh * seg * 5 * u_out + 4 * (mask.numel() + nh * mask.numel())
        print(f"heads3: {int(mask.sum())} active input pixels, {u_out} updated output pixels, {2.0 * u_out * 9 * cin * nh * seg / 1e9:.2f} GFLOP")
    elif which == "sparsify":
        n, h, w = 64, 224, 224
        prev = cl(torch.rand(n, 3, h, w, generator=g).to(dtype)).cuda()
        x = prev.clone()
        m0 = blob_mask(g, n, h, w, 0.1).cuda().bool().expand(n, 3, h, w)
        x[m0] = 0.5 * x[m0] + 0.25
        x = cl(x)
        p = prev.clone()
        delta = torch.empty_like(x)
        mask = torch.empty(n, 1, h, w, dtype=torch.int32, device="cuda")

        def run():
            p.copy_(prev)
            K.sparsify(x, p, delta, mask, 0.05)
        run()
        nbytes = 2 * 3 * (2 * mask.numel() + 2 * int(mask.sum())) + 4 * mask.numel()
    else:
        c, h, w = 96, 112, 112
        delta = cl((torch.randn(n, c, h, w, generator=g) * 0.3).to(dtype)).cuda()
        mask0 = blob_mask(g, n, h, w, 0.12).cuda()
        prev = cl(torch.randn(n, c, h, w, generator=g).to(dtype)).cuda()
        trunc = torch.zeros_like(prev)
        mask = mask0.clone()

        def run():
            mask.copy_(mask0)
            K.sparse_activation(delta, prev, trunc, mask, 0.02, 2, 0)
        nbytes = 2 * c * 6 * int(mask0.sum()) + 8 * mask0.numel()
    times = []
    for _ in range(reps):
        flush.fill_(1)
        torch.cuda._sleep(600000)         # the device stays busy while the host prepares the call: no idle time between the events
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    if _lib.lib.dc_umma_error() != 0:
        raise SystemExit("a bounded wait of a tensor-core kernel gave up")
    t = sorted(times)[len(times) // 2]
    print(f"{which}: median {t * 1000:.1f} us per launch, algorithmic {nbytes / 1e6:.1f} MB, {nbytes / t / 1e6:.0f} GB/s")


if __name__ == "__main__":
    main()
