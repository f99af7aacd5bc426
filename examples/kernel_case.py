"""One kernel of the delta path on a fixed, seeded, benchmark-shaped input, a few launches: the
small case that profiler captures are taken on (inputs larger than L2, well under 1 GB on the device).

    python examples/kernel_case.py pw     # tcgen05 pointwise 16->96 @112x112, fused ReLU6 + truncation, 32 streams (persistent CTAs over strided spans)
    python examples/kernel_case.py dw     # depthwise 3x3 96 ch @112x112 stride 2, fused ReLU6 + truncation, 32 streams
    python examples/kernel_case.py act    # stand-alone activation/truncation, 96 ch @112x112, 32 streams
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
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    t = sorted(times)[len(times) // 2]
    print(f"{which}: median {t * 1000:.1f} us per launch, algorithmic {nbytes / 1e6:.1f} MB, {nbytes / t / 1e6:.0f} GB/s")


if __name__ == "__main__":
    main()
