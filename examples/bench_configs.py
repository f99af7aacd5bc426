"""Frames/sec of the other benchmark configurations (ResNet-50 512x512, HRNet-W32 style 256x256,
CenterNet-R18 544x960), fp16, next to dense cuDNN on the same GPU: eager stepping, CUDA events.

    python examples/bench_configs.py [resnet50|hrnet|centernet ...] [--streams N] [--frames K] [--patches 0|1]

--patches 0 (default for resnet50) runs the stride-1 KxK layers on active-pixel work lists, the form for sparse maps;
--patches 1 (default for hrnet and centernet, whose randomly initialised maps saturate to fully active after the first
stages) runs them on patch tiles loaded by tiled TMA.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from examples.nets import build_pair  # noqa: E402
from deltacnn_b200.stepping import DepthPipelinedStep, MultiBranchStep, capture_groups, set_depth_thresholds  # noqa: E402
from examples.synthetic_video import make_video  # noqa: E402
from deltacnn_b200 import DCConv2d, DCThreshold  # noqa: E402


def run(name, streams, frames, input_threshold=0.03, patches=None, groups=1, stages=None):
    """``groups`` > 1: the streams are split into that many groups, each with its own model instance (own caches, same
    weights) and its own CUDA stream inside ONE captured graph, so kernels of different groups overlap (what bench.py
    does for MobileNetV2). The dense network is timed as one batch and as two concurrent half batches; the better
    one is reported. ``stages``: cut indices of a frame pipeline over the depth of the network (deltacnn_b200/stepping.py,
    DepthPipeline; the network's ``depth_stages`` says what the indices count); the pipeline is filled before the timed
    steps, and every timed step runs every layer once for every stream."""
    dev = torch.device("cuda")
    DCConv2d.patch_tiles = (name != "resnet50") if patches is None else bool(patches)
    vids = torch.stack([make_video(name, s).frames(frames + 3) for s in range(streams)], dim=1)     # (F, S, 3, H, W)
    heads = {"decode": True} if name in ("hrnet", "centernet") else {}      # key points / boxes decoded on the device
    G = max(1, min(groups, streams))
    bounds = [(g * streams) // G for g in range(G + 1)]
    fd = [vids[i].to(dev, torch.float16).contiguous(memory_format=torch.channels_last) for i in range(vids.shape[0])]
    DCThreshold.reset()
    dense, deltas = None, []
    for g in range(G):
        dense, delta = build_pair(name, vids[:4, 0], device=dev, dtype=torch.float16, **heads)
        deltas.append(delta)
    with torch.no_grad():
        for g, m in enumerate(deltas):
            sl = slice(bounds[g], bounds[g + 1])
            m(fd[0][sl])
            set_depth_thresholds(input_threshold, 0.01, 0.05, model=m)
            m(fd[1][sl])
        parts = [fd[1][bounds[g]:bounds[g + 1]] for g in range(G)]
        if stages:
            step = DepthPipelinedStep([m.depth_stages(stages) for m in deltas], parts, models=deltas)
        else:
            step = MultiBranchStep(deltas, parts)

        def load(frame):
            bufs = step.static_in
            for g in range(G):
                bufs[g].copy_(frame[bounds[g]:bounds[g + 1]], non_blocking=True)
        # frames 2, 1, 2, ... 2 before the timed ones: neighbouring frames, so every stage of a pipeline is busy
        for t in [2] + [1, 2] * ((len(stages) + 1) // 2 if stages else 0):
            load(fd[t]); step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for t in range(3, 3 + frames):
            load(fd[t]); step()
        e1.record()
        torch.cuda.synchronize()
        ms_delta = e0.elapsed_time(e1) / frames
        density = float(deltas[0].sparsify.mask.float().mean().item())
        torch.backends.cudnn.benchmark = True

        def dense_ms(parts):
            bnd = [(g * streams) // parts for g in range(parts + 1)]
            ins = [fd[0][bnd[g]:bnd[g + 1]].clone() for g in range(parts)]
            for x in ins:
                for _ in range(3):
                    dense(x)
            graph, _ = capture_groups([dense] * parts, ins)
            torch.cuda.synchronize()
            e0.record()
            for t in range(3, 3 + frames):
                for g in range(parts):
                    ins[g].copy_(fd[t][bnd[g]:bnd[g + 1]], non_blocking=True)
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / frames
        ms_dense = min(dense_ms(1), dense_ms(2) if streams >= 2 else float("inf"))
    from deltacnn_b200 import _lib
    if _lib.lib.dc_umma_error() != 0:
        raise RuntimeError(f"a bounded wait of a tensor-core kernel gave up (code {_lib.lib.dc_umma_error()})")
    return {"config": name, "streams": streams, "groups": G, "depth_stages": (len(stages) + 1) if stages else 1,
            "patch_tiles": DCConv2d.patch_tiles, "resolution": list(vids.shape[-2:]),
            "updated_input_pixels": density, "delta_fps": streams / ms_delta * 1000, "dense_cudnn_fps": streams / ms_dense * 1000,
            "ms_per_step_delta": ms_delta, "ms_per_step_dense": ms_dense}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("configs", nargs="*", default=["resnet50", "hrnet", "centernet"])
    ap.add_argument("--streams", type=int, default=4)
    ap.add_argument("--frames", type=int, default=8)
    ap.add_argument("--patches", type=int, default=None)
    ap.add_argument("--fuse-add-act", type=int, default=0, help="1: residual adds with activation run in the convolution epilogue")
    ap.add_argument("--groups", type=int, default=1, help="stream groups stepped concurrently inside one CUDA graph")
    ap.add_argument("--stages", default="", help="cut indices of a frame pipeline over the depth of the network (resnet50: into its "
                                                 "16 blocks; centernet: into 8 trunk blocks + 3 transposed convolutions)")
    a = ap.parse_args()
    DCConv2d.fuse_residual_activation = bool(a.fuse_add_act)
    cuts = [int(v) for v in a.stages.split(",") if v.strip()]
    for c in a.configs:
        print(json.dumps(run(c, a.streams, a.frames, patches=a.patches, groups=a.groups, stages=cuts or None)), flush=True)
