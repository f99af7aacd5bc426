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
from examples.runner import GraphedStep, set_depth_thresholds  # noqa: E402
from examples.synthetic_video import make_video  # noqa: E402
from deltacnn_b200 import DCConv2d, DCThreshold  # noqa: E402


def run(name, streams, frames, input_threshold=0.03, patches=None):
    dev = torch.device("cuda")
    DCConv2d.patch_tiles = (name != "resnet50") if patches is None else bool(patches)
    vids = torch.stack([make_video(name, s).frames(frames + 3) for s in range(streams)], dim=1)     # (F, S, 3, H, W)
    heads = {"decode": True} if name in ("hrnet", "centernet") else {}      # key points / boxes decoded on the device
    dense, delta = build_pair(name, vids[:4, 0], device=dev, dtype=torch.float16, **heads)
    fd = [vids[i].to(dev, torch.float16).contiguous(memory_format=torch.channels_last) for i in range(vids.shape[0])]
    DCThreshold.reset()
    with torch.no_grad():
        delta(fd[0])
        set_depth_thresholds(input_threshold, 0.01, 0.05)
        step = GraphedStep(delta, fd[1], warmup_frames=[fd[1]])
        step(fd[2])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for t in range(3, 3 + frames):
            step(fd[t])
        e1.record()
        torch.cuda.synchronize()
        ms_delta = e0.elapsed_time(e1) / frames
        density = float(delta.sparsify.mask.float().mean().item())
        torch.backends.cudnn.benchmark = True
        static = fd[0].clone()
        for _ in range(3):
            dense(static)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            dense(static)
        e0.record()
        for t in range(3, 3 + frames):
            static.copy_(fd[t]); g.replay()
        e1.record()
        torch.cuda.synchronize()
        ms_dense = e0.elapsed_time(e1) / frames
    return {"config": name, "streams": streams, "patch_tiles": DCConv2d.patch_tiles, "resolution": list(vids.shape[-2:]), "updated_input_pixels": density,
            "delta_fps": streams / ms_delta * 1000, "dense_cudnn_fps": streams / ms_dense * 1000,
            "ms_per_step_delta": ms_delta, "ms_per_step_dense": ms_dense}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("configs", nargs="*", default=["resnet50", "hrnet", "centernet"])
    ap.add_argument("--streams", type=int, default=4)
    ap.add_argument("--frames", type=int, default=8)
    ap.add_argument("--patches", type=int, default=None)
    ap.add_argument("--fuse-add-act", type=int, default=0, help="1: residual adds with activation run in the convolution epilogue")
    a = ap.parse_args()
    DCConv2d.fuse_residual_activation = bool(a.fuse_add_act)
    for c in a.configs:
        print(json.dumps(run(c, a.streams, a.frames, patches=a.patches)), flush=True)
