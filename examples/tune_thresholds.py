"""Tunes the per-layer thresholds of the benchmark's MobileNetV2 front to back on seeded synthetic streams
(deltacnn_b200.tuning, the procedure of the reference's readme.md:193-214) and writes ``thresholds_<name>.json`` in
the format DCThreshold.load_thresholds reads, beside the per-layer mask densities the table produces.

    python examples/tune_thresholds.py [--streams 4] [--frames 12] [--budget 1.02] [--name mobilenet_tuned]

The loss is the mean over frames of max|logits_delta - logits_dense| / max|logits_dense| (fp16 delta network
against the dense fp16 network of the same weights)."""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--streams", type=int, default=4)
    ap.add_argument("--frames", type=int, default=12)
    ap.add_argument("--budget", type=float, default=1.02, help="allowed loss factor per layer")
    ap.add_argument("--name", default="mobilenet_tuned")
    ap.add_argument("--out-dir", default=".")
    args = ap.parse_args()
    from deltacnn_b200 import DCThreshold
    from deltacnn_b200.tuning import tune_thresholds
    from examples.nets import build_pair
    from examples.synthetic_video import make_video
    dev = torch.device("cuda")
    vids = torch.stack([make_video("mobilenet", s).frames(args.frames) for s in range(args.streams)], dim=1)
    dense, delta = build_pair("mobilenet", vids[:8, 0], device=dev, dtype=torch.float16)
    frames = [vids[t].to(dev, torch.float16).contiguous(memory_format=torch.channels_last) for t in range(args.frames)]
    with torch.no_grad():
        refs = [dense(f).float() for f in frames]
        delta(frames[0])                         # registers every layer's threshold

    def calc_loss():
        delta.reset_layers()
        tot = 0.0
        with torch.no_grad():
            for f, r in zip(frames, refs):
                tot += ((delta(f).float() - r).abs().max() / r.abs().max()).item()
        return tot / len(frames)

    base = calc_loss()
    table = tune_thresholds(calc_loss, start=1e-3, step=2.0, max_loss_increase=args.budget, abs_slack=1e-3, log=print)
    final = calc_loss()
    cwd = os.getcwd()
    os.makedirs(args.out_dir, exist_ok=True)
    os.chdir(args.out_dir)
    try:
        DCThreshold.save_thresholds(args.name)
    finally:
        os.chdir(cwd)
    # input-mask density of the tuned table over the sequence
    dens = []
    delta.reset_layers()
    with torch.no_grad():
        for i, f in enumerate(frames):
            delta(f)
            if i > 0:
                dens.append(float(delta.sparsify.mask.float().mean().item()))
    summary = {"thresholds": table, "loss_at_zero_thresholds": base, "loss_tuned": final, "updated_input_pixels": sum(dens) / len(dens),
               "streams": args.streams, "frames": args.frames, "budget_per_layer": args.budget}
    with open(os.path.join(args.out_dir, f"thresholds_{args.name}_summary.json"), "w") as f:
        json.dump(summary, f, indent=1)
    print(json.dumps(summary))


if __name__ == "__main__":
    main()
