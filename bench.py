"""Benchmark of the delta-update inference path: MobileNetV2 224x224 fp16 over independent
synthetic video streams (about 10 % changed pixels per frame, per-layer thresholds 0.01-0.05),
frames/sec, beside dense cuDNN inference of the same network on the same GPU and the CPU
baseline. One step = one frame of every stream on this GPU (streams stacked on the batch axis,
one CUDA-graph replay). Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--streams S] [--impl reference]

N > 1 is launched with torch.distributed.run, one rank per GPU; streams are independent, so the
ranks share nothing on the data path (weak scaling: S streams per GPU).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "frames/sec (MobileNetV2 224x224 fp16 delta inference, ~10% updated pixels)"
UNIT = "frames/s"
THRESHOLDS = dict(input_threshold=0.05, first=0.01, last=0.05)
N_DISTINCT_FRAMES = 32          # per stream; played forward then backward (ping-pong) to any length


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--streams", type=int, default=64, help="streams per GPU")
    ap.add_argument("--branches", type=int, default=2, help="groups of streams stepped concurrently inside one CUDA graph")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the dense-cuDNN / CPU / reference-kernel side measurements")
    return ap.parse_args()


def pingpong(t, n):
    """Index into n distinct frames for time step t, bouncing at both ends (continuous motion)."""
    period = 2 * (n - 1)
    r = t % period
    return r if r < n else period - r


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for s in self.samples if len(s) >= 6 for i in range(4) if s[2 + i].lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons}


def make_streams(n_streams, first_seed):
    """(n_distinct, n_streams, 3, 224, 224) float32 frames of ``n_streams`` seeded videos."""
    import torch
    from examples.synthetic_video import make_video
    vids = [make_video("mobilenet", first_seed + s).frames(N_DISTINCT_FRAMES) for s in range(n_streams)]
    return torch.stack(vids, dim=1)


def cpu_delta_baseline(state_dict, frames32, seconds=15.0):
    """The CPU restatement of the delta path (oracle/, a port) on one stream, all host threads."""
    import torch
    from oracle.delta_net import build_oracle_net, Thresholds
    net = build_oracle_net("mobilenet", state_dict)
    n = frames32.shape[0]
    with torch.no_grad():
        net(frames32[0, :1])
        Thresholds.set_depth_table(**THRESHOLDS)
        net(frames32[1, :1])
        t0, done, t = time.perf_counter(), 0, 2
        while time.perf_counter() - t0 < seconds:
            net(frames32[pingpong(t, n), :1])
            t += 1
            done += 1
    dt = time.perf_counter() - t0
    return done / dt, done


def run_reference_arm(args, rank, world):
    """--impl reference: the reference's path has no CPU implementation of its own (its delta kernels
    are CUDA only), so this arm times the CPU port of it (oracle/) on the host cores."""
    if rank != 0:
        return
    import torch
    from examples.nets import build_pair
    torch.set_num_threads(os.cpu_count() or 1)
    frames = make_streams(1, 0)
    dense, _ = build_pair("mobilenet", frames[:8, 0], device="cpu")
    from oracle.delta_net import build_oracle_net, Thresholds
    net = build_oracle_net("mobilenet", dense.state_dict())
    n = frames.shape[0]
    with torch.no_grad():
        net(frames[0, :1])
        Thresholds.set_depth_table(**THRESHOLDS)
        for t in range(1, 1 + args.warmup):
            net(frames[pingpong(t, n), :1])
        steps = min(args.steps, 200)
        t0 = time.perf_counter()
        for t in range(1 + args.warmup, 1 + args.warmup + steps):
            net(frames[pingpong(t, n), :1])
        dt = time.perf_counter() - t0
    fps = steps / dt
    line = {"impl": "reference", "metric": METRIC, "value": fps, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": args.warmup, "ms_per_step": 1000 * dt / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "MobileNetV2 224x224, 1 stream, thresholds input 0.05 / layers 0.01-0.05 (CPU port of the delta path)"},
            "cpu_baseline": {"value": fps, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                             "sample": f"{steps} frames of one stream"},
            "e2e": {"value": fps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from deltacnn_b200 import DCThreshold
    from examples.nets import build_pair
    from examples.runner import MultiBranchStep, PipelinedStep, set_depth_thresholds

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    S, K_steps, W = args.streams, args.steps, max(args.warmup, 3)

    frames32 = make_streams(S, first_seed=rank * S)                     # (F, S, 3, H, W) fp32 on the host
    dense, delta = build_pair("mobilenet", frames32[:8, 0], device=dev, dtype=torch.float16)
    frames_dev = torch.stack([frames32[i].to(dev, torch.float16).contiguous(memory_format=torch.channels_last)
                              for i in range(frames32.shape[0])])
    host_frames = [frames_dev[i].cpu().pin_memory() for i in range(frames_dev.shape[0])]   # channels-last bytes, pinned
    F = frames_dev.shape[0]

    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    # The streams of this GPU are split into `branches` groups; every group has its own model instance
    # (own caches, same weights) and its own CUDA stream inside ONE captured graph, so kernels of
    # different groups overlap on the GPU and hide each other's launch and tail latencies.
    G = max(1, min(args.branches, S))
    bounds = [(g * S) // G for g in range(G + 1)]
    deltas = [delta]
    for _ in range(1, G):
        deltas.append(build_pair("mobilenet", frames32[:8, 0], device=dev, dtype=torch.float16)[1])
    with torch.no_grad():
        for g, m in enumerate(deltas):
            sl = slice(bounds[g], bounds[g + 1])
            m(frames_dev[0][sl])                                        # first frame: dense initialisation
            table = set_depth_thresholds(model=m, **THRESHOLDS)
            m(frames_dev[1][sl])                                        # one eager steady-state frame: buffers allocated
        step = MultiBranchStep(deltas, [frames_dev[1][bounds[g]:bounds[g + 1]] for g in range(G)])
    t_next = [2]

    def load(frame):
        for g in range(G):
            step.static_in[g].copy_(frame[bounds[g]:bounds[g + 1]], non_blocking=True)

    def run_steps(n):
        for _ in range(n):
            i = pingpong(t_next[0], F)
            t_next[0] += 1
            load(frames_dev[i])
            step.graph.replay()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(n, **kw):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        run_steps(n, **kw)
        e1.record(stream)
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    run_steps(W)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = timed(K_steps)
    clocks = sampler.stop() if rank == 0 else None

    # end to end through the module API: frames start in pinned host memory, logits end there; the upload
    # of the next frame overlaps the current step (two input buffers, two graphs of the same model)
    pipe = PipelinedStep(deltas, [frames_dev[1][bounds[g]:bounds[g + 1]] for g in range(G)], bounds, stream)

    def next_host_frame():
        f = host_frames[pingpong(t_next[0], F)]
        t_next[0] += 1
        return f

    def run_e2e(n):
        if pipe.uploaded == pipe.stepped:
            pipe.upload(next_host_frame())
        for _ in range(n):
            pipe.upload(next_host_frame())      # frame t+1 goes up ...
            pipe.step()                         # ... while frame t is processed

    def timed_e2e(n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        run_e2e(n)
        e1.record(stream)
        barrier()
        ms_ = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms_, op=dist.ReduceOp.MAX)
        return float(ms_.item())

    run_e2e(3)
    ms_e2e = timed_e2e(K_steps)
    d2h_bytes = sum(int(o.numel() * o.element_size()) for o in pipe.host_out[0])

    # measured fraction of updated input pixels over the frames used
    dens = []
    with torch.no_grad():
        for _ in range(4):
            run_steps(1)
            dens.append(sum(float(m.sparsify.mask.float().mean().item()) for m in deltas) / G)
    launches_per_step = count_launches(deltas, bounds, frames_dev, t_next, F)

    line = {
        "metric": METRIC, "value": world * S * K_steps / (ms / 1000.0), "unit": UNIT, "n_gpus": world, "steps": K_steps,
        "warmup": W, "ms_per_step": ms / K_steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": "configs[1]: MobileNetV2 224x224 fp16 delta inference, synthetic videos (3 moving 40x40 rectangles, sigma 0.005)",
                   "streams_per_gpu": S, "thresholds": THRESHOLDS, "updated_input_pixels": sum(dens) / len(dens),
                   "l2": "inputs larger than L2: a step touches a different frame (19 MB) and >1 GB of per-stream caches",
                   "bn": "BatchNorm calibrated on 8 frames of stream 0 and folded", "step": "one frame of every stream, one CUDA-graph replay", "concurrent_stream_groups": G},
        "e2e": {"value": world * S * K_steps / (ms_e2e / 1000.0), "unit": UNIT,
                "h2d_bytes_per_step": int(host_frames[0].numel() * host_frames[0].element_size()),
                "d2h_bytes_per_step": d2h_bytes},
        "gpu_launches": launches_per_step * K_steps,
        "clocks": clocks,
    }

    if rank == 0 and not args.no_extras and world == 1:
        line.update(side_measurements(args, dev, dense, deltas[0], frames_dev[:, bounds[0]:bounds[1]], frames_dev, frames32, stream, S, table, ms / K_steps))
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def count_launches(deltas, bounds, frames_dev, t_next, F):
    """Kernels of this library launched per step: counted by wrapping the C-ABI calls during one
    eager frame (pool = 2 launches when it updates its cache, fused conv epilogue = 2)."""
    import torch
    from deltacnn_b200 import _lib
    counts = [0]
    names = [n for n in _lib.EXPORTED_SYMBOLS if n not in ("dc_version", "dc_status_string", "dc_last_cuda_error", "dc_filter_umma_bytes", "dc_umma_error", "dc_conv_workspace_bytes", "dc_deconv_workspace_bytes", "dc_static_workspace_max_pixels")]
    originals = {}

    def wrap(name, fn):
        def inner(*a):
            counts[0] += 1
            return fn(*a)
        return inner

    for n in names:
        originals[n] = getattr(_lib.lib, n)
        setattr(_lib.lib, n, wrap(n, originals[n]))
    try:
        with torch.no_grad():
            frame = frames_dev[pingpong(t_next[0], F)]
            for g, m in enumerate(deltas):
                m(frame[bounds[g]:bounds[g + 1]])
        t_next[0] += 1
    finally:
        for n in names:
            setattr(_lib.lib, n, originals[n])
    return counts[0]


def side_measurements(args, dev, dense, delta, frames_group0, frames_dev, frames32, stream, S, table, ms_per_step):
    """Dense cuDNN baseline on the same GPU, CPU baselines, and the roofline of the dominant kernel."""
    import torch
    extra = {}
    F = frames_dev.shape[0]
    # dense cuDNN, same frames, CUDA graph; measured as one batch and as two concurrent half batches (the same
    # multi-stream treatment the delta path gets) -- the faster of the two is the baseline
    torch.backends.cudnn.benchmark = True
    from examples.runner import capture_groups

    def dense_ms(groups):
        bnd = [(g * S) // groups for g in range(groups + 1)]
        with torch.no_grad():
            ins = [frames_dev[0][bnd[g]:bnd[g + 1]].clone() for g in range(groups)]
            for x in ins:
                for _ in range(3):
                    dense(x)
            g_, _ = capture_groups([dense] * groups, ins)
            n = max(20, min(args.steps, 100))

            def go(k):
                for i in range(k):
                    f = frames_dev[i % F]
                    for g in range(groups):
                        ins[g].copy_(f[bnd[g]:bnd[g + 1]], non_blocking=True)
                    g_.replay()
            go(5)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            go(n)
            e1.record(stream)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n

    ms1, ms2 = dense_ms(1), dense_ms(2)
    dense_best = min(ms1, ms2)
    extra["dense_cudnn"] = {"value": S / (dense_best / 1000.0), "unit": UNIT, "ms_per_step": dense_best,
                            "ms_per_step_one_batch": ms1, "ms_per_step_two_concurrent_half_batches": ms2,
                            "how": f"same network, fp16 channels-last, {S} frames per step, cudnn.benchmark, CUDA graph"}
    extra["speedup_vs_dense_cudnn"] = dense_best / ms_per_step

    # CPU baselines on a bounded sample
    torch.set_num_threads(os.cpu_count() or 1)
    from examples.nets import build_pair
    dense_cpu, _ = build_pair("mobilenet", frames32[:8, 0], device="cpu")
    fps_port, n_port = cpu_delta_baseline(dense_cpu.state_dict(), frames32, seconds=12.0)
    extra["cpu_baseline"] = {"value": fps_port, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                             "sample": f"{n_port} frames of one stream through the CPU restatement of the delta path (oracle/)"}
    with torch.no_grad():
        for _ in range(3):
            dense_cpu(frames32[0, :1])
        t0, k = time.perf_counter(), 0
        while time.perf_counter() - t0 < 5.0:
            dense_cpu(frames32[k % F, :1]); k += 1
        extra["dense_cpu"] = {"value": k / (time.perf_counter() - t0), "unit": UNIT, "cores": torch.get_num_threads(),
                              "how": "dense PyTorch fp32 network, batch 1"}
    try:
        from examples.profile import roofline_of_dominant_kernel
        extra["roofline"] = roofline_of_dominant_kernel(delta, frames_group0, stream, peaks())
    except Exception as e:          # the roofline is reporting, never a reason to lose the bench line
        extra["roofline"] = {"error": repr(e)}
    return extra


if __name__ == "__main__":
    main()
