"""Benchmark of the delta-update inference path: MobileNetV2 224x224 fp16 over independent
synthetic video streams (about 10 % changed pixels per frame, per-layer thresholds 0.01-0.05),
frames/sec, beside dense cuDNN inference of the same network on the same GPU and the CPU
baseline. One step = one frame of every stream on this GPU (streams stacked on the batch axis,
one CUDA-graph replay). Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--streams S] [--total-streams T] [--impl reference]

N > 1 is launched with torch.distributed.run, one rank per GPU; streams are independent, so the
ranks share nothing on the data path. Default: S streams per GPU (weak scaling). With --total-streams T
the T streams of the job are dealt to the ranks round-robin (stream s runs on rank s mod N; strong scaling).
The timed block of K steps is repeated (--repeats) and the median is reported.
"""
import argparse
import hashlib
import json
import os
import struct
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The launcher gives every rank of a multi-GPU run a host thread pool of size one (OMP_NUM_THREADS=1). The CPU libraries
# then take other kernels for the BatchNorm calibration than in a single-GPU run, the folded weights differ in their last
# bits, and the output checksums of the same streams could not be compared between partitions. A small pool (set before
# torch is imported) keeps the calibration identical; the hot path does not use host threads.
if os.environ.get("OMP_NUM_THREADS") == "1" and "LOCAL_RANK" in os.environ:
    os.environ["OMP_NUM_THREADS"] = "4"

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
    ap.add_argument("--total-streams", type=int, default=0, help="streams of the whole job, dealt round-robin to the GPUs (0: --streams per GPU)")
    ap.add_argument("--branches", type=int, default=1, help="groups of streams stepped concurrently inside one CUDA graph")
    ap.add_argument("--stages", default="6,10,14",
                    help="frame pipeline over the depth of the network: indices into the network's feature blocks where a new "
                         "stage starts (stage s of a step works on the frame of s steps ago); empty: no pipeline")
    ap.add_argument("--repeats", type=int, default=5, help="repetitions of the timed block of --steps steps (median reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the dense-cuDNN / CPU / reference-kernel / roofline side measurements")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the ResNet-50 / HRNet / CenterNet side measurements")
    return ap.parse_args()


def pingpong(t, n):
    """Index into n distinct frames for time step t, bouncing at both ends (continuous motion)."""
    period = 2 * (n - 1)
    r = t % period
    return r if r < n else period - r


def stream_ids(rank, world, streams_per_gpu, total_streams=0):
    """Global ids (= video seeds) of the streams of ``rank``: a contiguous block of ``streams_per_gpu``, or with
    ``total_streams`` the ids s < total_streams with s mod world == rank."""
    if total_streams > 0:
        return [s for s in range(total_streams) if s % world == rank]
    return list(range(rank * streams_per_gpu, (rank + 1) * streams_per_gpu))


def stream_checksums(outputs):
    """One float64 number per stream (row) of a step's output: the sum of its elements."""
    return outputs.detach().double().reshape(outputs.shape[0], -1).sum(dim=1).cpu().tolist()


def combine_checksums(ids, sums):
    """Digest of per-stream checksums that does not depend on how the streams were dealt to ranks: sorted by
    stream id, packed as (id, float64) pairs, SHA-256."""
    h = hashlib.sha256()
    for i, v in sorted(zip(ids, sums)):
        h.update(struct.pack("<qd", int(i), float(v)))
    return h.hexdigest()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "50",
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
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def make_streams(n_streams, first_seed=0, seeds=None):
    """(n_distinct, n_streams, 3, 224, 224) float32 frames of seeded videos, quantised to the 256 levels of 8-bit
    video (the end-to-end leg uploads them as bytes); ``seeds`` lists the stream ids, default first_seed ..."""
    import torch
    from examples.synthetic_video import make_video
    seeds = list(range(first_seed, first_seed + n_streams)) if seeds is None else list(seeds)
    vids = [make_video("mobilenet", s).frames(N_DISTINCT_FRAMES) for s in seeds]
    frames = torch.stack(vids, dim=1)
    return torch.round(frames * 255.0) * (1.0 / 255.0)     # level * float32(1/255): the arithmetic of the 8-bit sparsify kernel


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
    are CUDA only), so this arm times the CPU port of it (oracle/) on the host cores. Nothing of the
    product is imported here: the dense network comes from examples.nets, which does not load the CUDA library."""
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
    assert "deltacnn_b200" not in sys.modules, "the reference arm must not load the product"
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
    from examples.nets import build_pair
    from deltacnn_b200.stepping import DepthPipeline, DepthPipelinedStep, MultiBranchStep, PipelinedStep, set_depth_thresholds

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ids = stream_ids(rank, world, args.streams, args.total_streams)
    S, K_steps, W = len(ids), args.steps, max(args.warmup, 3)
    total_streams = args.total_streams if args.total_streams > 0 else world * args.streams

    frames32 = make_streams(S, seeds=ids)                               # (F, S, 3, H, W) fp32 on the host, 8-bit levels
    calib = make_streams(1, 0)[:8, 0]                                   # BatchNorm is calibrated on stream 0 on every rank
    dense, delta = build_pair("mobilenet", calib, device=dev, dtype=torch.float16)
    frames_dev = torch.stack([frames32[i].to(dev, torch.float16).contiguous(memory_format=torch.channels_last)
                              for i in range(frames32.shape[0])])
    # the same frames as bytes, N,H,W,C, in pinned host memory: what the end-to-end leg uploads
    host_frames = [torch.round(frames32[i] * 255.0).to(torch.uint8).permute(0, 2, 3, 1).contiguous().pin_memory()
                   for i in range(frames32.shape[0])]
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
        deltas.append(build_pair("mobilenet", calib, device=dev, dtype=torch.float16)[1])
    for m in deltas:
        m.sparsify.set_u8_input(1.0 / 255.0, 0.0, torch.float16)      # 8-bit frames go straight into the sparsify kernel
    with torch.no_grad():
        for g, m in enumerate(deltas):
            sl = slice(bounds[g], bounds[g + 1])
            m(frames_dev[0][sl])                                        # first frame: dense initialisation
            table = set_depth_thresholds(model=m, **THRESHOLDS)
            m(frames_dev[1][sl])                                        # one eager steady-state frame: buffers allocated
        # With --stages every group's network is also cut into depth stages that work on consecutive frames at the
        # same time (deltacnn_b200/stepping.py, DepthPipeline): every step still runs every layer once for every stream, and
        # the logits a step returns belong to the frame of len(cuts) steps earlier.
        cuts = [int(v) for v in args.stages.split(",") if v.strip()]
        if cuts:
            step = DepthPipelinedStep([m.depth_stages(cuts) for m in deltas], [frames_dev[1][bounds[g]:bounds[g + 1]] for g in range(G)],
                                      models=deltas)
        else:
            step = MultiBranchStep(deltas, [frames_dev[1][bounds[g]:bounds[g + 1]] for g in range(G)])
    t_next = [2]
    last_frame = [frames_dev[1]]

    def load(frame):
        bufs = step.static_in
        for g in range(G):
            bufs[g].copy_(frame[bounds[g]:bounds[g + 1]], non_blocking=True)
        last_frame[0] = frame

    def run_steps(n):
        for _ in range(n):
            i = pingpong(t_next[0], F)
            t_next[0] += 1
            load(frames_dev[i])
            step()

    def drained_outputs():
        """Outputs that belong to the last loaded frame (the pipeline, if any, emptied by repeating that frame)."""
        if cuts:
            return step.drain([last_frame[0][bounds[g]:bounds[g + 1]] for g in range(G)])
        return step.static_out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        fn(n)
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
    reps = sorted(timed(run_steps, K_steps) for _ in range(max(1, args.repeats)))
    ms = reps[len(reps) // 2]

    # checksum of the outputs after the same number of steps on every run: comparable between runs that deal the
    # same streams differently to GPUs
    with torch.no_grad():
        out_now = torch.cat([o.float() for o in drained_outputs()], dim=0)
    sums = stream_checksums(out_now)
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, (ids, sums))
        all_ids = [i for part in gathered for i in part[0]]
        all_sums = [v for part in gathered for v in part[1]]
    else:
        all_ids, all_sums = ids, sums
    checksum = {"sha256_over_streams": combine_checksums(all_ids, all_sums), "streams": len(all_ids),
                "rank0_sum": float(sum(sums)), "steps_run": t_next[0] - 2,
                "first_streams": {str(i): v for i, v in sorted(zip(all_ids, all_sums))[:8]}}

    # end to end through the module API: 8-bit frames start in pinned host memory, logits end there; the upload
    # of the next frame overlaps the current step (two input buffers, two graphs of the same model)
    u8_example = [host_frames[1][bounds[g]:bounds[g + 1]].to(dev) for g in range(G)]
    with torch.no_grad():
        for g, m in enumerate(deltas):
            m(u8_example[g])                                            # one eager 8-bit frame before capture
    if cuts:
        depth_pipe = DepthPipeline([m.depth_stages(cuts) for m in deltas], u8_example, models=deltas)
        pipe = PipelinedStep(deltas, u8_example, bounds, stream, capture=depth_pipe.capture)
    else:
        pipe = PipelinedStep(deltas, u8_example, bounds, stream)

    def next_host_frame():
        f = host_frames[pingpong(t_next[0], F)]
        t_next[0] += 1
        return f

    def run_e2e(n):
        if pipe.uploaded == pipe.stepped:
            pipe.upload(next_host_frame())
        for _ in range(n):
            pipe.upload(next_host_frame())      # frame t+1 goes up ...
            pipe.step()                         # ... while frame t is processed and the result of frame t-1 comes down
        pipe.join()                             # the timed region ends when the last result has reached the host

    run_e2e(3)
    reps_e2e = sorted(timed(run_e2e, K_steps) for _ in range(max(1, args.repeats)))
    ms_e2e = reps_e2e[len(reps_e2e) // 2]
    clocks = sampler.stop() if rank == 0 else None
    d2h_bytes = sum(int(o.numel() * o.element_size()) for o in pipe.host_out[0])

    # measured fraction of updated input pixels over the frames used
    dens = []
    with torch.no_grad():
        for _ in range(4):
            run_steps(1)
            dens.append(sum(float(m.sparsify.mask.float().mean().item()) for m in deltas) / G)
        drained_outputs()
    launches_per_step = count_launches(deltas, bounds, frames_dev, t_next, F)

    # the same streams without the depth pipeline (two stream groups side by side): what the pipeline buys
    unpipelined = None
    if cuts and rank == 0 and world == 1 and not args.no_extras:
        with torch.no_grad():
            plain_models = [build_pair("mobilenet", calib, device=dev, dtype=torch.float16)[1] for _ in range(2)]
            half = [0, S // 2, S]
            for g, m in enumerate(plain_models):
                sl = slice(half[g], half[g + 1])
                m(frames_dev[0][sl])
                set_depth_thresholds(model=m, **THRESHOLDS)
                m(frames_dev[1][sl])
            plain = MultiBranchStep(plain_models, [frames_dev[1][half[g]:half[g + 1]] for g in range(2)])

        def run_plain(n):
            for k in range(n):
                f = frames_dev[pingpong(2 + k, F)]
                plain.load([f[half[g]:half[g + 1]] for g in range(2)])
                plain.graph.replay()

        run_plain(W)
        reps_plain = sorted(timed(run_plain, K_steps) for _ in range(3))
        unpipelined = {"value": total_streams * K_steps / (reps_plain[1] / 1000.0), "unit": UNIT, "ms_per_step": reps_plain[1] / K_steps,
                       "concurrent_stream_groups": 2, "what": "every step runs one frame through the whole network before the next starts"}
        del plain, plain_models

    line = {
        "metric": METRIC, "value": total_streams * K_steps / (ms / 1000.0), "unit": UNIT, "n_gpus": world, "steps": K_steps,
        "warmup": W, "ms_per_step": ms / K_steps, "higher_is_better": True,
        "scaling": "strong" if args.total_streams > 0 else "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": "configs[1]: MobileNetV2 224x224 fp16 delta inference, synthetic videos (3 moving 40x40 rectangles, sigma 0.005, 8-bit levels)",
                   "streams_per_gpu": S, "total_streams": total_streams,
                   "partition": "stream s on rank s mod N" if args.total_streams > 0 else "rank r runs streams r*S .. r*S+S-1",
                   "thresholds": THRESHOLDS, "updated_input_pixels": sum(dens) / len(dens),
                   "l2": "inputs larger than L2: a step touches a different frame (19 MB) and >1 GB of per-stream caches",
                   "bn": "BatchNorm calibrated on 8 frames of stream 0 and folded", "step": "one frame of every stream, one CUDA-graph replay",
                   "head": "classifier on the pooled delta (DCLinear), logits per stream", "concurrent_stream_groups": G,
                   "depth_pipeline": ({"stages": len(cuts) + 1, "cuts_in_feature_blocks": cuts, "latency_steps": len(cuts),
                                       "what": "every step runs every layer once for all streams; stage s works on the frame of s steps "
                                               "earlier, the stages are concurrent branches of the step's CUDA graph; the checksum is taken "
                                               "after the pipeline has been emptied"} if cuts else None)},
        "repeats": {"n": len(reps), "ms_per_step_min": reps[0] / K_steps, "ms_per_step_median": ms / K_steps,
                    "ms_per_step_max": reps[-1] / K_steps, "timed_region_ms_total": sum(reps)},
        "e2e": {"value": total_streams * K_steps / (ms_e2e / 1000.0), "unit": UNIT,
                "h2d_bytes_per_step": int(host_frames[0].numel() * host_frames[0].element_size()),
                "d2h_bytes_per_step": d2h_bytes, "input": "uint8 N,H,W,C frames from pinned host memory, normalised inside the sparsify kernel",
                "ms_per_step_min": reps_e2e[0] / K_steps, "ms_per_step_max": reps_e2e[-1] / K_steps},
        "gpu_launches": launches_per_step * K_steps,
        "output_checksum": checksum,
        "clocks": clocks,
    }
    if unpipelined is not None:
        line["unpipelined"] = unpipelined

    if rank == 0 and not args.no_extras and world == 1:
        line.update(side_measurements(args, dev, dense, deltas[0], frames_dev[:, bounds[0]:bounds[1]], frames_dev, frames32, stream, S,
                                      ms / K_steps, (bounds[1] - bounds[0]) / S))
        if "layer_density" in line:
            line["config"]["layer_density"] = line.pop("layer_density")
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def count_launches(deltas, bounds, frames_dev, t_next, F):
    """Kernels of this library launched per step: the C-ABI calls of one eager frame, or the library's kernels the
    profiler saw during one eager frame where that is more."""
    import torch
    from deltacnn_b200 import _lib
    counts = [0]
    skip = ("dc_version", "dc_status_string", "dc_last_cuda_error", "dc_filter_umma_bytes", "dc_umma_error", "dc_conv_workspace_bytes",
            "dc_deconv_workspace_bytes", "dc_static_workspace_max_pixels")
    names = [n for n in _lib.EXPORTED_SYMBOLS if n not in skip]
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
    # A call can launch more than one kernel (a layer wider than 256 channels truncates in a second kernel): where the
    # profiler is available, count the library's kernels (namespace dc) of one more eager frame instead of its calls.
    kernels = 0
    try:
        import warnings
        from torch.profiler import profile, ProfilerActivity
        with warnings.catch_warnings(), torch.no_grad(), profile(activities=[ProfilerActivity.CUDA]) as prof:
            warnings.simplefilter("ignore")
            frame = frames_dev[pingpong(t_next[0], F)]
            for g, m in enumerate(deltas):
                m(frame[bounds[g]:bounds[g + 1]])
            torch.cuda.synchronize()
        t_next[0] += 1
        kernels = sum(1 for e in prof.events() if "dc::" in e.name)
    except Exception:
        kernels = 0
    return max(counts[0], kernels)


def reference_kernels_gpu(delta, frames_group0, stream):
    """The reference's own CUDA kernels (built for this GPU by oracle/Makefile, test infrastructure) timed beside
    this library's on the same tensors and masks of one eager frame: one representative layer per kernel family.
    Per launch: L2 flushed, CUDA events on the stream the kernel runs on (the reference launches on the legacy
    default stream). The reference has no fused convolution epilogue, so its side of a fused layer is convolution
    plus activate_truncate."""
    import ctypes
    import torch
    import deltacnn_b200.cuda_kernels as K
    from oracle import ref_kernels as R
    if not R.available():
        return {"unavailable": "oracle/_ref/libdeltacnn_ref.so is not built"}
    lib = R.lib()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    legacy = torch.cuda.default_stream()
    captured = {}
    orig_conv, orig_sparsify = K.sparse_conv, K.sparsify
    want = {"stem 3x3/2 3->32 @224": (3, 32, 3), "depthwise 3x3 96 @112 s2": (96, 96, 3), "1x1 16->96 @112 (+act)": (16, 96, 1),
            "1x1 96->576 @14 (+act)": (96, 576, 1), "depthwise 3x3 576 @14": (576, 576, 3), "1x1 576->96 @14": (576, 96, 1)}

    def conv_hook(*a, **kw):
        x, filt = kw["x"], kw["filter"]
        for name, (ci, co, k) in want.items():
            if name not in captured and x.shape[1] == ci and filt.shape[3] == co and filt.shape[0] == k and \
                    ((name.endswith("@14") or "@14 " in name) == (x.shape[2] == 14)):
                ep = kw.get("epilogue")
                captured[name] = dict(kw, x=x.clone(), mask=kw["mask"].clone(), epilogue=ep)
        return orig_conv(*a, **kw)

    def sparsify_hook(inp, prev, d, m, thr):
        captured.setdefault("sparsify 3 @224", (inp.clone(), prev.clone(), thr))
        return orig_sparsify(inp, prev, d, m, thr)

    K.sparse_conv, K.sparsify = conv_hook, sparsify_hook
    try:
        with torch.no_grad():
            delta(frames_group0[5])
    finally:
        K.sparse_conv, K.sparsify = orig_conv, orig_sparsify

    def time_on(st, fn, reps=5):
        best = []
        for _ in range(reps):
            with torch.cuda.stream(st):
                flush.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(st)
                fn()
                e1.record(st)
            torch.cuda.synchronize()
            best.append(e0.elapsed_time(e1) * 1000.0)
        best.sort()
        return best[len(best) // 2]

    out = {}
    layers = {id(m): m for m in delta.modules()}
    convs = [m for m in delta.modules() if hasattr(m, "orig_weights") and m.orig_weights is not None]
    for name, c in captured.items():
        if name.startswith("sparsify"):
            x, prev, thr = c
            n, ch, h, w = x.shape
            d, m = torch.empty_like(x), torch.empty((n, 1, h, w), dtype=torch.int32, device=x.device)
            p1, p2 = prev.clone(), prev.clone()
            ours = time_on(stream, lambda: orig_sparsify(x, p1, d, m, thr))
            ref = time_on(legacy, lambda: lib.ref_sparsify(1, R._p(x), R._p(p2), R._p(d), R._p(m), ctypes.c_float(thr), n, h, w, ch, 0))
            out[name] = {"ours_us": round(ours, 2), "ref_us": round(ref, 2), "ref_kernel": "deltacnn_prepare_diff_mask_hp_kernel"}
            continue
        x, mask, filt = c["x"], c["mask"], c["filter"]
        conv = next(m for m in convs if m.weight.data_ptr() == filt.data_ptr())
        wt = conv.orig_weights                                        # torch layout
        n, ci, h, w = x.shape
        co = filt.shape[3]
        k = filt.shape[0]
        ho, wo = c["out"].shape[2], c["out"].shape[3]
        ep = c.get("epilogue")
        act = conv.activation_layer
        prev_o, trunc_o = (act.prev_out.clone(), act.out_truncated.clone()) if (ep is not None and act is not None) else (None, None)
        kw = dict(c)
        if ep is not None and act is not None:
            from deltacnn_b200 import DCThreshold
            kw["epilogue"] = K.make_epilogue(prev_o, trunc_o, DCThreshold.get(act), act.activation_int, 0)
        out_t, om_t = torch.empty_like(c["out"]), torch.empty_like(c["out_mask"])
        kw.update(out=out_t, out_mask=om_t)
        ours = time_on(stream, lambda: orig_conv(**kw))
        rf = R.ref_filter(wt)
        shape = R._ints(n, h, w, ci, ho, wo, co)
        pt, pb, pl, pr = K._pad4(c["padding"])
        geom = R._ints(k, k, c["stride"][0], c["stride"][1], pt, pl, pb, pr, 1, 1, c["groups"])
        ro = torch.empty_like(c["out"])
        rm = torch.empty_like(c["out_mask"])
        ref_conv = time_on(legacy, lambda: lib.ref_conv(1, R._p(x), R._p(ro), R._p(rf), R._p(None), R._p(mask), R._p(rm), shape, geom, 0))
        row = {"ours_us": round(ours, 2), "ref_conv_us": round(ref_conv, 2)}
        if ep is not None and act is not None:
            from deltacnn_b200 import DCThreshold
            p2, t2 = act.prev_out.clone(), act.out_truncated.clone()
            thr = float(DCThreshold.get(act))

            def ref_act():
                lib.ref_activate_truncate(1, R._p(ro), R._p(p2), R._p(t2), R._p(rm), ctypes.c_float(thr), n, ho, wo, co, act.activation_int, 0, 0)
            ref_conv_only = ref_conv
            lib.ref_conv(1, R._p(x), R._p(ro), R._p(rf), R._p(None), R._p(mask), R._p(rm), shape, geom, 1)
            row["ref_act_us"] = round(time_on(legacy, ref_act, reps=1), 2)      # once: the call consumes its mask
            row["ref_us"] = round(ref_conv_only + row["ref_act_us"], 2)
        else:
            row["ref_us"] = row["ref_conv_us"]
        if ep is not None and getattr(ep, "residual", None):
            row["ours_includes"] = "the residual add of the block (DCAdd) in the same kernel"
        row["active_input_pixels"] = round(float((mask != 0).float().mean().item()), 4)
        out[name] = row
    out["how"] = "one layer per kernel family, 32 streams, per-launch CUDA events with L2 flushed (cold, serialised); the reference's side of a fused layer is its convolution plus its activate_truncate kernel"
    return out


def other_configs():
    """Frames/sec of the other three configurations (fp16, CUDA graph on both sides) beside dense cuDNN."""
    import torch
    from examples import bench_configs
    from deltacnn_b200 import DCConv2d, DCThreshold
    out = {}
    # every configuration runs as a frame pipeline over its depth, like the MobileNetV2 step (cut indices: see the
    # network's depth_stages in examples/nets.py)
    for name, streams, cuts in (("resnet50", 16, [3, 7, 11, 14]), ("hrnet", 32, [1, 3, 5, 7, 9]), ("centernet", 32, [3, 7, 9])):
        try:
            DCThreshold.reset()
            r = bench_configs.run(name, streams, 6, stages=cuts)
            out[name] = {k: r[k] for k in ("streams", "resolution", "updated_input_pixels", "delta_fps", "dense_cudnn_fps", "patch_tiles",
                                           "depth_stages")}
            out[name]["speedup_vs_dense_cudnn"] = r["delta_fps"] / r["dense_cudnn_fps"]
        except Exception as e:
            out[name] = {"error": repr(e)}
        finally:
            DCConv2d.patch_tiles = False
            torch.cuda.empty_cache()
    return out


def config1_fp32(frames32, dev):
    """Configuration 1: MobileNetV2 fp32, batch 1, CUDA graph (the generic CUDA-core kernels), frames/sec at threshold 0.05."""
    import torch
    from deltacnn_b200 import DCThreshold
    from examples.nets import build_pair
    from deltacnn_b200.stepping import GraphedStep
    DCThreshold.reset()
    DCThreshold.t_default = 0.05
    try:
        dense, delta = build_pair("mobilenet", frames32[:8, 0], device=dev)
        fd = [frames32[i, :1].to(dev).contiguous(memory_format=torch.channels_last) for i in range(frames32.shape[0])]
        with torch.no_grad():
            delta(fd[0])
            step = GraphedStep(delta, fd[1], warmup_frames=[fd[1]])
            for t in range(2, 6):
                step(fd[t])
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n = 64
            e0.record()
            for t in range(n):
                step(fd[pingpong(6 + t, len(fd))])
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / n
            g = torch.cuda.CUDAGraph()
            static = fd[0].clone()
            for _ in range(3):
                dense(static)
            torch.cuda.synchronize()
            with torch.cuda.graph(g):
                dense(static)
            e0.record()
            for t in range(n):
                static.copy_(fd[pingpong(6 + t, len(fd))])
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            ms_dense = e0.elapsed_time(e1) / n
        return {"value": 1000.0 / ms, "unit": UNIT, "ms_per_frame": ms, "dense_cudnn_fp32_fps": 1000.0 / ms_dense,
                "how": "MobileNetV2 224x224 fp32, 1 stream, every threshold 0.05, CUDA graph, 64 frames"}
    finally:
        DCThreshold.t_default = 0.0
        DCThreshold.reset()


def side_measurements(args, dev, dense, delta, frames_group0, frames_dev, frames32, stream, S, ms_per_step, group_fraction):
    """Dense cuDNN baseline on the same GPU, CPU baselines, the reference's kernels on the same layers, the roofline
    of the dominant kernel and of the whole step, the other configurations."""
    import torch
    extra = {}
    F = frames_dev.shape[0]
    # dense cuDNN, same frames, CUDA graph; measured as one batch and as two concurrent half batches (the same
    # multi-stream treatment the delta path gets) -- the faster of the two is the baseline
    torch.backends.cudnn.benchmark = True
    from deltacnn_b200.stepping import capture_groups

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
    dense_cpu, _ = build_pair("mobilenet", make_streams(1, 0)[:8, 0], device="cpu")
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
    hbm, tensor, kind = peaks()
    for key, fn in (("roofline", lambda: None), ("ref_kernels_gpu", lambda: reference_kernels_gpu(delta, frames_group0, stream)),
                    ("config1_fp32", lambda: config1_fp32(frames32, dev))):
        try:                        # side measurements are reporting, never a reason to lose the bench line
            if key == "roofline":
                from examples.profile import roofline_report
                extra["roofline"], extra["layer_density"] = roofline_report(delta, frames_group0, stream, (hbm, kind), tensor, ms_per_step,
                                                                            group_fraction)
            else:
                extra[key] = fn()
        except Exception as e:
            extra[key] = {"error": repr(e)}
    if not args.no_other_configs:
        try:
            extra["other_configs"] = other_configs()
        except Exception as e:
            extra["other_configs"] = {"error": repr(e)}
    return extra


if __name__ == "__main__":
    main()
