"""Frame-step driver for a batch of independent video streams: first (dense) frame, threshold
table, and a CUDA-graph replay of the steady-state delta step."""
import torch

from deltacnn_b200 import DCThreshold, DCSparsify


def set_depth_thresholds(input_threshold=0.05, first=0.01, last=0.05, model=None):
    """Overwrite the registered thresholds (call after the first frame): the input DCSparsify gets
    ``input_threshold``; the activation layers get values rising linearly with depth from
    ``first`` to ``last``. With ``model`` only that model's layers are touched (several models may be
    registered at once). Returns the table as a list in registration order."""
    own = None if model is None else set(model.modules())
    keys = [k for k in DCThreshold.t.keys() if own is None or k in own]
    acts = [k for k in keys if not isinstance(k, DCSparsify)]
    table = []
    for k in keys:
        if isinstance(k, DCSparsify):
            v = input_threshold
        else:
            i = acts.index(k)
            v = first + (last - first) * (i / max(len(acts) - 1, 1))
        DCThreshold.t[k] = v
        table.append(v)
    return table


class GraphedStep:
    """Captures ``model(static_input)`` once and replays it per frame. The model must already have
    processed its first frame (caches allocated) and one eager steady-state frame (buffers
    allocated) before capture."""

    def __init__(self, model, example_input, warmup_frames=()):
        self.model = model
        self.static_in = example_input.clone()
        self.stream = torch.cuda.Stream()
        with torch.no_grad():
            for f in warmup_frames:
                self.model(f)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                self.static_out = self.model(self.static_in)

    def __call__(self, frame=None, non_blocking=True):
        if frame is not None:
            self.static_in.copy_(frame, non_blocking=non_blocking)
        self.graph.replay()
        return self.static_out


class MultiBranchStep:
    """One CUDA graph that steps several groups of streams concurrently: every group has its own model
    instance (own caches) and its own CUDA stream inside the capture, so the kernels of different groups
    overlap on the GPU. Streams of a video never interact, so the groups share nothing but the weights'
    values. Each model must already have processed its first frame and one steady-state frame."""

    def __init__(self, models, example_inputs):
        self.models = models
        self.static_in = [x.clone() for x in example_inputs]
        self.main = torch.cuda.Stream()
        self.side = [torch.cuda.Stream() for _ in models[1:]]
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph, stream=self.main):
            fork = torch.cuda.Event()
            fork.record(self.main)
            outs = [None] * len(models)
            joins = []
            for i, s in enumerate(self.side):
                s.wait_event(fork)
                with torch.cuda.stream(s):
                    outs[i + 1] = models[i + 1](self.static_in[i + 1])
                    ev = torch.cuda.Event()
                    ev.record(s)
                    joins.append(ev)
            outs[0] = models[0](self.static_in[0])
            for ev in joins:
                self.main.wait_event(ev)
        self.static_out = outs

    def load(self, frames, non_blocking=True):
        for dst, src in zip(self.static_in, frames):
            dst.copy_(src, non_blocking=non_blocking)

    def __call__(self, frames=None):
        if frames is not None:
            self.load(frames)
        self.graph.replay()
        return self.static_out
