"""Stepping many independent video streams through a delta network (host side; no reference counterpart: the
reference's examples call the model once per frame, example/mobilenet_deltacnn.py): the threshold table by depth, the
CUDA-graph replay of a steady-state frame step, several stream groups or several depth stages of the network as concurrent
branches of one graph, and double-buffered stepping from pinned host memory. Nothing here changes a layer's results."""
import torch

from .sparse_layers import DCThreshold, DCSparsify


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


def capture_groups(models, inputs, pool=None):
    """Capture one CUDA graph that runs ``models[g](inputs[g])`` for every group g, each group on its own
    stream inside the capture (fork from / join into the capturing stream), so kernels of different
    groups may overlap. Returns (graph, outputs)."""
    main = torch.cuda.Stream()
    side = [torch.cuda.Stream() for _ in models[1:]]
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.no_grad(), torch.cuda.graph(graph, stream=main, pool=pool):
        fork = torch.cuda.Event()
        fork.record(main)
        outs = [None] * len(models)
        joins = []
        for i, st in enumerate(side):
            st.wait_event(fork)
            with torch.cuda.stream(st):
                outs[i + 1] = models[i + 1](inputs[i + 1])
                ev = torch.cuda.Event()
                ev.record(st)
                joins.append(ev)
        outs[0] = models[0](inputs[0])
        for ev in joins:
            main.wait_event(ev)
    return graph, outs


class MultiBranchStep:
    """One CUDA graph that steps several groups of streams concurrently: every group has its own model
    instance (own caches) and its own CUDA stream inside the capture. Streams of a video never interact,
    so the groups share nothing but the weights' values. Each model must already have processed its first
    frame and one steady-state frame."""

    def __init__(self, models, example_inputs):
        self.models = models
        self.static_in = [x.clone() for x in example_inputs]
        self.graph, self.static_out = capture_groups(models, self.static_in)

    def load(self, frames, non_blocking=True):
        for dst, src in zip(self.static_in, frames):
            dst.copy_(src, non_blocking=non_blocking)

    def __call__(self, frames=None):
        if frames is not None:
            self.load(frames)
        self.graph.replay()
        return self.static_out


class DepthPipeline:
    """A frame pipeline over the depth of a network, inside one CUDA graph: the network of every stream group is cut
    into consecutive stages, and one step runs stage 0 on frame t, stage 1 on what stage 0 produced from frame t-1,
    stage 2 on what stage 1 produced one step earlier, and so on, all as concurrent branches of the graph. Every step
    still runs every layer once for every stream; the result a step returns belongs to the frame of
    ``latency_steps`` = stages - 1 steps earlier. A step of a delta network is a chain of short dependent kernels;
    the pipeline puts several such chains side by side without making the batch of any kernel smaller.

    Between two stages lie (delta, mask) pairs (one, or a list of them where the network has parallel branches). They
    are kept in two sets of buffers used in turn (two graphs, for even and odd steps): stage s writes the buffers of
    this step's parity while stage s+1 reads the others. The buffers start with all-zero masks, which every delta
    layer treats as "nothing changed", so the pipeline fills itself during the first steps and ``drain`` (steps that
    repeat the last frame, whose delta is zero) empties it.

    ``stages_per_group[g]`` are the stage callables of group g (first takes the frame batch, the others what the
    stage before returned); the models must have processed their first frame and one steady-state frame.
    Construction runs every stage once eagerly on ``example_inputs`` to learn the shapes between the stages: pass the
    frame the models saw last, so that this pass changes nothing. With ``models`` (the module of every group) the layer that ends a
    stage writes straight into the buffer of the step's parity: the module attributes that hold its output tensors
    are pointed at that buffer while the graph of a parity is captured. Without it, or where no such attribute is
    found, the stage's output is copied into the buffer."""

    def __init__(self, stages_per_group, example_inputs, models=None):
        self.stages = stages_per_group
        self.latency_steps = len(stages_per_group[0]) - 1
        self.shape = []                     # [group][stage boundary] -> what the stage returned (nested lists / tuples of tensors)
        self.between = []                   # [group][stage boundary][parity] -> the tensors of that structure, flattened
        self.owners = []                    # [group][stage boundary][tensor] -> [(module, attribute)] holding that tensor
        with torch.no_grad():
            for g, (fns, x) in enumerate(zip(stages_per_group, example_inputs)):
                shapes, row, own = [], [], []
                for fn in fns[:-1]:
                    x = fn(x)
                    leaves = _leaves(x)
                    shapes.append(x)
                    row.append([[torch.zeros_like(v) for v in leaves] for _ in range(2)])
                    found = [[] for _ in leaves]
                    if models is not None:
                        for mod in models[g].modules():
                            for attr, v in vars(mod).items():
                                for i, leaf in enumerate(leaves):
                                    if v is leaf:
                                        found[i].append((mod, attr))
                    own.append(found)
                fns[-1](x)
                self.shape.append(shapes)
                self.between.append(row)
                self.owners.append(own)
        torch.cuda.synchronize()

    def capture(self, inputs, parity, pool=None):
        """Graph of one step for the steps of ``parity``, reading the frames from ``inputs`` (one tensor per group).
        Returns (graph, outputs of the last stages)."""
        fns, ins, last = [], [], []

        def writer(fn, dst):
            def run(x):
                for v, d in zip(_leaves(fn(x)), dst):
                    if v.data_ptr() != d.data_ptr():      # a tensor no layer of this stage could be pointed at the buffer for
                        d.copy_(v)
                return None
            return run

        for g, stage_fns in enumerate(self.stages):
            n = len(stage_fns)
            for s, fn in enumerate(stage_fns):
                ins.append(inputs[g] if s == 0 else _like(self.shape[g][s - 1], iter(self.between[g][s - 1][1 - parity])))
                fns.append(fn if s == n - 1 else writer(fn, self.between[g][s][parity]))
                last.append(s == n - 1)
                if s < n - 1:
                    for found, buf in zip(self.owners[g][s], self.between[g][s][parity]):
                        for mod, attr in found:
                            setattr(mod, attr, buf)
        graph, outs = capture_groups(fns, ins, pool=pool)
        return graph, [o for o, is_last in zip(outs, last) if is_last]


def _leaves(x):
    """The tensors of a nested list / tuple structure, in order."""
    if torch.is_tensor(x):
        return [x]
    out = []
    for v in x:
        out += _leaves(v)
    return out


def _like(x, tensors):
    """The structure of ``x`` filled with the tensors the iterator ``tensors`` yields."""
    if torch.is_tensor(x):
        return next(tensors)
    return type(x)(_like(v, tensors) for v in x)


class DepthPipelinedStep:
    """Device-side stepping through a ``DepthPipeline``: two input buffers and two graphs used in turn."""

    def __init__(self, stages_per_group, example_inputs, models=None):
        self.pipe = DepthPipeline(stages_per_group, example_inputs, models)
        self.latency_steps = self.pipe.latency_steps
        self.inputs = [[x.clone() for x in example_inputs] for _ in range(2)]
        self.graphs, self.outputs = [], []
        pool = None
        for parity in range(2):
            g, outs = self.pipe.capture(self.inputs[parity], parity, pool)
            pool = g.pool()
            self.graphs.append(g)
            self.outputs.append(outs)
        self.t = 0

    @property
    def static_in(self):
        """Input buffers of the next step."""
        return self.inputs[self.t % 2]

    def __call__(self, frames=None):
        i = self.t % 2
        if frames is not None:
            for dst, src in zip(self.inputs[i], frames):
                dst.copy_(src, non_blocking=True)
        self.graphs[i].replay()
        self.t += 1
        return self.outputs[i]

    def drain(self, last_frames):
        """Steps that repeat the last frame (zero delta) until its result has left the pipeline and every buffer
        between two stages holds an all-zero mask again; returns the outputs, which now belong to that frame."""
        out = self.outputs[(self.t - 1) % 2]
        for _ in range(self.latency_steps + 1):
            out = self(last_frames)
        return out


class PipelinedStep:
    """End-to-end stepping from host memory: two sets of input buffers and two captured graphs of the
    same model group(s), so that the host->device copy of frame t+1 (on a copy stream) overlaps the delta
    step of frame t, and the result of frame t is copied back to pinned host memory behind it. The models
    must be warmed up (first frame and one steady-state frame done) before construction. ``bounds`` are
    the batch offsets of the groups inside a full frame batch."""

    def __init__(self, models, example_inputs, bounds, compute_stream, capture=None):
        self.compute = compute_stream
        self.copy = torch.cuda.Stream()
        self.bounds = bounds
        self.inputs = [[x.clone() for x in example_inputs] for _ in range(2)]
        self.graphs, self.outputs = [], []
        pool = None
        for i, bufs in enumerate(self.inputs):
            # ``capture(bufs, i, pool)``: another way to build the graph of the steps that read input buffer i
            # (``DepthPipeline.capture``: the buffer index is also the step's parity)
            g, outs = capture(bufs, i, pool) if capture is not None else capture_groups(models, bufs, pool=pool)
            pool = g.pool()
            self.graphs.append(g)
            self.outputs.append(outs)
        self.host_out = [[torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs] for outs in self.outputs]
        # results leave on a stream of their own: a small device copy on the compute stream frees the model's output
        # buffer for the next step, the copy to the host then runs beside that step
        self.down = torch.cuda.Stream()
        self.result = [[torch.empty_like(o) for o in outs] for outs in self.outputs]
        self.copied = [torch.cuda.Event(), torch.cuda.Event()]
        self.consumed = [torch.cuda.Event(), torch.cuda.Event()]
        self.stepped_ev = [torch.cuda.Event(), torch.cuda.Event()]
        self.downloaded = [torch.cuda.Event(), torch.cuda.Event()]
        for e in self.consumed + self.downloaded:
            e.record(self.compute)
        self.uploaded = 0      # frames uploaded so far
        self.stepped = 0       # frames processed so far

    def upload(self, host_frame):
        """Start the upload of the next frame batch (at most one ahead of step())."""
        assert self.uploaded - self.stepped < 2
        i = self.uploaded % 2
        self.copy.wait_event(self.consumed[i])            # the graph that last read these buffers is done
        with torch.cuda.stream(self.copy):
            for g, buf in enumerate(self.inputs[i]):
                buf.copy_(host_frame[self.bounds[g]:self.bounds[g + 1]], non_blocking=True)
            self.copied[i].record(self.copy)
        self.uploaded += 1

    def step(self):
        """Run the delta step on the oldest uploaded frame batch; returns the pinned host tensors the results are being
        copied to (valid once ``join()`` has been called and the compute stream synchronised, or after a device-wide
        synchronisation; overwritten two steps later)."""
        assert self.stepped < self.uploaded
        i = self.stepped % 2
        self.compute.wait_event(self.copied[i])
        self.compute.wait_event(self.downloaded[i])       # the results of two steps ago have left self.result[i]
        with torch.cuda.stream(self.compute):
            self.graphs[i].replay()
            self.consumed[i].record(self.compute)
            for dst, src in zip(self.result[i], self.outputs[i]):
                dst.copy_(src, non_blocking=True)
            self.stepped_ev[i].record(self.compute)
        self.down.wait_event(self.stepped_ev[i])
        with torch.cuda.stream(self.down):
            for dst, src in zip(self.host_out[i], self.result[i]):
                dst.copy_(src, non_blocking=True)
            self.downloaded[i].record(self.down)
        self.stepped += 1
        return self.host_out[i]

    def join(self):
        """Make the compute stream wait for the result copies in flight (so that an event recorded on it afterwards,
        or its synchronisation, covers them)."""
        for e in self.downloaded:
            self.compute.wait_event(e)
