"""CPU checks of the host side: the shared library loads and exports every symbol the header
declares, the module API keeps the reference's registry semantics, and nothing computes on a CPU."""
import json
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    import ctypes
    from deltacnn_b200 import _lib
    header = open(os.path.join(ROOT, "include", "deltacnn_b200.h")).read()
    declared = set(re.findall(r"\b(dc_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in the header"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/deltacnn_b200.h but not exported"
    assert declared == set(_lib.EXPORTED_SYMBOLS), "ctypes signature table and header disagree"
    assert lib.dc_version() >= 100
    lib.dc_status_string.restype = ctypes.c_char_p
    assert b"NULL" in lib.dc_status_string(1)


def test_no_cpu_fallback():
    import deltacnn_b200.cuda_kernels as K
    x = torch.zeros(1, 8, 4, 4).contiguous(memory_format=torch.channels_last)
    with pytest.raises(RuntimeError, match="CUDA"):
        K.sparsify(x, x.clone(), x.clone(), torch.zeros(1, 1, 4, 4, dtype=torch.int32), 0.1)
    with pytest.raises(RuntimeError, match="CUDA"):
        K.sparse_activation(x, x.clone(), x.clone(), torch.zeros(1, 1, 4, 4, dtype=torch.int32), 0.1, 1, 0)


def test_drop_in_module_names():
    import deltacnn
    from deltacnn.sparse_layers import DCConv2d, DCThreshold  # noqa: F401
    for name in ("DCModule", "DCSparsify", "DCDensify", "DCConv2d", "DCConvTranspose2d", "DCActivation", "DCMaxPooling",
                 "DCAdaptiveAveragePooling", "DCAdd", "DCUpsamplingNearest2d", "DCThreshold", "DCBackend", "DCBatchNorm2d",
                 "DCConcatenate", "DCTruncation", "sparse_conv", "sparse_deconv", "sparse_pooling", "sparse_activation",
                 "sparsify", "sparse_add_tensors", "sparse_add_to_dense_tensor", "sparse_upsample", "sparse_concatenate",
                 "sparse_mul_add", "DCPerformanceMetricsManager", "DCPerformanceMetrics"):
        assert hasattr(deltacnn, name), name


def test_threshold_registry_load_save(tmp_path, monkeypatch):
    from deltacnn_b200 import DCThreshold
    keys = [object() for _ in range(4)]
    for i, k in enumerate(keys):
        DCThreshold.set(k, 0.1 * i)
    DCThreshold.set(keys[0], 9.0)                    # first registration wins
    assert DCThreshold.get(keys[0]) == 0.0 and DCThreshold.get(object(), 7.0) == 7.0
    monkeypatch.chdir(tmp_path)
    DCThreshold.save_thresholds("t")
    saved = json.load(open(tmp_path / "thresholds_t.json"))
    assert [saved[str(i)] for i in range(4)] == [0.0, 0.1, 0.2, 0.30000000000000004]
    # a shorter file addresses the last layers; scale multiplies
    json.dump({"0": 1.0, "1": 2.0}, open(tmp_path / "short.json", "w"))
    DCThreshold.path, DCThreshold.scale = str(tmp_path / "short.json"), 0.5
    DCThreshold.load_thresholds()
    assert [DCThreshold.get(k) for k in keys] == [0.0, 0.1, 0.5, 1.0]
    DCThreshold.scale = 1.0


def test_constructor_signatures_and_backend_switch():
    from deltacnn_b200 import DCConv2d, DCConvTranspose2d, DCActivation, DCBackend, DCTruncation, DCSparsify
    c = DCConv2d(8, 16, 3, stride=2, padding=1, activation="relu6", delta_threshold=0.2)
    assert c.activation_layer is not None and c.activation_layer.delta_threshold == 0.2 and c.activation_int == 2
    d = DCConvTranspose2d(8, 8, 4, stride=2, padding=1, dense_out=True)
    assert d.densify_layer is not None
    assert DCActivation(activation="leaky").activation_int == 3
    assert DCTruncation.parse_string("rms") == DCTruncation.rms and DCBackend.parse_string("cudnn") == DCBackend.cudnn
    # cudnn backend: layers are plain torch layers on dense tensors, also on a CPU
    dense = DCConv2d(3, 4, 3, padding=1, backend=DCBackend.cudnn, activation="relu")
    y = dense(torch.randn(1, 3, 5, 5))
    assert y.shape == (1, 4, 5, 5) and (y >= 0).all()
    DCConv2d.backend = DCBackend.cudnn
    x = torch.randn(1, 3, 4, 4)
    assert DCSparsify()(x) is x
    with pytest.raises(NotImplementedError):
        DCConv2d.backend = DCBackend.delta_cudnn
        DCSparsify()(x)


def test_filter_layout():
    from deltacnn_b200.filter_conversion import convert_filter_out_channels_last
    w = torch.arange(2 * 3 * 4 * 5, dtype=torch.float32).view(2, 3, 4, 5)       # [co, ci, kh, kw]
    f = convert_filter_out_channels_last(w)
    assert f.shape == (4, 5, 3, 2) and f[1, 2, 0, 1] == w[1, 0, 1, 2]
    wt = torch.arange(2 * 3 * 4 * 4, dtype=torch.float32).view(2, 3, 4, 4)      # [ci, co, kh, kw]
    ft = convert_filter_out_channels_last(wt, transposed=True)
    assert ft.shape == (4, 4, 2, 3) and ft[3, 1, 1, 2] == wt[1, 2, 3, 1]


def test_threshold_tuning_front_to_back():
    """The front-to-back search of the reference's readme (3.5): each layer's threshold doubles until the loss
    leaves its budget, and the last accepted value is kept; earlier layers' choices are inputs to later ones."""
    from deltacnn_b200 import DCThreshold
    from deltacnn_b200.tuning import tune_thresholds
    DCThreshold.reset()
    keys = ["a", "b", "c"]
    for k in keys:
        DCThreshold.set(k, 0.0)
    sens = {"a": 10.0, "b": 1.0, "c": 0.0}                 # loss = 1 + sum sens * t^2 : "c" does not matter at all
    calls = []

    def loss():
        calls.append(dict(DCThreshold.t))
        return 1.0 + sum(sens[k] * DCThreshold.t[k] ** 2 for k in keys)

    table = tune_thresholds(loss, start=0.01, step=2.0, max_loss_increase=1.05, max_threshold=1.0)
    a, b, c = table
    assert a == 0.04 and 1.0 + 10 * 0.08 ** 2 > 1.05 >= 1.0 + 10 * a ** 2        # 0.08 would exceed the budget of layer a
    base_b = 1.0 + 10 * a ** 2
    assert base_b + b ** 2 <= base_b * 1.05 < base_b + (2 * b) ** 2
    assert c == 0.64                                        # insensitive layer: runs to the largest value <= max_threshold
    assert list(DCThreshold.t.values()) == table
    DCThreshold.reset()


def test_threshold_tuning_with_zero_start_loss_uses_the_absolute_slack():
    from deltacnn_b200 import DCThreshold
    from deltacnn_b200.tuning import tune_thresholds
    DCThreshold.reset()
    DCThreshold.set("x", 0.0)
    table = tune_thresholds(lambda: DCThreshold.t["x"], start=0.001, step=2.0, max_loss_increase=1.001, abs_slack=0.01)
    assert table == [0.008]
    DCThreshold.reset()


def test_performance_metrics_follow_the_reference_counter_definitions():
    """DCPerformanceMetricsManager computes the reference's DCMetrics counters (src/cuda/common.cuh:41-65) from masks.
    Checked on a hand-countable case and against the oracle's mask dilation on a random one."""
    from deltacnn_b200.cuda_kernels import DCPerformanceMetricsManager as M
    from oracle import delta_ops as O
    M.reset()
    M.enabled = True
    try:
        m = torch.zeros(1, 1, 16, 16, dtype=torch.int32)
        m[0, 0, 3, 4] = 1
        M.add_conv(m, 8, 16, (3, 3), (1, 1), (1, 1), (1, 1), 1, (16, 16))
        r = M.get_metrics()
        assert (r.tiles_active, r.tiles_total) == (1, 4)
        assert (r.inputs_active, r.inputs_total) == (1, 4 * 10 * 10)
        assert r.flops_theoretical == 9 * 8 * 16                       # nine output pixels see the one active tap
        assert r.flops_actual == 64 * 9 * 8 * 16                       # every pixel of the active 8x8 tile, all taps
        assert r.flops_dense == 256 * 9 * 8 * 16
        assert r.mem_write_actual == 9 * 16 and r.mem_write_dense == 256 * 16
        assert r.mem_read_actual == 1 * 8 + 9 * 8 * 16
        assert r.histogram[0] == 3 and r.histogram[1] == 1 and sum(r.histogram) == 4
        assert r.mode_sparse == 1 and r.mode_dense == 0
        # a random stride-2 case: updated pixels must be the oracle's out-mask
        M.reset()
        g = torch.Generator().manual_seed(0)
        m = (torch.rand(2, 1, 30, 34, generator=g) < 0.1).to(torch.int32)
        ho, wo = O.conv_out_size(30, 34, (3, 3), (2, 2), (1, 1), (1, 1))
        M.add_conv(m, 4, 6, (3, 3), (2, 2), (1, 1), (1, 1), 1, (ho, wo))
        om = O.dilate_mask(m, (3, 3), (2, 2), (1, 1), (1, 1))
        r = M.get_metrics()
        assert r.mem_write_actual == int(om.sum()) * 6
        assert r.tiles_total == 2 * 2 * 3 and r.inputs_total == r.tiles_total * 17 * 17
        # truncation layer: 2C read and written per masked pixel; two frames averaged
        M.reset()
        M.add_activation(m, 10, 0)
        M.add_activation(m, 10, 0)
        r = M.get_metrics(n_frames=2)
        assert r.mem_read_actual == 2 * 10 * int(m.sum()) and r.mem_write_actual == r.mem_read_actual
        d = r.to_dict()
        assert len(d["histogram"]) == 128 and "flops_ratio_actual" in d
    finally:
        M.enabled = False
        M.reset()


@pytest.mark.parametrize("name,size,cuts", [("mobilenet", 64, [5, 9, 13]), ("resnet50", 64, [3, 7, 11, 14]),
                                            ("hrnet", 64, [1, 3, 5, 7, 9]), ("centernet", 64, [3, 7, 9])])
def test_depth_stages_in_order_are_the_forward_pass(name, size, cuts):
    """The stage callables a network hands to the frame pipeline, called one after the other on one frame, are its
    forward pass (checked on the dense build of every example network, on the CPU)."""
    import torch
    from examples.nets import BUILDERS, DenseOps, init_weights
    net = BUILDERS[name](DenseOps)
    init_weights(net, 0)
    net.eval()
    x = torch.randn(1, 3, size, size)
    with torch.no_grad():
        want = net(x)
        y = x
        for stage in net.depth_stages(cuts):
            y = stage(y)
    want = list(want) if isinstance(want, (tuple, list)) else [want]
    got = list(y) if isinstance(y, (tuple, list)) else [y]
    assert len(want) == len(got) and all(torch.equal(a, b) for a, b in zip(want, got))
    with pytest.raises(AssertionError):
        net.depth_stages([4, 4])


def test_pipeline_buffers_follow_the_structure_between_stages():
    """The tensors a stage hands to the next one may be nested lists / tuples (parallel branches): the pipeline flattens
    them into its buffers and rebuilds the same structure from them."""
    import torch
    from deltacnn_b200.stepping import _leaves, _like
    a, b, c, d = (torch.full((2,), float(i)) for i in range(4))
    nested = [(a, b), [(c, d)]]
    flat = _leaves(nested)
    assert [t.data_ptr() for t in flat] == [a.data_ptr(), b.data_ptr(), c.data_ptr(), d.data_ptr()]
    other = [t + 10 for t in flat]
    rebuilt = _like(nested, iter(other))
    assert isinstance(rebuilt, list) and isinstance(rebuilt[0], tuple) and isinstance(rebuilt[1], list) and isinstance(rebuilt[1][0], tuple)
    assert [float(t[0]) for t in _leaves(rebuilt)] == [10.0, 11.0, 12.0, 13.0]
    assert _leaves(a) == [a] and _like(a, iter([b])) is b
