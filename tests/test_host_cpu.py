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
