"""Drop-in alias: ``import deltacnn`` resolves to deltacnn_b200, including the submodule
paths user code imports from (``deltacnn.sparse_layers``, ``deltacnn.cuda_kernels``,
``deltacnn.filter_conversion``)."""
import sys

import deltacnn_b200
from deltacnn_b200 import *  # noqa: F401,F403
from deltacnn_b200 import cuda_kernels, filter_conversion, sparse_layers

sys.modules[__name__ + ".sparse_layers"] = sparse_layers
sys.modules[__name__ + ".cuda_kernels"] = cuda_kernels
sys.modules[__name__ + ".filter_conversion"] = filter_conversion
