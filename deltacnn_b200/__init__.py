"""deltacnn_b200: the delta-update inference path of DeltaCNN on hand-written sm_100a kernels.

Exports the public names of the reference package (src/deltacnn/__init__.py:6-9). Importing
fails if the CUDA extension (libdeltacnn_b200.so) is not built: there is no fallback path.
"""
from .cuda_kernels import sparse_conv, sparse_deconv, sparse_pooling
from .cuda_kernels import sparse_activation, sparsify, sparse_add_tensors, sparse_add_to_dense_tensor, sparse_upsample, \
    sparse_concatenate, sparse_mul_add, sparse_densify, sparsify_u8, compact_mask, sparsify_dilated, linear_delta, \
    heatmap_argmax, centernet_decode, fused_inverted_residual, conv3x3_heads, conv3x3_heads_supported
from .sparse_layers import DCConv2d, DCConvTranspose2d, DCMaxPooling, DCAdaptiveAveragePooling, DCDensify, DCAdd, \
    DCActivation, DCUpsamplingNearest2d, DCSparsify, DCThreshold, DCBackend, DCModule, DCBatchNorm2d, DCConcatenate, \
    DCTruncation, DCLinear, DCHeatmapArgmax, DCCenterNetDecode, DCFusedInvertedResidual, DCFusedHeads
from .cuda_kernels import DCPerformanceMetricsManager, DCPerformanceMetrics
from .stepping import GraphedStep, MultiBranchStep, DepthPipeline, DepthPipelinedStep, PipelinedStep, set_depth_thresholds
