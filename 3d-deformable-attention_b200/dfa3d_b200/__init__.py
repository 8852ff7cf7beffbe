"""dfa3d_b200 -- B200 (sm_100a) implementation of the DFA3D operator behind the reference's API.

The compute lives in ``libdfa3d_b200.so`` (hand-written CUDA behind a C ABI, include/dfa3d_b200.h);
this package is the PyTorch-facing host side: ``ext`` mirrors the reference's extension module,
``functions`` its autograd Functions.  There is no fallback path: without the shared library the
operators raise.
"""
from . import _lib, ext  # noqa: F401
from .host import HostPipeline  # noqa: F401
from .functions import (  # noqa: F401
    DeformableAttn3DFromOffsetsFunction,
    DeformableAttn3DFromOffsetsFunction_fp32,
    MultiScale3DDeformableAttnFunction,
    MultiScaleDeformableAttnFunction,
    MultiScaleDeformableAttnFunction_fp16,
    MultiScaleDeformableAttnFunction_fp32,
    MultiScale3DDeformableAttnFunction_fp16,
    MultiScale3DDeformableAttnFunction_fp32,
    MultiScaleDepthScoreSampleFunction,
    MultiScaleDepthScoreSampleFunction_fp16,
    MultiScaleDepthScoreSampleFunction_fp32,
    WeightedMultiScaleDeformableAttnFunction,
    WeightedMultiScaleDeformableAttnFunction_fp16,
    WeightedMultiScaleDeformableAttnFunction_fp32,
)

__all__ = [
    "ext", "HostPipeline",
    "MultiScaleDepthScoreSampleFunction", "WeightedMultiScaleDeformableAttnFunction",
    "MultiScale3DDeformableAttnFunction",
    "MultiScaleDepthScoreSampleFunction_fp32", "WeightedMultiScaleDeformableAttnFunction_fp32",
    "MultiScale3DDeformableAttnFunction_fp32",
    "DeformableAttn3DFromOffsetsFunction", "DeformableAttn3DFromOffsetsFunction_fp32",
    "MultiScaleDeformableAttnFunction", "MultiScaleDeformableAttnFunction_fp32",
    "MultiScaleDepthScoreSampleFunction_fp16", "WeightedMultiScaleDeformableAttnFunction_fp16",
    "MultiScale3DDeformableAttnFunction_fp16", "MultiScaleDeformableAttnFunction_fp16",
]
