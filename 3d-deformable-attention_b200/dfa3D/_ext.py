"""The extension module of the drop-in package: the four entry points of the reference's compiled
``dfa3D._ext`` (DFA3D/dfa3D/ops/csrc/pybind.cpp:42-66), implemented by dfa3d_b200.ext, plus the two
entry points of the plain 2-D operator under the names the mmcv extension gives them."""
from dfa3d_b200.ext import (  # noqa: F401
    ms_deform_attn_backward,
    ms_deform_attn_forward,
    ms_depth_score_sample_backward,
    ms_depth_score_sample_forward,
    wms_deform_attn_backward,
    wms_deform_attn_forward,
)
