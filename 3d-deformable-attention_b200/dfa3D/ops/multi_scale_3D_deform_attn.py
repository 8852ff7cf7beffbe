"""Same module path and class names as DFA3D/dfa3D/ops/multi_scale_3D_deform_attn.py."""
from dfa3d_b200.functions import (  # noqa: F401
    MultiScale3DDeformableAttnFunction,
    MultiScaleDepthScoreSampleFunction,
    WeightedMultiScaleDeformableAttnFunction,
)
from .. import ext_loader

ext_module = ext_loader.load_ext(
    '_ext', ['wms_deform_attn_backward', 'wms_deform_attn_forward', 'ms_depth_score_sample_forward',
             'ms_depth_score_sample_backward'])
