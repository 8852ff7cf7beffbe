from .multi_scale_3D_deform_attn import (MultiScaleDepthScoreSampleFunction,
                                         WeightedMultiScaleDeformableAttnFunction)

__all__ = ['MultiScaleDepthScoreSampleFunction', 'WeightedMultiScaleDeformableAttnFunction']
