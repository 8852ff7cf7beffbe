"""Drop-in stand-in for the reference's ``dfa3D`` package, backed by dfa3d_b200.

Put this directory's parent on ``sys.path`` instead of the reference's DFA3D install and
``import dfa3D`` keeps working for its consumers:
  * ``dfa3D.ext_loader.load_ext('_ext', [...])``  (DFA3D/dfa3D/ext_loader.py:25-29) returns an object
    with the four extension functions;
  * ``dfa3D.ops.multi_scale_3D_deform_attn`` exports the three autograd Functions
    (DFA3D/dfa3D/ops/multi_scale_3D_deform_attn.py).
"""
from dfa3d_b200 import ext as _ext  # noqa: F401
