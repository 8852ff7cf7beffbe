"""ctypes binding of libdfa3d_b200.so (the C ABI declared in include/dfa3d_b200.h).

There is no CPU or pure-PyTorch fallback: if the shared library is missing or a call fails, an
exception is raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("DFA3D_B200_LIB") or os.path.join(_HERE, "libdfa3d_b200.so")

ABI_VERSION = 2
DTYPE_F32 = 0
DTYPE_BF16 = 1
DTYPE_F64 = 2
DTYPE_F16 = 3
MAX_LEVELS = 32
MAX_CHANNELS = 1024

ERROR_NAMES = {-1: "invalid argument", -2: "unsupported", -3: "CUDA error"}


class Problem(ctypes.Structure):
    """struct dfa3d_problem."""
    _fields_ = [(n, ctypes.c_int32) for n in
                ("B", "N", "H", "C", "D", "L", "Q", "P", "value_dtype", "dist_dtype")] + \
               [("dist_head_stride", ctypes.c_int64), ("dist_map_h", ctypes.c_int32),
                ("dist_map_w", ctypes.c_int32)]

    def __init__(self, *args, **kw):
        # the two dist-map fields default to 0 (dist laid out like value)
        super().__init__(*args, **kw)


_P = ctypes.POINTER(Problem)
_V = ctypes.c_void_p

# name -> number of pointer arguments after the problem descriptor (the stream included)
ENTRY_POINTS = {
    "dfa3d_depth_score_forward": 6,
    "dfa3d_depth_score_backward": 8,
    "dfa3d_wms_attn_forward": 8,
    "dfa3d_wms_attn_backward": 12,
    "dfa3d_fused_forward": 9,
    "dfa3d_fused_backward": 12,
    "dfa3d_msda_forward": 7,
    "dfa3d_msda_backward": 10,
    # double-precision instantiations (same argument lists)
    "dfa3d_depth_score_forward_f64": 6,
    "dfa3d_depth_score_backward_f64": 8,
    "dfa3d_wms_attn_forward_f64": 8,
    "dfa3d_wms_attn_backward_f64": 12,
    "dfa3d_fused_forward_f64": 9,
    "dfa3d_fused_backward_f64": 12,
    # ragged variants: the query-offset table is one more pointer, right after the descriptor
    "dfa3d_fused_forward_ragged": 10,
    "dfa3d_fused_backward_ragged": 13,
}
# entry points that take `int32_t num_anchors` right after the descriptor
ENTRY_POINTS_WITH_ANCHORS = {
    "dfa3d_attn3d_forward": 10,
    "dfa3d_attn3d_backward": 15,
    "dfa3d_attn3d_forward_ragged": 11,
    "dfa3d_attn3d_backward_ragged": 16,
}
_I32, _I64 = ctypes.c_int32, ctypes.c_int64
# entry points without a problem descriptor: explicit argument types
PLAIN_ENTRY_POINTS = {
    "dfa3d_rebatch_plan": [ctypes.c_void_p, _I32, _I32, _I32, _I32] + [ctypes.c_void_p] * 8,
    "dfa3d_rebatch_gather": [ctypes.c_void_p] * 4 + [_I32] * 4 + [_I64, _I64] + [ctypes.c_void_p] * 2
                            + [_I64, ctypes.c_void_p],
    "dfa3d_rebatch_combine": [ctypes.c_void_p] * 3 + [_I32] * 4 + [ctypes.c_void_p] * 3,
    "dfa3d_dist_from_logits": [ctypes.c_void_p] + [_I32] * 4 + [ctypes.c_void_p, _I32, ctypes.c_void_p]
                              + [_I32] * 4 + [ctypes.c_void_p] * 2,
    "dfa3d_dist_from_logits_backward": [ctypes.c_void_p] + [_I32] * 4 + [ctypes.c_void_p, _I32, ctypes.c_void_p]
                                       + [_I32] * 3 + [ctypes.c_void_p] * 3,
    "dfa3d_add_layer_norm_forward": [ctypes.c_void_p] * 4 + [_I64, _I32, ctypes.c_float] + [ctypes.c_void_p] * 5,
    "dfa3d_layer_norm_backward": [ctypes.c_void_p] * 5 + [_I64, _I32] + [ctypes.c_void_p] * 4,
    "dfa3d_column_sum": [ctypes.c_void_p, _I64, _I32, ctypes.c_void_p, ctypes.c_void_p],
}
ACT_SOFTMAX, ACT_SIGMOID = 0, 1

_lib = None
calls = 0      # successful entry-point calls so far (each launches at least one kernel)


def load():
    """Load the library once; raise with build instructions if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python 3d-deformable-attention_b200/build.py` "
            "(needs nvcc; targets sm_100a). dfa3d_b200 has no fallback implementation.")
    lib = ctypes.CDLL(LIB_PATH)
    lib.dfa3d_abi_version.restype = ctypes.c_int
    lib.dfa3d_abi_version.argtypes = []
    lib.dfa3d_last_error.restype = ctypes.c_char_p
    lib.dfa3d_last_error.argtypes = []
    for name, nptr in ENTRY_POINTS.items():
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [_P] + [_V] * nptr
    for name, nptr in ENTRY_POINTS_WITH_ANCHORS.items():
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [_P, ctypes.c_int32] + [_V] * nptr
    for name, argtypes in PLAIN_ENTRY_POINTS.items():
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = argtypes
    got = lib.dfa3d_abi_version()
    if got != ABI_VERSION:
        raise ImportError(f"libdfa3d_b200.so has ABI version {got}, this package expects {ABI_VERSION}")
    _lib = lib
    return lib


def call_plain(name, *args):
    """Invoke an entry point that takes no problem descriptor."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.dfa3d_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{name} failed ({ERROR_NAMES.get(rc, rc)}): {msg}")
    global calls
    calls += 1


def call(name, problem, *ptrs):
    """Invoke an entry point; raise RuntimeError carrying dfa3d_last_error() on failure."""
    lib = load()
    rc = getattr(lib, name)(ctypes.byref(problem), *ptrs)
    if rc != 0:
        msg = lib.dfa3d_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{name} failed ({ERROR_NAMES.get(rc, rc)}): {msg}")
    global calls
    calls += 1
