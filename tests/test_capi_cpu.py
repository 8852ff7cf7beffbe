"""The C-ABI library loads without a GPU, exports every symbol the public header declares, and its
host-side validation answers with error codes (no compute call is made here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "dfa3d_b200.h")


def declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(dfa3d_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for n in ("dfa3d_depth_score_forward", "dfa3d_depth_score_backward", "dfa3d_wms_attn_forward",
              "dfa3d_wms_attn_backward", "dfa3d_fused_forward", "dfa3d_fused_backward",
              "dfa3d_attn3d_forward", "dfa3d_attn3d_backward", "dfa3d_msda_forward",
              "dfa3d_msda_backward", "dfa3d_fused_forward_ragged", "dfa3d_fused_backward_ragged",
              "dfa3d_attn3d_forward_ragged", "dfa3d_attn3d_backward_ragged", "dfa3d_rebatch_plan",
              "dfa3d_rebatch_gather", "dfa3d_rebatch_combine",
              "dfa3d_last_error", "dfa3d_abi_version"):
        assert n in names


def test_library_exports_every_declared_symbol(lib_built):
    lib = ctypes.CDLL(lib_built)
    for n in declared_symbols():
        assert hasattr(lib, n), f"{n} declared in include/dfa3d_b200.h but not exported"


def test_binding_table_matches_header(lib_built):
    from dfa3d_b200 import _lib
    declared = set(declared_symbols()) - {"dfa3d_last_error", "dfa3d_abi_version"}
    bound = set(_lib.ENTRY_POINTS) | set(_lib.ENTRY_POINTS_WITH_ANCHORS) | set(_lib.PLAIN_ENTRY_POINTS)
    assert declared <= bound, declared - bound
    assert _lib.load().dfa3d_abi_version() == _lib.ABI_VERSION


def test_problem_struct_layout():
    from dfa3d_b200 import _lib
    assert ctypes.sizeof(_lib.Problem) == 10 * 4 + 8 + 2 * 4
    assert _lib.Problem.dist_head_stride.offset == 40
    assert _lib.Problem.dist_map_h.offset == 48 and _lib.Problem.dist_map_w.offset == 52


def test_validation_returns_codes_not_crashes(lib_built):
    from dfa3d_b200 import _lib
    lib = _lib.load()
    ok = _lib.Problem(1, 4, 1, 4, 2, 1, 1, 1, 0, 0, 2)
    # null descriptor
    assert lib.dfa3d_fused_forward(None, *([None] * 9)) == -1
    assert b"null" in lib.dfa3d_last_error()
    # null tensor pointer
    assert lib.dfa3d_fused_forward(ctypes.byref(ok), *([None] * 9)) == -1
    assert b"value" in lib.dfa3d_last_error()
    # too many levels -> unsupported
    bad = _lib.Problem(1, 4, 1, 4, 2, 33, 1, 1, 0, 0, 2)
    assert lib.dfa3d_fused_forward(ctypes.byref(bad), *([None] * 9)) == -2
    # bad enum
    bad = _lib.Problem(1, 4, 1, 4, 2, 1, 1, 1, 7, 0, 2)
    assert lib.dfa3d_fused_forward(ctypes.byref(bad), *([None] * 9)) == -1
    # bad head stride
    bad = _lib.Problem(1, 4, 1, 4, 2, 1, 1, 1, 0, 0, 3)
    assert lib.dfa3d_fused_backward(ctypes.byref(bad), *([None] * 12)) == -1
    # misaligned value pointer
    assert lib.dfa3d_fused_forward(ctypes.byref(ok), 8, 16, 16, 16, 16, 16, 16, None, None) == -1
    assert b"aligned" in lib.dfa3d_last_error()
    # empty problem: nothing to do, OK without touching the pointers
    empty = _lib.Problem(0, 4, 1, 4, 2, 1, 0, 1, 0, 0, 2)
    for name, n in _lib.ENTRY_POINTS.items():
        if name.endswith("_ragged"):     # the offset table is required even for an empty problem
            assert getattr(lib, name)(ctypes.byref(empty), *([None] * n)) == -1, name
            assert getattr(lib, name)(ctypes.byref(empty), 16, *([None] * (n - 1))) == 0, name
        elif name.endswith("_f64"):      # the double entry points want DFA3D_DTYPE_F64 in the descriptor
            assert getattr(lib, name)(ctypes.byref(empty), *([None] * n)) == -1, name
            assert b"F64" in lib.dfa3d_last_error()
            empty64 = _lib.Problem(0, 4, 1, 4, 2, 1, 0, 1, _lib.DTYPE_F64, _lib.DTYPE_F64, 2)
            assert getattr(lib, name)(ctypes.byref(empty64), *([None] * n)) == 0, name
        else:
            assert getattr(lib, name)(ctypes.byref(empty), *([None] * n)) == 0, name
    for name, n in _lib.ENTRY_POINTS_WITH_ANCHORS.items():
        if name.endswith("_ragged"):
            assert getattr(lib, name)(ctypes.byref(empty), 1, *([None] * n)) == -1, name
            assert getattr(lib, name)(ctypes.byref(empty), 1, 16, *([None] * (n - 1))) == 0, name
        else:
            assert getattr(lib, name)(ctypes.byref(empty), 1, *([None] * n)) == 0, name
    # re-batching entry points: sizes are checked before any pointer is used
    assert lib.dfa3d_rebatch_plan(None, 0, 1, 4, 1, *([None] * 8)) == -1
    assert lib.dfa3d_rebatch_plan(None, 2, 1, 4, 1, *([None] * 8)) == -1
    assert b"counts" in lib.dfa3d_last_error()
    assert lib.dfa3d_rebatch_gather(None, None, None, None, 2, 1, 4, 8, 0, 4, None, None, 0, None) == 0
    assert lib.dfa3d_rebatch_gather(None, None, None, None, 2, 1, 4, 0, 0, 4, None, None, 8, None) == -1
    assert lib.dfa3d_rebatch_combine(None, None, None, 2, 1, 0, 8, None, None, None) == 0
    assert lib.dfa3d_rebatch_combine(None, None, None, 2, 1, 4, 8, None, None, None) == -1
    # depth-distribution producer: logits, B, D, map_h, map_w, shapes, shape_stride, level_start, L, N,
    # activation, dist_dtype, dist, stream
    prod = lib.dfa3d_dist_from_logits
    assert prod(None, 0, 64, 4, 4, None, 2, None, 1, 16, 0, 0, None, None) == 0          # B = 0: nothing to do
    assert prod(None, 1, 64, 4, 4, None, 2, None, 1, 16, 0, 0, None, None) == -1 and b"logits" in lib.dfa3d_last_error()
    assert prod(None, 1, 257, 4, 4, None, 2, None, 1, 16, 0, 0, None, None) == -2 and b"256" in lib.dfa3d_last_error()
    assert prod(None, 1, 64, 4, 4, None, 2, None, 1, 16, 5, 0, None, None) == -1 and b"activation" in lib.dfa3d_last_error()
    assert prod(None, 1, 64, 4, 4, None, 4, None, 1, 16, 0, 0, None, None) == -1 and b"shape_stride" in lib.dfa3d_last_error()
    assert prod(None, 1, 64, 4, 4, None, 2, None, 1, 16, 0, 2, None, None) == -1 and b"dist_dtype" in lib.dfa3d_last_error()
    assert prod(None, 1, 64, 4, 4, None, 2, None, 1, 16, 0, _lib.DTYPE_F16, None, None) == -1 and b"logits" in lib.dfa3d_last_error()
    # half storage: value and dist together
    bad = _lib.Problem(1, 4, 1, 4, 2, 1, 1, 1, _lib.DTYPE_F16, 0, 2)
    assert lib.dfa3d_fused_forward(ctypes.byref(bad), *([None] * 9)) == -2 and b"fp16" in lib.dfa3d_last_error()
    half = _lib.Problem(1, 4, 1, 4, 2, 1, 1, 1, _lib.DTYPE_F16, _lib.DTYPE_F16, 2)
    assert lib.dfa3d_fused_forward(ctypes.byref(half), *([None] * 9)) == -1 and b"null" in lib.dfa3d_last_error()
    assert lib.dfa3d_dist_from_logits_backward(None, 1, 64, 0, 4, None, 2, None, 1, 16, 0, None, None, None) == -1
    # encoder-layer row operations: sizes first, then pointers
    ln_f, ln_b, cs = lib.dfa3d_add_layer_norm_forward, lib.dfa3d_layer_norm_backward, lib.dfa3d_column_sum
    assert ln_f(None, None, None, None, 0, 256, 1e-5, None, None, None, None, None) == 0
    assert ln_f(None, None, None, None, 4, 102, 1e-5, None, None, None, None, None) == -2 and b"multiple of 4" in lib.dfa3d_last_error()
    assert ln_f(None, None, None, None, 4, 2048, 1e-5, None, None, None, None, None) == -2
    assert ln_f(None, None, None, None, -1, 256, 1e-5, None, None, None, None, None) == -1
    assert ln_f(16, 16, 16, 16, 4, 256, 1e-5, None, 16, 16, 16, None) == -1 and b"together" in lib.dfa3d_last_error()
    assert ln_f(None, None, None, None, 4, 256, 1e-5, None, None, None, None, None) == -1 and b"null" in lib.dfa3d_last_error()
    assert ln_f(8, None, 16, 16, 4, 256, 1e-5, None, 16, 16, 16, None) == -1 and b"aligned" in lib.dfa3d_last_error()
    assert ln_b(None, None, None, None, None, 0, 256, None, None, None, None) == 0
    assert ln_b(None, None, None, None, None, 4, 256, None, None, None, None) == -1
    assert ln_b(None, None, None, None, None, 4, 130, None, None, None, None) == -2
    assert cs(None, 0, 8, None, None) == 0 and cs(None, 4, 0, None, None) == 0
    assert cs(None, 4, 6, None, None) == -2 and b"multiple of 4" in lib.dfa3d_last_error()
    assert cs(None, 4, 8, None, None) == -1 and cs(None, -1, 8, None, None) == -1
    # a dist map needs both of its sizes
    bad = _lib.Problem(1, 4, 1, 4, 2, 1, 1, 1, 0, 0, 2, 3, 0)
    assert lib.dfa3d_fused_forward(ctypes.byref(bad), *([None] * 9)) == -1 and b"dist_map" in lib.dfa3d_last_error()
    # the anchors must divide the points per level
    assert lib.dfa3d_attn3d_forward(ctypes.byref(ok), 3, *([None] * 10)) == -1
    assert b"num_anchors" in lib.dfa3d_last_error()
    with pytest.raises(RuntimeError, match="invalid argument"):
        _lib.call("dfa3d_fused_forward", ok, *([None] * 9))


def test_shim_rejects_cpu_tensors_like_the_reference(lib_built):
    import torch
    from dfa3d_b200 import ext, MultiScale3DDeformableAttnFunction
    from dfa3d_b200 import workloads as wl
    d = wl.make_inputs(wl.WORKLOADS["tiny"])
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ext.dfa3d_fused_forward(d["value"], d["dist"], d["shapes"], d["lsi"], d["loc"], d["attn"], 64)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        MultiScale3DDeformableAttnFunction.apply(d["value"], d["dist"], d["shapes"], d["lsi"], d["loc"],
                                                 d["attn"], 64)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ext.wms_deform_attn_forward(d["value"], d["shapes"][:, :2].contiguous(), d["lsi"],
                                    d["loc"][..., :2].contiguous(), d["attn"],
                                    torch.zeros(*d["attn"].shape, 4), 64)


def test_missing_library_fails_loudly(tmp_path):
    """No fallback path: without the shared library the package raises, it does not compute."""
    import subprocess
    import sys
    pkg = os.path.join(ROOT, "3d-deformable-attention_b200")
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "import torch, dfa3d_b200\n"
        "from dfa3d_b200 import _lib\n"
        "try:\n    _lib.load()\nexcept ImportError as e:\n    assert 'no fallback' in str(e); print('raised')\n"
        % pkg)
    env = dict(os.environ, DFA3D_B200_LIB=str(tmp_path / "absent.so"))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env)
    assert r.returncode == 0 and "raised" in r.stdout, r.stderr


def test_header_is_plain_c_and_the_library_links_from_c(lib_built, tmp_path):
    """include/dfa3d_b200.h compiles as C99 with warnings as errors, and a C program linked against
    the shared library can call it (version query and an argument check; no GPU needed)."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    src = tmp_path / "use_abi.c"
    src.write_text(r"""
#include <stdio.h>
#include <string.h>
#include "dfa3d_b200.h"
int main(void) {
  dfa3d_problem p;
  memset(&p, 0, sizeof p);
  p.B = 1; p.N = 4; p.H = 1; p.C = 4; p.D = 2; p.L = 1; p.Q = 1; p.P = 1; p.dist_head_stride = 2;
  if (dfa3d_abi_version() != DFA3D_ABI_VERSION) return 1;
  if (dfa3d_fused_forward(&p, 0, 0, 0, 0, 0, 0, 0, 0, 0) != DFA3D_ERR_INVALID_ARGUMENT) return 2;
  if (!strstr(dfa3d_last_error(), "value")) return 3;
  if (sizeof(dfa3d_problem) != 56) return 4;
  printf("abi %d ok\n", dfa3d_abi_version());
  return 0;
}
""")
    exe = tmp_path / "use_abi"
    libdir = os.path.dirname(lib_built)
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
                        str(src), "-o", str(exe), "-L", libdir, "-ldfa3d_b200", f"-Wl,-rpath,{libdir}"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and "ok" in r.stdout, (r.returncode, r.stdout, r.stderr)
