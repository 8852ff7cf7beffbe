"""Build the UNMODIFIED reference DFA3D CUDA op into ``oracle/_ref/`` (test infrastructure).

The reference ships only a CUDA implementation of its operator
(DFA3D/dfa3D/ops/csrc/cuda/cudabind.cpp:41-44,67-70 register CUDA impls only), so the strongest
checker for this repository is the reference op itself, compiled for sm_100a from the sources where
they lie in the reference checkout, and run on the GPU next to the new kernels.

What this script does, and nothing else:
  * compiles DFA3D/dfa3D/ops/csrc/{*.cpp, cuda/*.cu, cuda/*.cpp} with
    ``torch.utils.cpp_extension.load`` (name ``_ext``, arch sm_100a) -- the same file globs and
    include dirs as the reference's DFA3D/setup.py:176-181, minus its ``-std=c++14`` which
    torch 2.x headers reject;
  * "installs" the reference's own Python package next to the binary (``oracle/_ref/dfa3D``) and the
    BEVFormer-side copy of the autograd Functions (``oracle/_ref/bevformer_fn.py``), exactly as a
    ``pip install --target`` of the reference would, so that the reference can be driven through
    its own public API.  ``oracle/_ref/`` is git-ignored: no reference source enters the history.

Only tests, ``__graft_entry__`` and the reference arm of ``bench.py`` may import what this produces.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_OUT = os.path.join(HERE, "_ref")


def reference_root():
    """Where the reference checkout lies: $DFA3D_REFERENCE_ROOT, else a directory named ``reference``
    beside this repository."""
    env = os.environ.get("DFA3D_REFERENCE_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def is_built():
    pkg = os.path.join(REF_OUT, "dfa3D")
    return os.path.isdir(pkg) and any(
        f.startswith("_ext") and f.endswith(".so") for f in os.listdir(pkg))


def build(verbose=False):
    """Compile + install; returns the install dir.  No-op when already built."""
    if is_built():
        return REF_OUT
    root = reference_root()
    csrc = os.path.join(root, "DFA3D", "dfa3D", "ops", "csrc")
    if not os.path.isdir(csrc):
        raise FileNotFoundError(f"reference checkout not found at {root}: set DFA3D_REFERENCE_ROOT to the "
                                "directory that holds DFA3D/ and BEVFormer_DFA3D/")
    import glob
    from torch.utils import cpp_extension

    sources = (sorted(glob.glob(os.path.join(csrc, "*.cpp")))
               + sorted(glob.glob(os.path.join(csrc, "cuda", "*.cu")))
               + sorted(glob.glob(os.path.join(csrc, "cuda", "*.cpp"))))
    build_dir = os.path.join(REF_OUT, "_build")
    os.makedirs(build_dir, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    cpp_extension.load(
        name="_ext",
        sources=sources,
        extra_include_paths=[os.path.join(csrc, "common"), os.path.join(csrc, "common", "cuda")],
        extra_cflags=["-DWITH_CUDA", "-O2"],
        extra_cuda_cflags=["-DWITH_CUDA", "-O3", "-lineinfo",
                           "-gencode", "arch=compute_100a,code=sm_100a"],
        build_directory=build_dir,
        is_python_module=False,   # compile only; it is imported as dfa3D._ext below
        verbose=verbose,
    )
    # install: python package + binary
    pkg_src = os.path.join(root, "DFA3D", "dfa3D")
    pkg_dst = os.path.join(REF_OUT, "dfa3D")
    if os.path.isdir(pkg_dst):
        shutil.rmtree(pkg_dst)
    shutil.copytree(pkg_src, pkg_dst, ignore=shutil.ignore_patterns("csrc", "__pycache__"))
    for d, _, files in os.walk(pkg_dst):   # the checkout is read-only; make the install removable
        os.chmod(d, 0o755)
        for f in files:
            os.chmod(os.path.join(d, f), 0o644)
    shutil.copy(os.path.join(build_dir, "_ext.so"), os.path.join(pkg_dst, "_ext.so"))
    bev_fn = os.path.join(root, "BEVFormer_DFA3D", "projects", "mmdet3d_plugin", "bevformer",
                          "modules", "multi_scale_3ddeformable_attn_function.py")
    dst = os.path.join(REF_OUT, "bevformer_fn.py")
    if os.path.exists(dst):
        os.chmod(dst, 0o644)
    shutil.copyfile(bev_fn, dst)
    return REF_OUT


def load():
    """Import the installed reference.  Returns a namespace with the reference's own objects.

    Raises ImportError when ``oracle/_ref`` has not been built (it cannot be built on a machine
    without the reference checkout)."""
    if not is_built():
        raise ImportError("oracle/_ref is not built; run `python oracle/build_ref.py` where the "
                          "reference checkout is available")
    import importlib
    import types
    if REF_OUT not in sys.path:
        sys.path.insert(0, REF_OUT)
    mine = sys.modules.get("dfa3D")
    if mine is not None and not getattr(mine, "__file__", "").startswith(REF_OUT):
        raise ImportError("another `dfa3D` package is already imported in this process; the "
                          "reference build must be loaded in a process of its own")
    ops = importlib.import_module("dfa3D.ops.multi_scale_3D_deform_attn")
    ext = importlib.import_module("dfa3D._ext")
    bev = importlib.import_module("bevformer_fn")
    ns = types.SimpleNamespace(
        ext=ext,
        MultiScaleDepthScoreSampleFunction=ops.MultiScaleDepthScoreSampleFunction,
        WeightedMultiScaleDeformableAttnFunction=ops.WeightedMultiScaleDeformableAttnFunction,
        MultiScale3DDeformableAttnFunction_fp32=bev.MultiScale3DDeformableAttnFunction_fp32,
    )
    return ns


if __name__ == "__main__":
    out = build(verbose="-v" in sys.argv)
    print("reference op installed in", out)
