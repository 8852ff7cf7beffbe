"""Build libdfa3d_b200.so (CUDA kernels + C ABI) and libdfa3d_rates.so (memory-primitive rate probes,
measurement code) in-tree with nvcc for sm_100a.

No torch headers are involved: the library is plain CUDA C++ behind an ``extern "C"`` interface
(include/dfa3d_b200.h).  The result is written next to the Python package
(``dfa3d_b200/libdfa3d_b200.so``) so that it is found without any install step.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "dfa3d_b200", "libdfa3d_b200.so")
SOURCES = ["dfa3d_forward.cu", "dfa3d_backward.cu", "dfa3d_rebatch.cu", "dfa3d_dist_producer.cu",
           "dfa3d_fp64.cu", "dfa3d_layer_ops.cu", "dfa3d_capi.cu"]
RATES_SRC = os.path.join(CSRC, "rates", "dfa3d_rates.cu")
RATES_OUT = os.path.join(HERE, "dfa3d_b200", "libdfa3d_rates.so")
INCLUDE = os.path.join(HERE, "..", "include")
NVCC_FLAGS = ["-O3", "-I", INCLUDE, "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def needs_build():
    if not os.path.exists(OUT) or not os.path.exists(RATES_OUT):
        return True
    t = min(os.path.getmtime(OUT), os.path.getmtime(RATES_OUT))
    deps = [os.path.join(d, f) for d, _, fs in os.walk(CSRC) for f in fs]
    deps.append(os.path.join(HERE, "..", "include", "dfa3d_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every .cu of csrc/ in parallel and link the shared library.  Returns its path."""
    if not force and not needs_build():
        return OUT
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                                 text=True)))
    rates = subprocess.Popen([_nvcc(), *NVCC_FLAGS, "-shared", "-cudart", "shared", RATES_SRC, "-o", RATES_OUT],
                             stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    objs = []
    for src, obj, pr in procs:
        log, _ = pr.communicate()
        with open(os.path.join(objdir, src + ".log"), "w") as f:
            f.write(log)
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{log[-4000:]}")
        if verbose:
            print(log)
        objs.append(obj)
    cmd = [_nvcc(), "-shared", "-o", OUT, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
           "-cudart", "shared"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    log, _ = rates.communicate()
    with open(os.path.join(objdir, "dfa3d_rates.cu.log"), "w") as f:
        f.write(log)
    if rates.returncode != 0:
        raise RuntimeError(f"nvcc failed on dfa3d_rates.cu:\n{log[-4000:]}")
    return OUT


if __name__ == "__main__":
    print(build(force="-f" in sys.argv, verbose="-v" in sys.argv))
