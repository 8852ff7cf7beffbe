"""Rates of the memory primitives the DFA3D kernels are made of, measured on the GPU at hand.

``libdfa3d_rates.so`` (csrc/rates/dfa3d_rates.cu) replays the address stream of one operator launch --
the four 128-byte corner rows per sampling point in ``value`` / ``grad_value`` and the (z0, z0+1) pairs
of the four corner pixels in ``dist`` / ``grad_dist`` -- with pseudo-random uniform positions and none of
the arithmetic.  Timing each primitive alone and the ones a kernel needs together gives a lower bound
for that kernel that does not depend on how its arithmetic is written:

  forward  >= time(GATHER_ROWS + dist gathers)
  backward >= time(GATHER_ROWS + dist gathers + RED_ROWS + dist reductions)

    python -m dfa3d_b200.rates [--workload cfg2] [--cameras 6] [--reps 20] [--json]

Measurement code: the operator itself never loads this library.
"""
import argparse
import ctypes
import json
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdfa3d_rates.so")

GATHER_ROWS, RED_ROWS, GATHER_PAIRS, RED_PAIRS, GATHER_CELLS, RED_CELLS, BULK_RED_ROWS = \
    1, 2, 4, 8, 16, 32, 64


class RateProblem(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("B", "Q", "L", "P", "D")] + \
               [("level_h", ctypes.c_int32 * 8), ("level_w", ctypes.c_int32 * 8),
                ("ops", ctypes.c_int32), ("level_mask", ctypes.c_int32), ("dead_fraction", ctypes.c_float)]


_lib = None


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} not found: build it with "
                              "`python 3d-deformable-attention_b200/build.py`")
        lib = ctypes.CDLL(LIB_PATH)
        lib.dfa3d_rate_probe.restype = ctypes.c_int
        lib.dfa3d_rate_probe.argtypes = [ctypes.POINTER(RateProblem)] + [ctypes.c_void_p] * 8
        lib.dfa3d_rate_sizes.restype = ctypes.c_int
        lib.dfa3d_rate_sizes.argtypes = [ctypes.POINTER(RateProblem), ctypes.POINTER(ctypes.c_int64),
                                         ctypes.POINTER(ctypes.c_int64)]
        _lib = lib
    return _lib


class Prober:
    """Buffers of one problem shape (H = 8 heads, C = 32 fp32 channels, L*P = 32) and timed probes."""

    def __init__(self, levels, P, D, Q, B, device="cuda", dead_fraction=0.15, cells=True):
        assert len(levels) * P == 32, "the probe kernel covers L*P == 32"
        self.lib = load()
        self.dev = torch.device(device)
        self.pr = RateProblem(B=B, Q=Q, L=len(levels), P=P, D=D, ops=0, level_mask=(1 << len(levels)) - 1,
                              dead_fraction=dead_fraction)
        for i, (h, w) in enumerate(levels):
            self.pr.level_h[i], self.pr.level_w[i] = h, w
        n, nc = ctypes.c_int64(), ctypes.c_int64()
        assert self.lib.dfa3d_rate_sizes(ctypes.byref(self.pr), ctypes.byref(n), ctypes.byref(nc)) == 0
        self.N, self.NC = n.value, nc.value
        z = lambda *s: torch.zeros(*s, device=self.dev)
        self.value, self.grad_value = z(B, self.N, 8, 32), z(B, self.N, 8, 32)
        self.dist, self.grad_dist = z(B, self.N, D), z(B, self.N, D)
        self.cells = z(B, self.NC, D, 4) if cells else None
        self.grad_cells = z(B, self.NC, D, 4) if cells else None
        self.sink = z((Q * 8 + 7) // 8 * 8 * B)
        self.points = B * Q * 8 * 32

    def launch(self, ops, level_mask=None):
        self.pr.ops = ops
        self.pr.level_mask = (1 << self.pr.L) - 1 if level_mask is None else level_mask
        p = lambda t: None if t is None else t.data_ptr()
        rc = self.lib.dfa3d_rate_probe(ctypes.byref(self.pr), p(self.value), p(self.grad_value), p(self.dist),
                                       p(self.grad_dist), p(self.cells), p(self.grad_cells), p(self.sink),
                                       torch.cuda.current_stream(self.dev).cuda_stream)
        if rc != 0:
            raise RuntimeError(f"dfa3d_rate_probe failed with code {rc}")

    def time_ms(self, ops, level_mask=None, reps=20, warmup=3):
        """Median CUDA-event time of one probe launch."""
        for _ in range(warmup):
            self.launch(ops, level_mask)
        ts = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            self.launch(ops, level_mask)
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]


PROBES = (
    ("gather value rows (4 x 128 B per point)", GATHER_ROWS),
    ("reduce grad_value rows, red.global.add.v4.f32", RED_ROWS),
    ("reduce grad_value rows, cp.reduce.async.bulk from shared memory", BULK_RED_ROWS),
    ("gather dist pairs (4 x 8 B per point)", GATHER_PAIRS),
    ("reduce grad_dist pairs (4 x red.v2 per point)", RED_PAIRS),
    ("gather dist, corner-interleaved copy (1 x 32 B per point)", GATHER_CELLS),
    ("reduce grad_dist, corner-interleaved copy (2 x red.v4 per point)", RED_CELLS),
    ("forward stream: value rows + dist pairs", GATHER_ROWS | GATHER_PAIRS),
    ("forward stream, dist corner-interleaved", GATHER_ROWS | GATHER_CELLS),
    ("backward stream: gathers + row and pair reductions", GATHER_ROWS | GATHER_PAIRS | RED_ROWS | RED_PAIRS),
    ("backward stream, dist corner-interleaved", GATHER_ROWS | GATHER_CELLS | RED_ROWS | RED_CELLS),
)


def measure(levels, P, D, Q, B, reps=20, per_level=True):
    pb = Prober(levels, P, D, Q, B)
    rows = []
    for name, ops in PROBES:
        ms = pb.time_ms(ops, reps=reps)
        rows.append({"probe": name, "ops": ops, "levels": "all", "ms": ms,
                     "gpoints_per_s": pb.points / ms / 1e6})
    if per_level:
        # the same number of issued points, all on one level: few rows taking many updates against many
        for l in range(len(levels)):
            for name, ops in (("reduce grad_value rows, red.global.add.v4.f32", RED_ROWS),
                              ("gather value rows (4 x 128 B per point)", GATHER_ROWS)):
                ms = pb.time_ms(ops, level_mask=1 << l, reps=reps)
                rows.append({"probe": name, "ops": ops, "levels": f"level {l} only ({levels[l][0]}x{levels[l][1]})",
                             "ms": ms, "gpoints_per_s": pb.points / len(levels) / ms / 1e6})
    return rows


def floors(levels, P, D, Q, B, reps=10):
    """Lower bounds (ms) of the forward and the backward of this shape from their memory streams."""
    pb = Prober(levels, P, D, Q, B, cells=False)
    return {"forward_ms": pb.time_ms(GATHER_ROWS | GATHER_PAIRS, reps=reps),
            "backward_ms": pb.time_ms(GATHER_ROWS | GATHER_PAIRS | RED_ROWS | RED_PAIRS, reps=reps),
            "backward_reductions_only_ms": pb.time_ms(RED_ROWS | RED_PAIRS, reps=reps)}


def main():
    from . import workloads as wl
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--cameras", type=int, default=0)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args()
    w = wl.WORKLOADS[a.workload]
    B = a.cameras or w.B
    rows = measure(w.levels, w.P, w.D, w.Q, B, reps=a.reps)
    if a.json:
        print(json.dumps({"workload": w.name, "cameras": B, "gpu": torch.cuda.get_device_name(0), "rows": rows}))
        return
    print(f"# {w.name}: {B} cameras, Q={w.Q}, levels={w.levels}, D={w.D}; {torch.cuda.get_device_name(0)}")
    print("| probe | levels | ms | G points/s |")
    print("|---|---|---|---|")
    for r in rows:
        print(f"| {r['probe']} | {r['levels']} | {r['ms']:.3f} | {r['gpoints_per_s']:.2f} |")


if __name__ == "__main__":
    main()
