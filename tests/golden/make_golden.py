"""Generate the golden fixtures of tests/golden/ (committed next to this script).

Two sources, both independent of the CUDA kernels under test:

  --source grid_sample   (CPU, runs anywhere)  fp64 outputs of the independent grid_sample formulation
                         (oracle/grid_sample_form.py) on the small workloads; inputs are stored too.
  --source ref_cuda      (needs a GPU and oracle/_ref built by oracle/build_ref.py)  fp32 outputs of
                         the reference's unmodified CUDA op, driven through its own one-stage autograd
                         Function (forward + backward), on the small workloads and on cfg0.  For cfg0
                         the inputs are not stored (they are re-made from the seed); a checksum guards
                         against a change of the generator.

Usage:  python tests/golden/make_golden.py --source grid_sample
        python tests/golden/make_golden.py --source ref_cuda --out <dir>   (then copy the .npz files here)
"""
import argparse
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [os.path.join(ROOT, "3d-deformable-attention_b200"), os.path.join(ROOT, "oracle")]

from dfa3d_b200 import workloads as wl  # noqa: E402

SMALL = ("tiny", "odd")


def input_digest(d):
    h = hashlib.sha256()
    for k in ("value", "dist", "loc", "attn", "grad_out"):
        h.update(d[k].contiguous().numpy().tobytes())
    return h.hexdigest()


def from_grid_sample(out_dir):
    import grid_sample_form as G
    for name in SMALL:
        d = wl.make_inputs(wl.WORKLOADS[name], head_repeat=True)
        dd = {k: (v.double() if v.is_floating_point() else v) for k, v in d.items()}
        out, gv, gd, gl, ga = G.dfa3d_grid_sample_grads(dd["value"], dd["dist"], dd["shapes"], dd["lsi"],
                                                        dd["loc"], dd["attn"], dd["grad_out"])
        np.savez_compressed(
            os.path.join(out_dir, f"{name}_grid_sample_f64.npz"),
            **{"in_" + k: v.numpy() for k, v in d.items()},
            out=out.numpy(), grad_value=gv.numpy(), grad_dist=gd.numpy(), grad_loc=gl.numpy(),
            grad_attn=ga.numpy())
        print("wrote", name)


def from_ref_cuda(out_dir):
    import build_ref
    ref = build_ref.load()
    dev = "cuda"
    for name in SMALL + ("cfg0",):
        d = wl.make_inputs(wl.WORKLOADS[name], head_repeat=True)
        t = {k: v.to(dev) for k, v in d.items()}
        leaves = [t[k].clone().requires_grad_(True) for k in ("value", "dist", "loc", "attn")]
        out, ds = ref.MultiScale3DDeformableAttnFunction_fp32.apply(
            leaves[0], leaves[1], t["shapes"], t["lsi"], leaves[2], leaves[3], 64)
        out.backward(t["grad_out"])
        # two-stage API as well: gradient w.r.t. a given depth_score
        ds_leaf = ds.detach().clone().requires_grad_(True)
        v2 = t["value"].clone().requires_grad_(True)
        out2 = ref.WeightedMultiScaleDeformableAttnFunction.apply(
            v2, t["shapes"][:, :2].contiguous(), t["lsi"], t["loc"][..., :2].contiguous(), t["attn"],
            ds_leaf, 64)
        out2.backward(t["grad_out"])
        payload = dict(
            out=out, ds=ds, grad_value=leaves[0].grad, grad_dist=leaves[1].grad, grad_loc=leaves[2].grad,
            grad_attn=leaves[3].grad, grad_ds=ds_leaf.grad)
        payload = {k: v.detach().cpu().numpy() for k, v in payload.items()}
        if name in SMALL:
            payload.update({"in_" + k: v.numpy() for k, v in d.items()})
        payload["input_sha256"] = np.array(input_digest(d))
        payload["torch_version"] = np.array(torch.__version__)
        np.savez_compressed(os.path.join(out_dir, f"{name}_ref_cuda_f32.npz"), **payload)
        print("wrote", name)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", choices=("grid_sample", "ref_cuda"), required=True)
    ap.add_argument("--out", default=HERE)
    a = ap.parse_args()
    os.makedirs(a.out, exist_ok=True)
    (from_grid_sample if a.source == "grid_sample" else from_ref_cuda)(a.out)
