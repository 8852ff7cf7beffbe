"""Seeded synthetic inputs with the shapes and value distributions of the BEVFormer-DFA3D operator.

They stand in for the nuScenes-derived tensors the reference feeds its op (camera features, depth
distributions and projected BEV reference points): shapes come from the reference's configs
(BEVFormer_DFA3D/projects/configs/bevformer/bevformer_base_DFA3D.py: 256-d, 8 heads, 4 levels,
8 points, 200x200 BEV; 900x1600 images at strides 8/16/32/64 -> 116x200 ... 15x25, the same level
sizes as unittest_DFA3D.py:46-50).  Everything is drawn from a CPU ``torch.Generator`` so that the CPU
checker and the GPU see identical bits.
"""
from dataclasses import dataclass, field
from typing import List, Tuple

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    B: int                                   # batch * cameras
    levels: Tuple[Tuple[int, int], ...]      # (h, w) per level
    D: int                                   # depth bins
    Q: int                                   # queries per camera
    P: int                                   # sampling points per level
    H: int = 8                               # heads
    C: int = 32                              # channels per head
    seed: int = 0
    oob: bool = False                        # ~15 % of points with x or y outside [0,1]
    value_dtype: str = "fp32"                # "fp32" | "bf16" | "fp16" (value and dist storage)
    local: bool = False                      # locations clustered around per-query reference points

    @property
    def L(self):
        return len(self.levels)

    @property
    def N(self):
        return sum(h * w for h, w in self.levels)

    @property
    def points(self):
        """Sampled points = B*Q*H*L*P (the unit of the throughput metric)."""
        return self.B * self.Q * self.H * self.L * self.P

    def with_(self, **kw):
        d = dict(self.__dict__)
        d.update(kw)
        return Workload(**d)

    def algorithmic_bytes(self):
        """Compulsory HBM traffic (forward, backward): every input read once, every output written
        once, dist counted un-repeated (B,N,D), depth_score not materialised, no memset traffic."""
        e = 2 if self.value_dtype in ("bf16", "fp16") else 4
        pts = self.points
        value = self.B * self.N * self.H * self.C
        dist = self.B * self.N * self.D
        out = self.B * self.Q * self.H * self.C * 4
        fwd = value * e + dist * e + pts * 16 + out
        bwd = out + value * e + dist * e + pts * 16 + value * 4 + dist * 4 + pts * 16
        return fwd, bwd


_BASE_LEVELS = ((116, 200), (58, 100), (29, 50), (15, 25))

WORKLOADS = {
    # the benchmark configurations: cfg0 small parity case, cfg1 BEVFormer-small-like single level,
    # cfg2 BEVFormer-base shape (the headline), cfg3 the same with bf16 storage, cfg4op the operator
    # shapes of the encoder-stack configuration (D = 118 bins)
    "cfg0": Workload("cfg0", B=1, levels=((32, 32), (16, 16)), D=16, Q=512, P=4, seed=0),
    "cfg1": Workload("cfg1", B=6, levels=((23, 40),), D=64, Q=6000, P=8, seed=1),
    "cfg2": Workload("cfg2", B=6, levels=_BASE_LEVELS, D=64, Q=10000, P=8, seed=2, oob=True),
    "cfg3": Workload("cfg3", B=6, levels=_BASE_LEVELS, D=64, Q=10000, P=8, seed=3, oob=True,
                     value_dtype="bf16"),
    # cfg2 with BEVFormer-like locality instead of uniform locations (reported beside the headline):
    # neighbouring queries look at neighbouring pixels, a query's points stay within a few pixels of
    # its reference point (spatial_cross_attention.py:513-538 at initialisation)
    "cfg2local": Workload("cfg2local", B=6, levels=_BASE_LEVELS, D=64, Q=10000, P=8, seed=2, local=True),
    "cfg4op": Workload("cfg4op", B=6, levels=_BASE_LEVELS, D=118, Q=10000, P=8, seed=4, oob=True),
    # small cases for parity tests
    "tiny": Workload("tiny", B=2, levels=((5, 7), (3, 4)), D=5, Q=6, P=3, H=2, C=8, seed=11, oob=True),
    "odd": Workload("odd", B=3, levels=((9, 6), (4, 5), (2, 2)), D=7, Q=33, P=5, H=3, C=16, seed=12,
                    oob=True),
}


def level_tensors(w: Workload, device="cpu"):
    """(spatial_shapes_3D (L,3) int64 = (h,w,D), level_start_index (L) int64)."""
    shapes = torch.tensor([[h, ww, w.D] for h, ww in w.levels], dtype=torch.int64)
    hw = shapes[:, 0] * shapes[:, 1]
    lsi = torch.cat([hw.new_zeros(1), hw.cumsum(0)[:-1]])
    return shapes.to(device), lsi.to(device)


def make_inputs(w: Workload, seed=None, head_repeat=False):
    """CPU fp32 tensors: value (B,N,H,C), dist (B,N,D) [or (B,N,H,D) repeated over heads, the form the
    reference op needs], loc (B,Q,H,L,P,3), attn (B,Q,H,L,P), grad_out (B,Q,H*C), shapes, lsi.

    value ~ N(0,1); dist = softmax over D of N(0,1); x,y ~ U(0,1) (or U(-0.0423,1.0423): each axis in
    range with probability 0.922, so ~15 % of points leave the image); z ~ U(0,1);
    attn = softmax over L*P of N(0,1); grad_out ~ N(0,1).  With value_dtype == "bf16" / "fp16", value and dist
    are rounded to that type once (and returned as fp32 holding the rounded values)."""
    g = torch.Generator().manual_seed(w.seed if seed is None else seed)
    value = torch.randn(w.B, w.N, w.H, w.C, generator=g)
    dist = torch.randn(w.B, w.N, w.D, generator=g).softmax(-1)
    loc = torch.rand(w.B, w.Q, w.H, w.L, w.P, 3, generator=g)
    if w.oob:
        loc[..., :2] = loc[..., :2] * 1.0846 - 0.0423
    if w.local:
        # reference point of query q on a sqrt(Q) x sqrt(Q) grid over the image (row-major, so that
        # consecutive queries are neighbours), depth from a smooth ramp; offsets of up to ~4 pixels /
        # ~2 depth bins per (head, level, point), in units of each level's own size
        side = int(round(w.Q ** 0.5))
        q = torch.arange(w.Q)
        ref = torch.stack([((q % side).float() + 0.5) / side, ((q // side).float() + 0.5) / max(1, w.Q // side),
                           0.15 + 0.7 * (q.float() / w.Q)], -1).clamp(0, 1)          # (Q, 3)
        size = torch.tensor([[ww, h, w.D] for h, ww in w.levels], dtype=torch.float32)  # (L, 3) = (W, H, D)
        off = (loc - 0.5) * torch.tensor([8.0, 8.0, 4.0]) / size[None, None, None, :, None, :]
        loc = ref[None, :, None, None, None, :] + off
    attn = torch.randn(w.B, w.Q, w.H, w.L * w.P, generator=g).softmax(-1).view(w.B, w.Q, w.H, w.L, w.P)
    grad_out = torch.randn(w.B, w.Q, w.H * w.C, generator=g)
    if w.value_dtype == "bf16":
        value = value.bfloat16().float()
        dist = dist.bfloat16().float()
    elif w.value_dtype == "fp16":
        value = value.half().float()
        dist = dist.half().float()
    if head_repeat:
        dist = dist.view(w.B, w.N, 1, w.D).repeat(1, 1, w.H, 1)
    shapes, lsi = level_tensors(w)
    return dict(value=value, dist=dist, loc=loc, attn=attn, grad_out=grad_out,
                shapes=shapes, lsi=lsi)
