#!/usr/bin/env python
"""Benchmark of the DFA3D operator hot path: fused forward + fused backward, sampled points / s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one forward + backward of the operator over one batch of seeded synthetic inputs
(default workload ``cfg2``: 6 cameras, BEVFormer-base level shapes, 10 000 queries, 8 heads x 32
channels, 4 levels x 8 points, 64 depth bins, fp32, ~15 % of the points outside the image).  With
N > 1 every rank owns its own batch of camera frames (weak scaling, no data-path collective: frames
are independent); the job value is the points of all ranks over the slowest rank's time.

Printed by rank 0: ONE JSON line with
  value      device-resident throughput (inputs in HBM, CUDA-event timed, max over ranks)
  e2e        the same step through the host-buffer API (dfa3d_b200.HostPipeline: pinned HOST tensors
             in, pinned host tensors out; it calls the extension-level entry points, not the autograd
             Functions), host<->device copies inside the timed region; `copy_floor_ms` beside it is the
             same pipeline with the kernels left out
  roofline   the dominant kernel (backward) against the measured HBM copy bandwidth
  cpu_baseline  the CPU oracle (C + OpenMP port of the reference kernels) on a bounded sample
``--impl reference`` times the reference's own CUDA op (unmodified sources built for sm_100a into
oracle/_ref) through its own one-stage autograd Function on the same workload; when that build is
absent it times the CPU oracle port instead and says so.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.join(ROOT, "3d-deformable-attention_b200")]

import torch  # noqa: E402
import torch.distributed as dist_  # noqa: E402

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum of an ncu capture of the same
# kernels on 2 of the 6 cameras, times 3: cameras are independent and traffic grows in proportion).
# Keyed by workload; a workload without a capture reports null.
NCU_DRAM_TRAFFIC = {
    "cfg2": {"forward": 3 * (191.835392e6 + 17.074688e6), "backward": 3 * (262.928384e6 + 124.026624e6)},
    "cfg3": {"forward": 3 * (121.627904e6 + 14.459392e6), "backward": 3 * (220.926208e6 + 116.512768e6)},
}


def log(*a):
    print(*a, file=sys.stderr, flush=True)


# ----------------------------------------------------------------------------------------------
# clocks: sampled through NVML (read-only) while the timed region runs
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # NVML missing: report nulls, do not fail the bench
            log("clock sampling unavailable:", e)
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.001)

    def start(self):
        if self.nv:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()

    def stop(self):
        if self._thr:
            self._stop.set()
            self._thr.join()
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# ----------------------------------------------------------------------------------------------
def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s)"


def cpu_baseline(w, budget_cameras=1):
    """CPU oracle (C + OpenMP port of the reference kernels), fp32, fwd+bwd, on `budget_cameras`
    cameras of the workload.  Returns the cpu_baseline object."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np
    import dfa3d_oracle as O
    from dfa3d_b200 import workloads as wl
    ws = w.with_(B=budget_cameras)
    d = wl.make_inputs(ws, head_repeat=True)
    n = {k: v.numpy() for k, v in d.items()}
    O.lib()
    t0 = time.perf_counter()
    reps = 0
    while True:
        out, ds = O.dfa3d_forward(n["value"], n["dist"], n["shapes"], n["lsi"], n["loc"], n["attn"])
        O.dfa3d_backward(n["value"], n["dist"], n["shapes"], n["lsi"], n["loc"], n["attn"],
                         n["grad_out"], depth_score=ds)
        reps += 1
        el = time.perf_counter() - t0
        if el > 10.0 or (reps >= 5 and el > 2.0):      # a bounded sample: 2-10 s on all host threads
            break
    assert np.isfinite(out).all()
    cores = int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))
    return {"value": ws.points * reps / el, "unit": "sampled points/s", "cores": cores, "kind": "port",
            "sample": f"{budget_cameras} of {w.B} cameras of {w.name} (same per-camera shapes), fp32, "
                      f"fwd+bwd, {reps} repetitions in {el:.1f} s, C+OpenMP port of the reference "
                      f"kernels on {cores} host threads"}


# ----------------------------------------------------------------------------------------------
class OursRunner:
    """Device-resident step: fused forward, zeroing of the two accumulated gradients, fused backward,
    through the extension-level API (raw C-ABI calls on preallocated tensors)."""
    launches_per_step = 2

    def __init__(self, w, t):
        from dfa3d_b200 import ext
        self.ext, self.t, self.w = ext, t, w
        self.value = t["value"].bfloat16() if w.value_dtype == "bf16" else t["value"]
        self.dist = t["dist"].bfloat16() if w.value_dtype == "bf16" else t["dist"]
        self.gv = torch.zeros_like(t["value"]); self.gd = torch.zeros_like(t["dist"])
        self.gl = torch.empty_like(t["loc"]); self.ga = torch.empty_like(t["attn"])

    def forward(self):
        t = self.t
        self.out, _ = self.ext.dfa3d_fused_forward(self.value, self.dist, t["shapes"], t["lsi"], t["loc"],
                                                   t["attn"], 64, need_depth_score=False)

    def zero(self):
        self.gv.zero_(); self.gd.zero_()

    def backward(self):
        t = self.t
        self.ext.dfa3d_fused_backward(self.value, self.dist, t["shapes"], t["lsi"], t["loc"], t["attn"],
                                      t["grad_out"], self.gv, self.gd, self.gl, self.ga, 64)

    def e2e_step(self, host, pinned_out, join=True, copies_only=False):
        """Public host-buffer API (dfa3d_b200.HostPipeline): every input is copied host->device, the
        output and all four gradients device->host, per camera, overlapped with the kernels.
        join=False lets consecutive steps overlap (the caller joins after the last one)."""
        if getattr(self, "pipe", None) is None:
            from dfa3d_b200 import HostPipeline
            self.pipe = HostPipeline(self.t["shapes"], self.t["lsi"], self.t["loc"].device)
        self.pipe.run(host, pinned_out, join=join, copies_only=copies_only)

    def e2e_join(self):
        self.pipe.join()

    def function_step(self):
        """The same step through the one-stage autograd Function, the way the reference arm is driven:
        fresh leaves, output and depth_score allocated by forward, gradients allocated (and the two
        accumulated ones zeroed) by backward."""
        import dfa3d_b200
        t = self.t
        leaves = [self.value.detach().requires_grad_(True), self.dist.detach().requires_grad_(True),
                  t["loc"].detach().requires_grad_(True), t["attn"].detach().requires_grad_(True)]
        out, _ = dfa3d_b200.MultiScale3DDeformableAttnFunction_fp32.apply(
            leaves[0], leaves[1], t["shapes"], t["lsi"], leaves[2], leaves[3], 64)
        out.backward(t["grad_out"])


class ReferenceRunner:
    """The reference's CUDA op through its own one-stage autograd Function (dist repeated per head, as
    its kernels require; the repeat itself is not timed)."""
    launches_per_step = 4

    def __init__(self, w, t, ref):
        self.ref, self.t, self.w = ref, t, w
        self.dist_h = t["dist"].view(w.B, w.N, 1, w.D).repeat(1, 1, w.H, 1)
        self.leaves = [t["value"].clone().requires_grad_(True), self.dist_h.requires_grad_(True),
                       t["loc"].clone().requires_grad_(True), t["attn"].clone().requires_grad_(True)]

    def forward(self):
        for x in self.leaves:
            x.grad = None
        lv, t = self.leaves, self.t
        self.out, _ = self.ref.MultiScale3DDeformableAttnFunction_fp32.apply(
            lv[0], lv[1], t["shapes"], t["lsi"], lv[2], lv[3], 64)

    def zero(self):
        pass   # the reference Function zeroes inside backward

    def backward(self):
        self.out.backward(self.t["grad_out"])

    def e2e_join(self):
        pass

    def e2e_step(self, host, pinned_out, join=True, copies_only=False):
        dev = self.t["loc"].device
        w = self.w
        value = host["value"].to(dev, non_blocking=True).requires_grad_(True)
        dist = host["dist"].to(dev, non_blocking=True).view(w.B, w.N, 1, w.D).repeat(1, 1, w.H, 1)
        dist.requires_grad_(True)
        loc = host["loc"].to(dev, non_blocking=True).requires_grad_(True)
        attn = host["attn"].to(dev, non_blocking=True).requires_grad_(True)
        go = host["grad_out"].to(dev, non_blocking=True)
        out, _ = self.ref.MultiScale3DDeformableAttnFunction_fp32.apply(
            value, dist, self.t["shapes"], self.t["lsi"], loc, attn, 64)
        out.backward(go)
        for k, g in (("out", out.detach()), ("grad_value", value.grad), ("grad_dist", dist.grad.sum(2)),
                     ("grad_loc", loc.grad), ("grad_attn", attn.grad)):
            pinned_out[k].copy_(g, non_blocking=True)


# ----------------------------------------------------------------------------------------------
def measure_encoder_stack(rank, world, dev, steps, warmup):
    """Training step (forward, backward, gradient all-reduce, optimizer step) of the 6-layer
    spatial-cross-attention encoder stack on one frame (6 cameras) per GPU: 200x200 BEV queries, each
    camera sees 10 000 of them, BEVFormer-base level shapes, 118 depth bins, 256-d, FFN 512.  Data
    parallel over frames with NCCL all-reduce of the projection-layer gradients (torch DDP).  The
    process group must exist already when world > 1.  Returns the result dict (same on every rank)."""
    from dfa3d_b200 import _lib, modules, workloads as wl
    w = wl.WORKLOADS["cfg4op"]
    # projection GEMMs on the TF32 tensor cores, which is what the reference's stack (PyTorch 1.9,
    # where TF32 matmuls were on by default) ran them on; the DFA3D kernels themselves stay fp32
    tf32 = (torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32)
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    torch.manual_seed(0)                                   # identical initial weights on every rank
    layers, E, cams, Z, bev = 6, w.H * w.C, 6, 4, 200 * 200
    stack = modules.SCAEncoderStack(num_layers=layers, embed_dims=E, ffn_dims=512, num_cams=cams,
                                    num_heads=w.H, num_levels=w.L, num_points=w.P, dropout=0.1).to(dev)
    model = stack
    if world > 1:
        model = torch.nn.parallel.DistributedDataParallel(stack, device_ids=[dev.index],
                                                          broadcast_buffers=False)
    opt = torch.optim.AdamW(stack.parameters(), lr=2e-4, weight_decay=0.01)
    g = torch.Generator().manual_seed(w.seed + 1000 * rank)
    shapes, lsi = wl.level_tensors(w)
    mask = torch.zeros(cams, 1, bev, Z, dtype=torch.bool)
    for c in range(cams):                                  # each camera sees w.Q of the BEV queries
        mask[c, 0, torch.randperm(bev, generator=g)[:w.Q]] = True
    ref = torch.rand(cams, 1, bev, Z, 3, generator=g)
    ref[..., :2] = ref[..., :2] * 1.0846 - 0.0423
    kw = dict(key=None,
              value=torch.randn(cams, w.N, 1, E, generator=g).to(dev),
              value_dpt_dist=torch.randn(cams, w.N, 1, w.D, generator=g).softmax(-1).to(dev),
              reference_points_cam=ref.to(dev), bev_mask=mask.to(dev),
              spatial_shapes=shapes[:, :2].contiguous().to(dev), level_start_index=lsi.to(dev))
    query = torch.randn(1, bev, E, generator=g).to(dev)

    def step():
        opt.zero_grad(set_to_none=True)
        loss = model(query, **kw).float().pow(2).mean()
        loss.backward()
        opt.step()
        return loss.detach()

    def barrier():
        if world > 1:
            dist_.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    calls0 = _lib.calls
    e0.record()
    for _ in range(steps):
        loss = step()
    e1.record()
    barrier()
    own_launches = _lib.calls - calls0      # entry-point calls of the library (operator, re-batching, norms,
    tm = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)   # bias gradients)
    if world > 1:
        dist_.all_reduce(tm, op=dist_.ReduceOp.MAX)
    ms = float(tm.item()) / steps
    assert torch.isfinite(loss)
    torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = tf32
    return {"value": w.points * layers * world / (ms * 1e-3), "unit": "sampled points/s",
            "ms_per_step": ms, "n_gpus": world, "steps": steps, "loss": float(loss),
            "dtype": "f32 (projection GEMMs tf32)",
            "config": {"workload": "cfg4", "layers": layers, "frames_per_gpu": 1, "cameras": cams,
                       "bev_queries": bev, "queries_per_camera": w.Q, "depth_bins": w.D,
                       "embed_dims": E, "ffn_dims": 512,
                       "parallelism": f"dp{world}: NCCL all-reduce of projection gradients (DDP)"},
            "gpu_launches": own_launches}


def run_encoder_stack(a, rank, world, local):
    """--workload cfg4: the encoder-stack training step as the bench's only measurement."""
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist_.init_process_group("nccl", device_id=dev)
    sampler = ClockSampler(local)
    sampler.start()
    r = measure_encoder_stack(rank, world, dev, a.steps, a.warmup)
    clocks = sampler.stop()
    if rank == 0:
        print(json.dumps({
            "metric": "DFA3D fwd+bwd sampled points/s (encoder-stack training step)",
            "value": r["value"], "unit": r["unit"], "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": r["dtype"], "data": "synthetic", "config": r["config"],
            "clocks": clocks, "gpu_launches": r["gpu_launches"], "loss": r["loss"]}), flush=True)
    if world > 1:
        dist_.destroy_process_group()


def measure_query_blocks(a, w, rank, world, dev, steps, warmup):
    """Query-block mode: ONE batch of camera frames on all ranks.  The ranks form camera groups; inside
    a group the queries are split (dfa3d_b200.sharding.camera_query_grid).  value / dist are replicated
    by one NCCL broadcast (outside the timed region: they are the layer's inputs, resident before the op
    runs); a step is fused forward + backward on the rank's query block, one sub-group of cameras at a
    time, with the exchange of that sub-group's grad_value / grad_dist (partial sums over the group's
    query blocks) issued asynchronously while the next sub-group computes.  The exchange is an
    all-reduce (every rank of the group ends with the full gradient) or a reduce-scatter (every rank
    ends with its 1/group share of it).  Returns the result dict (identical on every rank)."""
    from dfa3d_b200 import ext, sharding, workloads as wl
    gi, ranks, cams, qi, qblocks = sharding.camera_query_grid(w.B, world, rank, a.camera_groups)
    ngroups = world // qblocks
    group = None
    if world > 1 and qblocks > 1:
        for g in range(ngroups):                                 # every rank creates every group
            pg = dist_.new_group(list(range(g * qblocks, (g + 1) * qblocks)))
            if g == gi:
                group = pg
    d = wl.make_inputs(w)                                        # same seed on every rank: same batch
    qs = sharding.shard_queries(w.Q, qblocks, qi)
    value = d["value"].to(dev) if rank == 0 else torch.empty_like(d["value"], device=dev)
    dist = d["dist"].to(dev) if rank == 0 else torch.empty_like(d["dist"], device=dev)
    if world > 1:
        dist_.broadcast(value, 0)
        dist_.broadcast(dist, 0)
    value, dist = value[cams].contiguous(), dist[cams].contiguous()
    loc = d["loc"][cams, qs].contiguous().to(dev)
    attn = d["attn"][cams, qs].contiguous().to(dev)
    go = d["grad_out"][cams, qs].contiguous().to(dev)
    shapes, lsi = d["shapes"].to(dev), d["lsi"].to(dev)
    ncam = value.shape[0]
    gv = torch.zeros_like(value); gd = torch.zeros_like(dist)
    gl = torch.empty_like(loc); ga = torch.empty_like(attn)
    out = torch.empty(ncam, loc.shape[1], w.H * w.C, device=dev)
    # cameras are exchanged in this many parts (one launch pair each); with nothing to exchange, one
    sub = max(1, min(a.exchange_groups, ncam)) if qblocks > 1 else 1
    bounds = [round(i * ncam / sub) for i in range(sub + 1)]
    scatter = a.exchange == "reduce_scatter" and qblocks > 1
    shards = []
    if scatter:                                                  # this rank's share of each part's gradient
        for g0, g1 in zip(bounds[:-1], bounds[1:]):
            n = gv[g0:g1].numel() + gd[g0:g1].numel()
            shards.append((torch.empty((n + qblocks - 1) // qblocks * qblocks, device=dev),
                           torch.empty((n + qblocks - 1) // qblocks, device=dev)))

    def step():
        works = []
        for i, (g0, g1) in enumerate(zip(bounds[:-1], bounds[1:])):
            sl = slice(g0, g1)
            ext.dfa3d_fused_forward(value[sl], dist[sl], shapes, lsi, loc[sl], attn[sl], 64,
                                    need_depth_score=False, out=out[sl])
            gv[sl].zero_(); gd[sl].zero_()
            ext.dfa3d_fused_backward(value[sl], dist[sl], shapes, lsi, loc[sl], attn[sl], go[sl], gv[sl],
                                     gd[sl], gl[sl], ga[sl], 64)
            if scatter:
                flat, mine = shards[i]
                nv = gv[sl].numel()
                flat[:nv].copy_(gv[sl].reshape(-1)); flat[nv:nv + gd[sl].numel()].copy_(gd[sl].reshape(-1))
                works.append(dist_.reduce_scatter_tensor(mine, flat, group=group, async_op=True))
            elif qblocks > 1:
                works += sharding.allreduce_sum_([gv[sl], gd[sl]], group=group, async_op=True)
        for wk in works:
            wk.wait()

    def barrier():
        if world > 1:
            dist_.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    ms = sharding.max_over_ranks(e0.elapsed_time(e1), device=dev) / steps
    # parity of the exchange: the exchanged gradient must satisfy the same adjoint identity as on one
    # GPU, <grad_out, out> summed over all ranks == <grad_value, value> summed over the camera groups
    lhs = (go.double() * out.double()).sum()
    if scatter:
        rhs = torch.zeros((), dtype=torch.float64, device=dev)
        for i, (g0, g1) in enumerate(zip(bounds[:-1], bounds[1:])):
            flat, mine = shards[i]
            n = mine.numel()
            vflat = torch.cat([value[g0:g1].reshape(-1), torch.zeros_like(gd[g0:g1]).reshape(-1)])
            vflat = torch.nn.functional.pad(vflat, (0, flat.numel() - vflat.numel()))
            rhs += (mine.double() * vflat[qi * n:(qi + 1) * n].double()).sum()
    else:
        rhs = (gv.double() * value.double()).sum() / qblocks      # every rank of the group holds the full sum
    both = torch.stack([lhs, rhs])
    if world > 1:
        dist_.all_reduce(both)
    lhs, rhs = both.tolist()
    assert abs(lhs - rhs) <= 1e-4 * abs(rhs), (lhs, rhs)
    exchanged = (gv.numel() + gd.numel()) * 4 if qblocks > 1 else 0
    return {"value": w.points / (ms * 1e-3), "unit": "sampled points/s", "ms_per_step": ms,
            "n_gpus": world, "steps": steps, "scaling": "strong",
            "mode": "query blocks: %d camera group(s) x %d query block(s); value/dist broadcast once; "
                    "grad_value/grad_dist exchanged inside a camera group by NCCL %s, in %d part(s) "
                    "overlapped with the kernels" % (ngroups, qblocks, a.exchange if qblocks > 1 else "(nothing)",
                                                     sub),
            "camera_groups": ngroups, "query_blocks": qblocks, "cameras_per_rank": ncam,
            "queries_per_rank": loc.shape[1], "points_total": w.points,
            "exchange_bytes_per_rank_step": exchanged, "gpu_launches": 2 * sub * steps}


def run_query_blocks(a, w, rank, world, local):
    """--scaling strong: the query-block mode as the bench's only measurement."""
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist_.init_process_group("nccl", device_id=dev)
    sampler = ClockSampler(local)
    sampler.start()
    r = measure_query_blocks(a, w, rank, world, dev, a.steps, a.warmup)
    clocks = sampler.stop()
    if rank == 0:
        print(json.dumps({
            "metric": "DFA3D fwd+bwd sampled points/s", "value": r["value"], "unit": r["unit"],
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": w.name, "mode": r["mode"], "camera_groups": r["camera_groups"],
                       "query_blocks": r["query_blocks"], "cameras": w.B,
                       "cameras_per_rank": r["cameras_per_rank"], "queries_per_rank": r["queries_per_rank"],
                       "points_total": w.points,
                       "exchange_bytes_per_rank_step": r["exchange_bytes_per_rank_step"]},
            "clocks": clocks, "gpu_launches": r["gpu_launches"]}), flush=True)
    if world > 1:
        dist_.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--e2e-steps", type=int, default=16)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the side measurements (cfg3, Function-level step, memory-stream floor)")
    ap.add_argument("--scaling", choices=("weak", "strong"), default="weak",
                    help="weak: 6 cameras per GPU (default, the headline); strong: one batch, queries "
                         "split over the GPUs with an all-reduce of the value/dist gradients")
    ap.add_argument("--exchange-groups", type=int, default=3,
                    help="strong scaling: number of camera groups whose gradient all-reduce overlaps "
                         "the next group's kernels")
    ap.add_argument("--camera-groups", type=int, default=0,
                    help="strong scaling: number of camera groups (0 = the largest that divides both "
                         "the GPUs and the cameras); queries are split inside a group")
    ap.add_argument("--exchange", choices=("all_reduce", "reduce_scatter"), default="all_reduce",
                    help="strong scaling: how a camera group combines its partial grad_value/grad_dist")
    ap.add_argument("--cameras", type=int, default=0,
                    help="override the workload's cameras per GPU (small cases for profiler captures)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)

    from dfa3d_b200 import workloads as wl
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != a.gpus:
        log(f"note: --gpus {a.gpus} but WORLD_SIZE={world}; using WORLD_SIZE")
    if torch.cuda.is_available():
        from dfa3d_b200 import sharding
        ncpu = sharding.bind_cpu_affinity_to_gpu(local)     # before any pinned allocation
        log(f"rank {rank}: bound to {ncpu} CPU cores local to GPU {local}" if ncpu else
            f"rank {rank}: CPU affinity unchanged")
    if a.workload == "cfg4":
        return run_encoder_stack(a, rank, world, local)
    w = wl.WORKLOADS[a.workload]
    if a.cameras > 0:
        w = w.with_(B=a.cameras)

    if a.scaling == "strong" and a.impl == "ours":
        return run_query_blocks(a, w, rank, world, local)

    ref = None
    if a.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        try:
            import warnings
            warnings.simplefilter("ignore")
            import build_ref
            ref = build_ref.load()
        except Exception as e:
            log("reference CUDA op unavailable:", e)
        if ref is None or not torch.cuda.is_available():
            # CPU arm: the oracle port on the host cores, rank 0 only
            if rank == 0:
                cb = cpu_baseline(w, 1)
                line = {"metric": "DFA3D fwd+bwd sampled points/s", "value": cb["value"],
                        "unit": "sampled points/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
                        "ms_per_step": None, "higher_is_better": True, "scaling": "weak",
                        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
                        "config": {"workload": w.name}, "cpu_baseline": cb,
                        "e2e": {"value": cb["value"], "unit": cb["unit"], "h2d_bytes_per_step": 0,
                                "d2h_bytes_per_step": 0},
                        "note": "reference CUDA op build (oracle/_ref) not present: timed the CPU port"}
                print(json.dumps(line), flush=True)
            return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: dfa3d_b200 has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist_.init_process_group("nccl", device_id=dev)

    d = wl.make_inputs(w, seed=w.seed + 1000 * rank)
    t = {k: v.to(dev) for k, v in d.items()}
    runner = OursRunner(w, t) if a.impl == "ours" else ReferenceRunner(w, t, ref)
    launches_per_step = runner.launches_per_step

    def step(events=None):
        if events is not None:
            events[0].record()
        runner.forward()
        if events is not None:
            events[1].record()
        runner.zero()
        if events is not None:
            events[2].record()
        runner.backward()
        if events is not None:
            events[3].record()

    def barrier():
        if world > 1:
            dist_.barrier()
        torch.cuda.synchronize()

    for _ in range(a.warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(a.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    t_begin.record()
    for i in range(a.steps):
        step(evs[i])
    t_end.record()
    barrier()
    clocks = sampler.stop()
    total_ms = t_begin.elapsed_time(t_end)
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / a.steps
    bwd_ms = sum(e[2].elapsed_time(e[3]) for e in evs) / a.steps
    tm = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist_.all_reduce(tm, op=dist_.ReduceOp.MAX)
    total_ms = float(tm.item())
    ms_per_step = total_ms / a.steps
    value = w.points * world / (ms_per_step * 1e-3)

    # ---- end to end from pinned host buffers through the public API -------------------------
    e2e = None
    if a.e2e_steps > 0:
        e2e = measure_e2e(a, w, d, dev, world, runner, barrier)

    extra = {}
    if a.impl == "ours" and not a.no_extras:
        # the same step through the autograd Function with its allocations: how the reference arm's
        # device-timed figure is taken
        for _ in range(2):
            runner.function_step()
        n = max(5, min(a.steps, 20))
        extra["function_level_ms"] = _timed(lambda i: runner.function_step(), n, dev, world, barrier)
        extra["function_level"] = ("MultiScale3DDeformableAttnFunction_fp32.apply + backward, "
                                   "allocations and depth_score output included")
        extra.update(measure_extras(a, w, dev, world, rank, barrier))
        if world > 1 and w.name == "cfg2":
            # the other way to use several GPUs: one batch, split by cameras and queries (strong scaling).
            # Its parity check compares all-reduced scalars, so it passes or fails on every rank alike.
            try:
                extra["query_blocks"] = measure_query_blocks(a, w, rank, world, dev,
                                                             max(10, min(a.steps, 50)), 3)
            except AssertionError as e:
                extra["query_blocks"] = {"error": f"adjoint identity violated: {e}"}
        if rank == 0 and w.L * w.P == 32 and w.H == 8 and w.C == 32 and w.value_dtype == "fp32":
            extra["memory_stream_floor"] = memory_stream_floor(w)
        if w.name == "cfg2":
            # the training configuration: 6-layer spatial-cross-attention encoder stack, one frame per GPU
            extra["encoder_stack"] = measure_encoder_stack(rank, world, dev, 5, 2)

    if rank == 0:
        report(a, w, world, launches_per_step, value, ms_per_step, fwd_ms, bwd_ms, clocks, e2e, extra)
    if world > 1:
        dist_.destroy_process_group()


def _timed(fn, n, dev, world, barrier):
    """n calls of fn bracketed by barrier + synchronize, CUDA events, max over ranks -> ms per call."""
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        fn(i)
    e1.record()
    barrier()
    tm = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist_.all_reduce(tm, op=dist_.ReduceOp.MAX)
    return float(tm.item()) / n


def measure_e2e(a, w, d, dev, world, runner, barrier):
    host = {k: d[k] for k in ("value", "dist", "loc", "attn", "grad_out")}
    if w.value_dtype == "bf16" and a.impl == "ours":     # bf16 storage starts on the host
        host["value"], host["dist"] = host["value"].bfloat16(), host["dist"].bfloat16()
    host = {k: v.pin_memory() for k, v in host.items()}
    pinned_out = {"out": torch.empty(w.B, w.Q, w.H * w.C).pin_memory(),
                  "grad_value": torch.empty_like(d["value"]).pin_memory(),
                  "grad_dist": torch.empty_like(d["dist"]).pin_memory(),
                  "grad_loc": torch.empty_like(d["loc"]).pin_memory(),
                  "grad_attn": torch.empty_like(d["attn"]).pin_memory()}
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = sum(v.numel() * v.element_size() for v in pinned_out.values())
    n = a.e2e_steps
    for _ in range(2):
        runner.e2e_step(host, pinned_out)
    # every step copies all inputs in and all results out; consecutive steps may overlap (the first
    # copies of step i+1 travel while the last results of step i leave), the last step is joined
    # before the clock stops
    last = n - 1
    e2e_ms = _timed(lambda i: runner.e2e_step(host, pinned_out, join=(i == last)), n, dev, world, barrier)
    assert torch.isfinite(pinned_out["out"]).all()
    res = {"value": w.points * world / (e2e_ms * 1e-3), "unit": "sampled points/s",
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": n}
    if a.impl == "ours":
        # one step at a time (each step joined and synchronised before the next starts)
        res["ms_per_step_one_at_a_time"] = _timed(
            lambda i: (runner.e2e_step(host, pinned_out), torch.cuda.synchronize()), n, dev, world, barrier)
        # the same copies in the same order with the kernels left out: what the host link allows
        res["copy_floor_ms"] = _timed(
            lambda i: runner.e2e_step(host, pinned_out, join=(i == last), copies_only=True), n, dev, world,
            barrier)
        res["copy_floor_gbs_each_way"] = h2d / (res["copy_floor_ms"] * 1e-3) / 1e9
        res["api"] = "dfa3d_b200.HostPipeline.run (extension-level entry points; not the autograd Functions)"
    return res


def measure_extras(a, w, dev, world, rank, barrier):
    """Driver-visible side measurements on this rank's shard, each the max over ranks:
    cfg3 (bf16 storage of value and dist) forward-only and forward+backward, and the headline step
    through the autograd Function with its allocations."""
    from dfa3d_b200 import workloads as wl
    extra = {}
    if w.name == "cfg2":
        w3 = wl.WORKLOADS["cfg3"].with_(B=w.B)
        d3 = wl.make_inputs(w3, seed=w3.seed + 1000 * rank)
        r3 = OursRunner(w3, {k: v.to(dev) for k, v in d3.items()})
        for _ in range(3):
            r3.forward(); r3.zero(); r3.backward()
        n = max(10, min(a.steps, 50))
        f_ms = _timed(lambda i: r3.forward(), n, dev, world, barrier)
        s_ms = _timed(lambda i: (r3.forward(), r3.zero(), r3.backward()), n, dev, world, barrier)
        extra["cfg3"] = {"workload": "cfg3: cfg2 shapes, bf16 value and dist, fp32 math and gradients",
                         "cameras_per_gpu": w3.B, "n_gpus": world, "steps": n,
                         "forward_only_ms": f_ms, "forward_only_points_per_s": w3.points * world / (f_ms * 1e-3),
                         "fwd_bwd_ms": s_ms, "fwd_bwd_points_per_s": w3.points * world / (s_ms * 1e-3)}
        del r3
        extra["few_points_per_item"] = measure_few_points(dev, world, barrier)
    return extra


def measure_few_points(dev, world, barrier):
    """The plain 2-D operator at the temporal self-attention shape (previous + current 200 x 200 BEV, 40 000
    queries, 8 heads x 32 channels, 1 level x 4 points: items of 4 points, several per warp) and with 32
    points per item (one item per warp) for comparison; same work on every rank, max over ranks."""
    from dfa3d_b200 import ext
    g = torch.Generator().manual_seed(7)
    B, side, Q, H, C = 2, 200, 40000, 8, 32
    shapes = torch.tensor([[side, side]], dtype=torch.int64, device=dev)
    lsi = torch.zeros(1, dtype=torch.int64, device=dev)
    value = torch.randn(B, side * side, H, C, generator=g).to(dev)
    go = torch.randn(B, Q, H * C, generator=g).to(dev)
    gv = torch.zeros_like(value)
    out = {"shape": "2 maps of 200x200, 40 000 queries, 8 heads x 32 channels, 1 level, plain 2-D operator"}
    for P in (4, 32):
        loc = torch.rand(B, Q, H, 1, P, 2, generator=g).to(dev)
        attn = torch.rand(B, Q, H, 1, P, generator=g).softmax(-1).to(dev)
        gl, ga = torch.empty_like(loc), torch.empty_like(attn)
        fwd = lambda i: ext.ms_deform_attn_forward(value, shapes, lsi, loc, attn, 64)
        bwd = lambda i: ext.ms_deform_attn_backward(value, shapes, lsi, loc, attn, go, gv, gl, ga, 64)
        for _ in range(3):
            fwd(0); bwd(0)
        f_ms, b_ms = _timed(fwd, 20, dev, world, barrier), _timed(bwd, 20, dev, world, barrier)
        pts = B * Q * H * P
        out[f"points_per_item_{P}"] = {"forward_ms": f_ms, "backward_ms": b_ms,
                                       "forward_points_per_s": pts / (f_ms * 1e-3),
                                       "backward_points_per_s": pts / (b_ms * 1e-3)}
    return out


def memory_stream_floor(w):
    """Lower bounds of the two kernels from the measured rates of the memory primitives they are made
    of (dfa3d_b200.rates replays a launch's address stream without the arithmetic)."""
    try:
        from dfa3d_b200 import rates
        f = rates.floors(w.levels, w.P, w.D, w.Q, w.B)
        f["what"] = ("probe launches with this workload's address stream: forward = value-row gathers + "
                     "dist-pair gathers; backward = the same gathers + grad_value row reductions + "
                     "grad_dist pair reductions; reductions only = what the L2 reduction units alone need")
        return f
    except Exception as e:          # measurement aid only: never fail the bench over it
        return {"unavailable": str(e)}


def report(a, w, world, launches_per_step, value, ms_per_step, fwd_ms, bwd_ms, clocks, e2e, extra=None):
    peak, peak_src = measured_peak_gbs()
    fwd_b, bwd_b = w.algorithmic_bytes()
    traffic = NCU_DRAM_TRAFFIC.get(w.name, {})
    line = {
        "metric": "DFA3D fwd+bwd sampled points/s", "value": value, "unit": "sampled points/s",
        "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 storage, f32 math" if w.value_dtype == "bf16" else "f32",
        "data": "synthetic",
        "config": {"workload": w.name, "cameras_per_gpu": w.B, "queries": w.Q, "heads": w.H,
                   "channels": w.C, "levels": [list(x) for x in w.levels], "points": w.P,
                   "depth_bins": w.D, "points_per_gpu_step": w.points,
                   "l2": ("inputs per step (%.0f MB) exceed the 126 MB L2; no explicit flush" % (fwd_b / 1e6))
                         if fwd_b > 126e6 else
                         ("inputs per step (%.1f MB) fit in the 126 MB L2 and no flush is made: a "
                          "parity-sized workload, not a bandwidth measurement" % (fwd_b / 1e6))},
        "kernel_ms": {"forward": fwd_ms, "backward": bwd_ms},
        "clocks": clocks,
        "gpu_launches": launches_per_step * a.steps,
        "e2e": e2e,
    }
    if a.impl == "ours":
        # items of 4 / 8 / 16 points (fp32, 16 / 32 / 64 channels) take the kernels in which a warp holds several
        packed = w.L * w.P in (4, 8, 16) and w.C in (16, 32, 64) and w.value_dtype == "fp32"
        line["roofline"] = {
            "kernel": "dfa3d_backward_packed_kernel" if packed else "dfa3d_backward_kernel", "bound": "hbm",
            "achieved": bwd_b / (bwd_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
            "frac": bwd_b / (bwd_ms * 1e-3) / 1e9 / peak, "traffic": traffic.get("backward"),
            "algorithmic_bytes": bwd_b, "peak_source": peak_src}
        line["roofline_forward"] = {
            "kernel": "dfa3d_forward_packed_kernel" if packed else "dfa3d_forward_kernel", "bound": "hbm",
            "achieved": fwd_b / (fwd_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
            "frac": fwd_b / (fwd_ms * 1e-3) / 1e9 / peak, "traffic": traffic.get("forward"),
            "algorithmic_bytes": fwd_b}
        line["roofline_step"] = {"frac": (fwd_b + bwd_b) / (ms_per_step * 1e-3) / 1e9 / peak,
                                 "algorithmic_bytes": fwd_b + bwd_b}
        floor = (extra or {}).get("memory_stream_floor") or {}
        if "backward_ms" in floor:
            # floor_ms: the launch's reductions alone at the measured L2 reduction rate (nothing the
            # kernel does can make them cheaper); stream_ms: all of its gathers and reductions replayed
            # without arithmetic
            line["roofline"]["floor_ms"] = floor["backward_reductions_only_ms"]
            line["roofline"]["frac_of_floor"] = floor["backward_reductions_only_ms"] / bwd_ms
            line["roofline"]["stream_ms"] = floor["backward_ms"]
            line["roofline_forward"]["stream_ms"] = floor["forward_ms"]
        if extra:
            line["extra"] = extra
        if world == 1 and not a.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(w, 1)
    else:
        line["impl"] = "reference"
        line["reference_kind"] = ("reference CUDA op (unmodified sources, sm_100a build in "
                                  "oracle/_ref) through its own autograd Function, same GPU")
        if world == 1 and not a.no_cpu_baseline:
            # the reference has no CPU implementation of this path; the CPU figure beside it is the
            # C + OpenMP port of its kernels
            line["cpu_baseline"] = cpu_baseline(w, 1)
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
