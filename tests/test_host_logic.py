"""Host-side logic that needs no GPU: location assembly, per-camera re-batching, module
initialisation, the dfa3D drop-in package, frame sharding and the world_size-2 gloo path."""
import math
import os
import subprocess
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dfa3d_b200 import modules, sharding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "3d-deformable-attention_b200")


def test_assemble_sampling_locations_matches_loops():
    g = torch.Generator().manual_seed(0)
    bs, Q, H, L, Z, P = 2, 3, 2, 2, 4, 2
    ref = torch.rand(bs, Q, Z, 3, generator=g)
    ouv = torch.randn(bs, Q, H, L, P * Z, 2, generator=g)
    od = torch.randn(bs, Q, H, L, P * Z, 1, generator=g)
    shapes = torch.tensor([[6, 9], [3, 5]])
    D = 7
    got = modules.assemble_sampling_locations(ref, ouv, od, shapes, D)
    assert got.shape == (bs, Q, H, L, P * Z, 3)
    for b in range(bs):
        for q in range(Q):
            for h in range(H):
                for l in range(L):
                    for j in range(P * Z):
                        z = j % Z          # the points of a level cycle through the anchors
                        hh, ww = shapes[l].tolist()
                        exp = torch.stack([ref[b, q, z, 0] + ouv[b, q, h, l, j, 0] / ww,
                                           ref[b, q, z, 1] + ouv[b, q, h, l, j, 1] / hh,
                                           ref[b, q, z, 2] + od[b, q, h, l, j, 0] / D])
                        torch.testing.assert_close(got[b, q, h, l, j], exp)


def test_point_sampling_matches_per_point_projection():
    """modules.point_sampling (encoder.py:421-476) against a projection written point by point."""
    g = torch.Generator().manual_seed(4)
    bs, cams, Q, Z = 2, 3, 11, 4
    ref = torch.rand(bs, Z, Q, 3, generator=g)
    pc_range = (-51.2, -51.2, -5.0, 51.2, 51.2, 3.0)
    d_bound = (2.0, 58.0, 0.5)
    img_shape = (928, 1600)
    lidar2img = torch.randn(bs, cams, 4, 4, generator=g) * 50
    cam_pts, mask = modules.point_sampling(ref, pc_range, lidar2img, img_shape, d_bound)
    assert cam_pts.shape == (cams, bs, Q, Z, 3) and mask.shape == (cams, bs, Q, Z)
    assert mask.dtype == torch.bool
    for j in range(bs):
        for i in range(cams):
            for q in range(Q):
                for z in range(Z):
                    p = ref[j, z, q]
                    world = torch.tensor([p[0] * 102.4 - 51.2, p[1] * 102.4 - 51.2, p[2] * 8.0 - 5.0, 1.0])
                    c = lidar2img[j, i] @ world
                    front = c[2] > 1e-5
                    x = c[0] / max(c[2].item(), 1e-5) / img_shape[1]
                    y = c[1] / max(c[2].item(), 1e-5) / img_shape[0]
                    dz = (c[2] - 2.0) / 56.0
                    got = cam_pts[i, j, q, z]
                    torch.testing.assert_close(got, torch.stack([x, y, dz]), rtol=1e-4, atol=1e-4)
                    assert bool(mask[i, j, q, z]) == bool(front and 0 < x < 1 and 0 < y < 1)


def test_module_initialisation_follows_reference():
    m = modules.MSDeformableAttention3D_DFA3D(embed_dims=64, num_heads=8, num_levels=2, num_points=4)
    assert not m.sampling_offsets.weight.any() and not m.attention_weights.weight.any()
    b = m.sampling_offsets.bias.view(8, 2, 4, 2)
    # head 0 points along +x, scaled by the point index (1..P)
    torch.testing.assert_close(b[0, 0, :, 0], torch.arange(1.0, 5.0))
    torch.testing.assert_close(b[0, 0, :, 1], torch.zeros(4))
    bd = m.sampling_offsets_depth.bias.view(8, 2, 4)
    th = 2 * math.pi / 8
    torch.testing.assert_close(bd[1, 1, 2], torch.tensor((math.cos(th) + math.sin(th)) / 2 * 3))
    names = {n for n, _ in m.named_parameters()}
    for n in ("sampling_offsets.weight", "sampling_offsets_depth.bias", "attention_weights.weight",
              "value_proj.weight"):
        assert n in names                 # same parameter names as the reference module


def test_dfa3D_drop_in_package_exposes_reference_names(lib_built):
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "from dfa3D import ext_loader\n"
        "ext = ext_loader.load_ext('_ext', ['wms_deform_attn_backward', 'wms_deform_attn_forward',"
        " 'ms_depth_score_sample_forward', 'ms_depth_score_sample_backward'])\n"
        "from dfa3D.ops.multi_scale_3D_deform_attn import (WeightedMultiScaleDeformableAttnFunction,"
        " MultiScaleDepthScoreSampleFunction, MultiScale3DDeformableAttnFunction)\n"
        "from dfa3D.ops import MultiScaleDepthScoreSampleFunction as A\n"
        "assert A is MultiScaleDepthScoreSampleFunction\n"
        "try:\n ext_loader.load_ext('_ext', ['nope'])\nexcept AssertionError as e:\n assert 'miss in module' in str(e)\n"
        "else:\n raise SystemExit('load_ext accepted a missing function')\n"
        "print('ok')\n" % PKG_DIR)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr


def test_shard_frames_partitions_everything():
    for n in (1, 6, 8, 48):
        for world in (1, 2, 3, 8):
            got = [i for r in range(world) for i in sharding.shard_frames(n, world, r)]
            assert got == list(range(n))
            sizes = [len(sharding.shard_frames(n, world, r)) for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    assert sharding.shard_cameras(8, 6, 4, 1) == slice(12, 24)
    with pytest.raises(ValueError):
        sharding.shard_frames(4, 2, 2)


def _gloo_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # frames of a global batch are split with whole frames per rank
        frames = sharding.shard_frames(5, world, rank)
        t = sharding.max_over_ranks(1.0 + rank)                 # slowest rank's time
        lin = torch.nn.Linear(3, 2)
        with torch.no_grad():
            lin.weight.fill_(1.0); lin.bias.fill_(0.0)
        x = torch.full((4, 3), float(rank + 1))
        lin(x).sum().backward()
        nb = sharding.allreduce_gradients(list(lin.parameters()), bucket_bytes=16)
        q.put((rank, list(frames), t, lin.weight.grad.clone(), lin.bias.grad.clone(), nb))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_world_size_2_gloo_sharding_and_gradient_allreduce():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted((q.get(timeout=120) for _ in range(world)), key=lambda x: x[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0][1] + res[1][1] == [0, 1, 2, 3, 4]
    assert res[0][2] == res[1][2] == 2.0
    # rank r's weight grad is 4*(r+1) per element: the average over the two ranks is 6
    for r in res:
        torch.testing.assert_close(r[3], torch.full((2, 3), 6.0))
        torch.testing.assert_close(r[4], torch.full((2,), 4.0))
        assert r[5] >= 2                                        # tiny buckets -> several collectives


def _gloo_query_block_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        qs = sharding.shard_queries(7, world, rank)
        # a stand-in "gradient": each rank contributes the sum of its query indices
        g = torch.full((3,), float(sum(range(7)[qs])))
        works = sharding.allreduce_sum_([g], async_op=True)
        for w in works:
            w.wait()
        q.put((rank, (qs.start, qs.stop), g.clone()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_world_size_2_gloo_query_block_exchange():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_gloo_query_block_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted((q.get(timeout=120) for _ in range(world)), key=lambda x: x[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0][1] == (0, 4) and res[1][1] == (4, 7)
    for r in res:                                   # every rank ends with the full sum 0+...+6
        torch.testing.assert_close(r[2], torch.full((3,), 21.0))
    assert sharding.allreduce_sum_([torch.ones(1)]) == []      # no process group: nothing to do


def test_camera_query_grid_covers_every_camera_query_pair_once():
    """The 2-D split of the query-block mode: camera groups x query blocks tile the batch exactly."""
    for cams, world in ((6, 1), (6, 2), (6, 4), (6, 8), (6, 3), (6, 6), (5, 4), (8, 8)):
        Q = 103
        seen = torch.zeros(cams, Q, dtype=torch.int32)
        sizes = set()
        for rank in range(world):
            gi, ranks, cs, qi, qblocks = sharding.camera_query_grid(cams, world, rank)
            assert rank in ranks and len(ranks) == qblocks and world % qblocks == 0
            qs = sharding.shard_queries(Q, qblocks, qi)
            seen[cs, qs] += 1
            sizes.add(cs.stop - cs.start)
        assert (seen == 1).all(), (cams, world)
        assert len(sizes) == 1                      # balanced: every group owns the same number of cameras
    # 8 GPUs, 6 cameras: 2 groups of 3 cameras x 4 query blocks; 2 GPUs: one camera group each, no exchange
    assert sharding.camera_query_grid(6, 8, 5)[:2] == (1, [4, 5, 6, 7])
    assert sharding.camera_query_grid(6, 2, 1)[3:] == (0, 1)
    with pytest.raises(ValueError):
        sharding.camera_query_grid(6, 8, 0, camera_groups=3)


def test_bev_reference_points_are_cell_and_pillar_centres():
    """modules.bev_reference_points against the closed forms of encoder.py:61-99."""
    H, W, Z, n, bs = 3, 5, 8, 4, 2
    r3 = modules.bev_reference_points(H, W, Z, n, "3d", bs, "cpu")
    r2 = modules.bev_reference_points(H, W, dim="2d", bs=bs, device="cpu")
    assert r3.shape == (bs, n, H * W, 3) and r2.shape == (bs, H * W, 1, 2)
    for y in range(H):
        for x in range(W):
            q = y * W + x
            assert torch.allclose(r2[1, q, 0], torch.tensor([(x + 0.5) / W, (y + 0.5) / H]))
            for k in range(n):
                z = (0.5 + k * (Z - 1.0) / (n - 1)) / Z
                assert torch.allclose(r3[0, k, q], torch.tensor([(x + 0.5) / W, (y + 0.5) / H, z]))


def test_layer_ops_refuse_cpu_tensors_and_keep_torch_parameter_names():
    """No fallback path: the row operations raise on CPU tensors; their modules keep torch's parameter names
    so that checkpoints of the reference's LayerNorm / Linear layers load."""
    import pytest
    import torch
    from dfa3d_b200.layer_ops import AddLayerNorm, Linear, column_sum, weight_gradient
    with pytest.raises(RuntimeError, match="float32 CUDA"):
        AddLayerNorm(128)(torch.zeros(2, 128))
    with pytest.raises(RuntimeError, match="float32 CUDA"):
        column_sum(torch.zeros(4, 8))
    assert list(AddLayerNorm(64).state_dict()) == list(torch.nn.LayerNorm(64).state_dict())
    assert list(Linear(8, 4).state_dict()) == list(torch.nn.Linear(8, 4).state_dict())
    # the sliced weight gradient equals the plain product (CPU tensors: pure torch arithmetic)
    g = torch.Generator().manual_seed(0)
    go, x = torch.randn(16384 + 7, 12, generator=g), torch.randn(16384 + 7, 20, generator=g)
    torch.testing.assert_close(weight_gradient(go, x), go.t() @ x, rtol=1e-4, atol=1e-3)
    torch.testing.assert_close(weight_gradient(go[:100], x[:100]), go[:100].t() @ x[:100])
