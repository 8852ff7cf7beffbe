"""Data-parallel plumbing around the operator: one process per GPU, camera frames sharded over ranks.

Every camera frame is independent in the forward and in the backward of the operator (all its tensors
carry the leading batch*camera dimension), so the operator itself needs no collective.  What is
needed across ranks: a partition of the frames that keeps the cameras of one frame together, the
maximum over ranks of a device-measured time, and -- for training configurations -- the all-reduce of
the projection-layer gradients (the reference gets this from mmcv's DistributedDataParallel wrapper,
BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/apis/mmdet_train.py:71-79).
"""
import torch
import torch.distributed as dist


def bind_cpu_affinity_to_gpu(index):
    """Pin the calling process to the CPU cores NVML reports as local to GPU `index` (its NUMA node).

    With one process per GPU this keeps each rank's pinned host buffers and its copy-issuing thread on
    the socket the GPU hangs off; host<->device streaming of several ranks then does not cross the
    inter-socket link.  Read-only NVML query plus sched_setaffinity on this process; returns the number
    of cores bound to, or 0 if NVML or the affinity call is unavailable (nothing is changed then)."""
    import os
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (w >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return 0
        os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:
        return 0


def shard_frames(num_frames, world_size, rank):
    """Contiguous, balanced partition of `num_frames` frames.  Returns range(start, stop); the first
    `num_frames % world_size` ranks get one frame more."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside [0, {world_size})")
    base, extra = divmod(num_frames, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def shard_cameras(num_frames, cams_per_frame, world_size, rank):
    """Slice of the flattened (frame, camera) batch dimension owned by `rank`: whole frames only."""
    fr = shard_frames(num_frames, world_size, rank)
    return slice(fr.start * cams_per_frame, fr.stop * cams_per_frame)


def shard_queries(num_queries, world_size, rank):
    """Query block of `rank` when ONE batch of frames is split over the ranks (strong scaling): a
    contiguous, balanced slice of the query dimension.  The value / depth-distribution tensors are
    then replicated (one broadcast) and the gradients with respect to them are partial sums that
    need one all-reduce (`allreduce_sum_`)."""
    r = shard_frames(num_queries, world_size, rank)
    return slice(r.start, r.stop)


def camera_query_grid(num_cameras, world_size, rank, camera_groups=0):
    """Two-dimensional split of ONE batch of camera frames over the ranks: `camera_groups` groups of
    ranks, each owning a contiguous block of cameras; inside a group the queries are split.  Gradients
    with respect to value / dist are then partial sums only over the ranks of one group, so the
    exchange moves 1/camera_groups of the bytes among world_size/camera_groups ranks.

    camera_groups = 0 picks the largest number of groups that divides both world_size and the number
    of cameras, so that every rank gets the same work (more groups = less to exchange; with world_size
    groups nothing at all).
    Returns (group index, ranks of this rank's group, camera slice, query block index, query blocks)."""
    g = int(camera_groups)
    if g <= 0:
        g = max(d for d in range(1, world_size + 1) if world_size % d == 0 and num_cameras % d == 0)
    if world_size % g != 0 or g > num_cameras:
        raise ValueError(f"camera_groups={g} must divide world_size={world_size} and not exceed "
                         f"the {num_cameras} cameras")
    per = world_size // g
    gi, qi = rank // per, rank % per
    cams = shard_frames(num_cameras, g, gi)
    return gi, list(range(gi * per, (gi + 1) * per)), slice(cams.start, cams.stop), qi, per


def allreduce_sum_(tensors, group=None, async_op=False):
    """In-place SUM all-reduce of each tensor over the group (the exchange step of the query-block
    mode: grad_value and grad_dist are partial sums over the ranks' query blocks).  Returns the list of
    work handles when async_op is set."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return []
    works = [dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group, async_op=async_op) for t in tensors]
    return [w for w in works if w is not None]


def max_over_ranks(value, device=None, group=None):
    """Maximum of a per-rank scalar (a device-measured duration) over the process group."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def allreduce_gradients(params, group=None, bucket_bytes=32 << 20):
    """Average the gradients of `params` over the group in flat buckets (one collective per bucket:
    sized for launch latency, NVSwitch gives every pair full bandwidth)."""
    if not (dist.is_available() and dist.is_initialized()):
        return 0
    world = dist.get_world_size(group)
    if world == 1:
        return 0
    grads = [p.grad for p in params if p.grad is not None]
    buckets, cur, cur_bytes = [], [], 0
    for g in grads:
        nb = g.numel() * g.element_size()
        if cur and (cur_bytes + nb > bucket_bytes or g.dtype != cur[0].dtype):
            buckets.append(cur); cur, cur_bytes = [], 0
        cur.append(g); cur_bytes += nb
    if cur:
        buckets.append(cur)
    for b in buckets:
        flat = torch.cat([g.reshape(-1) for g in b])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        flat.div_(world)
        off = 0
        for g in b:
            g.copy_(flat[off:off + g.numel()].view_as(g)); off += g.numel()
    return len(buckets)
