"""Forward + backward of the fused operator for tensors that live in pinned HOST memory.

Camera frames are independent in the operator, so a batch can stream through the GPU: while chunk i is
computed, chunk i+1 is copied in and the results of chunk i-1 are copied out (PCIe is full duplex).
Three CUDA streams and a ring of device-side slots do this; the wall time of a step approaches the
larger of the two copy directions instead of copy-in + compute + copy-out.  With ``join=False``
consecutive ``run()`` calls overlap as well: the first copies of the next batch go in while the last
results of the previous one go out, ordered only by the slots they share.

Every copy is one ``cudaMemcpyAsync`` (``Tensor.copy_(non_blocking=True)``) of one tensor's contiguous
camera range: five in and five out per chunk.
"""
import torch

from . import ext

_IN = ("value", "dist", "loc", "attn", "grad_out")
_OUT = ("out", "grad_value", "grad_dist", "grad_loc", "grad_attn")


class HostPipeline:
    """Reusable pipeline for one problem shape.

    ``run(host_in, host_out)``: ``host_in`` maps value (B,N,H,C), dist (B,N,D) or (B,N,H,D),
    loc (B,Q,H,L,P,3), attn (B,Q,H,L,P), grad_out (B,Q,H*C) to pinned host tensors; ``host_out``
    maps out, grad_value, grad_dist, grad_loc, grad_attn to pinned host tensors that receive the
    results.  value/dist may be bfloat16 or float16 (float16: both); all results are float32.

    Stream contract: all ``run()`` / ``join()`` calls of one pipeline must be issued from the same
    current stream (the pipeline orders its three side streams against that stream and against its own
    slot events, not against arbitrary other streams).  After ``run(..., join=True)`` the current stream
    waits for the results; after ``join=False`` the results of that call are complete only after
    ``join()`` (or a later ``run(join=True)``) and a synchronisation of the current stream, and the
    ``host_in`` tensors of that call must stay untouched until then.
    """

    def __init__(self, spatial_shapes_3d, level_start_index, device, cameras_per_chunk=2, slots=3,
                 im2col_step=64):
        self.device = torch.device(device)
        self.shapes = spatial_shapes_3d.to(self.device)
        self.lsi = level_start_index.to(self.device)
        self.step = im2col_step
        self.chunk = int(cameras_per_chunk)
        self.nslots = int(slots)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_cmp = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self._slots = None
        self._sig = None
        self._next = 0          # ring position; keeps advancing across run() calls

    def _make_slots(self, host_in):
        sig = tuple((k, tuple(host_in[k].shape[1:]), host_in[k].dtype) for k in _IN)
        if sig == self._sig:
            return
        if self._slots is not None:
            # the side streams may still be using the old slots: let them finish before the tensors go
            # back to the allocator (which would hand them out again on the caller's stream)
            for s in (self.s_in, self.s_cmp, self.s_out):
                s.synchronize()
        self._sig = sig
        c, dev = self.chunk, self.device
        self._slots = []
        self._next = 0
        for _ in range(self.nslots):
            s = {k: torch.empty((c,) + tuple(host_in[k].shape[1:]), dtype=host_in[k].dtype, device=dev)
                 for k in _IN}
            s["out"] = torch.empty((c,) + tuple(host_in["grad_out"].shape[1:]), device=dev)
            s["grad_value"] = torch.empty(s["value"].shape, device=dev)
            s["grad_dist"] = torch.empty(s["dist"].shape, device=dev)
            s["grad_loc"] = torch.empty_like(s["loc"])
            s["grad_attn"] = torch.empty_like(s["attn"])
            s["free"] = torch.cuda.Event()      # the slot's results have left the device
            s["used"] = False                   # `free` has been recorded at least once
            self._slots.append(s)

    def run(self, host_in, host_out, join=True, copies_only=False):
        """Enqueue one batch.  ``copies_only`` skips the kernels (same copies, same order): the time of
        such a run is the floor the host link sets for this pipeline."""
        for k in _IN:
            if not host_in[k].is_pinned():
                raise RuntimeError(f"host_in['{k}'] must be in pinned memory (tensor.pin_memory())")
        for k in _OUT:
            if not host_out[k].is_pinned():
                raise RuntimeError(f"host_out['{k}'] must be in pinned memory")
        B = host_in["value"].shape[0]
        cur = torch.cuda.current_stream(self.device)
        self._make_slots(host_in)                 # allocates on `cur`
        ready0 = torch.cuda.Event()
        ready0.record(cur)                        # whatever the caller enqueued so far (and the slots'
        self.s_in.wait_event(ready0)              # allocation) precedes this batch
        self.s_cmp.wait_event(ready0)
        self.s_out.wait_event(ready0)
        for c0 in range(0, B, self.chunk):
            c1 = min(B, c0 + self.chunk)
            n = c1 - c0
            s = self._slots[self._next % self.nslots]
            self._next += 1
            with torch.cuda.stream(self.s_in):
                if s["used"]:
                    self.s_in.wait_event(s["free"])
                for k in _IN:
                    s[k][:n].copy_(host_in[k][c0:c1], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(ready)
                if not copies_only:
                    ext.dfa3d_fused_forward(s["value"][:n], s["dist"][:n], self.shapes, self.lsi,
                                            s["loc"][:n], s["attn"][:n], self.step, need_depth_score=False,
                                            out=s["out"][:n])
                    s["grad_value"][:n].zero_()
                    s["grad_dist"][:n].zero_()
                    ext.dfa3d_fused_backward(s["value"][:n], s["dist"][:n], self.shapes, self.lsi,
                                             s["loc"][:n], s["attn"][:n], s["grad_out"][:n],
                                             s["grad_value"][:n], s["grad_dist"][:n], s["grad_loc"][:n],
                                             s["grad_attn"][:n], self.step)
                done = torch.cuda.Event()
                done.record(self.s_cmp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for k in _OUT:
                    host_out[k][c0:c1].copy_(s[k][:n], non_blocking=True)
                s["free"].record(self.s_out)
                s["used"] = True
        if join:
            self.join()
        return host_out

    def join(self):
        """Make the current stream wait for everything enqueued by earlier ``run()`` calls."""
        torch.cuda.current_stream(self.device).wait_stream(self.s_out)
