"""Forward + backward of the fused operator for tensors that live in pinned HOST memory.

Camera frames are independent in the operator, so a batch can stream through the GPU: while chunk i is
computed, chunk i+1 is copied in and the results of chunk i-1 are copied out (PCIe is full duplex).
Three CUDA streams and a ring of device-side slots do this; the wall time of a step approaches the
larger of the two copy directions instead of copy-in + compute + copy-out.
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
    results.  value/dist may be bfloat16; all results are float32.
    """

    def __init__(self, spatial_shapes_3d, level_start_index, device, cameras_per_chunk=1, slots=3,
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

    def _make_slots(self, host_in):
        sig = tuple((k, tuple(host_in[k].shape[1:]), host_in[k].dtype) for k in _IN)
        if sig == self._sig:
            return
        self._sig = sig
        c, dev = self.chunk, self.device
        self._slots = []
        for _ in range(self.nslots):
            s = {k: torch.empty((c,) + tuple(host_in[k].shape[1:]), dtype=host_in[k].dtype, device=dev)
                 for k in _IN}
            s["out"] = torch.empty((c,) + tuple(host_in["grad_out"].shape[1:]), device=dev)
            s["grad_value"] = torch.empty(s["value"].shape, device=dev)
            s["grad_dist"] = torch.empty(s["dist"].shape, device=dev)
            s["grad_loc"] = torch.empty_like(s["loc"])
            s["grad_attn"] = torch.empty_like(s["attn"])
            s["free"] = torch.cuda.Event()      # the slot's results have left the device
            self._slots.append(s)

    def run(self, host_in, host_out):
        for k in _IN:
            if not host_in[k].is_pinned():
                raise RuntimeError(f"host_in['{k}'] must be in pinned memory (tensor.pin_memory())")
        for k in _OUT:
            if not host_out[k].is_pinned():
                raise RuntimeError(f"host_out['{k}'] must be in pinned memory")
        B = host_in["value"].shape[0]
        self._make_slots(host_in)
        cur = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(cur)
        self.s_out.wait_stream(cur)
        i = 0
        for c0 in range(0, B, self.chunk):
            c1 = min(B, c0 + self.chunk)
            n = c1 - c0
            s = self._slots[i % self.nslots]
            with torch.cuda.stream(self.s_in):
                if i >= self.nslots:
                    self.s_in.wait_event(s["free"])
                for k in _IN:
                    s[k][:n].copy_(host_in[k][c0:c1], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(ready)
                ext.dfa3d_fused_forward(s["value"][:n], s["dist"][:n], self.shapes, self.lsi, s["loc"][:n],
                                        s["attn"][:n], self.step, need_depth_score=False, out=s["out"][:n])
                s["grad_value"][:n].zero_()
                s["grad_dist"][:n].zero_()
                ext.dfa3d_fused_backward(s["value"][:n], s["dist"][:n], self.shapes, self.lsi, s["loc"][:n],
                                         s["attn"][:n], s["grad_out"][:n], s["grad_value"][:n],
                                         s["grad_dist"][:n], s["grad_loc"][:n], s["grad_attn"][:n],
                                         self.step)
                done = torch.cuda.Event()
                done.record(self.s_cmp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for k in _OUT:
                    host_out[k][c0:c1].copy_(s[k][:n], non_blocking=True)
                s["free"].record(self.s_out)
            i += 1
        cur.wait_stream(self.s_out)
        return host_out
