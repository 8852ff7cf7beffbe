"""Row operations of the encoder layer around the attention operator, on the library's own kernels
(C entry points ``dfa3d_add_layer_norm_forward``, ``dfa3d_layer_norm_backward``, ``dfa3d_column_sum``).

The reference's layer (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/encoder.py:363-411,
custom_base_transformer_layer.py) applies ``norm(x + branch(x))`` after each block with torch's LayerNorm
and torch's Linear.  Here

  * ``AddLayerNorm`` is a LayerNorm (same parameters, same state dict keys as ``torch.nn.LayerNorm``)
    whose forward takes an optional residual: one kernel forms the sum and normalises it, one kernel
    produces the input gradient and the weight / bias gradients.
  * ``Linear`` is ``torch.nn.Linear`` whose bias gradient is a single column-sum kernel; the matrix
    products stay with cuBLAS (the weight gradient as a batch of row slices, see ``weight_gradient``).

float32 CUDA tensors only (under autocast the inputs are cast to float32, like the package's ``*_fp32``
Functions); like the rest of the package there is no fallback path.
"""
import torch
import torch.nn as nn
from torch.autograd.function import Function, once_differentiable

from . import _lib


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _check(t, name):
    if not t.is_cuda or t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be a float32 CUDA tensor, got {t.dtype} on {t.device}")


def column_sum(src):
    """(rows, cols) float32 -> (cols,): sum over the rows."""
    _check(src, "src")
    if src.dim() != 2:
        raise RuntimeError("column_sum takes a (rows, cols) matrix")
    src = src.contiguous()
    rows, cols = src.shape
    dst = torch.zeros(cols, dtype=torch.float32, device=src.device)
    with torch.cuda.device(src.device):
        _lib.call_plain("dfa3d_column_sum", src.data_ptr(), rows, cols, dst.data_ptr(), _stream(src))
    return dst


class AddLayerNormFunction(Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float32)
    def forward(ctx, x, residual, weight, bias, eps):
        """LayerNorm(x + residual) over the last dimension; residual may be None."""
        for t, n in ((x, "x"), (weight, "weight"), (bias, "bias")):
            _check(t, n)
        E = x.shape[-1]
        if weight.numel() != E or bias.numel() != E:
            raise RuntimeError(f"weight and bias must have {E} elements")
        x = x.contiguous()
        rows = x.numel() // E if E else 0
        summed = None
        if residual is not None:
            _check(residual, "residual")
            if residual.shape != x.shape:
                raise RuntimeError(f"residual {tuple(residual.shape)} does not match x {tuple(x.shape)}")
            residual = residual.contiguous()
            summed = torch.empty_like(x)
        y = torch.empty_like(x)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        weight, bias = weight.contiguous(), bias.contiguous()
        with torch.cuda.device(x.device):
            _lib.call_plain("dfa3d_add_layer_norm_forward", x.data_ptr(),
                            None if residual is None else residual.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                            rows, E, float(eps), None if summed is None else summed.data_ptr(), y.data_ptr(),
                            mean.data_ptr(), rstd.data_ptr(), _stream(x))
        ctx.save_for_backward(x if summed is None else summed, weight, mean, rstd)
        ctx.has_residual = residual is not None
        return y

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    @once_differentiable
    def backward(ctx, grad_y):
        inp, weight, mean, rstd = ctx.saved_tensors
        E = inp.shape[-1]
        grad_y = grad_y.contiguous()
        grad_in = torch.empty_like(inp)
        grad_wb = torch.zeros((2, E), dtype=torch.float32, device=inp.device)     # one fill for both
        grad_w, grad_b = grad_wb[0], grad_wb[1]
        with torch.cuda.device(inp.device):
            _lib.call_plain("dfa3d_layer_norm_backward", grad_y.data_ptr(), inp.data_ptr(), weight.data_ptr(),
                            mean.data_ptr(), rstd.data_ptr(), mean.numel(), E, grad_in.data_ptr(),
                            grad_w.data_ptr(), grad_b.data_ptr(), _stream(inp))
        return grad_in, (grad_in if ctx.has_residual else None), grad_w, grad_b, None


class AddLayerNorm(nn.LayerNorm):
    """``torch.nn.LayerNorm`` over the last dimension with an optional residual: ``forward(x, residual)``
    returns ``LayerNorm(x + residual)``."""

    def __init__(self, normalized_shape, eps=1e-5):
        super().__init__(normalized_shape, eps=eps, elementwise_affine=True)
        if len(self.normalized_shape) != 1:
            raise ValueError("AddLayerNorm normalises the last dimension only")

    def forward(self, x, residual=None):
        return AddLayerNormFunction.apply(x, residual, self.weight, self.bias, self.eps)


_SPLIT_ROWS, _SPLITS = 16384, 16


def weight_gradient(grad_out2, x2):
    """grad_out2 (rows, out)ᵀ @ x2 (rows, in) -> (out, in).  With many rows and a small result the product is
    one long reduction that cuBLAS runs on few CTAs (measured 60-206 us for 40 000-185 000 rows of 256-768
    columns, 4-7 times the time of reading the operands); as a batch of 16 row slices plus a sum of the 16
    partial results it takes 25-80 us."""
    rows = grad_out2.shape[0]
    if rows < _SPLIT_ROWS:
        return grad_out2.t() @ x2
    k = rows // _SPLITS
    head = k * _SPLITS
    w = torch.bmm(grad_out2[:head].view(_SPLITS, k, -1).transpose(1, 2), x2[:head].view(_SPLITS, k, -1)).sum(0)
    if head < rows:
        w.addmm_(grad_out2[head:].t(), x2[head:])
    return w


class LinearFunction(Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float32)
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        # written into a tensor of its own (F.linear returns a view of the 2-D product for inputs of more
        # dimensions, which an in-place activation after a custom Function must not modify)
        y = torch.empty(x.shape[:-1] + (weight.shape[0],), dtype=x.dtype, device=x.device)
        torch.addmm(bias, x.reshape(-1, x.shape[-1]), weight.t(), out=y.view(-1, weight.shape[0]))
        return y

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    @once_differentiable
    def backward(ctx, grad_out):
        x, weight = ctx.saved_tensors
        g2 = grad_out.reshape(-1, grad_out.shape[-1])
        grad_x = grad_w = grad_b = None
        if ctx.needs_input_grad[0]:
            grad_x = (g2 @ weight).view(x.shape)
        if ctx.needs_input_grad[1]:
            grad_w = weight_gradient(g2, x.reshape(-1, x.shape[-1]))
        if ctx.needs_input_grad[2]:
            grad_b = column_sum(g2)
        return grad_x, grad_w, grad_b


class Linear(nn.Linear):
    """``torch.nn.Linear`` (same parameters); the bias gradient is one column-sum kernel."""

    def forward(self, x):
        if self.bias is None or self.out_features % 4 != 0:
            return super().forward(x)
        return LinearFunction.apply(x, self.weight, self.bias)


def _time_ms(fn, launches=200):
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / launches


def measure(device="cuda"):
    """CUDA-event timings of the three kernels at the encoder stack's sizes, called through the C entry
    points on preallocated tensors, with torch's kernels for the same work beside them.  Returns a list of
    dicts (GB/s = bytes every operand and result is read / written once, over the time)."""
    out = []
    st = torch.cuda.current_stream(device).cuda_stream
    for rows, cols in ((184950, 256), (60000, 768), (60000, 512), (40000, 256)):
        src = torch.randn(rows, cols, device=device)
        dst = torch.zeros(cols, device=device)
        ms = _time_ms(lambda: _lib.call_plain("dfa3d_column_sum", src.data_ptr(), rows, cols, dst.data_ptr(), st))
        out.append({"kernel": "column_sum", "rows": rows, "cols": cols, "ms": ms,
                    "GB/s": rows * cols * 4 / ms / 1e6, "torch_ms": _time_ms(lambda: src.sum(0))})
    for rows, E in ((240000, 256), (40000, 256)):
        x, r, go = (torch.randn(rows, E, device=device) for _ in range(3))
        w, b = torch.ones(E, device=device), torch.zeros(E, device=device)
        s, y, gi = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
        mean, rstd = torch.empty(rows, device=device), torch.empty(rows, device=device)
        gwb = torch.zeros(2, E, device=device)
        fwd = lambda: _lib.call_plain("dfa3d_add_layer_norm_forward", x.data_ptr(), r.data_ptr(), w.data_ptr(),
                                      b.data_ptr(), rows, E, 1e-5, s.data_ptr(), y.data_ptr(), mean.data_ptr(),
                                      rstd.data_ptr(), st)
        bwd = lambda: _lib.call_plain("dfa3d_layer_norm_backward", go.data_ptr(), s.data_ptr(), w.data_ptr(),
                                      mean.data_ptr(), rstd.data_ptr(), rows, E, gi.data_ptr(), gwb[0].data_ptr(),
                                      gwb[1].data_ptr(), st)
        f_ms, b_ms = _time_ms(fwd), _time_ms(bwd)
        xs = (x + r).requires_grad_(True)
        ln = torch.nn.LayerNorm(E).to(device)
        t_f = _time_ms(lambda: torch.nn.functional.layer_norm(x + r, (E,), ln.weight, ln.bias))
        yy = ln(xs)
        t_b = _time_ms(lambda: torch.autograd.grad(yy, (xs, ln.weight, ln.bias), go, retain_graph=True))
        out.append({"kernel": "add_layer_norm_forward", "rows": rows, "cols": E, "ms": f_ms,
                    "GB/s": 4 * rows * E * 4 / f_ms / 1e6, "torch_ms": t_f})
        out.append({"kernel": "layer_norm_backward", "rows": rows, "cols": E, "ms": b_ms,
                    "GB/s": 3 * rows * E * 4 / b_ms / 1e6, "torch_ms": t_b})
    return out


if __name__ == "__main__":      # python -m dfa3d_b200.layer_ops   (with the package directory on PYTHONPATH)
    import json
    for line in measure():
        print(json.dumps(line))
