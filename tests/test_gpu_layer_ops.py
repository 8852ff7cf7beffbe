"""Encoder-layer row operations (residual add + LayerNorm, bias-gradient column sums) against torch's own
LayerNorm / Linear in float32 and float64."""
import pytest
import torch
import torch.nn.functional as F

from helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("with_residual", [False, True], ids=["plain", "residual"])
@pytest.mark.parametrize("rows,E", [(1, 128), (3, 4), (50, 32), (77, 200), (37, 256), (1000, 256), (5003, 384), (129, 640), (64, 1024)])
def test_add_layer_norm_matches_torch(lib_built, rows, E, with_residual):
    from dfa3d_b200.layer_ops import AddLayerNorm
    g = torch.Generator().manual_seed(rows + E)
    x = (torch.randn(rows, E, generator=g) * 2 + 0.5).to(DEV)
    r = torch.randn(rows, E, generator=g).to(DEV) if with_residual else None
    go = torch.randn(rows, E, generator=g).to(DEV)
    ln = AddLayerNorm(E).to(DEV)
    with torch.no_grad():
        ln.weight.copy_(torch.randn(E, generator=g)); ln.bias.copy_(torch.randn(E, generator=g))

    def run(fn, dtype):
        leaves = [t.detach().to(dtype).requires_grad_(True) if t is not None else None
                  for t in (x, r, ln.weight, ln.bias)]
        y = fn(*leaves)
        y.backward(go.to(dtype))
        return [y] + [t.grad for t in leaves if t is not None]

    def mine(a, b, w, bias):
        from dfa3d_b200.layer_ops import AddLayerNormFunction
        return AddLayerNormFunction.apply(a, b, w, bias, ln.eps)

    def torch_ln(a, b, w, bias):
        return F.layer_norm(a if b is None else a + b, (E,), w, bias, ln.eps)

    got, want = run(mine, torch.float32), run(torch_ln, torch.float64)
    names = ["y", "grad_x"] + (["grad_residual"] if with_residual else []) + ["grad_weight", "grad_bias"]
    for n, a, b in zip(names, got, want):
        # sums over rows (weight / bias gradients) carry the rounding of `rows` float32 additions
        tol = dict(rtol=2e-4, atol_frac=2e-6) if n.startswith("grad_w") or n.startswith("grad_b") \
            else dict(rtol=1e-4, atol_frac=1e-5) if n.startswith("grad") else dict(rtol=1e-5, atol_frac=2e-6)
        assert_close(n, a, b.float(), **tol)
    # the module form, 3-D input
    y3 = ln(x.view(1, rows, E), None if r is None else r.view(1, rows, E))
    assert y3.shape == (1, rows, E) and torch.equal(y3.view(rows, E), got[0])


def test_add_layer_norm_state_dict_is_layer_norm(lib_built):
    from dfa3d_b200.layer_ops import AddLayerNorm
    a, b = AddLayerNorm(256), torch.nn.LayerNorm(256)
    assert list(a.state_dict()) == list(b.state_dict())
    b.load_state_dict(a.state_dict())


def test_layer_op_argument_checks(lib_built):
    from dfa3d_b200.layer_ops import AddLayerNorm, column_sum
    with pytest.raises(RuntimeError, match="multiple of 4"):
        AddLayerNorm(102).to(DEV)(torch.zeros(4, 102, device=DEV))
    with pytest.raises(RuntimeError, match="float32 CUDA"):
        AddLayerNorm(128)(torch.zeros(4, 128))
    with pytest.raises(RuntimeError, match="does not match"):
        AddLayerNorm(128).to(DEV)(torch.zeros(4, 128, device=DEV), torch.zeros(3, 128, device=DEV))
    with pytest.raises(RuntimeError, match="multiple of 4"):
        column_sum(torch.zeros(4, 6, device=DEV))
    assert column_sum(torch.zeros(0, 8, device=DEV)).tolist() == [0.0] * 8
    empty = AddLayerNorm(128).to(DEV)(torch.zeros(0, 128, device=DEV))
    assert empty.shape == (0, 128)


@pytest.mark.parametrize("rows,cols", [(1, 4), (7, 12), (1000, 256), (40001, 512), (333, 772), (184950, 256)])
def test_column_sum_matches_torch(lib_built, rows, cols):
    from dfa3d_b200.layer_ops import column_sum
    g = torch.Generator().manual_seed(rows)
    src = torch.randn(rows, cols, generator=g).to(DEV)
    want = src.double().sum(0)
    assert_close("column_sum", column_sum(src), want.float(), rtol=1e-5, atol=float(rows) ** 0.5 * 1e-6)


@pytest.mark.parametrize("rows", [777, 16384 + 5])      # below and above the row count that splits the weight gradient
def test_linear_matches_torch_linear(lib_built, rows):
    from dfa3d_b200.layer_ops import Linear
    torch.manual_seed(3)
    mine, ref = Linear(256, 512).to(DEV), torch.nn.Linear(256, 512).to(DEV)
    ref.load_state_dict(mine.state_dict())
    x = torch.randn(2, rows, 256, device=DEV)
    go = torch.randn(2, rows, 512, device=DEV)
    outs = []
    for m in (mine, ref):
        xi = x.clone().requires_grad_(True)
        y = m(xi)
        y.backward(go)
        outs.append((y, xi.grad, m.weight.grad, m.bias.grad))
    for n, a, b in zip(("y", "grad_x", "grad_weight", "grad_bias"), *outs):
        assert_close(n, a, b, rtol=1e-4, atol_frac=1e-5)


def test_measure_times_every_row_kernel(lib_built):
    from dfa3d_b200 import layer_ops
    got = layer_ops.measure(DEV)
    assert {g["kernel"] for g in got} == {"column_sum", "add_layer_norm_forward", "layer_norm_backward"}
    assert all(g["ms"] > 0 and g["GB/s"] > 0 and g["torch_ms"] > 0 for g in got)


def test_layer_ops_compute_in_float32_under_autocast(lib_built):
    from dfa3d_b200.layer_ops import AddLayerNorm, Linear
    torch.manual_seed(0)
    ln, lin = AddLayerNorm(128).to(DEV), Linear(128, 64).to(DEV)
    x = torch.randn(9, 128, device=DEV, requires_grad=True)
    want = ln(lin(x).repeat(1, 2), x)
    with torch.autocast("cuda", dtype=torch.float16):
        got = ln(lin(x.half()).repeat(1, 2), x.half())
    assert got.dtype == torch.float32
    assert_close("autocast", got, want, rtol=5e-3, atol=5e-3)
    got.sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()


def test_residual_block_gradients_match_torch(lib_built):
    """A post-norm residual block as the encoder layer builds it -- norm(branch(q), q), twice, the residual
    feeding its own branch -- against the same block on torch.nn.LayerNorm / torch.nn.Linear: the input
    gradient (which sums the norm's gradient with the branch's) and every parameter gradient."""
    from dfa3d_b200.layer_ops import AddLayerNorm, Linear
    torch.manual_seed(11)
    E, rows = 128, 301
    mine = torch.nn.ModuleList([Linear(E, E), AddLayerNorm(E), Linear(E, E), AddLayerNorm(E)]).to(DEV)
    ref = torch.nn.ModuleList([torch.nn.Linear(E, E), torch.nn.LayerNorm(E), torch.nn.Linear(E, E),
                               torch.nn.LayerNorm(E)]).to(DEV)
    ref.load_state_dict(mine.state_dict())
    q0 = torch.randn(2, rows, E, device=DEV)
    go = torch.randn(2, rows, E, device=DEV)

    def run(m, fused):
        q = q0.clone().requires_grad_(True)
        x = m[1](m[0](q), q) if fused else m[1](m[0](q) + q)
        y = m[3](torch.relu(m[2](x)), x) if fused else m[3](torch.relu(m[2](x)) + x)
        y.backward(go)
        return [y, q.grad] + [p.grad for p in m.parameters()]

    for i, (a, b) in enumerate(zip(run(mine, True), run(ref, False))):
        assert_close(f"tensor {i}", a, b, rtol=2e-4, atol_frac=2e-5)
