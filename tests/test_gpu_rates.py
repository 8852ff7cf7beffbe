"""The memory-primitive rate probes run and report plausible figures (they are what the kernels' lower
bounds in the bench line are derived from)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_rate_probes_run_and_leave_the_expected_sums(lib_built):
    from dfa3d_b200 import rates
    levels, P, D, Q, B = ((12, 20), (6, 10), (3, 5), (2, 3)), 8, 16, 500, 2
    pb = rates.Prober(levels, P, D, Q, B, dead_fraction=0.15)
    # reductions add exactly 1 to every float they touch: the row probe and the bulk (TMA) row probe
    # must leave the same totals, 32 floats per live in-image corner row
    pb.launch(rates.RED_ROWS)
    torch.cuda.synchronize()
    rows = pb.grad_value.double().sum().item() / 32
    assert 0 < rows <= B * Q * 8 * 32 * 4 and rows == int(rows)
    pb.grad_value.zero_()
    pb.launch(rates.BULK_RED_ROWS)
    torch.cuda.synchronize()
    assert pb.grad_value.double().sum().item() / 32 == rows
    # pair reductions: 2 floats per live corner; the corner-interleaved copy takes 8 per live point
    pb.launch(rates.RED_PAIRS)
    pb.launch(rates.RED_CELLS)
    torch.cuda.synchronize()
    assert pb.grad_dist.double().sum().item() == 2 * rows
    live_points = pb.grad_cells.double().sum().item() / 8
    assert rows / 4 <= live_points <= B * Q * 8 * 32
    # restricting the stream to one level drops the other levels' rows
    pb.grad_value.zero_()
    pb.launch(rates.RED_ROWS, level_mask=1 << 3)
    torch.cuda.synchronize()
    assert 0 < pb.grad_value.double().sum().item() / 32 < rows
    assert not pb.grad_value[:, : 12 * 20 + 6 * 10 + 3 * 5].any()
    for ops in (rates.GATHER_ROWS, rates.GATHER_PAIRS, rates.GATHER_CELLS,
                rates.GATHER_ROWS | rates.GATHER_PAIRS | rates.RED_ROWS | rates.RED_PAIRS):
        assert pb.time_ms(ops, reps=3, warmup=1) > 0
    f = rates.floors(levels, P, D, Q, B, reps=3)
    assert 0 < f["backward_reductions_only_ms"] and 0 < f["forward_ms"] and 0 < f["backward_ms"]
