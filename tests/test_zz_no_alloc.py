"""The workspace-free per-tensor quantisation entry point (k3g_quant_fp8_tensor_noalloc).

It exists for hosts that cannot allocate or pass scratch memory at call time; its block maxima
live in a static device array inside the library.  Checked here through the C ABI against two
independent answers: the regular entry point (which takes a caller workspace) and the CPU oracle's
per-tensor quantiser -- identical bytes and an identical scale, on calls made back to back whose
inputs differ in size and magnitude, so a slot left over from one call would show up in the next.
Collected last on purpose: a failure here cannot hide another test's result.
"""
import numpy as np
import pytest

import k3o
from util import normal_bf16, rng, to_dev_bf16

pytestmark = pytest.mark.gpu


def _both(k3g, dev, x, grid, want_scale=True):
    import torch
    n = x.size
    dx = to_dev_bf16(x, dev)
    s = k3g.current_stream()
    y_ref = torch.empty(n, dtype=torch.uint8, device=dev); sc_ref = torch.zeros(1, device=dev)
    partials = torch.zeros(grid, dtype=torch.float32, device=dev)
    k3g.call("k3g_quant_fp8_tensor", dx, y_ref, sc_ref if want_scale else None, partials, n, grid, s)
    y = torch.full((n,), 0x55, dtype=torch.uint8, device=dev); sc = torch.zeros(1, device=dev)
    k3g.call("k3g_quant_fp8_tensor_noalloc", dx, y, sc if want_scale else None, n, grid, s)
    torch.cuda.synchronize()
    return y.cpu().numpy(), sc.item(), y_ref.cpu().numpy(), sc_ref.item()


def test_noalloc_matches_workspace_entry_point_and_oracle_twice_in_a_row(k3g, dev):
    big = normal_bf16(rng(1), (7168 * 300 + 5,), std=40.0)        # first call: large values, wide grid
    small = normal_bf16(rng(2), (7168 * 17,), std=0.01)           # second call: tiny values, narrow grid
    for x, grid in ((big, 2048), (small, 96)):
        y, sc, y_ref, sc_ref = _both(k3g, dev, x, grid)
        o_y, o_sc = k3o.quant_fp8_tensor(x)                       # the CPU oracle, independent of either CUDA entry
        assert sc == sc_ref and sc > 0 and np.float32(sc) == o_sc[0]
        assert np.array_equal(y, y_ref) and np.array_equal(y, o_y)
    assert abs(float(sc) * 448 - 0.01 * 5) < 0.05                 # the second scale reflects the small tensor only


@pytest.mark.parametrize("n", [1, 7, 8 * 4096 + 3, 7168 * 9 + 6])
@pytest.mark.parametrize("grid", [1, 2048])
def test_noalloc_ragged_sizes_at_both_grid_extremes(k3g, dev, n, grid):
    """A length that is not a multiple of eight (the scalar tail) with one block and with the full 2048: bytes equal
    to the workspace entry point's and to the oracle's; then the same call without a scale output."""
    x = normal_bf16(rng(n + grid), (n,), std=3.0)
    o_y, o_sc = k3o.quant_fp8_tensor(x)
    y, sc, y_ref, sc_ref = _both(k3g, dev, x, grid)
    assert np.float32(sc) == o_sc[0] and sc == sc_ref
    assert np.array_equal(y, o_y) and np.array_equal(y_ref, o_y)
    y2, _, y2_ref, _ = _both(k3g, dev, x, grid, want_scale=False)
    assert np.array_equal(y2, o_y) and np.array_equal(y2_ref, o_y)


def test_noalloc_rejects_grids_beyond_its_static_workspace(k3g, dev):
    import torch
    x = torch.zeros(4096, dtype=torch.bfloat16, device=dev); y = torch.zeros(4096, dtype=torch.uint8, device=dev)
    assert k3g.raw("k3g_quant_fp8_tensor_noalloc", x, y, None, 4096, 2049, k3g.current_stream()) == -5
    assert k3g.raw("k3g_quant_fp8_tensor_noalloc", x, y, None, 4096, 2048, k3g.current_stream()) == 0
    torch.cuda.synchronize()
    assert int(y.max()) == 0
