"""Parity of the FP8 quantisation kernels with the CPU oracle (bit-exact: integer scales,
exact maxima, one IEEE rounding per element)."""
import numpy as np
import pytest

import k3o
from util import normal_bf16, rng, to_dev_bf16

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(1, 32), (1, 3584), (7, 3584), (4096, 3584), (5, 7168), (3, 96), (129, 224)])
def test_moe_quant(k3g, dev, rows, cols):
    import torch
    g = rng(rows * 7 + cols)
    x = normal_bf16(g, (rows, cols), std=3.0)
    x[0, :32] = 0
    if rows > 2:
        x[2] = k3o.f32_to_bf16(np.full(cols, 7.0 * 2.0 ** 9, np.float32))     # amax exactly 7 * 2^k
    o_q, o_sf = k3o.moe_quant(x)
    q = torch.empty((rows, cols), dtype=torch.uint8, device=dev)
    sf = torch.full((rows, cols // 32), 0xAA, dtype=torch.uint8, device=dev)
    k3g.call("k3g_moe_quant", to_dev_bf16(x, dev), q, sf, rows, cols, 0, k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(sf.cpu().numpy(), o_sf)
    assert np.array_equal(q.cpu().numpy(), o_q)


def test_moe_quant_small_grid(k3g, dev):
    """The reference's manifest launches one thread per 32-element group; any grid must work."""
    import torch
    x = normal_bf16(rng(3), (513, 3584))
    o_q, o_sf = k3o.moe_quant(x)
    q = torch.empty((513, 3584), dtype=torch.uint8, device=dev); sf = torch.empty((513, 112), dtype=torch.uint8, device=dev)
    k3g.call("k3g_moe_quant", to_dev_bf16(x, dev), q, sf, 513, 3584, 57, k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(sf.cpu().numpy(), o_sf) and np.array_equal(q.cpu().numpy(), o_q)


@pytest.mark.parametrize("n,grid", [(8, 1), (4099, 3), (7168 * 33, 2048), (7168 * 4096, 2048), (13, 2)])
def test_quant_fp8_tensor(k3g, dev, n, grid):
    import torch
    x = normal_bf16(rng(n), (n,), std=2.0)
    o_y, o_scale = k3o.quant_fp8_tensor(x)
    y = torch.empty(n, dtype=torch.uint8, device=dev)
    scale = torch.zeros(1, dtype=torch.float32, device=dev)
    partials = torch.zeros(grid, dtype=torch.float32, device=dev)
    k3g.call("k3g_quant_fp8_tensor", to_dev_bf16(x, dev), y, scale, partials, n, grid, k3g.current_stream())
    torch.cuda.synchronize()
    assert scale.cpu().numpy()[0] == o_scale[0]
    assert np.array_equal(y.cpu().numpy(), o_y)


def test_quant_fp8_tensor_zero(k3g, dev):
    import torch
    x = torch.zeros(4096, dtype=torch.bfloat16, device=dev)
    y = torch.ones(4096, dtype=torch.uint8, device=dev); scale = torch.zeros(1, device=dev); partials = torch.zeros(4, device=dev)
    k3g.call("k3g_quant_fp8_tensor", x, y, scale, partials, 4096, 4, k3g.current_stream())
    torch.cuda.synchronize()
    assert scale.item() == 1.0 and int(y.max()) == 0
