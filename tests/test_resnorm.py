"""Parity of the residual-stream kernels (C ABI, sm_100a) with the CPU oracle.

Tolerances (from the acceptance statement of the path): UE8M0 scales bit-exact; E4M3 codes at
most 1 code apart on at most 1e-4 of the elements; bf16 outputs within 1e-2 relative.  The
kernels are written to the same accumulation order as the oracle and use the same IEEE-only
exponential in the attention-residual softmax, so these tests assert bit equality.
"""
import numpy as np
import pytest

import k3o
from util import bf16_bits, bf16_ulp_diff, fp8_code_diff, normal_bf16, rng, to_dev, to_dev_bf16

pytestmark = pytest.mark.gpu


def _inputs(seed, B, H):
    g = rng(seed)
    residual = normal_bf16(g, (B, H))
    delta = normal_bf16(g, (B, H))
    gamma = normal_bf16(g, (H,), mean=1.0, std=0.02)
    return residual, delta, gamma


def _run_resnorm(k3g, dev, residual, delta, gamma, eps, want_normed=True, grid_hint=0):
    import torch
    B, H = residual.shape
    out = torch.empty((B, H), dtype=torch.bfloat16, device=dev)
    q = torch.empty((B, H), dtype=torch.uint8, device=dev)
    sf = torch.empty((B, H // 32), dtype=torch.uint8, device=dev)
    normed = torch.empty((B, H), dtype=torch.bfloat16, device=dev) if want_normed else None
    k3g.call("k3g_resnorm_mxfp8", to_dev_bf16(residual, dev), to_dev_bf16(delta, dev), to_dev_bf16(gamma, dev), out, q, sf,
             normed, B, H, eps, grid_hint, k3g.current_stream())
    torch.cuda.synchronize()
    return bf16_bits(out), q.cpu().numpy(), sf.cpu().numpy(), (bf16_bits(normed) if want_normed else None)


@pytest.mark.parametrize("B,H", [(1, 7168), (3, 7168), (255, 7168), (257, 1024), (64, 2048), (33, 4096), (17, 8192)])
def test_resnorm_mxfp8_bit_exact(k3g, dev, B, H):
    residual, delta, gamma = _inputs(100 + B + H, B, H)
    o_out, o_q, o_sf, o_n = k3o.resnorm_mxfp8(residual, delta, gamma, 1e-6)
    g_out, g_q, g_sf, g_n = _run_resnorm(k3g, dev, residual, delta, gamma, 1e-6)
    assert np.array_equal(g_out, o_out)
    assert np.array_equal(g_n, o_n)
    assert np.array_equal(g_sf, o_sf)
    assert np.array_equal(g_q, o_q)


def test_resnorm_mxfp8_persistent_grid_and_no_normed(k3g, dev):
    residual, delta, gamma = _inputs(7, 1000, 7168)
    o_out, o_q, o_sf, _ = k3o.resnorm_mxfp8(residual, delta, gamma, 1e-6, want_normed=False)
    g_out, g_q, g_sf, _ = _run_resnorm(k3g, dev, residual, delta, gamma, 1e-6, want_normed=False, grid_hint=148 * 4)
    assert np.array_equal(g_out, o_out) and np.array_equal(g_sf, o_sf) and np.array_equal(g_q, o_q)


def test_resnorm_mxfp8_edge_values(k3g, dev):
    """Zero rows (amax 0 -> scale byte 127), huge and tiny magnitudes, exact 7 * 2^k group maxima."""
    B, H = 8, 7168
    residual, delta, gamma = _inputs(9, B, H)
    residual[0] = 0; delta[0] = 0
    residual[1] = k3o.f32_to_bf16(np.full(H, 3.0e38, np.float32)); delta[1] = 0
    residual[2] = k3o.f32_to_bf16(np.full(H, 1.0e-38, np.float32)); delta[2] = 0
    residual[3, ::2] = 0x8000   # negative zeros
    gamma_one = k3o.f32_to_bf16(np.ones(H, np.float32))
    for gm in (gamma, gamma_one):
        o = k3o.resnorm_mxfp8(residual, delta, gm, 1e-6)
        g = _run_resnorm(k3g, dev, residual, delta, gm, 1e-6)
        for a, b in zip(g, o):
            assert np.array_equal(a, b)
    assert (o[2][0] == 127).all()      # all-zero row: exponent 0


def test_resnorm_roundtrip_property_full_width(k3g, dev):
    """Size-independent property at the benchmark row count: dequantised codes reproduce the
    normed row within the E4M3 half-ulp (2^-4 relative of the group maximum)."""
    import torch
    B, H = 16384, 7168
    g = torch.Generator(device=dev); g.manual_seed(5)
    residual = torch.randn((B, H), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    delta = torch.randn((B, H), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    gamma = (1 + 0.02 * torch.randn((H,), generator=g, device=dev)).to(torch.bfloat16)
    out = torch.empty_like(residual); normed = torch.empty_like(residual)
    q = torch.empty((B, H), dtype=torch.uint8, device=dev); sf = torch.empty((B, H // 32), dtype=torch.uint8, device=dev)
    k3g.call("k3g_resnorm_mxfp8", residual, delta, gamma, out, q, sf, normed, B, H, 1e-6, 0, k3g.current_stream())
    torch.cuda.synchronize()
    assert torch.equal(out, (residual.float() + delta.float()).to(torch.bfloat16))
    deq = q.view(torch.float8_e4m3fn).float().view(B, H // 32, 32) * torch.exp2(sf.float() - 127).unsqueeze(-1)
    n = normed.float().view(B, H // 32, 32)
    amax = n.abs().amax(dim=-1, keepdim=True)
    assert ((deq - n).abs() <= amax * 2.0 ** -4 + 1e-30).all()
    # scale property: 448 * 2^e >= amax > 448 * 2^(e-1)
    e = sf.float().view(B, H // 32, 1) - 127
    assert (amax <= 448 * torch.exp2(e)).all() and (amax > 448 * torch.exp2(e - 1)).all()
    # the row check against the oracle on a seeded sample of rows
    rows = np.array([0, 1, 4095, 8191, 12345, 16383])
    o_out, o_q, o_sf, o_n = k3o.resnorm_mxfp8(bf16_bits(residual[rows]), bf16_bits(delta[rows]), bf16_bits(gamma), 1e-6)
    assert np.array_equal(bf16_bits(normed[rows]), o_n) and np.array_equal(sf[rows].cpu().numpy(), o_sf)
    assert np.array_equal(q[rows].cpu().numpy(), o_q)


@pytest.mark.parametrize("land_bf16", [True, False])
@pytest.mark.parametrize("nb,snapshot", [(0, 0), (0, 1), (1, 0), (3, 1), (8, 0)])
def test_land_add_attnres_rms(k3g, dev, land_bf16, nb, snapshot):
    import torch
    B, H = 67, 7168
    g = rng(200 + nb)
    partial = normal_bf16(g, (B, H)) if land_bf16 else g.standard_normal((B, H), dtype=np.float32)
    prefix = normal_bf16(g, (B, H))
    blocks = normal_bf16(g, (B, 8, H))
    sw = (g.standard_normal(H, dtype=np.float32) * 0.05).astype(np.float32)
    gamma = normal_bf16(g, (H,), mean=1.0, std=0.02)
    o_p2, o_n = k3o.land_add_attnres_rms(partial, prefix, blocks, sw, gamma, nb, snapshot, 1e-5)
    d_part = to_dev_bf16(partial, dev) if land_bf16 else to_dev(partial, dev)
    p2 = torch.empty((B, H), dtype=torch.bfloat16, device=dev); n = torch.empty_like(p2)
    k3g.call("k3g_land_add_attnres_rms", d_part, int(land_bf16), to_dev_bf16(prefix, dev), to_dev_bf16(blocks, dev),
             to_dev(sw, dev), to_dev_bf16(gamma, dev), p2, n, nb, snapshot, B, H, 1e-5, k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(p2), o_p2)
    assert np.array_equal(bf16_bits(n), o_n)     # the softmax uses the IEEE-only exp on both sides


@pytest.mark.parametrize("nb,snapshot", [(0, 1), (2, 1), (8, 1), (5, 0)])
def test_attnres_rms(k3g, dev, nb, snapshot):
    import torch
    B, H = 41, 7168
    g = rng(300 + nb)
    prefix = normal_bf16(g, (B, H))
    blocks = normal_bf16(g, (B, 8, H))
    sw = (g.standard_normal(H, dtype=np.float32) * 0.05).astype(np.float32)
    gamma = normal_bf16(g, (H,), mean=1.0, std=0.02)
    o_blocks = blocks.copy()
    o_n = k3o.attnres_rms(prefix, o_blocks, sw, gamma, nb, snapshot, 1e-5)
    d_blocks = to_dev_bf16(blocks, dev)
    n = torch.empty((B, H), dtype=torch.bfloat16, device=dev)
    k3g.call("k3g_attnres_rms", to_dev_bf16(prefix, dev), d_blocks, to_dev(sw, dev), to_dev_bf16(gamma, dev), n, nb, snapshot,
             B, H, 1e-5, k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(d_blocks), o_blocks)     # snapshot row stored (or untouched when nb == 8)
    assert bf16_ulp_diff(bf16_bits(n), o_n).max() == 0


@pytest.mark.parametrize("land_bf16", [True, False])
@pytest.mark.parametrize("two", [0, 1])
def test_land_add2(k3g, dev, land_bf16, two):
    import torch
    B, H = 129, 7168
    g = rng(400 + two)
    mk = (lambda: normal_bf16(g, (B, H))) if land_bf16 else (lambda: g.standard_normal((B, H), dtype=np.float32))
    p1, p2 = mk(), mk()
    prefix2 = normal_bf16(g, (B, H))
    o = k3o.land_add2(p1, p2, prefix2, two)
    up = (lambda a: to_dev_bf16(a, dev)) if land_bf16 else (lambda a: to_dev(a, dev))
    hidden = torch.empty((B, H), dtype=torch.bfloat16, device=dev)
    k3g.call("k3g_land_add2", up(p1), up(p2) if two else None, int(land_bf16), to_dev_bf16(prefix2, dev), hidden, two, B, H,
             k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(hidden), o)


def test_argument_errors(k3g, dev):
    import torch
    x = torch.zeros((4, 7168), dtype=torch.bfloat16, device=dev)
    q = torch.zeros((4, 7168), dtype=torch.uint8, device=dev); sf = torch.zeros((4, 224), dtype=torch.uint8, device=dev)
    s = k3g.current_stream()
    assert k3g.raw("k3g_resnorm_mxfp8", None, x, x[0], x, q, sf, None, 4, 7168, 1e-6, 0, s) == -1
    assert k3g.raw("k3g_resnorm_mxfp8", x, x, x[0], x, q, sf, None, 4, 7000, 1e-6, 0, s) == -2
    assert k3g.raw("k3g_resnorm_mxfp8", x.view(-1)[1:], x, x[0], x, q, sf, None, 3, 7168, 1e-6, 0, s) == -3
    assert k3g.raw("k3g_resnorm_mxfp8", x, x, x[0], x, q, sf, None, 0, 7168, 1e-6, 0, s) == 0      # empty input
    assert k3g.raw("k3g_attnres_rms", x, None, None, x[0], x, 9, 0, 4, 7168, 1e-5, s) == -4
