"""Parity of the remaining per-layer glue kernels (SiTU landing + latent RMSNorm, MLA output gate,
KDA state staging copy, latent cache gather) with the CPU oracle."""
import numpy as np
import pytest

import k3o
from util import bf16_bits, bf16_ulp_diff, normal_bf16, rng, to_dev, to_dev_bf16

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,L,n,h", [(1, 1, 6144, 3584), (5, 5, 6144, 3584), (37, 9, 6144, 3584), (9, 37, 256, 512), (6, 6, 1024, 8192), (0, 7, 64, 3584)])
def test_situ_rms(k3g, dev, B, L, n, h):
    import torch
    g = rng(B * 100 + L + h)
    sp = normal_bf16(g, (max(B, 1), 2 * n), std=3.0)[:B]
    lat = normal_bf16(g, (L, h)); gam = normal_bf16(g, (h,), mean=1.0, std=0.02)
    o_act, o_ln = k3o.situ_rms(np.ascontiguousarray(sp), lat, gam, n, h)
    act = torch.zeros((B, n), dtype=torch.bfloat16, device=dev); ln = torch.zeros((L, h), dtype=torch.bfloat16, device=dev)
    k3g.call("k3g_situ_rms", to_dev_bf16(np.ascontiguousarray(sp), dev) if B else ln, act if B else ln, to_dev_bf16(lat, dev), to_dev_bf16(gam, dev), ln,
             n, B, h, L, k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(ln), o_ln)                    # IEEE-only: bit exact
    if B:
        d = bf16_ulp_diff(bf16_bits(act), o_act)                  # tanh.approx / ex2.approx on the device: bf16 tolerance
        assert d.max() <= 2 and (d > 1).mean() < 1e-3
        a, b = k3o.bf16_to_f32(bf16_bits(act)).astype(np.float64), k3o.bf16_to_f32(o_act).astype(np.float64)
        assert np.all(np.abs(a - b) <= 1.6e-2 * np.abs(b) + 1e-30)


def test_situ_formula_equals_the_reference_form_on_every_bf16_input(k3g, dev):
    """The kernel's SiTU uses fewer instructions than the reference's formula; the two must be the same
    function.  Its domain is only 2^32 (g, u) pairs of bf16 values, so the whole domain is swept, 1024 values
    of g against all 65536 values of u per pass: infinities, NaNs, subnormals and the g < -87 range where the
    sigmoid's reciprocal is subnormal included.  NaN results only have to be NaN in both."""
    import torch
    bits = lambda lo, hi: (torch.arange(lo, hi, dtype=torch.int32, device=dev) << 16 >> 16).to(torch.int16)   # sign-extend 16 bits
    import ctypes
    import os
    so = os.path.join(os.path.dirname(os.path.abspath(__file__)), "native", "libk3g_probe.so")
    if not os.path.exists(so):
        import sys
        sys.path.insert(0, os.path.dirname(so))
        import build_probe
        build_probe.build()
    probe_fn = ctypes.CDLL(so).k3g_test_situ_probe                # test-only probe: both formulas from the library's own header
    probe_fn.restype = ctypes.c_int
    probe_fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]

    def probe(gt, ut, ot, literal):
        assert probe_fn(gt.data_ptr(), ut.data_ptr(), ot.data_ptr(), ut.numel(), literal, k3g.current_stream()) == 0
    u = bits(0, 65536).repeat(1024).view(torch.bfloat16)
    o0 = torch.empty(u.numel(), dtype=torch.bfloat16, device=dev); o1 = torch.empty_like(o0)
    for c in range(64):
        g = bits(c * 1024, (c + 1) * 1024).repeat_interleave(65536).view(torch.bfloat16)
        probe(g, u, o0, 0)
        probe(g, u, o1, 1)
        a, b = o0.view(torch.int16), o1.view(torch.int16)
        bad = (a != b) & ~(torch.isnan(o0) & torch.isnan(o1))
        if bool(bad.any()):
            i = int(torch.nonzero(bad)[0])
            raise AssertionError("g=%#06x u=%#06x kernel=%#06x reference form=%#06x (%d pairs differ in this pass)" % (
                int(g.view(torch.int16)[i]) & 0xffff, int(u.view(torch.int16)[i]) & 0xffff, int(a[i]) & 0xffff, int(b[i]) & 0xffff, int(bad.sum())))


@pytest.mark.parametrize("tokens,heads,hd", [(1, 24, 128), (33, 24, 128), (7, 16, 128), (5, 3, 64)])
def test_sigmoid_mul(k3g, dev, tokens, heads, hd):
    import torch
    g = rng(tokens + heads)
    n = heads * hd
    attn = normal_bf16(g, (tokens, n))
    tstride, hstride = heads * 2 * hd, 2 * hd                      # gate = second half of a per-head [q | gate] pair
    fused = normal_bf16(g, (tokens, heads * 2 * hd), std=2.0)
    gate_view = np.ascontiguousarray(fused.reshape(-1)[hd:])       # view starting at the first gate half
    want = k3o.sigmoid_mul(attn, np.concatenate([gate_view, np.zeros(hd, np.uint16)]), heads, hd, tstride, hstride)
    d_fused = to_dev_bf16(fused, dev)
    out = torch.zeros((tokens, n), dtype=torch.bfloat16, device=dev)
    k3g.call("k3g_sigmoid_mul", out, to_dev_bf16(attn, dev), d_fused.view(-1)[hd:], tokens, heads, hd, tstride, hstride, k3g.current_stream())
    torch.cuda.synchronize()
    d = bf16_ulp_diff(bf16_bits(out), want)
    assert d.max() <= 1 and (d > 0).mean() < 5e-3


@pytest.mark.parametrize("heads", [24, 12, 96])
def test_span_state_roundtrip_and_latent_gather(k3g, dev, heads):
    import torch
    g = rng(3)
    rec_floats = heads * 128 * 128
    line_bytes = rec_floats * 4 + 3 * 3 * heads * 128 * 2
    lines = torch.from_numpy(g.integers(0, 256, 3 * line_bytes, dtype=np.uint8)).to(dev)
    before = lines.clone()
    line_index = torch.tensor([2, 0, 1], dtype=torch.int32, device=dev); span_at = torch.tensor([1], dtype=torch.int32, device=dev)   # row 1 -> line 0
    guard = 4096                                                  # the copy must stop after `heads` heads
    buf = torch.zeros(rec_floats + guard, dtype=torch.float32, device=dev)
    s = k3g.current_stream()
    k3g.call("k3g_span_state", lines, line_index, line_bytes, span_at, buf, 0, heads, s)
    torch.cuda.synchronize()
    assert torch.equal(buf[:rec_floats].view(torch.uint8), before[:rec_floats * 4]) and torch.equal(lines, before)
    assert not buf[rec_floats:].any()
    buf += 1.0
    k3g.call("k3g_span_state", lines, line_index, line_bytes, span_at, buf, 1, heads, s)
    torch.cuda.synchronize()
    assert torch.equal(lines[:rec_floats * 4], buf[:rec_floats].view(torch.uint8)) and torch.equal(lines[rec_floats * 4:], before[rec_floats * 4:])
    assert k3g.raw("k3g_span_state", lines, line_index, rec_floats * 4 - 16, span_at, buf, 0, heads, s) == -2      # the line cannot hold that many heads
    # latent gather: 3 pages of 64 rows in shuffled order, 150 cached rows, 200 output rows
    page_stride = 64 * 576 * 2
    slab = normal_bf16(g, (4 * page_stride,))
    table = np.array([2, 0, 3, 1], np.int32); lens = np.array([150], np.int32)
    out = torch.full((200, 576), 7.0, dtype=torch.bfloat16, device=dev)
    k3g.call("k3g_latent_gather", to_dev_bf16(slab, dev), to_dev(table, dev), page_stride, to_dev(lens, dev), out, 200, s)
    torch.cuda.synchronize()
    want = np.zeros((200, 576), np.uint16)
    for t in range(150):
        o = table[t // 64] * page_stride + (t % 64) * 576
        want[t] = slab[o:o + 576]
    assert np.array_equal(bf16_bits(out), want)


@pytest.mark.parametrize("W,L,h", [(1, 5, 3584), (2, 9, 3584), (4, 13, 3584), (8, 6, 512), (4, 3, 4096)])
def test_reduce_scatter_folded_into_the_latent_norm(k3g, dev, W, L, h):
    """k3g_rs_situ_rms == k3g_rs_pull followed by k3g_situ_rms_amax, bit for bit, for every rank of a world emulated
    on one GPU (data kernels only: nothing waits)."""
    import torch
    g = rng(70 + W + L)
    s = k3g.current_stream()
    B, n = 7, 6144
    sp = to_dev_bf16(normal_bf16(g, (B, 2 * n), std=3.0), dev)
    gam = to_dev_bf16(normal_bf16(g, (h,), mean=1.0, std=0.02), dev)
    parts = [to_dev_bf16(normal_bf16(g, (W * L, h), std=1.0 / W), dev) for _ in range(W)]
    tab = torch.tensor([t.data_ptr() for t in parts], dtype=torch.int64, device=dev)
    items = (B * n + 4095) // 4096
    for rank in range(W):
        own = torch.zeros((L, h), dtype=torch.bfloat16, device=dev)
        k3g.call("k3g_rs_pull", parts[rank], own, tab, L * h, 2 * (W - 1), rank, W, 8, s)
        act0, act1 = torch.zeros((B, n), dtype=torch.bfloat16, device=dev), torch.zeros((B, n), dtype=torch.bfloat16, device=dev)
        ln0, ln1 = torch.zeros((L, h), dtype=torch.bfloat16, device=dev), torch.zeros((L, h), dtype=torch.bfloat16, device=dev)
        m0, m1 = torch.zeros(items, device=dev), torch.zeros(items, device=dev)
        k3g.call("k3g_situ_rms_amax", sp, act0, own, gam, ln0, n, B, h, L, m0, s)
        k3g.call("k3g_rs_situ_rms", sp, act1, parts[rank], tab, rank, W, gam, ln1, n, B, h, L, m1, s)
        torch.cuda.synchronize()
        assert torch.equal(ln0, ln1) and torch.equal(act0, act1) and torch.equal(m0, m1)
