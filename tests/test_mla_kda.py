"""Parity of MLA prep and the KDA conv / output-gate kernels with the CPU oracle."""
import numpy as np
import pytest

import k3o
from util import bf16_bits, bf16_ulp_diff, fp8_code_diff, normal_bf16, rng, to_dev, to_dev_bf16

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("partial_bf16", [True, False])
@pytest.mark.parametrize("B", [1, 5, 1027])
def test_mla_prep_reference_abi(k3g, dev, partial_bf16, B):
    import torch
    g = rng(B + int(partial_bf16))
    inner, fused = 3072, 5184
    partial = normal_bf16(g, (B, fused)) if partial_bf16 else g.standard_normal((B, fused), dtype=np.float32)
    gq = normal_bf16(g, (1536,), mean=1.0, std=0.02); gkv = normal_bf16(g, (512,), mean=1.0, std=0.02)
    pages, page_stride, layer_off = (B + 63) // 64 + 1, 64 * 576 * 3, 64 * 576
    slots = g.permutation(pages * 64)[:B].astype(np.int64)
    slots[::7] = -1                                              # rows without a cache slot
    slab0 = normal_bf16(g, (pages * page_stride,))
    o_slab = slab0.copy()
    o_q = k3o.mla_prep_head(partial, gq, gkv, slots, o_slab, layer_off, page_stride, 1e-5)
    o_gate = k3o.mla_prep_gate(partial, inner)
    d_slab = to_dev_bf16(slab0, dev)
    qn = torch.empty((B, 1536), dtype=torch.bfloat16, device=dev); gate = torch.empty((B, inner), dtype=torch.bfloat16, device=dev)
    d_part = to_dev_bf16(partial, dev) if partial_bf16 else to_dev(partial, dev)
    k3g.call("k3g_mla_prep", d_part, int(partial_bf16), to_dev_bf16(gq, dev), to_dev_bf16(gkv, dev), to_dev(slots, dev), d_slab, layer_off,
             page_stride, qn, gate, B, inner, 1e-5, k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(qn), o_q)
    assert np.array_equal(bf16_bits(d_slab), o_slab)          # appended rows written, everything else untouched
    assert np.array_equal(bf16_bits(gate), o_gate)


def _rope_table(T, theta=50000.0):
    j = np.arange(32, dtype=np.float32)
    inv = (1.0 / np.power(np.float32(theta), (2 * j) / np.float32(64))).astype(np.float32)
    ang = np.arange(T, dtype=np.float32)[:, None] * inv[None, :]
    return k3o.f32_to_bf16(np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32))


@pytest.mark.parametrize("T,heads", [(1, 16), (131, 16), (64, 32), (33, 8), (10, 4)])
def test_mla_prep_rope_pack(k3g, dev, T, heads):
    import torch
    g = rng(T + heads)
    kv = normal_bf16(g, (T, 576)); q = normal_bf16(g, (T, heads, 192))
    gkv = normal_bf16(g, (512,), mean=1.0, std=0.02)
    tab = _rope_table(T)
    k_init = normal_bf16(g, (T, heads, 192))                    # nope slots belong to the up-projection GEMM
    o_q, o_k, o_lat = k3o.mla_prep_rope_pack(kv, q, gkv, tab, 1e-6, k_out_init=k_init)
    q_out = torch.empty((T, heads, 192), dtype=torch.bfloat16, device=dev); k_out = to_dev_bf16(k_init, dev)
    lat = torch.empty((T, 512), dtype=torch.bfloat16, device=dev)
    k3g.call("k3g_mla_prep_rope_pack", to_dev_bf16(kv, dev), to_dev_bf16(q, dev), to_dev_bf16(gkv, dev), to_dev_bf16(tab, dev), q_out, k_out,
             lat, T, heads, 1e-6, k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(lat), o_lat)
    assert np.array_equal(bf16_bits(q_out), o_q)
    assert np.array_equal(bf16_bits(k_out), o_k)
    # position 0 rotates by angle 0: rope slices pass through unchanged
    assert np.array_equal(o_q[0, :, 128:], q[0, :, 128:])


@pytest.mark.parametrize("taps_bf16", [False, True])
@pytest.mark.parametrize("heads,rows,at,span,rpb", [(24, 40, 0, 40, 16), (24, 70, 3, 61, 32), (2, 9, 0, 2, 32), (2, 5, 1, 1, 4), (24, 300, 0, 300, 0),
                                                    (2, 9, 0, 9, 1), (24, 40, 0, 40, 2), (2, 70, 0, 70, 1)])
def test_span_conv_silu(k3g, dev, taps_bf16, heads, rows, at, span, rpb):
    import torch
    g = rng(heads * 1000 + span)
    inner = heads * 128
    stride = 4 * inner
    partial = normal_bf16(g, (rows, stride))
    cw = normal_bf16(g, (3, 4, inner), std=0.5) if taps_bf16 else (g.standard_normal((3, 4, inner), dtype=np.float32) * 0.5).astype(np.float32)
    win = normal_bf16(g, (3, 3, inner))
    wsm = g.standard_normal((rows, 256), dtype=np.float32)
    o_q, o_k, o_v, o_win = k3o.span_conv_silu(partial, stride, cw, win, inner, at, span)
    o_beta, o_flow = k3o.span_beta_flow(wsm, heads, at, span)
    outs = [torch.zeros((span, inner), dtype=torch.bfloat16, device=dev) for _ in range(3)]
    d_win = to_dev_bf16(win, dev)
    beta = torch.zeros((heads, span), dtype=torch.bfloat16, device=dev); flow = torch.zeros((span, 128), dtype=torch.bfloat16, device=dev)
    d_cw = to_dev_bf16(cw, dev) if taps_bf16 else to_dev(cw, dev)
    k3g.call("k3g_span_gather", to_dev_bf16(partial, dev), stride, d_cw, int(taps_bf16), d_win, to_dev(wsm, dev), outs[0], outs[1], outs[2],
             beta, flow, heads, at, span, rpb, k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(d_win), o_win)              # final state = last three inputs, bit exact
    assert np.array_equal(bf16_bits(beta), o_beta) and np.array_equal(bf16_bits(flow), o_flow)
    for got, want in zip(outs, (o_q, o_k, o_v)):
        d = bf16_ulp_diff(bf16_bits(got), want)                 # approximate sigmoid on the device: bf16 tolerance
        assert d.max() <= 1 and (d > 0).mean() < 2e-3
        a, b = k3o.bf16_to_f32(bf16_bits(got)), k3o.bf16_to_f32(want)
        assert np.all(np.abs(a - b) <= 1e-2 * np.abs(b) + 1e-30)


def test_span_conv_zero_state_matches_direct_convolution(k3g, dev):
    """Zero initial window = plain causal conv; checked against a float64 convolution."""
    import torch
    heads, span = 2, 50
    inner = heads * 128
    g = rng(77)
    x = normal_bf16(g, (span, 3 * inner)); cw = normal_bf16(g, (3, 4, inner), std=0.5)
    win = torch.zeros((3, 3, inner), dtype=torch.bfloat16, device=dev)
    outs = [torch.zeros((span, inner), dtype=torch.bfloat16, device=dev) for _ in range(3)]
    k3g.call("k3g_span_gather", to_dev_bf16(x, dev), 3 * inner, to_dev_bf16(cw, dev), 1, win, None, outs[0], outs[1], outs[2], None, None,
             heads, 0, span, 8, k3g.current_stream())
    torch.cuda.synchronize()
    xf = k3o.bf16_to_f32(x).astype(np.float64).reshape(span, 3, inner); wf = k3o.bf16_to_f32(cw).astype(np.float64)
    for s in range(3):
        xp = np.concatenate([np.zeros((3, inner)), xf[:, s]], 0)
        y = sum(xp[t:t + span] * wf[s, t] for t in range(4))
        ref = y / (1 + np.exp(-y))
        got = k3o.bf16_to_f32(bf16_bits(outs[s])).astype(np.float64)
        assert np.all(np.abs(got - ref) <= 2e-2 * np.abs(ref) + 1e-3)
    assert np.array_equal(bf16_bits(win).reshape(3, 3, inner), x.reshape(span, 3, inner)[-3:].transpose(1, 0, 2))


@pytest.mark.parametrize("heads,rows,at,span", [(24, 10, 0, 10), (24, 300, 17, 256), (2, 3, 1, 1), (8, 65, 0, 65)])
def test_kda_out_gate(k3g, dev, heads, rows, at, span):
    import torch
    g = rng(heads + span)
    inner = heads * 128
    attn = normal_bf16(g, (span, inner)); gate = normal_bf16(g, (rows, 4 * inner))
    gamma_o = (1 + 0.1 * g.standard_normal(128, dtype=np.float32)).astype(np.float32)
    o_gated, o_q, o_sf = k3o.kda_out_gate(attn, gate, 4 * inner, 3 * inner, gamma_o, heads, at, span, rows, 1e-6, quant=True)
    gated = torch.zeros((rows, inner), dtype=torch.bfloat16, device=dev)
    q = torch.zeros((rows, inner), dtype=torch.uint8, device=dev); sf = torch.zeros((rows, inner // 32), dtype=torch.uint8, device=dev)
    k3g.call("k3g_kda_out_gate", to_dev_bf16(attn, dev), to_dev_bf16(gate, dev), 4 * inner, 3 * inner, to_dev(gamma_o, dev), gated, q, sf,
             heads, at, span, 1e-6, k3g.current_stream())
    torch.cuda.synchronize()
    gb = bf16_bits(gated)
    d = bf16_ulp_diff(gb, o_gated)
    assert d.max() <= 1 and (d > 0).mean() < 5e-3               # approximate sigmoid: bf16 tolerance
    assert not gb[:at].any() and not gb[at + span:].any()       # rows outside [at, at + span) untouched
    # the MXFP8 epilogue is exact on the kernel's own bf16 row: scales and codes bit for bit
    s_q, s_sf = k3o.moe_quant(gb[at:at + span])
    assert np.array_equal(sf.cpu().numpy()[at:at + span], s_sf)
    assert np.array_equal(q.cpu().numpy()[at:at + span], s_q)
    # and against the all-CPU oracle: scales equal except where a group maximum moved by the 1-ulp sigmoid
    sf_bad = (sf.cpu().numpy()[at:at + span] != o_sf[at:at + span]).mean()
    cd = fp8_code_diff(q.cpu().numpy()[at:at + span], o_q[at:at + span])
    assert sf_bad < 1e-3 and (cd > 1).mean() < 1e-3
    # quant-only and gated-only launches give the same bytes
    q2 = torch.zeros_like(q); sf2 = torch.zeros_like(sf); g2 = torch.zeros_like(gated)
    k3g.call("k3g_kda_out_gate", to_dev_bf16(attn, dev), to_dev_bf16(gate, dev), 4 * inner, 3 * inner, to_dev(gamma_o, dev), None, q2, sf2,
             heads, at, span, 1e-6, k3g.current_stream())
    k3g.call("k3g_kda_out_gate", to_dev_bf16(attn, dev), to_dev_bf16(gate, dev), 4 * inner, 3 * inner, to_dev(gamma_o, dev), g2, None, None,
             heads, at, span, 1e-6, k3g.current_stream())
    torch.cuda.synchronize()
    assert torch.equal(q2, q) and torch.equal(sf2, sf) and torch.equal(g2, gated)
