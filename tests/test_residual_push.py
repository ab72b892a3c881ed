"""The residual kernels the reference's default program actually runs: landing add + mix + RMSNorm
with the normed row pushed to every rank (kern_k3_attnres_rms_push) and the per-candidate-count
residual kernel that consumes the statistics it hands over (kern_k3_land_add_attnres_rms_nbK)."""
import numpy as np
import pytest

import k3o
from util import bf16_bits, normal_bf16, rng, to_dev, to_dev_bf16


def _case(seed, B, H=7168):
    g = rng(seed)
    d = dict(blocks=normal_bf16(g, (B, 8, H)), sw=(g.standard_normal(H, dtype=np.float32) * 0.05).astype(np.float32),
             sw_mlp=(g.standard_normal(H, dtype=np.float32) * 0.05).astype(np.float32), gamma=normal_bf16(g, (H,), mean=1.0, std=0.02),
             p1=normal_bf16(g, (B, H), std=0.5), p2=normal_bf16(g, (B, H), std=0.5), prefix2=normal_bf16(g, (B, H)),
             partial=normal_bf16(g, (B, H), std=0.5))
    return d


@pytest.mark.parametrize("nb,nb_stats", [(1, 1), (4, 4), (4, 2), (8, 8), (3, 0)])
def test_oracle_stats_handoff_is_bit_neutral(nb, nb_stats):
    """CPU: statistics written by the push kernel equal what the consumer would recompute, so the
    consumer's output does not depend on how many candidates the hand-off covers."""
    d = _case(nb, 5)
    blocks = d["blocks"].copy()
    hidden, _, stats = k3o.attnres_rms_push(blocks, d["sw"], d["gamma"], nb, 0, d["sw_mlp"], d["p1"], d["p2"], d["prefix2"], 1, 1e-5)
    plain = k3o.land_add_attnres_rms(d["partial"], hidden, blocks, d["sw_mlp"], d["gamma"], nb, 0, 1e-5)
    fed = k3o.land_add_attnres_rms_stats(d["partial"], hidden, blocks, d["sw_mlp"], d["gamma"], nb, 0, 1e-5, stats, nb_stats)
    assert np.array_equal(plain[0], fed[0]) and np.array_equal(plain[1], fed[1])
    assert np.array_equal(hidden, k3o.land_add2(d["p1"], d["p2"], d["prefix2"], 1))     # the folded K1c


@pytest.mark.gpu
@pytest.mark.parametrize("W,nb,snapshot,two", [(1, 0, 1, 0), (2, 1, 0, 1), (4, 4, 1, 1), (4, 8, 1, 1), (8, 3, 0, 0)])
def test_attnres_rms_push_emulated_ranks(k3g, dev, W, nb, snapshot, two):
    import torch
    B, H = 13, 7168
    cases = [_case(100 * W + r, B) for r in range(W)]
    normed_all = [torch.zeros((W * B, H), dtype=torch.bfloat16, device=dev) for _ in range(W)]
    tab = torch.tensor([t.data_ptr() for t in normed_all], dtype=torch.int64, device=dev)
    want_rows = []
    for r, d in enumerate(cases):
        o_blocks = d["blocks"].copy()
        o_hidden, o_normed, o_stats = k3o.attnres_rms_push(o_blocks, d["sw"], d["gamma"], nb, snapshot, d["sw_mlp"], d["p1"], d["p2"], d["prefix2"],
                                                           two, 1e-5)
        want_rows.append(o_normed)
        blocks = to_dev_bf16(d["blocks"], dev)
        hidden = torch.zeros((B, H), dtype=torch.bfloat16, device=dev)
        stats = torch.zeros((B, 8, 2), dtype=torch.float32, device=dev)
        k3g.call("k3g_attnres_rms_push", blocks, to_dev(d["sw"], dev), to_dev_bf16(d["gamma"], dev), normed_all[r], tab, nb, snapshot, B, r, W,
                 to_dev(d["sw_mlp"], dev), stats, to_dev_bf16(d["p1"], dev), to_dev_bf16(d["p2"], dev) if two else None,
                 to_dev_bf16(d["prefix2"], dev), hidden, two, H, 1e-5, k3g.current_stream())
        torch.cuda.synchronize()
        assert np.array_equal(bf16_bits(hidden), o_hidden)
        assert np.array_equal(bf16_bits(blocks), o_blocks)
        assert np.array_equal(stats.cpu().numpy().view(np.uint32), o_stats.view(np.uint32))
        # the consumer fed with the device statistics == the consumer that recomputes them
        pre = to_dev_bf16(o_hidden, dev)
        out = [torch.zeros((B, H), dtype=torch.bfloat16, device=dev) for _ in range(4)]
        if nb > 0:
            k3g.call("k3g_land_add_attnres_rms_stats", to_dev_bf16(d["partial"], dev), 1, pre, blocks, to_dev(d["sw_mlp"], dev),
                     to_dev_bf16(d["gamma"], dev), out[0], out[1], nb, 0, B, H, 1e-5, stats, nb, k3g.current_stream())
            k3g.call("k3g_land_add_attnres_rms", to_dev_bf16(d["partial"], dev), 1, pre, blocks, to_dev(d["sw_mlp"], dev),
                     to_dev_bf16(d["gamma"], dev), out[2], out[3], nb, 0, B, H, 1e-5, k3g.current_stream())
            torch.cuda.synchronize()
            assert torch.equal(out[0], out[2]) and torch.equal(out[1], out[3])
            o_p2, o_n = k3o.land_add_attnres_rms(d["partial"], o_hidden, o_blocks, d["sw_mlp"], d["gamma"], nb, 0, 1e-5)
            assert np.array_equal(bf16_bits(out[1]), o_n)
    want = np.concatenate(want_rows)
    for r in range(W):
        assert np.array_equal(bf16_bits(normed_all[r]), want)     # every rank holds the full gathered matrix


def _rowmax(bits):
    """max |x| per row of a bf16 bit array, as f32 (the bit-pattern maximum the amax pass takes)."""
    m = (bits & 0x7fff).max(axis=-1).astype(np.uint32)
    return (m << 16).view(np.float32)


@pytest.mark.gpu
@pytest.mark.parametrize("W", [1, 4])
def test_producer_side_amax_equals_two_pass_quantisation(k3g, dev, W):
    """Row maxima left by the producers (push kernel: gathered over the emulated ranks; per-count residual kernel;
    SiTU items) fed to the apply launch give exactly the bytes and scale of the two-pass per-tensor quantisation."""
    import torch
    B, H, nb = 9, 7168, 3
    s = k3g.current_stream()
    cases = [_case(500 + 10 * W + r, B) for r in range(W)]
    normed_all = [torch.zeros((W * B, H), dtype=torch.bfloat16, device=dev) for _ in range(W)]
    rowmax_all = [torch.full((W * B,), -1.0, dtype=torch.float32, device=dev) for _ in range(W)]
    tab = torch.tensor([t.data_ptr() for t in normed_all], dtype=torch.int64, device=dev)
    mtab = torch.tensor([t.data_ptr() for t in rowmax_all], dtype=torch.int64, device=dev)
    for r, d in enumerate(cases):
        blocks = to_dev_bf16(d["blocks"], dev)
        hidden = torch.zeros((B, H), dtype=torch.bfloat16, device=dev); stats = torch.zeros((B, 8, 2), dtype=torch.float32, device=dev)
        k3g.call("k3g_attnres_rms_push_amax", blocks, to_dev(d["sw"], dev), to_dev_bf16(d["gamma"], dev), normed_all[r], tab, nb, 1, B, r, W,
                 to_dev(d["sw_mlp"], dev), stats, to_dev_bf16(d["p1"], dev), to_dev_bf16(d["p2"], dev), to_dev_bf16(d["prefix2"], dev), hidden, 1,
                 H, 1e-5, rowmax_all[r], mtab, s)
        # consumer of the same layer: per-count residual kernel with its own row maxima
        p2o, nrm = torch.zeros((B, H), dtype=torch.bfloat16, device=dev), torch.zeros((B, H), dtype=torch.bfloat16, device=dev)
        rowmax = torch.full((B,), -1.0, dtype=torch.float32, device=dev)
        k3g.call("k3g_land_add_attnres_rms_stats_amax", to_dev_bf16(d["partial"], dev), 1, hidden, blocks, to_dev(d["sw_mlp"], dev),
                 to_dev_bf16(d["gamma"], dev), p2o, nrm, nb + 1, 0, B, H, 1e-5, stats, nb, rowmax, s)
        torch.cuda.synchronize()
        assert np.array_equal(rowmax.cpu().numpy(), _rowmax(bf16_bits(nrm)))
        n = B * H
        y0, y1 = torch.zeros(n, dtype=torch.uint8, device=dev), torch.zeros(n, dtype=torch.uint8, device=dev)
        sc0, sc1, part = torch.zeros(1, device=dev), torch.zeros(1, device=dev), torch.zeros(64, device=dev)
        k3g.call("k3g_quant_fp8_tensor", nrm, y0, sc0, part, n, 64, s)
        k3g.call("k3g_quant_fp8_apply", nrm, y1, sc1, rowmax, B, n, 64, s)
        torch.cuda.synchronize()
        assert torch.equal(y0, y1) and torch.equal(sc0, sc1)
    for r in range(W):
        assert torch.equal(normed_all[r], normed_all[0]) and torch.equal(rowmax_all[r], rowmax_all[0])
    assert np.array_equal(rowmax_all[0].cpu().numpy(), _rowmax(bf16_bits(normed_all[0])))
    n = W * B * H
    y0, y1 = torch.zeros(n, dtype=torch.uint8, device=dev), torch.zeros(n, dtype=torch.uint8, device=dev)
    sc0, sc1, part = torch.zeros(1, device=dev), torch.zeros(1, device=dev), torch.zeros(2048, device=dev)
    k3g.call("k3g_quant_fp8_tensor", normed_all[0], y0, sc0, part, n, 2048, s)
    k3g.call("k3g_quant_fp8_apply", normed_all[0], y1, sc1, rowmax_all[0], W * B, n, 2048, s)
    torch.cuda.synchronize()
    assert torch.equal(y0, y1) and torch.equal(sc0, sc1)


@pytest.mark.gpu
@pytest.mark.parametrize("B,n", [(7, 6144), (3, 1000 * 8), (1, 64)])
def test_situ_item_maxima(k3g, dev, B, n):
    import torch
    g = rng(B + n)
    s = k3g.current_stream()
    sp = to_dev_bf16(normal_bf16(g, (B, 2 * n), std=3.0), dev)
    h = 3584
    lat, gam = to_dev_bf16(normal_bf16(g, (B, h)), dev), to_dev_bf16(normal_bf16(g, (h,), mean=1.0, std=0.02), dev)
    act0, act1 = torch.zeros((B, n), dtype=torch.bfloat16, device=dev), torch.zeros((B, n), dtype=torch.bfloat16, device=dev)
    ln0, ln1 = torch.zeros((B, h), dtype=torch.bfloat16, device=dev), torch.zeros((B, h), dtype=torch.bfloat16, device=dev)
    items = (B * n + 4095) // 4096
    imax = torch.full((items,), -1.0, dtype=torch.float32, device=dev)
    k3g.call("k3g_situ_rms", sp, act0, lat, gam, ln0, n, B, h, B, s)
    k3g.call("k3g_situ_rms_amax", sp, act1, lat, gam, ln1, n, B, h, B, imax, s)
    torch.cuda.synchronize()
    assert torch.equal(act0, act1) and torch.equal(ln0, ln1)
    flat = np.concatenate([bf16_bits(act1).reshape(-1), np.zeros(items * 4096 - B * n, np.uint16)]).reshape(items, 4096)
    assert np.array_equal(imax.cpu().numpy(), _rowmax(flat))
    y0, y1 = torch.zeros(B * n, dtype=torch.uint8, device=dev), torch.zeros(B * n, dtype=torch.uint8, device=dev)
    sc0, sc1, part = torch.zeros(1, device=dev), torch.zeros(1, device=dev), torch.zeros(32, device=dev)
    k3g.call("k3g_quant_fp8_tensor", act1, y0, sc0, part, B * n, 32, s)
    k3g.call("k3g_quant_fp8_apply", act1, y1, sc1, imax, items, B * n, 32, s)
    torch.cuda.synchronize()
    assert torch.equal(y0, y1) and torch.equal(sc0, sc1)


@pytest.mark.gpu
@pytest.mark.parametrize("W,nb,snapshot", [(1, 0, 0), (2, 3, 0), (4, 4, 0), (4, 2, 1), (8, 8, 0)])
def test_reduce_scatter_folded_into_the_residual_kernel(k3g, dev, W, nb, snapshot):
    """k3g_rs_land_add_attnres_rms == k3g_rs_pull followed by k3g_land_add_attnres_rms_stats_amax, bit for bit, for
    every rank of a world emulated on one GPU (data kernels only: nothing waits), and == the oracle chain."""
    import torch
    B, H = 11, 7168
    g = rng(900 + W + nb)
    s = k3g.current_stream()
    parts = [normal_bf16(g, (W * B, H), std=0.5 / W) for _ in range(W)]
    d_parts = [to_dev_bf16(p, dev) for p in parts]
    tab = torch.tensor([t.data_ptr() for t in d_parts], dtype=torch.int64, device=dev)
    for rank in range(W):
        d = _case(1000 + rank, B)
        blocks, prefix = to_dev_bf16(d["blocks"], dev), to_dev_bf16(d["prefix2"], dev)
        sw, gamma = to_dev(d["sw_mlp"], dev), to_dev_bf16(d["gamma"], dev)
        # statistics as the push kernel of the same layer would have left them
        o_blocks = d["blocks"].copy()
        _, _, o_stats = k3o.attnres_rms_push(o_blocks, d["sw"], d["gamma"], nb, 0, d["sw_mlp"], d["p1"], d["p2"], d["prefix2"], 1, 1e-5)
        stats = to_dev(o_stats, dev)
        own = torch.zeros((B, H), dtype=torch.bfloat16, device=dev)
        k3g.call("k3g_rs_pull", d_parts[rank], own, tab, B * H, 2 * (W - 1), rank, W, 8, s)
        a = [torch.zeros((B, H), dtype=torch.bfloat16, device=dev) for _ in range(4)]
        m0, m1 = torch.zeros(B, device=dev), torch.zeros(B, device=dev)
        k3g.call("k3g_land_add_attnres_rms_stats_amax", own, 1, prefix, blocks, sw, gamma, a[0], a[1], nb, snapshot, B, H, 1e-5, stats, nb, m0, s)
        k3g.call("k3g_rs_land_add_attnres_rms", d_parts[rank], tab, rank, W, prefix, blocks, sw, gamma, a[2], a[3], nb, snapshot, B, H, 1e-5,
                 stats, nb, m1, s)
        torch.cuda.synchronize()
        assert torch.equal(a[0], a[2]) and torch.equal(a[1], a[3]) and torch.equal(m0, m1)
        o_own = k3o.rs_pull(parts, rank, 2 * (W - 1))
        o_p2, o_n = k3o.land_add_attnres_rms(o_own.reshape(B, H), d["prefix2"], d["blocks"], d["sw_mlp"], d["gamma"], nb, snapshot, 1e-5)
        assert np.array_equal(bf16_bits(a[2]), o_p2) and np.array_equal(bf16_bits(a[3]), o_n)
