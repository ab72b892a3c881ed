"""Parity of the once-per-prefill helpers (row copies, embedding, zero fill, length record, argmax), the f32
landings (SiTU on an f32 partial, band landing, stand-alone latent RMSNorm) and the first layer's push form
with the CPU oracle."""
import numpy as np
import pytest

import k3o
from util import bf16_bits, bf16_ulp_diff, normal_bf16, rng, to_dev, to_dev_bf16

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,n", [(1, 33792), (5, 1024), (3, 1028), (7, 250), (0, 64)])
def test_land_situ(k3g, dev, B, n):
    import torch
    g = rng(B * 7 + n)
    p = (g.standard_normal((B, 2 * n), dtype=np.float32) * 3.0).astype(np.float32)
    want = k3o.land_situ(p, n)
    act = torch.zeros((max(B, 1), n), dtype=torch.bfloat16, device=dev)
    k3g.call("k3g_land_situ", to_dev(p, dev) if B else act, act, n, B, k3g.current_stream())
    torch.cuda.synchronize()
    if B:
        d = bf16_ulp_diff(bf16_bits(act), want)                # tanh.approx / ex2.approx on the device: bf16 tolerance
        assert d.max() <= 2 and (d > 1).mean() < 1e-3


@pytest.mark.parametrize("B,n,off,ldc", [(4, 1024, 2048, 4096), (3, 250, 3, 301), (2, 64, 0, 64)])
def test_land_band(k3g, dev, B, n, off, ldc):
    import torch
    g = rng(B + n + off)
    p = g.standard_normal((B, ldc), dtype=np.float32)
    o = torch.zeros((B, n), dtype=torch.bfloat16, device=dev)
    k3g.call("k3g_land", to_dev(p, dev), o, n, off, ldc, B, k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(o), k3o.land(p, n, off, ldc))


@pytest.mark.parametrize("B,h", [(1, 3584), (9, 3584), (4, 512), (3, 8192), (5, 4104)])
def test_rms(k3g, dev, B, h):
    import torch
    g = rng(B * 3 + h)
    x = normal_bf16(g, (B, h), std=2.0); gam = normal_bf16(g, (h,), mean=1.0, std=0.02)
    o = torch.zeros((B, h), dtype=torch.bfloat16, device=dev)
    k3g.call("k3g_rms", to_dev_bf16(x, dev), to_dev_bf16(gam, dev), o, h, B, k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(o), k3o.rms(x, gam))          # IEEE-only: bit exact


def test_row_copies_and_zero_fill(k3g, dev):
    import torch
    g = rng(11)
    s = k3g.current_stream()
    for row_bytes in (14336, 48, 10):                              # vector path, small vector path, byte path
        rows, own = 11, 4
        src = g.integers(0, 256, (rows, row_bytes), dtype=np.uint8)
        d_src = to_dev(src, dev)
        for rank in range(4):                                      # rank 2 and 3 run past the end: last row repeated
            dst = torch.zeros((own, row_bytes), dtype=torch.uint8, device=dev)
            k3g.call("k3g_rank_rows", dst, d_src, rank, own, row_bytes, rows, s)
            torch.cuda.synchronize()
            assert np.array_equal(dst.cpu().numpy(), k3o.rank_rows(src, rank, own))
        plan = np.array([0, 3, 9, 10], np.int32)
        for rank in range(4):
            dst = torch.zeros((own, row_bytes), dtype=torch.uint8, device=dev)
            k3g.call("k3g_own_rows", dst, d_src, to_dev(plan, dev), rank, own, row_bytes, rows, s)
            torch.cuda.synchronize()
            assert np.array_equal(dst.cpu().numpy(), k3o.own_rows(src, plan, rank, own))
        for lo, hi in ((3, 9), (0, rows), (5, 5), (7, 2)):
            buf = d_src.clone()
            k3g.call("k3g_zero_rows", buf, row_bytes, lo, hi, s)
            torch.cuda.synchronize()
            assert np.array_equal(buf.cpu().numpy(), k3o.zero_rows(src, lo, hi))


def test_embedding_copy_rows_last_row_lens(k3g, dev):
    import torch
    g = rng(12)
    s = k3g.current_stream()
    for hidden in (7168, 100, 7):
        table = normal_bf16(g, (50, hidden))
        ids = g.integers(0, 50, 33).astype(np.int64)
        out = torch.zeros((33, hidden), dtype=torch.bfloat16, device=dev)
        k3g.call("k3g_embedding", to_dev(ids, dev), to_dev_bf16(table, dev), out, 33, hidden, s)
        torch.cuda.synchronize()
        assert np.array_equal(bf16_bits(out), k3o.embedding(ids, table))
        last = torch.zeros(hidden, dtype=torch.bfloat16, device=dev)
        k3g.call("k3g_last_row", last, to_dev_bf16(table, dev), hidden, hidden, 50, s)
        torch.cuda.synchronize()
        assert np.array_equal(bf16_bits(last), table[49])
    src = normal_bf16(g, (9, 4 * 768))
    dst = torch.zeros((9, 768), dtype=torch.bfloat16, device=dev)
    k3g.call("k3g_copy_rows", dst, to_dev_bf16(src, dev).view(-1)[2 * 768:], 768, 4 * 768, 768, 8, s)       # band 2 of a fused row
    torch.cuda.synchronize()
    want = np.zeros((9, 768), np.uint16); want[:8] = src[:8, 2 * 768:3 * 768]
    assert np.array_equal(bf16_bits(dst), want)
    lens = torch.full((8,), -1, dtype=torch.int32, device=dev)
    k3g.call("k3g_fmha_lens", to_dev(np.array([12345, 7], np.int32), dev), lens, 4096, s)
    torch.cuda.synchronize()
    assert np.array_equal(lens.cpu().numpy(), k3o.fmha_lens([12345], 4096))


@pytest.mark.parametrize("B,n,parts", [(1, 163840, 64), (3, 1000, 64), (2, 4096, 7), (4, 37, 64), (2, 8, 1)])
def test_argmax(k3g, dev, B, n, parts):
    import torch
    g = rng(n + parts)
    x = g.standard_normal((B, n), dtype=np.float32)
    x[0, n // 3] = x[0].max() + 1.0
    x[0, n - 1] = x[0, n // 3]                                   # tie: the smaller index wins
    if B > 1:
        x[1, :] = -np.inf
        x[1, n // 2:] = -3.0e38
    if B > 2:
        x[2, 5 % n] = np.inf
    pmax = torch.zeros((B, parts), dtype=torch.float32, device=dev); pidx = torch.zeros((B, parts), dtype=torch.int32, device=dev)
    out = torch.full((B,), -1, dtype=torch.int64, device=dev)
    k3g.call("k3g_argmax_f32", to_dev(x, dev), pmax, pidx, out, B, n, parts, k3g.current_stream())
    torch.cuda.synchronize()
    want = k3o.argmax_f32(x)
    assert np.array_equal(out.cpu().numpy(), want)
    assert want[0] == n // 3


@pytest.mark.parametrize("nb,snapshot", [(0, 1), (3, 1), (2, 0)])
def test_push_first_layer_form(k3g, dev, nb, snapshot):
    """p1 == NULL: the row is the prefix itself (op attnres_rms_push_first_v3) -- K1a with the normed row stored into
    this rank's slice of every rank's gathered buffer (the peers' copies emulated on one GPU)."""
    import torch
    g = rng(40 + nb)
    B, H, W, rank = 5, 7168, 4, 2
    prefix = normal_bf16(g, (B, H)); blocks = normal_bf16(g, (B, 8, H))
    sw = (g.standard_normal(H, dtype=np.float32) * 0.05).astype(np.float32); gamma = normal_bf16(g, (H,), mean=1.0, std=0.02)
    want_blocks = blocks.copy()
    want = k3o.attnres_rms(prefix, want_blocks, sw, gamma, nb, snapshot, 1e-5)
    copies = [torch.zeros((W * B, H), dtype=torch.bfloat16, device=dev) for _ in range(W)]
    tab = torch.tensor([c.data_ptr() for c in copies], dtype=torch.int64, device=dev)
    d_blocks = to_dev_bf16(blocks, dev)
    k3g.call("k3g_attnres_rms_push", d_blocks, to_dev(sw, dev), to_dev_bf16(gamma, dev), copies[rank], tab, nb, snapshot, B, rank, W,
             None, None, None, None, to_dev_bf16(prefix, dev), None, 0, H, 1e-5, k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(d_blocks), want_blocks)
    for c in copies:
        got = bf16_bits(c)
        assert np.array_equal(got[rank * B:(rank + 1) * B], want)
        assert not got[:rank * B].any() and not got[(rank + 1) * B:].any()
