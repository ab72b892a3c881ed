"""Load-time derived tables (fills, casts, rope table, conv taps transpose, scoring vector, small-projection block, packed
scale words, MLA expansion weight) against the CPU oracle."""
import numpy as np
import pytest

import k3o
from util import bf16_bits, bf16_ulp_diff, normal_bf16, rng, to_dev, to_dev_bf16

pytestmark = pytest.mark.gpu


def test_fills_iota_casts(k3g, dev):
    import torch
    s = k3g.current_stream()
    for kind, dt, val in ((0, torch.bfloat16, 1.0), (1, torch.float32, -2.5), (2, torch.int32, -7), (3, torch.int64, 1 << 40), (4, torch.uint8, 200)):
        p = torch.zeros(1003, dtype=dt, device=dev)
        k3g.call("k3g_fill", p, 1000, kind, float(val) if kind < 2 else 0.0, int(val) if kind >= 2 else 0, s)
        torch.cuda.synchronize()
        assert bool((p[:1000] == val).all()) and bool((p[1000:] == 0).all())
    p = torch.full((40,), -1, dtype=torch.int32, device=dev)
    k3g.call("k3g_iota_i32", p, 13, 5, 3, 3, s)
    torch.cuda.synchronize()
    want = np.full(40, -1, np.int32); want[0:39:3] = 5 + 3 * np.arange(13)
    assert np.array_equal(p.cpu().numpy(), want)
    w = normal_bf16(rng(1), (777,))
    for plus in (0, 1):
        o = torch.zeros(777, dtype=torch.float32, device=dev)
        k3g.call("k3g_cast_bf16_f32", to_dev_bf16(w, dev), o, 777, plus, s)
        torch.cuda.synchronize()
        assert np.array_equal(o.cpu().numpy(), (k3o.bf16_to_f32(w) + np.float32(plus)).astype(np.float32))


def test_rope_table(k3g, dev):
    import torch
    rows, half = 4096, 32
    t = torch.zeros((rows, 2 * half), dtype=torch.bfloat16, device=dev)                  # one buffer, cos | sin halves
    k3g.call("k3g_rope_table", t, t.view(-1)[half:], rows, half, 2 * half, 50000.0, k3g.current_stream())
    torch.cuda.synchronize()
    cos, sin = k3o.rope_table(rows, half, 50000.0)
    got = bf16_bits(t)
    for g, w in ((got[:, :half], cos), (got[:, half:], sin)):
        d = bf16_ulp_diff(np.ascontiguousarray(g), w)      # device powf / cosf / sinf vs libm: last-ulp differences in f32
        a, b = k3o.bf16_to_f32(np.ascontiguousarray(g)), k3o.bf16_to_f32(w)
        assert np.abs(a - b).max() <= 8e-3 and (d > 0).mean() < 0.05                      # large angles: f32 argument error
    assert np.array_equal(got[0, :half], k3o.f32_to_bf16(np.ones(half, np.float32)))      # row 0: cos 1, sin 0
    assert not got[0, half:].any()


def test_conv_taps_scoring_wsm(k3g, dev):
    import torch
    g = rng(2)
    s = k3g.current_stream()
    inner = 3072
    q, k, v = (g.standard_normal((inner, 4), dtype=np.float32) for _ in range(3))
    cw = torch.zeros((3, 4, inner), dtype=torch.float32, device=dev)
    k3g.call("k3g_conv_taps", to_dev(q, dev), to_dev(k, dev), to_dev(v, dev), cw, inner, s)
    norm, proj = normal_bf16(g, (7168,)), normal_bf16(g, (7168,))
    sw = torch.zeros(7168, dtype=torch.float32, device=dev)
    k3g.call("k3g_scoring", to_dev_bf16(norm, dev), to_dev_bf16(proj, dev), sw, 7168, s)
    b, fa = normal_bf16(g, (24, 7168)), normal_bf16(g, (128, 7168))
    w = torch.full((256, 7168), 1.0, dtype=torch.bfloat16, device=dev)
    k3g.call("k3g_wsm", to_dev_bf16(b, dev), to_dev_bf16(fa, dev), w, 24, 7168, s)
    torch.cuda.synchronize()
    assert np.array_equal(cw.cpu().numpy(), k3o.conv_taps(q, k, v))
    assert np.array_equal(sw.cpu().numpy(), k3o.scoring(norm, proj))
    assert np.array_equal(bf16_bits(w), k3o.wsm(b, fa, 24))


@pytest.mark.parametrize("interleave", [0, 1])
def test_mega_sf_pack_and_kvb_aug(k3g, dev, interleave):
    import torch
    g = rng(3 + interleave)
    s = k3g.current_stream()
    raw = g.integers(0, 256, (3, 256, 12), dtype=np.uint8)
    out = torch.zeros((3, 3, 256), dtype=torch.int32, device=dev)
    k3g.call("k3g_mega_sf_pack", to_dev(raw, dev), out, 3, 256, 12, interleave, s)
    heads = 2
    wkv = normal_bf16(g, (heads * 256, 512))
    aug = torch.full((heads * 320, 576), 3.0, dtype=torch.bfloat16, device=dev)
    k3g.call("k3g_kvb_aug", to_dev_bf16(wkv, dev), aug, heads, s)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), k3o.mega_sf_pack(raw, interleave))
    assert np.array_equal(bf16_bits(aug), k3o.kvb_aug(wkv, heads))
