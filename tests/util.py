"""Shared helpers of the parity tests: seeded inputs, bf16 <-> torch plumbing, comparisons."""
import numpy as np

import k3o


def rng(seed):
    return np.random.Generator(np.random.Philox(seed))


def normal_bf16(g, shape, mean=0.0, std=1.0):
    return k3o.f32_to_bf16((g.standard_normal(shape, dtype=np.float32) * std + mean).astype(np.float32))


def to_dev_bf16(h, dev):
    import torch
    return torch.from_numpy(h.view(np.int16)).to(dev).view(torch.bfloat16)


def to_dev(a, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def bf16_bits(t):
    """torch bf16 tensor -> numpy uint16 bit patterns."""
    import torch
    return t.detach().view(torch.int16).cpu().numpy().view(np.uint16)


def bf16_ulp_diff(a, b):
    """Distance in bf16 ulps between two uint16 bit-pattern arrays (sign-magnitude aware)."""
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, -(x & 0x7FFF), x & 0x7FFF)
    return np.abs(key(a) - key(b))


def fp8_code_diff(a, b):
    """Distance in E4M3 codes (sign-magnitude aware)."""
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x80, -(x & 0x7F), x & 0x7F)
    return np.abs(key(a) - key(b))


def router_picks_differ_only_at_near_ties(S, bias, idx_a, idx_b, ulps=4):
    """Two top-k results for the same logits may differ only where the competing biased scores (sigmoid + bias, an
    f32 quantity) lie within `ulps` f32 ulps of each other: at every position where the picks differ, the two
    experts' scores must be that close.  Returns (rows that differ, worst gap in ulps); raises on a wider gap."""
    sig = 1.0 / (1.0 + np.exp(-S.astype(np.float64))) + bias.astype(np.float64)
    rows = np.nonzero((idx_a != idx_b).any(axis=1))[0]
    worst = 0.0
    for b in rows:
        for r in np.nonzero(idx_a[b] != idx_b[b])[0]:
            x, y = sig[b, idx_a[b, r]], sig[b, idx_b[b, r]]
            gap = abs(x - y) / float(np.spacing(np.float32(max(abs(x), abs(y)))))
            worst = max(worst, gap)
            assert gap < ulps, "row %d pick %d: experts %d / %d have scores %.9g / %.9g, %.1f ulps apart" % (b, r, idx_a[b, r], idx_b[b, r], x, y, gap)
    return len(rows), worst
