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
