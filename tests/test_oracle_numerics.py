"""CPU checks of the oracle's numeric primitives against independent implementations."""
import math

import ml_dtypes
import numpy as np

import k3o


def all_bf16_finite():
    h = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    f = k3o.bf16_to_f32(h)
    return h[np.isfinite(f)], f[np.isfinite(f)]


def test_bf16_roundtrip_matches_ml_dtypes():
    g = np.random.Generator(np.random.Philox(1))
    x = (g.standard_normal(200000, dtype=np.float32) * np.float32(10.0) ** g.integers(-30, 30, 200000)).astype(np.float32)
    x = np.concatenate([x, np.array([0.0, -0.0, np.inf, -np.inf, 1.00390625, 1.01171875, 3.3895314e38], np.float32)])
    ours = k3o.f32_to_bf16(x)
    ref = x.astype(ml_dtypes.bfloat16).view(np.uint16)
    assert np.array_equal(ours, ref)
    lib = k3o.lib()
    for v in x[:2000]:
        assert lib.k3o_f32_to_bf16(float(v)) == int(np.float32(v).astype(ml_dtypes.bfloat16).view(np.uint16))


def test_e4m3_encode_matches_ml_dtypes_on_every_bf16_times_scales():
    lib = k3o.lib()
    _, f = all_bf16_finite()
    for scale in (1.0, 0.5, 2.0 ** -6, 2.0 ** -9, 3.0, 448.0):
        x = (f * np.float32(scale)).astype(np.float32)
        x = x[np.isfinite(x)]
        ref = np.clip(x, -448.0, 448.0).astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
        ours = np.array([lib.k3o_e4m3_encode(float(v)) for v in x[::7]], np.uint8)
        assert np.array_equal(ours, ref[::7]), scale
    assert lib.k3o_e4m3_encode(float("nan")) == 0x7F
    assert lib.k3o_e4m3_encode(float("inf")) == 0x7E and lib.k3o_e4m3_encode(-1e30) == 0xFE
    assert lib.k3o_e4m3_encode(464.0) == 0x7E and lib.k3o_e4m3_encode(447.9) == 0x7E
    # ties to even at the subnormal step 2^-9: 0.5 * 2^-9 -> 0, 1.5 * 2^-9 -> 2
    assert lib.k3o_e4m3_encode(2.0 ** -10) == 0 and lib.k3o_e4m3_encode(1.5 * 2.0 ** -9) == 2


def test_e4m3_decode_is_inverse():
    lib = k3o.lib()
    for c in range(256):
        v = lib.k3o_e4m3_decode(c)
        if math.isnan(v):
            assert c & 0x7F == 0x7F
            continue
        assert lib.k3o_e4m3_encode(v) == c or (v == 0.0)
    assert np.allclose(k3o.e4m3_to_f32(np.arange(256, dtype=np.uint8))[:0x7F],
                       [lib.k3o_e4m3_decode(c) for c in range(0x7F)])


def test_ue8m0_integer_formula_equals_reference_float_formula_on_every_bf16():
    """source/k3_moe_prefill_v4.cu:130-131 evaluates ceil(log2(amax / 448)) in f32; the oracle and
    the kernels use exact integer arithmetic.  They agree on every non-negative bf16 amax."""
    lib = k3o.lib()
    h = np.arange(0, 0x7F80, dtype=np.uint32).astype(np.uint16)   # +0 .. largest finite
    f = k3o.bf16_to_f32(h)
    for v in f:
        assert lib.k3o_ue8m0_exp(float(v)) == lib.k3o_ue8m0_exp_float_formula(float(v)), v
    assert lib.k3o_ue8m0_exp(448.0) == 0 and lib.k3o_ue8m0_exp(450.0) == 1 and lib.k3o_ue8m0_exp(224.0) == -1
    assert lib.k3o_ue8m0_exp(0.0) == 0 and lib.k3o_ue8m0_exp(1e-38) == -127


def test_rsqrt_and_det_exp_accuracy():
    lib = k3o.lib()
    g = np.random.Generator(np.random.Philox(2))
    for v in np.exp(g.uniform(-20, 20, 5000)).astype(np.float32):
        exact = 1.0 / math.sqrt(float(v))
        got = lib.k3o_rsqrt_rn(float(v))
        assert got == float(np.float32(exact)), v
    for v in g.uniform(-80, 80, 20000).astype(np.float32):
        got, exact = lib.k3o_det_exp(float(v)), math.exp(float(v))
        assert abs(got - exact) <= 4e-7 * exact, (v, got, exact)
    assert lib.k3o_det_sigmoid(0.0) == 0.5
