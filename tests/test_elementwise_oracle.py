"""CPU checks of the element-wise oracle: it agrees with plain float64 math up to the
16-bit rounding it models, and its rounding points are where the reference kernels
round (sum before variance, scaled value before the weight product)."""
import numpy as np

from oracle import elementwise_oracle as eo


def test_rms_norm_against_float64():
    rng = np.random.default_rng(0)
    for dtype, tol in (("bfloat16", 2 ** -7), ("float16", 2 ** -10)):
        x = eo.round_to_dtype(rng.standard_normal((5, 256)).astype(np.float32), dtype)
        r = eo.round_to_dtype(rng.standard_normal((5, 256)).astype(np.float32), dtype)
        w = eo.round_to_dtype(1 + 0.1 * rng.standard_normal(256).astype(np.float32), dtype)
        out, res = eo.fused_add_rms_norm(x, r, w, 1e-6, dtype)
        z = (x.astype(np.float64) + r.astype(np.float64))
        assert np.array_equal(res, eo.round_to_dtype(z.astype(np.float32), dtype))
        zz = res.astype(np.float64)
        ref = zz / np.sqrt((zz ** 2).mean(-1, keepdims=True) + 1e-6) * w.astype(np.float64)
        assert np.max(np.abs(out - ref) / np.maximum(np.abs(ref), 1e-3)) <= 2.5 * tol
        assert np.array_equal(out, eo.round_to_dtype(out, dtype))     # representable in the dtype


def test_silu_and_mul_against_float64():
    rng = np.random.default_rng(1)
    for dtype, tol in (("bfloat16", 2 ** -7), ("float16", 2 ** -10)):
        x = eo.round_to_dtype(rng.standard_normal((3, 64)).astype(np.float32) * 3, dtype)
        out = eo.silu_and_mul(x, dtype)
        a, b = x[:, :32].astype(np.float64), x[:, 32:].astype(np.float64)
        ref = a / (1 + np.exp(-a)) * b
        assert np.max(np.abs(out - ref) / np.maximum(np.abs(ref), 1e-3)) <= 2.5 * tol


def test_all_reduce_order_and_rounding():
    parts = [np.array([1.0, 256.0], dtype=np.float32), np.array([2 ** -9, 1.0], dtype=np.float32),
             np.array([2 ** -9, 1.0], dtype=np.float32)]
    out = eo.all_reduce(parts, "bfloat16")
    # fp32 accumulation, one rounding at the end: 1 + 2^-8 rounds to 1, 258 rounds to 258
    assert out.tolist() == [1.0, 258.0]
