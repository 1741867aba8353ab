"""CPU checks of the element-wise oracle: it agrees with plain float64 math up to the
16-bit rounding it models, and its rounding points are where the reference kernels
round (sum before variance, scaled value before the weight product)."""
import os

import numpy as np
import pytest

from oracle import elementwise_oracle as eo
from tests import helpers as H

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("tag,dtype", [("bf16", "bfloat16"), ("f16", "float16")])
def test_oracle_against_recorded_reference_outputs(tag, dtype):
    """Outputs recorded from the reference's RMSNorm.forward_static and
    SiluAndMul.forward_native.  The *_native restatements must reproduce them (one 16-bit
    unit of slack where numpy's and torch's fp32 reductions / exp round differently); the
    kernel-order functions must stay within the reference's kernel-vs-torch tolerance."""
    g = np.load(os.path.join(GOLDEN, f"elementwise_{tag}.npz"))
    f = lambda name: H.from_bits16(g[name], dtype)
    x, res, w, eps = f("x_bits"), f("res_bits"), f("w_bits"), float(g["eps"])
    want_plain, want_fused, want_res = f("rms_bits"), f("fused_bits"), f("new_res_bits")
    ulp = 2.0 ** -7 if dtype == "bfloat16" else 2.0 ** -10

    def close_1ulp(got, want):
        exact = np.mean(got == want)
        return exact >= 0.97 and np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-6)) <= ulp

    got_plain = eo.rms_norm_native(x, w, eps, dtype)
    got_fused, got_res = eo.rms_norm_native(x, w, eps, dtype, residual=res)
    assert np.array_equal(got_res, want_res)            # one fp32 add, one rounding: exact
    assert close_1ulp(got_plain, want_plain) and close_1ulp(got_fused, want_fused)
    gu = f("gate_up_bits")
    assert close_1ulp(eo.silu_and_mul_native(gu, dtype), f("act_bits"))
    # kernel-order functions against the same recordings, at atol = rtol = 1e-2
    tol = lambda got, want: np.all(np.abs(got - want) <= 1e-2 + 1e-2 * np.abs(want))
    assert tol(eo.rms_norm(x, w, eps, dtype), want_plain)
    k_out, k_res = eo.fused_add_rms_norm(x, res, w, eps, dtype)
    assert np.array_equal(k_res, want_res) and tol(k_out, want_fused)
    assert tol(eo.silu_and_mul(gu, dtype), f("act_bits"))


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
