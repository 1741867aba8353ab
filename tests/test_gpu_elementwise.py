"""fused_add_rms_norm / rms_norm / silu_and_mul against the numpy restatement of the
reference kernels' rounding (oracle/elementwise_oracle.py).  Tolerance: the reference's
own kernel tests use atol = rtol = 1e-2 (tests/kernels/core/test_layernorm.py,
test_activation.py); here results must also agree to one 16-bit ulp on at least
99.9 % of the elements (the fp32 sum of squares is taken in a different order)."""
import numpy as np
import pytest

from oracle import elementwise_oracle as eo
from tests import gpu_utils as G

pytestmark = pytest.mark.gpu


def _close(got, want, dtype):
    got, want = got.astype(np.float32), want.astype(np.float32)
    assert np.allclose(got, want, atol=1e-2, rtol=1e-2)
    ulp = 2.0 ** (-7 if dtype == "bfloat16" else -10)
    near = np.abs(got - want) <= ulp * np.maximum(np.abs(want), 1e-30) * 1.0001
    assert near.mean() >= 0.999, near.mean()


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("tokens,hidden", [(1, 4096), (7, 768), (64, 8192), (33, 5120), (2, 8)])
def test_fused_add_rms_norm(dtype, tokens, hidden):
    import torch
    from vllm_b200 import _custom_ops as ops
    rng = np.random.default_rng(tokens * 131 + hidden)
    x = eo.round_to_dtype(rng.standard_normal((tokens, hidden)).astype(np.float32), dtype)
    r = eo.round_to_dtype(rng.standard_normal((tokens, hidden)).astype(np.float32) * 3, dtype)
    w = eo.round_to_dtype(1 + 0.1 * rng.standard_normal(hidden).astype(np.float32), dtype)
    want, want_res = eo.fused_add_rms_norm(x, r, w, 1e-5, dtype)
    xt, rt, wt = G.t16(x, dtype), G.t16(r, dtype), G.t16(w, dtype)
    ops.fused_add_rms_norm(xt, rt, wt, 1e-5)
    torch.cuda.synchronize()
    assert np.array_equal(G.n16(rt), want_res)          # the sum is rounded once: exact
    _close(G.n16(xt), want, dtype)
    # plain rms_norm, out of place, and a strided input view
    out = torch.empty_like(xt)
    ops.rms_norm(out, G.t16(x, dtype), wt, 1e-5)
    _close(G.n16(out), eo.rms_norm(x, w, 1e-5, dtype), dtype)
    if hidden % 16 == 0:
        wide = G.t16(np.concatenate([x, x], axis=1), dtype)
        view, res2 = wide[:, :hidden], G.t16(r, dtype)
        ops.fused_add_rms_norm(view, res2, wt, 1e-5)
        _close(G.n16(view.contiguous()), want, dtype)
        assert np.array_equal(G.n16(wide[:, hidden:].contiguous()), x)   # the other half is untouched


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("tokens,d", [(1, 14336), (64, 14336), (5, 8), (300, 1024)])
def test_silu_and_mul(dtype, tokens, d):
    import torch
    from vllm_b200 import _custom_ops as ops
    rng = np.random.default_rng(tokens + d)
    x = eo.round_to_dtype(rng.standard_normal((tokens, 2 * d)).astype(np.float32) * 2, dtype)
    xt = G.t16(x, dtype)
    out = torch.empty((tokens, d), dtype=xt.dtype, device=xt.device)
    ops.silu_and_mul(out, xt)
    torch.cuda.synchronize()
    _close(G.n16(out), eo.silu_and_mul(x, dtype), dtype)


def test_argument_checks():
    import torch
    from vllm_b200 import _custom_ops as ops
    x = torch.zeros((2, 12), dtype=torch.bfloat16, device="cuda")
    w = torch.ones(12, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        ops.fused_add_rms_norm(x, torch.zeros_like(x), w, 1e-5)      # hidden % 8 != 0
    with pytest.raises(RuntimeError):
        ops.silu_and_mul(torch.zeros((2, 5), dtype=torch.bfloat16, device="cuda"),
                         torch.zeros((2, 12), dtype=torch.bfloat16, device="cuda"))
