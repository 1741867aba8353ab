"""CPU restatement (numpy) of the element-wise steps next to the row-parallel GEMM.

Test infrastructure only: imported by tests/ and by nothing that ships.

Parity pinned on the reference's torch implementations: `rms_norm_native` and
`silu_and_mul_native` restate RMSNorm.forward_static
(vllm/model_executor/layers/layernorm.py:180-224) and SiluAndMul.forward_native
(vllm/model_executor/layers/activation.py:84-87) and are checked bit for bit against
outputs recorded from them (tests/golden/elementwise_*.npz, made by
tests/golden/make_golden.py).  `rms_norm`, `fused_add_rms_norm` and `silu_and_mul`
follow the rounding points of the reference's CUDA kernels as read from their source
(csrc/layernorm_kernels.cu:17-58,60-149, csrc/activation_kernels.cu:22-38: the sum is
rounded to 16 bits before the variance is taken, where the torch path takes it from the
unrounded sum); those kernels cannot run in this environment, so these three are held to
the recorded torch outputs at the tolerance the reference uses between its kernels and
its torch path (atol = rtol = 1e-2, tests/kernels/core/test_layernorm.py).
"""
from __future__ import annotations

import numpy as np

from .marlin_oracle import round_to_dtype  # noqa: F401  (re-exported for the tests)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float, dtype: str) -> np.ndarray:
    """rms_norm_kernel, csrc/layernorm_kernels.cu:17-58: variance in fp32 from the 16-bit
    input, out = ((T)(x * rstd)) * weight with the product rounded to 16 bits."""
    x = x.astype(np.float32)
    var = (x.astype(np.float64) ** 2).mean(axis=-1, keepdims=True)
    rstd = (1.0 / np.sqrt(var + eps)).astype(np.float32)
    y = round_to_dtype(x * rstd, dtype)
    return round_to_dtype(y * weight.astype(np.float32), dtype)


def fused_add_rms_norm(x: np.ndarray, residual: np.ndarray, weight: np.ndarray, eps: float,
                       dtype: str):
    """fused_add_rms_norm_kernel, csrc/layernorm_kernels.cu:60-149.  Returns
    (normalised, new residual): z = (T)(x + residual); residual = z; out as rms_norm(z)."""
    z = round_to_dtype(x.astype(np.float32) + residual.astype(np.float32), dtype)
    return rms_norm(z, weight, eps, dtype), z


def silu_and_mul(x: np.ndarray, dtype: str) -> np.ndarray:
    """act_and_mul_kernel with silu_kernel, csrc/activation_kernels.cu:22-38:
    out = ((T)(a / (1 + exp(-a)))) * b with a, b the two halves of the last axis."""
    d = x.shape[-1] // 2
    a, b = x[..., :d].astype(np.float32), x[..., d:].astype(np.float32)
    s = round_to_dtype(a / (1.0 + np.exp(-a, dtype=np.float32)), dtype)
    return round_to_dtype(s * b, dtype)


def rms_norm_native(x: np.ndarray, weight: np.ndarray, eps: float, dtype: str,
                    residual: np.ndarray | None = None):
    """RMSNorm.forward_static (layernorm.py:180-224): fp32 sum with the residual, new residual
    = the sum rounded to 16 bits, variance from the UNROUNDED fp32 sum, x * rsqrt(var + eps) in
    fp32 rounded to 16 bits, then the product with the weight rounded again.  Returns the
    output, or (output, new residual) when a residual is given."""
    x32 = x.astype(np.float32)
    new_res = None
    if residual is not None:
        x32 = x32 + residual.astype(np.float32)
        new_res = round_to_dtype(x32, dtype)
    var = np.mean(x32 * x32, axis=-1, keepdims=True, dtype=np.float32)
    y = round_to_dtype(x32 * (np.float32(1.0) / np.sqrt(var + np.float32(eps))), dtype)
    out = round_to_dtype(y * weight.astype(np.float32), dtype)
    return out if residual is None else (out, new_res)


def silu_and_mul_native(x: np.ndarray, dtype: str) -> np.ndarray:
    """SiluAndMul.forward_native (activation.py:84-87): F.silu on the 16-bit first half
    (computed in fp32, rounded to 16 bits), times the second half, rounded."""
    d = x.shape[-1] // 2
    a, b = x[..., :d].astype(np.float32), x[..., d:].astype(np.float32)
    s = round_to_dtype(a / (np.float32(1.0) + np.exp(-a)), dtype)
    return round_to_dtype(s * b, dtype)


def all_reduce(parts: list[np.ndarray], dtype: str) -> np.ndarray:
    """SUM of 16-bit partials in rank order with fp32 accumulation, one rounding."""
    acc = np.zeros(parts[0].shape, dtype=np.float32)
    for p in parts:
        acc = acc + p.astype(np.float32)
    return round_to_dtype(acc, dtype)
