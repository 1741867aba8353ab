"""CPU restatement (numpy) of the element-wise steps next to the row-parallel GEMM.

Test infrastructure only: imported by tests/ and by nothing that ships.

Parity UNPINNED: these follow the rounding points of the reference's CUDA kernels
as read from their source (csrc/layernorm_kernels.cu:17-58,60-149,
csrc/activation_kernels.cu:22-38); the kernels cannot run in this environment and
the reference's pure-torch fall-backs round at different points (variance from the
unrounded sum, layernorm.py forward_native), so no golden vector of the reference
backs them.  The tolerances in the tests are those of the reference's own kernel
tests (atol = rtol = 1e-2, tests/kernels/core/test_layernorm.py).
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


def all_reduce(parts: list[np.ndarray], dtype: str) -> np.ndarray:
    """SUM of 16-bit partials in rank order with fp32 accumulation, one rounding."""
    acc = np.zeros(parts[0].shape, dtype=np.float32)
    for p in parts:
        acc = acc + p.astype(np.float32)
    return round_to_dtype(acc, dtype)
