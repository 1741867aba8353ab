"""Shared builders for the parity tests: synthetic quantized layers in the
formats the ops consume, produced with the CPU oracle."""
from __future__ import annotations

import functools

import numpy as np

from oracle import marlin_oracle as mo

TYPE_IDS = {"uint4b8": mo.UINT4B8_ID, "uint8b128": mo.UINT8B128_ID, "uint4": mo.UINT4_ID,
            "uint8": mo.UINT8_ID}
TYPE_BITS = {"uint4b8": 4, "uint8b128": 8, "uint4": 4, "uint8": 8}
TYPE_BIAS = {"uint4b8": 8, "uint8b128": 128, "uint4": 0, "uint8": 0}

# north-star tolerances for the GEMM
MAX_ABS_FRAC = 2e-2
MEAN_REL = 5e-3


def to_bits16(x: np.ndarray, dtype: str) -> np.ndarray:
    """float32 array (already representable) -> uint16 bit patterns."""
    if dtype == "float16":
        return x.astype(np.float16).view(np.uint16)
    return (mo.round_to_bf16(x).view(np.uint32) >> 16).astype(np.uint16)


def from_bits16(bits: np.ndarray, dtype: str) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    if dtype == "float16":
        return bits.view(np.float16).astype(np.float32)
    return (bits.astype(np.uint32) << 16).view(np.float32)


class Layer:
    """One synthetic quantized layer in op-ready (numpy) form."""


@functools.lru_cache(maxsize=16)
def make_layer(size_k: int, size_n: int, qtype: str, group_size: int, act_order: bool,
               dtype: str, seed: int = 0, with_bias: bool = False) -> Layer:
    rng = np.random.default_rng(seed + 7919 * size_k + size_n)
    bits = TYPE_BITS[qtype]
    has_zp = qtype in ("uint4", "uint8")
    G = 1 if group_size in (-1, size_k) else size_k // group_size
    L = Layer()
    L.size_k, L.size_n, L.qtype, L.bits, L.dtype = size_k, size_n, qtype, bits, dtype
    L.group_size, L.num_groups, L.act_order, L.has_zp = group_size, G, act_order, has_zp
    L.type_id, L.type_bias = TYPE_IDS[qtype], TYPE_BIAS[qtype]
    # codes as stored in the checkpoint (row k of the original weight)
    q = rng.integers(0, 1 << bits, size=(size_k, size_n), dtype=np.int32)
    scales = mo.round_to_dtype(rng.uniform(0.002, 0.02, size=(G, size_n)).astype(np.float32), dtype)
    L.q, L.scales = q, scales
    L.zeros = rng.integers(0, 1 << bits, size=(G, size_n), dtype=np.int32) if has_zp else None
    if act_order:
        assert G > 1
        g_idx = (np.arange(size_k) // group_size)[rng.permutation(size_k)].astype(np.int32)
        L.g_idx_ckpt = g_idx
        L.g_idx, L.sort_idx = mo.sort_g_idx(g_idx)
        q_sorted = q[L.sort_idx.astype(np.int64), :]
    else:
        L.g_idx_ckpt = L.g_idx = L.sort_idx = None
        q_sorted = q
    L.gptq_qweight = mo.gptq_pack(q, bits)
    L.awq_qweight = mo.awq_pack(q, bits)
    L.marlin_q = mo.marlin_weights(q_sorted, bits)
    L.marlin_s = mo.marlin_permute_scales(scales, size_k, size_n, group_size if G > 1 else -1)
    L.marlin_zp = mo.marlin_zero_points(L.zeros, G, size_n, bits) if has_zp else None
    if with_bias:
        L.bias = mo.round_to_dtype(10 * rng.standard_normal(size_n).astype(np.float32), dtype)
        L.marlin_bias = mo.marlin_permute_bias(L.bias)
    else:
        L.bias = L.marlin_bias = None
    # dense dequantised weight in checkpoint row order (w[k] multiplies a[:, k])
    g_of_k = L.g_idx_ckpt if act_order else None
    L.w = mo.dequantize(q, scales, dtype, bias=L.type_bias, zeros=L.zeros, g_idx=g_of_k,
                        group_size=group_size if G > 1 else -1)
    return L


def make_activations(size_m: int, size_k: int, dtype: str, seed: int = 1) -> np.ndarray:
    rng = np.random.default_rng(seed + 31 * size_m + size_k)
    return mo.round_to_dtype(rng.standard_normal((size_m, size_k)).astype(np.float32), dtype)


def gemm_errors(out: np.ndarray, ref: np.ndarray):
    """(max-abs error / max|ref|, mean|err| / mean|ref|)."""
    err = np.abs(out.astype(np.float64) - ref.astype(np.float64))
    return float(err.max() / max(np.abs(ref).max(), 1e-30)), float(err.mean() / max(np.abs(ref).mean(), 1e-30))
