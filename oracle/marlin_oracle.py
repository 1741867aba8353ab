"""CPU oracle for the weight-only quantized linear path (Marlin surface).

TEST INFRASTRUCTURE ONLY.  This module is a numpy restatement of the
reference's CPU packers and of its dequantise-then-matmul result.  It is the
checker for the CUDA kernels: only the test-suite, the smoke entry and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it.
Nothing in the shipped package calls into it.

Parity status: PINNED.  Every function here is compared bit-for-bit with the
output of the reference's own Python (imported once, on CPU) through the
fixtures under ``tests/golden/`` — see ``tests/golden/make_golden.py``.

Each function cites the reference location it restates (paths relative to the
reference project root).
"""

from __future__ import annotations

import numpy as np

# ---------------------------------------------------------------------------
# ScalarType ids   (vllm/scalar_type.py:136-164, csrc/core/scalar_type.hpp:124-157)
# ---------------------------------------------------------------------------


def scalar_type_id(exponent: int, mantissa: int, signed: bool, bias: int,
                   finite_values_only: bool = False, nan_repr: int = 1) -> int:
    """64-bit id: exponent(8) | mantissa(8) | signed(1) | bias(32) |
    finite_only(1) | nan_repr(8), packed low to high
    (vllm/scalar_type.py:136-164).  nan_repr 1 == IEEE_754, the default."""
    val, off = 0, 0
    for member, width in ((exponent, 8), (mantissa, 8), (int(signed), 1),
                          (bias, 32), (int(finite_values_only), 1),
                          (nan_repr, 8)):
        val |= (int(member) & ((1 << width) - 1)) << off
        off += width
    return val


UINT4B8_ID = scalar_type_id(0, 4, False, 8)
UINT4_ID = scalar_type_id(0, 4, False, 0)
UINT8B128_ID = scalar_type_id(0, 8, False, 128)
UINT8_ID = scalar_type_id(0, 8, False, 0)


def scalar_type_min_max(mantissa: int, signed: bool, bias: int):
    """Integer ScalarType min()/max() (vllm/scalar_type.py:93-118,170-182)."""
    bits = mantissa + int(signed)
    raw_min = -(1 << (bits - 1)) if signed else 0
    raw_max = (1 << mantissa) - 1
    return raw_min - bias, raw_max - bias


# ---------------------------------------------------------------------------
# checkpoint-format packers  (quant_utils.py:524-633)
# ---------------------------------------------------------------------------

_INTERLEAVE = {4: np.array([0, 2, 4, 6, 1, 3, 5, 7]), 8: np.array([0, 2, 1, 3])}


def pack_factor(num_bits: int) -> int:
    assert num_bits in (4, 8)
    return 32 // num_bits


def pack_rows(q: np.ndarray, num_bits: int) -> np.ndarray:
    """GPTQ packing along K: word r of column n holds k = r*pf + i at bit
    i*bits (quant_utils.py:524-545, gptq_pack 605-611)."""
    pf = pack_factor(num_bits)
    K, N = q.shape
    assert K % pf == 0
    u = q.astype(np.uint32).reshape(K // pf, pf, N)
    out = np.zeros((K // pf, N), dtype=np.uint32)
    for i in range(pf):
        out |= u[:, i, :] << np.uint32(num_bits * i)
    return out.view(np.int32)


def unpack_rows(packed: np.ndarray, num_bits: int) -> np.ndarray:
    pf = pack_factor(num_bits)
    R, N = packed.shape
    u = packed.view(np.uint32)
    mask = np.uint32((1 << num_bits) - 1)
    out = np.empty((R, pf, N), dtype=np.int32)
    for i in range(pf):
        out[:, i, :] = (u >> np.uint32(num_bits * i)) & mask
    return out.reshape(R * pf, N)


def pack_cols(q: np.ndarray, num_bits: int) -> np.ndarray:
    """Packing along N: word w of row k holds n = w*pf + i at bit i*bits
    (quant_utils.py:548-571)."""
    pf = pack_factor(num_bits)
    K, N = q.shape
    assert N % pf == 0
    u = q.astype(np.uint32).reshape(K, N // pf, pf)
    out = np.zeros((K, N // pf), dtype=np.uint32)
    for i in range(pf):
        out |= u[:, :, i] << np.uint32(num_bits * i)
    return out.view(np.int32)


def unpack_cols(packed: np.ndarray, num_bits: int) -> np.ndarray:
    """Inverse of pack_cols (quant_utils.py:574-602)."""
    pf = pack_factor(num_bits)
    K, W = packed.shape
    u = packed.view(np.uint32)
    mask = np.uint32((1 << num_bits) - 1)
    out = np.empty((K, W, pf), dtype=np.int32)
    for i in range(pf):
        out[:, :, i] = (u >> np.uint32(num_bits * i)) & mask
    return out.reshape(K, W * pf)


def gptq_pack(q: np.ndarray, num_bits: int) -> np.ndarray:
    return pack_rows(q, num_bits)


def awq_pack(q: np.ndarray, num_bits: int) -> np.ndarray:
    """AWQ packing: inside every run of pf columns the values are stored in
    the order [0,2,4,6,1,3,5,7] (4-bit) / [0,2,1,3] (8-bit), then packed along
    N (quant_utils.py:614-633)."""
    K, N = q.shape
    il = _INTERLEAVE[num_bits]
    shuffled = q.reshape(K, N // len(il), len(il))[:, :, il].reshape(K, N)
    return pack_cols(shuffled, num_bits)


def awq_unpack(packed: np.ndarray, num_bits: int) -> np.ndarray:
    il = _INTERLEAVE[num_bits]
    inv = np.argsort(il)
    flat = unpack_cols(packed, num_bits)
    K, N = flat.shape
    return flat.reshape(K, N // len(il), len(il))[:, :, inv].reshape(K, N)


# ---------------------------------------------------------------------------
# Marlin weight layout  (marlin_utils_test.py:32-93; device restatement in
# csrc/quantization/gptq_marlin/gptq_marlin_repack.cu:115-202)
# ---------------------------------------------------------------------------


def marlin_tile_coords(num_bits: int):
    """For one 16(K) x 64(N) tile return (rows, cols), each of shape
    [words, pf]: the tile-local (k, n) of the value stored in sub-field t of
    word w.

    4-bit: word w = lane*4 + sub, nibble t.  8-bit: word w = lane*8 + sub*2 +
    half, byte t.  lane = 4*c + q owns column c (+8) of 16-column sub-tile
    `sub` and rows 2q + {0,1,8,9}; this is the mma.m16n8k16 B-fragment
    ownership (marlin_utils_test.py:63-93)."""
    lane = np.arange(32)
    c, q = lane // 4, lane % 4
    row_of_rr = np.stack([2 * q, 2 * q + 1, 2 * q + 8, 2 * q + 9], axis=1)  # [32,4]
    if num_bits == 4:
        # position p = 4*block + rr inside the 8 values of (lane, sub);
        # stored order is p = [0,2,4,6,1,3,5,7][t]
        p = _INTERLEAVE[4]
        block, rr = p // 4, p % 4
        rows = np.empty((32, 4, 8), dtype=np.int64)
        cols = np.empty((32, 4, 8), dtype=np.int64)
        for sub in range(4):
            rows[:, sub, :] = row_of_rr[:, rr]
            cols[:, sub, :] = 16 * sub + c[:, None] + 8 * block[None, :]
        return rows.reshape(128, 8), cols.reshape(128, 8)
    # 8-bit: two words per (lane, sub); half == block; byte order rr=[0,2,1,3]
    rr = _INTERLEAVE[8]
    rows = np.empty((32, 4, 2, 4), dtype=np.int64)
    cols = np.empty((32, 4, 2, 4), dtype=np.int64)
    for sub in range(4):
        for half in range(2):
            rows[:, sub, half, :] = row_of_rr[:, rr]
            cols[:, sub, half, :] = (16 * sub + c + 8 * half)[:, None]
    return rows.reshape(256, 4), cols.reshape(256, 4)


def marlin_weights(q: np.ndarray, num_bits: int) -> np.ndarray:
    """Dense codes [K, N] -> Marlin int32 [K/16, N*16/pf]
    (marlin_utils_test.py:32-60 with the permutation of 63-93)."""
    K, N = q.shape
    assert K % 16 == 0 and N % 64 == 0
    pf = pack_factor(num_bits)
    rows, cols = marlin_tile_coords(num_bits)          # [W, pf]
    W = rows.shape[0]
    tiles = q.astype(np.uint32).reshape(K // 16, 16, N // 64, 64).transpose(0, 2, 1, 3)
    vals = tiles[:, :, rows, cols]                     # [K/16, N/64, W, pf]
    out = np.zeros((K // 16, N // 64, W), dtype=np.uint32)
    for t in range(pf):
        out |= vals[..., t] << np.uint32(num_bits * t)
    return out.reshape(K // 16, N * 16 // pf).view(np.int32)


def marlin_unpack(packed: np.ndarray, size_k: int, size_n: int, num_bits: int) -> np.ndarray:
    """Marlin int32 [K/16, N*16/pf] -> dense codes [K, N] (inverse of
    marlin_weights; used to check what a kernel reads from the layout)."""
    pf = pack_factor(num_bits)
    rows, cols = marlin_tile_coords(num_bits)
    W = rows.shape[0]
    u = packed.view(np.uint32).reshape(size_k // 16, size_n // 64, W)
    mask = np.uint32((1 << num_bits) - 1)
    tiles = np.empty((size_k // 16, size_n // 64, 16, 64), dtype=np.int32)
    for t in range(pf):
        tiles[:, :, rows[:, t], cols[:, t]] = (u >> np.uint32(num_bits * t)) & mask
    return tiles.transpose(0, 2, 1, 3).reshape(size_k, size_n)


def gptq_marlin_repack(b_q_weight: np.ndarray, perm: np.ndarray | None,
                       size_k: int, size_n: int, num_bits: int) -> np.ndarray:
    """Oracle of the device op: GPTQ [K/pf, N] (+ optional row gather
    ``perm``: output row k reads input row perm[k]) -> Marlin layout
    (gptq_marlin_repack.cu:251-322; expected value built as in
    tests/kernels/quantization/test_marlin_gemm.py:121-156)."""
    q = unpack_rows(b_q_weight, num_bits)
    assert q.shape == (size_k, size_n)
    if perm is not None and perm.size:
        q = q[perm.astype(np.int64), :]
    return marlin_weights(q, num_bits)


def awq_marlin_repack(b_q_weight: np.ndarray, size_k: int, size_n: int,
                      num_bits: int) -> np.ndarray:
    """AWQ [K, N/pf] -> Marlin layout (awq_marlin_repack.cu:189-248;
    test_marlin_gemm.py:183-209)."""
    q = awq_unpack(b_q_weight, num_bits)
    assert q.shape == (size_k, size_n)
    return marlin_weights(q, num_bits)


# ---------------------------------------------------------------------------
# scale / zero-point / bias permutations  (marlin_utils.py:278-370)
# ---------------------------------------------------------------------------

# grouped scales: inside each 64-column chunk position 8*i + j holds column i + 8*j
_SCALE_PERM = np.array([i + 8 * j for i in range(8) for j in range(8)])
# channel-wise scales and bias: inside each 32-column chunk position 8*i + jj
# holds column 2*i + [0,1,8,9,16,17,24,25][jj]
_SCALE_PERM_SINGLE = np.array(
    [2 * i + j for i in range(4) for j in (0, 1, 8, 9, 16, 17, 24, 25)])


def marlin_permute_scales(s: np.ndarray, size_k: int, size_n: int, group_size: int) -> np.ndarray:
    """marlin_utils.py:288-298."""
    if group_size < size_k and group_size != -1:
        out = s.reshape(-1, 64)[:, _SCALE_PERM]
    else:
        out = s.reshape(-1, 32)[:, _SCALE_PERM_SINGLE]
    return np.ascontiguousarray(out.reshape(-1, size_n))


def marlin_unpermute_scales(s: np.ndarray, size_k: int, size_n: int, group_size: int) -> np.ndarray:
    if group_size < size_k and group_size != -1:
        inv = np.argsort(_SCALE_PERM)
        out = s.reshape(-1, 64)[:, inv]
    else:
        inv = np.argsort(_SCALE_PERM_SINGLE)
        out = s.reshape(-1, 32)[:, inv]
    return np.ascontiguousarray(out.reshape(-1, size_n))


def marlin_permute_bias(b: np.ndarray) -> np.ndarray:
    """marlin_utils.py:301-305."""
    return np.ascontiguousarray(b.reshape(-1, 32)[:, _SCALE_PERM_SINGLE].reshape(b.shape))


def marlin_unpermute_bias(b: np.ndarray) -> np.ndarray:
    inv = np.argsort(_SCALE_PERM_SINGLE)
    return np.ascontiguousarray(b.reshape(-1, 32)[:, inv].reshape(b.shape))


def marlin_zero_points(zp: np.ndarray, num_groups: int, size_n: int, num_bits: int) -> np.ndarray:
    """Integer zero-points [G, N] -> int32 [G, N/pf]: 64-chunk scale
    permutation, then the per-pf interleave, then column packing
    (marlin_utils.py:326-346)."""
    il = _INTERLEAVE[num_bits]
    z = zp.reshape(-1, 64)[:, _SCALE_PERM]
    z = z.reshape(-1, len(il))[:, il].reshape(num_groups, size_n)
    return pack_cols(np.ascontiguousarray(z), num_bits)


def marlin_zero_points_unpack(zp_packed: np.ndarray, num_groups: int, size_n: int,
                              num_bits: int) -> np.ndarray:
    il = _INTERLEAVE[num_bits]
    z = unpack_cols(zp_packed, num_bits)
    z = z.reshape(-1, len(il))[:, np.argsort(il)].reshape(-1, 64)
    z = z[:, np.argsort(_SCALE_PERM)]
    return np.ascontiguousarray(z.reshape(num_groups, size_n))


def awq_to_marlin_zero_points(q_zp_packed: np.ndarray, num_groups: int, size_n: int,
                              num_bits: int) -> np.ndarray:
    """AWQ-packed zero-points [G, N/pf] -> Marlin zero-points
    (marlin_utils.py:349-370)."""
    zp = awq_unpack(q_zp_packed, num_bits)
    return marlin_zero_points(zp, num_groups, size_n, num_bits)


def sort_g_idx(g_idx: np.ndarray):
    """marlin_utils.py:273-275.  A stable sort is used here; callers that
    compare against a device run must hand the SAME sort indices to both
    sides (ties may be broken differently by other sorts)."""
    order = np.argsort(g_idx, kind="stable").astype(np.int32)
    return g_idx[order], order


# ---------------------------------------------------------------------------
# 16-bit float rounding helpers (numpy has no bfloat16)
# ---------------------------------------------------------------------------


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bfloat16, returned as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return rounded.view(np.float32)


def round_to_dtype(x: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "float16":
        return x.astype(np.float16).astype(np.float32)
    if dtype == "bfloat16":
        return round_to_bf16(x)
    raise ValueError(dtype)


# ---------------------------------------------------------------------------
# dequantise-then-matmul  (quant_utils.py:434-441 for w_ref;
# test_marlin_gemm.py:355 for the product)
# ---------------------------------------------------------------------------


def dequantize(q: np.ndarray, scales: np.ndarray, dtype: str, *, bias: int = 0,
               zeros: np.ndarray | None = None, g_idx: np.ndarray | None = None,
               group_size: int = -1) -> np.ndarray:
    """w[k, n] = dtype( dtype(q[k, n] - b) * s[g(k), n] ) as float32, with
    b = the type's bias (8 / 128) or zeros[g(k), n], and g(k) = g_idx[k] when
    given, else k // group_size (0 when group_size == -1)
    (quant_utils.py:434-441: ``(w_q - zp).to(orig_type) * w_s``)."""
    K, N = q.shape
    if g_idx is not None and g_idx.size:
        g = g_idx.astype(np.int64)
    elif group_size in (-1, K) or scales.shape[0] == 1:
        g = np.zeros(K, dtype=np.int64)
    else:
        g = np.arange(K, dtype=np.int64) // group_size
    centred = q.astype(np.int32) - (zeros[g, :].astype(np.int32) if zeros is not None else bias)
    w_int = round_to_dtype(centred.astype(np.float32), dtype)   # exact: |values| < 256
    s = round_to_dtype(scales.astype(np.float32), dtype)[g, :]
    return round_to_dtype(w_int * s, dtype)


def dequantize_zp_float(q: np.ndarray, scales: np.ndarray, zeros: np.ndarray, group_size: int,
                        dtype: str) -> np.ndarray:
    """HQQ-style float zero-points: w[k, n] = dtype( dtype(q[k, n] - zp[g, n]) * s[g, n] ), the
    arithmetic of the reference's test (tests/kernels/quantization/test_marlin_gemm.py:520-525:
    ``(b_flat - zp_flat) * s_flat`` in 16-bit tensors).  The CUDA kernels compute
    q * s - dtype(zp * s) with one fma (marlin_template.h:174-181,1235-1240); the two agree
    within the GEMM tolerance."""
    K = q.shape[0]
    g = np.arange(K, dtype=np.int64) // group_size
    z = round_to_dtype(zeros.astype(np.float32), dtype)[g, :]
    s = round_to_dtype(scales.astype(np.float32), dtype)[g, :]
    centred = round_to_dtype(q.astype(np.float32) - z, dtype)
    return round_to_dtype(centred * s, dtype)


def fp8_e4m3fn_decode(codes: np.ndarray) -> np.ndarray:
    """float8_e4m3fn bit patterns -> float32: sign, 4 exponent bits (bias 7), 3 mantissa bits, no
    infinities; exponent 0 is subnormal (m / 8 * 2^-6); 0x7f / 0xff are NaN."""
    c = codes.astype(np.uint32)
    sign = np.where(c & 0x80, -1.0, 1.0).astype(np.float32)
    e = ((c >> 3) & 0xF).astype(np.int32)
    m = (c & 0x7).astype(np.float32)
    mag = np.where(e == 0, m / 8.0 * 2.0 ** -6, (1.0 + m / 8.0) * np.exp2((e - 7).astype(np.float32)))
    out = (sign * mag).astype(np.float32)
    out[(c & 0x7F) == 0x7F] = np.nan
    return out


def fp8_fuse_exponent_bias(scales: np.ndarray, dtype: str) -> np.ndarray:
    """marlin_utils_fp8.py:26-37: the kernels move the fp8 exponent field into the 16-bit format
    without re-biasing; the factor 2^(bias16 - 7) rides on the scales (2^8 fp16, 2^120 bf16)."""
    factor = np.float32(2.0 ** 8) if dtype == "float16" else np.float32(2.0 ** 120)
    return round_to_dtype(scales.astype(np.float32) * factor, dtype)


def dequantize_fp8(codes: np.ndarray, scales: np.ndarray, group_size: int, dtype: str) -> np.ndarray:
    """w[k, n] = dtype( dtype(fp8 value) * s[g(k), n] ) (marlin_utils_fp8.py:325-334:
    ``fp8_weight.to(dtype) * repeated_scales``); `scales` without the fused exponent bias."""
    K = codes.shape[0]
    g = np.zeros(K, dtype=np.int64) if group_size in (-1, K) else np.arange(K) // group_size
    s = round_to_dtype(scales.astype(np.float32), dtype)[g, :]
    return round_to_dtype(fp8_e4m3fn_decode(codes) * s, dtype)


# ---- float4_e2m1f weights: NVFP4 (fp8-e4m3 scales per 16, one global scale) and MXFP4 (e8m0
# ---- scales per 32) --------------------------------------------------------------------------
FP4_E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def fp4_e2m1_decode(codes: np.ndarray) -> np.ndarray:
    """4-bit codes s e e m -> float32: exponent 0 is subnormal (m / 2), bias 1, no inf / NaN
    (the table the reference builds through float8 in marlin_utils_fp4.py:316-324)."""
    c = codes.astype(np.int64)
    mag = FP4_E2M1_VALUES[c & 7]
    return np.where(c & 8, -mag, mag).astype(np.float32)


def _fp4_scale_source_index(size_n: int) -> np.ndarray:
    """Where each byte of a processed row pair comes from.  The reference regroups two
    consecutive scale rows (groups 2 g', 2 g' + 1) of the 64-column-permuted matrix so that a
    thread's eight scales of both groups are 16 adjacent bytes, then swaps the middle two of
    every four (marlin_utils_fp4.py:41-50, 66-75).  Returns src[F] = rr * N + p0: byte F of the
    2 N-byte pair block holds element p0 of row rr of the pair."""
    F = np.arange(2 * size_n)
    swap = np.array([0, 2, 1, 3])
    L = (F & ~3) | swap[F & 3]
    c, rr, jj = L // 16, (L % 16) // 8, L % 8
    return rr * size_n + 8 * c + jj


def nvfp4_process_scales(s_perm: np.ndarray) -> np.ndarray:
    """Permuted scales [G, N] (non-negative, fp8-e4m3 representable) -> the byte matrix the
    kernel reads: regrouped (see _fp4_scale_source_index), each value as the high byte of
    (fp16(s * 2^7) bits << 1): five exponent bits and three mantissa bits
    (marlin_utils_fp4.py:52-62)."""
    G, N = s_perm.shape
    pairs = s_perm.astype(np.float32).reshape(G // 2, 2 * N)[:, _fp4_scale_source_index(N)]
    bits = (pairs * np.float32(128.0)).astype(np.float16).view(np.uint16)
    return ((bits >> 7) & 0xFF).astype(np.uint8).reshape(G, N)


def nvfp4_unprocess_scales(b: np.ndarray) -> np.ndarray:
    """Inverse of nvfp4_process_scales: byte matrix [G, N] -> permuted scales (float32)."""
    G, N = b.shape
    vals = (b.astype(np.uint16) << 7).view(np.float16).astype(np.float32) / np.float32(128.0)
    out = np.empty((G // 2, 2 * N), dtype=np.float32)
    out[:, _fp4_scale_source_index(N)] = vals.reshape(G // 2, 2 * N)
    return out.reshape(G, N)


def mxfp4_process_scales(e_perm: np.ndarray) -> np.ndarray:
    """Permuted e8m0 exponent bytes [G, N] -> regrouped bytes (marlin_utils_fp4.py:65-77)."""
    G, N = e_perm.shape
    return e_perm.reshape(G // 2, 2 * N)[:, _fp4_scale_source_index(N)].reshape(G, N).astype(np.uint8)


def mxfp4_unprocess_scales(b: np.ndarray) -> np.ndarray:
    """Regrouped e8m0 bytes -> permuted scale values 2^(e - 127) (float32)."""
    G, N = b.shape
    out = np.empty((G // 2, 2 * N), dtype=np.float32)
    out[:, _fp4_scale_source_index(N)] = np.exp2(b.astype(np.float32) - 127.0).reshape(G // 2, 2 * N)
    return out.reshape(G, N)


def nvfp4_process_global_scale(g: float, dtype: str) -> np.ndarray:
    """marlin_utils_fp4.py:80-90: the kernel leaves the fp4 exponent un-rebiased (2^-14 fp16,
    2^-126 bf16) and the scales carry 2^7; the global scale makes up for both."""
    bias = 14 if dtype == "float16" else 126
    return round_to_dtype(np.float32(g) * np.float32(2.0 ** (bias - 7)), dtype)


def nvfp4_unprocess_global_scale(g_processed: float, dtype: str) -> np.float32:
    bias = 14 if dtype == "float16" else 126
    return np.float32(np.float32(g_processed) * np.float32(2.0 ** (7 - bias)))


def dequantize_fp4(codes: np.ndarray, scales: np.ndarray, group_size: int, dtype: str,
                   global_scale=None) -> np.ndarray:
    """w[k, n] in the reference's order of roundings (marlin_utils_fp4.py:329-333, 375):
    dtype( dtype(fp4 * global) * s[g(k), n] ); without a global scale dtype(fp4 * s)."""
    K = codes.shape[0]
    g = np.arange(K) // group_size
    w = fp4_e2m1_decode(codes)
    if global_scale is not None:
        w = round_to_dtype(w * round_to_dtype(np.float32(global_scale), dtype), dtype)
    return round_to_dtype(w * round_to_dtype(scales.astype(np.float32), dtype)[g, :], dtype)


# ---- mixture of experts ---------------------------------------------------------------------
def moe_align_block_size(topk_ids: np.ndarray, block_size: int, num_experts: int):
    """tests/kernels/moe/test_moe_align_block_size.py:92-170 (the golden torch implementation of
    the reference's CUDA op): (token, slot) ids sorted by expert (stable), every expert's run
    padded with `numel` to a multiple of block_size; the expert of every block (0 for blocks
    past the end); the padded total."""
    flat = topk_ids.reshape(-1)
    numel = flat.size
    max_padded = numel + num_experts * (block_size - 1)
    sorted_ids = np.full(max_padded, numel, dtype=np.int32)
    expert_ids = np.zeros(-(-max_padded // block_size), dtype=np.int32)
    pos = blk = 0
    for e in range(num_experts):
        ids = np.nonzero(flat == e)[0]
        if ids.size == 0:
            continue
        sorted_ids[pos:pos + ids.size] = ids
        nb = -(-ids.size // block_size)
        expert_ids[blk:blk + nb] = e
        pos += nb * block_size
        blk += nb
    return sorted_ids, expert_ids, np.array([pos], dtype=np.int32)


def moe_marlin_gemm_ref(a: np.ndarray, w_experts, sorted_ids: np.ndarray, expert_ids: np.ndarray,
                        num_padded: int, topk_weights: np.ndarray | None, block_size: int,
                        top_k: int, size_m: int, bias_experts=None) -> np.ndarray:
    """moe_wna16_marlin_gemm as the kernel indexes it (marlin_moe_wna16/marlin_template.h:459-530,
    920-930, 1500-1550): block b of `block_size` sorted ids uses expert expert_ids[b] (-1:
    skipped); id < size_m * top_k reads row id // top_k of A and writes row id of the output
    (times topk_weights[id] if given).  fp32; rows never written are NaN."""
    n = w_experts[0].shape[1]
    out = np.full((size_m * top_k, n), np.nan, dtype=np.float32)
    for b in range(int(num_padded) // block_size):
        e = int(expert_ids[b])
        if e < 0:
            continue
        for i in sorted_ids[b * block_size:(b + 1) * block_size]:
            if i < size_m * top_k:
                v = a[i // top_k].astype(np.float32) @ w_experts[e].astype(np.float32)
                if bias_experts is not None:
                    v = v + bias_experts[e].astype(np.float32)
                out[i] = v * (np.float32(topk_weights[i]) if topk_weights is not None else np.float32(1))
    return out


def gemm_ref(a: np.ndarray, w: np.ndarray, bias: np.ndarray | None = None) -> np.ndarray:
    """fp32-accumulated product of 16-bit operands held as float32."""
    out = a.astype(np.float32) @ w.astype(np.float32)
    if bias is not None:
        out = out + bias.astype(np.float32)[None, :]
    return out


def marlin_gemm_ref(a: np.ndarray, b_q_weight: np.ndarray, b_scales: np.ndarray, *,
                    size_k: int, size_n: int, num_bits: int, dtype: str,
                    type_bias: int = 0, b_zeros: np.ndarray | None = None,
                    g_idx: np.ndarray | None = None, perm: np.ndarray | None = None,
                    b_bias: np.ndarray | None = None) -> np.ndarray:
    """Reference result of ``gptq_marlin_gemm`` computed from the SAME device
    tensors the op receives (Marlin-layout weights, permuted scales / zeros /
    bias, sorted g_idx and the sort permutation), by undoing the layouts and
    running dequantise-then-matmul in float32.

    With act-order the weights are stored in sorted-row order, so the product
    is sum_k' a[:, perm[k']] * w_sorted[k', :] with g_idx indexing sorted rows
    (gptq_marlin.cu:549-564, marlin_template.h:979-1045)."""
    q = marlin_unpack(b_q_weight, size_k, size_n, num_bits)
    num_groups = b_scales.shape[0]
    group_size = size_k // num_groups if num_groups > 1 else -1
    has_act_order = g_idx is not None and g_idx.size > 0
    # channel-wise permutation is used when there is a single group
    s = marlin_unpermute_scales(b_scales, size_k, size_n, group_size if num_groups > 1 else -1)
    zeros = None
    if b_zeros is not None and b_zeros.size:
        zeros = marlin_zero_points_unpack(b_zeros, num_groups, size_n, num_bits)
    w = dequantize(q, s, dtype, bias=type_bias, zeros=zeros,
                   g_idx=g_idx if has_act_order else None, group_size=group_size)
    a_used = a[:, perm.astype(np.int64)] if has_act_order else a
    bias = marlin_unpermute_bias(b_bias) if b_bias is not None else None
    return gemm_ref(a_used, w, bias)


def permute_cols(a: np.ndarray, perm: np.ndarray) -> np.ndarray:
    """csrc/permute_cols.cu:14-88: out[m, k] = a[m, perm[k]]."""
    return a[:, perm.astype(np.int64)]


def algorithmic_bytes(size_m: int, size_n: int, size_k: int, num_bits: int,
                      num_groups: int, has_zp: bool, has_act_order: bool) -> int:
    """Bytes one GEMM call must move: packed weights + scales (+ zero-points)
    (+ g_idx and perm) + activations + output, 16-bit floats."""
    b = size_k * size_n * num_bits // 8 + num_groups * size_n * 2
    if has_zp:
        b += num_groups * size_n * num_bits // 8
    if has_act_order:
        b += 2 * size_k * 4
    return b + 2 * size_m * size_k + 2 * size_m * size_n
