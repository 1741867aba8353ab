"""The numpy oracle against the fixtures recorded from the reference's own
Python packers (tests/golden/make_golden.py).  Integer outputs must be
bit-exact."""
import glob
import os

import numpy as np
import pytest

from oracle import marlin_oracle as mo

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    return np.load(os.path.join(GOLDEN, name))


def _f16(bits, is_bf16):
    bits = np.asarray(bits, dtype=np.uint16)
    if is_bf16:
        return (bits.astype(np.uint32) << 16).view(np.float32)
    return bits.view(np.float16).astype(np.float32)


def test_scalar_type_ids_and_ranges():
    g = _load("scalar_types.npz")
    table = {"uint4b8": (4, False, 8), "uint4": (4, False, 0),
             "uint8b128": (8, False, 128), "uint8": (8, False, 0)}
    for name, sid, lo, hi, bits in zip(g["names"], g["ids"], g["mins"], g["maxs"], g["size_bits"]):
        mant, signed, bias = table[str(name)]
        assert mo.scalar_type_id(0, mant, signed, bias) == int(sid)
        assert mo.scalar_type_min_max(mant, signed, bias) == (int(lo), int(hi))
        assert mant == int(bits)
    # known answers held by the reference's tests/test_scalartype.py:13-17
    assert mo.scalar_type_min_max(4, False, 8) == (-8, 7)
    assert mo.scalar_type_min_max(8, False, 128) == (-128, 127)
    assert mo.scalar_type_min_max(4, False, 0) == (0, 15)
    assert mo.UINT4B8_ID == 1125899907892224
    assert mo.UINT4_ID == 1125899906843648
    assert mo.UINT8B128_ID == 1125899923621888


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "repack_*.npz"))))
def test_repack_matches_reference(path):
    g = np.load(path)
    bits = int(os.path.basename(path).split("_")[1][1:])
    q = g["q"]
    K, N = q.shape
    assert np.array_equal(mo.gptq_pack(q, bits), g["gptq_in"])
    assert np.array_equal(mo.awq_pack(q, bits), g["awq_in"])
    assert np.array_equal(mo.marlin_weights(q, bits), g["expect"])
    assert np.array_equal(mo.gptq_marlin_repack(g["gptq_in"], None, K, N, bits), g["expect"])
    assert np.array_equal(mo.gptq_marlin_repack(g["gptq_in"], np.empty(0, np.int32), K, N, bits), g["expect"])
    assert np.array_equal(mo.awq_marlin_repack(g["awq_in"], K, N, bits), g["expect"])
    assert np.array_equal(mo.gptq_marlin_repack(g["gptq_in"], g["sort_idx"], K, N, bits), g["expect_perm"])
    assert np.array_equal(mo.marlin_unpack(g["expect"], K, N, bits), q)
    # the flat permutation implied by marlin_tile_coords equals get_weight_perm
    rows, cols = mo.marlin_tile_coords(bits)
    flat = (cols // 16) * 256 + rows * 16 + (cols % 16)
    assert np.array_equal(flat.reshape(-1), g["weight_perm"])


def test_known_answer_tile():
    # a 16x64 tile with q[k, n] = (k*64 + n) % 16 repacks to words that start
    # with 0x88008800 (value recorded from the reference packer)
    k, n = np.meshgrid(np.arange(16), np.arange(64), indexing="ij")
    q = ((k * 64 + n) % 16).astype(np.int32)
    out = mo.marlin_weights(q, 4).view(np.uint32)
    assert [hex(v) for v in out[0, :4]] == ["0x88008800"] * 4


def test_scale_zero_bias_permutations():
    g = _load("perms.npz")
    K, N = 512, 256
    assert np.array_equal(mo.marlin_permute_scales(g["s_grouped"], K, N, 128), g["s_grouped_perm"])
    assert np.array_equal(mo.marlin_permute_scales(g["s_channel"], K, N, -1), g["s_channel_perm"])
    assert np.array_equal(mo.marlin_permute_scales(g["s_channel"], K, N, K), g["s_channel_perm_gk"])
    assert np.array_equal(mo.marlin_permute_bias(g["bias"]), g["bias_perm"])
    assert np.array_equal(mo.marlin_unpermute_scales(g["s_grouped_perm"], K, N, 128), g["s_grouped"])
    assert np.array_equal(mo.marlin_unpermute_scales(g["s_channel_perm"], K, N, -1), g["s_channel"])
    assert np.array_equal(mo.marlin_unpermute_bias(g["bias_perm"]), g["bias"])
    for bits in (4, 8):
        G = K // 128
        assert np.array_equal(mo.marlin_zero_points(g[f"zp{bits}"], G, N, bits), g[f"zp{bits}_marlin"])
        assert np.array_equal(mo.awq_pack(g[f"zp{bits}"], bits), g[f"zp{bits}_awq_in"])
        assert np.array_equal(mo.awq_to_marlin_zero_points(g[f"zp{bits}_awq_in"], G, N, bits),
                              g[f"zp{bits}_awq_marlin"])
        assert np.array_equal(mo.marlin_zero_points_unpack(g[f"zp{bits}_marlin"], G, N, bits), g[f"zp{bits}"])


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "gemm_*.npz"))))
def test_dequant_and_gemm_match_reference(path):
    g = np.load(path)
    is_bf16 = bool(g["is_bf16"])
    dtype = "bfloat16" if is_bf16 else "float16"
    M, K, N = int(g["M"]), int(g["K"]), int(g["N"])
    bits = int(g["size_bits"])
    a = _f16(g["a_bits"], is_bf16)
    w_ref = _f16(g["w_ref_bits"], is_bf16)
    s = _f16(g["marlin_s_bits"], is_bf16)
    type_bias = {mo.UINT4B8_ID: 8, mo.UINT8B128_ID: 128, mo.UINT4_ID: 0, mo.UINT8_ID: 0}[int(g["type_id"])]
    act = bool(g["act_order"])
    zeros = g["marlin_zp"] if "marlin_zp" in g.files else None
    g_idx = g["g_idx"] if act else None
    perm = g["sort_idx"] if act else None

    # the dequantised weights recovered from the Marlin tensors equal w_ref
    # (rows in sorted order for act-order)
    q = mo.marlin_unpack(g["marlin_q_w"], K, N, bits)
    G = s.shape[0]
    gs = K // G if G > 1 else -1
    s_lin = mo.marlin_unpermute_scales(s, K, N, gs)
    z_lin = mo.marlin_zero_points_unpack(zeros, G, N, bits) if zeros is not None else None
    w = mo.dequantize(q, s_lin, dtype, bias=type_bias, zeros=z_lin, g_idx=g_idx, group_size=gs)
    if act:
        # w_ref rows are in checkpoint (shuffled) order; sorted row k' is row perm[k']
        assert np.array_equal(w, w_ref[perm.astype(np.int64), :])
    else:
        assert np.array_equal(w, w_ref)

    out = mo.marlin_gemm_ref(a, g["marlin_q_w"], s, size_k=K, size_n=N, num_bits=bits, dtype=dtype,
                             type_bias=type_bias, b_zeros=zeros, g_idx=g_idx, perm=perm)
    ref = g["out_ref"]
    assert out.shape == (M, N)
    # same operands, fp32 accumulation in a different order only
    assert np.max(np.abs(out - ref)) <= 1e-4 * max(1.0, np.max(np.abs(ref)))


def test_bf16_rounding_helper():
    x = np.array([1.0, 1.00390625, 1.005859375, 3.1415926, -2.7182818, 65504.0], dtype=np.float32)
    import torch
    want = torch.from_numpy(x).bfloat16().float().numpy()
    assert np.array_equal(mo.round_to_bf16(x), want)


def test_hqq_float_zero_points_match_reference():
    """Float zero-points: packers, scale-layout permutation of the zero-points, and the
    dequantised weights / product of the reference's test formula."""
    g = _load("hqq_u4_g64_f16.npz")
    K, N, gs = int(g["K"]), int(g["N"]), int(g["group_size"])
    q = g["q"]
    assert np.array_equal(mo.gptq_pack(q, 4), g["gptq_in"])
    assert np.array_equal(mo.gptq_marlin_repack(g["gptq_in"], None, K, N, 4), g["marlin_q_w"])
    s, z = _f16(g["scale_bits"], False), _f16(g["zero_bits"], False)
    assert np.array_equal(mo.marlin_permute_scales(s, K, N, gs), _f16(g["marlin_s_bits"], False))
    assert np.array_equal(mo.marlin_permute_scales(z, K, N, gs), _f16(g["marlin_zp_bits"], False))
    w = mo.dequantize_zp_float(q, s, z, gs, "float16")
    assert np.array_equal(w, _f16(g["w_ref_bits"], False))
    out = mo.gemm_ref(_f16(g["a_bits"], False), w)
    assert np.allclose(out, g["out_ref"], rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("name", ["fp8_g128_bf16", "fp8_gm1_f16"])
def test_fp8_weights_match_reference(name):
    """float8_e4m3fn weights: decode table, packing, Marlin layout, fused-bias scales and the
    dequantised weights of the reference's marlin_quant_fp8_torch steps."""
    g = _load(name + ".npz")
    K, N, gs, bf = int(g["K"]), int(g["N"]), int(g["group_size"]), bool(g["is_bf16"])
    dtype = "bfloat16" if bf else "float16"
    codes = g["codes"]
    assert np.array_equal(mo.pack_rows(codes.astype(np.int32), 8), g["packed"])
    assert np.array_equal(mo.marlin_weights(codes.astype(np.int32), 8), g["marlin_q_w"])
    assert np.array_equal(mo.gptq_marlin_repack(g["packed"], None, K, N, 8), g["marlin_q_w"])
    s = _f16(g["scales_bits"], bf)
    fused = mo.fp8_fuse_exponent_bias(mo.marlin_permute_scales(s, K, N, gs), dtype)
    assert np.array_equal(fused, _f16(g["marlin_s_bits"], bf))
    w = mo.dequantize_fp8(codes, s, gs, dtype)
    assert np.array_equal(w, _f16(g["w_ref_bits"], bf))
    out = mo.gemm_ref(_f16(g["a_bits"], bf), w)
    assert np.allclose(out, g["out_ref"], rtol=1e-5, atol=1e-4)


def test_fp8_decode_known_values():
    c = np.array([0x00, 0x01, 0x07, 0x08, 0x38, 0x7E, 0x80, 0xB8, 0xFE], dtype=np.uint8)
    want = [0.0, 2.0 ** -9, 7 * 2.0 ** -9, 2.0 ** -6, 1.0, 448.0, -0.0, -1.0, -448.0]
    assert mo.fp8_e4m3fn_decode(c).tolist() == want
    assert np.isnan(mo.fp8_e4m3fn_decode(np.array([0x7F, 0xFF], dtype=np.uint8))).all()


@pytest.mark.parametrize("name", ["nvfp4_g16_f16", "nvfp4_g16_bf16", "mxfp4_g32_bf16"])
def test_fp4_weights_match_reference(name):
    """float4_e2m1f weights (NVFP4 / MXFP4): Marlin words, the processed scale bytes and global
    scale decoded back to values, and the dequantised weights of the reference's
    rand_marlin_weight_nvfp4_like / _mxfp4_like; the forward transforms reproduce the bytes."""
    g = _load(name + ".npz")
    K, N, gs, bf = int(g["K"]), int(g["N"]), int(g["group_size"]), bool(g["is_bf16"])
    nv = bool(g["is_nvfp4"])
    dtype = "bfloat16" if bf else "float16"
    codes = g["codes"]
    assert np.array_equal(mo.marlin_weights(codes.astype(np.int32), 4), g["marlin_q_w"])
    b = g["marlin_s_bytes"]
    assert b.shape == (K // gs, N)
    if nv:
        s = mo.marlin_unpermute_scales(mo.nvfp4_unprocess_scales(b), K, N, gs)
        gl = mo.nvfp4_unprocess_global_scale(_f16(g["global_scale_bits"], bf)[0], dtype)
        w = mo.dequantize_fp4(codes, s, gs, dtype, global_scale=gl)
        assert np.array_equal(mo.nvfp4_process_scales(mo.marlin_permute_scales(s, K, N, gs)), b)
        assert float(np.ravel(mo.nvfp4_process_global_scale(gl, dtype))[0]) == float(_f16(g["global_scale_bits"], bf)[0])
    else:
        s = mo.marlin_unpermute_scales(mo.mxfp4_unprocess_scales(b), K, N, gs)
        w = mo.dequantize_fp4(codes, s, gs, dtype)
        e = np.round(np.log2(mo.marlin_permute_scales(s, K, N, gs))).astype(np.int64) + 127
        assert np.array_equal(mo.mxfp4_process_scales(e.astype(np.uint8)), b)
    assert np.array_equal(w, _f16(g["w_ref_bits"], bf))
    out = mo.gemm_ref(_f16(g["a_bits"], bf), w)
    assert np.allclose(out, g["out_ref"], rtol=1e-5, atol=1e-4)


def test_fp4_decode_table():
    c = np.arange(16, dtype=np.uint8)
    want = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    assert mo.fp4_e2m1_decode(c).tolist() == want


def test_moe_align_block_size_matches_reference():
    """The oracle's moe_align_block_size against the reference's golden torch implementation."""
    g = _load("moe_align.npz")
    for i in range(int(g["cases"])):
        m, topk, e, bs = (int(x) for x in g[f"cfg_{i}"])
        s, ex, n = mo.moe_align_block_size(g[f"topk_ids_{i}"], bs, e)
        assert int(n[0]) == int(g[f"num_{i}"].reshape(-1)[0]), i
        assert np.array_equal(s, g[f"sorted_{i}"]), i
        assert np.array_equal(ex, g[f"experts_{i}"]), i
