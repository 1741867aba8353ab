"""CPU tests of the host side: library loading / exported symbols, the torch
restatements of the permutation helpers against the oracle, parameter sharding,
and the layer bookkeeping of the quantized linear methods."""
import os
import re

import numpy as np
import pytest
import torch

from oracle import marlin_oracle as mo
from tests import helpers as H

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_exports_every_declared_symbol():
    from vllm_b200 import _lib
    lib = _lib.load()
    header = open(os.path.join(ROOT, "include", "b200q.h")).read()
    declared = set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", header)) - {"b200q_stream_t"}
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/b200q.h but not exported"
    assert set(_lib.EXPORTS) <= declared
    assert lib.b200q_version() >= 100
    # pure host query: no GPU needed
    assert lib.b200q_marlin_gemm_scratch_bytes(16, 4096, 4096, 0) > 0
    assert lib.b200q_marlin_gemm_scratch_bytes(16, 4096, 4096, 1) >= \
        lib.b200q_marlin_gemm_scratch_bytes(16, 4096, 4096, 0) + 16 * 4096 * 2


def test_ops_registered_with_reference_schemas():
    from vllm_b200 import _custom_ops as ops
    ns = getattr(torch.ops, ops.ops_namespace())
    schema = str(ns.gptq_marlin_gemm.default._schema)
    for piece in ("Tensor a", "Tensor? c_or_none", "Tensor b_q_weight", "Tensor? b_bias_or_none",
                  "Tensor b_scales", "Tensor? global_scale", "Tensor? b_zeros_or_none",
                  "Tensor? g_idx_or_none", "Tensor? perm_or_none", "Tensor workspace",
                  "int b_q_type", "SymInt size_m", "SymInt size_n", "SymInt size_k",
                  "bool is_k_full", "bool use_atomic_add", "bool use_fp32_reduce",
                  "bool is_zp_float"):
        assert piece in schema, (piece, schema)
    assert "SymInt size_k, SymInt size_n, int num_bits" in str(ns.gptq_marlin_repack.default._schema)
    assert "SymInt size_k, SymInt size_n, int num_bits" in str(ns.awq_marlin_repack.default._schema)
    # fake (meta) kernels give the output shapes
    with torch._subclasses.fake_tensor.FakeTensorMode():
        q = torch.empty((32, 128), dtype=torch.int32)
        out = ns.gptq_marlin_repack(q, torch.empty(0, dtype=torch.int32), 256, 128, 4)
        assert tuple(out.shape) == (16, 256)


def test_scalar_types():
    from vllm_b200.scalar_type import ScalarType, scalar_types
    assert scalar_types.uint4b8.id == mo.UINT4B8_ID and scalar_types.uint4.id == mo.UINT4_ID
    assert scalar_types.uint8b128.id == mo.UINT8B128_ID and scalar_types.uint8.id == mo.UINT8_ID
    assert (scalar_types.uint4b8.min(), scalar_types.uint4b8.max()) == (-8, 7)
    assert (scalar_types.uint8b128.min(), scalar_types.uint8b128.max()) == (-128, 127)
    assert (scalar_types.uint4.min(), scalar_types.uint4.max()) == (0, 15)
    assert ScalarType.from_id(mo.UINT8B128_ID) is scalar_types.uint8b128
    assert scalar_types.uint4b8.size_bits == 4 and str(scalar_types.uint4b8) == "uint4b8"
    # float8_e4m3fn: the id the reference's ScalarType.float_(4, 3, True, EXTD_RANGE_MAX_MIN) yields
    f8 = scalar_types.float8_e4m3fn
    assert f8.id == 2814749767172868 and f8.size_bits == 8 and f8.is_floating_point()
    assert ScalarType.from_id(f8.id) is f8 and str(f8) == "float8_e4m3fn"


def test_fp8_host_helpers_match_oracle():
    from vllm_b200 import marlin_utils_fp8 as f8
    rng = np.random.default_rng(5)
    codes = rng.integers(0, 256, size=(64, 32)).astype(np.uint8)            # [K, N]
    t = torch.from_numpy(codes).view(torch.float8_e4m3fn)
    assert np.array_equal(f8.pack_fp8_to_int32(t, True).numpy(), mo.pack_rows(codes.astype(np.int32), 8))
    assert np.array_equal(f8.pack_fp8_to_int32(t.T.contiguous(), False).T.numpy(),
                          mo.pack_rows(codes.astype(np.int32), 8))
    for dt, name in ((torch.float16, "float16"), (torch.bfloat16, "bfloat16")):
        s = torch.from_numpy(rng.uniform(0.002, 0.02, size=(2, 32)).astype(np.float32)).to(dt)
        got = f8.fp8_fused_exponent_bias_into_scales(s).float().numpy()
        assert np.array_equal(got, mo.fp8_fuse_exponent_bias(s.float().numpy(), name))
    finite = codes[(codes & 0x7F) != 0x7F]
    assert np.array_equal(torch.from_numpy(finite).view(torch.float8_e4m3fn).float().numpy(),
                          mo.fp8_e4m3fn_decode(finite))


def test_torch_permutations_match_oracle():
    from vllm_b200 import marlin_utils as mu
    rng = np.random.default_rng(3)
    K, N = 512, 256
    s = torch.from_numpy(rng.random((K // 128, N), dtype=np.float32)).half()
    assert np.array_equal(mu.marlin_permute_scales(s, K, N, 128).numpy(),
                          mo.marlin_permute_scales(s.numpy(), K, N, 128))
    s1 = s[:1].contiguous()
    assert np.array_equal(mu.marlin_permute_scales(s1, K, N, -1).numpy(),
                          mo.marlin_permute_scales(s1.numpy(), K, N, -1))
    b = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).half()
    assert np.array_equal(mu.marlin_permute_bias(b).numpy(), mo.marlin_permute_bias(b.numpy()))
    for bits in (4, 8):
        G = K // 128
        zp = torch.from_numpy(rng.integers(0, 1 << bits, size=(G, N), dtype=np.int32))
        assert np.array_equal(mu.marlin_zero_points(zp, G, N, bits).numpy(),
                              mo.marlin_zero_points(zp.numpy(), G, N, bits))
        packed = mu.pack_cols(zp, bits, G, N)
        assert np.array_equal(packed.numpy(), mo.pack_cols(zp.numpy(), bits))
        assert torch.equal(mu.unpack_cols(packed, bits, G, N), zp)
        awq = torch.from_numpy(mo.awq_pack(zp.numpy(), bits))
        assert np.array_equal(mu.awq_to_marlin_zero_points(awq, G, N, bits).numpy(),
                              mo.awq_to_marlin_zero_points(awq.numpy(), G, N, bits))
    g_idx = torch.from_numpy((np.arange(K) // 128)[rng.permutation(K)].astype(np.int32))
    sorted_g, order = mu.marlin_sort_g_idx(g_idx)
    assert torch.equal(sorted_g, g_idx[order.long()]) and bool((sorted_g[1:] >= sorted_g[:-1]).all())


def test_support_checks_and_helpers():
    from vllm_b200 import marlin_utils as mu
    from vllm_b200.scalar_type import scalar_types
    assert mu.marlin_is_k_full(False, True) and mu.marlin_is_k_full(True, False)
    assert not mu.marlin_is_k_full(True, True)
    assert mu.marlin_repeat_scales_on_all_ranks(True, 128, False)
    assert mu.marlin_repeat_scales_on_all_ranks(False, -1, True)
    assert not mu.marlin_repeat_scales_on_all_ranks(False, 128, True)
    assert mu.check_marlin_supports_shape(4096, 4096, 4096, 128) == (True, None)
    assert not mu.check_marlin_supports_shape(4096 + 32, 4096, 4096, 128)[0]
    assert not mu.check_marlin_supports_shape(4096, 4096 + 64, 4096 + 64, 128)[0]
    with pytest.raises(ValueError):
        mu.verify_marlin_supports_shape(4096, 1792 + 64, 14336, 128)
    assert mu.check_marlin_supported(scalar_types.uint4b8, 128, device_capability=100)
    assert not mu.check_marlin_supported(scalar_types.uint4b8, 16, device_capability=100)
    assert mu.query_marlin_supported_quant_types(True, device_capability=100) == [scalar_types.uint4]
    assert mu.query_marlin_supported_quant_types(False, device_capability=90) == []
    assert not mu.should_use_atomic_add_reduce(16, 4096, 4096, torch.device("cuda"), torch.float16)


def test_parameter_sharding():
    from vllm_b200.parameter import ShardedParameter, permute_param_layout_
    full = torch.arange(32 * 24, dtype=torch.int32).reshape(32, 24)
    # packed along dim 0 by 8: 32 packed rows == 256 unpacked; output dim 1
    p = ShardedParameter(torch.empty(16, 24, dtype=torch.int32), input_dim=0, output_dim=1,
                         packed_dim=0, packed_factor=8)
    p.load_row_parallel_weight(full, tp_rank=1, tp_size=2)
    assert torch.equal(p.data, full[16:32])
    p = ShardedParameter(torch.empty(32, 12, dtype=torch.int32), input_dim=0, output_dim=1)
    p.load_column_parallel_weight(full, tp_rank=1, tp_size=2)
    assert torch.equal(p.data, full[:, 12:])
    # merged: two logical matrices of 16 and 8 output columns, this rank holds 8 + 4
    p = ShardedParameter(torch.zeros(32, 12, dtype=torch.int32), input_dim=0, output_dim=1)
    p.load_merged_column_weight(full[:, :16], 0, 8, tp_rank=1, tp_size=2)
    p.load_merged_column_weight(full[:, 16:], 8, 4, tp_rank=1, tp_size=2)
    assert torch.equal(p.data, torch.cat([full[:, 8:16], full[:, 20:24]], dim=1))
    # packed output dim (AWQ-style): offsets given in unpacked columns
    p = ShardedParameter(torch.zeros(4, 6, dtype=torch.int32), input_dim=0, output_dim=1,
                         packed_dim=1, packed_factor=8)
    loaded = torch.arange(4 * 8, dtype=torch.int32).reshape(4, 8)    # 64 unpacked columns
    p.load_merged_column_weight(loaded, shard_offset=16, shard_size=32, tp_rank=1, tp_size=2)
    assert torch.equal(p.data[:, 2:6], loaded[:, 4:8]) and int(p.data[:, :2].abs().sum()) == 0
    # replicated parameter (no input dim) is copied whole
    p = ShardedParameter(torch.empty(4, 24, dtype=torch.int32), input_dim=None, output_dim=1)
    p.load_row_parallel_weight(full[:4], tp_rank=1, tp_size=2)
    assert torch.equal(p.data, full[:4])
    # layout permutation
    p = ShardedParameter(torch.arange(6).reshape(2, 3).clone(), input_dim=1, output_dim=0,
                         packed_dim=1, packed_factor=8)
    permute_param_layout_(p, input_dim=0, output_dim=1, packed_dim=0)
    assert tuple(p.data.shape) == (3, 2) and p.packed_dim == 0


def test_gptq_layer_parameter_shapes():
    from vllm_b200.linear import ColumnParallelLinear, QKVParallelLinear, RowParallelLinear
    from vllm_b200.quantization import AWQMarlinConfig, GPTQMarlinConfig
    qc = GPTQMarlinConfig(4, 128, desc_act=True)
    col = ColumnParallelLinear(4096, 28672, quant_config=qc, params_dtype=torch.bfloat16,
                               tp_rank=3, tp_size=8, device="meta")
    assert tuple(col.qweight.shape) == (512, 3584) and tuple(col.scales.shape) == (32, 3584)
    assert tuple(col.g_idx.shape) == (4096,)
    row = RowParallelLinear(14336, 4096, quant_config=qc, params_dtype=torch.bfloat16,
                            tp_rank=3, tp_size=8, device="meta")
    # act-order + row-parallel: scales replicated (all 112 groups), K sharded
    assert tuple(row.qweight.shape) == (1792 // 8, 4096) and tuple(row.scales.shape) == (112, 4096)
    assert row.scales.input_dim is None and tuple(row.g_idx.shape) == (1792,)
    qc2 = GPTQMarlinConfig(4, 128, desc_act=False)
    row2 = RowParallelLinear(14336, 4096, quant_config=qc2, params_dtype=torch.bfloat16,
                             tp_rank=0, tp_size=8, device="meta")
    assert tuple(row2.scales.shape) == (14, 4096) and row2.scales.input_dim == 0
    qkv = QKVParallelLinear(4096, 128, 32, 8, quant_config=qc2, params_dtype=torch.bfloat16,
                            tp_rank=0, tp_size=8, device="meta")
    assert qkv.output_partition_sizes == [512, 128, 128] and tuple(qkv.qweight.shape) == (512, 768)
    awq = AWQMarlinConfig(4, 128)
    a = ColumnParallelLinear(3584, 37888, quant_config=awq, params_dtype=torch.float16,
                             tp_rank=0, tp_size=1, device="meta")
    assert tuple(a.qweight.shape) == (3584, 37888 // 8) and tuple(a.qzeros.shape) == (28, 37888 // 8)
    with pytest.raises(ValueError):
        RowParallelLinear(14336 + 128, 4096, quant_config=qc2, tp_rank=0, tp_size=8, device="meta")
    with pytest.raises(ValueError):
        GPTQMarlinConfig(3, 128, False)
    assert GPTQMarlinConfig(4, -1, desc_act=True).desc_act is False


def test_fp4_scale_processing_matches_reference_bytes():
    """This package's nvfp4 / mxfp4 scale and global-scale transforms (torch, CPU) reproduce the
    bytes the reference's functions produced for the golden fixtures."""
    import os
    import torch
    from oracle import marlin_oracle as mo
    from vllm_b200 import marlin_utils_fp4 as f4
    golden = os.path.join(os.path.dirname(__file__), "golden")
    for name in ("nvfp4_g16_f16", "nvfp4_g16_bf16", "mxfp4_g32_bf16"):
        g = np.load(os.path.join(golden, name + ".npz"))
        bf, nv = bool(g["is_bf16"]), bool(g["is_nvfp4"])
        td = torch.bfloat16 if bf else torch.float16
        b = g["marlin_s_bytes"]
        if nv:
            s_perm = torch.from_numpy(mo.nvfp4_unprocess_scales(b)).to(td)
            got = f4.nvfp4_marlin_process_scales(s_perm).view(torch.uint8).numpy()
            bits = np.asarray(g["global_scale_bits"], dtype=np.uint16)
            gp = (bits.astype(np.uint32) << 16).view(np.float32) if bf else bits.view(np.float16).astype(np.float32)
            gl = mo.nvfp4_unprocess_global_scale(gp[0], "bfloat16" if bf else "float16")
            again = f4.nvfp4_marlin_process_global_scale(torch.tensor(float(gl), dtype=td))
            assert float(again) == float(gp[0])
        else:
            s_perm = torch.from_numpy(mo.mxfp4_unprocess_scales(b)).to(td)
            got = f4.mxfp4_marlin_process_scales(s_perm).view(torch.uint8).numpy()
        assert np.array_equal(got, b), name


def test_moe_align_block_size_torch_matches_reference_golden():
    """This package's device-side moe_align_block_size (torch ops, here on CPU tensors) against the
    outputs of the reference's golden implementation."""
    import os
    from vllm_b200 import fused_moe
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "moe_align.npz"))
    for i in range(int(g["cases"])):
        m, topk, e, bs = (int(x) for x in g[f"cfg_{i}"])
        s, ex, n = fused_moe.moe_align_block_size(torch.from_numpy(g[f"topk_ids_{i}"]), bs, e)
        assert int(n[0]) == int(g[f"num_{i}"].reshape(-1)[0]), i
        assert np.array_equal(s.numpy(), g[f"sorted_{i}"]), i
        assert np.array_equal(ex.numpy(), g[f"experts_{i}"]), i
