"""gptq_marlin_gemm with float8_e4m3fn weights (W8A16-fp8: 8-bit Marlin layout, scales carrying
the exponent re-bias factor), the op contract of marlin_utils_fp8.py:40-90.  Golden inputs from
the reference's Python, every finite code value, and random shapes against the oracle."""
import os

import numpy as np
import pytest

from oracle import marlin_oracle as mo
from tests import gpu_utils as G
from tests import helpers as H

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _run(a, marlin_q, marlin_s, M, N, K, dtype):
    import torch
    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import marlin_utils as mu
    from vllm_b200.scalar_type import scalar_types
    dev = torch.device("cuda")
    empty = torch.empty(0, dtype=torch.int32, device=dev)
    ws = mu.marlin_make_workspace_new(dev)
    out = ops.gptq_marlin_gemm(
        G.t16(a, dtype), None, G.ti32(marlin_q), None, G.t16(marlin_s, dtype), None, empty, empty,
        empty, ws, scalar_types.float8_e4m3fn, M, N, K, is_k_full=True, use_atomic_add=False,
        use_fp32_reduce=True, is_zp_float=False)
    torch.cuda.synchronize()
    assert int(ws.abs().sum().item()) == 0
    return G.n16(out)


def _bits(b, bf):
    b = np.asarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32) if bf else b.view(np.float16).astype(np.float32)


@pytest.mark.parametrize("name", ["fp8_g128_bf16", "fp8_gm1_f16"])
def test_golden_inputs(name):
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    bf = bool(g["is_bf16"])
    dtype = "bfloat16" if bf else "float16"
    M, K, N = int(g["M"]), int(g["K"]), int(g["N"])
    got = _run(_bits(g["a_bits"], bf), g["marlin_q_w"], _bits(g["marlin_s_bits"], bf), M, N, K, dtype)
    mf, mr = H.gemm_errors(got, g["out_ref"])
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL, (mf, mr)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("gs", [-1, 128])
def test_every_code_value_is_exact(dtype, gs):
    """A one-hot activation row picks single weights: with unit scales every finite fp8 value
    (subnormals included) must come out exactly."""
    K, N = 256, 64
    codes = np.zeros((K, N), dtype=np.uint8)
    vals = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=np.uint8)   # 254 finite codes
    codes[:vals.size, 0] = vals
    codes[:, 1:] = 0x38                                                             # 1.0 elsewhere
    groups = 1 if gs == -1 else K // gs
    s = np.ones((groups, N), dtype=np.float32)
    a = np.zeros((vals.size, K), dtype=np.float32)
    a[np.arange(vals.size), np.arange(vals.size)] = 1.0
    got = _run(a, mo.marlin_weights(codes.astype(np.int32), 8),
               mo.fp8_fuse_exponent_bias(mo.marlin_permute_scales(s, K, N, gs), dtype),
               vals.size, N, K, dtype)
    assert np.array_equal(got[:, 0], mo.fp8_e4m3fn_decode(vals))
    assert np.array_equal(got[:, 1], np.ones(vals.size, dtype=np.float32))


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("M,K,N,gs", [(1, 128, 64, -1), (16, 256, 192, 128), (40, 512, 128, 128),
                                      (64, 256, 64, -1), (130, 1024, 256, 128)])
def test_random_shapes(dtype, M, K, N, gs):
    rng = np.random.default_rng(M + K + N)
    codes = rng.integers(0, 256, size=(K, N)).astype(np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x30
    groups = 1 if gs == -1 else K // gs
    s = mo.round_to_dtype(rng.uniform(0.002, 0.02, size=(groups, N)).astype(np.float32), dtype)
    a = mo.round_to_dtype(rng.standard_normal((M, K)).astype(np.float32), dtype)
    w = mo.dequantize_fp8(codes, s, gs, dtype)
    got = _run(a, mo.marlin_weights(codes.astype(np.int32), 8),
               mo.fp8_fuse_exponent_bias(mo.marlin_permute_scales(s, K, N, gs), dtype), M, N, K, dtype)
    mf, mr = H.gemm_errors(got, mo.gemm_ref(a, w))
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL, (mf, mr)


@pytest.mark.parametrize("dtype_name,gs", [("bfloat16", 128), ("float16", -1)])
def test_host_helpers_end_to_end(dtype_name, gs):
    """marlin_quant_fp8_torch (device repack) + apply_fp8_marlin_linear against a @ weight_ref,
    and prepare_fp8_layer_for_marlin from an fp8 checkpoint tensor."""
    import torch
    from vllm_b200 import marlin_utils as mu
    from vllm_b200 import marlin_utils_fp8 as f8
    dtype = getattr(torch, dtype_name)
    torch.manual_seed(3)
    N, K, M = 256, 512, 24
    w = torch.randn((N, K), dtype=dtype, device="cuda")
    a = torch.randn((M, K), dtype=dtype, device="cuda")
    w_ref, mq, ms = f8.marlin_quant_fp8_torch(w, gs)
    ws = mu.marlin_make_workspace_new(a.device)
    out = f8.apply_fp8_marlin_linear(a, mq, ms, ws, N, K, None)
    ref = a.float() @ w_ref.float()
    mf, mr = H.gemm_errors(out.float().cpu().numpy(), ref.cpu().numpy())
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL, (mf, mr)

    class Layer(torch.nn.Module):
        pass
    layer = Layer()
    layer.output_size_per_partition, layer.input_size_per_partition, layer.orig_dtype = N, K, dtype
    g = K if gs == -1 else gs
    scales = w.view(N, -1, g).abs().max(-1)[0] / 448                    # [N, K / g]
    layer.weight = torch.nn.Parameter((w / scales.repeat_interleave(g, 1)).to(torch.float8_e4m3fn),
                                      requires_grad=False)              # [N, K] checkpoint layout
    layer.weight_scale = torch.nn.Parameter(scales.float(), requires_grad=False)
    f8.prepare_fp8_layer_for_marlin(layer, size_k_first=False)
    assert torch.equal(layer.weight, mq) and torch.equal(layer.weight_scale, ms)
