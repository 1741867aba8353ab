"""gptq_marlin_gemm with float4_e2m1f weights: NVFP4 (float8_e4m3fn scales per 16 values + a
global scale) and MXFP4 (float8_e8m0fnu scales per 32), the op contract of
marlin_utils_fp4.py:93-133.  Golden inputs from the reference's Python, every code value, random
shapes through this package's own host preparation, and the reference's error messages."""
import os

import numpy as np
import pytest

from oracle import marlin_oracle as mo
from tests import gpu_utils as G
from tests import helpers as H

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _bits(b, bf):
    b = np.asarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32) if bf else b.view(np.float16).astype(np.float32)


def _run(a, marlin_q, s_bytes, global_scale, nv, M, N, K, dtype, bias=None):
    import torch
    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import marlin_utils as mu
    from vllm_b200.scalar_type import scalar_types
    dev = torch.device("cuda")
    ws = mu.marlin_make_workspace_new(dev)
    s = torch.from_numpy(np.ascontiguousarray(s_bytes)).to(dev)
    s = s.view(torch.float8_e4m3fn if nv else torch.float8_e8m0fnu)
    gs = G.t16(np.asarray([global_scale], dtype=np.float32), dtype) if nv else None
    out = ops.gptq_marlin_gemm(
        G.t16(a, dtype), None, G.ti32(marlin_q), None if bias is None else G.t16(bias, dtype), s, gs,
        None, None, None, ws, scalar_types.float4_e2m1f, M, N, K, is_k_full=True,
        use_atomic_add=False, use_fp32_reduce=True, is_zp_float=False)
    torch.cuda.synchronize()
    assert int(ws.abs().sum().item()) == 0
    return G.n16(out)


@pytest.mark.parametrize("name", ["nvfp4_g16_f16", "nvfp4_g16_bf16", "mxfp4_g32_bf16"])
def test_golden_inputs(name):
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    bf, nv = bool(g["is_bf16"]), bool(g["is_nvfp4"])
    dtype = "bfloat16" if bf else "float16"
    M, K, N = int(g["M"]), int(g["K"]), int(g["N"])
    gl = float(_bits(g["global_scale_bits"], bf)[0]) if nv else None
    got = _run(_bits(g["a_bits"], bf), g["marlin_q_w"], g["marlin_s_bytes"], gl, nv, M, N, K, dtype)
    mf, mr = H.gemm_errors(got, g["out_ref"])
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL, (mf, mr)


@pytest.mark.parametrize("kind,dtype", [("nv", "float16"), ("nv", "bfloat16"), ("mx", "bfloat16")])
def test_every_code_value_is_exact(kind, dtype):
    """A one-hot activation row picks single weights: with unit scales all sixteen codes must come
    out exactly, in every nibble position of a packed word."""
    nv = kind == "nv"
    gs = 16 if nv else 32
    K, N = 128, 64
    rng = np.random.default_rng(3)
    codes = rng.integers(0, 16, size=(K, N), dtype=np.int64)
    codes[:16, 0] = np.arange(16)
    q = mo.marlin_weights(codes.astype(np.int32), 4)
    ones = np.ones((K // gs, N), dtype=np.float32)
    if nv:
        s_bytes = mo.nvfp4_process_scales(mo.marlin_permute_scales(ones, K, N, gs))
        gl = float(np.ravel(mo.nvfp4_process_global_scale(1.0, dtype))[0])
    else:
        s_bytes = mo.mxfp4_process_scales(np.full((K // gs, N), 127, dtype=np.uint8))
        gl = None
    a = np.eye(K, dtype=np.float32)[:64]                 # rows 0..63 pick k = 0..63
    got = _run(a, q, s_bytes, gl, nv, 64, N, K, dtype)
    assert np.array_equal(got, mo.fp4_e2m1_decode(codes[:64]))


CASES = [
    # M, K, N, kind, dtype
    (1, 128, 64, "nv", "float16"),
    (7, 256, 128, "nv", "bfloat16"),
    (16, 512, 256, "mx", "bfloat16"),
    (33, 1024, 192, "nv", "float16"),
    (64, 2048, 512, "mx", "bfloat16"),
    (100, 512, 320, "nv", "bfloat16"),
    (257, 4096, 1024, "nv", "float16"),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(map(str, c)))
def test_random_shapes_through_host_preparation(case):
    """rand_marlin_weight_*_like of this package (GPU repack operator, scale processing) ->
    operator -> product with the returned reference weights; the processed scale bytes agree with
    the oracle's transform."""
    import torch
    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import marlin_utils as mu
    from vllm_b200 import marlin_utils_fp4 as f4
    from vllm_b200.scalar_type import scalar_types
    M, K, N, kind, dtype = case
    td = torch.bfloat16 if dtype == "bfloat16" else torch.float16
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(M + K)
    weight = torch.randn((N, K), dtype=td, device=dev, generator=gen)
    a = torch.randn((M, K), dtype=td, device=dev, generator=gen)
    bias = torch.randn((N,), dtype=td, device=dev, generator=gen) if M % 2 else None
    if kind == "nv":
        w_ref, q, s, gs = f4.rand_marlin_weight_nvfp4_like(weight, 16)
    else:
        w_ref, q, s = f4.rand_marlin_weight_mxfp4_like(weight, 32)
        gs = None
    ws = mu.marlin_make_workspace_new(dev)
    out = ops.gptq_marlin_gemm(a, None, q, None if bias is None else mu.marlin_permute_bias(bias), s, gs,
                               None, None, None, ws, scalar_types.float4_e2m1f, M, N, K)
    torch.cuda.synchronize()
    ref = a.float() @ w_ref.float()
    if bias is not None:
        ref = ref + bias.float()
    mf, mr = H.gemm_errors(G.n16(out), ref.cpu().numpy())
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL, (case, mf, mr)
    # the bytes decode (oracle) to scales that reproduce the reference weights' groups
    b = s.contiguous().view(torch.uint8).cpu().numpy()
    again = mo.nvfp4_process_scales(mo.nvfp4_unprocess_scales(b)) if kind == "nv" else \
        mo.mxfp4_process_scales(np.round(np.log2(mo.mxfp4_unprocess_scales(b))).astype(np.int64).astype(np.uint8) + 127)
    assert np.array_equal(again, b)


def test_reference_error_messages():
    import torch
    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import marlin_utils as mu
    from vllm_b200.scalar_type import scalar_types
    dev = torch.device("cuda")
    M, K, N = 4, 128, 64
    a = torch.zeros((M, K), dtype=torch.float16, device=dev)
    q = torch.zeros((K // 16, N * 2), dtype=torch.int32, device=dev)
    ws = mu.marlin_make_workspace_new(dev)
    s_nv = torch.zeros((K // 16, N), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    s_mx = torch.zeros((K // 32, N), dtype=torch.uint8, device=dev).view(torch.float8_e8m0fnu)
    gs = torch.ones(1, dtype=torch.float16, device=dev)
    call = lambda s, g, x=a: ops.gptq_marlin_gemm(x, None, q, None, s, g, None, None, None, ws,
                                                  scalar_types.float4_e2m1f, M, N, K)
    with pytest.raises(RuntimeError, match="global_scale parameter must be passed for nvfp4"):
        call(s_nv, None)
    with pytest.raises(RuntimeError, match="global_scale can only be used for nvfp4"):
        call(s_mx, gs, a.to(torch.bfloat16))
    with pytest.raises(RuntimeError, match="bfloat16 activations"):
        call(s_mx, None)
    with pytest.raises(RuntimeError, match="float8_e4m3fn or float8_e8m0fnu"):
        call(torch.zeros((K // 16, N), dtype=torch.float16, device=dev), None)
    # global_scale with an integer weight type
    s16 = torch.ones((1, N), dtype=torch.float16, device=dev)
    with pytest.raises(RuntimeError, match="global_scale can only be used for nvfp4"):
        ops.gptq_marlin_gemm(a, None, q, None, s16, gs, None, None, None, ws, scalar_types.uint4b8, M, N, K)
