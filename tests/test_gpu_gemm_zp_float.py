"""gptq_marlin_gemm with float zero-points (HQQ: uint4 codes, fp16 scales and zero-points in
the scales' layout, group 64), as tests/kernels/quantization/test_marlin_gemm.py:463-534 runs
it.  Golden inputs from the reference's Python plus random shapes against the oracle."""
import os

import numpy as np
import pytest

from oracle import marlin_oracle as mo
from tests import gpu_utils as G
from tests import helpers as H

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _run(a, marlin_q, marlin_s, marlin_zp, M, N, K):
    import torch
    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import marlin_utils as mu
    from vllm_b200.scalar_type import scalar_types
    dev = torch.device("cuda")
    empty = torch.empty(0, dtype=torch.int32, device=dev)
    ws = mu.marlin_make_workspace_new(dev)
    out = ops.gptq_marlin_gemm(
        G.t16(a, "float16"), None, G.ti32(marlin_q), None, G.t16(marlin_s, "float16"), None,
        G.t16(marlin_zp, "float16"), empty, empty, ws, scalar_types.uint4, M, N, K,
        is_k_full=True, use_atomic_add=False, use_fp32_reduce=True, is_zp_float=True)
    torch.cuda.synchronize()
    assert int(ws.abs().sum().item()) == 0
    return G.n16(out)


def test_golden_inputs():
    g = np.load(os.path.join(GOLDEN, "hqq_u4_g64_f16.npz"))
    f16 = lambda b: np.asarray(b, dtype=np.uint16).view(np.float16).astype(np.float32)
    M, K, N = int(g["M"]), int(g["K"]), int(g["N"])
    got = _run(f16(g["a_bits"]), g["marlin_q_w"], f16(g["marlin_s_bits"]), f16(g["marlin_zp_bits"]),
               M, N, K)
    mf, mr = H.gemm_errors(got, g["out_ref"])
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL, (mf, mr)


@pytest.mark.parametrize("M,K,N", [(1, 128, 64), (13, 256, 192), (33, 512, 128), (64, 256, 64),
                                   (100, 1024, 256), (257, 128, 128)])
def test_random_shapes(M, K, N):
    gs = 64
    rng = np.random.default_rng(M * 7 + K + N)
    q = rng.integers(0, 10, size=(K, N), dtype=np.int32)        # the reference test draws codes in [0, 10)
    s = mo.round_to_dtype(rng.standard_normal((K // gs, N)).astype(np.float32), "float16")
    z = mo.round_to_dtype(rng.standard_normal((K // gs, N)).astype(np.float32), "float16")
    a = mo.round_to_dtype(rng.standard_normal((M, K)).astype(np.float32), "float16")
    w = mo.dequantize_zp_float(q, s, z, gs, "float16")
    got = _run(a, mo.marlin_weights(q, 4), mo.marlin_permute_scales(s, K, N, gs),
               mo.marlin_permute_scales(z, K, N, gs), M, N, K)
    mf, mr = H.gemm_errors(got, mo.gemm_ref(a, w))
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL, (mf, mr)


def test_needs_float16():
    import torch
    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import marlin_utils as mu
    from vllm_b200.scalar_type import scalar_types
    dev = torch.device("cuda")
    K, N = 128, 64
    empty = torch.empty(0, dtype=torch.int32, device=dev)
    with pytest.raises(RuntimeError, match="float16"):
        ops.gptq_marlin_gemm(
            torch.zeros((1, K), dtype=torch.bfloat16, device=dev), None,
            torch.zeros((K // 16, N * 2), dtype=torch.int32, device=dev), None,
            torch.ones((K // 64, N), dtype=torch.bfloat16, device=dev), None,
            torch.ones((K // 64, N), dtype=torch.bfloat16, device=dev), empty, empty,
            mu.marlin_make_workspace_new(dev), scalar_types.uint4, 1, N, K, is_zp_float=True)
