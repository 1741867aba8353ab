"""torch.library.opcheck on the operators registered from C++ (schema, fake kernel and
autograd registration consistency), as the reference does for each of its ops
(tests/kernels/utils.py:1300 `opcheck`, used at tests/kernels/quantization/
test_marlin_gemm.py:141,196,310,419 and tests/kernels/core/test_permute_cols.py)."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu

# what the reference's helper runs by default; the autograd tests do not apply to these
# inference-only ops
CHECKS = ("test_schema", "test_autograd_registration", "test_faketensor")


@pytest.fixture(scope="module")
def env():
    import torch

    from tests import gpu_utils as G
    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import marlin_utils as mu
    return torch, G, ops, mu, getattr(torch.ops, ops.ops_namespace())


def test_opcheck_repack_and_permute(env):
    torch, G, ops, mu, ns = env
    K, N = 256, 128
    L = H.make_layer(K, N, "uint4b8", 64, True, "float16")
    torch.library.opcheck(ns.gptq_marlin_repack,
                          (G.ti32(L.gptq_qweight), G.ti32(L.sort_idx), K, N, 4), test_utils=CHECKS)
    torch.library.opcheck(ns.gptq_marlin_repack,
                          (G.ti32(L.gptq_qweight), G.ti32(None), K, N, 4), test_utils=CHECKS)
    torch.library.opcheck(ns.awq_marlin_repack, (G.ti32(L.awq_qweight), K, N, 4),
                          test_utils=CHECKS)
    a = torch.randn((5, K), dtype=torch.float16, device="cuda")
    torch.library.opcheck(ns.permute_cols, (a, G.ti32(L.sort_idx)), test_utils=CHECKS)


@pytest.mark.parametrize("m", [1, 48, 200])
def test_opcheck_gemm(env, m):
    """M = 1 takes the decode kernel, 48 and 200 the tensor-core kernel."""
    torch, G, ops, mu, ns = env
    K, N = 512, 256
    L = H.make_layer(K, N, "uint4b8", 128, True, "bfloat16")
    a = torch.randn((m, K), dtype=torch.bfloat16, device="cuda")
    ws = mu.marlin_make_workspace_new(torch.device("cuda"))
    args = (a, None, G.ti32(L.marlin_q), None, G.t16(L.marlin_s, "bfloat16"), None, G.ti32(None),
            G.ti32(L.g_idx), G.ti32(L.sort_idx), ws, L.type_id, m, N, K, True, False, True, False)
    torch.library.opcheck(ns.gptq_marlin_gemm, args, test_utils=CHECKS)
    assert int(ws.abs().sum().item()) == 0


def test_cpp_checks_raise_like_the_reference(env):
    """The C++ checks turn into RuntimeError with the reference's messages."""
    torch, G, ops, mu, ns = env
    K, N = 512, 256
    L = H.make_layer(K, N, "uint4b8", 128, False, "float16")
    ws = mu.marlin_make_workspace_new(torch.device("cuda"))
    e = G.ti32(None)
    a = torch.randn((4, K), dtype=torch.float16, device="cuda")
    good = [a, None, G.ti32(L.marlin_q), None, G.t16(L.marlin_s, "float16"), None, e, e, e, ws,
            L.type_id, 4, N, K, True, False, True, False]
    bad = list(good)
    bad[12] = N + 64                                     # size_n does not match the weights
    with pytest.raises(RuntimeError, match="size_n"):
        ns.gptq_marlin_gemm(*bad)
    bad = list(good)
    bad[0] = a.float()                                   # unsupported activation dtype
    with pytest.raises(RuntimeError):
        ns.gptq_marlin_gemm(*bad)
    bad = list(good)
    bad[9] = ws[:8]                                      # workspace below the number of SMs
    with pytest.raises(RuntimeError, match="workspace"):
        ns.gptq_marlin_gemm(*bad)
    with pytest.raises(RuntimeError, match="num_bits"):
        ns.gptq_marlin_repack(G.ti32(L.gptq_qweight), e, K, N, 5)


def test_opcheck_moe_wna16_marlin_gemm():
    import torch
    from oracle import marlin_oracle as mo
    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import marlin_utils as mu
    from vllm_b200.scalar_type import scalar_types
    dev = torch.device("cuda")
    M, K, N, E, topk, bs = 6, 128, 64, 4, 2, 16
    rng = np.random.default_rng(0)
    topk_ids = np.stack([rng.permutation(E)[:topk] for _ in range(M)]).astype(np.int32)
    sorted_ids, expert_ids, num = mo.moe_align_block_size(topk_ids, bs, E)
    a = torch.randn((M, K), dtype=torch.float16, device=dev)
    q = torch.randint(-2**31, 2**31 - 1, (E, K // 16, N * 2), dtype=torch.int32, device=dev)
    s = torch.rand((E, 1, N), dtype=torch.float16, device=dev)
    args = (a, None, q, None, s, None, None, None, None, mu.marlin_make_workspace_new(dev),
            torch.from_numpy(sorted_ids).to(dev), torch.from_numpy(expert_ids).to(dev),
            torch.from_numpy(num).to(dev), torch.ones(M * topk, device=dev), bs, topk, False, False,
            scalar_types.uint4b8.id, M, N, K, True, False, True, False)
    op = getattr(torch.ops, ops._MOE_NS).moe_wna16_marlin_gemm.default
    torch.library.opcheck(op, args, test_utils=("test_schema", "test_autograd_registration", "test_faketensor"))
