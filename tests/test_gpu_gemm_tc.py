"""GPU parity of the tensor-core (tcgen05) path of gptq_marlin_gemm, M > 64:
ragged M and N tails, every weight type, group sizes, act-order, bias, strided
A, and a full-size Llama-3-8B layer checked through linearity (a size-independent
property) plus an oracle-checked corner."""
import numpy as np
import pytest

from oracle import marlin_oracle as mo
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_utils as G
    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import _lib
    from vllm_b200 import marlin_utils as mu
    assert torch.cuda.is_available()
    return torch, G, ops, mu, _lib.load()


def _check(out, ref, what=""):
    max_frac, mean_rel = H.gemm_errors(out, ref)
    assert max_frac <= H.MAX_ABS_FRAC and mean_rel <= H.MEAN_REL, (
        f"{what}: max-abs/max|ref| = {max_frac:.3e}, mean rel = {mean_rel:.3e}")


CASES = [
    # M, K, N, type, group, act_order, dtype
    (65, 64, 64, "uint4b8", -1, False, "float16"),
    (96, 128, 192, "uint4b8", 32, False, "bfloat16"),
    (127, 1024, 448, "uint4b8", 128, True, "bfloat16"),
    (129, 512, 256, "uint4", 64, False, "float16"),
    (255, 2048, 320, "uint4", 128, False, "bfloat16"),
    (256, 1024, 1024, "uint8b128", -1, False, "bfloat16"),
    (300, 1024, 576, "uint8b128", 128, True, "float16"),
    (513, 4096, 512, "uint4b8", 128, False, "float16"),
    (1024, 3584, 1152, "uint4", -1, False, "float16"),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(map(str, c)))
def test_tc_gemm(env, case):
    torch, G, ops, mu, lib = env
    M, K, N, qtype, group, act, dtype = case
    L = H.make_layer(K, N, qtype, group, act, dtype, with_bias=(M % 2 == 1))
    a = H.make_activations(M, K, dtype)
    out = G.run_gemm(ops, mu, L, a)
    assert lib.b200q_device_error(1) == 0, "a hand-off wait timed out in the tensor-core kernel"
    _check(out, mo.gemm_ref(a, L.w, L.bias), str(case))


def test_tc_gemm_strided_a(env):
    torch, G, ops, mu, lib = env
    M, K, N = 200, 1024, 2048
    L = H.make_layer(K, N, "uint4b8", 128, False, "bfloat16")
    big = torch.randn((M + 16, 2 * K), dtype=torch.bfloat16, device="cuda")
    a = big[8:M + 8, 8:K + 8]
    out = G.run_gemm(ops, mu, L, None, a_tensor=a)
    assert lib.b200q_device_error(1) == 0
    _check(out, mo.gemm_ref(G.n16(a), L.w), "strided A")


def test_tc_gemm_full_size_linearity(env):
    """Llama-3-8B gate_up at M = 4096: f(a1 + a2) == f(a1) + f(a2) up to 16-bit
    rounding of the outputs, f agrees with the decode-regime kernels on the first
    rows, and a corner agrees with the oracle."""
    torch, G, ops, mu, lib = env
    from vllm_b200.scalar_type import scalar_types
    M, K, N = 4096, 4096, 28672
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(5)
    q = torch.randint(-2**31, 2**31 - 1, (K // 16, N * 2), dtype=torch.int32, device=dev, generator=gen)
    s = (torch.rand((K // 128, N), device=dev, generator=gen) * 0.018 + 0.002).to(torch.bfloat16)
    ws = mu.marlin_make_workspace_new(torch.device(dev))
    e = torch.empty(0, dtype=torch.int32, device=dev)
    f = lambda a: ops.gptq_marlin_gemm(a, None, q, None, s, None, e, e, e, ws, scalar_types.uint4b8,
                                       a.shape[0], N, K, True, False, True, False)
    # integer-valued activations keep the sums of two inputs exact in bf16
    a1 = torch.randint(-3, 4, (M, K), device=dev, generator=gen).to(torch.bfloat16)
    a2 = torch.randint(-3, 4, (M, K), device=dev, generator=gen).to(torch.bfloat16)
    y1, y2, y12 = f(a1).float(), f(a2).float(), f(a1 + a2).float()
    torch.cuda.synchronize()
    assert lib.b200q_device_error(1) == 0
    scale = y12.abs().max().item()
    assert (y12 - (y1 + y2)).abs().max().item() <= 2e-2 * scale
    small = f(a1[:16].contiguous()).float()        # decode kernel on the same rows
    assert (small - y1[:16]).abs().max().item() <= 2e-2 * scale
    # oracle on a corner: first 64 columns, 48 rows
    qn = q[:, :128].cpu().numpy()                  # first 64-column tile of every k-tile
    sn_perm = s[:, :64].float().cpu().numpy()
    w_codes = mo.marlin_unpack(np.ascontiguousarray(qn), K, 64, 4)
    s_lin = mo.marlin_unpermute_scales(sn_perm, K, 64, 128)
    w = mo.dequantize(w_codes, s_lin, "bfloat16", bias=8, group_size=128)
    ref = mo.gemm_ref(a1[:48].float().cpu().numpy(), w)
    _check(y1[:48, :64].cpu().numpy(), ref, "corner vs oracle")


def test_tc_gemm_many_tiles_per_cta(env):
    """M = 32768: ~100 tiles per CTA and an activation matrix larger than L2, so
    the producer is the slow role and stage barriers complete late — the regime in
    which a hand-off that skips barrier phases goes wrong.  Sampled rows must agree
    with the decode-regime kernel run on those rows alone."""
    torch, G, ops, mu, lib = env
    from vllm_b200.scalar_type import scalar_types
    M, K, N = 32768, 4096, 2048
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(11)
    q = torch.randint(-2**31, 2**31 - 1, (K // 16, N * 2), dtype=torch.int32, device=dev, generator=gen)
    s = (torch.rand((K // 128, N), device=dev, generator=gen) * 0.018 + 0.002).to(torch.bfloat16)
    a = torch.randn((M, K), device=dev, dtype=torch.bfloat16, generator=gen)
    ws = mu.marlin_make_workspace_new(torch.device(dev))
    e = torch.empty(0, dtype=torch.int32, device=dev)
    f = lambda x: ops.gptq_marlin_gemm(x, None, q, None, s, None, e, e, e, ws, scalar_types.uint4b8,
                                       x.shape[0], N, K, True, False, True, False)
    for _ in range(2):
        big = f(a).float()
        torch.cuda.synchronize()
        assert lib.b200q_device_error(1) == 0, "a hand-off wait timed out"
        scale = big.abs().max().item()
        for r0 in (0, 5000, 16384, 32768 - 16):
            small = f(a[r0:r0 + 16].contiguous()).float()
            assert (small - big[r0:r0 + 16]).abs().max().item() <= 2e-2 * scale, r0
