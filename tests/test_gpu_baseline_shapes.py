"""Full-size shapes of the benchmark configurations, checked through properties
that do not need a full CPU reference: every kernel family must agree on the
same layer (decode kernel at small M vs tensor-core kernel at large M on shared
rows), and an oracle-checked corner of the output (first 64 columns) pins the
absolute values.  Config 3 (Qwen2-7B AWQ uint4 + zero-points, and W8A16
uint8b128 channel-wise) and config 4 (Llama-3-70B shards) shapes."""
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
    return torch, G, ops, mu, _lib.load()


def _random_layer(torch, K, N, bits, G_, has_zp, tdt, gen):
    pf = 32 // bits
    q = torch.randint(-2**31, 2**31 - 1, (K // 16, N * 16 // pf), dtype=torch.int32, device="cuda",
                      generator=gen)
    s = (torch.rand((G_, N), device="cuda", generator=gen) * 0.018 + 0.002).to(tdt)
    z = torch.randint(-2**31, 2**31 - 1, (G_, N // pf), dtype=torch.int32, device="cuda",
                      generator=gen) if has_zp else torch.empty(0, dtype=torch.int32, device="cuda")
    return q, s, z


def _corner_ref(a_np, q, s, z, K, bits, group, has_zp, dtype, type_bias):
    """Oracle product for the first 64 output columns."""
    words = 16 * 64 * bits // 32
    qn = np.ascontiguousarray(q[:, :words].cpu().numpy())
    codes = mo.marlin_unpack(qn, K, 64, bits)
    G_ = s.shape[0]
    s_lin = mo.marlin_unpermute_scales(s[:, :64].float().cpu().numpy(), K, 64, group if G_ > 1 else -1)
    zeros = None
    if has_zp:
        zeros = mo.marlin_zero_points_unpack(np.ascontiguousarray(z[:, :64 * bits // 32].cpu().numpy()),
                                             G_, 64, bits)
    w = mo.dequantize(codes, s_lin, dtype, bias=type_bias, zeros=zeros,
                      group_size=group if G_ > 1 else -1)
    return mo.gemm_ref(a_np, w)


CASES = [
    # name, K, N, qtype, group, dtype, Ms
    ("qwen2_awq_gate_up", 3584, 37888, "uint4", 128, "float16", (1, 32, 512, 2048)),
    ("qwen2_awq_down", 18944, 3584, "uint4", 128, "float16", (1, 32, 512, 2048)),
    ("qwen2_w8_qkv", 3584, 4608, "uint8b128", -1, "float16", (1, 32, 512, 2048)),
    ("qwen2_w8_o", 3584, 3584, "uint8b128", -1, "float16", (1, 32, 512)),
    ("llama70b_gate_up_tp8", 8192, 7168, "uint4b8", 128, "bfloat16", (1, 16, 128, 1024)),
    ("llama70b_down_tp8", 3584, 8192, "uint4b8", 128, "bfloat16", (1, 16, 128, 1024)),
    ("llama70b_down_tp2", 14336, 8192, "uint4b8", 128, "bfloat16", (16, 8192)),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_full_size_layer_consistency(env, case):
    torch, G, ops, mu, lib = env
    from vllm_b200.scalar_type import ScalarType
    name, K, N, qtype, group, dtype, Ms = case
    bits, has_zp = H.TYPE_BITS[qtype], qtype in ("uint4", "uint8")
    tdt = torch.float16 if dtype == "float16" else torch.bfloat16
    G_ = K // group if group > 0 else 1
    gen = torch.Generator(device="cuda").manual_seed(7)
    q, s, z = _random_layer(torch, K, N, bits, G_, has_zp, tdt, gen)
    ws = mu.marlin_make_workspace_new(torch.device("cuda"))
    e = torch.empty(0, dtype=torch.int32, device="cuda")
    qt = ScalarType.from_id(H.TYPE_IDS[qtype])
    f = lambda x: ops.gptq_marlin_gemm(x, None, q, None, s, None, z, e, e, ws, qt, x.shape[0], N, K,
                                       True, False, True, False)
    m_max = max(Ms)
    a = torch.randn((m_max, K), device="cuda", dtype=tdt, generator=gen)
    full = f(a).float()
    torch.cuda.synchronize()
    assert lib.b200q_device_error(1) == 0
    scale = full.abs().max().item()
    # oracle corner: first 48 rows (or fewer) x first 64 columns
    rows = min(48, m_max)
    ref = _corner_ref(G.n16(a[:rows]), q, s, z, K, bits, group, has_zp, dtype, H.TYPE_BIAS[qtype])
    mf, mr = H.gemm_errors(full[:rows, :64].cpu().numpy(), ref)
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL, (name, mf, mr)
    # every smaller M (other kernels / tile shapes) reproduces the same rows
    for m in Ms:
        if m == m_max:
            continue
        part = f(a[:m].contiguous()).float()
        assert (part - full[:m]).abs().max().item() <= 2e-2 * scale, (name, m)
    assert int(ws.abs().sum().item()) == 0


# Config 2: the benchmarked sweep itself.  Llama-3-8B layers, uint4b8, group 128, act-order
# (desc_act): the op receives the sorted g_idx and the sort permutation, exactly what the bench
# passes, so this is the path whose time is reported (activation gather + grouped kernel, every
# kernel family over M), plus the partial-K form of the same layer (is_k_full = False: groups
# looked up through g_idx), as tests/kernels/quantization/test_marlin_gemm.py:212-361 crosses
# act_order with is_k_full.
CONFIG2 = [("qkv", 4096, 6144), ("o", 4096, 4096), ("gate_up", 4096, 28672), ("down", 14336, 4096)]
CONFIG2_MS = (1, 16, 64, 256, 4096)


@pytest.mark.parametrize("layer", CONFIG2, ids=lambda c: c[0])
def test_config2_act_order_full_size(env, layer):
    torch, G, ops, mu, lib = env
    from vllm_b200.scalar_type import scalar_types
    name, K, N = layer
    group, dtype, tdt = 128, "bfloat16", torch.bfloat16
    gen = torch.Generator(device="cuda").manual_seed(11)
    q, s, _ = _random_layer(torch, K, N, 4, K // group, False, tdt, gen)
    g = (torch.arange(K, device="cuda") // group)[torch.randperm(K, device="cuda", generator=gen)]
    order = torch.argsort(g, stable=True)
    g_idx, perm = g[order].to(torch.int32).contiguous(), order.to(torch.int32).contiguous()
    ws = mu.marlin_make_workspace_new(torch.device("cuda"))
    e = torch.empty(0, dtype=torch.int32, device="cuda")

    def f(x, k_full=True):
        return ops.gptq_marlin_gemm(x, None, q, None, s, None, e, g_idx, perm, ws,
                                    scalar_types.uint4b8, x.shape[0], N, K, k_full, False, True,
                                    False)

    m_max = max(CONFIG2_MS)
    a = torch.randn((m_max, K), device="cuda", dtype=tdt, generator=gen)
    full = f(a).float()
    torch.cuda.synchronize()
    assert lib.b200q_device_error(1) == 0
    scale = full.abs().max().item()
    # oracle corner: the kernel multiplies the gathered columns a[:, perm] with the rows in
    # sorted order, whose groups are then contiguous
    rows = 48
    a_sorted = G.n16(a[:rows][:, order])
    ref = _corner_ref(a_sorted, q, s, None, K, 4, group, False, dtype, 8)
    mf, mr = H.gemm_errors(full[:rows, :64].cpu().numpy(), ref)
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL, (name, mf, mr)
    for m in CONFIG2_MS:
        part = f(a[:m].contiguous()).float()
        torch.cuda.synchronize()
        assert (part - full[:m]).abs().max().item() <= 2e-2 * scale, (name, m)
        if m <= rows:
            mf, mr = H.gemm_errors(part[:, :64].cpu().numpy(), ref[:m])
            assert mf <= H.MAX_ABS_FRAC and mr <= 2 * H.MEAN_REL, (name, m, mf, mr)
    # partial-K form (group looked up per row): same numbers, other kernel
    for m in (1, 16, 64):
        part = f(a[:m].contiguous(), k_full=False).float()
        torch.cuda.synchronize()
        assert (part - full[:m]).abs().max().item() <= 2e-2 * scale, (name, m, "lookup")
    assert lib.b200q_device_error(1) == 0
    assert int(ws.abs().sum().item()) == 0
