"""moe_wna16_marlin_gemm (the Marlin GEMM over blocks of tokens sorted by expert) and the
fused_marlin_moe layer built on it, against the oracle: every block size, weight types with and
without zero-points, channel-wise and grouped scales, bias, router weights, experts without
tokens, expert parallelism (-1 blocks), and the two-GEMM layer against a numpy composite."""
import numpy as np
import pytest

from oracle import marlin_oracle as mo
from tests import gpu_utils as G
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _experts(E, K, N, qtype, group, dtype, with_bias=False, seed=0):
    return [H.make_layer(K, N, qtype, group, False, dtype, seed=seed + 101 * e, with_bias=with_bias)
            for e in range(E)]


def _stack(torch, layers, dtype):
    q = torch.stack([G.ti32(L.marlin_q) for L in layers])
    s = torch.stack([G.t16(L.marlin_s, dtype) for L in layers])
    z = torch.stack([G.ti32(L.marlin_zp) for L in layers]) if layers[0].has_zp else None
    b = torch.stack([G.t16(L.marlin_bias, dtype) for L in layers]) if layers[0].marlin_bias is not None else None
    return q, s, z, b


CASES = [
    # M, K, N, E, topk, block, type, group, dtype, bias, mul
    (5, 128, 64, 4, 2, 16, "uint4b8", -1, "float16", False, False),
    (33, 256, 128, 8, 4, 8, "uint4b8", 128, "bfloat16", False, True),
    (64, 512, 256, 3, 2, 64, "uint4b8", 64, "float16", True, True),
    (7, 256, 192, 16, 1, 32, "uint8b128", 128, "bfloat16", False, False),
    (100, 1024, 128, 6, 3, 48, "uint4", 128, "float16", False, True),
    (40, 512, 128, 4, 2, 16, "uint8", -1, "bfloat16", True, False),
    (256, 2048, 512, 8, 2, 64, "uint4b8", 128, "bfloat16", False, True),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(map(str, c)))
def test_moe_gemm(case):
    import torch
    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import marlin_utils as mu
    from vllm_b200.scalar_type import scalar_types
    M, K, N, E, topk, bs, qtype, group, dtype, with_bias, mul = case
    rng = np.random.default_rng(M * 7 + E)
    layers = _experts(E, K, N, qtype, group, dtype, with_bias)
    a = H.make_activations(M, K, dtype)
    topk_ids = np.stack([rng.permutation(E)[:topk] for _ in range(M)]).astype(np.int32)
    if topk == 1 and E > 2:
        topk_ids[topk_ids == 1] = 0               # an expert without tokens
    tw = rng.uniform(0.1, 1.0, size=(M * topk,)).astype(np.float32)
    sorted_ids, expert_ids, num = mo.moe_align_block_size(topk_ids, bs, E)
    dev = torch.device("cuda")
    q, s, z, b = _stack(torch, layers, dtype)
    out = ops.moe_wna16_marlin_gemm(
        G.t16(a, dtype), None, q, b, s, None, z, None, None, mu.marlin_make_workspace_new(dev),
        torch.from_numpy(sorted_ids).to(dev), torch.from_numpy(expert_ids).to(dev),
        torch.from_numpy(num).to(dev), torch.from_numpy(tw).to(dev), bs, topk, mul, False,
        getattr(scalar_types, qtype), M, N, K)
    torch.cuda.synchronize()
    got = G.n16(out)
    ref = mo.moe_marlin_gemm_ref(a, [L.w for L in layers], sorted_ids, expert_ids, int(num[0]),
                                 tw if mul else None, bs, topk, M,
                                 [L.bias for L in layers] if with_bias else None)
    assert not np.isnan(ref).any()                # every (token, slot) is in some block
    mf, mr = H.gemm_errors(got, ref)
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL, (case, mf, mr)


def test_moe_gemm_expert_parallel_blocks_are_skipped():
    """Blocks whose expert id is -1 (expert on another rank) leave their output rows untouched."""
    import torch
    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import marlin_utils as mu
    from vllm_b200.scalar_type import scalar_types
    M, K, N, E, topk, bs, dtype = 24, 256, 128, 4, 2, 16, "float16"
    rng = np.random.default_rng(5)
    layers = _experts(E, K, N, "uint4b8", 128, dtype)
    a = H.make_activations(M, K, dtype)
    topk_ids = np.stack([rng.permutation(E)[:topk] for _ in range(M)]).astype(np.int32)
    sorted_ids, expert_ids, num = mo.moe_align_block_size(topk_ids, bs, E)
    local = expert_ids.copy()
    local[expert_ids >= 2] = -1                   # experts 2, 3 live elsewhere
    dev = torch.device("cuda")
    q, s, _, _ = _stack(torch, layers, dtype)
    out = torch.full((M * topk, N), 7.0, dtype=torch.float16, device=dev)
    ops.moe_wna16_marlin_gemm(
        G.t16(a, dtype), out, q, None, s, None, None, None, None, mu.marlin_make_workspace_new(dev),
        torch.from_numpy(sorted_ids).to(dev), torch.from_numpy(local).to(dev),
        torch.from_numpy(num).to(dev), torch.ones(M * topk, device=dev), bs, topk, False, True,
        scalar_types.uint4b8, M, N, K)
    torch.cuda.synchronize()
    got = G.n16(out)
    ref = mo.moe_marlin_gemm_ref(a, [L.w for L in layers], sorted_ids, local, int(num[0]), None, bs, topk, M)
    skipped = np.isnan(ref).all(axis=1)
    assert skipped.any() and (~skipped).any()
    assert np.all(got[skipped] == 7.0)
    mf, mr = H.gemm_errors(got[~skipped], ref[~skipped])
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL, (mf, mr)


@pytest.mark.parametrize("M,E,topk,dtype", [(4, 8, 2, "bfloat16"), (96, 4, 2, "float16"), (300, 8, 4, "bfloat16")])
def test_fused_marlin_moe_layer(M, E, topk, dtype):
    """align -> gate_up GEMM -> silu * up -> down GEMM with router weights -> sum over top-k,
    against the same steps in numpy (16-bit rounding after each GEMM and the activation)."""
    import torch
    from vllm_b200 import fused_moe
    from vllm_b200.scalar_type import scalar_types
    K, N = 256, 128
    rng = np.random.default_rng(M + E)
    w1 = _experts(E, K, 2 * N, "uint4b8", 128, dtype, seed=1)
    w2 = _experts(E, N, K, "uint4b8", 128, dtype, seed=2)
    a = H.make_activations(M, K, dtype)
    topk_ids = np.stack([rng.permutation(E)[:topk] for _ in range(M)]).astype(np.int32)
    tw = rng.uniform(0.1, 1.0, size=(M, topk)).astype(np.float32)
    dev = torch.device("cuda")
    q1, s1, _, _ = _stack(torch, w1, dtype)
    q2, s2, _, _ = _stack(torch, w2, dtype)
    out = fused_moe.fused_marlin_moe(G.t16(a, dtype), q1, q2, s1, s2, torch.from_numpy(tw).to(dev),
                                     torch.from_numpy(topk_ids).to(dev), scalar_types.uint4b8)
    torch.cuda.synchronize()
    ref = np.zeros((M, K), dtype=np.float32)
    for t in range(M):
        for j in range(topk):
            e = int(topk_ids[t, j])
            h = mo.round_to_dtype(a[t].astype(np.float32) @ w1[e].w.astype(np.float32), dtype)
            act = mo.round_to_dtype(h[:N] / (1.0 + np.exp(-h[:N])) * h[N:], dtype)
            y = mo.round_to_dtype((act @ w2[e].w.astype(np.float32)) * tw[t, j], dtype)
            ref[t] += y
    mf, mr = H.gemm_errors(G.n16(out), ref)
    assert mf <= 3e-2 and mr <= 1.5e-2, (mf, mr)


def test_moe_error_messages():
    import torch
    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import marlin_utils as mu
    from vllm_b200.scalar_type import scalar_types
    dev = torch.device("cuda")
    M, K, N, E = 4, 128, 64, 2
    a = torch.zeros((M, K), dtype=torch.float16, device=dev)
    q = torch.zeros((E, K // 16, N * 2), dtype=torch.int32, device=dev)
    s = torch.ones((E, 1, N), dtype=torch.float16, device=dev)
    ids = torch.zeros(64, dtype=torch.int32, device=dev)
    ex = torch.zeros(8, dtype=torch.int32, device=dev)
    num = torch.zeros(1, dtype=torch.int32, device=dev)
    tw = torch.ones(M, dtype=torch.float32, device=dev)
    ws = mu.marlin_make_workspace_new(dev)
    with pytest.raises(RuntimeError, match="unsupported moe_block_size=24"):
        ops.moe_wna16_marlin_gemm(a, None, q, None, s, None, None, None, None, ws, ids, ex, num, tw, 24, 1,
                                  False, False, scalar_types.uint4b8, M, N, K)
    with pytest.raises(RuntimeError, match="actual_size_n"):
        ops.moe_wna16_marlin_gemm(a, None, q, None, s, None, None, None, None, ws, ids, ex, num, tw, 16, 1,
                                  False, False, scalar_types.uint4b8, M, 2 * N, K)
