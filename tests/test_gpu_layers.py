"""GPU parity of the layer stack: checkpoint-format parameters -> per-shard repack
(MarlinLinearKernel / AWQMarlinLinearMethod) -> GEMM, against the CPU oracle.
Tensor parallelism is emulated on one GPU by building every rank's shard in this
process: row-parallel partial outputs must sum to, and column-parallel outputs
concatenate to, the unsharded result."""
import numpy as np
import pytest

from oracle import marlin_oracle as mo
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_utils as G
    assert torch.cuda.is_available()
    return torch, G


def _load_gptq(torch, layer, L, ckpt_g_idx):
    tdt = torch.float16 if L.dtype == "float16" else torch.bfloat16
    layer.weight_loader(layer.qweight, torch.from_numpy(L.gptq_qweight).cuda())
    layer.weight_loader(layer.scales, torch.from_numpy(L.scales).to(tdt).cuda())
    layer.weight_loader(layer.g_idx, torch.from_numpy(ckpt_g_idx).cuda())
    layer.process_weights_after_loading()


@pytest.mark.parametrize("act_order", [False, True])
@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("M", [3, 200])
def test_gptq_layers_tp_emulated(env, act_order, dtype, M):
    torch, G = env
    from vllm_b200.linear import ColumnParallelLinear, RowParallelLinear
    from vllm_b200.quantization import GPTQMarlinConfig
    K, N, g, tp = 1024, 768, 128, 2
    tdt = torch.float16 if dtype == "float16" else torch.bfloat16
    L = H.make_layer(K, N, "uint4b8", g, act_order, dtype)
    a_np = H.make_activations(M, K, dtype)
    a = G.t16(a_np, dtype)
    ref = mo.gemm_ref(a_np, L.w)
    qc = GPTQMarlinConfig(4, g, desc_act=act_order)
    ckpt_g_idx = L.g_idx_ckpt if act_order else (np.arange(K) // g).astype(np.int32)
    kw = dict(quant_config=qc, params_dtype=tdt, device="cuda")

    full = ColumnParallelLinear(K, N, tp_rank=0, tp_size=1, **kw)
    _load_gptq(torch, full, L, ckpt_g_idx)
    # the device repack of the checkpoint tensor reproduces the oracle's Marlin layout
    assert np.array_equal(full.qweight.data.cpu().numpy(), L.marlin_q)
    out = G.n16(full(a))
    mf, mr = H.gemm_errors(out, ref)
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL

    cols = []
    for r in range(tp):
        c = ColumnParallelLinear(K, N, tp_rank=r, tp_size=tp, **kw)
        _load_gptq(torch, c, L, ckpt_g_idx)
        cols.append(G.n16(c(a)))
    mf, mr = H.gemm_errors(np.concatenate(cols, axis=1), ref)
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL

    total = np.zeros_like(ref)
    for r in range(tp):
        rl = RowParallelLinear(K, N, tp_rank=r, tp_size=tp, reduce_results=False, **kw)
        _load_gptq(torch, rl, L, ckpt_g_idx)
        if act_order:
            assert rl.is_k_full is False   # group lookup path
        total += G.n16(rl(a[:, r * K // tp:(r + 1) * K // tp].contiguous()))
    mf, mr = H.gemm_errors(total, ref)
    assert mf <= H.MAX_ABS_FRAC and mr <= 2 * H.MEAN_REL   # two 16-bit roundings of partial sums


def test_awq_layer(env):
    torch, G = env
    from vllm_b200.linear import ColumnParallelLinear
    from vllm_b200.quantization import AWQMarlinConfig
    K, N, g, M = 1024, 512, 128, 33
    L = H.make_layer(K, N, "uint4", g, False, "float16")
    a_np = H.make_activations(M, K, "float16")
    layer = ColumnParallelLinear(K, N, bias=True, quant_config=AWQMarlinConfig(4, g),
                                 params_dtype=torch.float16, device="cuda", tp_rank=0, tp_size=1)
    layer.weight_loader(layer.qweight, torch.from_numpy(L.awq_qweight).cuda())
    layer.weight_loader(layer.scales, torch.from_numpy(L.scales).half().cuda())
    layer.weight_loader(layer.qzeros, torch.from_numpy(mo.awq_pack(L.zeros, 4)).cuda())
    bias = np.linspace(-2, 2, N).astype(np.float16).astype(np.float32)
    layer.bias.data.copy_(torch.from_numpy(bias).half())
    layer.process_weights_after_loading()
    assert np.array_equal(layer.qweight.data.cpu().numpy(), L.marlin_q)
    assert np.array_equal(layer.qzeros.data.cpu().numpy(), L.marlin_zp)
    out = G.n16(layer(G.t16(a_np, "float16")))
    mf, mr = H.gemm_errors(out, mo.gemm_ref(a_np, L.w, bias))
    assert mf <= H.MAX_ABS_FRAC and mr <= H.MEAN_REL
