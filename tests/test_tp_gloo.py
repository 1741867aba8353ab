"""Tensor-parallel sharding and the row-parallel all-reduce with two gloo ranks
on CPU.  The CUDA GEMM cannot run here, so each rank's shard (still in checkpoint
format, as the loaders left it) is multiplied with the CPU oracle; what is under
test is the sharding arithmetic — packed rows, group scales, replicated scales
and g_idx slices for act-order — and the collective plumbing."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from oracle import marlin_oracle as mo
from tests import helpers as H


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_shard_product(a, layer, bits, type_bias, group_size, act_order, dtype="float16"):
    q = mo.unpack_rows(layer.qweight.data.numpy(), bits)
    scales = layer.scales.data.float().numpy()
    if act_order:
        w = mo.dequantize(q, scales, dtype, bias=type_bias, g_idx=layer.g_idx.data.numpy())
    else:
        w = mo.dequantize(q, scales, dtype, bias=type_bias, group_size=group_size)
    return mo.gemm_ref(a, w)


def _worker(rank, world, port, act_order, out_q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from vllm_b200 import distributed as D
    from vllm_b200.linear import MergedColumnParallelLinear, RowParallelLinear
    from vllm_b200.quantization import GPTQMarlinConfig
    D.initialize_model_parallel(world)
    assert D.get_tensor_model_parallel_rank() == rank and D.get_tensor_model_parallel_world_size() == world
    K, N, M, g = 512, 256, 5, 128
    L = H.make_layer(K, N, "uint4b8", g, act_order, "float16")
    a = H.make_activations(M, K, "float16")
    full = mo.gemm_ref(a, L.w)
    qc = GPTQMarlinConfig(4, g, desc_act=act_order)
    ckpt_g_idx = L.g_idx_ckpt if act_order else (np.arange(K) // g).astype(np.int32)

    # ---- row-parallel: shard K, sum over ranks -------------------------------------------
    row = RowParallelLinear(K, N, quant_config=qc, params_dtype=torch.float16)
    row.weight_loader(row.qweight, torch.from_numpy(L.gptq_qweight))
    row.weight_loader(row.scales, torch.from_numpy(L.scales.astype(np.float16)))
    row.weight_loader(row.g_idx, torch.from_numpy(ckpt_g_idx))
    k0, k1 = rank * K // world, (rank + 1) * K // world
    assert torch.equal(row.g_idx.data, torch.from_numpy(ckpt_g_idx[k0:k1]))
    expected_groups = K // g if act_order else (K // world) // g
    assert row.scales.shape[0] == expected_groups
    partial = _oracle_shard_product(a[:, k0:k1], row, 4, 8, g, act_order) if act_order else \
        mo.gemm_ref(a[:, k0:k1], mo.dequantize(mo.unpack_rows(row.qweight.data.numpy(), 4),
                                               row.scales.data.float().numpy(), "float16", bias=8,
                                               group_size=g))
    summed = D.tensor_model_parallel_all_reduce(torch.from_numpy(partial))
    assert summed.data_ptr() != torch.from_numpy(partial).data_ptr()
    err_row = float(np.abs(summed.numpy() - full).max() / np.abs(full).max())

    # ---- merged column-parallel: two logical matrices, shard N, gather -----------------------
    col = MergedColumnParallelLinear(K, [N // 2, N // 2], quant_config=qc, params_dtype=torch.float16)
    for name, t in (("qweight", L.gptq_qweight), ("scales", L.scales.astype(np.float16))):
        for sid in range(2):
            part = torch.from_numpy(np.ascontiguousarray(t[:, sid * N // 2:(sid + 1) * N // 2]))
            col.weight_loader(getattr(col, name), part, sid)
    col.weight_loader(col.g_idx, torch.from_numpy(ckpt_g_idx), 0)
    out = _oracle_shard_product(a, col, 4, 8, g, act_order) if act_order else \
        mo.gemm_ref(a, mo.dequantize(mo.unpack_rows(col.qweight.data.numpy(), 4),
                                     col.scales.data.float().numpy(), "float16", bias=8, group_size=g))
    gathered = D.tensor_model_parallel_all_gather(torch.from_numpy(out)).numpy()
    # rank r holds columns [r*N/4, (r+1)*N/4) of each half
    h = N // 2 // world
    cols = np.concatenate([np.r_[r * h:(r + 1) * h, N // 2 + r * h:N // 2 + (r + 1) * h]
                           for r in range(world)])
    err_col = float(np.abs(gathered - full[:, cols]).max() / np.abs(full).max())
    out_q.put((rank, err_row, err_col))
    dist.destroy_process_group()


@pytest.mark.parametrize("act_order", [False, True])
def test_two_rank_sharding_and_all_reduce(act_order):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, act_order, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err_row, err_col in results:
        assert err_row < 1e-4 and err_col < 1e-4, (rank, err_row, err_col)


def _worker_forward(rank, world, port, out_q):
    """RowParallelLinear.forward on CPU (16-bit weights, torch matmul): with no peer link
    (reduce_link() is None) the layer falls back to the process group; reduce=False
    returns the partial sum; the bias is added on rank 0 only."""
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from vllm_b200 import distributed as D
    from vllm_b200.linear import RowParallelLinear
    D.initialize_model_parallel(world)
    ok = D.reduce_link() is None
    torch.manual_seed(0)
    K, N, M = 64, 32, 3
    w = torch.randn(N, K)
    b = torch.randn(N)
    x = torch.randn(M, K)
    layer = RowParallelLinear(K, N, bias=True, params_dtype=torch.float32)
    layer.weight_loader(layer.weight, w)
    layer.bias.data.copy_(b)
    k0, k1 = rank * K // world, (rank + 1) * K // world
    part = layer(x[:, k0:k1], reduce=False)
    want_part = x[:, k0:k1] @ w[:, k0:k1].t() + (b if rank == 0 else 0)
    ok &= bool(torch.allclose(part, want_part, atol=1e-5))
    full = layer(x[:, k0:k1])
    ok &= bool(torch.allclose(full, x @ w.t() + b, atol=1e-4))
    whole = RowParallelLinear(K, N, input_is_parallel=False, params_dtype=torch.float32)
    whole.weight_loader(whole.weight, w)
    ok &= bool(torch.allclose(whole(x), x @ w.t(), atol=1e-4))
    out_q.put((rank, bool(ok)))
    dist.destroy_process_group()


def test_row_parallel_forward_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_forward, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok in results), results
