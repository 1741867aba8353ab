"""Peer-memory all-reduce (b200q_all_reduce) against NCCL on 2+ GPUs: exact
equality on integer-valued inputs (as the reference's
tests/distributed/test_custom_all_reduce.py:60-82 does), several sizes, repeated
calls (the epoch counters), CUDA-graph replay, and a row-parallel quantized layer
whose output goes through it.  Skipped when fewer than two GPUs are visible."""
import os
import socket

import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"   # also on the exception path below
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from vllm_b200 import _lib
    from vllm_b200 import distributed as D
    D.initialize_model_parallel(world)
    assert D.enable_custom_all_reduce(dev)
    lib = _lib.load()
    ok = True
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    for dtype in (torch.bfloat16, torch.float16):
        for shape in ((1, 4096), (16, 4096), (64, 8192), (5, 8)):
            for rep in range(3):
                x = torch.randint(-8, 9, shape, device=dev, generator=gen).to(dtype)
                want = x.clone()
                dist.all_reduce(want)
                got = D.tensor_model_parallel_all_reduce(x)
                ok &= bool(torch.equal(got, want)) and got.data_ptr() != x.data_ptr()
    # too large for the one-shot path: falls back to NCCL
    big = torch.ones((1024, 8192), device=dev, dtype=torch.bfloat16)
    ok &= bool((D.tensor_model_parallel_all_reduce(big) == world).all())
    # CUDA graph replay: the kernel advances its own epochs
    x = torch.randint(-8, 9, (16, 4096), device=dev, generator=gen).to(torch.bfloat16)
    want = x.clone()
    dist.all_reduce(want)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        y = D.tensor_model_parallel_all_reduce(x)
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y = D.tensor_model_parallel_all_reduce(x)
        y2 = D.tensor_model_parallel_all_reduce(y)
    for _ in range(5):
        g.replay()
    torch.cuda.synchronize()
    ok &= bool(torch.equal(y, want)) and bool(torch.equal(y2, want * world))
    # a row-parallel quantized layer end to end
    import numpy as np
    from oracle import marlin_oracle as mo
    from tests import gpu_utils as G
    from tests import helpers as H
    from vllm_b200.linear import RowParallelLinear
    from vllm_b200.quantization import GPTQMarlinConfig
    K, N, M, gsz = 2048, 1024, 16, 128
    L = H.make_layer(K, N, "uint4b8", gsz, False, "bfloat16")
    a_np = H.make_activations(M, K, "bfloat16")
    layer = RowParallelLinear(K, N, quant_config=GPTQMarlinConfig(4, gsz, False),
                              params_dtype=torch.bfloat16, device=dev)
    layer.weight_loader(layer.qweight, torch.from_numpy(L.gptq_qweight).to(dev))
    layer.weight_loader(layer.scales, torch.from_numpy(L.scales).to(torch.bfloat16).to(dev))
    layer.weight_loader(layer.g_idx, torch.from_numpy((np.arange(K) // gsz).astype(np.int32)).to(dev))
    layer.process_weights_after_loading()
    a = G.t16(a_np, "bfloat16", device=dev)
    shard = a[:, rank * K // world:(rank + 1) * K // world].contiguous()
    out = layer(shard)                      # GEMM with the all-reduce in its epilogue
    torch.cuda.synchronize()
    mf, mr = H.gemm_errors(G.n16(out), mo.gemm_ref(a_np, L.w))
    ok &= mf <= H.MAX_ABS_FRAC and mr <= 2 * H.MEAN_REL
    # the fused kernel gives the bits of GEMM followed by the stand-alone all-reduce, for
    # every decode size, for sizes that take the in-place kernel (M = 48), and under graph replay
    for m in (1, 3, 8, 16, 32, 48):
        part = layer.quant_method.apply(layer, shard[:m].contiguous(), None)
        want = D.tensor_model_parallel_all_reduce(part)
        got = layer(shard[:m].contiguous())
        ok &= bool(torch.equal(got, want))
    # many rows: blocks of rows with NCCL's all-reduce beside the next block's GEMM give the bits of
    # GEMM followed by one all-reduce, eagerly and under graph replay
    big = torch.randn((1280, K // world), device=dev, generator=gen).to(torch.bfloat16)
    want_big = D.tensor_model_parallel_all_reduce(layer.quant_method.apply(layer, big, None))
    D.OVERLAP_MIN_ROWS = 1024               # (the default threshold is 8192 rows)
    got_big = layer(big)
    torch.cuda.synchronize()
    ok &= got_big.shape == want_big.shape and bool(torch.equal(got_big, want_big))
    g3 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g3):
        o3 = layer(big)
    for _ in range(3):
        g3.replay()
    torch.cuda.synchronize()
    ok &= bool(torch.equal(o3, want_big))
    del g3
    xs = shard[:16].contiguous()
    want = D.tensor_model_parallel_all_reduce(layer.quant_method.apply(layer, xs, None))
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer(xs)
    torch.cuda.current_stream().wait_stream(side)
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2):
        o1 = layer(xs)
        o2 = layer(xs)
    for _ in range(7):
        g2.replay()
    torch.cuda.synchronize()
    ok &= bool(torch.equal(o1, want)) and bool(torch.equal(o2, want))
    # all-reduce + residual add + RMSNorm in one kernel == the three steps one after another
    from vllm_b200 import _custom_ops as ops
    car = D._CUSTOM_AR
    common = torch.Generator(device=dev).manual_seed(77)        # same residual / weight on every rank
    for (m, n) in ((1, 4096), (48, 4096), (5, 1024), (64, 4096)):
        part = torch.randn((m, n), device=dev, generator=gen).to(torch.bfloat16)
        res = torch.randn((m, n), device=dev, generator=common).to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(n, device=dev, generator=common)).to(torch.bfloat16)
        want_x, want_res = D.tensor_model_parallel_all_reduce(part), res.clone()
        ops.fused_add_rms_norm(want_x, want_res, w, 1e-5)
        got_x, got_res = part.clone(), res.clone()
        ok &= car.all_reduce_add_rms_norm(got_x, got_res, w, 1e-5)
        torch.cuda.synchronize()
        ok &= bool(torch.equal(got_x, want_x)) and bool(torch.equal(got_res, want_res))
    ok &= lib.b200q_device_error(1) == 0
    # leave in order: nothing in flight, graphs that hold link kernels gone, the peer buffers
    # released on every rank, then the process group, then a normal return
    torch.cuda.synchronize()
    dist.barrier()
    del g, g2, layer
    D.destroy_model_parallel()
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    q.put((rank, bool(ok)))


def _worker_guarded(rank, world, port, q):
    """Report an exception of the worker instead of dying silently (the parent would otherwise
    wait for its time-out while the other rank blocks in a collective)."""
    try:
        _worker(rank, world, port, q)
    except BaseException:                      # noqa: BLE001 - everything goes to the parent
        import traceback
        q.put((rank, traceback.format_exc()))
        q.close()
        q.join_thread()
        os._exit(1)


@pytest.mark.parametrize("twoshot", [False, True])
def test_custom_all_reduce_matches_nccl(twoshot, monkeypatch):
    """twoshot: the owner-reduces variant, forced on for every size and for two ranks."""
    import queue

    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    if twoshot:                      # read by the library in the child processes
        monkeypatch.setenv("B200Q_DEBUG", "twoshot_any")
    world = min(4, torch.cuda.device_count()) if twoshot else 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_guarded, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in procs:
            results.append(q.get(timeout=150))
            if results[-1][1] is not True:       # a failed check or a traceback: stop waiting
                break
    except queue.Empty:
        results.append(("timeout", "no report within 150 s; exit codes %s" % [p.exitcode for p in procs]))
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.kill()                             # exactly the children started above
    assert len(results) == world and all(ok is True for _, ok in results), results
