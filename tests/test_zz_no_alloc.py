"""b200q_marlin_gemm_noalloc — the GEMM entry point for callers that cannot
allocate device memory (plugins living inside another framework's fixed memory
plan, code that runs during stream capture, processes whose device memory is
owned elsewhere).  Its scratch is a fixed array inside the library instead of a
caller buffer.

The test calls it through the C ABI, twice in a row (the array keeps the
previous call's contents, so the second call sees a dirty scratch), and
compares with b200q_marlin_gemm given caller scratch: the two run the same
kernels, so the results must agree bit for bit — well inside the GEMM tolerance
used elsewhere (max-abs <= 2e-2 * max|ref|).  The file name sorts last so that
a failure here cannot hide the other tests in a run that stops at the first
failure.
"""
import ctypes

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _call(lib, fn_name, a, q, s, g_idx, perm, c, ws, L, M, stream, scratch=None):
    vp = ctypes.c_void_p
    from vllm_b200 import _lib
    ptr = lambda t: None if t is None else vp(t.data_ptr())
    head = [ptr(a), a.stride(0), ptr(q), ptr(s), None, ptr(g_idx), ptr(perm), None, ptr(c)]
    if scratch is not None:
        head += [ptr(scratch), scratch.numel()]
    tail = [ptr(ws), ws.numel(), L.type_id, _lib.BF16 if L.dtype == "bfloat16" else _lib.F16,
            M, L.size_n, L.size_k, L.num_groups, _lib.FLAG_K_FULL | _lib.FLAG_FP32_REDUCE,
            vp(stream)]
    return getattr(lib, fn_name)(*head, *tail)


@pytest.mark.parametrize("act_order", [False, True])
def test_noalloc_matches_caller_scratch(act_order):
    import torch

    from tests import gpu_utils as G
    from vllm_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    M, K, N = 16, 4096, 4096          # split slices: exercises the partial-sum scratch
    L = H.make_layer(K, N, "uint4b8", 128, act_order, "bfloat16")
    a_np = H.make_activations(M, K, "bfloat16")
    a = G.t16(a_np, "bfloat16")
    q, s = G.ti32(L.marlin_q), G.t16(L.marlin_s, "bfloat16")
    g_idx = G.ti32(L.g_idx) if act_order else None
    perm = G.ti32(L.sort_idx) if act_order else None
    ws = torch.zeros(2 * torch.cuda.get_device_properties(0).multi_processor_count,
                     dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    nbytes = lib.b200q_marlin_gemm_scratch_bytes(M, N, K, int(act_order))
    assert nbytes <= lib.b200q_marlin_gemm_noalloc_max_scratch()
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    c_ref = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    _lib.check(_call(lib, "b200q_marlin_gemm", a, q, s, g_idx, perm, c_ref, ws, L, M, stream,
                     scratch=scratch), "b200q_marlin_gemm")
    torch.cuda.synchronize()
    ref = G.n16(c_ref)

    for attempt in range(2):
        c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        _lib.check(_call(lib, "b200q_marlin_gemm_noalloc", a, q, s, g_idx, perm, c, ws, L, M,
                         stream), "b200q_marlin_gemm_noalloc")
        torch.cuda.synchronize()
        out = G.n16(c)
        assert int(ws.abs().sum().item()) == 0
        max_frac, _ = H.gemm_errors(out, ref)
        assert max_frac <= H.MAX_ABS_FRAC, f"call {attempt}: {max_frac}"
        assert np.array_equal(out, ref), f"call {attempt} differs from the caller-scratch result"


def test_noalloc_rejects_oversized_problem():
    import torch

    from vllm_b200 import _lib
    lib = _lib.load()
    # N = 57344 needs more partial-sum scratch than the built-in 16 MiB
    M, K, N = 1, 128, 57344
    assert lib.b200q_marlin_gemm_scratch_bytes(M, N, K, 0) > lib.b200q_marlin_gemm_noalloc_max_scratch()
    dev = torch.device("cuda")
    a = torch.zeros((M, K), dtype=torch.float16, device=dev)
    q = torch.zeros((K // 16, N * 2), dtype=torch.int32, device=dev)
    s = torch.zeros((1, N), dtype=torch.float16, device=dev)
    c = torch.zeros((M, N), dtype=torch.float16, device=dev)
    ws = torch.zeros(512, dtype=torch.int32, device=dev)
    vp = ctypes.c_void_p
    rc = lib.b200q_marlin_gemm_noalloc(
        vp(a.data_ptr()), K, vp(q.data_ptr()), vp(s.data_ptr()), None, None, None, None,
        vp(c.data_ptr()), vp(ws.data_ptr()), ws.numel(), H.TYPE_IDS["uint4b8"], _lib.F16, M, N, K, 1,
        _lib.FLAG_K_FULL, vp(torch.cuda.current_stream().cuda_stream))
    assert rc == _lib.ESCRATCH
    assert b"built-in scratch" in lib.b200q_last_error()
