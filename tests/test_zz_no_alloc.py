"""b200q_marlin_gemm_noalloc — the GEMM entry point for callers that cannot
allocate device memory (plugins living inside another framework's fixed memory
plan, code that runs during stream capture, processes whose device memory is
owned elsewhere).  Its scratch is a fixed array inside the library instead of a
caller buffer.

The test calls it through the C ABI, twice in a row (the array keeps the
previous call's contents, so the second call sees a dirty scratch), and
compares with the CPU oracle (GEMM tolerance: max-abs <= 2e-2 * max|ref|, mean
relative error <= 5e-3) and with b200q_marlin_gemm given caller scratch of the
same size: the two run the same kernels with the same plan, so they must agree
bit for bit.  The file name sorts last so that
a failure here cannot hide the other tests in a run that stops at the first
failure.
"""
import ctypes

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _call(lib, fn_name, a, q, s, g_idx, perm, c, ws, L, M, stream, flags, scratch=None):
    vp = ctypes.c_void_p
    from vllm_b200 import _lib
    ptr = lambda t: None if t is None else vp(t.data_ptr())
    head = [ptr(a), a.stride(0), ptr(q), ptr(s), None, ptr(g_idx), ptr(perm), None, ptr(c)]
    if scratch is not None:
        head += [ptr(scratch), scratch.numel()]
    tail = [ptr(ws), ws.numel(), L.type_id, _lib.BF16 if L.dtype == "bfloat16" else _lib.F16,
            M, L.size_n, L.size_k, L.num_groups, flags, vp(stream)]
    return getattr(lib, fn_name)(*head, *tail)


# Every kernel family that keeps something in the scratch, on a 4096 x 4096 layer whose column
# slices are shared by several CTAs (so fp32 partial sums go through the array):
#   stream      decode kernel, M = 16: partial sums of split slices
#   stream_act  the same with act-order: + the gathered activations at the array's tail
#   lookup      act-order layer holding part of K (is_k_full = False), M = 16: the
#               reference-order kernel's partial sums
#   tensor      M = 256: the tensor-core kernel's k-split partials
CASES = [("stream", 16, False, True), ("stream_act", 16, True, True), ("lookup", 16, True, False),
         ("tensor", 256, False, True)]


@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_noalloc_matches_caller_scratch(case):
    import torch

    from oracle import marlin_oracle as mo
    from tests import gpu_utils as G
    from vllm_b200 import _lib
    name, M, act_order, k_full = case
    lib = _lib.load()
    dev = torch.device("cuda")
    K, N = 4096, 4096
    L = H.make_layer(K, N, "uint4b8", 128, act_order, "bfloat16")
    a_np = H.make_activations(M, K, "bfloat16")
    a = G.t16(a_np, "bfloat16")
    q, s = G.ti32(L.marlin_q), G.t16(L.marlin_s, "bfloat16")
    g_idx = G.ti32(L.g_idx) if act_order else None
    perm = G.ti32(L.sort_idx) if act_order else None
    ws = torch.zeros(2 * torch.cuda.get_device_properties(0).multi_processor_count,
                     dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    flags = (_lib.FLAG_K_FULL if k_full else 0) | _lib.FLAG_FP32_REDUCE

    assert (lib.b200q_marlin_gemm_scratch_bytes(M, N, K, int(act_order))
            <= lib.b200q_marlin_gemm_noalloc_max_scratch())
    # the caller-scratch arm gets a buffer of the built-in array's size, so that both arms
    # plan the same k-split and bit equality is the right expectation
    scratch = torch.empty(lib.b200q_marlin_gemm_noalloc_max_scratch(), dtype=torch.uint8, device=dev)
    c_ref = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    _lib.check(_call(lib, "b200q_marlin_gemm", a, q, s, g_idx, perm, c_ref, ws, L, M, stream, flags,
                     scratch=scratch), "b200q_marlin_gemm")
    torch.cuda.synchronize()
    ref = G.n16(c_ref)
    oracle = mo.gemm_ref(a_np, L.w)          # the reference's dequantise-then-matmul, on the CPU

    for attempt in range(2):
        c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        _lib.check(_call(lib, "b200q_marlin_gemm_noalloc", a, q, s, g_idx, perm, c, ws, L, M,
                         stream, flags), "b200q_marlin_gemm_noalloc")
        torch.cuda.synchronize()
        out = G.n16(c)
        assert lib.b200q_device_error(1) == 0
        assert int(ws.abs().sum().item()) == 0
        max_frac, mean_rel = H.gemm_errors(out, oracle)
        assert max_frac <= H.MAX_ABS_FRAC and mean_rel <= H.MEAN_REL, (name, attempt, max_frac, mean_rel)
        assert np.array_equal(out, ref), f"{name}, call {attempt}: differs from the caller-scratch result"


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
