"""torch-side helpers of the GPU parity tests (imported only by tests marked gpu)."""
from __future__ import annotations

import numpy as np
import torch

from tests import helpers as H


def t16(x: np.ndarray, dtype: str, device="cuda") -> torch.Tensor:
    bits = torch.from_numpy(H.to_bits16(x, dtype).view(np.int16).copy())
    return bits.view(torch.float16 if dtype == "float16" else torch.bfloat16).to(device)


def n16(t: torch.Tensor) -> np.ndarray:
    dtype = "float16" if t.dtype == torch.float16 else "bfloat16"
    return H.from_bits16(t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16), dtype)


def ti32(x: np.ndarray | None, device="cuda") -> torch.Tensor:
    if x is None:
        return torch.empty(0, dtype=torch.int32, device=device)
    return torch.from_numpy(np.ascontiguousarray(x).view(np.int32).copy()).to(device)


def run_gemm(ops, mu, L, a_np, *, is_k_full=True, use_atomic_add=False, use_fp32_reduce=True,
             workspace=None, a_tensor=None):
    """Run gptq_marlin_gemm on layer L (tests.helpers.Layer) and return a numpy float32 result."""
    from vllm_b200.scalar_type import ScalarType
    dev = "cuda"
    a = a_tensor if a_tensor is not None else t16(a_np, L.dtype)
    ws = workspace if workspace is not None else mu.marlin_make_workspace_new(torch.device(dev))
    out = ops.gptq_marlin_gemm(
        a, None, ti32(L.marlin_q), None if L.marlin_bias is None else t16(L.marlin_bias, L.dtype),
        t16(L.marlin_s, L.dtype), None, ti32(L.marlin_zp), ti32(L.g_idx), ti32(L.sort_idx), ws,
        ScalarType.from_id(L.type_id), a.shape[0], L.size_n, L.size_k, is_k_full=is_k_full,
        use_atomic_add=use_atomic_add, use_fp32_reduce=use_fp32_reduce, is_zp_float=False)
    torch.cuda.synchronize()
    assert int(ws.abs().sum().item()) == 0, "workspace not returned to zero"
    return n16(out)
