"""Operator surface of the quantized linear path.

Registers ``gptq_marlin_gemm``, ``gptq_marlin_repack``, ``awq_marlin_repack``
and ``permute_cols`` as torch custom ops with the reference's schemas
(csrc/torch_bindings.cpp:304-327) and provides the Python wrappers of
vllm/_custom_ops.py:1134-1232,1326-1334.  The operators are defined and
implemented in C++ (vllm_b200/csrc/torch_bindings.cpp, built to
lib/b200q_torch.so): argument checks, per-stream scratch, the current CUDA
stream, then the C ABI of libb200q.so, where the CUDA kernels live.  Nothing
here computes on the host, and a missing library is an import-time error.
This module adds the fake (meta) kernels and the Python-level wrappers.

Namespace: the ops are defined in ``torch.ops._C`` (the reference's namespace)
unless another extension already defined them there, in which case — or when
``VLLM_B200_OPS_NAMESPACE`` is set — they go to that / the ``b200q`` namespace.
``ops_namespace()`` tells which.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib
from .scalar_type import ScalarType

_L = _lib.load()  # raises if the CUDA library is absent


def _pick_namespace() -> str:
    forced = os.environ.get("VLLM_B200_OPS_NAMESPACE")
    if forced:
        return forced
    try:
        torch.ops._C.gptq_marlin_repack  # noqa: B018 - defined by someone else?
        return "b200q"
    except (AttributeError, RuntimeError):
        return "_C"


_NS = _pick_namespace()


def _pick_moe_namespace() -> str:
    """The reference keeps its mixture-of-experts operators in `_moe_C`."""
    try:
        torch.ops._moe_C.moe_wna16_marlin_gemm  # noqa: B018 - defined by someone else?
        return "b200q_moe"
    except (AttributeError, RuntimeError):
        return "_moe_C" if _NS == "_C" else "b200q_moe"


_MOE_NS = _pick_moe_namespace()


def _load_torch_extension(ns: str) -> None:
    path = os.path.join(os.path.dirname(_lib.LIB_PATH), "b200q_torch.so")
    if not os.path.exists(path):
        raise _lib.B200QError(
            f"{path} is missing: build it with `python -m vllm_b200.build` (g++ against this "
            "torch). The operators have no Python or CPU implementation.")
    try:
        ext = ctypes.CDLL(path)          # first by hand: dlopen's own message on failure
    except OSError as exc:
        raise _lib.B200QError(f"cannot load {path}: {exc}; rebuild it with "
                              "`python -m vllm_b200.build --force`") from exc
    torch.ops.load_library(path)         # lists it in torch.ops.loaded_libraries
    rc = ext.b200q_torch_register(ns.encode())
    if rc != 0:
        raise _lib.B200QError(f"operator names in torch.ops.{ns} are taken by another extension; "
                              "set VLLM_B200_OPS_NAMESPACE to a free namespace")
    if ext.b200q_torch_register_moe(_MOE_NS.encode()) != 0:
        raise _lib.B200QError(f"torch.ops.{_MOE_NS}.moe_wna16_marlin_gemm is taken by another extension")


_load_torch_extension(_NS)


def ops_namespace() -> str:
    return _NS


def _ptr(t: torch.Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(device: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class _on_device:
    """Make ``device`` current for the duration of a library call (the library
    launches on the current device)."""

    def __init__(self, device: torch.device):
        self.idx = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


# fake (meta) kernels: shapes only (vllm/_custom_ops.py:524-545,
# gptq_marlin_repack.cu:324-334, awq_marlin_repack.cu:250-260)
@torch.library.register_fake(f"{_NS}::gptq_marlin_gemm")
def _gptq_marlin_gemm_fake(a, c_or_none, b_q_weight, b_bias_or_none, b_scales, global_scale,
                           b_zeros_or_none, g_idx_or_none, perm_or_none, workspace, b_q_type,
                           size_m, size_n, size_k, is_k_full=True, use_atomic_add=False,
                           use_fp32_reduce=False, is_zp_float=False):
    return torch.empty((size_m, size_n), device=a.device, dtype=a.dtype)


@torch.library.register_fake(f"{_NS}::gptq_marlin_gemm_all_reduce")
def _gptq_marlin_gemm_all_reduce_fake(a, c_or_none, b_q_weight, b_bias_or_none, b_scales,
                                      global_scale, b_zeros_or_none, g_idx_or_none, perm_or_none,
                                      workspace, b_q_type, size_m, size_n, size_k, is_k_full,
                                      use_atomic_add, use_fp32_reduce, is_zp_float, peer_ptrs, state,
                                      rank, world, max_message_bytes):
    return torch.empty((size_m, size_n), device=a.device, dtype=a.dtype)


@torch.library.register_fake(f"{_NS}::gptq_marlin_repack")
def _gptq_marlin_repack_fake(b_q_weight, perm, size_k, size_n, num_bits):
    pf = 32 // num_bits
    return torch.empty((size_k // 16, size_n * 16 // pf), dtype=b_q_weight.dtype,
                       device=b_q_weight.device)


@torch.library.register_fake(f"{_NS}::awq_marlin_repack")
def _awq_marlin_repack_fake(b_q_weight, size_k, size_n, num_bits):
    pf = 32 // num_bits
    return torch.empty((size_k // 16, size_n * 16 // pf), dtype=b_q_weight.dtype,
                       device=b_q_weight.device)


@torch.library.register_fake(f"{_NS}::permute_cols")
def _permute_cols_fake(A, perm):
    return torch.empty((A.size(0), A.size(1)), dtype=A.dtype, device=A.device)


@torch.library.register_fake(f"{_MOE_NS}::moe_wna16_marlin_gemm")
def _moe_wna16_marlin_gemm_fake(a, c_or_none, b_q_weight, b_bias_or_none, b_scales, global_scale,
                                b_zeros_or_none, g_idx_or_none, perm_or_none, workspace,
                                sorted_token_ids, expert_ids, num_tokens_past_padded, topk_weights,
                                moe_block_size, top_k, mul_topk_weights, is_ep, b_q_type_id, size_m,
                                size_n, size_k, is_full_k, use_atomic_add, use_fp32_reduce, is_zp_float):
    return torch.empty((size_m * top_k, size_n), dtype=a.dtype, device=a.device)


_ops = getattr(torch.ops, _NS)
_moe_ops = getattr(torch.ops, _MOE_NS)

# ---------------------------------------------------------------------------
# Python wrappers with the reference's signatures
# ---------------------------------------------------------------------------


def gptq_marlin_repack(b_q_weight: torch.Tensor, perm: torch.Tensor, size_k: int, size_n: int,
                       num_bits: int) -> torch.Tensor:
    return _ops.gptq_marlin_repack(b_q_weight, perm, size_k, size_n, num_bits)


def awq_marlin_repack(b_q_weight: torch.Tensor, size_k: int, size_n: int,
                      num_bits: int) -> torch.Tensor:
    return _ops.awq_marlin_repack(b_q_weight, size_k, size_n, num_bits)


def gptq_marlin_moe_repack(b_q_weight: torch.Tensor, perm: torch.Tensor, size_k: int, size_n: int,
                           num_bits: int) -> torch.Tensor:
    """Per-expert loop over the dense repack (vllm/_custom_ops.py:1151-1169)."""
    num_experts = b_q_weight.shape[0]
    out = torch.empty((num_experts, size_k // 16, size_n * (num_bits // 2)),
                      device=b_q_weight.device, dtype=b_q_weight.dtype)
    for e in range(num_experts):
        out[e] = gptq_marlin_repack(b_q_weight[e], perm[e], size_k, size_n, num_bits)
    return out


def awq_marlin_moe_repack(b_q_weight: torch.Tensor, perm: torch.Tensor, size_k: int, size_n: int,
                          num_bits: int) -> torch.Tensor:
    """Per-expert loop over the dense repack (vllm/_custom_ops.py:1172-1190)."""
    num_experts = b_q_weight.shape[0]
    out = torch.empty((num_experts, size_k // 16, size_n * (num_bits // 2)),
                      device=b_q_weight.device, dtype=b_q_weight.dtype)
    for e in range(num_experts):
        out[e] = awq_marlin_repack(b_q_weight[e], size_k, size_n, num_bits)
    return out


def gptq_marlin_gemm(a: torch.Tensor, c: torch.Tensor | None, b_q_weight: torch.Tensor,
                     b_bias: torch.Tensor | None, b_scales: torch.Tensor,
                     global_scale: torch.Tensor | None, b_zeros: torch.Tensor | None,
                     g_idx: torch.Tensor | None, perm: torch.Tensor | None,
                     workspace: torch.Tensor, b_q_type: ScalarType, size_m: int, size_n: int,
                     size_k: int, is_k_full: bool = True, use_atomic_add: bool = False,
                     use_fp32_reduce: bool = False, is_zp_float: bool = False,
                     reduce_link=None) -> torch.Tensor:
    """reduce_link (not in the reference): a CustomAllreduce whose peer-memory link the op uses
    to SUM all-reduce the output across the tensor-parallel ranks (row-parallel layers): one
    operator, and at decode sizes one kernel, instead of GEMM then all-reduce."""
    if reduce_link is not None:
        return _ops.gptq_marlin_gemm_all_reduce(
            a, c, b_q_weight, b_bias, b_scales, global_scale, b_zeros, g_idx, perm, workspace,
            b_q_type.id, size_m, size_n, size_k, is_k_full, use_atomic_add, use_fp32_reduce,
            is_zp_float, reduce_link.peer_ptrs, reduce_link.state, reduce_link.rank,
            reduce_link.world_size, reduce_link.max_size)
    return _ops.gptq_marlin_gemm(a, c, b_q_weight, b_bias, b_scales, global_scale, b_zeros, g_idx,
                                 perm, workspace, b_q_type.id, size_m, size_n, size_k, is_k_full,
                                 use_atomic_add, use_fp32_reduce, is_zp_float)


def moe_wna16_marlin_gemm(input: torch.Tensor, output: torch.Tensor | None, b_qweight: torch.Tensor,
                          b_bias: torch.Tensor | None, b_scales: torch.Tensor,
                          global_scale: torch.Tensor | None, b_qzeros: torch.Tensor | None,
                          g_idx: torch.Tensor | None, perm: torch.Tensor | None,
                          workspace: torch.Tensor, sorted_token_ids: torch.Tensor,
                          expert_ids: torch.Tensor, num_tokens_past_padded: torch.Tensor,
                          topk_weights: torch.Tensor, moe_block_size: int, top_k: int,
                          mul_topk_weights: bool, is_ep: bool, b_q_type: ScalarType, size_m: int,
                          size_n: int, size_k: int, is_k_full: bool = True,
                          use_atomic_add: bool = False, use_fp32_reduce: bool = True,
                          is_zp_float: bool = False) -> torch.Tensor:
    """vllm/_custom_ops.py:1907-1963: the Marlin GEMM over blocks of tokens sorted by expert;
    returns [size_m * top_k, size_n]."""
    return _moe_ops.moe_wna16_marlin_gemm(
        input, output, b_qweight, b_bias, b_scales, global_scale, b_qzeros, g_idx, perm, workspace,
        sorted_token_ids, expert_ids, num_tokens_past_padded, topk_weights, moe_block_size, top_k,
        mul_topk_weights, is_ep, b_q_type.id, size_m, size_n, size_k, is_k_full, use_atomic_add,
        use_fp32_reduce, is_zp_float)


def _dtype_code(t: torch.Tensor) -> int:
    _check(t.dtype in (torch.float16, torch.bfloat16), "only float16 and bfloat16 are supported")
    return _lib.BF16 if t.dtype == torch.bfloat16 else _lib.F16


def fused_add_rms_norm(input: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                       epsilon: float) -> None:
    """In place: residual += input; input = rms_norm(residual) * weight
    (vllm/_custom_ops.py:336-339)."""
    _check(input.is_cuda and input.stride(-1) == 1, "input must be a CUDA tensor with unit inner stride")
    _check(residual.is_contiguous() and weight.is_contiguous(), "residual / weight must be contiguous")
    _check(residual.dtype == input.dtype == weight.dtype, "dtypes must match")
    n = input.size(-1)
    x2 = input.view(-1, n)
    with _on_device(input.device):
        rc = _L.b200q_fused_add_rms_norm(_ptr(x2), x2.stride(0), _ptr(residual), _ptr(weight),
                                         float(epsilon), x2.size(0), n, _dtype_code(input),
                                         _stream(input.device))
    _lib.check(rc, "fused_add_rms_norm")


def rms_norm(out: torch.Tensor, input: torch.Tensor, weight: torch.Tensor, epsilon: float) -> None:
    """out = rms_norm(input) * weight (vllm/_custom_ops.py:328-333)."""
    _check(out.is_contiguous() and out.shape == input.shape and out.dtype == input.dtype,
           "out must be contiguous with the shape and dtype of input")
    out.copy_(input)
    n = out.size(-1)
    with _on_device(out.device):
        rc = _L.b200q_fused_add_rms_norm(_ptr(out), n, None, _ptr(weight), float(epsilon),
                                         out.numel() // n, n, _dtype_code(out), _stream(out.device))
    _lib.check(rc, "rms_norm")


def silu_and_mul(out: torch.Tensor, input: torch.Tensor) -> None:
    """out = silu(input[..., :d]) * input[..., d:] (vllm/_custom_ops.py, torch.ops._C.silu_and_mul)."""
    d = input.size(-1) // 2
    _check(input.is_cuda and input.is_contiguous() and out.is_contiguous(), "tensors must be contiguous")
    _check(out.size(-1) == d and out.numel() * 2 == input.numel() and out.dtype == input.dtype,
           "out must be [..., d] for input [..., 2 * d]")
    with _on_device(input.device):
        rc = _L.b200q_silu_and_mul(_ptr(out), _ptr(input), out.numel() // d, d, _dtype_code(input),
                                   _stream(input.device))
    _lib.check(rc, "silu_and_mul")


def permute_cols(a: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
    return _ops.permute_cols(a, perm)
