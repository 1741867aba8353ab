"""Operator surface of the quantized linear path.

Registers ``gptq_marlin_gemm``, ``gptq_marlin_repack``, ``awq_marlin_repack``
and ``permute_cols`` as torch custom ops with the reference's schemas
(csrc/torch_bindings.cpp:304-327) and provides the Python wrappers of
vllm/_custom_ops.py:1134-1232,1326-1334.  The CUDA implementations live in
libb200q.so and are reached through its C ABI; nothing here computes on the
host, and a missing library is an import-time error.

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
from . import custom_all_reduce as _car
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
_libdef = torch.library.Library(_NS, "FRAGMENT")

_libdef.define(
    "gptq_marlin_gemm(Tensor a, Tensor? c_or_none, Tensor b_q_weight, "
    "Tensor? b_bias_or_none, Tensor b_scales, Tensor? global_scale, "
    "Tensor? b_zeros_or_none, Tensor? g_idx_or_none, Tensor? perm_or_none, "
    "Tensor workspace, int b_q_type, SymInt size_m, SymInt size_n, "
    "SymInt size_k, bool is_k_full, bool use_atomic_add, "
    "bool use_fp32_reduce, bool is_zp_float) -> Tensor")
_libdef.define(
    "gptq_marlin_repack(Tensor b_q_weight, Tensor perm, SymInt size_k, "
    "SymInt size_n, int num_bits) -> Tensor")
_libdef.define(
    "awq_marlin_repack(Tensor b_q_weight, SymInt size_k, SymInt size_n, "
    "int num_bits) -> Tensor")
_libdef.define("permute_cols(Tensor A, Tensor perm) -> Tensor")


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


# ---------------------------------------------------------------------------
# repack  (gptq_marlin_repack.cu:251-342, awq_marlin_repack.cu:189-268)
# ---------------------------------------------------------------------------


def _repack_out_shape(size_k: int, size_n: int, num_bits: int):
    pf = 32 // num_bits
    return (size_k // 16, size_n * 16 // pf)


def _gptq_marlin_repack_cuda(b_q_weight, perm, size_k, size_n, num_bits):
    _check(size_k % 16 == 0, f"size_k = {size_k} is not divisible by tile_k_size = 16")
    _check(size_n % 64 == 0, f"size_n = {size_n} is not divisible by tile_n_size = 64")
    _check(num_bits in (4, 8), f"num_bits must be 4 or 8. Got = {num_bits}")
    pf = 32 // num_bits
    _check(b_q_weight.is_cuda, "b_q_weight is not on GPU")
    _check(b_q_weight.is_contiguous(), "b_q_weight is not contiguous")
    _check(b_q_weight.dtype == torch.int32, "b_q_weight type is not kInt")
    _check(b_q_weight.dim() == 2 and b_q_weight.size(0) == size_k // pf,
           f"Shape mismatch: b_q_weight.size(0) = {b_q_weight.size(0)}, size_k = {size_k}, "
           f"pack_factor = {pf}")
    _check(b_q_weight.size(1) == size_n,
           f"b_q_weight.size(1) = {b_q_weight.size(1)} is not size_n = {size_n}")
    _check(perm.is_cuda, "perm is not on GPU")
    _check(perm.is_contiguous(), "perm is not contiguous")
    _check(perm.dtype == torch.int32, "perm type is not at::kInt")
    has_perm = perm.numel() > 0
    _check(not has_perm or perm.numel() == size_k, f"perm.numel() = {perm.numel()} is not size_k")
    out = torch.empty(_repack_out_shape(size_k, size_n, num_bits), dtype=torch.int32,
                      device=b_q_weight.device)
    with _on_device(b_q_weight.device):
        rc = _L.b200q_gptq_marlin_repack(_ptr(b_q_weight), _ptr(perm) if has_perm else None,
                                         _ptr(out), size_k, size_n, num_bits,
                                         _stream(b_q_weight.device))
    _lib.check(rc, "gptq_marlin_repack")
    return out


def _awq_marlin_repack_cuda(b_q_weight, size_k, size_n, num_bits):
    _check(size_k % 16 == 0, f"size_k = {size_k} is not divisible by tile_k_size = 16")
    _check(size_n % 64 == 0, f"size_n = {size_n} is not divisible by tile_n_size = 64")
    _check(num_bits in (4, 8), f"num_bits must be 4 or 8. Got = {num_bits}")
    pf = 32 // num_bits
    _check(b_q_weight.is_cuda, "b_q_weight is not on GPU")
    _check(b_q_weight.is_contiguous(), "b_q_weight is not contiguous")
    _check(b_q_weight.dtype == torch.int32, "b_q_weight type is not kInt")
    _check(b_q_weight.dim() == 2 and b_q_weight.size(0) == size_k,
           f"b_q_weight.size(0) = {b_q_weight.size(0)} is not size_k = {size_k}")
    _check(b_q_weight.size(1) == size_n // pf,
           f"Shape mismatch: b_q_weight.size(1) = {b_q_weight.size(1)}, size_n = {size_n}, "
           f"pack_factor = {pf}")
    out = torch.empty(_repack_out_shape(size_k, size_n, num_bits), dtype=torch.int32,
                      device=b_q_weight.device)
    with _on_device(b_q_weight.device):
        rc = _L.b200q_awq_marlin_repack(_ptr(b_q_weight), _ptr(out), size_k, size_n, num_bits,
                                        _stream(b_q_weight.device))
    _lib.check(rc, "awq_marlin_repack")
    return out


def _permute_cols_cuda(A, perm):
    _check(A.is_cuda and perm.is_cuda, "permute_cols: tensors must be on GPU")
    _check(A.dim() == 2 and A.stride(1) == 1, "A must be a row major tensor")
    _check(A.dtype in (torch.float16, torch.bfloat16), "A must be a 16-bit float tensor")
    _check(perm.dtype == torch.int32 and perm.is_contiguous() and perm.numel() == A.size(1),
           "perm must be a contiguous int32 tensor of A.size(1) entries")
    out = torch.empty((A.size(0), A.size(1)), dtype=A.dtype, device=A.device)
    with _on_device(A.device):
        rc = _L.b200q_permute_cols(_ptr(A), A.stride(0), _ptr(perm), _ptr(out), A.size(0),
                                   A.size(1), _stream(A.device))
    _lib.check(rc, "permute_cols")
    return out


# ---------------------------------------------------------------------------
# GEMM  (gptq_marlin.cu:674-959)
# ---------------------------------------------------------------------------


def _gptq_marlin_gemm_cuda(a, c_or_none, b_q_weight, b_bias_or_none, b_scales, global_scale,
                           b_zeros_or_none, g_idx_or_none, perm_or_none, workspace, b_q_type,
                           size_m, size_n, size_k, is_k_full, use_atomic_add, use_fp32_reduce,
                           is_zp_float):
    try:
        qt = ScalarType.from_id(b_q_type)
    except ValueError:
        raise RuntimeError(
            "b_q_type must be uint4b8, uint8b128 (has_zp = False) or u4, u8 (has_zp = True); "
            f"id {b_q_type} is not supported") from None
    pf = 32 // qt.size_bits
    _check(a.dim() == 2 and a.size(0) == size_m,
           f"Shape mismatch: a.size(0) = {a.size(0)}, size_m = {size_m}")
    _check(a.size(1) == size_k, f"Shape mismatch: a.size(1) = {a.size(1)}, size_k = {size_k}")
    _check(size_k % 16 == 0, f"size_k = {size_k} is not divisible by tile_size = 16")
    _check(size_k // 16 == b_q_weight.size(0),
           f"Shape mismatch: b_q_weight.size(0) = {b_q_weight.size(0)}, size_k = {size_k}, "
           "tile_size = 16")
    _check(b_q_weight.size(1) % 16 == 0,
           f"b_q_weight.size(1) = {b_q_weight.size(1)} is not divisible by tile_size = 16")
    actual_n = b_q_weight.size(1) // 16 * pf
    _check(size_n == actual_n, f"size_n = {size_n}, actual_size_n = {actual_n}")
    _check(a.is_cuda, "A is not on GPU")
    _check(a.stride(1) == 1, "A.stride(1) is not 1")
    _check(a.stride(0) % 8 == 0, "A.stride(0) must divisible by 8")
    _check(a.data_ptr() % 16 == 0, "A must aligned to 16 bytes")
    _check(b_q_weight.is_cuda, "b_q_weight is not on GPU")
    _check(b_q_weight.is_contiguous(), "b_q_weight is not contiguous")
    _check(b_scales.is_cuda, "b_scales is not on GPU")
    _check(b_scales.is_contiguous(), "b_scales is not contiguous")
    _check(a.dtype in (torch.float16, torch.bfloat16),
           "gpt_marlin_gemm only supports bfloat16 and float16")
    _check(b_scales.dtype == a.dtype, "b_scales must have the dtype of a")

    if c_or_none is not None:
        c = c_or_none
        _check(c.is_cuda, "c is not on GPU")
        _check(c.is_contiguous(), "c is not contiguous")
        _check(c.size(0) == size_m, f"Shape mismatch: c.size(0) = {c.size(0)}, size_m = {size_m}")
        _check(c.size(1) == size_n, f"Shape mismatch: c.size(1) = {c.size(1)}, size_n = {size_n}")
        _check(c.dtype == a.dtype, "c must have the dtype of a")
    else:
        c = torch.empty((size_m, size_n), dtype=a.dtype, device=a.device)
    if size_m == 0:
        return c

    _check(b_scales.dim() == 2, f"b_scales rank = {b_scales.dim()} is not 2")
    _check(b_scales.size(1) == size_n,
           f"b_scales dim 1 = {b_scales.size(1)} is not size_n = {size_n}")
    num_groups = b_scales.size(0)

    g_idx = perm = None
    if g_idx_or_none is not None and perm_or_none is not None:
        g_idx, perm = g_idx_or_none, perm_or_none
        _check(g_idx.is_cuda, "g_idx is not on GPU")
        _check(g_idx.is_contiguous(), "g_idx is not contiguous")
        _check(perm.is_cuda, "perm is not on GPU")
        _check(perm.is_contiguous(), "perm is not contiguous")
        _check((g_idx.size(-1) == 0 and perm.size(-1) == 0)
               or (g_idx.size(-1) == size_k and perm.size(-1) == size_k),
               f"Unexpected g_idx.size(-1) = {g_idx.size(-1)} and perm.size(-1) = "
               f"{perm.size(-1)}, where size_k = {size_k}")
        if g_idx.size(-1) == 0:
            g_idx = perm = None
        else:
            _check(g_idx.dtype == torch.int32 and perm.dtype == torch.int32,
                   "g_idx and perm must be int32")
    _check(global_scale is None, "global_scale can only be used for nvfp4 format.")

    bias = None
    if b_bias_or_none is not None:
        bias = b_bias_or_none
        _check(bias.is_cuda, "b_bias is not on GPU")
        _check(bias.is_contiguous(), "b_bias is not contiguous")
        _check(bias.size(0) == size_n, "b_bias.size(0) != size_n")
        _check(bias.dtype == a.dtype, "b_bias must have the dtype of a")

    zeros = None
    if b_zeros_or_none is not None:
        _check(b_zeros_or_none.is_cuda, "b_zeros is not on GPU")
        _check(b_zeros_or_none.is_contiguous(), "b_zeros is not contiguous")
        if b_zeros_or_none.size(-1) > 0:
            zeros = b_zeros_or_none
    if zeros is not None:
        _check(qt.bias == 0, f"b_q_type must be u4 or u8 when has_zp = True. Got = {qt}")
        _check(zeros.dim() == 2, f"b_zeros rank = {zeros.dim()} is not 2")
        _check(zeros.size(0) == num_groups,
               f"b_zeros dim 0 = {zeros.size(0)} is not num_groups = {num_groups}")
        if is_zp_float:
            _check(a.dtype == torch.float16,
                   "Computation type must be float16 (half) when using float zero points.")
            _check(zeros.size(1) == size_n, f"b_zeros dim 1 = {zeros.size(1)} is not size_n = {size_n}")
            _check(zeros.dtype == a.dtype, "float zero-points must have the dtype of a")
        else:
            _check(zeros.size(1) == size_n // pf,
                   f"b_zeros dim 1 = {zeros.size(1)} is not size_n / pack_factor = {size_n // pf}")
            _check(zeros.dtype == torch.int32, "b_zeros must be int32")
    else:
        _check(qt.bias != 0 or qt.is_floating_point(),
               "b_q_type must be uint4b8, uint8b128, float8_e4m3fn or float4_e2m1f when "
               f"has_zp = False. Got = {qt}")

    _check(size_n % 64 == 0, f"size_n = {size_n}, is not divisible by min_thread_n = 64")
    _check(workspace.is_cuda and workspace.dtype == torch.int32, "workspace must be int32 on GPU")
    with _on_device(a.device):
        sms = _L.b200q_sm_count()
        _check(workspace.numel() >= sms,
               f"workspace.numel = {workspace.numel()} is below min_workspace_size = {sms}")
        nbytes = _L.b200q_marlin_gemm_preferred_scratch_bytes(size_m, size_n, size_k,
                                                             int(g_idx is not None))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=a.device)
        flags = ((_lib.FLAG_K_FULL if is_k_full else 0)
                 | (_lib.FLAG_ATOMIC_ADD if use_atomic_add else 0)
                 | (_lib.FLAG_FP32_REDUCE if use_fp32_reduce else 0)
                 | (_lib.FLAG_ZP_FLOAT if (is_zp_float and zeros is not None) else 0))
        args = (_ptr(a), a.stride(0), _ptr(b_q_weight), _ptr(b_scales), _ptr(zeros), _ptr(g_idx),
                _ptr(perm), _ptr(bias), _ptr(c), _ptr(scratch), nbytes, _ptr(workspace),
                workspace.numel(), b_q_type, _lib.BF16 if a.dtype == torch.bfloat16 else _lib.F16,
                size_m, size_n, size_k, num_groups, flags)
        scope = _car.active_scope()
        if scope is not None and scope.accepts(c):
            # row-parallel layer: the GEMM all-reduces its own output over the peer link
            rc = _L.b200q_marlin_gemm_all_reduce(*args, *scope.link_args(), _stream(a.device))
            scope.done = True
        else:
            rc = _L.b200q_marlin_gemm(*args, _stream(a.device))
    _lib.check(rc, "gptq_marlin_gemm")
    return c


_libdef.impl("gptq_marlin_gemm", _gptq_marlin_gemm_cuda, "CUDA")
_libdef.impl("gptq_marlin_repack", _gptq_marlin_repack_cuda, "CUDA")
_libdef.impl("awq_marlin_repack", _awq_marlin_repack_cuda, "CUDA")
_libdef.impl("permute_cols", _permute_cols_cuda, "CUDA")


# fake (meta) kernels: shapes only (vllm/_custom_ops.py:524-545,
# gptq_marlin_repack.cu:324-334, awq_marlin_repack.cu:250-260)
@torch.library.register_fake(f"{_NS}::gptq_marlin_gemm")
def _gptq_marlin_gemm_fake(a, c_or_none, b_q_weight, b_bias_or_none, b_scales, global_scale,
                           b_zeros_or_none, g_idx_or_none, perm_or_none, workspace, b_q_type,
                           size_m, size_n, size_k, is_k_full=True, use_atomic_add=False,
                           use_fp32_reduce=False, is_zp_float=False):
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


_ops = getattr(torch.ops, _NS)

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
                     use_fp32_reduce: bool = False, is_zp_float: bool = False) -> torch.Tensor:
    return _ops.gptq_marlin_gemm(a, c, b_q_weight, b_bias, b_scales, global_scale, b_zeros, g_idx,
                                 perm, workspace, b_q_type.id, size_m, size_n, size_k, is_k_full,
                                 use_atomic_add, use_fp32_reduce, is_zp_float)


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
