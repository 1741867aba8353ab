"""Host-side helpers for float4_e2m1f weights on the Marlin path (NVFP4: fp8-e4m3 scales per 16
values and one global scale; MXFP4: e8m0 scales per 32), mirroring
vllm/model_executor/layers/quantization/utils/marlin_utils_fp4.py: the scale layout and value
transforms the kernel expects, random test weights, layer preparation and the apply function."""
from __future__ import annotations

import torch

from . import _custom_ops as ops
from .marlin_utils import (USE_FP32_REDUCE_DEFAULT, marlin_make_workspace_new, marlin_permute_bias,
                           marlin_permute_scales, should_use_atomic_add_reduce)
from .scalar_type import scalar_types

FP4_MARLIN_SUPPORTED_GROUP_SIZES = [16]


def is_fp4_marlin_supported() -> bool:
    return torch.cuda.is_available()


def _regroup_index(size_n: int, device) -> torch.Tensor:
    """src[F]: which element of a pair of permuted scale rows (rr * N + p0) lands at byte F of the
    pair's 2 N-byte block.  A thread's eight scales of both groups of the pair become 16 adjacent
    bytes, and the middle two of every four change places (the order the kernel's byte-to-16-bit
    expansion returns them in; marlin_utils_fp4.py:41-50)."""
    f = torch.arange(2 * size_n, device=device)
    swap = torch.tensor([0, 2, 1, 3], device=device)
    lin = (f & ~3) | swap[f & 3]
    return ((lin % 16) // 8) * size_n + 8 * (lin // 16) + lin % 8


def _regroup(marlin_scales: torch.Tensor) -> torch.Tensor:
    groups, size_n = marlin_scales.shape
    assert groups % 2 == 0, "fp4 scales are regrouped in pairs of groups"
    pairs = marlin_scales.reshape(groups // 2, 2 * size_n)
    return pairs[:, _regroup_index(size_n, marlin_scales.device)].reshape(groups, size_n)


def nvfp4_marlin_process_scales(marlin_scales: torch.Tensor) -> torch.Tensor:
    """Permuted scales [G, N] -> float8_e4m3fn-typed bytes in the kernel's layout.  The scales
    are assumed non-negative: s * 2^7 as fp16 then has its top exponent bit set whenever s > 0,
    and bits 14..7 of it (five exponent, three mantissa bits) are what is stored
    (marlin_utils_fp4.py:28-62)."""
    s = _regroup(marlin_scales.to(torch.half))
    bits = (s * (2 ** 7)).view(torch.int16).to(torch.int32) & 0xFFFF
    return ((bits >> 7) & 0xFF).to(torch.uint8).view(torch.float8_e4m3fn)


def mxfp4_marlin_process_scales(marlin_scales: torch.Tensor) -> torch.Tensor:
    """Permuted power-of-two scales [G, N] -> float8_e8m0fnu in the kernel's layout
    (marlin_utils_fp4.py:65-77)."""
    return _regroup(marlin_scales).to(torch.float8_e8m0fnu)


def nvfp4_marlin_process_global_scale(global_scale: torch.Tensor) -> torch.Tensor:
    """The kernel leaves the fp4 exponent un-rebiased (2^-14 as fp16, 2^-126 as bf16) and the
    stored scales carry a factor 2^7: the global scale makes up for both
    (marlin_utils_fp4.py:80-90)."""
    assert global_scale.dtype in (torch.half, torch.bfloat16)
    bias = 14 if global_scale.dtype == torch.half else 126
    return global_scale * (2.0 ** (bias - 7))


def apply_fp4_marlin_linear(input: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
                            weight_scale_2: torch.Tensor | None, workspace: torch.Tensor,
                            size_n: int, size_k: int, bias: torch.Tensor | None = None,
                            use_fp32_reduce: bool = USE_FP32_REDUCE_DEFAULT) -> torch.Tensor:
    """marlin_utils_fp4.py:93-133."""
    x = input.reshape(-1, input.shape[-1])
    use_atomic_add = should_use_atomic_add_reduce(m=x.size(0), n=size_n, k=size_k,
                                                  device=input.device, dtype=input.dtype)
    out = ops.gptq_marlin_gemm(x, None, weight, bias, weight_scale, weight_scale_2, None, None, None,
                               workspace, scalar_types.float4_e2m1f, x.size(0), size_n, size_k,
                               use_atomic_add=use_atomic_add, use_fp32_reduce=use_fp32_reduce)
    return out.reshape(input.shape[:-1] + (size_n,))


def _fp4_codes_to_dtype(codes: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    table = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=dtype, device=codes.device)
    mag = table[(codes & 7).long()]
    return torch.where((codes & 8) != 0, -mag, mag)


def _repack_fp4(fp4_bytes: torch.Tensor, size_k: int, size_n: int) -> torch.Tensor:
    """[N, K / 2] bytes (low nibble first) -> Marlin layout through the 4-bit repack operator."""
    packed = fp4_bytes.view(torch.int32).T.contiguous()
    return ops.gptq_marlin_repack(packed, torch.empty(0, dtype=torch.int, device=fp4_bytes.device),
                                  size_k, size_n, 4)


def rand_marlin_weight_nvfp4_like(weight: torch.Tensor, group_size: int):
    """Random fp4 codes with scales shaped like `weight`'s ([N, K]); returns (weight_ref [K, N],
    marlin_qweight, marlin_scales, global_scale) as marlin_utils_fp4.py:304-349."""
    size_n, size_k = weight.shape
    scales = weight.view(size_n, -1, group_size).abs().max(-1)[0] / 6
    global_scale = scales.max() / 448
    scales = (scales / global_scale).to(torch.float8_e4m3fn)
    fp4 = torch.randint(0, 256, (size_n, size_k // 2), dtype=torch.uint8, device=weight.device)
    lo, hi = _fp4_codes_to_dtype(fp4 & 15, weight.dtype), _fp4_codes_to_dtype(fp4 >> 4, weight.dtype)
    ref = torch.stack([lo, hi], dim=2).view(size_n, size_k)
    ref = ref * global_scale.to(weight.dtype) * scales.repeat_interleave(group_size, 1).to(weight.dtype)
    marlin_scales = nvfp4_marlin_process_scales(
        marlin_permute_scales(scales.T.to(weight.dtype), size_k, size_n, group_size))
    return (ref.T, _repack_fp4(fp4, size_k, size_n), marlin_scales,
            nvfp4_marlin_process_global_scale(global_scale.to(weight.dtype)))


def rand_marlin_weight_mxfp4_like(weight: torch.Tensor, group_size: int):
    """As above with e8m0 scales 2^-27 .. 2^-3 and no global scale (marlin_utils_fp4.py:352-397)."""
    size_n, size_k = weight.shape
    scales = torch.randint(100, 125, (size_n, size_k // group_size), dtype=torch.uint8,
                           device=weight.device).view(torch.float8_e8m0fnu)
    fp4 = torch.randint(0, 256, (size_n, size_k // 2), dtype=torch.uint8, device=weight.device)
    lo, hi = _fp4_codes_to_dtype(fp4 & 15, weight.dtype), _fp4_codes_to_dtype(fp4 >> 4, weight.dtype)
    ref = torch.stack([lo, hi], dim=2).view(size_n, size_k)
    ref = ref * scales.repeat_interleave(group_size, 1).to(weight.dtype)
    marlin_scales = mxfp4_marlin_process_scales(
        marlin_permute_scales(scales.T.to(weight.dtype), size_k, size_n, group_size))
    return ref.T, _repack_fp4(fp4, size_k, size_n), marlin_scales


def prepare_fp4_layer_for_marlin(layer: torch.nn.Module) -> None:
    """Repack layer.weight ([N, K / 2] bytes) and bring layer.weight_scale (and, for NVFP4,
    layer.weight_scale_2) into the kernel's form (marlin_utils_fp4.py:136-200)."""
    n, k = layer.output_size_per_partition, layer.input_size_per_partition
    is_nvfp4 = hasattr(layer, "weight_scale_2")
    group_size = 16 if is_nvfp4 else 32
    dtype = layer.params_dtype
    device = layer.weight.device
    layer.workspace = marlin_make_workspace_new(device)
    layer.weight = torch.nn.Parameter(_repack_fp4(layer.weight.data, k, n), requires_grad=False)
    scales = layer.weight_scale.data.T.contiguous()
    scales = scales.to(dtype) if is_nvfp4 else scales.view(torch.float8_e8m0fnu).to(dtype)
    scales = marlin_permute_scales(scales, k, n, group_size)
    if is_nvfp4:
        layer.weight_scale = torch.nn.Parameter(nvfp4_marlin_process_scales(scales), requires_grad=False)
        layer.weight_scale_2 = torch.nn.Parameter(
            nvfp4_marlin_process_global_scale(layer.weight_scale_2.data.to(dtype)), requires_grad=False)
    else:
        layer.weight_scale = torch.nn.Parameter(mxfp4_marlin_process_scales(scales), requires_grad=False)
    if getattr(layer, "bias", None) is not None:
        layer.bias = torch.nn.Parameter(marlin_permute_bias(layer.bias.data), requires_grad=False)
