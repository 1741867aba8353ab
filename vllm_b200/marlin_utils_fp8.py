"""Host-side helpers for float8_e4m3fn weights on the Marlin path (W8A16-fp8), mirroring
vllm/model_executor/layers/quantization/utils/marlin_utils_fp8.py: packing of fp8 weights into
the 8-bit GPTQ word format, the exponent re-bias factor that rides on the scales, the CPU
reference quantiser used by the tests, and the linear apply function."""
from __future__ import annotations

import torch

from . import _custom_ops as ops
from .marlin_utils import (USE_FP32_REDUCE_DEFAULT, marlin_make_workspace_new,
                           marlin_permute_scales, should_use_atomic_add_reduce)
from .scalar_type import scalar_types


def is_fp8_marlin_supported() -> bool:
    return torch.cuda.is_available()


def fp8_fused_exponent_bias_into_scales(scales: torch.Tensor) -> torch.Tensor:
    """The kernel moves the fp8 exponent field into the 16-bit format without re-biasing; the
    factor 2^(bias16 - bias8) = 2^8 (fp16) / 2^120 (bf16) is folded into the scales
    (marlin_utils_fp8.py:26-37)."""
    target_exponent = {torch.float16: 5, torch.bfloat16: 8}[scales.dtype]
    exponent_bias = 2 ** (target_exponent - 1) - 2 ** (4 - 1)
    return scales * (torch.ones_like(scales) * 2) ** exponent_bias


def pack_fp8_to_int32(fp8_tensor: torch.Tensor, size_k_first: bool = True) -> torch.Tensor:
    """fp8 weights -> int32 words of four consecutive K values (GPTQ 8-bit packing,
    marlin_utils_fp8.py:304-318).  Returns [K / 4, N] for size_k_first, else [N, K / 4]."""
    assert fp8_tensor.dtype == torch.float8_e4m3fn and fp8_tensor.ndim == 2
    t = (fp8_tensor.T if size_k_first else fp8_tensor).contiguous()    # [N, K]
    words = t.view(torch.int32)                                         # [N, K / 4]
    return words.T.contiguous() if size_k_first else words


def marlin_quant_fp8_torch(weight: torch.Tensor, group_size: int):
    """Per-group (or per-channel, group_size = -1) absmax quantisation of weight [N, K] to fp8,
    Marlin repack and scale preparation (marlin_utils_fp8.py:321-352).  Returns
    (weight_ref [K, N], marlin_qweight, marlin_scales)."""
    size_n, size_k = weight.shape
    g = size_k if group_size == -1 else group_size
    scales = weight.view(size_n, -1, g).abs().max(-1)[0] / 448
    rep = scales.repeat_interleave(g, 1)
    fp8_weight = (weight / rep).to(torch.float8_e4m3fn)
    weight_ref = fp8_weight.to(weight.dtype) * rep
    packed = pack_fp8_to_int32(fp8_weight, False).T.contiguous()
    marlin_qweight = ops.gptq_marlin_repack(
        packed, torch.empty(0, dtype=torch.int, device=weight.device), size_k, size_n, 8)
    marlin_scales = fp8_fused_exponent_bias_into_scales(
        marlin_permute_scales(scales.T.contiguous(), size_k, size_n, group_size))
    return weight_ref.T, marlin_qweight, marlin_scales


def prepare_fp8_layer_for_marlin(layer: torch.nn.Module, size_k_first: bool = True) -> None:
    """Repack layer.weight (fp8, [K, N] or [N, K]) and prepare layer.weight_scale (per tensor,
    per channel or per group) for the kernel (marlin_utils_fp8.py:82-170; block-wise scales of
    other shapes are not handled here)."""
    n, k = layer.output_size_per_partition, layer.input_size_per_partition
    device = layer.weight.device
    layer.workspace = marlin_make_workspace_new(device)
    qweight = pack_fp8_to_int32(layer.weight, size_k_first)
    if not size_k_first:
        qweight = qweight.T.contiguous()
    layer.weight = torch.nn.Parameter(
        ops.gptq_marlin_repack(qweight, torch.empty(0, dtype=torch.int, device=device), k, n, 8),
        requires_grad=False)
    scales = layer.weight_scale.to(layer.orig_dtype)
    if scales.numel() == 1:                       # per tensor
        scales = scales.view(1, 1).repeat_interleave(n, 1)
    elif scales.numel() == n:                     # per channel
        scales = scales.view(1, n)
    else:                                         # per group: [N, K / g] or [K / g, N]
        scales = scales if scales.shape[-1] == n else scales.T
    group_size = -1 if scales.shape[0] == 1 else k // scales.shape[0]
    marlin_scales = marlin_permute_scales(scales.contiguous(), k, n, group_size)
    layer.weight_scale = torch.nn.Parameter(fp8_fused_exponent_bias_into_scales(marlin_scales),
                                            requires_grad=False)


def apply_fp8_marlin_linear(input: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
                            workspace: torch.Tensor, size_n: int, size_k: int,
                            bias: torch.Tensor | None,
                            use_fp32_reduce: bool = USE_FP32_REDUCE_DEFAULT) -> torch.Tensor:
    """marlin_utils_fp8.py:40-79."""
    reshaped_x = input.reshape(-1, input.shape[-1])
    out_shape = input.shape[:-1] + (size_n,)
    use_atomic_add = should_use_atomic_add_reduce(m=reshaped_x.size(0), n=size_n, k=size_k,
                                                  device=input.device, dtype=input.dtype)
    output = ops.gptq_marlin_gemm(
        reshaped_x, None, weight, bias, weight_scale, None, None, None, None, workspace,
        scalar_types.float8_e4m3fn, size_m=reshaped_x.size(0), size_n=size_n, size_k=size_k,
        use_atomic_add=use_atomic_add, use_fp32_reduce=use_fp32_reduce)
    return output.reshape(out_shape)
