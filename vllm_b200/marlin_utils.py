"""Host-side preparation for the Marlin-layout quantized linear: workspace,
scale / zero-point / bias permutations, support checks and the ``apply_*``
entry points.  Mirrors the interface of
vllm/model_executor/layers/quantization/utils/marlin_utils.py (names, argument
meaning, error behaviour); the tensor work runs on whatever device the inputs
live on, with torch ops only.
"""
from __future__ import annotations

import os

import torch

from . import _custom_ops as ops
from .scalar_type import ScalarType, scalar_types

GPTQ_MARLIN_TILE = 16
GPTQ_MARLIN_MIN_THREAD_N = 64
GPTQ_MARLIN_MIN_THREAD_K = 128
GPTQ_MARLIN_MAX_PARALLEL = 16
MARLIN_SUPPORTED_GROUP_SIZES = [-1, 32, 64, 128]
USE_FP32_REDUCE_DEFAULT = True


# ---------------------------------------------------------------------------
# support queries  (marlin_utils.py:35-189)
# ---------------------------------------------------------------------------


def query_marlin_supported_quant_types(has_zp: bool | None = None,
                                       include_fp_type: bool = True,
                                       device_capability: int | None = None):
    """Weight types the GEMM accepts (marlin_utils.py:35-72, integer types
    only: the fp8 / fp4 weight types are not part of this build)."""
    if device_capability is None and torch.cuda.is_available():
        major, minor = torch.cuda.get_device_capability()
        device_capability = major * 10 + minor
    if device_capability is not None and device_capability < 100:
        return []
    if has_zp is None:
        return [scalar_types.uint4, scalar_types.uint4b8, scalar_types.uint8b128]
    if has_zp:
        return [scalar_types.uint4]
    return [scalar_types.uint4b8, scalar_types.uint8b128]


def verify_marlin_supports_shape(output_size_per_partition: int, input_size_per_partition: int,
                                 input_size: int, group_size: int) -> None:
    """marlin_utils.py:126-158 — raises ValueError on an unsupported shard."""
    if output_size_per_partition % GPTQ_MARLIN_MIN_THREAD_N != 0:
        raise ValueError(
            f"Weight output_size_per_partition = {output_size_per_partition} is not divisible "
            f"by min_thread_n = {GPTQ_MARLIN_MIN_THREAD_N}. Consider reducing "
            "tensor_parallel_size or running with --quantization gptq.")
    if input_size_per_partition % GPTQ_MARLIN_MIN_THREAD_K != 0:
        raise ValueError(
            f"Weight input_size_per_partition = {input_size_per_partition} is not divisible "
            f"by min_thread_k = {GPTQ_MARLIN_MIN_THREAD_K}. Consider reducing "
            "tensor_parallel_size or running with --quantization gptq.")
    if group_size < input_size and input_size_per_partition % group_size != 0:
        raise ValueError(
            f"Weight input_size_per_partition = {input_size_per_partition} is not divisible by "
            f"group_size = {group_size}. Consider reducing tensor_parallel_size or running "
            "with --quantization gptq.")


def check_marlin_supports_shape(output_size_per_partition: int, input_size_per_partition: int,
                                input_size: int, group_size: int) -> tuple[bool, str | None]:
    try:
        verify_marlin_supports_shape(output_size_per_partition, input_size_per_partition,
                                     input_size, group_size)
    except ValueError as e:
        return False, str(e)
    return True, None


def check_marlin_supported(quant_type: ScalarType, group_size: int, has_zp: bool = False,
                           device_capability: int | None = None) -> bool:
    supported = query_marlin_supported_quant_types(has_zp, True, device_capability)
    return quant_type in supported and group_size in MARLIN_SUPPORTED_GROUP_SIZES


# ---------------------------------------------------------------------------
# workspace and small helpers  (marlin_utils.py:237-275)
# ---------------------------------------------------------------------------


def marlin_make_workspace_new(device: torch.device, max_blocks_per_sm: int = 2) -> torch.Tensor:
    """Zero-initialised int32 counters, one per CTA the GEMM may launch.  The
    GEMM accepts any length >= #SMs (what the reference allocates,
    marlin_utils.py:237-245) and sizes its work to fit; the extra length lets the
    tensor-core kernel split K on problems with few output tiles (four counters per tile)."""
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    return torch.zeros(max(sms * max_blocks_per_sm, 1024), dtype=torch.int, device=device,
                       requires_grad=False)


def marlin_is_k_full(act_order: bool, is_row_parallel: bool) -> bool:
    return (not act_order) or (act_order and not is_row_parallel)


def marlin_repeat_scales_on_all_ranks(act_order: bool, group_size: int,
                                      is_row_parallel: bool) -> bool:
    is_channelwise = group_size == -1
    return act_order or (is_channelwise and is_row_parallel)


def marlin_make_empty_g_idx(device: torch.device) -> torch.Tensor:
    return torch.nn.Parameter(torch.empty(0, dtype=torch.int, device=device), requires_grad=False)


def marlin_make_empty_zp(device: torch.device) -> torch.Tensor:
    return torch.nn.Parameter(torch.empty(0, dtype=torch.int, device=device), requires_grad=False)


def marlin_sort_g_idx(g_idx: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    g_idx_sort_indices = torch.argsort(g_idx).to(torch.int)
    return g_idx[g_idx_sort_indices], g_idx_sort_indices


# ---------------------------------------------------------------------------
# permutations  (marlin_utils.py:278-370)
# ---------------------------------------------------------------------------


def get_scale_perms() -> tuple[list[int], list[int]]:
    # grouped: position 8*i + j of a 64-column chunk holds column i + 8*j
    scale_perm = [i + 8 * j for i in range(8) for j in range(8)]
    # channel-wise / bias: position 8*i + jj of a 32-column chunk holds column
    # 2*i + [0,1,8,9,16,17,24,25][jj]
    scale_perm_single = [2 * i + j for i in range(4) for j in (0, 1, 8, 9, 16, 17, 24, 25)]
    return scale_perm, scale_perm_single


def _idx(values, device) -> torch.Tensor:
    return torch.tensor(values, dtype=torch.long, device=device)


def marlin_permute_scales(s: torch.Tensor, size_k: int, size_n: int,
                          group_size: int) -> torch.Tensor:
    scale_perm, scale_perm_single = get_scale_perms()
    if group_size < size_k and group_size != -1:
        s = s.reshape(-1, 64)[:, _idx(scale_perm, s.device)]
    else:
        s = s.reshape(-1, 32)[:, _idx(scale_perm_single, s.device)]
    return s.reshape(-1, size_n).contiguous()


def marlin_permute_bias(s: torch.Tensor) -> torch.Tensor:
    _, scale_perm_single = get_scale_perms()
    return s.reshape(-1, 32)[:, _idx(scale_perm_single, s.device)].reshape(s.shape).contiguous()


_INTERLEAVE = {4: [0, 2, 4, 6, 1, 3, 5, 7], 8: [0, 2, 1, 3]}


def pack_cols(q_w: torch.Tensor, num_bits: int, size_k: int, size_n: int) -> torch.Tensor:
    """Pack along the last dim, value i of a word at bit i*num_bits
    (quant_utils.py:548-571)."""
    assert q_w.shape == (size_k, size_n)
    pf = 32 // num_bits
    assert size_n % pf == 0
    v = q_w.to(torch.int64).reshape(size_k, size_n // pf, pf)
    shifts = torch.arange(pf, device=q_w.device, dtype=torch.int64) * num_bits
    word = (v << shifts).sum(dim=-1) & 0xFFFFFFFF
    word = torch.where(word >= 1 << 31, word - (1 << 32), word)
    return word.to(torch.int32).contiguous()


def unpack_cols(packed_q_w: torch.Tensor, num_bits: int, size_k: int,
                size_n: int) -> torch.Tensor:
    """Inverse of pack_cols (quant_utils.py:574-602)."""
    pf = 32 // num_bits
    assert size_n % pf == 0
    assert packed_q_w.shape == (size_k, size_n // pf), (
        f"packed_q_w.shape = {tuple(packed_q_w.shape)} size_k = {size_k}, size_n = {size_n} "
        f"pack_Factor = {pf}")
    shifts = torch.arange(pf, device=packed_q_w.device, dtype=torch.int64) * num_bits
    v = (packed_q_w.to(torch.int64) & 0xFFFFFFFF).unsqueeze(-1) >> shifts
    return (v & ((1 << num_bits) - 1)).to(torch.int32).reshape(size_k, size_n).contiguous()


def marlin_zero_points(zp: torch.Tensor, size_k: int, size_n: int, num_bits: int) -> torch.Tensor:
    """Integer zero-points [size_k (= groups), size_n] -> packed Marlin
    zero-points (marlin_utils.py:326-346)."""
    scale_perm, _ = get_scale_perms()
    il = _INTERLEAVE[num_bits]
    zp = zp.reshape(-1, 64)[:, _idx(scale_perm, zp.device)]
    zp = zp.reshape(-1, len(il))[:, _idx(il, zp.device)].reshape(-1, size_n).contiguous()
    return pack_cols(zp, num_bits, size_k, size_n)


def awq_to_marlin_zero_points(q_zp_packed: torch.Tensor, size_k: int, size_n: int,
                              num_bits: int) -> torch.Tensor:
    """AWQ-packed zero-points -> Marlin zero-points (marlin_utils.py:349-370)."""
    q_zp = unpack_cols(q_zp_packed, num_bits, size_k, size_n)
    il = _INTERLEAVE[num_bits]
    undo = sorted(range(len(il)), key=il.__getitem__)
    q_zp = q_zp.reshape(-1, len(il))[:, _idx(undo, q_zp.device)].reshape(-1, size_n).contiguous()
    return marlin_zero_points(q_zp, size_k, size_n, num_bits)


def moe_awq_to_marlin_zero_points(q_zp_packed: torch.Tensor, size_k: int, size_n: int,
                                  num_bits: int) -> torch.Tensor:
    out = [awq_to_marlin_zero_points(q_zp_packed[e], size_k, size_n, num_bits)
           for e in range(q_zp_packed.shape[0])]
    return torch.stack(out)


def marlin_moe_permute_scales(s: torch.Tensor, size_k: int, size_n: int,
                              group_size: int) -> torch.Tensor:
    return torch.stack([marlin_permute_scales(s[e], size_k, size_n, group_size)
                        for e in range(s.shape[0])])


# ---------------------------------------------------------------------------
# apply  (marlin_utils.py:412-530)
# ---------------------------------------------------------------------------


def should_use_atomic_add_reduce(m: int, n: int, k: int, device: torch.device,
                                 dtype: torch.dtype) -> bool:
    """Heuristic of marlin_utils.py:412-432.  The GEMM here reduces split
    slices with a fixed-order fp32 sum whatever this returns; the flag is
    forwarded for interface fidelity."""
    if n >= 2048 or k < 2048 or device.type != "cuda":
        return False
    return os.environ.get("VLLM_MARLIN_USE_ATOMIC_ADD", "0") == "1"


def apply_gptq_marlin_linear(input: torch.Tensor, weight: torch.Tensor,
                             weight_scale: torch.Tensor, weight_zp: torch.Tensor,
                             g_idx: torch.Tensor, g_idx_sort_indices: torch.Tensor,
                             workspace: torch.Tensor, wtype: ScalarType,
                             output_size_per_partition: int, input_size_per_partition: int,
                             is_k_full: bool, bias: torch.Tensor | None = None,
                             use_fp32_reduce: bool = USE_FP32_REDUCE_DEFAULT,
                             reduce_link=None) -> torch.Tensor:
    """reduce_link (not in the reference): a peer-memory link; the output is then all-reduced
    over it by the same op (row-parallel layers)."""
    reshaped_x = input.reshape(-1, input.shape[-1])
    out_shape = input.shape[:-1] + (output_size_per_partition,)
    use_atomic_add = should_use_atomic_add_reduce(
        m=reshaped_x.size(0), n=output_size_per_partition, k=reshaped_x.size(1),
        device=input.device, dtype=input.dtype)
    output = ops.gptq_marlin_gemm(
        reshaped_x, None, weight, bias, weight_scale, None, weight_zp, g_idx,
        g_idx_sort_indices, workspace, wtype, size_m=reshaped_x.shape[0],
        size_n=output_size_per_partition, size_k=input_size_per_partition, is_k_full=is_k_full,
        use_atomic_add=use_atomic_add, use_fp32_reduce=use_fp32_reduce, is_zp_float=False,
        reduce_link=reduce_link)
    return output.reshape(out_shape)


def apply_awq_marlin_linear(input: torch.Tensor, weight: torch.Tensor,
                            weight_scale: torch.Tensor, weight_zp: torch.Tensor,
                            g_idx: torch.Tensor, g_idx_sort_indices: torch.Tensor,
                            workspace: torch.Tensor, quant_type: ScalarType,
                            output_size_per_partition: int, input_size_per_partition: int,
                            bias: torch.Tensor | None = None,
                            use_fp32_reduce: bool = USE_FP32_REDUCE_DEFAULT,
                            reduce_link=None) -> torch.Tensor:
    reshaped_x = input.reshape(-1, input.shape[-1])
    out_shape = input.shape[:-1] + (output_size_per_partition,)
    use_atomic_add = should_use_atomic_add_reduce(
        m=reshaped_x.size(0), n=output_size_per_partition, k=reshaped_x.size(1),
        device=input.device, dtype=input.dtype)
    output = ops.gptq_marlin_gemm(
        reshaped_x, None, weight, bias, weight_scale, None, weight_zp, g_idx,
        g_idx_sort_indices, workspace, quant_type, size_m=reshaped_x.shape[0],
        size_n=output_size_per_partition, size_k=input_size_per_partition,
        use_atomic_add=use_atomic_add, use_fp32_reduce=use_fp32_reduce, is_zp_float=False,
        reduce_link=reduce_link)
    return output.reshape(out_shape)
