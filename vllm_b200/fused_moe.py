"""Mixture-of-experts layer over the Marlin GEMM, mirroring
vllm/model_executor/layers/fused_moe/fused_marlin_moe.py and moe_align_block_size.py: tokens are
sorted by expert into blocks, two grouped GEMMs (gate_up, then down with the router weights) run
over the blocks, and the top-k outputs of a token are summed."""
from __future__ import annotations

import torch

from . import _custom_ops as ops
from .marlin_utils import marlin_make_workspace_new
from .scalar_type import ScalarType, scalar_types


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int,
                         expert_map: torch.Tensor | None = None):
    """Sort the (token, slot) pairs by expert and pad every expert's run to a multiple of
    block_size (fused_moe/moe_align_block_size.py:13-86; the reference does this in a CUDA op,
    here it is a handful of torch ops on the device: no host synchronisation).
    Returns (sorted_token_ids [numel + E (block_size - 1)] padded with numel, expert_ids per block,
    num_tokens_post_padded [1])."""
    numel = topk_ids.numel()
    dev = topk_ids.device
    max_padded = numel + num_experts * (block_size - 1)
    max_blocks = -(-max_padded // block_size)
    flat = topk_ids.flatten().to(torch.int64)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)[:num_experts]
    padded = (counts + block_size - 1) // block_size * block_size
    ends = torch.cumsum(padded, 0)
    starts = ends - padded
    run_starts = torch.cumsum(counts, 0) - counts
    sorted_experts = flat[order]
    pos = starts[sorted_experts] + (torch.arange(numel, device=dev) - run_starts[sorted_experts])
    sorted_ids = torch.full((max_padded,), numel, dtype=torch.int32, device=dev)
    sorted_ids[pos] = order.to(torch.int32)
    block_first = torch.arange(max_blocks, device=dev) * block_size
    expert_ids = torch.searchsorted(ends, block_first, right=True).clamp(max=num_experts - 1)
    expert_ids = torch.where(block_first < ends[-1], expert_ids, 0).to(torch.int32)   # unused blocks: 0
    if expert_map is not None:
        expert_ids = expert_map[expert_ids.long()].to(torch.int32)
    return sorted_ids, expert_ids, ends[-1:].to(torch.int32)


def fused_marlin_moe(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
                     w1_scale: torch.Tensor, w2_scale: torch.Tensor, topk_weights: torch.Tensor,
                     topk_ids: torch.Tensor, quant_type: ScalarType = scalar_types.uint4b8,
                     bias1: torch.Tensor | None = None, bias2: torch.Tensor | None = None,
                     w1_zeros: torch.Tensor | None = None, w2_zeros: torch.Tensor | None = None,
                     global_num_experts: int = -1, expert_map: torch.Tensor | None = None,
                     apply_router_weight_on_input: bool = False,
                     workspace: torch.Tensor | None = None) -> torch.Tensor:
    """hidden_states [M, K]; w1 [E, K/16, 2N*16/pf] (gate and up), w2 [E, N/16, K*16/pf], scales
    [E, groups, 2N] / [E, groups, K] in Marlin form; topk_weights fp32 [M, topk], topk_ids
    [M, topk].  silu(gate) * up between the GEMMs; returns [M, K]
    (fused_marlin_moe.py:186-340)."""
    M, K = hidden_states.shape
    E = w1.size(0)
    topk = topk_ids.size(1)
    pf = 32 // quant_type.size_bits
    N = w2.size(1) * 16
    assert w1.size(2) // 16 * pf == 2 * N and w2.size(2) // 16 * pf == K
    assert topk_weights.dtype == torch.float32
    # the reference walks 8, 16, 32, 48, 64 (fused_marlin_moe.py:286-288); here blocks of up to 32
    # ids run the decode kernel, which is faster than the 48 / 64 path even when an expert's
    # weights are then read twice
    for block_size_m in (8, 16, 32):
        if M * topk / E / block_size_m < 0.9:
            break
    if global_num_experts == -1:
        global_num_experts = E
    sorted_ids, expert_ids, num_post_padded = moe_align_block_size(topk_ids, block_size_m,
                                                                   global_num_experts, expert_map)
    if workspace is None:
        workspace = marlin_make_workspace_new(hidden_states.device)
    tw = topk_weights.reshape(-1).contiguous()
    cache1 = ops.moe_wna16_marlin_gemm(
        hidden_states, None, w1, bias1, w1_scale, None, w1_zeros, None, None, workspace, sorted_ids,
        expert_ids, num_post_padded, tw, block_size_m, topk, apply_router_weight_on_input,
        expert_map is not None, quant_type, M, 2 * N, K)
    cache2 = torch.empty((M * topk, N), dtype=hidden_states.dtype, device=hidden_states.device)
    ops.silu_and_mul(cache2, cache1)
    out = torch.zeros((M * topk, K), dtype=hidden_states.dtype, device=hidden_states.device) \
        if expert_map is not None else None
    out = ops.moe_wna16_marlin_gemm(
        cache2, out, w2, bias2, w2_scale, None, w2_zeros, None, None, workspace, sorted_ids,
        expert_ids, num_post_padded, tw, block_size_m, 1, not apply_router_weight_on_input,
        expert_map is not None, quant_type, M * topk, K, N)
    return out.view(M, topk, K).sum(dim=1)
