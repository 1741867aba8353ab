"""GPTQ checkpoints on the Marlin kernels: config and linear method.  Parameter
shapes, sharding rules and the load -> repack -> apply life cycle follow
vllm/model_executor/layers/quantization/gptq_marlin.py:92-466 (linear layers only)."""
from __future__ import annotations

import torch

from vllm_b200 import _custom_ops as ops
from vllm_b200.marlin_utils import (apply_gptq_marlin_linear, check_marlin_supported,
                                    marlin_is_k_full, marlin_make_empty_g_idx,
                                    marlin_make_workspace_new, marlin_permute_bias,
                                    marlin_permute_scales, marlin_repeat_scales_on_all_ranks,
                                    marlin_sort_g_idx, verify_marlin_supports_shape)
from vllm_b200.parameter import ShardedParameter
from vllm_b200.scalar_type import scalar_types


class GPTQMarlinConfig:
    # (num_bits, is_sym) -> quant_type
    TYPE_MAP = {(4, True): scalar_types.uint4b8, (8, True): scalar_types.uint8b128}

    def __init__(self, weight_bits: int, group_size: int, desc_act: bool, is_sym: bool = True,
                 lm_head_quantized: bool = False) -> None:
        if desc_act and group_size == -1:
            # no reordering is needed when there is a single group (gptq_marlin.py:118-121)
            desc_act = False
        if (weight_bits, is_sym) not in self.TYPE_MAP:
            raise ValueError(f"Unsupported quantization config: bits={weight_bits}, sym={is_sym}")
        self.weight_bits = weight_bits
        self.pack_factor = 32 // weight_bits
        self.group_size = group_size
        self.desc_act = desc_act
        self.is_sym = is_sym
        self.lm_head_quantized = lm_head_quantized
        self.quant_type = self.TYPE_MAP[(weight_bits, is_sym)]
        if not check_marlin_supported(self.quant_type, group_size, has_zp=False,
                                      device_capability=100):
            raise ValueError(f"GPTQ config not supported by Marlin: {self}")

    @classmethod
    def from_config(cls, config: dict) -> "GPTQMarlinConfig":
        return cls(config["bits"], config["group_size"], config.get("desc_act", False),
                   config.get("sym", True), config.get("lm_head", False))

    @classmethod
    def get_name(cls) -> str:
        return "gptq_marlin"

    def get_quant_method(self, layer: torch.nn.Module, prefix: str = ""):
        return GPTQMarlinLinearMethod(self)

    def __repr__(self) -> str:
        return (f"GPTQMarlinConfig(quant_type={self.quant_type}, group_size={self.group_size}, "
                f"desc_act={self.desc_act}, lm_head_quantized={self.lm_head_quantized})")


class GPTQMarlinLinearMethod:
    supports_reduce_link = True   # apply() can all-reduce its output over a peer link

    def __init__(self, quant_config: GPTQMarlinConfig) -> None:
        self.quant_config = quant_config

    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int,
                       output_partition_sizes: list[int], input_size: int, output_size: int,
                       params_dtype: torch.dtype, **extra_weight_attrs) -> None:
        qc = self.quant_config
        output_size_per_partition = sum(output_partition_sizes)
        is_row_parallel = input_size != input_size_per_partition
        weight_loader = extra_weight_attrs.get("weight_loader")
        device = extra_weight_attrs.get("device")
        verify_marlin_supports_shape(output_size_per_partition, input_size_per_partition,
                                     input_size, qc.group_size if qc.group_size != -1 else input_size)
        group_size = qc.group_size if qc.group_size != -1 else input_size
        if marlin_repeat_scales_on_all_ranks(qc.desc_act, qc.group_size, is_row_parallel):
            scales_input_dim, scales_size = None, input_size // group_size       # replicated
        else:
            scales_input_dim, scales_size = 0, input_size_per_partition // group_size

        layer.register_parameter("qweight", ShardedParameter(
            torch.empty(input_size_per_partition // qc.pack_factor, output_size_per_partition,
                        dtype=torch.int32, device=device),
            input_dim=0, output_dim=1, packed_dim=0, packed_factor=qc.pack_factor,
            weight_loader=weight_loader))
        layer.register_parameter("g_idx", ShardedParameter(
            torch.empty(input_size_per_partition, dtype=torch.int32, device=device),
            input_dim=0, weight_loader=weight_loader))
        layer.register_parameter("scales", ShardedParameter(
            torch.empty(scales_size, output_size_per_partition, dtype=params_dtype, device=device),
            input_dim=scales_input_dim, output_dim=1, weight_loader=weight_loader))
        layer.register_parameter("qzeros", ShardedParameter(
            torch.empty(scales_size, output_size_per_partition // qc.pack_factor,
                        dtype=torch.int32, device=device),
            input_dim=scales_input_dim, output_dim=1, packed_dim=1, packed_factor=qc.pack_factor,
            weight_loader=weight_loader))
        # what the load -> repack -> apply steps below need to know about the shard
        layer.input_size_per_partition = input_size_per_partition
        layer.output_size_per_partition = output_size_per_partition
        layer.is_k_full = marlin_is_k_full(qc.desc_act, is_row_parallel)

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        """Checkpoint layout -> kernel layout, once per layer: sort the act-order groups,
        repack the codes on the device (rows visited in sorted order), permute scales and
        bias.  The symmetric types carry no zero-points (qzeros is dropped)."""
        qc = self.quant_config
        device = layer.qweight.device
        k, n = layer.input_size_per_partition, layer.output_size_per_partition

        def replace(name, data):
            delattr(layer, name)
            layer.register_parameter(name, torch.nn.Parameter(data, requires_grad=False))

        layer.workspace = marlin_make_workspace_new(device)
        if qc.desc_act:
            g_idx, sort_indices = marlin_sort_g_idx(layer.g_idx.data)
        else:
            g_idx = sort_indices = marlin_make_empty_g_idx(device)
        replace("g_idx", g_idx)
        layer.g_idx_sort_indices = sort_indices
        replace("qweight", ops.gptq_marlin_repack(layer.qweight.data.contiguous(), perm=sort_indices,
                                                   size_k=k, size_n=n, num_bits=qc.weight_bits))
        replace("scales", marlin_permute_scales(layer.scales.data.contiguous(), size_k=k, size_n=n,
                                                group_size=qc.group_size))
        replace("qzeros", marlin_make_empty_g_idx(device))
        if getattr(layer, "bias", None) is not None:
            layer.bias.data = marlin_permute_bias(layer.bias)

    def apply(self, layer: torch.nn.Module, x: torch.Tensor,
              bias: torch.Tensor | None = None, reduce_link=None) -> torch.Tensor:
        return apply_gptq_marlin_linear(
            input=x, weight=layer.qweight, weight_scale=layer.scales, weight_zp=layer.qzeros,
            g_idx=layer.g_idx, g_idx_sort_indices=layer.g_idx_sort_indices,
            workspace=layer.workspace, wtype=self.quant_config.quant_type,
            input_size_per_partition=layer.input_size_per_partition,
            output_size_per_partition=layer.output_size_per_partition,
            is_k_full=layer.is_k_full, bias=bias, reduce_link=reduce_link)
