"""AWQ checkpoints on the Marlin kernels: config and linear method
(vllm/model_executor/layers/quantization/awq_marlin.py:66-413, linear layers only).
AWQ packs along the output dim with its own nibble interleave and always carries
zero-points; there is no act-order."""
from __future__ import annotations

import torch

from vllm_b200 import _custom_ops as ops
from vllm_b200.marlin_utils import (apply_awq_marlin_linear, awq_to_marlin_zero_points,
                                    check_marlin_supported, marlin_make_empty_g_idx,
                                    marlin_make_workspace_new, marlin_permute_bias,
                                    marlin_permute_scales, verify_marlin_supports_shape)
from vllm_b200.parameter import ShardedParameter
from vllm_b200.scalar_type import scalar_types


class AWQMarlinConfig:
    TYPE_MAP = {4: scalar_types.uint4, 8: scalar_types.uint8}

    def __init__(self, weight_bits: int, group_size: int, zero_point: bool = True,
                 lm_head_quantized: bool = False) -> None:
        if weight_bits not in self.TYPE_MAP:
            raise ValueError(f"Unsupported num_bits = {weight_bits}")
        if not zero_point:
            raise ValueError("AWQ Marlin needs zero_point = True")
        self.weight_bits = weight_bits
        self.pack_factor = 32 // weight_bits
        self.group_size = group_size
        self.zero_point = zero_point
        self.lm_head_quantized = lm_head_quantized
        self.quant_type = self.TYPE_MAP[weight_bits]
        if not check_marlin_supported(self.quant_type, group_size, has_zp=True,
                                      device_capability=100):
            raise ValueError(f"AWQ config not supported by Marlin: {self}")

    @classmethod
    def from_config(cls, config: dict) -> "AWQMarlinConfig":
        return cls(config["bits"], config["group_size"], config.get("zero_point", True),
                   config.get("lm_head", False))

    @classmethod
    def get_name(cls) -> str:
        return "awq_marlin"

    def get_quant_method(self, layer: torch.nn.Module, prefix: str = ""):
        return AWQMarlinLinearMethod(self)

    def __repr__(self) -> str:
        return (f"AWQMarlinConfig(quant_type={self.quant_type}, group_size={self.group_size}, "
                f"zero_point={self.zero_point})")


class AWQMarlinLinearMethod:
    supports_reduce_link = True   # apply() can all-reduce its output over a peer link

    def __init__(self, quant_config: AWQMarlinConfig) -> None:
        self.quant_config = quant_config

    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int,
                       output_partition_sizes: list[int], input_size: int, output_size: int,
                       params_dtype: torch.dtype, **extra_weight_attrs) -> None:
        qc = self.quant_config
        output_size_per_partition = sum(output_partition_sizes)
        weight_loader = extra_weight_attrs.get("weight_loader")
        device = extra_weight_attrs.get("device")
        group_size = qc.group_size if qc.group_size != -1 else input_size
        verify_marlin_supports_shape(output_size_per_partition, input_size_per_partition,
                                     input_size, group_size)
        num_groups = input_size_per_partition // group_size
        layer.register_parameter("qweight", ShardedParameter(
            torch.empty(input_size_per_partition, output_size_per_partition // qc.pack_factor,
                        dtype=torch.int32, device=device),
            input_dim=0, output_dim=1, packed_dim=1, packed_factor=qc.pack_factor,
            weight_loader=weight_loader))
        layer.register_parameter("qzeros", ShardedParameter(
            torch.empty(num_groups, output_size_per_partition // qc.pack_factor,
                        dtype=torch.int32, device=device),
            input_dim=0, output_dim=1, packed_dim=1, packed_factor=qc.pack_factor,
            weight_loader=weight_loader))
        layer.register_parameter("scales", ShardedParameter(
            torch.empty(num_groups, output_size_per_partition, dtype=params_dtype, device=device),
            input_dim=0, output_dim=1, weight_loader=weight_loader))
        layer.input_size_per_partition = input_size_per_partition
        layer.output_size_per_partition = output_size_per_partition
        layer.num_groups = num_groups

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        qc = self.quant_config
        device = layer.qweight.device
        k, n = layer.input_size_per_partition, layer.output_size_per_partition

        def replace(name, data):
            delattr(layer, name)
            layer.register_parameter(name, torch.nn.Parameter(data, requires_grad=False))

        layer.workspace = marlin_make_workspace_new(device)
        replace("qweight", ops.awq_marlin_repack(layer.qweight.data.contiguous(), size_k=k,
                                                  size_n=n, num_bits=qc.quant_type.size_bits))
        replace("scales", marlin_permute_scales(layer.scales.data, size_k=k, size_n=n,
                                                group_size=qc.group_size))
        replace("qzeros", awq_to_marlin_zero_points(layer.qzeros.data, size_k=layer.num_groups,
                                                    size_n=n, num_bits=qc.quant_type.size_bits))
        layer.g_idx = marlin_make_empty_g_idx(device)
        layer.g_idx_sort_indices = marlin_make_empty_g_idx(device)
        if getattr(layer, "bias", None) is not None:
            layer.bias.data = marlin_permute_bias(layer.bias)

    def apply(self, layer: torch.nn.Module, x: torch.Tensor,
              bias: torch.Tensor | None = None, reduce_link=None) -> torch.Tensor:
        return apply_awq_marlin_linear(
            input=x, weight=layer.qweight, weight_scale=layer.scales, weight_zp=layer.qzeros,
            g_idx=layer.g_idx, g_idx_sort_indices=layer.g_idx_sort_indices,
            workspace=layer.workspace, quant_type=self.quant_config.quant_type,
            output_size_per_partition=layer.output_size_per_partition,
            input_size_per_partition=layer.input_size_per_partition, bias=bias,
            reduce_link=reduce_link)
