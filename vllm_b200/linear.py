"""Tensor-parallel linear layers over a pluggable (quantized) linear method.

Follows the reference's layer contract (vllm/model_executor/layers/linear.py):
``ColumnParallelLinear`` shards the output dim and needs no collective,
``RowParallelLinear`` shards the input dim and all-reduces its output
(linear.py:1388-1416); the quant method owns ``create_weights``,
``process_weights_after_loading`` and ``apply`` (linear.py:155-193).  Weights
are sharded in checkpoint format and each shard is repacked on its own rank.
"""
from __future__ import annotations

import torch

from . import distributed as D
import torch.nn.functional as F

from .distributed import (divide, reduce_link, get_tensor_model_parallel_rank,
                          get_tensor_model_parallel_world_size, tensor_model_parallel_all_gather,
                          tensor_model_parallel_all_reduce)
from .parameter import ShardedParameter


class UnquantizedLinearMethod:
    """Plain 16-bit weights [out, in] and torch's matmul."""

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size,
                       output_size, params_dtype, **extra_weight_attrs):
        layer.register_parameter("weight", ShardedParameter(
            torch.empty(sum(output_partition_sizes), input_size_per_partition, dtype=params_dtype,
                        device=extra_weight_attrs.get("device")),
            input_dim=1, output_dim=0, weight_loader=extra_weight_attrs.get("weight_loader")))

    def process_weights_after_loading(self, layer):
        pass

    def apply(self, layer, x, bias=None):
        return F.linear(x, layer.weight, bias)


class LinearBase(torch.nn.Module):
    def __init__(self, input_size: int, output_size: int, params_dtype: torch.dtype | None = None,
                 quant_config=None, prefix: str = "", device=None,
                 tp_rank: int | None = None, tp_size: int | None = None):
        super().__init__()
        self.input_size, self.output_size = input_size, output_size
        self.params_dtype = params_dtype or torch.get_default_dtype()
        self.prefix = prefix
        self.device = device
        # explicit rank / size let one process build several shards (tests, single-GPU emulation)
        self.tp_size = tp_size if tp_size is not None else get_tensor_model_parallel_world_size()
        self.tp_rank = tp_rank if tp_rank is not None else get_tensor_model_parallel_rank()
        self.quant_method = (quant_config.get_quant_method(self, prefix=prefix)
                             if quant_config is not None else UnquantizedLinearMethod())

    def process_weights_after_loading(self) -> None:
        self.quant_method.process_weights_after_loading(self)


class ColumnParallelLinear(LinearBase):
    """Y = X A + b with A split along its output dim: rank i holds A_i, computes Y_i = X A_i
    (linear.py:414-583)."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False,
                 gather_output: bool = False, output_sizes: list[int] | None = None, **kw):
        super().__init__(input_size, output_size, **kw)
        self.gather_output = gather_output
        self.output_sizes = output_sizes or [output_size]
        self.output_partition_sizes = [divide(s, self.tp_size) for s in self.output_sizes]
        self.output_size_per_partition = sum(self.output_partition_sizes)
        self.input_size_per_partition = input_size
        self.quant_method.create_weights(
            layer=self, input_size_per_partition=input_size,
            output_partition_sizes=self.output_partition_sizes, input_size=input_size,
            output_size=output_size, params_dtype=self.params_dtype,
            weight_loader=self.weight_loader, device=self.device)
        if bias:
            self.bias = ShardedParameter(
                torch.zeros(self.output_size_per_partition, dtype=self.params_dtype,
                            device=self.device), output_dim=0, weight_loader=self.weight_loader)
        else:
            self.register_parameter("bias", None)

    def weight_loader(self, param: ShardedParameter, loaded_weight: torch.Tensor,
                      loaded_shard_id: int | None = None) -> None:
        """loaded_shard_id selects one of the fused logical matrices (``output_sizes``); the
        loaded tensor is that matrix in full (all ranks' columns)."""
        if loaded_shard_id is None:
            if len(self.output_sizes) == 1:
                param.load_column_parallel_weight(loaded_weight, self.tp_rank, self.tp_size)
                return
            # a fused checkpoint tensor: split it into its logical matrices first
            offset = 0
            for i, size in enumerate(self.output_sizes):
                s, o = param.adjust_for_packing(param.output_dim, size, offset)
                part = loaded_weight if param.output_dim is None else \
                    loaded_weight.narrow(param.output_dim, o, s)
                self.weight_loader(param, part, i)
                offset += size
            return
        if param.output_dim is None:
            param.load_column_parallel_weight(loaded_weight, self.tp_rank, self.tp_size)
            return
        shard_offset = sum(self.output_partition_sizes[:loaded_shard_id])
        shard_size = self.output_partition_sizes[loaded_shard_id]
        param.load_merged_column_weight(loaded_weight, shard_offset, shard_size, self.tp_rank,
                                        self.tp_size)

    def forward(self, input_: torch.Tensor) -> torch.Tensor:
        out = self.quant_method.apply(self, input_, self.bias)
        if self.gather_output and self.tp_size > 1:
            out = tensor_model_parallel_all_gather(out)
        return out


class MergedColumnParallelLinear(ColumnParallelLinear):
    """Several column-parallel matrices fused along the output dim (gate_up_proj;
    linear.py:586)."""

    def __init__(self, input_size: int, output_sizes: list[int], **kw):
        super().__init__(input_size, sum(output_sizes), output_sizes=list(output_sizes), **kw)


class QKVParallelLinear(ColumnParallelLinear):
    """Fused q / k / v projection (linear.py:867): heads are split across ranks; KV heads are
    replicated when there are fewer of them than ranks."""

    def __init__(self, hidden_size: int, head_size: int, total_num_heads: int,
                 total_num_kv_heads: int | None = None, **kw):
        total_num_kv_heads = total_num_kv_heads or total_num_heads
        tp = kw.get("tp_size") or get_tensor_model_parallel_world_size()
        if total_num_kv_heads < tp:
            raise NotImplementedError("KV-head replication (fewer KV heads than ranks)")
        self.head_size = head_size
        self.num_heads = divide(total_num_heads, tp)
        self.num_kv_heads = divide(total_num_kv_heads, tp)
        sizes = [total_num_heads * head_size, total_num_kv_heads * head_size,
                 total_num_kv_heads * head_size]
        super().__init__(hidden_size, sum(sizes), output_sizes=sizes, **kw)


class RowParallelLinear(LinearBase):
    """Y = X A + b with A split along its input dim and X along its last dim: rank i computes
    X_i A_i, the partial results are summed by an all-reduce (linear.py:1242-1424).  Bias is
    added on rank 0 only, before the reduction (linear.py:1404)."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False,
                 input_is_parallel: bool = True, reduce_results: bool = True, **kw):
        super().__init__(input_size, output_size, **kw)
        self.input_is_parallel = input_is_parallel
        self.reduce_results = reduce_results
        self.input_size_per_partition = divide(input_size, self.tp_size)
        self.output_size_per_partition = output_size
        self.quant_method.create_weights(
            layer=self, input_size_per_partition=self.input_size_per_partition,
            output_partition_sizes=[output_size], input_size=input_size, output_size=output_size,
            params_dtype=self.params_dtype, weight_loader=self.weight_loader, device=self.device)
        if bias:
            self.bias = ShardedParameter(torch.zeros(output_size, dtype=self.params_dtype,
                                                     device=self.device),
                                         weight_loader=self.weight_loader)
        else:
            self.register_parameter("bias", None)

    def weight_loader(self, param: ShardedParameter, loaded_weight: torch.Tensor,
                      loaded_shard_id=None) -> None:
        param.load_row_parallel_weight(loaded_weight, self.tp_rank, self.tp_size)

    def forward(self, input_: torch.Tensor, all_reduce=tensor_model_parallel_all_reduce,
                reduce: bool = True) -> torch.Tensor:
        """reduce=False returns this rank's partial sum (for a caller that fuses the all-reduce
        with what follows, e.g. residual add + RMSNorm)."""
        if not self.input_is_parallel and self.tp_size > 1:
            input_ = input_.chunk(self.tp_size, dim=-1)[self.tp_rank].contiguous()
        bias = self.bias if (self.tp_rank == 0 or self.tp_size == 1) else None
        if not (reduce and self.reduce_results and self.tp_size > 1):
            return self.quant_method.apply(self, input_, bias)
        if all_reduce is not tensor_model_parallel_all_reduce:
            return all_reduce(self.quant_method.apply(self, input_, bias))
        # GEMM -> all-reduce is one op (one kernel at decode sizes) where the peer link is up
        # and the output fits its slots
        link = reduce_link()
        rows = input_.numel() // input_.shape[-1]
        if (link is not None and getattr(self.quant_method, "supports_reduce_link", False)
                and link.fits(rows, self.output_size_per_partition, input_.dtype)):
            return self.quant_method.apply(self, input_, bias, reduce_link=link)
        if input_.dim() == 2 and rows >= D.OVERLAP_MIN_ROWS and input_.is_cuda:
            # many rows: NCCL's all-reduce of one block of rows runs beside the GEMM of the next
            return D.overlapped_row_parallel(lambda x: self.quant_method.apply(self, x, bias), input_)
        return all_reduce(self.quant_method.apply(self, input_, bias))
