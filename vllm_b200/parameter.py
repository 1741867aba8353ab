"""Parameters that know how they are sharded across tensor-parallel ranks.

A compact counterpart of the reference's parameter classes
(vllm/model_executor/parameter.py: ``PackedvLLMParameter``,
``GroupQuantScaleParameter``, ``ChannelQuantScaleParameter``,
``RowvLLMParameter``): the metadata is what the quantized linear methods rely on
— which dim is the input (K) dim, which the output (N) dim, and along which dim
and by what factor several codes are packed into one int32.
"""
from __future__ import annotations

import torch


class ShardedParameter(torch.nn.Parameter):
    """input_dim / output_dim: index of the K / N dimension (None = replicated
    along it); packed_dim / packed_factor: packing of sub-byte codes."""

    def __new__(cls, data: torch.Tensor, **kwargs):
        return super().__new__(cls, data=data, requires_grad=False)

    def __init__(self, data: torch.Tensor, input_dim: int | None = None,
                 output_dim: int | None = None, packed_dim: int | None = None,
                 packed_factor: int = 1, weight_loader=None):
        self.input_dim = input_dim
        self.output_dim = output_dim
        self.packed_dim = packed_dim
        self.packed_factor = packed_factor
        self.weight_loader = weight_loader

    # shard sizes / offsets given in unpacked elements are scaled down along the packed dim
    def adjust_for_packing(self, dim: int | None, size: int, offset: int) -> tuple[int, int]:
        if dim is not None and dim == self.packed_dim:
            assert size % self.packed_factor == 0 and offset % self.packed_factor == 0
            return size // self.packed_factor, offset // self.packed_factor
        return size, offset

    def load_column_parallel_weight(self, loaded: torch.Tensor, tp_rank: int, tp_size: int) -> None:
        """Shard along the output dim (parameter.py load_column_parallel_weight)."""
        if self.output_dim is None or tp_size == 1:
            self._copy(loaded)
            return
        size = self.data.shape[self.output_dim]
        self._copy(loaded.narrow(self.output_dim, tp_rank * size, size))

    def load_row_parallel_weight(self, loaded: torch.Tensor, tp_rank: int, tp_size: int) -> None:
        """Shard along the input dim; parameters without one are replicated."""
        if self.input_dim is None or tp_size == 1:
            self._copy(loaded)
            return
        size = self.data.shape[self.input_dim]
        self._copy(loaded.narrow(self.input_dim, tp_rank * size, size))

    def load_merged_column_weight(self, loaded: torch.Tensor, shard_offset: int, shard_size: int,
                                  tp_rank: int, tp_size: int) -> None:
        """One logical matrix (e.g. gate or up, q / k / v) of a fused layer: goes to
        [shard_offset, shard_offset + shard_size) of this rank's output dim; offsets are in
        unpacked output columns of the local partition (linear.py:586-700)."""
        assert self.output_dim is not None
        size, offset = self.adjust_for_packing(self.output_dim, shard_size, shard_offset)
        src = loaded
        if tp_size > 1:
            src = loaded.narrow(self.output_dim, tp_rank * size, size)
        self.data.narrow(self.output_dim, offset, size).copy_(src)

    def _copy(self, src: torch.Tensor) -> None:
        if self.data.shape != src.shape:
            raise ValueError(f"shape mismatch: parameter {tuple(self.data.shape)} vs loaded "
                             f"{tuple(src.shape)}")
        self.data.copy_(src)


def permute_param_layout_(param: ShardedParameter, input_dim: int, output_dim: int,
                          packed_dim: int | None = None) -> ShardedParameter:
    """Make (input_dim, output_dim) the parameter's dim order (2-D parameters), as
    vllm/model_executor/parameter.py:558-613 does before handing weights to a kernel."""
    cur_in, cur_out = param.input_dim, param.output_dim
    if cur_in is None or cur_out is None:
        # replicated along one dim: the data already has the canonical [in?, out] order
        param.input_dim = input_dim if cur_in is not None else None
        param.output_dim = output_dim if cur_out is not None else None
        return param
    if (cur_in, cur_out) != (input_dim, output_dim):
        param.data = param.data.t().contiguous()
        if param.packed_dim is not None:
            param.packed_dim = {cur_in: input_dim, cur_out: output_dim}[param.packed_dim]
        param.input_dim, param.output_dim = input_dim, output_dim
    if packed_dim is not None and param.packed_dim is not None:
        assert param.packed_dim == packed_dim, "unexpected packed dim"
    return param
