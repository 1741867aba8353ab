"""Tensor-parallel group state and the row-parallel all-reduce.

One process per GPU; the group is a ``torch.distributed`` process group (NCCL
over NVLink / NVSwitch on GPUs, gloo in CPU tests).  Mirrors the call chain
``tensor_model_parallel_all_reduce`` -> ``GroupCoordinator.all_reduce`` of the
reference (vllm/distributed/communication_op.py:12-14,
vllm/distributed/parallel_state.py:452-479): out-of-place semantics, a no-op
for a group of one.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_TP_GROUP = None
_TP_RANK = 0
_TP_SIZE = 1
_CUSTOM_AR = None


def initialize_model_parallel(tensor_model_parallel_size: int | None = None, group=None) -> None:
    """Use the default (or given) process group as the TP group.  TP ranks are
    the innermost dimension of the rank layout, as in
    vllm/distributed/parallel_state.py:1262-1275; only TP is modelled here."""
    global _TP_GROUP, _TP_RANK, _TP_SIZE
    if not dist.is_initialized():
        _TP_GROUP, _TP_RANK, _TP_SIZE = None, 0, 1
        return
    _TP_GROUP = group if group is not None else dist.group.WORLD
    _TP_SIZE = dist.get_world_size(_TP_GROUP)
    _TP_RANK = dist.get_rank(_TP_GROUP)
    if tensor_model_parallel_size is not None and tensor_model_parallel_size != _TP_SIZE:
        raise ValueError(f"tensor_model_parallel_size = {tensor_model_parallel_size} but the "
                         f"process group has {_TP_SIZE} ranks")


def enable_custom_all_reduce(device: torch.device, max_size: int = 1 << 21) -> bool:
    """Set up the peer-memory all-reduce for small messages (decode).  Collective: call on
    every rank after initialize_model_parallel.  Returns whether it is active."""
    global _CUSTOM_AR
    if _TP_SIZE < 2:
        return False
    from .custom_all_reduce import CustomAllreduce
    _CUSTOM_AR = CustomAllreduce(_TP_GROUP, device, max_size)
    return not _CUSTOM_AR.disabled


def reduce_link():
    """The peer-memory link of the TP group (a CustomAllreduce), or None when it is not up.
    A row-parallel layer hands it to the quantized GEMM op that all-reduces its own output
    (gptq_marlin_gemm_all_reduce) where the output fits (link.fits)."""
    if _CUSTOM_AR is None or _CUSTOM_AR.disabled:
        return None
    return _CUSTOM_AR


def destroy_model_parallel() -> None:
    """Forget the group and release the peer-memory buffers (call on every rank, with no
    kernel of this rank still using the link)."""
    global _TP_GROUP, _TP_RANK, _TP_SIZE, _CUSTOM_AR
    if _CUSTOM_AR is not None:
        _CUSTOM_AR.close()
    _TP_GROUP, _TP_RANK, _TP_SIZE, _CUSTOM_AR = None, 0, 1, None


def get_tensor_model_parallel_world_size() -> int:
    return _TP_SIZE


def get_tensor_model_parallel_rank() -> int:
    return _TP_RANK


def tensor_model_parallel_all_reduce(input_: torch.Tensor) -> torch.Tensor:
    """SUM all-reduce over the TP group; returns a new tensor (the reference's op
    is out-of-place, parallel_state.py:117-126)."""
    if _TP_SIZE == 1:
        return input_
    if _CUSTOM_AR is not None:
        out = _CUSTOM_AR.custom_all_reduce(input_)
        if out is not None:
            return out
    out = input_.clone()
    dist.all_reduce(out, op=dist.ReduceOp.SUM, group=_TP_GROUP)
    return out


_OVERLAP_STREAMS: dict = {}
# measured on 2 B200s: below 8192 rows the blocks are too short for NCCL's kernel to find free SMs
# beside the persistent GEMM kernel (4096 rows, o-proj: 232 us plain, 254 us in two blocks, 380 us
# in four), at 8192 rows four blocks win (down-proj of the 70B shard, alternating runs on one box: 1681 / 1734 us
# plain, 1576 / 1635 us in four blocks, 1755 us in two)
OVERLAP_MIN_ROWS = 8192
OVERLAP_CHUNKS = 4


def overlapped_row_parallel(gemm, input_: torch.Tensor, chunks: int = OVERLAP_CHUNKS) -> torch.Tensor:
    """Row-parallel GEMM over many rows with the collective hidden behind the compute: the rows are
    cut into `chunks` blocks, block j's all-reduce (NCCL, on a second stream) runs while block
    j + 1 is multiplied.  `gemm(x_block) -> partial output block`.  Works under CUDA-graph capture
    (the second stream forks from and joins the capturing stream)."""
    rows = input_.shape[0]
    step = -(-rows // chunks)
    cur = torch.cuda.current_stream(input_.device)
    key = (input_.device.index, cur.cuda_stream)
    side = _OVERLAP_STREAMS.get(key)
    if side is None:
        side = _OVERLAP_STREAMS[key] = torch.cuda.Stream(device=input_.device)
    outs = []
    for r0 in range(0, rows, step):
        part = gemm(input_[r0:r0 + step])
        done = torch.cuda.Event()
        done.record(cur)
        with torch.cuda.stream(side):
            side.wait_event(done)
            dist.all_reduce(part, op=dist.ReduceOp.SUM, group=_TP_GROUP)
        part.record_stream(side)
        outs.append(part)
    cur.wait_stream(side)
    return torch.cat(outs, dim=0) if len(outs) > 1 else outs[0]


def tensor_model_parallel_all_gather(input_: torch.Tensor, dim: int = -1) -> torch.Tensor:
    if _TP_SIZE == 1:
        return input_
    parts = [torch.empty_like(input_) for _ in range(_TP_SIZE)]
    dist.all_gather(parts, input_.contiguous(), group=_TP_GROUP)
    return torch.cat(parts, dim=dim)


def divide(numerator: int, denominator: int) -> int:
    if numerator % denominator != 0:
        raise ValueError(f"{numerator} is not divisible by {denominator}")
    return numerator // denominator
