"""Low-latency all-reduce for the row-parallel output at decode sizes.

Mirrors the role (and the interface names) of the reference's ``CustomAllreduce``
(vllm/distributed/device_communicators/custom_all_reduce.py:50-283): small
messages are reduced by one kernel over peer-mapped buffers instead of NCCL.
The peer mapping comes from torch's symmetric-memory allocator (plumbing); the
kernel is ``b200q_all_reduce`` of this package.  Larger messages, or a group
without peer access, fall back to the NCCL process group in
``vllm_b200.distributed``.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib


class CustomAllreduce:
    # messages above this go to NCCL (the reference caps its one-stage kernel at 256-512 KiB,
    # csrc/custom_all_reduce.cuh:592-593, and the whole path at 1-2 MiB on compute capability 10.0)
    def __init__(self, group, device: torch.device, max_size: int = 1 << 19) -> None:
        import torch.distributed._symmetric_memory as symm_mem
        self.lib = _lib.load()
        self.group = group
        self.device = device
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self.max_size = max_size
        self.disabled = True
        if self.world_size < 2 or self.world_size > 8:
            return
        symm_mem.enable_symm_mem_for_group(group.group_name)
        self.data = symm_mem.empty(self.lib.b200q_all_reduce_buffer_bytes(self.world_size, max_size),
                                   dtype=torch.uint8, device=device)
        self.data_hdl = symm_mem.rendezvous(self.data, group.group_name)
        nflag = self.lib.b200q_all_reduce_flag_bytes() // 4
        self.flags = symm_mem.empty(nflag, dtype=torch.int32, device=device)
        self.flags.zero_()
        self.flags_hdl = symm_mem.rendezvous(self.flags, group.group_name)
        self.epochs = torch.zeros(self.lib.b200q_all_reduce_epoch_bytes() // 4, dtype=torch.int32,
                                  device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)          # every rank's flags are zero before anyone signals
        self.disabled = False

    def should_custom_ar(self, inp: torch.Tensor) -> bool:
        if self.disabled or not inp.is_cuda or inp.dtype not in (torch.float16, torch.bfloat16):
            return False
        nbytes = inp.numel() * inp.element_size()
        return (nbytes % 16 == 0 and 0 < nbytes <= self.max_size and inp.is_contiguous()
                and inp.data_ptr() % 16 == 0)

    def custom_all_reduce(self, inp: torch.Tensor) -> torch.Tensor | None:
        """Out-of-place SUM all-reduce, or None when the input does not qualify.  The input is
        read where it is (no staging copy): the kernel pushes it into the peers' buffers."""
        if not self.should_custom_ar(inp):
            return None
        out = torch.empty_like(inp)
        vp = ctypes.c_void_p
        rc = self.lib.b200q_all_reduce(
            vp(self.data_hdl.buffer_ptrs_dev), vp(self.flags_hdl.buffer_ptrs_dev),
            vp(self.epochs.data_ptr()), self.rank, self.world_size, self.max_size,
            vp(inp.data_ptr()), vp(out.data_ptr()), inp.numel(),
            _lib.BF16 if inp.dtype == torch.bfloat16 else _lib.F16,
            vp(torch.cuda.current_stream(self.device).cuda_stream))
        _lib.check(rc, "b200q_all_reduce")
        return out
