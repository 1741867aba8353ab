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
import os

import torch
import torch.distributed as dist

from . import _lib


class CustomAllreduce:
    # messages above this go to NCCL: 2 MiB, the reference's cap for its own peer-memory path on
    # compute capability 10.0 (vllm/distributed/device_communicators/all_reduce_utils.py:40-45)
    def __init__(self, group, device: torch.device, max_size: int = 1 << 21) -> None:
        # The kernels use plain peer stores only.  Without this setting torch's rendezvous also
        # binds the buffer to an NVLink multicast object, which nothing here needs and which
        # must not outlive a rank that exits while its peers still run.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
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
        self.data.zero_()                  # flag 0 marks a packet that was never written
        self.data_hdl = symm_mem.rendezvous(self.data, group.group_name)
        self.state = torch.zeros(self.lib.b200q_all_reduce_state_bytes() // 4, dtype=torch.int32,
                                 device=device)
        # the ranks' receive buffers as a device tensor, for the torch op that takes the link
        self.peer_ptrs = torch.tensor(list(self.data_hdl.buffer_ptrs), dtype=torch.int64,
                                      device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)          # every rank's buffer is zero before anyone sends
        self.disabled = False

    def close(self) -> None:
        """Drop the symmetric buffer and its handle; the object stays, disabled."""
        self.disabled = True
        self.data_hdl = None
        self.data = None
        self.state = None
        self.peer_ptrs = None

    def fits(self, rows: int, cols: int, dtype: torch.dtype) -> bool:
        """Whether a [rows, cols] output of this dtype can be all-reduced over the link."""
        nbytes = rows * cols * 2
        return (not self.disabled and dtype in (torch.float16, torch.bfloat16)
                and nbytes % 16 == 0 and 0 < nbytes <= self.max_size)

    def link_args(self) -> tuple:
        """The link as the C ABI takes it (peer_bufs, state, rank, world, max_message_bytes)."""
        vp = ctypes.c_void_p
        return (vp(self.peer_ptrs.data_ptr()), vp(self.state.data_ptr()), self.rank,
                self.world_size, self.max_size)

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
            vp(self.peer_ptrs.data_ptr()), vp(self.state.data_ptr()), self.rank,
            self.world_size, self.max_size,
            vp(inp.data_ptr()), vp(out.data_ptr()), inp.numel(),
            _lib.BF16 if inp.dtype == torch.bfloat16 else _lib.F16,
            vp(torch.cuda.current_stream(self.device).cuda_stream))
        _lib.check(rc, "b200q_all_reduce")
        return out

    def all_reduce_add_rms_norm(self, inp: torch.Tensor, residual: torch.Tensor | None,
                                weight: torch.Tensor, epsilon: float) -> bool:
        """In place and in one kernel: inp = all_reduce(inp); residual += inp;
        inp = rms_norm(residual) * weight (residual None: plain rms_norm of the sum).
        Returns False (nothing done) when the input does not qualify."""
        if not self.should_custom_ar(inp) or inp.size(-1) % 8 != 0:
            return False
        n = inp.size(-1)
        vp = ctypes.c_void_p
        rc = self.lib.b200q_all_reduce_fused_add_rms_norm(
            vp(self.peer_ptrs.data_ptr()), vp(self.state.data_ptr()), self.rank,
            self.world_size, self.max_size, vp(inp.data_ptr()),
            vp(residual.data_ptr()) if residual is not None else None, vp(weight.data_ptr()),
            float(epsilon), inp.numel() // n, n,
            _lib.BF16 if inp.dtype == torch.bfloat16 else _lib.F16,
            vp(torch.cuda.current_stream(self.device).cuda_stream))
        _lib.check(rc, "b200q_all_reduce_fused_add_rms_norm")
        return True
