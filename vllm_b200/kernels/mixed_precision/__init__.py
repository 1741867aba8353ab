"""Kernel selection for weight-only quantized linears.  The reference walks a
priority list of backends (kernels/mixed_precision/__init__.py:36-105) and ends up
on Marlin on compute capability 10.0; this build has exactly one backend."""
from __future__ import annotations

import os

from .marlin import MarlinLinearKernel
from .MPLinearKernel import MPLinearKernel, MPLinearLayerConfig

_POSSIBLE_KERNELS: list[type[MPLinearKernel]] = [MarlinLinearKernel]


def choose_mp_linear_kernel(config: MPLinearLayerConfig,
                            compute_capability: int | None = None) -> type[MPLinearKernel]:
    disabled = os.environ.get("VLLM_DISABLED_KERNELS", "").split(",")
    failure_reasons = []
    for kernel in _POSSIBLE_KERNELS:
        if kernel.__name__ in disabled:
            failure_reasons.append(f" {kernel.__name__} disabled by environment variable")
            continue
        if compute_capability is not None and kernel.get_min_capability() > compute_capability:
            failure_reasons.append(f"{kernel.__name__} requires capability "
                                   f"{kernel.get_min_capability()}, current compute capability "
                                   f"is {compute_capability}")
            continue
        ok, reason = kernel.can_implement(config)
        if ok:
            return kernel
        failure_reasons.append(f" {kernel.__name__} cannot implement due to: {reason}")
    raise ValueError("Failed to find a kernel that can implement the WNA16 linear layer. "
                     "Reasons: \n" + "\n".join(failure_reasons))


__all__ = ["MPLinearKernel", "MPLinearLayerConfig", "MarlinLinearKernel", "choose_mp_linear_kernel"]
