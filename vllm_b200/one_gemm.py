"""Run one quantized GEMM shape a few times (uint4b8, group 128, bf16): the small,
self-contained process to put under a profiler.

    python -m vllm_b200.one_gemm K N M [repeats]
"""
import sys

import torch
from vllm_b200 import _custom_ops as ops, marlin_utils as mu
from vllm_b200.scalar_type import scalar_types as st


def main():
    K, N, M = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    reps = int(sys.argv[4]) if len(sys.argv) > 4 else 4
    dt = torch.bfloat16
    dev = torch.device("cuda")
    ws = mu.marlin_make_workspace_new(dev)
    q = torch.randint(-2**31, 2**31 - 1, (K // 16, N * 2), dtype=torch.int32, device=dev)
    s = (torch.rand((K // 128, N), device=dev) * 0.018 + 0.002).to(dt)
    a = torch.randn((M, K), device=dev, dtype=dt)
    e = torch.empty(0, dtype=torch.int32, device=dev)
    for _ in range(reps):
        out = ops.gptq_marlin_gemm(a, None, q, None, s, None, e, e, e, ws, st.uint4b8, M, N, K, True, False, True, False)
    torch.cuda.synchronize()
    print("done", out.float().abs().mean().item())


if __name__ == "__main__":
    main()
