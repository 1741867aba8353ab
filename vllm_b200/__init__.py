"""B200-native (sm_100a) weight-only quantized linear kernels behind the
reference's ``gptq_marlin_gemm`` / ``gptq_marlin_repack`` /
``awq_marlin_repack`` operator surface.

Importing the package does not load the CUDA library; ``vllm_b200._custom_ops``
does, and raises if it is missing (there is no CPU fallback).
"""

__version__ = "0.1.0"
