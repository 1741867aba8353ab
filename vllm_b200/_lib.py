"""ctypes loader for libb200q.so — the C ABI declared in include/b200q.h.

The library is looked up in-tree (``vllm_b200/lib``).  A missing library is a
hard error: there is no fallback path.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libb200q.so")

# names that include/b200q.h declares; checked at load time
EXPORTS = (
    "b200q_last_error",
    "b200q_version",
    "b200q_sm_count",
    "b200q_kernel_launches",
    "b200q_device_error",
    "b200q_gptq_marlin_repack",
    "b200q_awq_marlin_repack",
    "b200q_permute_cols",
    "b200q_marlin_gemm_scratch_bytes",
    "b200q_marlin_gemm_preferred_scratch_bytes",
    "b200q_marlin_gemm",
    "b200q_marlin_gemm_fp4",
    "b200q_moe_wna16_marlin_gemm",
    "b200q_marlin_gemm_noalloc_max_scratch",
    "b200q_marlin_gemm_noalloc",
    "b200q_all_reduce_state_bytes",
    "b200q_all_reduce_buffer_bytes",
    "b200q_all_reduce_set_poll_limit",
    "b200q_all_reduce",
    "b200q_marlin_gemm_all_reduce",
    "b200q_fused_add_rms_norm",
    "b200q_all_reduce_fused_add_rms_norm",
    "b200q_silu_and_mul",
)

OK, EINVAL, EUNSUPPORTED, ECUDA, ESCRATCH = 0, -1, -2, -3, -4
F16, BF16 = 0, 1
FLAG_K_FULL, FLAG_ATOMIC_ADD, FLAG_FP32_REDUCE, FLAG_ZP_FLOAT = 1, 2, 4, 8
FP4_SCALES_E4M3, FP4_SCALES_E8M0 = 1, 2

_lib = None


class B200QError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise B200QError(
            f"{LIB_PATH} is missing: build it with `python -m vllm_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for these ops.")
    lib = ctypes.CDLL(LIB_PATH)
    missing = [n for n in EXPORTS if not hasattr(lib, n)]
    if missing:
        raise B200QError(f"{LIB_PATH} lacks symbols {missing}; rebuild it")
    c = ctypes
    vp, i64, i32, u32 = c.c_void_p, c.c_int64, c.c_int, c.c_uint
    lib.b200q_last_error.restype = c.c_char_p
    lib.b200q_last_error.argtypes = []
    lib.b200q_version.restype = i32
    lib.b200q_sm_count.restype = i32
    lib.b200q_kernel_launches.restype = c.c_ulonglong
    lib.b200q_device_error.restype = i32
    lib.b200q_device_error.argtypes = [i32]
    lib.b200q_kernel_launches.argtypes = []
    lib.b200q_gptq_marlin_repack.restype = i32
    lib.b200q_gptq_marlin_repack.argtypes = [vp, vp, vp, i64, i64, i32, vp]
    lib.b200q_awq_marlin_repack.restype = i32
    lib.b200q_awq_marlin_repack.argtypes = [vp, vp, i64, i64, i32, vp]
    lib.b200q_permute_cols.restype = i32
    lib.b200q_permute_cols.argtypes = [vp, i64, vp, vp, i64, i64, vp]
    lib.b200q_marlin_gemm_scratch_bytes.restype = c.c_size_t
    lib.b200q_marlin_gemm_scratch_bytes.argtypes = [i64, i64, i64, i32]
    lib.b200q_marlin_gemm_preferred_scratch_bytes.restype = c.c_size_t
    lib.b200q_marlin_gemm_preferred_scratch_bytes.argtypes = [i64, i64, i64, i32]
    lib.b200q_marlin_gemm.restype = i32
    lib.b200q_marlin_gemm.argtypes = [
        vp, i64, vp, vp, vp, vp, vp, vp, vp, vp, c.c_size_t, vp, i64, i64, i32,
        i64, i64, i64, i64, u32, vp]
    lib.b200q_marlin_gemm_fp4.restype = i32
    lib.b200q_marlin_gemm_fp4.argtypes = [
        vp, i64, vp, vp, vp, i32, vp, vp, vp, c.c_size_t, vp, i64, i32, i64, i64, i64, i64, vp]
    lib.b200q_moe_wna16_marlin_gemm.restype = i32
    lib.b200q_moe_wna16_marlin_gemm.argtypes = [
        vp, i64, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i32, i64, i64, i32, i64, i64,
        i64, i64, vp]
    lib.b200q_marlin_gemm_all_reduce.restype = i32
    lib.b200q_marlin_gemm_all_reduce.argtypes = [
        vp, i64, vp, vp, vp, vp, vp, vp, vp, vp, c.c_size_t, vp, i64, i64, i32,
        i64, i64, i64, i64, u32, vp, vp, i32, i32, i64, vp]
    lib.b200q_marlin_gemm_noalloc_max_scratch.restype = c.c_size_t
    lib.b200q_marlin_gemm_noalloc_max_scratch.argtypes = []
    lib.b200q_marlin_gemm_noalloc.restype = i32
    lib.b200q_marlin_gemm_noalloc.argtypes = [
        vp, i64, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, i64, i64, i64, i64, u32, vp]
    lib.b200q_all_reduce_state_bytes.restype = c.c_size_t
    lib.b200q_all_reduce.restype = i32
    lib.b200q_fused_add_rms_norm.restype = i32
    lib.b200q_fused_add_rms_norm.argtypes = [vp, i64, vp, vp, c.c_float, i64, i64, i32, vp]
    lib.b200q_all_reduce_fused_add_rms_norm.restype = i32
    lib.b200q_all_reduce_fused_add_rms_norm.argtypes = [vp, vp, i32, i32, i64, vp, vp, vp, c.c_float,
                                                        i64, i64, i32, vp]
    lib.b200q_silu_and_mul.restype = i32
    lib.b200q_silu_and_mul.argtypes = [vp, vp, i64, i64, i32, vp]
    lib.b200q_all_reduce_set_poll_limit.restype = None
    lib.b200q_all_reduce_set_poll_limit.argtypes = [c.c_uint32]
    lib.b200q_all_reduce_buffer_bytes.restype = c.c_size_t
    lib.b200q_all_reduce_buffer_bytes.argtypes = [i32, i64]
    lib.b200q_all_reduce.argtypes = [vp, vp, i32, i32, i64, vp, vp, i64, i32, vp]
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    """Turn a non-zero status into the exception type the reference op raises
    (TORCH_CHECK -> RuntimeError, TORCH_CHECK_NOT_IMPLEMENTED ->
    NotImplementedError)."""
    if status == OK:
        return
    msg = load().b200q_last_error().decode("utf-8", "replace")
    if status == EUNSUPPORTED:
        raise NotImplementedError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: {msg}")
