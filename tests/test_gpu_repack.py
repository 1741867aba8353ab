"""GPU parity: repack ops and permute_cols against the CPU oracle, bit-exact.
Shapes follow the reference's tests/kernels/quantization/test_marlin_gemm.py:88-209
and tests/kernels/core/test_permute_cols.py."""
import glob
import os

import numpy as np
import pytest

from oracle import marlin_oracle as mo
from tests import helpers as H

pytestmark = pytest.mark.gpu

MNK_FACTORS = [(1, 1, 1), (1, 4, 8), (26, 37, 13), (257, 13, 11)]


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_utils as G
    from vllm_b200 import _custom_ops as ops
    assert torch.cuda.is_available()
    return torch, G, ops


@pytest.mark.parametrize("n_chunk", [64, 256])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("act_order", [False, True])
@pytest.mark.parametrize("mnk", MNK_FACTORS)
def test_gptq_marlin_repack(env, n_chunk, bits, act_order, mnk):
    torch, G, ops = env
    _, nf, kf = mnk
    K, N = 128 * kf, n_chunk * nf
    rng = np.random.default_rng(K * 131 + N + bits)
    q = rng.integers(0, 1 << bits, size=(K, N), dtype=np.int32)
    packed = mo.gptq_pack(q, bits)
    if act_order:
        g_idx = (np.arange(K) // 32)[rng.permutation(K)].astype(np.int32)
        _, sort_idx = mo.sort_g_idx(g_idx)
    else:
        sort_idx = None
    want = mo.gptq_marlin_repack(packed, sort_idx, K, N, bits)
    got = ops.gptq_marlin_repack(G.ti32(packed), G.ti32(sort_idx), K, N, bits)
    torch.cuda.synchronize()
    assert got.dtype == torch.int32 and tuple(got.shape) == want.shape
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("n_chunk", [64, 256])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("mnk", MNK_FACTORS)
def test_awq_marlin_repack(env, n_chunk, bits, mnk):
    torch, G, ops = env
    _, nf, kf = mnk
    K, N = 128 * kf, n_chunk * nf
    rng = np.random.default_rng(K * 17 + N + bits)
    q = rng.integers(0, 1 << bits, size=(K, N), dtype=np.int32)
    packed = mo.awq_pack(q, bits)
    want = mo.awq_marlin_repack(packed, K, N, bits)
    got = ops.awq_marlin_repack(G.ti32(packed), K, N, bits)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "repack_*.npz"))))
def test_repack_golden(env, path):
    """Device ops against the fixtures recorded from the reference packers."""
    torch, G, ops = env
    g = np.load(path)
    bits = int(os.path.basename(path).split("_")[1][1:])
    K, N = g["q"].shape
    got = ops.gptq_marlin_repack(G.ti32(g["gptq_in"]), G.ti32(None), K, N, bits).cpu().numpy()
    assert np.array_equal(got, g["expect"])
    got = ops.gptq_marlin_repack(G.ti32(g["gptq_in"]), G.ti32(g["sort_idx"]), K, N, bits).cpu().numpy()
    assert np.array_equal(got, g["expect_perm"])
    got = ops.awq_marlin_repack(G.ti32(g["awq_in"]), K, N, bits).cpu().numpy()
    assert np.array_equal(got, g["expect"])


def test_repack_full_size_roundtrip(env):
    """Llama-3-70B gate_up shard width at full K: the device repack must decode
    back to the packed input (size-independent property; the oracle is only run
    on a corner)."""
    torch, G, ops = env
    K, N, bits = 8192, 7168, 4
    gen = torch.Generator(device="cuda").manual_seed(0)
    packed = torch.randint(-2**31, 2**31 - 1, (K // 8, N), dtype=torch.int32, device="cuda", generator=gen)
    out = ops.gptq_marlin_repack(packed, G.ti32(None), K, N, bits)
    torch.cuda.synchronize()
    # checksum: every nibble value must occur equally often in input and output
    def nibble_hist(t):
        u = t.view(torch.uint8).flatten()
        lo = torch.bincount((u & 15).to(torch.int64), minlength=16)
        hi = torch.bincount((u >> 4).to(torch.int64), minlength=16)
        return (lo + hi).cpu().numpy()
    assert np.array_equal(nibble_hist(packed), nibble_hist(out))
    corner_in = packed[:32, :128].cpu().numpy()          # 256 rows x 128 cols
    want = mo.gptq_marlin_repack(np.ascontiguousarray(corner_in), None, 256, 128, 4)
    got = out[:16].cpu().numpy().reshape(16, N // 64, 128)[:, :2, :].reshape(16, 256)
    assert np.array_equal(got, want)


def test_repack_rejects_bad_shapes(env):
    torch, G, ops = env
    x = torch.zeros((16, 64), dtype=torch.int32, device="cuda")
    empty = G.ti32(None)
    with pytest.raises(RuntimeError):
        ops.gptq_marlin_repack(x, empty, 120, 64, 4)      # size_k % 16
    with pytest.raises(RuntimeError):
        ops.gptq_marlin_repack(x, empty, 128, 96, 4)      # size_n % 64
    with pytest.raises(RuntimeError):
        ops.gptq_marlin_repack(x, empty, 128, 64, 3)      # bits
    with pytest.raises(RuntimeError):
        ops.awq_marlin_repack(x, 128, 64, 4)              # wrong packed shape


@pytest.mark.parametrize("shape", [(1, 512), (544, 4096), (67, 8192), (3, 28672)])
@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_permute_cols(env, shape, dtype):
    torch, G, ops = env
    tdt = torch.float16 if dtype == "float16" else torch.bfloat16
    x = torch.randn(shape, dtype=tdt, device="cuda")
    perm = torch.randperm(shape[1], device="cuda").to(torch.int32)
    y = ops.permute_cols(x, perm)
    torch.cuda.synchronize()
    assert torch.equal(y, x[:, perm.long()])
    # strided input
    big = torch.randn((shape[0] + 2, shape[1] + 16), dtype=tdt, device="cuda")
    view = big[1:shape[0] + 1, 8:shape[1] + 8]
    y = ops.permute_cols(view, perm)
    assert torch.equal(y, view[:, perm.long()])
