"""Generate the golden fixtures in this directory from the reference's own
Python packers (CPU only).

Usage:  python tests/golden/make_golden.py <path-to-reference-checkout> [hqq|fp8|fp4|moe|elementwise]
        (with `hqq` / `fp8` / `fp4` / `moe` / `elementwise` only that fixture is rewritten)

The reference checkout is only needed to (re)generate the fixtures; the tests
read the committed ``*.npz`` files and never import the reference.  All inputs
are seeded, so a rerun reproduces the files byte for byte (up to zip
metadata).

What is recorded (every array is the reference's output for the stated
inputs):
  scalar_types.npz   ids and min/max of uint4b8 / uint4 / uint8b128 / uint8
  repack_*.npz       gptq_pack / awq_pack inputs, sort indices, and the
                     expected Marlin layout from marlin_weights(get_weight_perm)
  perms.npz          marlin_permute_scales (grouped and channel-wise),
                     marlin_permute_bias, marlin_zero_points,
                     awq_to_marlin_zero_points
  gemm_*.npz         marlin_quantize / awq_marlin_quantize outputs (w_ref,
                     Marlin weights, scales, zero-points, g_idx, sort indices),
                     an activation matrix and the fp32 product a @ w_ref
  hqq_u4_g64_f16.npz float zero-points (HQQ): codes, scales, zero-points, their Marlin
                     forms from gptq_pack / marlin_weights / marlin_permute_scales, and
                     the dequantised weights and product computed as the reference's
                     test does (tests/kernels/quantization/test_marlin_gemm.py:463-534)
  fp8_g128_bf16.npz, fp8_gm1_f16.npz
                     float8_e4m3fn weights: the steps of marlin_quant_fp8_torch
                     (marlin_utils_fp8.py:321-352) with the CUDA repack op replaced by the CPU
                     marlin_weights: codes, scales, weight_ref, packed words, Marlin words,
                     permuted scales with the exponent bias fused in, and the product
  nvfp4_g16_{f16,bf16}.npz, mxfp4_g32_bf16.npz
                     float4_e2m1f weights: rand_marlin_weight_nvfp4_like / _mxfp4_like
                     (marlin_utils_fp4.py:304-397) run on CPU with the CUDA repack op replaced by
                     the CPU marlin_weights: the random codes, weight_ref, Marlin words, the
                     processed scale bytes, the processed global scale, and the product
  moe_align.npz      torch_moe_align_block_size (the reference's golden torch implementation of its
                     CUDA op, tests/kernels/moe/test_moe_align_block_size.py:92-170): routing tables,
                     sorted ids, block experts, padded totals
  elementwise_{bf16,f16}.npz
                     the reference's torch implementations of the steps next to the
                     row-parallel GEMM: RMSNorm.forward_static with and without a residual
                     (vllm/model_executor/layers/layernorm.py:180-224) and
                     SiluAndMul.forward_native (vllm/model_executor/layers/activation.py:84-87),
                     inputs and outputs as 16-bit patterns
"""

import os
import sys

import numpy as np


def _bits16(t):
    """torch fp16/bf16 tensor -> uint16 bit pattern."""
    import torch
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def make_hqq(here, mu, mt, qu) -> None:
    import torch
    torch.manual_seed(7)
    M, K, N, g = 19, 256, 128, 64
    a = torch.randn((M, K), dtype=torch.float16)
    b_weight = torch.randint(0, 10, (N, K), dtype=torch.uint8)            # [N, K] as in the test
    scale = torch.randn((N, K // g), dtype=torch.float16)
    zero = torch.randn((N, K // g), dtype=torch.float16)
    q_kn = b_weight.transpose(1, 0).contiguous().to(torch.int32)          # [K, N]
    gptq_w_q = qu.gptq_pack(q_kn, 4, K, N)
    marlin_q = mt.marlin_weights(q_kn, K, N, 4, mt.get_weight_perm(4))    # what the repack op returns
    marlin_s = mu.marlin_permute_scales(scale.transpose(1, 0).contiguous(), K, N, g)
    marlin_zp = mu.marlin_permute_scales(zero.transpose(1, 0).contiguous(), K, N, g)
    b_flat = b_weight.reshape(-1, g)
    dequant = (b_flat - zero.reshape(-1, 1)) * scale.reshape(-1, 1)       # fp16 arithmetic
    w_ref = dequant.reshape(b_weight.shape).transpose(1, 0).contiguous()  # [K, N]
    np.savez_compressed(
        os.path.join(here, "hqq_u4_g64_f16.npz"),
        M=np.int64(M), K=np.int64(K), N=np.int64(N), group_size=np.int64(g),
        a_bits=_bits16(a), q=q_kn.numpy(), gptq_in=gptq_w_q.numpy(), marlin_q_w=marlin_q.numpy(),
        scale_bits=_bits16(scale.transpose(1, 0).contiguous()),
        zero_bits=_bits16(zero.transpose(1, 0).contiguous()),
        marlin_s_bits=_bits16(marlin_s), marlin_zp_bits=_bits16(marlin_zp),
        w_ref_bits=_bits16(w_ref), out_ref=(a.float() @ w_ref.float()).numpy())


def make_fp8(here, mu, mt) -> None:
    import torch
    from vllm.model_executor.layers.quantization.utils import marlin_utils_fp8 as f8
    torch.manual_seed(11)
    for name, dtype, g, M, K, N in (("fp8_g128_bf16", torch.bfloat16, 128, 7, 256, 128),
                                    ("fp8_gm1_f16", torch.float16, -1, 21, 128, 192)):
        weight = torch.randn((N, K), dtype=dtype)                         # [N, K] as in the reference
        a = torch.randn((M, K), dtype=dtype)
        if g != -1:
            scales = weight.view(N, -1, g).abs().max(-1)[0] / 448
            rep = scales.repeat_interleave(g, 1)
        else:
            scales = weight.view(N, 1, K).abs().max(-1)[0] / 448
            rep = scales.repeat_interleave(K, 1)
        fp8_weight = (weight / rep).to(torch.float8_e4m3fn)
        weight_ref = fp8_weight.to(dtype) * rep
        packed = f8.pack_fp8_to_int32(fp8_weight, False).T.contiguous()   # [K / 4, N]
        codes = fp8_weight.view(torch.uint8).T.contiguous()               # [K, N]
        marlin_q = mt.marlin_weights(codes.to(torch.int32), K, N, 8, mt.get_weight_perm(8))
        marlin_s = f8.fp8_fused_exponent_bias_into_scales(
            mu.marlin_permute_scales(scales.T.contiguous(), K, N, g))
        np.savez_compressed(
            os.path.join(here, name + ".npz"),
            M=np.int64(M), K=np.int64(K), N=np.int64(N), group_size=np.int64(g),
            is_bf16=np.int64(dtype == torch.bfloat16), a_bits=_bits16(a), codes=codes.numpy(),
            scales_bits=_bits16(scales.T.contiguous()), packed=packed.numpy(),
            marlin_q_w=marlin_q.numpy(), marlin_s_bits=_bits16(marlin_s),
            w_ref_bits=_bits16(weight_ref.T.contiguous()),
            out_ref=(a.float() @ weight_ref.T.float()).numpy())


def make_fp4(here, mt) -> None:
    import torch
    from vllm.model_executor.layers.quantization.utils import marlin_utils_fp4 as f4

    captured = {}

    def cpu_repack(b_q_weight, perm, size_k, size_n, num_bits):
        # GPTQ words [K / 8, N] -> codes [K, N] -> the CPU Marlin packer
        shifts = torch.arange(0, 32, num_bits, dtype=torch.int32)
        codes = ((b_q_weight.unsqueeze(1) >> shifts.view(1, -1, 1)) & ((1 << num_bits) - 1))
        codes = codes.reshape(size_k, size_n).to(torch.int32)
        captured["codes"] = codes
        return mt.marlin_weights(codes, size_k, size_n, num_bits, mt.get_weight_perm(num_bits))

    f4.ops.gptq_marlin_repack = cpu_repack
    torch.manual_seed(13)
    for name, dtype, nv, g, M, K, N in (("nvfp4_g16_f16", torch.float16, True, 16, 9, 128, 128),
                                        ("nvfp4_g16_bf16", torch.bfloat16, True, 16, 23, 256, 192),
                                        ("mxfp4_g32_bf16", torch.bfloat16, False, 32, 17, 256, 128)):
        weight = torch.randn((N, K), dtype=dtype)
        a = torch.randn((M, K), dtype=dtype)
        if nv:
            w_ref, q, s, gs = f4.rand_marlin_weight_nvfp4_like(weight, g)
            gs_bits = _bits16(gs.reshape(1))
        else:
            w_ref, q, s = f4.rand_marlin_weight_mxfp4_like(weight, g)
            gs_bits = np.zeros(0, dtype=np.uint16)
        np.savez_compressed(
            os.path.join(here, name + ".npz"),
            M=np.int64(M), K=np.int64(K), N=np.int64(N), group_size=np.int64(g),
            is_bf16=np.int64(dtype == torch.bfloat16), is_nvfp4=np.int64(nv), a_bits=_bits16(a),
            codes=captured["codes"].numpy().astype(np.uint8), marlin_q_w=q.numpy(),
            marlin_s_bytes=s.contiguous().view(torch.uint8).numpy(), global_scale_bits=gs_bits,
            w_ref_bits=_bits16(w_ref.contiguous()),
            out_ref=(a.float() @ w_ref.float()).numpy())


def make_moe_align(here, ref_root) -> None:
    """Outputs of the reference's golden torch implementation of moe_align_block_size
    (tests/kernels/moe/test_moe_align_block_size.py:92-170) for seeded routing tables."""
    import importlib.util
    import torch
    spec = importlib.util.spec_from_file_location(
        "ref_test_moe_align", os.path.join(ref_root, "tests/kernels/moe/test_moe_align_block_size.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    torch.manual_seed(17)
    out = {}
    for i, (m, topk, e, bs) in enumerate(((5, 2, 4, 16), (33, 4, 8, 8), (64, 2, 3, 64), (7, 1, 16, 32),
                                          (128, 6, 32, 48))):
        topk_ids = torch.stack([torch.randperm(e)[:topk] for _ in range(m)]).to(torch.int32)
        if i == 2:
            topk_ids[topk_ids == 1] = 0                                   # an expert without tokens
        s, ex, n = mod.torch_moe_align_block_size(topk_ids, bs, e)
        out[f"topk_ids_{i}"] = topk_ids.numpy()
        out[f"cfg_{i}"] = np.array([m, topk, e, bs], dtype=np.int64)
        out[f"sorted_{i}"] = s.numpy()
        out[f"experts_{i}"] = ex.numpy()
        out[f"num_{i}"] = n.numpy()
    np.savez_compressed(os.path.join(here, "moe_align.npz"), cases=np.int64(5), **out)


def make_elementwise(here) -> None:
    import torch
    from vllm.model_executor.layers.activation import SiluAndMul
    from vllm.model_executor.layers.layernorm import RMSNorm
    for tag, dt in (("bf16", torch.bfloat16), ("f16", torch.float16)):
        torch.manual_seed(11)
        tokens, hidden, eps = 7, 512, 1e-5
        x = torch.randn((tokens, hidden), dtype=torch.float32).to(dt)
        res = torch.randn((tokens, hidden), dtype=torch.float32).to(dt)
        w = (1 + 0.1 * torch.randn(hidden, dtype=torch.float32)).to(dt)
        plain = RMSNorm.forward_static(x, eps, hidden, dt, w, None)
        fused, new_res = RMSNorm.forward_static(x, eps, hidden, dt, w, res)
        gate_up = (3 * torch.randn((tokens, 2 * hidden), dtype=torch.float32)).to(dt)
        act = SiluAndMul.forward_native(gate_up)
        np.savez_compressed(
            os.path.join(here, f"elementwise_{tag}.npz"), eps=np.float64(eps),
            x_bits=_bits16(x), res_bits=_bits16(res), w_bits=_bits16(w),
            rms_bits=_bits16(plain), fused_bits=_bits16(fused), new_res_bits=_bits16(new_res),
            gate_up_bits=_bits16(gate_up), act_bits=_bits16(act))


def main(ref_root: str, only: str | None = None) -> None:
    sys.path.insert(0, ref_root)
    import torch
    from vllm.model_executor.layers.quantization.utils import marlin_utils as mu
    from vllm.model_executor.layers.quantization.utils import marlin_utils_test as mt
    from vllm.model_executor.layers.quantization.utils import quant_utils as qu
    from vllm.scalar_type import scalar_types

    here = os.path.dirname(os.path.abspath(__file__))
    if only == "hqq":
        make_hqq(here, mu, mt, qu)
        print("hqq fixture written to", here)
        return
    if only == "fp8":
        make_fp8(here, mu, mt)
        print("fp8 fixtures written to", here)
        return
    if only == "moe":
        make_moe_align(here, ref_root)
        print("moe fixture written to", here)
        return
    if only == "fp4":
        make_fp4(here, mt)
        print("fp4 fixtures written to", here)
        return
    if only == "elementwise":
        make_elementwise(here)
        print("elementwise fixtures written to", here)
        return
    types = {"uint4b8": scalar_types.uint4b8, "uint4": scalar_types.uint4,
             "uint8b128": scalar_types.uint8b128, "uint8": scalar_types.uint8}

    # ---- scalar types -----------------------------------------------------
    np.savez(os.path.join(here, "scalar_types.npz"),
             names=np.array(list(types)),
             ids=np.array([t.id for t in types.values()], dtype=np.int64),
             mins=np.array([t.min() for t in types.values()], dtype=np.int64),
             maxs=np.array([t.max() for t in types.values()], dtype=np.int64),
             size_bits=np.array([t.size_bits for t in types.values()], dtype=np.int64))

    # ---- repack -----------------------------------------------------------
    rng = np.random.default_rng(0)
    for bits in (4, 8):
        for (K, N) in ((128, 64), (256, 192)):
            q = torch.from_numpy(rng.integers(0, 1 << bits, size=(K, N), dtype=np.int32))
            g_idx = torch.from_numpy((np.arange(K) // 32)[rng.permutation(K)].astype(np.int32))
            gptq_in = qu.gptq_pack(q, bits, K, N)
            awq_in = qu.awq_pack(q, bits, K, N)
            wperm = mt.get_weight_perm(bits)
            expect = mt.marlin_weights(q, K, N, bits, wperm)
            q_sorted, g_sorted, sort_idx = qu.sort_weights(q, g_idx)
            expect_perm = mt.marlin_weights(q_sorted, K, N, bits, wperm)
            np.savez_compressed(
                os.path.join(here, f"repack_b{bits}_k{K}_n{N}.npz"),
                q=q.numpy(), gptq_in=gptq_in.numpy(), awq_in=awq_in.numpy(),
                expect=expect.numpy(), g_idx=g_idx.numpy(),
                sort_idx=sort_idx.numpy(), g_sorted=g_sorted.numpy(),
                expect_perm=expect_perm.numpy(),
                weight_perm=wperm.numpy())

    # ---- scale / zero-point / bias permutations ---------------------------
    K, N = 512, 256
    s_grouped = torch.from_numpy(rng.random((K // 128, N), dtype=np.float32)).half()
    s_channel = torch.from_numpy(rng.random((1, N), dtype=np.float32)).half()
    bias = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).half()
    out = dict(
        s_grouped=s_grouped.numpy(), s_channel=s_channel.numpy(), bias=bias.numpy(),
        s_grouped_perm=mu.marlin_permute_scales(s_grouped, K, N, 128).numpy(),
        s_channel_perm=mu.marlin_permute_scales(s_channel, K, N, -1).numpy(),
        s_channel_perm_gk=mu.marlin_permute_scales(s_channel, K, N, K).numpy(),
        bias_perm=mu.marlin_permute_bias(bias).numpy())
    for bits in (4, 8):
        G = K // 128
        zp = torch.from_numpy(rng.integers(0, 1 << bits, size=(G, N), dtype=np.int32))
        awq_zp = qu.awq_pack(zp, bits, G, N)
        out[f"zp{bits}"] = zp.numpy()
        out[f"zp{bits}_marlin"] = mu.marlin_zero_points(zp, G, N, bits).numpy()
        out[f"zp{bits}_awq_in"] = awq_zp.numpy()
        out[f"zp{bits}_awq_marlin"] = mu.awq_to_marlin_zero_points(awq_zp, G, N, bits).numpy()
    np.savez_compressed(os.path.join(here, "perms.npz"), **out)

    # ---- quantise + GEMM expected values ----------------------------------
    torch.manual_seed(0)
    cases = [
        # name, type, dtype, group, act_order, M, K, N
        ("u4b8_g128_f16", "uint4b8", torch.float16, 128, False, 16, 256, 128),
        ("u4b8_g32_bf16", "uint4b8", torch.bfloat16, 32, False, 5, 128, 64),
        ("u4b8_gm1_f16", "uint4b8", torch.float16, -1, False, 26, 256, 64),
        ("u4b8_g64_act_bf16", "uint4b8", torch.bfloat16, 64, True, 9, 256, 128),
        ("u8b128_gm1_f16", "uint8b128", torch.float16, -1, False, 3, 128, 128),
        ("u8b128_g128_act_f16", "uint8b128", torch.float16, 128, True, 17, 256, 64),
        ("u4_g128_f16", "uint4", torch.float16, 128, False, 33, 256, 128),
        ("u4_g64_bf16", "uint4", torch.bfloat16, 64, False, 1, 128, 192),
    ]
    for name, tname, dtype, g, act, M, K, N in cases:
        t = types[tname]
        w = torch.randn((K, N), dtype=dtype)
        a = torch.randn((M, K), dtype=dtype)
        rec = dict(type_id=np.int64(t.id), size_bits=np.int64(t.size_bits),
                   group_size=np.int64(g), act_order=np.int64(act),
                   is_bf16=np.int64(dtype == torch.bfloat16),
                   M=np.int64(M), K=np.int64(K), N=np.int64(N))
        if tname in ("uint4", "uint8"):
            w_ref, mq, ms, mzp = mt.awq_marlin_quantize(w, t, g)
            rec["marlin_zp"] = mzp.numpy()
        else:
            w_ref, mq, ms, g_idx, sort_idx, _ = mt.marlin_quantize(w, t, g, act)
            rec["g_idx"] = g_idx.numpy().astype(np.int32)
            rec["sort_idx"] = sort_idx.numpy().astype(np.int32)
        rec["a_bits"] = _bits16(a)
        rec["w_ref_bits"] = _bits16(w_ref)
        rec["marlin_q_w"] = mq.numpy()
        rec["marlin_s_bits"] = _bits16(ms)
        rec["out_ref"] = (a.float() @ w_ref.float()).numpy()
        np.savez_compressed(os.path.join(here, f"gemm_{name}.npz"), **rec)
    make_hqq(here, mu, mt, qu)
    make_fp8(here, mu, mt)
    make_fp4(here, mt)
    make_moe_align(here, ref_root)
    make_elementwise(here)
    print("golden fixtures written to", here)


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        sys.exit(__doc__)
    main(sys.argv[1], sys.argv[2] if len(sys.argv) == 3 else None)
