"""The end-to-end decode harness on a tiny Llama-shaped model: the quantized
model's prefill logits agree with a dense model built from the weights the
kernels see, and CUDA-graph decode reproduces eager decode."""
import pytest

pytestmark = pytest.mark.gpu


def test_tiny_llama_matches_dense_and_graph_replay():
    import torch
    import torch.nn.functional as F

    from vllm_b200.e2e_llama import LlamaConfig, LlamaDecoder, generate
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_layers=2, num_heads=4,
                      num_kv_heads=2, head_dim=64, vocab_size=1000)
    B, T, NEW = 3, 24, 6
    model = LlamaDecoder(cfg, max_seq=T + NEW + 1, batch=B, seed=1)
    prompts = torch.randint(0, cfg.vocab_size, (B, T), device="cuda")

    # effective dense weights: push an identity through each quantized layer
    def dense(lin, k):
        eye = torch.eye(k, dtype=torch.bfloat16, device="cuda")
        return lin(eye).float()            # [k, n] == dequantised weights in bf16

    x = model.embed[prompts].float()
    for layer in model.layers:
        wq, wo = dense(layer.qkv_proj, 256), dense(layer.o_proj, 256)
        wgu, wd = dense(layer.gate_up_proj, 256), dense(layer.down_proj, 512)
        h = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)
        qkv = h.bfloat16().float() @ wq
        q, k, v = qkv.split([256, 128, 128], dim=-1)
        q = q.view(B, T, 4, 64).transpose(1, 2)
        k = k.view(B, T, 2, 64).transpose(1, 2)
        v = v.view(B, T, 2, 64).transpose(1, 2)
        from vllm_b200.e2e_llama import apply_rope
        q, k = apply_rope(q, model.cos[:T], model.sin[:T]), apply_rope(k, model.cos[:T], model.sin[:T])
        attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        x = x + attn.transpose(1, 2).reshape(B, T, -1).bfloat16().float() @ wo
        h = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)
        g, u = (h.bfloat16().float() @ wgu).chunk(2, dim=-1)
        x = x + (F.silu(g) * u).bfloat16().float() @ wd
    xl = x[:, -1]
    ref_last = xl * torch.rsqrt(xl.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)   # final norm (weight 1)

    # the model's own final-norm output after prefill
    if model.use_fa:
        model.fa["seqlens"].zero_()
        y = model._run_layers(model.embed[prompts], None, None, model.fa, None, T)
    else:
        y = model._run_layers(model.embed[prompts], model.cos[:T], model.sin[:T], None, None, T)
    got_last = y[:, -1].float()
    err = (got_last - ref_last).abs().max().item()
    assert err <= 3e-2 * ref_last.abs().max().item(), err

    eager, _, _ = generate(model, prompts, NEW, use_graph=False)
    graphed, _, _ = generate(model, prompts, NEW, use_graph=True)
    assert torch.equal(eager, graphed)
    if model.use_fa:
        # the torch attention path of the harness gives the same tokens as the library kernel
        # up to ties; compare the first generated token, which depends on prefill only
        plain = LlamaDecoder(cfg, max_seq=T + NEW + 1, batch=B, seed=1, use_flash_attn=False)
        toks, _, _ = generate(plain, prompts, 2, use_graph=False)
        assert (toks[:, 0] == eager[:, 0]).float().mean().item() >= 0.66
