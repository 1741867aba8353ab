"""Minimal Llama-architecture decoder whose every projection runs through the
quantized linear layers of this package — the harness for the end-to-end decode
measurement (random-init Llama-3-8B shape, GPTQ uint4b8 g128).

Only what the measurement needs is here: RMSNorm, RoPE, grouped-query attention
over a static KV cache (torch SDPA), SiLU-gated MLP, greedy sampling; the layer
order, the four projections per block and the (hidden, residual) hand-over between
blocks follow the reference's model (vllm/model_executor/models/llama.py:73-347).
The residual add + RMSNorm and SiLU * mul steps next to the projections run through
this package's kernels; after a row-parallel projection the all-reduce is either
inside the GEMM kernel (up to 32 rows) or inside the add + RMSNorm kernel.
Attention is library code: flash_attn's kv-cache kernel (rotary embedding, cache
append and attention in one launch) when the package is importable, else torch SDPA.  Embedding and lm_head stay 16-bit
and replicated (the reference quantizes lm_head only when the checkpoint says
so, gptq_marlin.py:198).  Attention, norms and sampling use stock torch ops: they
are outside the hot path this package replaces.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

try:  # library attention kernel; the torch path below is the fall-back
    from flash_attn import flash_attn_with_kvcache as _fa_kvcache
except Exception:  # pragma: no cover - depends on the image
    _fa_kvcache = None

from . import _custom_ops as ops
from . import distributed as D
from .linear import MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear
from .quantization import GPTQMarlinConfig


@dataclass
class LlamaConfig:
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 128256
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5


def _fill_random_gptq(layer, gen) -> None:
    """Seeded random codes and scales in checkpoint format, then the regular
    load-time transform (device repack, scale permutation)."""
    q = layer.qweight
    q.data.copy_(torch.randint(-2**31, 2**31 - 1, q.shape, dtype=torch.int32, device=q.device,
                               generator=gen))
    s = layer.scales
    s.data.copy_((torch.rand(s.shape, device=s.device, generator=gen) * 0.018 + 0.002).to(s.dtype))
    layer.process_weights_after_loading()


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    v = x.float()
    v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    return (v * w.float()).to(x.dtype)


class DecoderLayer(torch.nn.Module):
    def __init__(self, cfg: LlamaConfig, qc, dtype, device, gen, tp_rank, tp_size):
        super().__init__()
        kw = dict(quant_config=qc, params_dtype=dtype, device=device, tp_rank=tp_rank, tp_size=tp_size)
        h = cfg.hidden_size
        self.cfg = cfg
        self.qkv_proj = QKVParallelLinear(h, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, **kw)
        self.o_proj = RowParallelLinear(cfg.num_heads * cfg.head_dim, h, **kw)
        self.gate_up_proj = MergedColumnParallelLinear(h, [cfg.intermediate_size] * 2, **kw)
        self.down_proj = RowParallelLinear(cfg.intermediate_size, h, **kw)
        for lin in (self.qkv_proj, self.o_proj, self.gate_up_proj, self.down_proj):
            _fill_random_gptq(lin, gen)
        self.input_norm = torch.nn.Parameter(torch.ones(h, dtype=dtype, device=device), False)
        self.post_norm = torch.nn.Parameter(torch.ones(h, dtype=dtype, device=device), False)
        self.n_q = self.qkv_proj.num_heads
        self.n_kv = self.qkv_proj.num_kv_heads

    def _row_parallel_then_norm(self, proj, inp, residual, weight):
        """proj(inp) summed over the tensor-parallel ranks, added to the residual, normalised.
        Returns the normalised activations [rows, hidden]; the residual is updated in place."""
        eps = self.cfg.rms_eps
        rows = inp.shape[0]
        car = D._CUSTOM_AR
        if proj.tp_size > 1 and car is not None and rows > 32:
            part = proj(inp, reduce=False)
            if car.all_reduce_add_rms_norm(part, residual, weight, eps):
                return part
            out = D.tensor_model_parallel_all_reduce(part)
        else:
            out = proj(inp)          # all-reduce inside the GEMM kernel (or NCCL without a link)
        ops.fused_add_rms_norm(out, residual, weight, eps)
        return out

    def forward(self, x, residual, cos, sin, k_cache, v_cache, pos_index, attn_mask, prefill_len,
                next_norm):
        """x: [B, T, H], normalised input of the block; residual: [B * T, H], updated in place.
        prefill (prefill_len = T > 0): causal attention inside the prompt, KV written to [0, T).
        decode (T == 1): KV written at pos_index, attention over the cache under attn_mask
        [1, 1, 1, S].  Returns the input of the next block, normalised with `next_norm`."""
        cfg = self.cfg
        B, T, _ = x.shape
        qkv = self.qkv_proj(x.view(B * T, -1)).view(B, T, -1)
        q, k, v = qkv.split([self.n_q * cfg.head_dim, self.n_kv * cfg.head_dim,
                             self.n_kv * cfg.head_dim], dim=-1)
        if isinstance(pos_index, dict):
            # flash_attn: caches are [B, S, kv heads, D]; rotary, append at seqlens, attention
            fa = pos_index
            attn = _fa_kvcache(q.view(B, T, self.n_q, cfg.head_dim), k_cache, v_cache,
                               k=k.view(B, T, self.n_kv, cfg.head_dim),
                               v=v.view(B, T, self.n_kv, cfg.head_dim), rotary_cos=fa["cos"],
                               rotary_sin=fa["sin"], cache_seqlens=fa["seqlens"], causal=True,
                               rotary_interleaved=False)
            return self._mlp_tail(attn.reshape(B * T, -1), residual, next_norm, B, T)
        q = q.view(B, T, self.n_q, cfg.head_dim).transpose(1, 2)
        k = k.view(B, T, self.n_kv, cfg.head_dim).transpose(1, 2)
        v = v.view(B, T, self.n_kv, cfg.head_dim).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        if prefill_len:
            k_cache[:, :, :T].copy_(k)
            v_cache[:, :, :T].copy_(v)
            attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        else:
            k_cache.index_copy_(2, pos_index, k)
            v_cache.index_copy_(2, pos_index, v)
            attn = F.scaled_dot_product_attention(q, k_cache, v_cache, attn_mask=attn_mask,
                                                  enable_gqa=True)
        return self._mlp_tail(attn.transpose(1, 2).reshape(B * T, -1), residual, next_norm, B, T)

    def _mlp_tail(self, attn, residual, next_norm, B, T):
        h = self._row_parallel_then_norm(self.o_proj, attn, residual, self.post_norm)
        gu = self.gate_up_proj(h)
        act = torch.empty((B * T, gu.shape[-1] // 2), dtype=gu.dtype, device=gu.device)
        ops.silu_and_mul(act, gu)
        h = self._row_parallel_then_norm(self.down_proj, act, residual, next_norm)
        return h.view(B, T, -1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE; cos / sin: [T, head_dim / 2] for the positions of x's T axis."""
    x1, x2 = x.float().chunk(2, dim=-1)
    c, s = cos[None, None], sin[None, None]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


class LlamaDecoder(torch.nn.Module):
    def __init__(self, cfg: LlamaConfig, max_seq: int, batch: int, dtype=torch.bfloat16,
                 device="cuda", seed: int = 0, tp_rank: int = 0, tp_size: int = 1,
                 use_flash_attn: bool = True):
        super().__init__()
        self.cfg, self.max_seq, self.batch = cfg, max_seq, batch
        gen = torch.Generator(device=device).manual_seed(seed)       # same weights on every rank
        gen_shard = torch.Generator(device=device).manual_seed(seed * 1000 + 17 + tp_rank)
        qc = GPTQMarlinConfig(4, 128, desc_act=False)
        self.embed = (torch.randn(cfg.vocab_size, cfg.hidden_size, device=device, generator=gen)
                      * 0.02).to(dtype)
        self.lm_head = (torch.randn(cfg.vocab_size, cfg.hidden_size, device=device, generator=gen)
                        * 0.02).to(dtype)
        self.final_norm = torch.ones(cfg.hidden_size, dtype=dtype, device=device)
        self.layers = torch.nn.ModuleList(
            DecoderLayer(cfg, qc, dtype, device, gen_shard, tp_rank, tp_size)
            for _ in range(cfg.num_layers))
        n_kv = self.layers[0].n_kv
        self.use_fa = _fa_kvcache is not None and use_flash_attn
        cache_shape = ((batch, max_seq, n_kv, cfg.head_dim) if self.use_fa
                       else (batch, n_kv, max_seq, cfg.head_dim))
        self.k_cache = [torch.zeros(cache_shape, dtype=dtype, device=device)
                        for _ in range(cfg.num_layers)]
        self.v_cache = [torch.zeros_like(k) for k in self.k_cache]
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=device).float()
                                        / cfg.head_dim))
        ang = torch.arange(max_seq, device=device).float()[:, None] * inv[None]
        self.cos, self.sin = ang.cos(), ang.sin()
        self.fa = {"cos": self.cos.to(dtype), "sin": self.sin.to(dtype),
                   "seqlens": torch.zeros(batch, dtype=torch.int32, device=device)}

    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, T] -> next token ids [B]."""
        B, T = tokens.shape
        if self.use_fa:
            self.fa["seqlens"].zero_()
            x = self._run_layers(self.embed[tokens], None, None, self.fa, None, T)
            return (x[:, -1] @ self.lm_head.t()).argmax(-1)
        x = self._run_layers(self.embed[tokens], self.cos[:T], self.sin[:T], None, None, T)
        return (x[:, -1] @ self.lm_head.t()).argmax(-1)

    def _run_layers(self, emb, cos, sin, pos_index, attn_mask, prefill_len):
        """emb [B, T, H] -> final-norm output [B, T, H]."""
        B, T, H = emb.shape
        residual = emb.reshape(B * T, H).clone()
        x = torch.empty_like(residual)
        ops.rms_norm(x, residual, self.layers[0].input_norm, self.cfg.rms_eps)
        x = x.view(B, T, H)
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            next_norm = self.layers[i + 1].input_norm if i + 1 < n else self.final_norm
            x = layer(x, residual, cos, sin, self.k_cache[i], self.v_cache[i], pos_index, attn_mask,
                      prefill_len, next_norm)
        return x

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor, pos_index: torch.Tensor,
                    attn_mask: torch.Tensor) -> torch.Tensor:
        """One token per sequence.  tokens [B]; pos_index int64 [1] (cache slot to write);
        attn_mask bool [1, 1, 1, max_seq] with the valid cache slots set."""
        if self.use_fa:
            self.fa["seqlens"].copy_(pos_index.to(torch.int32).expand(tokens.shape[0]))
            x = self._run_layers(self.embed[tokens][:, None], None, None, self.fa, None, 0)
            return (x[:, 0] @ self.lm_head.t()).argmax(-1)
        cos, sin = self.cos.index_select(0, pos_index), self.sin.index_select(0, pos_index)
        x = self._run_layers(self.embed[tokens][:, None], cos, sin, pos_index, attn_mask, 0)
        return (x[:, 0] @ self.lm_head.t()).argmax(-1)


@torch.no_grad()
def generate(model: LlamaDecoder, prompts: torch.Tensor, new_tokens: int, use_graph: bool = True):
    """Greedy decode.  Returns (tokens [B, new_tokens], prefill_ms, decode_ms), timed with CUDA
    events; the decode loop replays one captured CUDA graph per step."""
    dev = prompts.device
    B, T = prompts.shape
    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    out = torch.empty(B, new_tokens, dtype=torch.long, device=dev)
    cur = torch.empty(B, dtype=torch.long, device=dev)
    pos = torch.zeros(1, dtype=torch.long, device=dev)
    mask = torch.zeros(1, 1, 1, model.max_seq, dtype=torch.bool, device=dev)
    e[0].record()
    cur.copy_(model.prefill(prompts))
    out[:, 0] = cur
    e[1].record()
    mask[..., :T] = True
    graph, nxt = None, None
    if use_graph:
        pos.fill_(T)
        mask[..., T] = True
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            nxt = model.decode_step(cur, pos, mask)       # warm-up outside capture
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            nxt = model.decode_step(cur, pos, mask)
        mask[..., T] = False
        torch.cuda.synchronize()
    e[2].record()
    for i in range(1, new_tokens):
        p = T + i - 1                                      # slot of the token fed in this step
        pos.fill_(p)
        mask[..., p] = True
        if graph is not None:
            graph.replay()
        else:
            nxt = model.decode_step(cur, pos, mask)
        cur.copy_(nxt)
        out[:, i] = cur
    e[3].record()
    torch.cuda.synchronize()
    return out, e[0].elapsed_time(e[1]), e[2].elapsed_time(e[3])
