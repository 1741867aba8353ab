"""End-to-end decode throughput of a random-init Llama-3-8B-shaped model whose
linear layers are GPTQ uint4b8 g128 on this package's kernels.

    python bench_e2e.py [--batch 64] [--prompt 512] [--new 128] [--layers 32]
    python -m torch.distributed.run --nproc-per-node N ... bench_e2e.py   (tensor parallel)

Offline batch of `batch` sequences with `prompt` uniform-random token ids each,
greedy decoding of `new` tokens.  Prints one JSON line: decode tokens/s =
batch * new / decode time (CUDA events, max over ranks), prefill time, and the
weight-streaming floor for context.  Weights and tokens are synthetic and seeded.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=128)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    import torch

    from vllm_b200 import distributed as D
    from vllm_b200.e2e_llama import LlamaConfig, LlamaDecoder, generate

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        D.initialize_model_parallel(world)
        if os.environ.get("E2E_NCCL_ONLY", "0") != "1":
            D.enable_custom_all_reduce(dev)   # row-parallel outputs up to 512 KiB: peer-memory all-reduce
    cfg = LlamaConfig(num_layers=args.layers)
    model = LlamaDecoder(cfg, max_seq=args.prompt + args.new + 1, batch=args.batch, device=dev,
                         tp_rank=rank, tp_size=world)
    gen = torch.Generator(device=dev).manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt), device=dev, generator=gen)
    # one extra token: the first comes from prefill, then `new` timed decode steps
    out, prefill_ms, decode_ms = generate(model, prompts, args.new + 1, use_graph=not args.no_graph)
    t = torch.tensor([prefill_ms, decode_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    prefill_ms, decode_ms = t.tolist()
    if rank == 0:
        w_bytes = cfg.num_layers * sum(k * n // 2 + (k // 128) * n * 2 for k, n in
                                       [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096)])
        print(json.dumps({
            "metric": "llama3_8b_gptq_decode_tokens_per_s", "value": args.batch * args.new / decode_ms * 1e3,
            "unit": "tokens/s", "n_gpus": world, "ms_per_decode_step": decode_ms / args.new,
            "prefill_ms": prefill_ms, "batch": args.batch, "prompt": args.prompt, "new_tokens": args.new,
            "layers": cfg.num_layers, "quantized_weight_bytes_per_step": w_bytes,
            "cuda_graph": not args.no_graph, "data": "synthetic",
            "checksum": int(out.sum().item()) % 1000003}), flush=True)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
