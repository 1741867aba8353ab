"""Benchmark of the weight-only quantized linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the Llama-3-8B-shaped GPTQ layer sweep — bf16 activations,
uint4b8 weights, group 128, desc_act (act-order) — over the four layers
QKV 4096->6144, O 4096->4096, gate_up 4096->28672, down 14336->4096 and
M in {1, 4, 16, 64, 256, 1024, 4096}.  One step = one GEMM call per (layer, M).
For N > 1 every rank runs the same per-GPU shapes as a tensor-parallel shard
(weak scaling) and the row-parallel layers (O, down) all-reduce their output
over NCCL.

The headline value is the algorithmic HBM GB/s of the decode regime (M <= 64);
TFLOP/s of the M >= 1024 calls, the per-shape table, the roofline fractions
against the measured peaks, the end-to-end figure through the torch op with
host buffers, and a CPU baseline are reported in the same JSON line.

Inputs are synthetic and seeded; each (layer, M) rotates over a pool of
distinct weight tensors larger than L2, so weights always come from HBM.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYERS = [("qkv", 4096, 6144, False), ("o", 4096, 4096, True),
          ("gate_up", 4096, 28672, False), ("down", 14336, 4096, True)]  # name, K, N, row-parallel
MS = [1, 4, 16, 64, 256, 1024, 4096]
GROUP = 128
BITS = 4
POOL_BYTES = 400_000_000  # per layer: > 3 x the 126 MB L2
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
METRIC = "w4a16_gemm_hbm_gbs_m_le_64"


def algorithmic_bytes(m: int, n: int, k: int, act_order: bool = True) -> int:
    """Packed weights + scales + g_idx/perm + activations + output (16-bit)."""
    g = k // GROUP
    return k * n * BITS // 8 + g * n * 2 + (8 * k if act_order else 0) + 2 * m * k + 2 * m * n


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                mhz.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx,
                "samples": len(mhz), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------
# CPU arm: the reference's dequantise-then-matmul path, restated by the oracle
# ---------------------------------------------------------------------------


def cpu_sample(layers, m: int, seed: int = 0):
    """Run unpack -> dequantise (act-order groups) -> fp32 matmul on the host for
    the given layers at M = m.  Returns (algorithmic bytes, seconds)."""
    import numpy as np

    from oracle import marlin_oracle as mo
    rng = np.random.default_rng(seed)
    total_bytes, total_s = 0, 0.0
    for _, k, n, _ in layers:
        qweight = rng.integers(-2**31, 2**31 - 1, size=(k // 8, n), dtype=np.int64).astype(np.int32)
        scales = rng.uniform(0.002, 0.02, size=(k // GROUP, n)).astype(np.float32)
        g_idx = (np.arange(k) // GROUP)[rng.permutation(k)].astype(np.int32)
        a = rng.standard_normal((m, k)).astype(np.float32)
        t0 = time.perf_counter()
        q = mo.unpack_rows(qweight, BITS)
        w = mo.dequantize(q, scales, "bfloat16", bias=8, g_idx=g_idx)
        out = mo.gemm_ref(mo.round_to_bf16(a), w)
        total_s += time.perf_counter() - t0
        total_bytes += algorithmic_bytes(m, n, k)
        del q, w, out
    return total_bytes, total_s


def run_reference(args, world, rank):
    if rank != 0:
        return
    layers = [LAYERS[0]]  # bounded sample: the QKV layer at M = 16
    for _ in range(args.warmup):
        cpu_sample(layers, 16)
    t_bytes, t_s = 0, 0.0
    for i in range(args.steps):
        b, s = cpu_sample(layers, 16, seed=i)
        t_bytes += b
        t_s += s
    value = t_bytes / t_s / 1e9
    sample = "QKV 4096->6144 at M=16 per step (unpack + act-order dequant + fp32 matmul, numpy)"
    emit({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_s / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(world),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })


def workload_config(world):
    return {"workload": "llama3_8b_gptq_uint4b8_g128_actorder_layer_sweep",
            "layers_k_n": [[k, n] for _, k, n, _ in LAYERS], "m_values": MS,
            "group_size": GROUP, "act_order": True,
            "parallelism": "tp%d_weak (per-GPU shard shapes fixed; O/down all-reduce over NVLink peer "
                           "memory up to 512 KiB - inside the GEMM kernel at M <= 32 - NCCL above)" % world
            if world > 1 else "single_gpu",
            "l2_policy": "weight pool of >= 400 MB per layer rotated per call (inputs larger than L2)"}


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------


class LayerPool:
    """Device-resident pool of distinct random quantized copies of one layer."""

    def __init__(self, torch, dev, dt, name, k, n, row_parallel, gen):
        self.name, self.k, self.n, self.row_parallel = name, k, n, row_parallel
        wbytes = k * n * BITS // 8
        self.copies = int(min(64, max(8, -(-POOL_BYTES // wbytes))))
        pf = 32 // BITS
        self.q = [torch.randint(-2**31, 2**31 - 1, (k // 16, n * 16 // pf), dtype=torch.int32,
                                device=dev, generator=gen) for _ in range(self.copies)]
        self.s = [(torch.rand((k // GROUP, n), device=dev, generator=gen) * 0.018 + 0.002).to(dt)
                  for _ in range(self.copies)]
        # act-order: sorted group ids as the GEMM sees them, and the sort permutation
        g = (torch.arange(k, device=dev) // GROUP)[torch.randperm(k, device=dev, generator=gen)]
        order = torch.argsort(g, stable=True)
        self.g_idx = g[order].to(torch.int32).contiguous()
        self.perm = order.to(torch.int32).contiguous()


def run_ours(args, world, rank, local_rank):
    import torch

    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import _lib
    from vllm_b200 import marlin_utils as mu
    from vllm_b200.scalar_type import scalar_types

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    custom_ar = ar_link = None
    if world > 1:
        import torch.distributed as dist

        from vllm_b200 import distributed as D
        dist.init_process_group("nccl", device_id=dev)
        D.initialize_model_parallel(world)
        if os.environ.get("BENCH_NCCL_ONLY", "0") != "1" and D.enable_custom_all_reduce(dev):
            custom_ar = D._CUSTOM_AR
            ar_link = D.fused_all_reduce_scope().link_args()
    lib = _lib.load()
    dt = torch.bfloat16
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    pools = [LayerPool(torch, dev, dt, *layer, gen) for layer in LAYERS]
    ws = mu.marlin_make_workspace_new(dev)
    max_scratch = max(lib.b200q_marlin_gemm_preferred_scratch_bytes(m, p.n, p.k, 1)
                      for p in pools for m in MS)
    scratch = torch.empty(max_scratch, dtype=torch.uint8, device=dev)
    a_dev = {(p.k, m): torch.randn((m, p.k), device=dev, dtype=dt, generator=gen)
             for p in pools for m in MS}
    c_dev = {(p.n, m): torch.empty((m, p.n), device=dev, dtype=dt) for p in pools for m in MS}
    vp = ctypes.c_void_p
    flags = _lib.FLAG_K_FULL | _lib.FLAG_FP32_REDUCE
    qtype = scalar_types.uint4b8

    def raw_call(p, m, copy):
        """One GEMM through the C ABI on the current stream, inputs resident in HBM."""
        a, c = a_dev[(p.k, m)], c_dev[(p.n, m)]
        fused = (custom_ar is not None and p.row_parallel and m * p.n * 2 <= custom_ar.max_size)
        args = (vp(a.data_ptr()), p.k, vp(p.q[copy].data_ptr()), vp(p.s[copy].data_ptr()), None,
                vp(p.g_idx.data_ptr()), vp(p.perm.data_ptr()), None, vp(c.data_ptr()),
                vp(scratch.data_ptr()), max_scratch, vp(ws.data_ptr()), ws.numel(), qtype.id,
                _lib.BF16, m, p.n, p.k, p.k // GROUP, flags)
        cur = vp(torch.cuda.current_stream().cuda_stream)
        if fused:
            # GEMM and all-reduce in one call: one kernel at M <= 32, GEMM + peer-memory
            # all-reduce kernel above
            rc = lib.b200q_marlin_gemm_all_reduce(*args, *ar_link, cur)
        else:
            rc = lib.b200q_marlin_gemm(*args, cur)
        _lib.check(rc, "b200q_marlin_gemm")
        if not fused and dist is not None and p.row_parallel:
            dist.all_reduce(c)

    shapes = [(p, m) for p in pools for m in MS]
    use_graphs = os.environ.get("BENCH_NO_GRAPH", "0") != "1"
    stream = torch.cuda.Stream(device=dev)

    def make_runner(p, m, count, first_copy):
        """Callable that issues `count` calls rotating over the pool; a CUDA graph
        when enabled (host launch cost would otherwise exceed the kernel time)."""
        def body():
            for i in range(count):
                raw_call(p, m, (first_copy + i) % p.copies)
        if not use_graphs or count == 0:
            return body, 0
        before = lib.b200q_kernel_launches()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            body()
        return g.replay, lib.b200q_kernel_launches() - before

    with torch.cuda.stream(stream):
        for p, m in shapes:                      # eager pass: attribute set-up, NCCL warm-up
            raw_call(p, m, 0)
    torch.cuda.synchronize()
    warm = [make_runner(p, m, args.warmup, 0)[0] for p, m in shapes]
    timed = [make_runner(p, m, args.steps, args.warmup) for p, m in shapes]
    launches = sum(n for _, n in timed)

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident throughput ---------------------------------------------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)                      # let the sampler come up; warm-up load is sampled too
    with torch.cuda.stream(stream):
        for w in warm:
            w()
    sync_all()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in shapes]
    t_all0, t_all1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    align = torch.zeros(1, device=dev) if dist is not None else None
    if not use_graphs:
        before = lib.b200q_kernel_launches()
    with torch.cuda.stream(stream):
        t_all0.record()
        for (e0, e1), (fn, _) in zip(ev, timed):
            if align is not None:
                # ranks drift apart over the shapes without a collective; without this the whole
                # drift would be booked on the first row-parallel shape that follows
                dist.all_reduce(align)
            e0.record()
            fn()
            e1.record()
        t_all1.record()
    sync_all()
    if not use_graphs:
        launches = lib.b200q_kernel_launches() - before
    clocks = sampler.stop()
    ms = torch.tensor([e0.elapsed_time(e1) for e0, e1 in ev] + [t_all0.elapsed_time(t_all1)],
                      dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = ms.tolist()
    total_ms, ms = ms[-1], ms[:-1]

    # ---- end to end: torch op, host buffers ------------------------------------------------
    e2e_steps = max(1, min(args.steps, 5))
    a_host = {key: t.cpu().pin_memory() for key, t in a_dev.items()}
    c_host = {key: torch.empty(t.shape, dtype=dt).pin_memory() for key, t in c_dev.items()}
    empty = torch.empty(0, dtype=torch.int32, device=dev)

    def e2e_call(p, m, copy):
        a = a_host[(p.k, m)].to(dev, non_blocking=True)
        out = ops.gptq_marlin_gemm(a, None, p.q[copy], None, p.s[copy], None, empty, p.g_idx, p.perm,
                                   ws, qtype, m, p.n, p.k, is_k_full=True, use_atomic_add=False,
                                   use_fp32_reduce=True, is_zp_float=False)
        if dist is not None and p.row_parallel:
            out = D.tensor_model_parallel_all_reduce(out)
        c_host[(p.n, m)].copy_(out, non_blocking=True)

    for p, m in shapes:
        e2e_call(p, m, 0)
    sync_all()
    ev2 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in shapes]
    for (e0, e1), (p, m) in zip(ev2, shapes):
        e0.record()
        for i in range(e2e_steps):
            e2e_call(p, m, (1 + i) % p.copies)
        e1.record()
    sync_all()
    ms2 = torch.tensor([e0.elapsed_time(e1) for e0, e1 in ev2], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
    ms2 = ms2.tolist()
    decode = run_decode(world, rank, dev) if os.environ.get("BENCH_NO_DECODE", "0") != "1" else None
    if rank == 0:
        report(args, world, shapes, ms, total_ms, ms2, e2e_steps, launches, clocks, decode)
    if dist is not None:
        # CUDA graphs that captured NCCL kernels are still alive: tearing the communicator down
        # under them can block, so leave together and let process exit release everything
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def run_decode(world, rank, dev):
    """Third part of the metric: greedy decode of a Llama-3-8B-shaped model (random weights, GPTQ
    uint4b8 g128) whose projections all run through this library, tensor-parallel over the ranks.
    Batch 64, prompt 512, CUDA-graph decode steps timed with CUDA events, max over ranks."""
    import torch
    try:
        from vllm_b200.e2e_llama import LlamaConfig, LlamaDecoder, generate
        batch, prompt, new = 64, 512, 64
        cfg = LlamaConfig()
        model = LlamaDecoder(cfg, max_seq=prompt + new + 2, batch=batch, device=dev, tp_rank=rank,
                             tp_size=world)
        gen = torch.Generator(device=dev).manual_seed(0)
        prompts = torch.randint(0, cfg.vocab_size, (batch, prompt), device=dev, generator=gen)
        _, prefill_ms, decode_ms = generate(model, prompts, new + 1, use_graph=True)
        t = torch.tensor([prefill_ms, decode_ms], dtype=torch.float64, device=dev)
        if world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        prefill_ms, decode_ms = t.tolist()
        del model
        torch.cuda.empty_cache()
        return {"metric": "llama3_8b_gptq_decode_tokens_per_s", "value": batch * new / decode_ms * 1e3,
                "unit": "tokens/s", "ms_per_decode_step": decode_ms / new, "prefill_ms": prefill_ms,
                "batch": batch, "prompt": prompt, "new_tokens": new, "tensor_parallel": world,
                "data": "synthetic (random-init weights of the Llama-3-8B architecture)",
                "note": "projections, residual add + RMSNorm, SiLU*mul and the row-parallel all-reduce "
                        "are this library's kernels; attention is a library kernel"}
    except Exception as exc:  # the GEMM sweep above is the primary result
        return {"error": repr(exc)[:300]}


def report(args, world, shapes, ms, total_ms, ms2, e2e_steps, launches, clocks, decode=None):
    peaks = load_peaks()
    k_steps = args.steps
    rows = []
    dec_b = dec_t = ten_f = ten_t = e2e_b = e2e_t = str_b = str_t = 0.0
    for (p, m), t, t2 in zip(shapes, ms, ms2):
        b, f = algorithmic_bytes(m, p.n, p.k), 2.0 * m * p.n * p.k
        us = 1e3 * t / k_steps
        rows.append({"layer": p.name, "k": p.k, "n": p.n, "m": m, "us": round(us, 2),
                     "gbs": round(b / us / 1e3, 1), "tflops": round(f / us / 1e6, 2),
                     "e2e_us": round(1e3 * t2 / e2e_steps, 2)})
        if m <= 64:
            dec_b += b * k_steps
            dec_t += t
            e2e_b += b * e2e_steps
            e2e_t += t2
        if m <= 16:                      # the launches of the streaming decode kernel
            str_b += b * k_steps
            str_t += t
        if m >= 1024:
            ten_f += f * k_steps
            ten_t += t
    value = world * dec_b / dec_t / 1e6            # GB/s, all ranks
    tflops = world * ten_f / ten_t / 1e9
    per_gpu_gbs, per_gpu_tf = value / world, tflops / world
    stream_gbs = str_b / str_t / 1e6  # per GPU: every rank runs the same shapes
    # DRAM bytes of one launch of the dominant decode kernel from the ncu capture summarised in
    # profiles/gemm_stream_gate_up_m16.txt (gate_up, M = 16: 60.9 MB for 61.6 MB algorithmic)
    traffic = 60.9e6
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": k_steps,
        "warmup": args.warmup, "ms_per_step": total_ms / k_steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(world),
        "tflops_m_ge_1024": tflops,
        "roofline": {"bound": "hbm", "achieved": stream_gbs, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": stream_gbs / peaks["hbm_gbs"], "traffic": traffic,
                     "traffic_launch": "gemm_stream_kernel, gate_up 4096->28672, M=16: DRAM bytes of one "
                                       "launch under ncu (61.6e6 algorithmic)",
                     "peak_source": peaks["source"],
                     "scope": "dominant kernel gemm_stream_kernel: the M <= 16 calls (each = act-order "
                              "gather + decode GEMM), algorithmic bytes / CUDA-event time, per GPU",
                     "frac_m_le_64": per_gpu_gbs / peaks["hbm_gbs"]},
        "roofline_tensor": {"bound": "tensor", "achieved": per_gpu_tf, "peak": peaks["bf16_tflops"],
                            "unit": "TFLOP/s", "frac": per_gpu_tf / peaks["bf16_tflops"],
                            "traffic": None, "peak_source": peaks["source"],
                            "scope": "M >= 1024 calls"},
        "e2e": {"value": world * e2e_b / e2e_t / 1e6, "unit": "GB/s",
                "h2d_bytes_per_step": sum(2 * m * p.k for p, m in shapes),
                "d2h_bytes_per_step": sum(2 * m * p.n for p, m in shapes),
                "steps": e2e_steps,
                "path": "torch op gptq_marlin_gemm; A from pinned host memory, C back to pinned "
                        "host memory every call; weights resident (the op takes device tensors)"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "decode": decode,
        "per_shape": rows,
    }
    if world == 1:
        b, s = cpu_sample(LAYERS, 16)
        line["cpu_baseline"] = {
            "value": b / s / 1e9, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
            "sample": "the four layers at M=16, one pass (unpack + act-order dequant + fp32 matmul, "
                      "numpy restatement of the reference's CPU path), %.1f s" % s}
    emit(line)


_RESULT_FD = 1


def emit(line: dict) -> None:
    """Write the result line to the process's original stdout."""
    os.write(_RESULT_FD, (json.dumps(line) + "\n").encode())


def main():
    # libraries (NCCL's version banner, for one) print to file descriptor 1: keep it for the
    # single result line and send everything else to stderr
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node %d for --gpus %d"
                         % (args.gpus, args.gpus))
    if args.impl == "reference":
        run_reference(args, world, rank)
    else:
        run_ours(args, world, rank, local_rank)


if __name__ == "__main__":
    main()
