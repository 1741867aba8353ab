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
MS4 = [1, 16, 128, 1024, 8192]  # BASELINE config 4 (Llama-3-70B shards)
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
    layers = LAYERS  # bounded sample: the four layers at M = 16, the set cpu_baseline uses
    for _ in range(args.warmup):
        cpu_sample(layers, 16)
    t_bytes, t_s = 0, 0.0
    for i in range(args.steps):
        b, s = cpu_sample(layers, 16, seed=i)
        t_bytes += b
        t_s += s
    value = t_bytes / t_s / 1e9
    sample = ("the four layers at M=16 per step (unpack + act-order dequant + fp32 matmul, numpy "
              "restatement of the reference's CPU path)")
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
                           "memory up to 2 MiB - inside the GEMM kernel at M <= 32 - NCCL above)" % world
            if world > 1 else "single_gpu",
            "l2_policy": "weight pool of >= 400 MB per layer rotated per call (inputs larger than L2)"}


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------


class LayerPool:
    """Device-resident pool of distinct random quantized copies of one layer."""

    def __init__(self, torch, dev, dt, name, k, n, row_parallel, gen, act_order=True, min_copies=8):
        self.name, self.k, self.n, self.row_parallel = name, k, n, row_parallel
        self.act_order = act_order
        wbytes = k * n * BITS // 8
        self.copies = int(min(64, max(min_copies, -(-POOL_BYTES // wbytes))))
        pf = 32 // BITS
        self.q = [torch.randint(-2**31, 2**31 - 1, (k // 16, n * 16 // pf), dtype=torch.int32,
                                device=dev, generator=gen) for _ in range(self.copies)]
        self.s = [(torch.rand((k // GROUP, n), device=dev, generator=gen) * 0.018 + 0.002).to(dt)
                  for _ in range(self.copies)]
        self.g_idx = self.perm = None
        if not act_order:
            return
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
            ar_link = custom_ar.link_args()
    lib = _lib.load()
    dt = torch.bfloat16
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    pools = [LayerPool(torch, dev, dt, *layer, gen,
                       act_order=os.environ.get("BENCH_NO_ACT_ORDER", "0") != "1")
             for layer in LAYERS]
    # BASELINE config 4: the Llama-3-70B layers as tensor-parallel shards of this world size
    # (gate_up column-parallel, down row-parallel with the all-reduce), no act-order
    pools4 = [] if os.environ.get("BENCH_NO_CONFIG4", "0") == "1" else [
        LayerPool(torch, dev, dt, "gate_up_70b", 8192, 57344 // world, False, gen, act_order=False,
                  min_copies=2),
        LayerPool(torch, dev, dt, "down_70b", 28672 // world, 8192, True, gen, act_order=False,
                  min_copies=2)]
    all_shapes = [(p, m) for p in pools for m in MS] + [(p, m) for p in pools4 for m in MS4]
    ws = mu.marlin_make_workspace_new(dev)
    max_scratch = max(lib.b200q_marlin_gemm_preferred_scratch_bytes(m, p.n, p.k, 1)
                      for p, m in all_shapes)
    scratch = torch.empty(max_scratch, dtype=torch.uint8, device=dev)
    a_dev = {(p.k, m): torch.randn((m, p.k), device=dev, dtype=dt, generator=gen)
             for p, m in all_shapes}
    c_dev = {(p.n, m): torch.empty((m, p.n), device=dev, dtype=dt) for p, m in all_shapes}
    vp = ctypes.c_void_p
    flags = _lib.FLAG_K_FULL | _lib.FLAG_FP32_REDUCE
    qtype = scalar_types.uint4b8

    ar_side = torch.cuda.Stream(device=dev) if dist is not None else None

    def raw_call(p, m, copy, reduce=True):
        """One GEMM through the C ABI on the current stream, inputs resident in HBM.
        reduce=False leaves the row-parallel output un-reduced (GEMM-only timing)."""
        a, c = a_dev[(p.k, m)], c_dev[(p.n, m)]
        fused = (reduce and custom_ar is not None and p.row_parallel
                 and m * p.n * 2 <= custom_ar.max_size)
        args = (vp(a.data_ptr()), p.k, vp(p.q[copy].data_ptr()), vp(p.s[copy].data_ptr()), None,
                vp(p.g_idx.data_ptr()) if p.act_order else None,
                vp(p.perm.data_ptr()) if p.act_order else None, None, vp(c.data_ptr()),
                vp(scratch.data_ptr()), max_scratch, vp(ws.data_ptr()), ws.numel(), qtype.id,
                _lib.BF16, m, p.n, p.k, p.k // GROUP, flags)
        if (reduce and not fused and dist is not None and p.row_parallel
                and m >= D.OVERLAP_MIN_ROWS):
            # what RowParallelLinear does with many rows: blocks of rows, NCCL's all-reduce of a
            # block on a second stream beside the GEMM of the next block
            step = -(-m // D.OVERLAP_CHUNKS)
            cur_s = torch.cuda.current_stream()
            for r0 in range(0, m, step):
                rows = min(step, m - r0)
                blk = list(args)
                blk[0] = vp(a.data_ptr() + r0 * p.k * 2)
                blk[8] = vp(c.data_ptr() + r0 * p.n * 2)
                blk[15] = rows
                _lib.check(lib.b200q_marlin_gemm(*blk, vp(cur_s.cuda_stream)), "b200q_marlin_gemm")
                done = torch.cuda.Event()
                done.record(cur_s)
                with torch.cuda.stream(ar_side):
                    ar_side.wait_event(done)
                    dist.all_reduce(c[r0:r0 + rows])
            cur_s.wait_stream(ar_side)
            return
        cur = vp(torch.cuda.current_stream().cuda_stream)
        if fused:
            # GEMM and all-reduce in one call: one kernel at M <= 32, GEMM + peer-memory
            # all-reduce kernel above
            rc = lib.b200q_marlin_gemm_all_reduce(*args, *ar_link, cur)
        else:
            rc = lib.b200q_marlin_gemm(*args, cur)
        _lib.check(rc, "b200q_marlin_gemm")
        if reduce and not fused and dist is not None and p.row_parallel:
            dist.all_reduce(c)

    ar_check = run_ar_check(torch, dist, D, lib, dev, custom_ar, ar_link, rank, world) \
        if world > 1 else None

    shapes = [(p, m) for p in pools for m in MS]
    use_graphs = os.environ.get("BENCH_NO_GRAPH", "0") != "1"
    stream = torch.cuda.Stream(device=dev)

    def make_runner(p, m, count, first_copy, reduce=True):
        """Callable that issues `count` calls rotating over the pool; a CUDA graph
        when enabled (host launch cost would otherwise exceed the kernel time)."""
        def body():
            for i in range(count):
                raw_call(p, m, (first_copy + i) % p.copies, reduce)
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
        # the synchronisation above left the GPU idle: one more untimed replay of the first shape's
        # warm-up graph, so that the timed region starts on a busy device like every later shape
        warm[0]()
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

    # ---- extra timings outside the headline: GEMM-only for row-parallel shapes (here, in the
    # thermal state of the pass above), config 4 (further down) ------------------------------
    def time_shapes(shape_list, steps, reduce=True):
        """CUDA-event time per call (ms, max over ranks) of each (pool, M): a graph of `steps`
        calls after one of 3 warm-up calls, ranks aligned before each."""
        fns = []
        for p, m in shape_list:
            w, _ = make_runner(p, m, 3, 0, reduce)
            t, n_l = make_runner(p, m, steps, 3, reduce)
            fns.append((w, t, n_l))
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in shape_list]
        with torch.cuda.stream(stream):
            for w, _, _ in fns:
                w()
        sync_all()
        with torch.cuda.stream(stream):
            for (e0, e1), (_, t, _) in zip(evs, fns):
                if align is not None:
                    dist.all_reduce(align)
                e0.record()
                t()
                e1.record()
        sync_all()
        out = torch.tensor([e0.elapsed_time(e1) / steps for e0, e1 in evs], dtype=torch.float64,
                           device=dev)
        if dist is not None:
            dist.all_reduce(out, op=dist.ReduceOp.MAX)
        return out.tolist(), sum(n_l for _, _, n_l in fns)

    extra = {}
    if dist is not None:
        rp = [(p, m) for p, m in shapes if p.row_parallel]
        g2, n2g = time_shapes(rp, args.steps, reduce=False)
        launches += n2g
        extra["gemm_only"] = (rp, g2)

    # ---- end to end: torch op, host buffers ------------------------------------------------
    e2e_steps = max(1, min(args.steps, 20))
    if os.environ.get("BENCH_NO_E2E", "0") == "1":
        e2e_steps = 0
    a_host = {key: t.cpu().pin_memory() for key, t in a_dev.items()}
    c_host = {key: torch.empty(t.shape, dtype=dt).pin_memory() for key, t in c_dev.items()}
    empty = torch.empty(0, dtype=torch.int32, device=dev)

    def e2e_call(p, m, copy):
        a = a_host[(p.k, m)].to(dev, non_blocking=True)
        # what RowParallelLinear does: the op all-reduces its own output where it fits the link
        link = None
        if dist is not None and p.row_parallel and custom_ar is not None \
                and custom_ar.fits(m, p.n, dt):
            link = custom_ar
        out = ops.gptq_marlin_gemm(a, None, p.q[copy], None, p.s[copy], None, empty, p.g_idx, p.perm,
                                   ws, qtype, m, p.n, p.k, is_k_full=True, use_atomic_add=False,
                                   use_fp32_reduce=True, is_zp_float=False, reduce_link=link)
        if dist is not None and p.row_parallel and link is None:
            out = D.tensor_model_parallel_all_reduce(out)
        c_host[(p.n, m)].copy_(out, non_blocking=True)

    if e2e_steps:
        for p, m in shapes:
            e2e_call(p, m, 0)
    sync_all()

    copy_in, copy_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def e2e_pipelined(p, m):
        """The same e2e_steps calls as a three-stage pipeline inside one captured graph: the
        copy of step i + 1's activations (copy-in stream, two device buffers) and the copy of
        step i - 1's result (copy-out stream) run beside the operator call of step i, as a
        serving loop with separate copy streams does.  Every step still moves its own A from
        pinned host memory and its own C back to pinned host memory."""
        cur = torch.cuda.current_stream()
        a_buf = [torch.empty_like(a_dev[(p.k, m)]) for _ in range(2)]
        link = None
        if dist is not None and p.row_parallel and custom_ar is not None \
                and custom_ar.fits(m, p.n, dt):
            link = custom_ar
        copy_in.wait_stream(cur)
        copy_out.wait_stream(cur)
        gemm_done = [None, None]
        for i in range(e2e_steps):
            with torch.cuda.stream(copy_in):
                if gemm_done[i % 2] is not None:
                    copy_in.wait_event(gemm_done[i % 2])       # the buffer's previous reader
                a_buf[i % 2].copy_(a_host[(p.k, m)], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(copy_in)
            cur.wait_event(ready)
            copy = (1 + i) % p.copies
            out = ops.gptq_marlin_gemm(a_buf[i % 2], None, p.q[copy], None, p.s[copy], None, empty,
                                       p.g_idx, p.perm, ws, qtype, m, p.n, p.k, is_k_full=True,
                                       use_atomic_add=False, use_fp32_reduce=True, is_zp_float=False,
                                       reduce_link=link)
            if dist is not None and p.row_parallel and link is None:
                out = D.tensor_model_parallel_all_reduce(out)
            done = torch.cuda.Event()
            done.record(cur)
            gemm_done[i % 2] = done
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                c_host[(p.n, m)].copy_(out, non_blocking=True)
            out.record_stream(copy_out)
        cur.wait_stream(copy_in)
        cur.wait_stream(copy_out)

    def time_e2e(graphs):
        """ms per shape for e2e_steps calls of (copy A from pinned host memory, operator, copy C
        to pinned host memory), max over ranks.  graphs=True: the calls of a shape are captured
        once in a CUDA graph and replayed (how a serving engine issues decode steps: the host
        cost of the operator call is paid at capture), with the copies on their own streams;
        False: issued call by call on one stream."""
        runs = []
        for p, m in shapes:
            def body(p=p, m=m):
                for i in range(e2e_steps):
                    e2e_call(p, m, (1 + i) % p.copies)
            if graphs and e2e_steps:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    e2e_pipelined(p, m)
                runs.append(g.replay)
            else:
                runs.append(body)
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in shapes]
        sync_all()
        with torch.cuda.stream(stream):
            for (e0, e1), run in zip(evs, runs):
                if align is not None and graphs:
                    dist.all_reduce(align)
                e0.record()
                run()
                e1.record()
        sync_all()
        out = torch.tensor([e0.elapsed_time(e1) for e0, e1 in evs], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(out, op=dist.ReduceOp.MAX)
        return out.tolist()

    ms2 = time_e2e(use_graphs)
    ms2_eager = time_e2e(False)
    extra["e2e_eager"] = ms2_eager

    shapes4 = [(p, m) for p in pools4 for m in MS4]
    if shapes4:
        with torch.cuda.stream(stream):
            for p, m in shapes4:
                raw_call(p, m, 0)
        torch.cuda.synchronize()
        steps4 = max(1, min(args.steps, 5))
        t4, n4 = time_shapes(shapes4, steps4)
        launches += n4
        g4 = None
        if dist is not None:
            g4, n4g = time_shapes([(p, m) for p, m in shapes4 if p.row_parallel], steps4, reduce=False)
            launches += n4g
        extra["config4"] = (shapes4, t4, g4, steps4)
    if os.environ.get("BENCH_NO_FP4", "0") != "1":
        extra["fp4"] = time_fp4(torch, ops, dev, dt, stream, gen, ws, min(args.steps, 10))
        extra["moe"] = time_moe(torch, ops, dev, dt, stream, gen, ws, min(args.steps, 10))
    decode = run_decode(world, rank, dev) if os.environ.get("BENCH_NO_DECODE", "0") != "1" else None
    if rank == 0:
        report(args, world, shapes, ms, total_ms, ms2, e2e_steps, launches, clocks, decode,
               ar_check=ar_check, extra=extra)
    if dist is not None:
        # CUDA graphs that captured NCCL kernels are still alive: tearing the communicator down
        # under them can block, so leave together and let process exit release everything
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def time_fp4(torch, ops, dev, dt, stream, gen, ws, steps):
    """NVFP4 (float4_e2m1f weights, float8_e4m3fn scales per 16 values, one global scale) on the
    Llama-3-8B gate_up shape through the torch operator, device-resident inputs, a CUDA graph of
    `steps` calls over rotating weight copies: us per call at M = 1, 16, 64, 1024.  Random codes
    and scale bytes of the processed form (the kernel's time does not depend on the values)."""
    from vllm_b200.scalar_type import scalar_types
    k, n, group = 4096, 28672, 16
    copies = 8
    qs = [torch.randint(-2**31, 2**31 - 1, (k // 16, n * 2), dtype=torch.int32, device=dev,
                        generator=gen) for _ in range(copies)]
    # scale bytes: exponent field 0b1xxxx (what non-zero scales look like after processing)
    ss = [(torch.randint(0, 64, (k // group, n), dtype=torch.uint8, device=dev, generator=gen) | 0x80)
          .view(torch.float8_e4m3fn) for _ in range(copies)]
    gs = torch.full((1,), 2.0 ** -7, dtype=dt, device=dev)
    rows = []
    for m in (1, 16, 64, 1024):
        a = torch.randn((m, k), dtype=dt, device=dev, generator=gen)

        def body():
            for i in range(steps):
                ops.gptq_marlin_gemm(a, None, qs[i % copies], None, ss[i % copies], gs, None, None, None,
                                     ws, scalar_types.float4_e2m1f, m, n, k)
        with torch.cuda.stream(stream):
            body()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            body()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            g.replay()
            e0.record()
            g.replay()
            e1.record()
        torch.cuda.synchronize()
        us = 1e3 * e0.elapsed_time(e1) / steps
        b = k * n // 2 + (k // group) * n + 2 * m * k + 2 * m * n      # weights, scale bytes, A, C
        rows.append({"m": m, "us": round(us, 2), "gbs": round(b / us / 1e3, 1),
                     "tflops": round(2.0 * m * n * k / us / 1e6, 2)})
    return {"workload": "nvfp4 (float4_e2m1f, group 16) gate_up 4096->28672, reference-order kernel",
            "steps": steps, "per_shape": rows}


def time_moe(torch, ops, dev, dt, stream, gen, ws, steps):
    """moe_wna16_marlin_gemm on a Mixtral-8x7B-shaped gate_up projection (8 experts, top-2,
    4096 -> 2 x 14336, uint4b8 g128): us per call at 16 and 256 tokens, device-resident inputs,
    a CUDA graph of `steps` calls over two weight sets (940 MB: larger than L2).  The bytes counted
    are the weights and scales of the experts that received tokens."""
    from vllm_b200 import fused_moe
    from vllm_b200.scalar_type import scalar_types
    e, topk, k, n, group = 8, 2, 4096, 28672, 128
    qs = [torch.randint(-2**31, 2**31 - 1, (e, k // 16, n * 2), dtype=torch.int32, device=dev,
                        generator=gen) for _ in range(2)]
    ss = [(torch.rand((e, k // group, n), device=dev, generator=gen) * 0.018 + 0.002).to(dt)
          for _ in range(2)]
    rows = []
    for m in (16, 256):
        a = torch.randn((m, k), dtype=dt, device=dev, generator=gen)
        topk_ids = torch.stack([torch.randperm(e, device=dev, generator=gen)[:topk] for _ in range(m)])
        tw = torch.rand((m * topk,), device=dev, generator=gen)
        for bs in (8, 16, 32):                      # as fused_moe.fused_marlin_moe picks it
            if m * topk / e / bs < 0.9:
                break
        sorted_ids, expert_ids, num = fused_moe.moe_align_block_size(topk_ids.to(torch.int32), bs, e)
        used = int(torch.unique(topk_ids).numel())

        def body():
            for i in range(steps):
                ops.moe_wna16_marlin_gemm(a, None, qs[i % 2], None, ss[i % 2], None, None, None, None, ws,
                                          sorted_ids, expert_ids, num, tw, bs, topk, False, False,
                                          scalar_types.uint4b8, m, n, k)
        with torch.cuda.stream(stream):
            body()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            body()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            g.replay()
            e0.record()
            g.replay()
            e1.record()
        torch.cuda.synchronize()
        us = 1e3 * e0.elapsed_time(e1) / steps
        b = used * (k * n // 2 + (k // group) * n * 2) + 2 * m * k + 2 * m * topk * n
        rows.append({"tokens": m, "block": bs, "experts_used": used, "us": round(us, 2),
                     "gbs": round(b / us / 1e3, 1),
                     "tflops": round(2.0 * m * topk * n * k / us / 1e6, 2)})
    return {"workload": "moe_wna16_marlin_gemm: 8 experts, top-2, gate_up 4096 -> 28672, uint4b8 g128, "
                        "reference-order kernel", "steps": steps, "per_shape": rows}


def run_ar_check(torch, dist, D, lib, dev, custom_ar, ar_link, rank, world):
    """Value check of the peer-memory all-reduce kernels before anything is timed: each is
    compared, bit for bit, with NCCL's all-reduce of the same un-reduced partials, on
    integer-valued inputs whose sums are exact in fp16 (the method of the reference's
    tests/distributed/test_custom_all_reduce.py:60-82).  Cases: the GEMM with the all-reduce
    in its epilogue (M = 1, 16, 32) and followed by the all-reduce kernel (M = 48), the
    stand-alone kernel at one-shot and two-shot sizes, and all-reduce + residual add +
    RMSNorm in one kernel.  A mismatch ends the run with a non-zero exit code."""
    from vllm_b200 import _custom_ops as ops
    from vllm_b200 import _lib
    from vllm_b200 import marlin_utils as mu
    from vllm_b200.scalar_type import scalar_types
    if custom_ar is None:
        return {"cases": 0, "ok": True, "note": "peer-memory all-reduce not active (NCCL only)"}
    import ctypes
    vp = ctypes.c_void_p
    dt = torch.float16
    gen = torch.Generator(device=dev).manual_seed(4321 + rank)
    cases, bad = 0, []
    cur = lambda: vp(torch.cuda.current_stream().cuda_stream)
    # ---- GEMM + all-reduce: K shard of 256 rows, unit scales, activations in {-1, 0, 1} ----
    K, N = 256, 4096
    q = torch.randint(-2**31, 2**31 - 1, (K // 16, N * 2), dtype=torch.int32, device=dev, generator=gen)
    s_ = torch.ones((K // GROUP, N), dtype=dt, device=dev)
    ws = mu.marlin_make_workspace_new(dev)
    nscr = lib.b200q_marlin_gemm_preferred_scratch_bytes(64, N, K, 0)
    scratch = torch.empty(nscr, dtype=torch.uint8, device=dev)
    flags = _lib.FLAG_K_FULL | _lib.FLAG_FP32_REDUCE
    for m in (1, 16, 32, 48):
        a = torch.randint(-1, 2, (m, K), device=dev, generator=gen).to(dt)
        part, got = torch.empty((m, N), dtype=dt, device=dev), torch.empty((m, N), dtype=dt, device=dev)
        args = lambda c: (vp(a.data_ptr()), K, vp(q.data_ptr()), vp(s_.data_ptr()), None, None, None,
                          None, vp(c.data_ptr()), vp(scratch.data_ptr()), nscr, vp(ws.data_ptr()),
                          ws.numel(), scalar_types.uint4b8.id, _lib.F16, m, N, K, K // GROUP, flags)
        _lib.check(lib.b200q_marlin_gemm(*args(part), cur()), "b200q_marlin_gemm")
        _lib.check(lib.b200q_marlin_gemm_all_reduce(*args(got), *ar_link, cur()),
                   "b200q_marlin_gemm_all_reduce")
        dist.all_reduce(part)
        torch.cuda.synchronize()
        cases += 1
        if not torch.equal(got, part):
            bad.append("gemm_all_reduce m=%d" % m)
    # ---- stand-alone kernel: one-shot sizes, and 512 KiB (two-shot from four ranks up) ----
    for shape in ((1, 4096), (16, 4096), (64, 4096), (256, 4096)):
        x = torch.randint(-8, 9, shape, device=dev, generator=gen).to(dt)
        want = x.clone()
        dist.all_reduce(want)
        got = custom_ar.custom_all_reduce(x)
        torch.cuda.synchronize()
        cases += 1
        if got is None or not torch.equal(got, want):
            bad.append("all_reduce %dx%d" % shape)
    # ---- all-reduce + residual add + RMSNorm in one kernel vs NCCL, then the local kernel ----
    common = torch.Generator(device=dev).manual_seed(99)         # same on every rank
    for (m, n) in ((1, 4096), (64, 4096)):
        part = torch.randint(-4, 5, (m, n), device=dev, generator=gen).to(dt)
        res = torch.randint(-4, 5, (m, n), device=dev, generator=common).to(dt)
        w = (1 + 0.125 * torch.randint(-2, 3, (n,), device=dev, generator=common)).to(dt)
        want_x, want_res = part.clone(), res.clone()
        dist.all_reduce(want_x)
        ops.fused_add_rms_norm(want_x, want_res, w, 1e-5)
        got_x, got_res = part.clone(), res.clone()
        done = custom_ar.all_reduce_add_rms_norm(got_x, got_res, w, 1e-5)
        torch.cuda.synchronize()
        cases += 1
        if not (done and torch.equal(got_x, want_x) and torch.equal(got_res, want_res)):
            bad.append("all_reduce_add_rms_norm %dx%d" % (m, n))
    err = lib.b200q_device_error(1)
    flag = torch.tensor([len(bad) + (1 if err else 0)], dtype=torch.int64, device=dev)
    dist.all_reduce(flag)
    if int(flag.item()) != 0:
        sys.stderr.write("rank %d: all-reduce value check FAILED: %s (device error 0x%x)\n"
                         % (rank, bad, err))
        if rank == 0:
            emit({"metric": METRIC, "ar_check": {"cases": cases, "ok": False, "failed": bad}})
        dist.barrier()
        sys.stdout.flush()
        os._exit(3)
    return {"cases": cases, "ok": True,
            "what": "bitwise equality with NCCL all-reduce on integer-valued fp16 inputs"}


def run_decode(world, rank, dev):
    """Third part of the metric: greedy decode of a Llama-3-8B-shaped model (random weights, GPTQ
    uint4b8 g128) whose projections all run through this library, tensor-parallel over the ranks.
    Batch 64, prompt 512, CUDA-graph decode steps timed with CUDA events, max over ranks."""
    import torch
    try:
        from vllm_b200.e2e_llama import LlamaConfig, LlamaDecoder, generate
        batch, prompt, new = 64, 512, 128
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


def report(args, world, shapes, ms, total_ms, ms2, e2e_steps, launches, clocks, decode=None,
           ar_check=None, extra=None):
    peaks = load_peaks()
    k_steps = args.steps
    div = lambda a, b: a / b if b else 0.0          # --only leaves some classes empty
    rows = []
    dec_b = dec_t = ten_f = ten_t = e2e_b = e2e_t = str_b = str_t = 0.0
    for (p, m), t, t2 in zip(shapes, ms, ms2):
        b, f = algorithmic_bytes(m, p.n, p.k), 2.0 * m * p.n * p.k
        us = 1e3 * t / k_steps
        rows.append({"layer": p.name, "k": p.k, "n": p.n, "m": m, "us": round(us, 2),
                     "gbs": round(b / us / 1e3, 1), "tflops": round(f / us / 1e6, 2),
                     "e2e_us": round(div(1e3 * t2, e2e_steps), 2)})
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
    value = world * div(dec_b, dec_t) / 1e6        # GB/s, all ranks
    tflops = world * div(ten_f, ten_t) / 1e9
    per_gpu_gbs, per_gpu_tf = value / world, tflops / world
    stream_gbs = div(str_b, str_t) / 1e6  # per GPU: every rank runs the same shapes
    # DRAM bytes (read + write) of one launch of the dominant decode kernel, from the ncu capture
    # summarised in profiles/gemm_stream_gate_up_m16.txt: gate_up with act-order, M = 16,
    # 60.73 MB read + 0.32 MB written for 61.6 MB algorithmic (the gather kernel in front of it
    # adds 0.15 MB: profiles/permute_cols_gate_up_m16.txt)
    traffic = 61.04e6
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": k_steps,
        "warmup": args.warmup, "ms_per_step": total_ms / k_steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(world),
        "tflops_m_ge_1024": tflops,
        "roofline": {"bound": "hbm", "achieved": stream_gbs, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": stream_gbs / peaks["hbm_gbs"], "traffic": traffic,
                     "traffic_launch": "gemm_stream_kernel, gate_up 4096->28672 with act-order, M=16: "
                                       "dram__bytes_read.sum + dram__bytes_write.sum of one launch "
                                       "under ncu (61.6e6 algorithmic bytes for the call)",
                     "peak_source": peaks["source"],
                     "scope": "dominant kernel gemm_stream_kernel: the M <= 16 calls (each = act-order "
                              "gather + decode GEMM), algorithmic bytes / CUDA-event time, per GPU",
                     "frac_m_le_64": per_gpu_gbs / peaks["hbm_gbs"]},
        "roofline_tensor": {"bound": "tensor", "achieved": per_gpu_tf, "peak": peaks["bf16_tflops"],
                            "unit": "TFLOP/s", "frac": per_gpu_tf / peaks["bf16_tflops"],
                            "traffic": None, "peak_source": peaks["source"],
                            "scope": "M >= 1024 calls"},
        "e2e": {"value": world * div(e2e_b, e2e_t) / 1e6, "unit": "GB/s",
                "h2d_bytes_per_step": sum(2 * m * p.k for p, m in shapes),
                "d2h_bytes_per_step": sum(2 * m * p.n for p, m in shapes),
                "steps": e2e_steps,
                "path": "torch op gptq_marlin_gemm (C++ registration; gptq_marlin_gemm_all_reduce "
                        "for row-parallel layers at N > 1); A from pinned host memory, C back to "
                        "pinned host memory every call; weights resident (the op takes device "
                        "tensors); the calls of a shape are captured in one CUDA graph and replayed: "
                        "every step copies its A in and its C out, on copy streams beside the "
                        "operator call of the neighbouring steps (two device buffers for A); "
                        "eager_value = the same calls issued one by one on one stream"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "decode": decode,
        "per_shape": rows,
    }
    if ar_check is not None:
        line["ar_check"] = ar_check
    extra = extra or {}
    if "e2e_eager" in extra:
        eb = et = 0.0
        for (p, m), t2, row in zip(shapes, extra["e2e_eager"], rows):
            row["e2e_eager_us"] = round(div(1e3 * t2, e2e_steps), 2)
            if m <= 64:
                eb += algorithmic_bytes(m, p.n, p.k) * e2e_steps
                et += t2
        line["e2e"]["eager_value"] = world * div(eb, et) / 1e6
    if "gemm_only" in extra:
        # row-parallel shapes without their all-reduce: what the collective costs at this N
        rp, g2 = extra["gemm_only"]
        by_key = {(p.name, m): t for (p, m), t in zip(rp, g2)}
        for row in rows:
            if (row["layer"], row["m"]) in by_key:
                row["us_gemm_only"] = round(1e3 * by_key[(row["layer"], row["m"])], 2)
    if "config4" in extra:
        shapes4, t4, g4, steps4 = extra["config4"]
        rows4, gi = [], 0
        for (p, m), t in zip(shapes4, t4):
            b, f = algorithmic_bytes(m, p.n, p.k, act_order=False), 2.0 * m * p.n * p.k
            us = 1e3 * t
            row = {"layer": p.name, "k": p.k, "n": p.n, "m": m, "us": round(us, 2),
                   "gbs": round(b / us / 1e3, 1), "tflops": round(f / us / 1e6, 2),
                   "frac_hbm": round(b / us / 1e3 / peaks["hbm_gbs"], 3),
                   "frac_tensor": round(f / us / 1e6 / peaks["bf16_tflops"], 3)}
            if g4 is not None and p.row_parallel:
                row["us_gemm_only"] = round(1e3 * g4[gi], 2)
                gi += 1
            rows4.append(row)
        line["config4"] = {
            "workload": "llama3_70b_gptq_uint4b8_g128 tensor-parallel shards at tp=%d: gate_up "
                        "8192->57344/tp (column-parallel), down 28672/tp->8192 (row-parallel + "
                        "all-reduce)" % world,
            "m_values": MS4, "steps": steps4, "per_shape": rows4}
    if "fp4" in extra:
        for row in extra["fp4"]["per_shape"]:
            row["frac_hbm"] = round(row["gbs"] / peaks["hbm_gbs"], 3)
        line["fp4"] = extra["fp4"]
    if "moe" in extra:
        for row in extra["moe"]["per_shape"]:
            row["frac_hbm"] = round(row["gbs"] / peaks["hbm_gbs"], 3)
        line["moe"] = extra["moe"]
    if world == 1 and e2e_steps:
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
    ap.add_argument("--only", default=None, metavar="LAYER:M",
                    help="profiling aid: time one (layer, M) of the sweep alone, e.g. gate_up:16, "
                         "without the end-to-end / decode / config-4 / CPU parts; the line it "
                         "prints is not a benchmark result")
    args = ap.parse_args()
    if args.only:
        name, m = args.only.split(":")
        global LAYERS, MS
        LAYERS = [layer for layer in LAYERS if layer[0] == name]
        MS = [int(m)]
        if not LAYERS:
            raise SystemExit("--only: unknown layer %r" % name)
        for key in ("BENCH_NO_DECODE", "BENCH_NO_CONFIG4", "BENCH_NO_E2E", "BENCH_NO_FP4"):
            os.environ[key] = "1"
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
