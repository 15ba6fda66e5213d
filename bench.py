#!/usr/bin/env python
"""Benchmark of the int4 dequant decode product (M=1) on LLaMA-7B layer shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode product ``y = x @ W`` (M=1, fp16) on every layer of a pool of
synthetic GPTQ v2 layers (groupsize 128, no act-order): ``--copies`` distinct copies of each of
the three LLaMA-7B shapes 4096x4096, 4096x11008, 11008x4096.  The pool is several times larger
than L2, so every launch streams its weights from HBM.  The reported value is algorithmic
bytes (every operand once) per second, summed over ranks; ranks are independent replicas with
their own pool (the path has no cross-GPU exchange).

``--impl reference`` times the reference's own decode path on the same pool: its ``quant_cuda``
kernels, compiled unmodified for sm_100a into oracle/_ref/ (oracle/build_ref.py), driven as
``matmul_utils_4bit._matmul4bit_v2`` drives them in its default ``faster_mode='old_faster'``
(matmul_utils_4bit.py:84-87).  Where that extension was never built the arm falls back to the CPU
restatement of the reference's composition (reconstruct to fp16 + fp32 matmul,
matmul_utils_4bit.py:114-127; oracle/q4_oracle.py) on this box's host cores; the reference itself
has no CPU implementation of the path.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from alpaca_lora_4bit_b200 import synth  # noqa: E402

SHAPES = [(4096, 4096), (4096, 11008), (11008, 4096)]
GROUPSIZE = 128
METRIC = "int4_dequant_gemv_m1_gbs"
UNIT = "GB/s"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi, every sample stamped with the host
    time it arrived.  The sampler is started ahead of the load (nvidia-smi needs up to a few seconds before
    its first line on a box with many GPUs); ``summary(t0, t1)`` keeps the samples of that window."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index, enabled=True):
        self.index, self.rows, self.proc, self.enabled = index, [], None, enabled

    def __enter__(self):
        if not self.enabled:
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def wait_ready(self, timeout=10.0):
        """Blocks until the first sample has arrived (or ``timeout`` seconds have passed)."""
        t0 = time.time()
        while self.proc is not None and not self.rows and time.time() - t0 < timeout and self.proc.poll() is None:
            time.sleep(0.01)

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self, t0=None, t1=None):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, r in self.rows:
            if (t0 is not None and t < t0) or (t1 is not None and t > t1):
                continue
            try:
                sm.append(float(r[0])); mx = max(mx, float(r[1]))
            except Exception:
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def ncu_dram_bytes_per_launch():
    """DRAM bytes (read + write) of one launch of the decode kernel, averaged over the three layer shapes, and the
    kernel the capture was taken on: the ``dram_bytes_<KxN>`` and ``kernel`` lines of the ncu summary under
    profiles/ (written from ``dram__bytes_read.sum + dram__bytes_write.sum`` of one capture per shape).  None when
    the summary is missing or names another kernel than the one that runs now."""
    path = os.path.join(ROOT, "profiles", "gemv_ws_kernel_c1_m1.md")
    try:
        vals, kernel = {}, None
        with open(path) as f:
            for line in f:
                line = line.strip().strip("`")
                if line.startswith("dram_bytes_"):
                    k, v = line.split("=")
                    vals[k.strip()[len("dram_bytes_"):]] = int(v.strip().replace(",", ""))
                elif line.startswith("kernel ="):
                    kernel = line.split("=", 1)[1].strip()
        want = [f"{K}x{N}" for K, N in [(4096, 4096), (4096, 11008), (11008, 4096)]]
        if kernel != DECODE_KERNEL or any(w not in vals for w in want):
            return None
        return round(sum(vals[w] for w in want) / 3)
    except OSError:
        return None


DECODE_KERNEL = "gemv_ws_kernel<16,2,1>"


def make_pool(copies, device, seed):
    """``copies`` x 3 layers generated on the device (same distributions as synth.make_layer)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    pool = []
    for _ in range(copies):
        for K, N in SHAPES:
            G = K // GROUPSIZE
            qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 8, N), generator=gen, device=device, dtype=torch.int64).to(torch.int32)
            zl = torch.randint(0, 15, (G, N), generator=gen, device=device, dtype=torch.int64)
            sh = torch.arange(8, device=device, dtype=torch.int64) * 4
            zw = (zl.reshape(G, N // 8, 8) << sh).sum(-1)
            zw = torch.where(zw >= 2 ** 31, zw - 2 ** 32, zw).to(torch.int32)
            sc = (torch.rand((G, N), generator=gen, device=device) * 0.018 + 0.002).half()
            pool.append(synth.QuantLayer(qw, zw, sc, None, K, N, GROUPSIZE))
    return pool


def bytes_per_step(copies):
    return copies * sum(synth.gemv_bytes(1, K, N, GROUPSIZE) for K, N in SHAPES)


def run_ours(args, rank, world, local_rank):
    from alpaca_lora_4bit_b200 import _lib, matmul_utils_4bit as mm4b
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    L = _lib.lib()
    pool = make_pool(args.copies, dev, 1234 + rank)
    gen = torch.Generator(device=dev).manual_seed(99 + rank)
    xs = {K: torch.randn((1, K), generator=gen, device=dev).half() for K in sorted({k for k, _ in SHAPES})}
    ys = [torch.empty((1, l.N), dtype=torch.float16, device=dev) for l in pool]
    ws = _lib.workspace(dev, max(L.q4_gemv_workspace_bytes(1, K, N) for K, N in SHAPES))
    stream = torch.cuda.Stream(dev)
    n_launch = len(pool)

    def step():
        st = torch.cuda.current_stream(dev).cuda_stream
        for l, y in zip(pool, ys):
            rc = L.q4_gemv(xs[l.K].data_ptr(), l.qweight.data_ptr(), y.data_ptr(), l.scales.data_ptr(),
                           l.qzeros.data_ptr(), None, None, 1, l.K, l.N, l.K // GROUPSIZE, GROUPSIZE,
                           _lib.Q4_F16, 0, ws.data_ptr(), ws.numel(), st)
            if rc:
                _lib.check(rc, "gemv")

    def barrier():
        if world > 1:
            torch.distributed.barrier()

    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # The timed region of the default run lasts a few milliseconds, nvidia-smi delivers a sample every
        # 50 ms: the warm-up replays of the same graph therefore run for at least 0.4 s right up to the timed
        # region, and the clock record is the samples from the start of that load to the end of the timed
        # region (rank 0 samples its own GPU; every rank runs the same load).
        with ClockSampler(local_rank, enabled=(rank == 0)) as clk:
            clk.wait_ready()
            barrier()
            t_load = time.time()
            n_warm = 0
            while n_warm < max(args.warmup, 3) or time.time() - t_load < args.load_seconds:
                graph.replay()
                n_warm += 1
                if n_warm % 64 == 0:
                    stream.synchronize()
            stream.synchronize()
            barrier()
            torch.cuda.synchronize(dev)
            e0.record(stream)
            for _ in range(args.steps):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
            t_end = time.time()
            time.sleep(0.06)                     # the sample that covers the end of the region
        clocks = clk.summary(t_load + 0.05, t_end + 0.06)
        torch.cuda.synchronize(dev)
        barrier()
        ms = e0.elapsed_time(e1)

        # per-shape breakdown (same graph-free launches, one event pair per shape), rank 0 only
        per_shape = {}
        if rank == 0:
            for K, N in SHAPES:
                sel = [(l, y) for l, y in zip(pool, ys) if (l.K, l.N) == (K, N)]
                g2 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g2, stream=stream):
                    st = torch.cuda.current_stream(dev).cuda_stream
                    for l, y in sel:
                        L.q4_gemv(xs[K].data_ptr(), l.qweight.data_ptr(), y.data_ptr(), l.scales.data_ptr(),
                                  l.qzeros.data_ptr(), None, None, 1, K, N, K // GROUPSIZE, GROUPSIZE,
                                  _lib.Q4_F16, 0, ws.data_ptr(), ws.numel(), st)
                reps = 20
                graph.replay()          # evict this shape's weights from L2 with the whole pool
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                tot = 0.0
                for _ in range(reps):
                    graph.replay()
                    a.record(stream); g2.replay(); b.record(stream)
                    stream.synchronize()
                    tot += a.elapsed_time(b)
                us = tot / reps / len(sel) * 1e3
                per_shape[f"{K}x{N}"] = {"us_per_launch": round(us, 3),
                                         "gbs": round(synth.gemv_bytes(1, K, N, GROUPSIZE) / us / 1e3, 1)}

        # the same pool at the other batch sizes of the decode sweep (C1: M in {1, 4, 8, 16}), rank 0 only
        m_sweep = {}
        if rank == 0:
            wsm = _lib.workspace(dev, max(L.q4_gemv_workspace_bytes(16, K, N) for K, N in SHAPES))
            for M in (4, 8, 16):
                xm = {K: torch.randn((M, K), generator=gen, device=dev).half() for K in sorted({k for k, _ in SHAPES})}
                ym = [torch.empty((M, l.N), dtype=torch.float16, device=dev) for l in pool]
                gm = torch.cuda.CUDAGraph()
                with torch.cuda.stream(stream):
                    for capture in (False, True):
                        ctx = torch.cuda.graph(gm, stream=stream) if capture else contextlib.nullcontext()
                        with ctx:
                            st = torch.cuda.current_stream(dev).cuda_stream
                            for l, y in zip(pool, ym):
                                L.q4_gemv(xm[l.K].data_ptr(), l.qweight.data_ptr(), y.data_ptr(), l.scales.data_ptr(),
                                          l.qzeros.data_ptr(), None, None, M, l.K, l.N, l.K // GROUPSIZE, GROUPSIZE,
                                          _lib.Q4_F16, 0, wsm.data_ptr(), wsm.numel(), st)
                        stream.synchronize()
                    for _ in range(3):
                        gm.replay()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                    for _ in range(10):
                        gm.replay()
                    b.record(stream)
                    stream.synchronize()
                us = a.elapsed_time(b) / 10 / len(pool) * 1e3
                byt = sum(synth.gemv_bytes(M, l.K, l.N, GROUPSIZE) for l in pool) / len(pool)
                m_sweep[str(M)] = {"us_per_launch": round(us, 3), "gbs": round(byt / us / 1e3, 1)}
                del xm, ym, gm

    # ---- end to end through the Python operator surface, host buffers in, host buffers out
    for l in pool:
        l.g_idx = (torch.arange(l.K, device=dev) // GROUPSIZE).to(torch.int32)
    # One step = one pass over the pool: the step's inputs (one activation vector per layer width) go
    # host -> device from pinned memory, every layer runs through the public no-grad entry point, and
    # the step's result (all output vectors, gathered on the device) comes back in one device -> host copy.
    xh = {K: torch.randn((1, K)).half().pin_memory() for K in sorted({k for k, _ in SHAPES})}
    yh = torch.empty((1, sum(l.N for l in pool)), dtype=torch.float16).pin_memory()
    h2d = sum(v.numel() * 2 for v in xh.values())
    d2h = yh.numel() * 2

    def e2e_step():
        xd = {K: v.to(dev, non_blocking=True) for K, v in xh.items()}
        outs = [mm4b.matmul4bit(xd[l.K], l.qweight, l.scales, l.qzeros, l.g_idx, GROUPSIZE) for l in pool]
        yh.copy_(torch.cat(outs, dim=1), non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()

    def timed_host(fn, n):
        barrier()
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        torch.cuda.synchronize(dev)
        dt = (time.perf_counter() - t0) * 1e3
        barrier()
        return dt

    with torch.no_grad():
        for _ in range(3):
            e2e_step()
        e2e_steps = max(3, min(args.steps, 50))
        e2e_eager_ms = timed_host(e2e_step, e2e_steps)
        # The same step as a decode loop runs it in production: the host -> device copies, the per-layer calls of
        # the public entry point and the gather of the outputs recorded once as a CUDA graph (the entry point
        # allocates its outputs from the graph's pool and keeps its workspace per stream, so it can be captured),
        # then one replay plus the device -> host copy per step.  Host buffers in, host buffer out, every step.
        e2e_graph, yd = None, None
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                e2e_step()                                     # the stream's decode workspace exists before the capture
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    xd = {K: v.to(dev, non_blocking=True) for K, v in xh.items()}
                    outs = [mm4b.matmul4bit(xd[l.K], l.qweight, l.scales, l.qzeros, l.g_idx, GROUPSIZE) for l in pool]
                    yd = torch.cat(outs, dim=1)
            torch.cuda.current_stream(dev).wait_stream(side)
            e2e_graph = g
        except Exception as exc:                               # capture is an optimisation of the caller, not a requirement
            print(f"bench: the end-to-end step could not be captured ({type(exc).__name__}: {exc}); eager calls only", file=sys.stderr)

        def e2e_graph_step():
            e2e_graph.replay()
            yh.copy_(yd, non_blocking=True)
            torch.cuda.current_stream(dev).synchronize()

        if e2e_graph is not None:
            ref_out = torch.cat([mm4b.matmul4bit(xh[l.K].to(dev), l.qweight, l.scales, l.qzeros, l.g_idx, GROUPSIZE) for l in pool], dim=1).cpu()
            for _ in range(3):
                e2e_graph_step()
            assert torch.equal(yh, ref_out), "graph replay of the end-to-end step disagrees with the eager calls"
            e2e_ms = timed_host(e2e_graph_step, e2e_steps)
        else:
            e2e_ms = e2e_eager_ms

    if world > 1:
        t = torch.tensor([ms, e2e_ms, e2e_eager_ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms, e2e_ms, e2e_eager_ms = float(t[0]), float(t[1]), float(t[2])
    return dict(ms=ms, e2e_ms=e2e_ms, e2e_eager_ms=e2e_eager_ms, e2e_graphed=e2e_graph is not None, e2e_steps=e2e_steps,
                n_launch=n_launch, clocks=clocks, per_shape=per_shape, m_sweep=m_sweep, h2d=h2d, d2h=d2h)


def run_finetune(args, rank, world, local_rank):
    """LLaMA-7B-shape LoRA finetune step (C3): 32 layers, g128 int4 base, LoRA r=8 alpha=16 on q_proj/v_proj,
    micro-batch 4 x 256 uniform token ids per rank, fp16 autocast, gradient checkpointing, AdamW; data parallel
    with one NCCL all-reduce of the flat LoRA-gradient buffer.  Token ids come from pinned host memory every
    step and the loss is read back every step (inside the timed region)."""
    from alpaca_lora_4bit_b200 import finetune_step as fs
    dev = torch.device("cuda", local_rank)
    big = args.finetune_config == "70b"
    shape = fs.LlamaShape.llama2_70b() if big else fs.LlamaShape.llama_7b()
    if args.finetune_layers:
        shape.num_hidden_layers = args.finetune_layers
    # 80 random layers at unit gain overflow bf16 attention around layer 64: the deep model is built at gain 0.5
    model = fs.build_quant_llama(shape, dev, groupsize=128, act_order=big, seed=0, gain=0.5 if big else 1.0)
    if big:
        fs.add_lora(model, ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"], r=16, alpha=32,
                    std_a=0.02, std_b=0.01, seed=1)
    else:
        fs.add_lora(model, ["q_proj", "v_proj"], r=8, alpha=16, std_a=0.02, std_b=0.01, seed=1)
    if not args.finetune_stock_elementwise:
        from alpaca_lora_4bit_b200 import fused_ops
        # RMSNorm, SwiGLU, rotary: one kernel each way; gate and up as one layer where no adapter sits on them
        fused_ops.patch_llama(model, fuse_gate_up=not args.finetune_separate_gate_up)
    fs.apply_gradient_checkpointing(model)
    model.train()
    ft = fs.LoraFinetuner(model, lr=3e-4, autocast_dtype=torch.bfloat16 if big else torch.float16)
    B, T = (1, 2048) if big else (4, 256)
    gen = torch.Generator().manual_seed(1000 + rank)
    steps, warm = args.finetune_steps, 3
    ids_host = [torch.randint(0, shape.vocab_size, (B, T), generator=gen).pin_memory() for _ in range(steps + warm)]
    loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()

    def one(i):
        ids = ids_host[i].to(dev, non_blocking=True)
        loss = ft.step(ids)
        loss_host.copy_(loss.float().reshape(1), non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
        return float(loss_host[0])

    for i in range(warm):
        one(i)
    graphed = False
    if not args.finetune_eager:
        graphed = ft.capture(ids_host[0].to(dev))
        if world > 1:                                   # all ranks must take the same path
            flag = torch.tensor([1 if graphed else 0], device=dev)
            torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
            if int(flag[0]) == 0:
                ft._graph, graphed = None, False
        for i in range(warm):
            one(i)
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    losses = [one(warm + i) for i in range(steps)]
    e1.record()
    torch.cuda.synchronize(dev)
    if world > 1:
        torch.distributed.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t[0])
    tokens = B * T * world * steps
    p_lin = fs.quant_linear_params(model) + shape.vocab_size * shape.hidden_size
    flops_per_token = 4 * p_lin                      # forward 2P + backward-dx 2P, recompute not counted
    tps = tokens / (ms * 1e-3)
    out = {"metric": "llama2_70b_lora_finetune_tokens_per_s" if big else "llama7b_lora_finetune_tokens_per_s", "value": round(tps, 1), "unit": "tokens/s", "n_gpus": world,
           "steps": steps, "ms_per_step": round(ms / steps, 2), "layers": shape.num_hidden_layers,
           "micro_batch": [B, T], "lora": ("r=16 alpha=32 on q,k,v,o,gate,up,down; act-order g_idx; bf16 autocast" if big else
                                             "r=8 alpha=16 q_proj,v_proj, dropout 0 (as the reference forces under checkpointing)"),
           "lora_params": fs.lora_param_count(model), "allreduce_bytes_per_step": 4 * fs.lora_param_count(model) if world > 1 else 0,
           "model_tflops_per_s": round(tps * flops_per_token / 1e12, 1), "loss_first_last": [round(losses[0], 4), round(losses[-1], 4)], "launch": "cuda_graph" if graphed else "eager",
           "elementwise": "stock transformers modules" if args.finetune_stock_elementwise else "fused RMSNorm / SwiGLU / rotary kernels",
           "gate_up": "two layers" if (args.finetune_stock_elementwise or args.finetune_separate_gate_up or big) else "one fused layer [K, 2 I]",
           "h2d_bytes_per_step": B * T * 8, "d2h_bytes_per_step": 4}
    if args.finetune_profile and local_rank == 0:
        # device time per kernel of ONE eager step (torch.profiler; outside the timed region, after it)
        import collections
        from torch.profiler import ProfilerActivity, profile
        ids = ids_host[0].to(dev)
        ft._eager_step(ids)
        torch.cuda.synchronize(dev)
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            ft._eager_step(ids)
            torch.cuda.synchronize(dev)
        agg = collections.defaultdict(lambda: [0.0, 0])
        for e in prof.events():
            if e.device_type == torch.autograd.DeviceType.CUDA:
                agg[e.name][0] += e.device_time
                agg[e.name][1] += 1
        total = sum(v[0] for v in agg.values())
        out["kernels"] = {"sum_ms": round(total / 1e3, 2), "launches": sum(v[1] for v in agg.values()),
                          "top": [[name[:96], c, round(t / 1e3, 3), round(100 * t / total, 1)]
                                  for name, (t, c) in sorted(agg.items(), key=lambda kv: -kv[1][0])[:24]]}
    del ft, model
    torch.cuda.empty_cache()
    return out


def run_gemm(args, local_rank, reference_only=False):
    """C2: fused dequant-GEMM at M=2048 on LLaMA-13B layer shapes, act-order g128, forward and backward, next to the
    reference's composition (reconstruct to a dense fp16 buffer + library GEMM, matmul_utils_4bit.py:114-127) run
    twice: with this library's reconstruct kernel and with the reference's own (``vecquant4recons_v2`` of its
    extension built unmodified into oracle/_ref, where present).  Also the M=1024 products of the LLaMA-7B step.
    Tensor-core roofline: 2*M*K*N flop against the measured bf16 GEMM peak.  ``reference_only``: the reference
    composition alone (the ``--impl reference`` arm; nothing of this library runs)."""
    dev = torch.device("cuda", local_rank)
    gen = torch.Generator(device=dev).manual_seed(7)
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak = float(json.load(f)["bf16_tflops"])
        kind = "measured"
    except Exception:
        peak, kind = 1590.0, "fallback"
    ref = None
    try:
        from oracle import build_ref
        ref = build_ref.load()
    except Exception:
        ref = None
    if not reference_only:
        from alpaca_lora_4bit_b200 import quant_cuda

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize(dev)
        return a.elapsed_time(b) / reps

    out = {"peak_tflops": peak, "peak_kind": kind, "shapes": {}}
    cases = [(2048, 5120, 5120, True), (2048, 5120, 13824, True), (2048, 13824, 5120, True),
             (1024, 4096, 4096, False), (1024, 4096, 11008, False), (1024, 11008, 4096, False)]
    if getattr(args, "gemm_shape", ""):
        dims = [int(v) for v in args.gemm_shape.lower().split("x")]
        # KxN: the act-order M=2048 case of that layer; MxKxN: that many rows with sequential groups (the finetune shapes)
        cases = [(2048, dims[0], dims[1], True)] if len(dims) == 2 else [(dims[0], dims[1], dims[2], False)]
    for M, K, N, act in cases:
        G = K // 128
        qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 8, N), device=dev, dtype=torch.int64, generator=gen).to(torch.int32)
        zw = (torch.randint(0, 2 ** 31 - 1, (G, N // 8), device=dev, dtype=torch.int64, generator=gen) & 0x66666666).to(torch.int32)
        sc = (torch.rand((G, N), device=dev, generator=gen) * 0.018 + 0.002).half()
        gi = ((torch.randperm(K, device=dev, generator=gen) if act else torch.arange(K, device=dev)) // 128).int()
        x = torch.randn((M, K), device=dev, generator=gen).half()
        dy = torch.randn((M, N), device=dev, generator=gen).half()
        y = torch.empty((M, N), device=dev, dtype=torch.float16)
        dx = torch.empty((M, K), device=dev, dtype=torch.float16)
        w = torch.empty((K, N), device=dev, dtype=torch.float16)
        fl = 2.0 * M * K * N / 1e9
        row = {"M": M, "act_order": act}
        tm = timed(lambda: torch.matmul(x, w, out=y))
        tmb = timed(lambda: torch.matmul(dy, w.t(), out=dx))
        if ref is not None:
            trr = timed(lambda: ref.vecquant4recons_v2(qw, w, sc, zw, gi))
            row.update({"reference_recons_us": round(trr * 1e3, 1),
                        "reference_recons_plus_library_gemm_fwd_tflops": round(fl / (trr + tm), 1),
                        "reference_recons_plus_library_gemm_bwd_tflops": round(fl / (trr + tmb), 1)})
        if not reference_only:
            r = 16                                         # LoRA r=16, alpha=32: A ~ N(0, 0.02) [16, K], B ~ N(0, 0.02) [N, 16]
            la = (torch.randn((r, K), device=dev, generator=gen) * 0.02).half()
            lb = (torch.randn((N, r), device=dev, generator=gen) * 0.02).half()
            u = torch.nn.functional.pad((x @ la.t()) * 2.0, (0, 64 - r)).contiguous()
            v = torch.nn.functional.pad((dy @ lb) * 2.0, (0, 64 - r)).contiguous()
            tf = timed(lambda: quant_cuda.gemm(x, qw, y, sc, zw, gi))
            tb = timed(lambda: quant_cuda.gemm(dy, qw, dx, sc, zw, gi, transpose=True))
            tfl = timed(lambda: quant_cuda.gemm(x, qw, y, sc, zw, gi, lora_u=u, lora_w=lb))
            tbl = timed(lambda: quant_cuda.gemm(dy, qw, dx, sc, zw, gi, transpose=True, lora_u=v, lora_w=la))
            tr = timed(lambda: quant_cuda.vecquant4recons_v2(qw, w, sc, zw, gi))
            row.update({
                "fused_fwd_tflops": round(fl / tf, 1), "fused_bwd_tflops": round(fl / tb, 1),
                "fused_fwd_frac": round(fl / tf / peak, 3), "fused_bwd_frac": round(fl / tb / peak, 3),
                "fused_fwd_with_lora_r16_tflops": round(fl / tfl, 1), "fused_bwd_with_lora_r16_tflops": round(fl / tbl, 1),
                "recons_plus_library_gemm_fwd_tflops": round(fl / (tr + tm), 1),
                "recons_plus_library_gemm_bwd_tflops": round(fl / (tr + tmb), 1), "recons_us": round(tr * 1e3, 1)})
            if ref is not None:
                row["fused_over_reference_composition"] = [round((trr + tm) / tf, 2), round((trr + tmb) / tb, 2)]
        out["shapes"][f"M{M}_{K}x{N}"] = row
        del qw, zw, sc, gi, x, dy, y, dx, w
    torch.cuda.empty_cache()
    return out


def reference_gpu(args):
    """The reference's own decode path on this GPU: its compiled ``quant_cuda`` kernels (oracle/_ref, built
    unmodified from the reference sources) driven exactly as ``matmul_utils_4bit._matmul4bit_v2`` drives them
    in its default ``faster_mode='old_faster'`` (matmul_utils_4bit.py:84-87,94): zero-filled fp32 y, x.half(),
    scales.float() per call, the kernel on the legacy default stream, y.to(dtype).  Returns None when the
    extension is not there or there is no GPU."""
    from oracle import build_ref
    if not torch.cuda.is_available():
        return None
    ref = build_ref.load()
    if ref is None:
        return None
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    pool = make_pool(args.copies, dev, 1234)
    gen = torch.Generator(device=dev).manual_seed(99)
    xs = {K: torch.randn((1, K), generator=gen, device=dev).half() for K in sorted({k for k, _ in SHAPES})}

    def matmul4bit_v2(x, l):
        y = torch.zeros((x.shape[0], l.N), dtype=torch.float32, device=x.device)
        ref.vecquant4matmul_old_faster(x.half(), l.qweight, y, l.scales.float(), l.qzeros, GROUPSIZE, x.shape[-1] // 2)
        return y.to(x.dtype)

    def step():
        return [matmul4bit_v2(xs[l.K], l) for l in pool]

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize(dev)
    steps = max(1, min(args.steps, 50))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / steps
    # the same end-to-end step as this library's arm: inputs in from pinned memory, all outputs back in one copy
    xh = {K: torch.randn((1, K)).half().pin_memory() for K in sorted({k for k, _ in SHAPES})}
    yh = torch.empty((1, sum(l.N for l in pool)), dtype=torch.float16).pin_memory()
    t0 = time.perf_counter()
    for _ in range(steps):
        xd = {K: v.to(dev, non_blocking=True) for K, v in xh.items()}
        outs = [matmul4bit_v2(xd[l.K], l) for l in pool]
        yh.copy_(torch.cat(outs, dim=1), non_blocking=True)
        torch.cuda.synchronize(dev)
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    bps = bytes_per_step(args.copies)
    return {"gbs": bps / (ms * 1e-3) / 1e9, "ms": ms, "e2e_gbs": bps / (e2e_ms * 1e-3) / 1e9, "launches": len(pool),
            "h2d": sum(v.numel() * 2 for v in xh.values()), "d2h": yh.numel() * 2}


def cpu_reference(reps=3, threads=None):
    """The reference composition on the host cores, on the one-layer configuration it is defined for (K = N = 4096,
    groups of 128, M = 16 rows, everything from one seed): reconstruct W to fp16 (three roundings, as the
    reference's kernel), forward ``y = x @ W`` and backward ``dx = dy @ W.T`` in fp32 - oracle/q4_oracle.py, best
    of ``reps`` after one warm-up, each part timed on its own.  Returns the decode metric of the forward path
    (algorithmic bytes of the 16-row product over reconstruct + forward time) and the parts."""
    from oracle import q4_oracle as orc
    if threads:
        torch.set_num_threads(threads)
    K, N, M = 4096, 4096, 16
    layer = synth.make_layer(K, N, GROUPSIZE, False, seed=0)
    x = synth.make_acts(M, K, seed=1)
    dy = synth.make_acts(M, N, seed=2)

    def best_of(fn):
        fn()
        best = float("inf")
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            best = min(best, time.perf_counter() - t0)
        return best

    w = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    t_rec = best_of(lambda: orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx))
    t_fwd = best_of(lambda: orc.matmul_recons(x, w))
    t_bwd = best_of(lambda: orc.matmul_recons(dy, w, transpose=True))
    gbs = synth.gemv_bytes(M, K, N, GROUPSIZE) / (t_rec + t_fwd) / 1e9
    parts = {"reconstruct_s": round(t_rec, 5), "forward_s": round(t_fwd, 5), "backward_s": round(t_bwd, 5),
             "total_s": round(t_rec + t_fwd + t_bwd, 5), "threads": torch.get_num_threads(), "cpu_count": os.cpu_count()}
    return gbs, t_rec + t_fwd, torch.get_num_threads(), parts


CPU_SAMPLE = ("one 4096x4096 g128 layer, M=16 (the reference's single-layer CPU configuration): fp16 reconstruct + fp32 "
              "forward, best of the repetitions; backward dx = dy @ W.T timed beside it")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--copies", type=int, default=8, help="distinct copies of each layer shape per GPU")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-gemm", action="store_true", help="skip the M=2048 fused GEMM leg")
    ap.add_argument("--gemm-shape", default="", help="restrict the GEMM leg to one shape: KxN (M=2048, act-order), e.g. 5120x13824, or MxKxN (sequential groups), "
                         "e.g. 1024x4096x4096 (for profiler captures)")
    ap.add_argument("--load-seconds", type=float, default=0.4,
                    help="keep replaying the decode graph for at least this long before the timed region, so that the clock "
                         "sampler sees the GPU under this load (0 for profiler captures: warm-up replays only)")
    ap.add_argument("--decode-shape", default="", help="decode pool of one KxN layer shape instead of the three LLaMA-7B shapes, "
                                                       "e.g. 8192x28672 (for profiler captures; not the headline workload)")
    ap.add_argument("--finetune-steps", type=int, default=30, help="timed LoRA finetune steps (0 = skip)")
    ap.add_argument("--finetune-config", default="7b", choices=["7b", "70b"],
                    help="7b: LLaMA-7B, r=8 LoRA on q/v, 4 x 256 tokens, fp16 (C3); 70b: LLaMA-2-70B GQA, act-order, r=16 LoRA on "
                         "all seven projections, 1 x 2048 tokens, bf16 autocast (C4; 35 GB of int4 weights per GPU)")
    ap.add_argument("--finetune-eager", action="store_true", help="do not capture the finetune step as a CUDA graph")
    ap.add_argument("--finetune-profile", action="store_true",
                    help="after the timed steps run one eager step under torch.profiler and add its per-kernel device times as finetune.kernels")
    ap.add_argument("--finetune-stock-elementwise", action="store_true",
                    help="leave RMSNorm, SwiGLU and the rotary embedding to the stock transformers modules")
    ap.add_argument("--finetune-separate-gate-up", action="store_true",
                    help="keep gate_proj and up_proj two layers (default: one fused layer where no adapter sits on them)")
    ap.add_argument("--finetune-layers", type=int, default=0, help="override the number of decoder layers (0 = 32)")
    args = ap.parse_args()
    if args.decode_shape:
        SHAPES[:] = [tuple(int(v) for v in args.decode_shape.lower().split("x"))]

    # The one JSON line must be alone on stdout: libraries that write to file descriptor 1 on their own
    # (NCCL prints its version there) are sent to stderr until the line is printed.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(obj) + "\n").encode())

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    shapes_txt = "LLaMA-7B shapes 4096x4096+4096x11008+11008x4096" if not args.decode_shape else f"one shape {args.decode_shape} (not the headline workload)"
    config = {"workload": f"C1 decode GEMV M=1, {shapes_txt}, g128, "
                          f"{args.copies} copies each per GPU (pool > 2x L2, no flush needed)",
              "l2_policy": "inputs larger than L2", "launch": "cuda_graph", "parallelism": f"replicas x{world}"}

    if args.impl == "reference":
        if rank != 0:
            return
        rg = reference_gpu(args)
        if rg is not None:
            line = {"impl": "reference", "metric": METRIC, "value": round(rg["gbs"], 1), "unit": UNIT, "n_gpus": 1,
                    "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(rg["ms"], 5), "higher_is_better": True,
                    "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                    "config": dict(config, launch="eager, legacy default stream (as the reference launches)",
                                   parallelism="one GPU (the reference arm does not replicate)"),
                    "reference_path": "the reference's quant_cuda kernels, built unmodified for sm_100a (oracle/_ref), driven as "
                                      "matmul_utils_4bit._matmul4bit_v2 does with faster_mode='old_faster'",
                    "cpu_baseline": {"value": round(rg["gbs"], 1), "unit": UNIT, "cores": 0, "kind": "reference",
                                     "sample": "the whole workload, on the GPU: the reference has no CPU implementation of this path"},
                    "e2e": {"value": round(rg["gbs"], 1), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    # the same step as this library's end-to-end leg (inputs from pinned host memory, outputs back in one copy)
                    "e2e_with_host_copies": {"value": round(rg["e2e_gbs"], 1), "unit": UNIT, "h2d_bytes_per_step": rg["h2d"],
                                             "d2h_bytes_per_step": rg["d2h"]},
                    "gpu_launches": 0}
            if not args.no_gemm:
                line["gemm"] = run_gemm(args, 0, reference_only=True)     # reconstruct (its kernel) + library GEMM
            emit(line)
            return
        steps = max(1, min(args.steps, 5))
        gbs, sec, threads, parts = cpu_reference(reps=max(1, min(args.warmup, 2)) + steps)
        line = {"impl": "reference", "metric": METRIC, "value": round(gbs, 4), "unit": UNIT, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
                "data": "synthetic", "config": config,
                "cpu_baseline": dict({"value": round(gbs, 4), "unit": UNIT, "cores": threads, "kind": "port", "sample": CPU_SAMPLE}, **parts),
                "e2e": {"value": round(gbs, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        emit(line)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the kernels have no CPU path")
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    r = run_ours(args, rank, world, local_rank)
    gm = run_gemm(args, local_rank) if (rank == 0 and not args.no_gemm) else None
    ft = run_finetune(args, rank, world, local_rank) if args.finetune_steps > 0 else None
    if rank == 0:
        peak, peak_kind = load_peaks()
        bps = bytes_per_step(args.copies)
        value = bps * world * args.steps / (r["ms"] * 1e-3) / 1e9
        per_launch_us = r["ms"] * 1e3 / (args.steps * r["n_launch"])
        achieved = bps / r["n_launch"] / (per_launch_us * 1e-6) / 1e9
        e2e = bps * world * r["e2e_steps"] / (r["e2e_ms"] * 1e-3) / 1e9
        line = {"metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(r["ms"] / args.steps, 5), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": config,
                "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                             "frac": round(achieved / peak, 4), "traffic": None if args.decode_shape else ncu_dram_bytes_per_launch(),
                             "algorithmic_bytes_per_launch": round(bps / r["n_launch"]), "peak_kind": peak_kind,
                             "kernel": DECODE_KERNEL, "avg_launch_us": round(per_launch_us, 3),
                             "frac_of_nominal_8000": round(achieved / 8000.0, 4)},
                "per_shape": r["per_shape"], "m_sweep": r["m_sweep"],
                "e2e": {"value": round(e2e, 1), "unit": UNIT, "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"],
                        "api": "matmul_utils_4bit.matmul4bit per layer; per step the activation vectors come from pinned host memory and all "
                               "outputs go back in one copy; weights resident" +
                               ("; the step (copies in, the calls, the gather) is recorded once as a CUDA graph and replayed" if r["e2e_graphed"] else ""),
                        "launch": "cuda_graph" if r["e2e_graphed"] else "eager",
                        "eager_value": round(bps * world * r["e2e_steps"] / (r["e2e_eager_ms"] * 1e-3) / 1e9, 1)},
                "gpu_launches": args.steps * r["n_launch"], "clocks": r["clocks"]}
        if gm is not None:
            line["gemm"] = gm
        if ft is not None:
            line["finetune"] = ft
        if world == 1 and not args.no_cpu:
            gbs, sec, threads, parts = cpu_reference(reps=5)
            line["cpu_baseline"] = dict({"value": round(gbs, 4), "unit": UNIT, "cores": threads, "kind": "port", "sample": CPU_SAMPLE}, **parts)
        emit(line)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
