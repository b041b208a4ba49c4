#!/usr/bin/env python
"""Benchmark of the hybrid-attention hot path on B200.

Workload (the "full 64-layer hybrid stack decode" configuration): 64 layers in
the pattern 3 x Gated DeltaNet + 1 x Gated Attention, attention/DeltaNet
operators only, batch 32 sequences with ragged contexts uniform in
[8192, 32768] on a paged F16 KV cache (64-token pages, shuffled page table),
24Q/4KV heads of 256, 16K/48V DeltaNet heads of 128x128 FP32 state, conv k=4 over
10240 channels; seed 4; synthetic N(0,1) data.  One step = one decode step of
every sequence through all 64 layers (KV append + attend + gate; conv update +
delta rule).  Every step streams the whole KV cache and all recurrent state
(~50 GB), far more than the 126 MB L2, so no explicit L2 flush is needed.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

The timed region replays the step as one CUDA graph (rl_stack_decode); a second pass over the
same steps with CUDA events between the kernels supplies the per-kernel durations behind the
roofline object.  e2e goes through rl_stack_decode_host with pinned host buffers.

N > 1 (under torchrun, one rank per GPU): by default the batch is sharded by sequence -- every
rank owns 32 sequences of its own; there is no data-path collective (weak scaling).
--shard heads / --shard splitkv divide ONE batch of 32 over the ranks instead (strong scaling,
NCCL all_gather of head outputs / of attention partials merged by rl_lse_combine).
--workload selects single-operator lines (N = 1).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_LAYERS, N_Q, N_KV, HD = 64, 24, 4, 256
N_V, N_K, DK, DV, CONV_K = 48, 16, 128, 128, 4
CONV_DIM = 2 * N_K * DK + N_V * DV
PAGE = 64


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--ctx-min", type=int, default=8192)
    ap.add_argument("--ctx-max", type=int, default=32768)
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--seed", type=int, default=4)
    ap.add_argument("--workload", default="stack",
                    choices=["stack", "compact_decode", "f16_decode", "delta_step", "attn_prefill", "delta_prefill",
                             "stack_prefill"],
                    help="stack = the headline workload; the others time one operator at the shapes of "
                         "the single-layer configurations: 131 072-token compact-KV decode, 4 096-token F16 decode, one "
                         "DeltaNet step, 8 192-token prefills (secondary lines, N=1 only)")
    ap.add_argument("--shard", default="seq", choices=["seq", "heads", "splitkv"],
                    help="N > 1: seq = every rank owns 32 sequences of its own (weak scaling, no collective); "
                         "heads = ONE batch of 32 divided by KV / value heads (up to 4 ways) and then by sequence, "
                         "head outputs all-gathered over NCCL every step (strong scaling); "
                         "splitkv = ONE batch of 32, every rank holds 1/N of each sequence's KV pages and 1/N of "
                         "the DeltaNet heads; attention partials (o, max, sum) are all-gathered over NCCL and "
                         "merged by rl_lse_combine (strong scaling)")
    ap.add_argument("--wht-len", type=int, default=128)
    ap.add_argument("--op-batch", type=int, default=0, help="operator workloads: override the batch")
    ap.add_argument("--op-ctx", type=int, default=0, help="operator workloads: override the context")
    ap.add_argument("--chunk", type=int, default=None,
                    help="query rows per prefill call: attn_prefill default 8192, stack_prefill default 1024 "
                         "(the reference's chunk cap)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="plain launches instead of graph replay in the timed region")
    return ap.parse_args()


def contexts(args, rank):
    import torch
    g = torch.Generator().manual_seed(args.seed + 1000 * rank)
    return torch.randint(args.ctx_min, args.ctx_max + 1, (args.batch,), generator=g).tolist()


def workload_name(args):
    return ("hybrid_stack_decode: %d layers (3 DeltaNet + 1 GatedAttn), batch %d, ragged ctx U[%d,%d], "
            "paged F16 KV page 64" % (args.layers, args.batch, args.ctx_min, args.ctx_max))


def algorithmic_bytes(args, ctx):
    """Bytes one step must move, per kernel family (per layer-launch, and per step)."""
    B = len(ctx)
    n_attn = args.layers // 4
    n_delta = args.layers - n_attn
    attn_launch = sum(ctx) * N_KV * HD * 2 * 2 + B * N_Q * HD * 4 * 3
    delta_launch = B * (2 * N_V * DK * DV * 4 + 2 * (N_K * DK * 4) + N_V * DV * 4 * 2 + N_V * 8)
    conv_launch = B * (2 * CONV_DIM * CONV_K * 4 + 2 * CONV_DIM * 4) + CONV_DIM * CONV_K * 4
    append_launch = B * N_KV * HD * (4 + 2) * 2
    return {"attn_decode": attn_launch, "delta_rule": delta_launch, "conv1d_update": conv_launch,
            "kv_append": append_launch,
            "step": n_attn * (attn_launch + append_launch) + n_delta * (delta_launch + conv_launch)}


# --------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []
        self.first = 0

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self, wait_s=3.0):
        """Samples taken before this call (start-up of the tool, warm-up steps) are not reported;
        waits (bounded) until the tool has produced its first sample."""
        t0 = time.time()
        while self.proc and not self.lines and time.time() - t0 < wait_s:
            time.sleep(0.02)
        self.first = len(self.lines)

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines[self.first:]:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm),
                "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------
def cpu_reference_leg(args, ctx, seconds_budget=12.0, quiet=False):
    """Time the reference's CPU implementation of one step's operators on host cores.

    Attention: ops::attn_decode (scalar, one thread: the reference has no other CPU
    attention) on whole sequences of the workload; DeltaNet: ops::conv1d_update +
    ops::delta_recurrent_step_simd (AVX, WorkerPool threads) for the whole batch of one
    layer.  The per-layer costs are scaled to the 16 + 48 layers of a step.
    """
    import numpy as np

    import oracle as orc
    kind = "reference" if orc.Reference.available() else "port"
    impl = orc.Reference() if kind == "reference" else orc.Oracle()
    rng = np.random.default_rng(args.seed)
    # attention sample: the two shortest sequences of the batch, full context
    order = sorted(range(len(ctx)), key=lambda b: ctx[b])[:2]
    t_attn_tok = []
    for b in order:
        n = ctx[b]
        k = rng.standard_normal((n, N_KV, HD), dtype=np.float32).astype(np.float16).astype(np.float32)
        v = rng.standard_normal((n, N_KV, HD), dtype=np.float32).astype(np.float16).astype(np.float32)
        q = rng.standard_normal((N_Q, HD), dtype=np.float32)
        t0 = time.perf_counter()
        reps = 0
        while True:
            impl.attn_decode(q, k, v)
            reps += 1
            if time.perf_counter() - t0 > seconds_budget / 4:
                break
        t_attn_tok.append((time.perf_counter() - t0) / reps / n)
        del k, v
    attn_s_per_tok = float(np.mean(t_attn_tok))
    # DeltaNet sample: one layer, whole batch
    B = len(ctx)
    S = (rng.standard_normal((B, N_V, DK, DV), dtype=np.float32) * 0.02).astype(np.float32)
    cst = np.zeros((B, CONV_DIM, CONV_K), np.float32)
    w = (rng.standard_normal((CONV_DIM, CONV_K), dtype=np.float32) * 0.5).astype(np.float32)
    x = rng.standard_normal((B, CONV_DIM), dtype=np.float32)
    beta = rng.random((B, N_V), dtype=np.float32)
    g = -rng.random((B, N_V), dtype=np.float32)
    rep = N_V // N_K
    t0 = time.perf_counter()
    reps = 0
    while True:
        for b in range(B):
            mixed = impl.conv1d_update(x[b], w, cst[b])
            qq = np.repeat(mixed[:N_K * DK].reshape(N_K, DK), rep, axis=0)
            kk = np.repeat(mixed[N_K * DK:2 * N_K * DK].reshape(N_K, DK), rep, axis=0)
            vv = mixed[2 * N_K * DK:].reshape(N_V, DV)
            if kind == "reference":
                impl.delta_step(S[b], qq, kk, vv, beta[b], g[b], simd=True)
            else:
                impl.delta_step(S[b], qq, kk, vv, beta[b], g[b])
        reps += 1
        if time.perf_counter() - t0 > seconds_budget / 4:
            break
    delta_layer_s = (time.perf_counter() - t0) / reps
    n_attn = args.layers // 4
    n_delta = args.layers - n_attn
    step_s = n_attn * attn_s_per_tok * sum(ctx) + n_delta * delta_layer_s
    cores = impl.num_threads() if kind == "reference" else 1
    isa = impl.simd_name() if kind == "reference" else "scalar C"
    return {"value": len(ctx) / step_s, "unit": "seq-steps/s", "cores": cores, "kind": kind,
            "sample": ("ops::attn_decode (scalar, 1 thread) on the 2 shortest sequences (%d, %d tokens) of one "
                       "layer, scaled by tokens to 32 seq x %d layers; conv1d_update + delta_recurrent_step_simd "
                       "(%s, %d threads) on one whole layer x %d layers" %
                       (ctx[order[0]], ctx[order[1]], n_attn, isa, cores, n_delta)),
            "step_seconds": step_s, "attn_us_per_token_layer": attn_s_per_tok * 1e6,
            "delta_ms_per_layer_batch": delta_layer_s * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ctx = contexts(args, 0)
    steps = []
    for _ in range(max(0, args.warmup)):
        cpu_reference_leg(args, ctx, seconds_budget=2.0)
    base = None
    for _ in range(max(1, args.steps)):
        base = cpu_reference_leg(args, ctx, seconds_budget=max(2.0, 60.0 / max(1, args.steps)))
        steps.append(base["step_seconds"])
    step_s = sum(steps) / len(steps)
    value = len(ctx) * args.gpus / step_s
    line = {"impl": "reference", "metric": "hybrid-layer decode steps/sec", "value": value,
            "unit": "seq-steps/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(args), "l2": "inputs larger than L2",
                       "note": "reference CPU operators on host cores; each step is a bounded sample scaled to the "
                               "whole step; N ranks would each run the same CPU work, so value scales by n_gpus"},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": value, "unit": "seq-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    line["cpu_baseline"]["value"] = value
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
def run_operator(args):
    """Secondary lines: one operator at its single-layer benchmark shapes (single GPU)."""
    import torch

    import __graft_entry__ as ge
    ge.build()
    from rapidllm_b200 import _lib, ops
    torch.cuda.set_device(0)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    gen = torch.Generator(device="cuda").manual_seed(args.seed)
    wl = args.workload
    if args.chunk is None:
        args.chunk = 1024 if wl == "stack_prefill" else 8192
    if wl == "attn_prefill":
        T = args.op_ctx or 8192
        n_pages = (T + PAGE - 1) // PAGE
        cg = torch.Generator().manual_seed(args.seed)
        table = torch.randperm(n_pages, generator=cg).int().cuda()
        q = torch.randn(T, N_Q, HD, device="cuda", generator=gen).bfloat16()
        k = torch.randn(T, N_KV, HD, device="cuda", generator=gen).bfloat16()
        v = torch.randn(T, N_KV, HD, device="cuda", generator=gen).bfloat16()
        gate = torch.randn(T, N_Q, HD, device="cuda", generator=gen)
        kp, vp = ops.new_pool(n_pages, N_KV), ops.new_pool(n_pages, N_KV)

        def call():
            for p0 in range(0, T, args.chunk):
                sl = slice(p0, min(T, p0 + args.chunk))
                ops.attn_prefill(q[sl], kp, vp, table, p0, k[sl], v[sl], gate[sl])
        for _ in range(max(3, args.warmup)):
            call()
        _lib.check_device()
        sampler = ClockSampler(0)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            call()
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        _lib.check_device()
        ms = e0.elapsed_time(e1) / args.steps
        flops = 4.0 * N_Q * HD * T * (T + 1) / 2
        tpeak = float(peaks.get("bf16_tflops", 1590.0))
        achieved = flops / (ms * 1e-3) / 1e12
        # The back-to-back loop above runs under the 1 kW power cap (the SM clock drops to ~1.7 GHz within a
        # few calls).  The burst peak it is divided by is a best-of-10 of single GEMMs, so the like-for-like
        # figure is taken too: single calls after 20 ms of idle, best and median.
        import time as _time
        singles = []
        for _ in range(10):
            torch.cuda.synchronize()
            _time.sleep(0.02)
            b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            b0.record()
            call()
            b1.record()
            torch.cuda.synchronize()
            singles.append(b0.elapsed_time(b1))
        singles.sort()
        speak = float(peaks.get("bf16_tflops_sustained", 1400.0))
        print(json.dumps({
            "metric": "attention prefill tokens/sec (one layer)", "value": T / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic", "dtype": "f16 (bf16 in)",
            "config": {"workload": "gated attention chunked prefill, T %d in chunks of %d, 24Q/4KV hd256, causal, "
                       "writes F16 KV" % (T, args.chunk), "l2": "K/V of one layer fit L2 by design (32 MB)"},
            "clocks": clocks, "gpu_launches": args.steps * 2 * ((T + args.chunk - 1) // args.chunk),
            "roofline": {"bound": "tensor", "kernel": "attn_prefill_kernel", "achieved": achieved, "peak": tpeak,
                         "unit": "TFLOP/s", "frac": achieved / tpeak, "flops_per_step": flops, "traffic": None,
                         "peak_sustained": speak, "frac_of_sustained_peak": achieved / speak,
                         "single_calls_after_idle": {"ms_best": singles[0], "ms_median": singles[len(singles) // 2],
                                                     "frac_best": flops / (singles[0] * 1e-3) / 1e12 / tpeak,
                                                     "frac_median": flops / (singles[len(singles) // 2] * 1e-3) / 1e12 / tpeak},
                         "note": "achieved = back-to-back loop (power-capped clocks); frac divides it by the burst peak, "
                                 "frac_of_sustained_peak by the cuBLAS figure taken under the same cap"}}),
            flush=True)
        return
    if wl == "stack_prefill":
        # a prompt of T tokens through all layers' mixers in chunks (the reference's launch_prefill loop);
        # every chunk reuses one set of synthetic per-layer inputs (values do not change the work)
        from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
        T, chunk = args.op_ctx or 8192, min(args.chunk, args.op_ctx or 8192)
        types = (QWEN35_LAYER_TYPES * ((args.layers + 3) // 4))[:args.layers]
        pages = (T + PAGE - 1) // PAGE
        cache = HybridCache(types, n_pages=pages, n_slots=1, max_batch=1, max_pages_per_seq=pages)
        cg = torch.Generator().manual_seed(args.seed)
        row = torch.randperm(pages, generator=cg).int().cuda()
        t = {}
        for name, (shape, dtype) in cache.prefill_shapes(chunk).items():
            if name in ("attn_o", "delta_o"):
                t[name] = torch.empty(shape, dtype=dtype, device="cuda")
            elif name == "delta_beta":
                t[name] = torch.sigmoid(torch.randn(shape, device="cuda", generator=gen))
            elif name == "delta_g":
                t[name] = -torch.nn.functional.softplus(torch.randn(shape, device="cuda", generator=gen))
            else:
                t[name] = (torch.randn(shape, device="cuda", generator=gen) * (0.5 if name == "conv_w" else 1.0)).to(dtype)
        ws = torch.empty(max(256, max(_lib.lib().rl_stack_prefill_workspace_bytes(cache._h, p0, chunk)
                                      for p0 in range(0, T, chunk))), dtype=torch.uint8, device="cuda")
        n_chunks = (T + chunk - 1) // chunk

        def call():
            for p0 in range(0, T, chunk):
                n = min(chunk, T - p0)
                if n == chunk:
                    cache.prefill(t, row, 0, p0, n, ws)
                else:
                    cache.prefill({k_: (v_ if k_ == "conv_w" else v_[:, :n].contiguous()) for k_, v_ in t.items()}, row, 0,
                                  p0, n, ws)
        for _ in range(max(3, args.warmup)):
            call()
        _lib.check_device()
        sampler = ClockSampler(0)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            call()
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        _lib.check_device()
        ms = e0.elapsed_time(e1) / args.steps
        flops_attn = cache.n_attn * 4.0 * N_Q * HD * T * (T + 1) / 2
        tpeak = float(peaks.get("bf16_tflops", 1590.0))
        # per chunk: attention layers 2 launches (KV write, prefill), DeltaNet layers 3 (conv, prepare, scan)
        launches = n_chunks * (cache.n_attn * 2 + cache.n_delta * 3)
        print(json.dumps({
            "metric": "prompt tokens/sec through the hybrid stack's mixers", "value": T / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
            "dtype": "f16 attention (bf16 in) / f16 hi+lo + f32 state DeltaNet",
            "config": {"workload": "chunked prefill, %d layers (%d attention + %d DeltaNet), one sequence of %d tokens in "
                       "chunks of %d, mixers only (no projections / MLP)" % (len(types), cache.n_attn, cache.n_delta, T, chunk),
                       "l2": "per-chunk inputs of all layers (%.1f GB) exceed L2" %
                             (sum(x.numel() * x.element_size() for x in t.values()) / 1e9)},
            "clocks": clocks, "gpu_launches": args.steps * launches,
            "roofline": {"bound": "tensor", "kernel": "attn_prefill_kernel (attention layers only)",
                         "achieved": flops_attn / (ms * 1e-3) / 1e12, "peak": tpeak, "unit": "TFLOP/s",
                         "frac": flops_attn / (ms * 1e-3) / 1e12 / tpeak, "flops_per_step": flops_attn, "traffic": None,
                         "note": "whole-stack time in the denominator; the DeltaNet layers' chunk-to-chunk scan is "
                                 "latency-bound and takes most of it"}}), flush=True)
        return
    if wl == "delta_prefill":
        T = args.op_ctx or 8192
        S = torch.zeros(N_V, DK, DV, device="cuda")
        q = torch.randn(T, N_K, DK, device="cuda", generator=gen)
        k = torch.randn(T, N_K, DK, device="cuda", generator=gen)
        v = torch.randn(T, N_V, DV, device="cuda", generator=gen)
        beta = torch.sigmoid(torch.randn(T, N_V, device="cuda", generator=gen))
        gl = -torch.nn.functional.softplus(torch.randn(T, N_V, device="cuda", generator=gen))
        ws = torch.empty(_lib.lib().rl_delta_chunk_workspace_bytes(
            __import__("ctypes").byref(_lib.DeltaChunkParams(n_v=N_V, dk=DK, dv=DV, seq=T, chunk=64, eps_l2=1e-6,
                                                              n_qk=N_K, head_map=1))), dtype=torch.uint8, device="cuda")

        def call():
            S.zero_()
            ops.delta_chunk_prefill(S, q, k, v, beta, gl, workspace=ws)
        for _ in range(max(3, args.warmup)):
            call()
        _lib.check_device()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            call()
        e1.record()
        torch.cuda.synchronize()
        _lib.check_device()
        ms = e0.elapsed_time(e1) / args.steps
        n_chunks = (T + 63) // 64
        # tensor-core MMAs actually issued by the scan kernel per (chunk, head), M = 128:
        # D: 4 (N64,K16) + 16; O: 16 + 8; S: 8 (N128)  -> flops = 2*128*N*16 each
        flops = n_chunks * N_V * (2 * 128 * 16) * ((4 + 16 + 16 + 8) * 64 + 8 * 128)
        tpeak = float(peaks.get("bf16_tflops", 1590.0))
        achieved = flops / (ms * 1e-3) / 1e12
        print(json.dumps({
            "metric": "DeltaNet prefill tokens/sec (one layer)", "value": T / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
            "dtype": "f16 hi+lo operands / f32 state",
            "config": {"workload": "gated DeltaNet chunked (WY, chunk 64) prefill, T %d, batch 1, 16K/48V heads 128x128"
                       % T, "l2": "operands streamed once (0.5 GB workspace)",
                       "note": "one CTA per value head walks %d chunks in order: bound by the chunk-to-chunk "
                               "dependency, not by tensor throughput" % n_chunks},
            "gpu_launches": args.steps * 2,
            "roofline": {"bound": "tensor", "kernel": "delta_chunk_scan_kernel", "achieved": achieved, "peak": tpeak,
                         "unit": "TFLOP/s", "frac": achieved / tpeak, "flops_per_step": flops, "traffic": None}}),
            flush=True)
        return
    if wl in ("compact_decode", "f16_decode"):
        if wl == "compact_decode":
            B, ctx = 4, 131072
        else:
            B, ctx = 1, 4096
        B, ctx = args.op_batch or B, args.op_ctx or ctx
        pages = ctx // PAGE
        n_pages = B * pages
        cg = torch.Generator().manual_seed(args.seed)
        table = torch.randperm(n_pages, generator=cg).int().reshape(B, pages).cuda()
        lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        q = torch.randn(B, N_Q, HD, device="cuda", generator=gen)
        gate = torch.randn(B, N_Q, HD, device="cuda", generator=gen)
        if wl == "compact_decode":
            signs = None
            if args.wht_len == 256:
                signs = (2.0 * torch.bernoulli(torch.full((256,), 0.5, device="cuda"), generator=gen) - 1.0)
            pool = ops.new_compact_pool(n_pages, N_KV)
            step = 8192
            for b in range(B):
                for t0 in range(0, ctx, step):
                    k = torch.randn(step, N_KV, HD, device="cuda", generator=gen)
                    v = torch.randn(step, N_KV, HD, device="cuda", generator=gen)
                    ops.kv_compact_append(pool, table[b], k, v, args.wht_len, signs, pos0=t0)
            per_tok = _lib.lib().rl_kv_compact_page_bytes() // PAGE
            call = lambda: ops.attn_decode(q, pool, None, table, lens, gate, wht_len=args.wht_len, signs=signs,
                                           workspace=ws, out=out)
            kernel = "attn_decode_tq_kernel"
            name = "gated attention decode over q8k_tq3v cache, batch %d, ctx %d, 24Q/4KV hd256, wht %d" % (
                B, ctx, args.wht_len)
        else:
            kp, vp = ops.new_pool(n_pages, N_KV), ops.new_pool(n_pages, N_KV)
            kp.normal_(generator=gen)
            vp.normal_(generator=gen)
            per_tok = HD * 2 * 2
            call = lambda: ops.attn_decode(q, kp, vp, table, lens, gate, workspace=ws, out=out)
            kernel = "attn_decode_f16_kernel"
            name = "gated attention decode over F16 cache, batch %d, ctx %d, 24Q/4KV hd256" % (B, ctx)
        ws = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
        out = torch.empty_like(q)
        bytes_per_step = B * ctx * N_KV * per_tok + B * N_Q * HD * 4 * 3
        unit_per_step = B
    else:
        B = 1
        S = torch.randn(B, N_V, DK, DV, device="cuda", generator=gen) * 0.02
        cst = torch.zeros(B, CONV_DIM, CONV_K, device="cuda")
        w = torch.randn(CONV_DIM, CONV_K, device="cuda", generator=gen) * 0.5
        x = torch.randn(B, CONV_DIM, device="cuda", generator=gen)
        beta = torch.sigmoid(torch.randn(B, N_V, device="cuda", generator=gen))
        gl = -torch.nn.functional.softplus(torch.randn(B, N_V, device="cuda", generator=gen))
        od = torch.empty(B, N_V, DV, device="cuda")

        def call():
            mixed = ops.conv1d_update(x, w, cst)
            qk = mixed[:, :2 * N_K * DK].view(B, 2, N_K, DK)
            ops.delta_recurrent_step(S, qk[:, 0].contiguous(), qk[:, 1].contiguous(),
                                     mixed[:, 2 * N_K * DK:].reshape(B, N_V, DV).contiguous(), beta, gl, out=od)
        kernel = "delta_decode_kernel (+ conv1d_update4_kernel)"
        name = "gated DeltaNet decode step, batch 1, 16K/48V heads 128x128 FP32 state + conv k4 x 10240 (state stays in L2)"
        bytes_per_step = algorithmic_bytes(args, [1])["delta_rule"] + algorithmic_bytes(args, [1])["conv1d_update"]
        unit_per_step = 1
    for _ in range(max(3, args.warmup)):
        call()
    _lib.check_device()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if bytes_per_step < (512 << 20) else None
    sampler = ClockSampler(0)
    sampler.start()
    # Everything is enqueued without a host synchronisation in between, so the device never waits
    # for the host inside a timed interval (an untimed call goes first to get the host ahead).
    call()
    evs = []
    for _ in range(args.steps):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        call()
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    tot = sum(e0.elapsed_time(e1) for e0, e1 in evs)
    clocks = sampler.stop()
    _lib.check_device()
    ms = tot / args.steps
    achieved = bytes_per_step / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "hybrid-layer decode steps/sec", "value": unit_per_step / (ms * 1e-3), "unit": "seq-steps/s (one layer)",
        "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
        "dtype": "q8 K / tq3 V" if wl == "compact_decode" else ("f16 KV" if wl == "f16_decode" else "f32 state"),
        "config": {"workload": name, "l2": "256 MB buffer written between iterations" if flush is not None
                   else "inputs larger than L2", "timed": "operator call incl. its merge kernel"},
        "clocks": clocks, "gpu_launches": args.steps * 2,
        "roofline": {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "frac_of_8TBs_nominal": achieved / 8000.0,
                     "bytes_per_launch": bytes_per_step,
                     # dram read + write of one ncu capture at this workload's default size
                     # (profiles/attn_decode_tq_kernel.compact_decode.md); traffic grows with tokens
                     "traffic": int(1.007 * bytes_per_step) if wl == "compact_decode" else None}}), flush=True)


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload != "stack":
        run_operator(args)
        return
    import torch
    import torch.distributed as dist

    import __graft_entry__ as ge
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if local == 0:
        ge.build()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist.barrier()
    from rapidllm_b200 import _lib, ops
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
    if not _lib.lib().rl_b200_available():
        raise SystemExit("no sm_100 device: the CUDA path is the only path")

    heads_mode = args.shard == "heads" and world > 1
    split_mode = args.shard == "splitkv" and world > 1
    head_ways = 1
    attn_head_ways = 1
    pos_local = None
    if heads_mode:
        # head shards first (at most one KV head per rank), then sequence shards
        from rapidllm_b200.shard import plan_heads, plan_sequences
        head_ways = attn_head_ways = min(world, N_KV)
        hshard = plan_heads(rank % head_ways, head_ways)
        seqs = plan_sequences(rank // head_ways, world // head_ways, args.batch)
        ctx = [contexts(args, 0)[b] for b in seqs]
    elif split_mode:
        # every rank: a contiguous range of whole pages of each of the 32 sequences (the last rank
        # holds the tail and appends the new token) and 1/N of the DeltaNet heads
        if N_K % world:
            raise SystemExit("splitkv needs a world size that divides the %d DeltaNet key heads" % N_K)
        head_ways = world
        full = contexts(args, 0)
        ctx, pos_local = [], []
        from rapidllm_b200.shard import token_range_of_part
        for c in full:
            first, n_local = token_range_of_part(c, world, rank, PAGE)   # c counts the token being decoded
            ctx.append(max(1, n_local))
            pos_local.append(n_local - 1 if rank == world - 1 else n_local)
    else:
        ctx = contexts(args, rank)
    B = len(ctx)
    pages = [(c + PAGE - 1) // PAGE for c in ctx]
    max_pages = max(pages)
    n_pages = sum(pages)
    types = (QWEN35_LAYER_TYPES * ((args.layers + 3) // 4))[:args.layers]
    cache = HybridCache(types, n_pages=n_pages, n_slots=B, max_batch=B, max_pages_per_seq=max_pages,
                        max_seq_len=max(ctx), n_q=N_Q // attn_head_ways, n_kv=N_KV // attn_head_ways,
                        n_v=N_V // head_ways, n_k=N_K // head_ways)
    gen = torch.Generator(device="cuda").manual_seed(args.seed + 1000 * rank)
    for a in range(cache.n_attn):
        cache.k_pool(a).normal_(generator=gen)
        cache.v_pool(a).normal_(generator=gen)
    for d in range(cache.n_delta):
        cache.state(d).normal_(0.0, 0.02, generator=gen)
        cache.conv(d).normal_(generator=gen)
    cg = torch.Generator().manual_seed(args.seed + 1000 * rank)
    perm = torch.randperm(n_pages, generator=cg).int()
    table = torch.zeros(B, max_pages, dtype=torch.int32)
    at = 0
    for b, p in enumerate(pages):
        table[b, :p] = perm[at:at + p]
        at += p
    sh = cache.io_shapes(B)
    host = {}
    for n in ("attn_q", "attn_gate", "attn_k", "attn_v", "delta_qkv"):
        host[n] = torch.randn(sh[n], generator=cg).pin_memory()
    host["delta_beta"] = torch.sigmoid(torch.randn(sh["delta_beta"], generator=cg)).pin_memory()
    host["delta_g"] = (-torch.nn.functional.softplus(torch.randn(sh["delta_g"], generator=cg))).pin_memory()
    host["attn_o"] = torch.zeros(sh["attn_o"]).pin_memory()
    host["delta_o"] = torch.zeros(sh["delta_o"]).pin_memory()
    host["page_table"] = table.pin_memory()
    host["pos"] = torch.tensor(pos_local if split_mode else [c - 1 for c in ctx], dtype=torch.int32).pin_memory()
    conv_w = torch.randn(sh["conv_w"], generator=cg) * 0.5
    cache.set_conv_w(conv_w)
    dev = {n: x.cuda() for n, x in host.items()}
    dev["conv_w"] = conv_w.cuda()
    stream = torch.cuda.current_stream()

    gathered = None
    if heads_mode:
        gathered = (torch.empty((world,) + tuple(dev["attn_o"].shape), device="cuda"),
                    torch.empty((world,) + tuple(dev["delta_o"].shape), device="cuda"))
    if split_mode:
        dev["attn_ml"] = torch.zeros(sh["attn_ml"], device="cuda")
        dev["no_append"] = rank != world - 1
        gathered = (torch.empty((world,) + tuple(dev["attn_o"].shape), device="cuda"),
                    torch.empty((world,) + tuple(dev["delta_o"].shape), device="cuda"),
                    torch.empty((world,) + tuple(dev["attn_ml"].shape), device="cuda"))
        gate_rows = dev["attn_gate"].reshape(-1, HD)

    def exchange():
        # what a tensor-parallel model does with the mixer outputs: every rank gets every head slice
        if heads_mode:
            dist.all_gather_into_tensor(gathered[0], dev["attn_o"])
            dist.all_gather_into_tensor(gathered[1], dev["delta_o"])
        if split_mode:
            # partial (o, max, sum) of every rank's token range -> log-sum-exp merge + gate on every rank
            dist.all_gather_into_tensor(gathered[0], dev["attn_o"])
            dist.all_gather_into_tensor(gathered[2], dev["attn_ml"])
            dist.all_gather_into_tensor(gathered[1], dev["delta_o"])
            ops.lse_combine(gathered[0].view(world, -1, HD), gathered[2].view(world, -1, 2), gate_rows)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---------------- device-resident timing ----------------
    # Timed region: K steps back to back through rl_stack_decode (graph replay after the
    # second warm-up step), no host synchronisation between steps.
    if args.no_graph:
        cache.set_graph(False)
    sampler = ClockSampler(local)
    sampler.start()                              # the tool needs a moment to come up: start it before the warm-up
    for _ in range(max(3, args.warmup)):
        cache.decode(dev, B)
        exchange()
    _lib.check_device()
    sampler.mark()                               # may sleep: before the barrier, so that the ranks leave it together
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        cache.decode(dev, B)
        exchange()
    e1.record(stream)
    sync_all()
    ms = e0.elapsed_time(e1)
    _lib.check_device()
    # Second pass over the same K steps with CUDA events between the kernels (plain launches):
    # the per-kernel durations behind the roofline and the family shares.
    cache.set_timing(True)
    cache.decode(dev, B)
    sync_all()
    fam = {}
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record(stream)
    for _ in range(args.steps):
        cache.decode(dev, B)
        exchange()
        for k, v in cache.timing().items():      # waits for this step's last event
            fam[k] = fam.get(k, 0.0) + v
    e3.record(stream)
    sync_all()
    clocks = sampler.stop()
    ms_events = e2.elapsed_time(e3) / args.steps
    _lib.check_device()
    cache.set_timing(False)
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    ms_per_step = ms_max / args.steps
    total_seqs = args.batch if (heads_mode or split_mode) else B * world
    value = total_seqs / (ms_per_step * 1e-3)

    # ---------------- end to end through the host-buffer entry point ----------------
    e2e = None
    if not args.no_e2e and not heads_mode and not split_mode:
        for _ in range(2):
            cache.decode_host(host, B)
        sync_all()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            cache.decode_host(host, B)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        t = torch.tensor([dt], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
        h2d = sum(host[n].numel() * host[n].element_size() for n in
                  ("attn_q", "attn_gate", "attn_k", "attn_v", "delta_qkv", "delta_beta", "delta_g",
                   "page_table", "pos"))
        d2h = sum(host[n].numel() * host[n].element_size() for n in ("attn_o", "delta_o"))
        e2e = {"value": B * world / (dt / args.steps), "unit": "seq-steps/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": dt / args.steps * 1e3}
        _lib.check_device()

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        ab = algorithmic_bytes(args, ctx)
        if heads_mode:
            ab = {k: v / head_ways for k, v in ab.items()}
        if split_mode:
            ab["delta_rule"] /= world
            ab["conv1d_update"] /= world
            ab["step"] = ab["attn_decode"] * cache.n_attn + (ab["delta_rule"] + ab["conv1d_update"]) * cache.n_delta
        n_attn = cache.n_attn
        attn_ms_per_launch = fam["attn_decode"] / args.steps / max(1, n_attn)
        achieved = ab["attn_decode"] / (attn_ms_per_launch * 1e-3) / 1e9
        families = {}
        for k, nl in (("attn_decode", n_attn), ("attn_combine", n_attn), ("kv_append", n_attn),
                      ("delta_rule", cache.n_delta), ("conv1d_update", cache.n_delta)):
            per = fam[k] / args.steps / max(1, nl)
            families[k] = {"ms_per_launch": round(per, 5), "share": round(fam[k] / args.steps / ms_events, 4)}
            if k in ab:
                families[k]["gbs"] = round(ab[k] / (per * 1e-3) / 1e9, 1) if per > 0 else None
        line = {
            "metric": "hybrid-layer decode steps/sec", "value": value, "unit": "seq-steps/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong" if (heads_mode or split_mode) else "weak", "vs_baseline": None,
            "dtype": "f16 KV / f32 state", "data": "synthetic",
            "config": {"workload": workload_name(args), "l2": "inputs larger than L2 (%.1f GB streamed per step)"
                       % (ab["step"] / 1e9),
                       "parallelism": ("heads x%d then sequences x%d, NCCL all_gather of head outputs"
                                       % (head_ways, world // head_ways)) if heads_mode
                       else ("split-KV x%d (token ranges of every sequence) + DeltaNet heads x%d, NCCL all_gather of "
                             "attention partials merged by rl_lse_combine" % (world, world)) if split_mode
                       else "sequence-sharded x%d, no collective" % world,
                       "ctx_tokens_rank0": sum(ctx), "cache_bytes_rank0": cache.bytes},
            "clocks": clocks,
            "gpu_launches": (cache.launches_per_step + (1 if split_mode else 0)) * args.steps,
            "step_hbm_gbs": ab["step"] * world / (ms_per_step * 1e-3) / 1e9,   # rank 0's bytes x ranks
            "roofline": {"bound": "hbm", "kernel": "attn_decode_f16_kernel", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "frac_of_8TBs_nominal": achieved / 8000.0,
                         "peak_source": "MEASURED_PEAKS.json hbm_gbs (of measured)" if peaks else "fallback 6650 (of fallback)",
                         "bytes_per_launch": ab["attn_decode"], "ms_per_launch": attn_ms_per_launch,
                         # ncu dram read+write of a batch-8 capture was 1.0246 x its algorithmic bytes
                         # (profiles/attn_decode_f16_kernel.stack_decode.md); traffic grows with tokens
                         "traffic": int(1.0246 * ab["attn_decode"]),
                         "traffic_source": "ncu capture of a batch-8 launch scaled by algorithmic bytes"},
            "kernel_families": families,
            "kernel_timing_pass": {"ms_per_step": ms_events, "note": "same K steps repeated as plain launches "
                                   "with CUDA events between the kernels; roofline and shares come from this pass"},
            "graph_replay": not args.no_graph,
        }
        if e2e:
            line["e2e"] = e2e
        if world == 1 and not args.no_cpu_baseline:
            cb = cpu_reference_leg(args, ctx)
            line["cpu_baseline"] = cb
        print(json.dumps(line), flush=True)
    cache.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
