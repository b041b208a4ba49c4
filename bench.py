#!/usr/bin/env python
"""Benchmark of the hybrid-attention hot path on B200.

Headline workload (the "full 64-layer hybrid stack decode" configuration): 64 layers in
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

N = 1 also times the single-operator configurations (F16 decode at ctx 4096 and 4 x 131072,
one DeltaNet step, compact-KV decode at 4 x 131072 in both V layouts, attention prefill of 8192
tokens in one chunk and in chunks of 1024, the chunked DeltaNet prefill, the chunked prefill of
the whole stack) and attaches them to the line under "operators", each with its own roofline
and clock record (--no-operators skips them; --workload NAME prints one of them alone).

N > 1 (under torchrun, one rank per GPU): ONE batch of 32 is divided over the ranks (strong
scaling): KV heads and DeltaNet value heads 2- or 4-way, at N = 8 also the sequences 2-way
(--shard heads), or token ranges of every sequence plus DeltaNet heads (--shard splitkv).  The
per-layer outputs are all-gathered by the library (rl_stack_set_gather: NCCL on a side stream,
beside the following layers).  Before timing, rank 0 checks the gathered outputs of the first
attention and the first DeltaNet layer for two sequences against the unsharded operators on the
same inputs; a mismatch ends the run with a non-zero exit.  --shard seq gives every rank a whole
batch of its own (weak scaling, same contexts on every rank, no collective).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
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
# tolerances of the sharded-step check (those of the tests: fp16-KV attention / FP32 DeltaNet)
ATTN_MAX_ABS, ATTN_REL_L2, DELTA_MAX_ABS = 2e-2, 1e-3, 1e-4
OPERATORS = ["f16_decode", "f16_decode_long", "delta_step", "compact_decode", "compact_decode_wht256",
             "attn_prefill", "attn_prefill_chunk1024", "delta_prefill", "stack_prefill", "stack_prefill_chunk4096", "stack_long_compact", "stack_long_f16"]


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--ctx-min", type=int, default=8192)
    ap.add_argument("--ctx-max", type=int, default=32768)
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--seed", type=int, default=4)
    ap.add_argument("--workload", default="stack", choices=["stack"] + OPERATORS,
                    help="stack = the headline workload (with the operator lines attached at N = 1); an operator "
                         "name prints that operator's line alone (N = 1)")
    ap.add_argument("--shard", default="auto", choices=["auto", "seq", "heads", "splitkv"],
                    help="N > 1: auto = heads; heads = ONE batch of 32 divided by KV / value heads (up to 4 ways) and "
                         "then by sequence; splitkv = ONE batch of 32, every rank holds 1/N of each sequence's KV "
                         "pages and 1/N of the DeltaNet heads, attention partials merged by log-sum-exp; "
                         "seq = every rank owns a whole batch of 32 (weak scaling, no collective)")
    ap.add_argument("--layers-per-exchange", type=int, default=0,
                    help="N > 1: layers whose outputs one grouped all-gather carries (0 = 4)")
    ap.add_argument("--reserve-sms", type=int, default=0,
                    help="N > 1: SMs the step's persistent kernels leave to the exchange kernels")
    ap.add_argument("--op-seconds", type=float, default=1.0, help="least length of an operator's timed region")
    ap.add_argument("--op-batch", type=int, default=0, help="--workload NAME: override the batch")
    ap.add_argument("--op-ctx", type=int, default=0, help="--workload NAME: override the context / token count")
    ap.add_argument("--chunk", type=int, default=None, help="--workload NAME: query rows per prefill call")
    ap.add_argument("--emulate-ranks", type=int, default=0,
                    help="N = 1 only: time rank 0's share of a step divided over this many ranks (--shard heads or "
                         "splitkv), without the exchange: the per-rank kernel time of a multi-GPU run on one GPU")
    ap.add_argument("--no-operators", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="N > 1: skip the sharded-step check")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="plain launches instead of graph replay in the timed region")
    return ap.parse_args()


def contexts(args):
    import torch
    g = torch.Generator().manual_seed(args.seed)
    return torch.randint(args.ctx_min, args.ctx_max + 1, (args.batch,), generator=g).tolist()


def workload_name(args):
    return ("hybrid_stack_decode: %d layers (3 DeltaNet + 1 GatedAttn), batch %d, ragged ctx U[%d,%d], "
            "paged F16 KV page 64" % (args.layers, args.batch, args.ctx_min, args.ctx_max))


def algorithmic_bytes(n_layers, ctx, n_q=N_Q, n_kv=N_KV, n_v=N_V, n_k=N_K):
    """Bytes one step must move, per kernel family (per layer-launch, and per step)."""
    B = len(ctx)
    n_attn = n_layers // 4
    n_delta = n_layers - n_attn
    conv_dim = 2 * n_k * DK + n_v * DV
    attn_launch = sum(ctx) * n_kv * HD * 2 * 2 + B * n_q * HD * 4 * 3
    # fused DeltaNet step: state read + write, the conv rings (three older taps read, one tap written per
    # channel), the channels' inputs and taps' weights, beta, g, o
    conv_launch = B * conv_dim * (3 * 4 + 4 + 4) + conv_dim * CONV_K * 4
    delta_launch = B * (2 * n_v * DK * DV * 4 + n_v * DV * 4 + n_v * 8) + conv_launch
    append_launch = B * n_kv * HD * (4 + 2) * 2
    return {"attn_decode": attn_launch, "delta_rule": delta_launch, "conv_part_of_delta_rule": conv_launch,
            "kv_append": append_launch,
            "step": n_attn * (attn_launch + append_launch) + n_delta * delta_launch}


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        return {}


# --------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi (query only) every 50 ms for the whole run; a timed region reports the samples
    between the cursor() it took before and the one after."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

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
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def cursor(self, wait_s=3.0):
        """Index of the next sample; the first call waits (bounded) for the tool to come up."""
        t0 = time.time()
        while self.proc and not self.lines and time.time() - t0 < wait_s:
            time.sleep(0.02)
        return len(self.lines)

    def window(self, first, last=None):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines[first:last]:
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

    def stop(self):
        if not self.proc:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)


# --------------------------------------------------------------------------------------
def cpu_reference_leg(args, ctx, seconds_budget=12.0):
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


def shard_mode(args, world):
    if world <= 1:
        return "single"
    return "heads" if args.shard == "auto" else args.shard


def run_reference(args):
    """The reference arm: the reference's own CPU operators on this box's host cores, on the same
    workload.  The CPU path is single-process: with N ranks sharing one batch the job is still that
    one batch (value does not grow with N); in --shard seq every rank owns a batch of its own."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ctx = contexts(args)
    steps = []
    for _ in range(max(0, args.warmup)):
        cpu_reference_leg(args, ctx, seconds_budget=2.0)
    base = None
    for _ in range(max(1, args.steps)):
        base = cpu_reference_leg(args, ctx, seconds_budget=max(2.0, 60.0 / max(1, args.steps)))
        steps.append(base["step_seconds"])
    step_s = sum(steps) / len(steps)
    weak = shard_mode(args, args.gpus) == "seq"
    value = len(ctx) * (args.gpus if weak else 1) / step_s
    line = {"impl": "reference", "metric": "hybrid-layer decode steps/sec", "value": value,
            "unit": "seq-steps/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak" if weak or args.gpus == 1 else "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(args), "l2": "inputs larger than L2",
                       "note": "reference CPU operators on host cores; each step is a bounded sample scaled to the "
                               "whole step"},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": value, "unit": "seq-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    line["cpu_baseline"]["value"] = value
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# Single-operator workloads.  Each returns one entry: ms per call, the operator's own metric, its
# roofline (achieved = algorithmic bytes or flops / CUDA-event time) and the clock record of its
# timed region.  The timed region is at least --op-seconds long so that it holds >= 10 clock samples.
def _timed(call, sampler, seconds, warmup, graph_calls=0):
    """Warm up, then time back-to-back calls for >= `seconds` with two CUDA events.  graph_calls > 0:
    `call` is captured once per that many invocations into a CUDA graph that is replayed (short
    operators: keeps the device busy back to back, as a serving loop would)."""
    import torch
    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    per = 1
    run = call
    if graph_calls:
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(graph_calls):                 # on the side stream once, outside capture
                call()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=side):
            for _ in range(graph_calls):
                call()
        per, run = graph_calls, g.replay
        run()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run()
    e1.record()
    torch.cuda.synchronize()
    est = max(e0.elapsed_time(e1), 1e-3)
    reps = max(3, min(200000, int(math.ceil(seconds * 1e3 / est))))
    c0 = sampler.cursor()
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    c1 = sampler.cursor()
    return e0.elapsed_time(e1) / (reps * per), reps * per, sampler.window(c0, c1)


def _hbm_roofline(kernel, bytes_per_launch, ms, peaks, traffic=None, traffic_source=None):
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = bytes_per_launch / (ms * 1e-3) / 1e9
    r = {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak, "unit": "GB/s",
         "frac": achieved / peak, "frac_of_8TBs_nominal": achieved / 8000.0,
         "peak_source": "MEASURED_PEAKS.json hbm_gbs (of measured)" if peaks else "fallback 6650 (of fallback)",
         "bytes_per_launch": bytes_per_launch, "traffic": traffic}
    if traffic_source:
        r["traffic_source"] = traffic_source
    return r


def _tensor_roofline(kernel, flops, ms, peaks, note=None):
    tpeak = float(peaks.get("bf16_tflops", 1590.0))
    speak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    achieved = flops / (ms * 1e-3) / 1e12
    r = {"bound": "tensor", "kernel": kernel, "achieved": achieved, "peak": tpeak, "unit": "TFLOP/s",
         "frac": achieved / tpeak, "peak_sustained": speak, "frac_of_sustained_peak": achieved / speak,
         "peak_source": "MEASURED_PEAKS.json bf16_tflops (burst) / bf16_tflops_sustained (of measured)" if peaks
         else "fallback 1590 / 1400 (of fallback)",
         "flops_per_launch": flops, "traffic": None}
    if note:
        r["note"] = note
    return r


def op_decode(name, args, sampler, peaks, gen):
    """Decode attention of one layer: F16 cache (batch 1 x ctx 4096 = the single-layer CPU
    configuration; batch 4 x 131072) or the compact q8-K / TQ3-V cache (batch 4 x 131072)."""
    import torch

    from rapidllm_b200 import _lib, ops
    compact = name.startswith("compact")
    wht = 256 if name.endswith("wht256") else 128
    B, ctx = (1, 4096) if name == "f16_decode" else (4, 131072)
    B, ctx = args.op_batch or B, args.op_ctx or ctx
    pages = (ctx + PAGE - 1) // PAGE
    per_tok = (_lib.lib().rl_kv_compact_page_bytes() // PAGE) if compact else HD * 2 * 2
    bytes_per_launch = B * ctx * N_KV * per_tok + B * N_Q * HD * 4 * 3
    # short calls rotate over enough independent input sets to exceed L2
    n_sets = max(1, min(64, int(math.ceil(300e6 / bytes_per_launch)))) if bytes_per_launch < 300e6 else 1
    cg = torch.Generator().manual_seed(args.seed)
    sets = []
    signs = None
    if compact and wht == 256:
        signs = 2.0 * torch.bernoulli(torch.full((256,), 0.5, device="cuda"), generator=gen) - 1.0
    lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    for _ in range(n_sets):
        n_pages = B * pages
        table = torch.randperm(n_pages, generator=cg).int().reshape(B, pages).cuda()
        q = torch.randn(B, N_Q, HD, device="cuda", generator=gen)
        gate = torch.randn(B, N_Q, HD, device="cuda", generator=gen)
        if compact:
            pool = ops.new_compact_pool(n_pages, N_KV)
            step = 8192
            for b in range(B):
                for t0 in range(0, ctx, step):
                    n = min(step, ctx - t0)
                    k = torch.randn(n, N_KV, HD, device="cuda", generator=gen)
                    v = torch.randn(n, N_KV, HD, device="cuda", generator=gen)
                    ops.kv_compact_append(pool, table[b], k, v, wht, signs, pos0=t0)
            sets.append((q, gate, pool, None, table))
        else:
            kp, vp = ops.new_pool(n_pages, N_KV), ops.new_pool(n_pages, N_KV)
            kp.normal_(generator=gen)
            vp.normal_(generator=gen)
            sets.append((q, gate, kp, vp, table))
    ws = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
    out = torch.empty(B, N_Q, HD, device="cuda")
    state = {"i": 0}

    def call():
        q, gate, kp, vp, table = sets[state["i"] % n_sets]
        state["i"] += 1
        ops.attn_decode(q, kp, vp, table, lens, gate, wht_len=wht, signs=signs, workspace=ws, out=out)
    ms, calls, clocks = _timed(call, sampler, args.op_seconds, max(3, args.warmup), graph_calls=n_sets if n_sets > 1 else 8)
    _lib.check_device()
    kernel = "attn_decode_tq_kernel" if compact else "attn_decode_f16_kernel"
    traffic = int(1.007 * bytes_per_launch) if compact else int(1.0246 * bytes_per_launch)
    return {
        "workload": "gated attention decode over the %s cache, batch %d, ctx %d, 24Q/4KV hd256%s" % (
            "q8k_tq3v" if compact else "F16", B, ctx, (", V transform length %d" % wht) if compact else ""),
        "ms": ms, "value": B / (ms * 1e-3), "unit": "seq-steps/s (one layer)", "calls_timed": calls,
        "dtype": "q8 K / tq3 V" if compact else "f16 KV", "gpu_launches_per_call": 2,
        "l2": ("rotates over %d independent input sets, %.0f MB in all" % (n_sets, n_sets * bytes_per_launch / 1e6))
        if n_sets > 1 else "inputs larger than L2",
        "timed": "operator call incl. its merge kernel, CUDA-graph replay back to back",
        "roofline": _hbm_roofline(kernel + " (+ merge)", bytes_per_launch, ms, peaks, traffic,
                                  "ncu dram read+write of a smaller capture of this kernel scaled by algorithmic bytes"),
        "clocks": clocks}


def op_delta_step(args, sampler, peaks, gen):
    """One Gated DeltaNet decode step of one layer, batch 1: conv window + l2 norms + delta rule (one kernel)."""
    import torch

    from rapidllm_b200 import _lib
    B = args.op_batch or 1
    bytes_per_launch = algorithmic_bytes(4, [1] * B)["delta_rule"]
    n_sets = max(1, min(96, int(math.ceil(300e6 / bytes_per_launch))))
    sets = []
    for _ in range(n_sets):
        S = torch.randn(B, N_V, DK, DV, device="cuda", generator=gen) * 0.02
        ring = torch.zeros(B, CONV_DIM, CONV_K, device="cuda")
        phase = torch.zeros(B, dtype=torch.int32, device="cuda")
        x = torch.randn(B, CONV_DIM, device="cuda", generator=gen)
        sets.append((S, ring, phase, x))
    w = torch.randn(CONV_DIM, CONV_K, device="cuda", generator=gen) * 0.5
    beta = torch.sigmoid(torch.randn(B, N_V, device="cuda", generator=gen))
    gl = -torch.nn.functional.softplus(torch.randn(B, N_V, device="cuda", generator=gen))
    od = torch.empty(B, N_V, DV, device="cuda")
    p = _lib.GdnDecodeParams(n_v=N_V, n_qk=N_K, dk=DK, dv=DV, conv_k=CONV_K, batch=B, n_slots=B,
                             head_map=_lib.RL_HEADS_GROUPED, eps_l2=1e-6)
    state = {"i": 0}
    L = _lib.lib()
    vp = ctypes.c_void_p

    def call():
        S, ring, phase, x = sets[state["i"] % n_sets]
        state["i"] += 1
        st = vp(torch.cuda.current_stream().cuda_stream)
        _lib.check(L.rl_gdn_decode(vp(S.data_ptr()), vp(ring.data_ptr()), vp(phase.data_ptr()), None, vp(x.data_ptr()),
                                   vp(w.data_ptr()), vp(beta.data_ptr()), vp(gl.data_ptr()), vp(od.data_ptr()),
                                   ctypes.byref(p), st))
        _lib.check(L.rl_gdn_phase_advance(vp(phase.data_ptr()), None, 1, B, B, 1, st))
    ms, calls, clocks = _timed(call, sampler, args.op_seconds, max(3, args.warmup), graph_calls=n_sets)
    _lib.check_device()
    return {
        "workload": "gated DeltaNet decode step, batch %d, 16K/48V heads 128x128 FP32 state + conv k4 x 10240" % B,
        "ms": ms, "value": B / (ms * 1e-3), "unit": "seq-steps/s (one layer)", "calls_timed": calls,
        "dtype": "f32 state", "gpu_launches_per_call": 2,
        "l2": "rotates over %d independent states, %.0f MB in all" % (n_sets, n_sets * bytes_per_launch / 1e6),
        "timed": "fused conv + delta rule kernel and the ring-phase kernel, CUDA-graph replay back to back",
        "roofline": _hbm_roofline("gdn_decode_kernel", bytes_per_launch, ms, peaks),
        "clocks": clocks}


def op_attn_prefill(name, args, sampler, peaks, gen):
    """Causal attention prefill of T tokens of one layer in chunks (tcgen05 / TMEM), writes F16 KV."""
    import torch

    from rapidllm_b200 import _lib, ops
    T = args.op_ctx or 8192
    chunk = args.chunk or (1024 if name.endswith("1024") else T)
    n_pages = (T + PAGE - 1) // PAGE
    cg = torch.Generator().manual_seed(args.seed)
    table = torch.randperm(n_pages, generator=cg).int().cuda()
    q = torch.randn(T, N_Q, HD, device="cuda", generator=gen).bfloat16()
    k = torch.randn(T, N_KV, HD, device="cuda", generator=gen).bfloat16()
    v = torch.randn(T, N_KV, HD, device="cuda", generator=gen).bfloat16()
    gate = torch.randn(T, N_Q, HD, device="cuda", generator=gen)
    kp, vp = ops.new_pool(n_pages, N_KV), ops.new_pool(n_pages, N_KV)

    def call():
        for p0 in range(0, T, chunk):
            sl = slice(p0, min(T, p0 + chunk))
            ops.attn_prefill(q[sl], kp, vp, table, p0, k[sl], v[sl], gate[sl])
    ms, calls, clocks = _timed(call, sampler, args.op_seconds, max(3, args.warmup))
    _lib.check_device()
    flops = 4.0 * N_Q * HD * T * (T + 1) / 2
    return {
        "workload": "gated attention chunked prefill, T %d in chunks of %d, 24Q/4KV hd256, causal, writes F16 KV" % (T, chunk),
        "ms": ms, "value": T / (ms * 1e-3), "unit": "tokens/s (one layer)", "calls_timed": calls,
        "dtype": "f16 (bf16 in)", "gpu_launches_per_call": 2 * ((T + chunk - 1) // chunk),
        "l2": "K/V of one layer (32 MB) fit L2 by design; q/gate/o (%.0f MB) are streamed" % (T * N_Q * HD * 10 / 1e6),
        "timed": "KV append + prefill kernel of every chunk, back to back (power-capped clocks)",
        "roofline": _tensor_roofline("attn_prefill_kernel", flops, ms, peaks,
                                     "flops = 4 n_q hd T (T + 1) / 2 (the masked half is not counted)"),
        "clocks": clocks}


def op_delta_prefill(args, sampler, peaks, gen):
    """Chunked (WY form, chunk 64) Gated DeltaNet prefill of T tokens of one layer."""
    import torch

    from rapidllm_b200 import _lib, ops
    T = args.op_ctx or 8192
    S = torch.zeros(N_V, DK, DV, device="cuda")
    q = torch.randn(T, N_K, DK, device="cuda", generator=gen)
    k = torch.randn(T, N_K, DK, device="cuda", generator=gen)
    v = torch.randn(T, N_V, DV, device="cuda", generator=gen)
    beta = torch.sigmoid(torch.randn(T, N_V, device="cuda", generator=gen))
    gl = -torch.nn.functional.softplus(torch.randn(T, N_V, device="cuda", generator=gen))
    ws = torch.empty(_lib.lib().rl_delta_chunk_workspace_bytes(
        ctypes.byref(_lib.DeltaChunkParams(n_v=N_V, dk=DK, dv=DV, seq=T, chunk=64, eps_l2=1e-6,
                                           n_qk=N_K, head_map=1))), dtype=torch.uint8, device="cuda")

    def call():
        S.zero_()
        ops.delta_chunk_prefill(S, q, k, v, beta, gl, workspace=ws)
    ms, calls, clocks = _timed(call, sampler, args.op_seconds, max(3, args.warmup))
    _lib.check_device()
    n_chunks = (T + 63) // 64
    mma = _lib.lib().rl_delta_chunk_mma_flops()
    flops = float(n_chunks) * N_V * mma
    return {
        "workload": "gated DeltaNet chunked (WY, chunk 64) prefill, T %d, batch 1, 16K/48V heads 128x128" % T,
        "ms": ms, "value": T / (ms * 1e-3), "unit": "tokens/s (one layer)", "calls_timed": calls,
        "dtype": "f16 hi+lo operands / f32 state", "gpu_launches_per_call": 1 + 2 * (1 if n_chunks < 32 else (2 if n_chunks < 64 else (3 if n_chunks < 128 else 4))),
        "l2": "operands streamed once (%.2f GB workspace)" % (ws.numel() / 1e9),
        "timed": "keys + prepare + scan kernels of one call, back to back",
        "roofline": _tensor_roofline("delta_chunk_scan_kernel + delta_chunk_prepare_kernel", flops, ms, peaks,
                                     "flops = tensor-core MMAs the scan kernel issues per (chunk, value head) x chunks x "
                                     "heads; the chunk-to-chunk dependency, not tensor throughput, bounds the operator"),
        "clocks": clocks}


def op_stack_prefill(args, sampler, peaks, gen, chunk=1024):
    """A prompt of T tokens through the mixers of all 64 layers in chunks of 1024 (the reference's chunk cap) or of
    4096 (what the memory of this part allows: fewer, longer calls of every kernel)."""
    import torch

    from rapidllm_b200 import _lib
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
    T = args.op_ctx or 8192
    chunk = min(args.chunk or chunk, T)
    types = (QWEN35_LAYER_TYPES * ((args.layers + 3) // 4))[:args.layers]
    pages = (T + PAGE - 1) // PAGE
    cache = HybridCache(types, n_pages=pages, n_slots=1, max_batch=1, max_pages_per_seq=pages)
    cg = torch.Generator().manual_seed(args.seed)
    row = torch.randperm(pages, generator=cg).int().cuda()
    t = {}
    for nm, (shape, dtype) in cache.prefill_shapes(chunk).items():
        if nm in ("attn_o", "delta_o"):
            t[nm] = torch.empty(shape, dtype=dtype, device="cuda")
        elif nm == "delta_beta":
            t[nm] = torch.sigmoid(torch.randn(shape, device="cuda", generator=gen))
        elif nm == "delta_g":
            t[nm] = -torch.nn.functional.softplus(torch.randn(shape, device="cuda", generator=gen))
        else:
            t[nm] = (torch.randn(shape, device="cuda", generator=gen) * (0.5 if nm == "conv_w" else 1.0)).to(dtype)
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
    ms, calls, clocks = _timed(call, sampler, args.op_seconds, max(3, args.warmup))
    _lib.check_device()
    flops_attn = cache.n_attn * 4.0 * N_Q * HD * T * (T + 1) / 2
    entry = {
        "workload": "chunked prefill, %d layers (%d attention + %d DeltaNet), one sequence of %d tokens in chunks of %d, "
                    "mixers only (no projections / MLP)" % (len(types), cache.n_attn, cache.n_delta, T, chunk),
        "ms": ms, "value": T / (ms * 1e-3), "unit": "tokens/s", "calls_timed": calls,
        "dtype": "f16 attention (bf16 in) / f16 hi+lo + f32 state DeltaNet",
        # attention: append + prefill (+ the merge of the divided last wave from the second chunk on);
        # DeltaNet: conv, keys, prepare, scan
        "gpu_launches_per_call": n_chunks * (cache.n_attn * 2 + cache.n_delta * 4) + (n_chunks - 1) * cache.n_attn,
        "l2": "per-chunk inputs of all layers (%.1f GB) exceed L2" % (sum(x.numel() * x.element_size() for x in t.values()) / 1e9),
        "timed": "rl_stack_prefill of every chunk, back to back",
        "roofline": _tensor_roofline("attn_prefill_kernel (attention layers' flops only)", flops_attn, ms, peaks,
                                     "whole-stack time in the denominator; the DeltaNet layers take most of it"),
        "clocks": clocks}
    cache.close()
    return entry


def op_stack_long(args, sampler, peaks, gen, compact=True):
    """The 64-layer stack decode at the metric's context range, ragged ctx U[32768, 131072]: batch 32 on the
    compact cache (q8-K / TQ3-V pages inside rl_cache, every sequence past the F16 window), or batch 8 on the
    F16 cache (the batch whose 43 GB of pages fit beside the rest)."""
    import torch

    from rapidllm_b200 import _lib, ops
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
    B = args.op_batch or (32 if compact else 8)
    lo, hi = 32768, args.op_ctx or 131072
    cg = torch.Generator().manual_seed(args.seed)
    ctx = torch.randint(lo, hi + 1, (B,), generator=cg).tolist()
    pages = [(c + PAGE - 1) // PAGE for c in ctx]
    max_pages, n_pages = max(pages), sum(pages)
    types = (QWEN35_LAYER_TYPES * ((args.layers + 3) // 4))[:args.layers]
    window = 8192
    if compact:
        cache = HybridCache(types, n_pages=n_pages, n_slots=B, max_batch=B, max_pages_per_seq=max_pages, max_seq_len=max(ctx),
                            kv_dtype=_lib.RL_KV_Q8K_TQ3V, wht_len=128, window_tokens=window)
    else:
        cache = HybridCache(types, n_pages=n_pages, n_slots=B, max_batch=B, max_pages_per_seq=max_pages, max_seq_len=max(ctx))
    perm = torch.randperm(n_pages, generator=cg).int()
    table = torch.zeros(B, max_pages, dtype=torch.int32)
    at = 0
    for b, p in enumerate(pages):
        table[b, :p] = perm[at:at + p]
        at += p
    table_d = table.cuda()
    if compact:
        # layer 0's pages are quantised from N(0,1) rows, the other layers get a copy (same page table)
        p0 = cache.k_pool(0)
        step = 8192
        for b in range(B):
            for t0 in range(0, ctx[b] - 1, step):
                n = min(step, ctx[b] - 1 - t0)
                k = torch.randn(n, N_KV, HD, device="cuda", generator=gen)
                v = torch.randn(n, N_KV, HD, device="cuda", generator=gen)
                ops.kv_compact_append(p0, table_d[b], k, v, 128, None, pos0=t0)
        for a in range(1, cache.n_attn):
            cache.k_pool(a).copy_(p0)
    else:
        for a in range(cache.n_attn):
            cache.k_pool(a).normal_(generator=gen)
            cache.v_pool(a).normal_(generator=gen)
    for d in range(cache.n_delta):
        cache.state(d).normal_(0.0, 0.02, generator=gen)
        cache.conv(d).normal_(generator=gen)
    sh = cache.io_shapes(B)
    dev = {n: torch.randn(sh[n], device="cuda", generator=gen) for n in ("attn_q", "attn_gate", "attn_k", "attn_v", "delta_qkv")}
    dev["delta_beta"] = torch.sigmoid(torch.randn(sh["delta_beta"], device="cuda", generator=gen))
    dev["delta_g"] = -torch.nn.functional.softplus(torch.randn(sh["delta_g"], device="cuda", generator=gen))
    dev["conv_w"] = torch.randn(sh["conv_w"], device="cuda", generator=gen) * 0.5
    dev["attn_o"], dev["delta_o"] = torch.zeros(sh["attn_o"], device="cuda"), torch.zeros(sh["delta_o"], device="cuda")
    dev["page_table"] = table_d
    dev["pos"] = torch.tensor([c - 1 for c in ctx], dtype=torch.int32, device="cuda")
    dev["kv_window_ok"] = False

    def call():
        cache.decode(dev, B)
    ms, calls, clocks = _timed(call, sampler, args.op_seconds, max(3, args.warmup))
    _lib.check_device()
    finite = bool(torch.isfinite(dev["attn_o"]).all() and torch.isfinite(dev["delta_o"]).all())
    per_tok = (_lib.lib().rl_kv_compact_page_bytes() // PAGE) if compact else HD * 2 * 2
    ab = algorithmic_bytes(args.layers, ctx)
    attn_bytes = sum(ctx) * N_KV * per_tok + B * N_Q * HD * 4 * 3
    step_bytes = cache.n_attn * (attn_bytes + ab["kv_append"]) + cache.n_delta * ab["delta_rule"]
    entry = {
        "workload": ("hybrid_stack_decode on the compact cache: %d layers, batch %d, ragged ctx U[%d,%d], q8-K / TQ3-V pages "
                     "(358 B per token and head) + F16 window of %d tokens, page 64" % (len(types), B, lo, hi, window))
        if compact else ("hybrid_stack_decode: %d layers, batch %d, ragged ctx U[%d,%d], paged F16 KV page 64"
                         % (len(types), B, lo, hi)),
        "ms": ms, "value": B / (ms * 1e-3), "unit": "seq-steps/s", "calls_timed": calls,
        "dtype": "q8 K / tq3 V / f32 state" if compact else "f16 KV / f32 state", "gpu_launches_per_call": cache.launches_per_step,
        "l2": "inputs larger than L2 (%.1f GB streamed per step)" % (step_bytes / 1e9),
        "timed": "rl_stack_decode (graph replay), back to back", "outputs_finite": finite,
        "ctx_tokens": sum(ctx), "cache_bytes": cache.bytes,
        "roofline": _hbm_roofline("whole step (%s dominates)" % ("attn_decode_tq_kernel" if compact else "attn_decode_f16_kernel"),
                                  step_bytes, ms, peaks),
        "clocks": clocks}
    cache.close()
    return entry


def run_one_operator(name, args, sampler, peaks):
    import torch
    gen = torch.Generator(device="cuda").manual_seed(args.seed)
    if name in ("f16_decode", "f16_decode_long", "compact_decode", "compact_decode_wht256"):
        return op_decode(name, args, sampler, peaks, gen)
    if name == "delta_step":
        return op_delta_step(args, sampler, peaks, gen)
    if name in ("attn_prefill", "attn_prefill_chunk1024"):
        return op_attn_prefill(name, args, sampler, peaks, gen)
    if name == "delta_prefill":
        return op_delta_prefill(args, sampler, peaks, gen)
    if name in ("stack_prefill", "stack_prefill_chunk4096"):
        return op_stack_prefill(args, sampler, peaks, gen, chunk=4096 if name.endswith("4096") else 1024)
    if name in ("stack_long_compact", "stack_long_f16"):
        return op_stack_long(args, sampler, peaks, gen, compact=name == "stack_long_compact")
    raise SystemExit("unknown operator %s" % name)


def run_operators(args, sampler, peaks):
    import torch
    out = {}
    for name in OPERATORS:
        t0 = time.time()
        try:
            out[name] = run_one_operator(name, args, sampler, peaks)
            out[name]["wall_s"] = round(time.time() - t0, 1)
        except Exception as e:                       # one operator failing must not lose the headline
            out[name] = {"error": "%s: %s" % (type(e).__name__, e)}
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
    return out


def operator_line(name, args):
    """--workload NAME: that operator alone as a line of its own."""
    import torch

    import __graft_entry__ as ge
    ge.build()
    torch.cuda.set_device(0)
    peaks = load_peaks()
    sampler = ClockSampler(0).start()
    e = run_one_operator(name, args, sampler, peaks)
    sampler.stop()
    print(json.dumps({
        "metric": "hybrid-layer decode steps/sec" if "decode" in name or name == "delta_step" else "prefill tokens/sec",
        "value": e["value"], "unit": e["unit"], "n_gpus": 1, "steps": e["calls_timed"], "warmup": max(3, args.warmup),
        "ms_per_step": e["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
        "dtype": e["dtype"], "config": {"workload": e["workload"], "l2": e["l2"], "timed": e["timed"]},
        "clocks": e["clocks"], "gpu_launches": e["calls_timed"] * e["gpu_launches_per_call"],
        "roofline": e["roofline"]}), flush=True)


# --------------------------------------------------------------------------------------
def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload != "stack":
        operator_line(args.workload, args)
        return
    import numpy as np
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
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, Comm, HybridCache
    from rapidllm_b200.shard import StepPlan
    if not _lib.lib().rl_b200_available():
        raise SystemExit("no sm_100 device: the CUDA path is the only path")
    sampler = ClockSampler(local).start()           # the tool needs a moment to come up: start it first
    peaks = load_peaks()

    mode = shard_mode(args, world)
    strong = mode in ("heads", "splitkv")
    plan = StepPlan(mode if world > 1 else "seq", rank if strong else 0, world if strong else 1, args.batch)
    emulated = world == 1 and args.emulate_ranks > 1
    if emulated:
        plan = StepPlan("heads" if args.shard == "auto" else args.shard, 0, args.emulate_ranks, args.batch)
    split_mode = mode == "splitkv" or (emulated and plan.mode == "splitkv")
    ctx_full = contexts(args)                       # tokens attended per sequence, the one being decoded included
    seqs = list(plan.seqs)
    last_part = (not split_mode) or (rank == world - 1 and not emulated)
    # tokens of every local sequence this rank holds after the step, and the value of pos[] it passes
    hist, ctx, pos_local = [], [], []
    for b in seqs:
        first, n_loc = plan.token_range(ctx_full[b], PAGE)
        n_hist = n_loc - 1 if last_part else n_loc          # rows already cached here before the step
        hist.append((first, max(0, n_hist)))
        ctx.append(max(1, n_loc))
        pos_local.append(max(0, n_hist))
    B = len(seqs)
    pages = [(c + PAGE - 1) // PAGE for c in ctx]
    max_pages = max(pages)
    n_pages = sum(pages)
    types = (QWEN35_LAYER_TYPES * ((args.layers + 3) // 4))[:args.layers]
    n_q_l, n_kv_l, n_v_l, n_k_l = len(plan.q_heads), len(plan.kv_heads), len(plan.v_heads), len(plan.k_heads)
    cache = HybridCache(types, n_pages=n_pages, n_slots=B, max_batch=B, max_pages_per_seq=max_pages,
                        max_seq_len=max(ctx), n_q=n_q_l, n_kv=n_kv_l, n_v=n_v_l, n_k=n_k_l)
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
    # The whole problem's step inputs from one seed (the same on every rank), then this rank's slices.
    A, D = cache.n_attn, cache.n_delta
    fg = torch.Generator().manual_seed(args.seed + 17)
    full = {"attn_q": torch.randn(A, args.batch, N_Q, HD, generator=fg), "attn_gate": torch.randn(A, args.batch, N_Q, HD, generator=fg),
            "attn_k": torch.randn(A, args.batch, N_KV, HD, generator=fg), "attn_v": torch.randn(A, args.batch, N_KV, HD, generator=fg),
            "delta_qkv": torch.randn(D, args.batch, CONV_DIM, generator=fg),
            "delta_beta": torch.sigmoid(torch.randn(D, args.batch, N_V, generator=fg)),
            "delta_g": -torch.nn.functional.softplus(torch.randn(D, args.batch, N_V, generator=fg)),
            "conv_w": torch.randn(D, CONV_DIM, CONV_K, generator=fg) * 0.5}
    mine = {n: x.contiguous() for n, x in plan.slice_io(full).items()}
    sh = cache.io_shapes(B)
    for n in ("attn_q", "attn_gate", "attn_k", "attn_v", "delta_qkv", "delta_beta", "delta_g", "conv_w"):
        assert tuple(mine[n].shape) == tuple(sh[n]), (n, mine[n].shape, sh[n])
    host = {n: mine[n].pin_memory() for n in ("attn_q", "attn_gate", "attn_k", "attn_v", "delta_qkv", "delta_beta", "delta_g")}
    host["attn_o"] = torch.zeros(sh["attn_o"]).pin_memory()
    host["delta_o"] = torch.zeros(sh["delta_o"]).pin_memory()
    host["page_table"] = table.pin_memory()
    host["pos"] = torch.tensor(pos_local, dtype=torch.int32).pin_memory()
    cache.set_conv_w(mine["conv_w"])
    dev = {n: x.cuda() for n, x in host.items()}
    dev["conv_w"] = mine["conv_w"].cuda()
    stream = torch.cuda.current_stream()

    # ---------------- the exchange of a sharded step (library side) ----------------
    comm, gathered = None, None
    if strong:
        def bcast(raw):
            t = torch.zeros(_lib.COMM_ID_BYTES, dtype=torch.uint8, device="cuda")
            if raw is not None:
                t.copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
            dist.broadcast(t, 0)
            return bytes(t.cpu().numpy().tobytes())
        comm = Comm(rank, world, bcast)
        gs = cache.gather_shapes(B, world)
        names = ["attn_o_all", "delta_o_all"] + (["attn_ml_all", "attn_o_final"] if split_mode else [])
        gathered = {n: torch.zeros(gs[n], device="cuda") for n in names}
        cache.set_gather(comm, gathered, args.layers_per_exchange, args.reserve_sms)
    if split_mode:
        dev["attn_ml"] = torch.zeros(sh["attn_ml"], device="cuda")
        dev["no_append"] = not last_part

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---------------- check of the sharded step: first layer of each kind, two sequences ----------------
    check = None
    if strong and not args.no_check:
        check = sharded_step_check(args, plan, cache, dev, gathered, full, ctx_full, hist, table, seqs, rank, world)
    if args.no_graph:
        cache.set_graph(False)

    # ---------------- device-resident timing ----------------
    # Timed region: K steps back to back through rl_stack_decode (graph replay after the
    # second warm-up step), no host synchronisation between steps.
    for _ in range(max(3, args.warmup)):
        cache.decode(dev, B)
    _lib.check_device()
    c0 = sampler.cursor()                            # may sleep: before the barrier, so that the ranks leave it together
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        cache.decode(dev, B)
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
        for k, v in cache.timing().items():      # waits for this step's last event
            fam[k] = fam.get(k, 0.0) + v
    e3.record(stream)
    sync_all()
    clocks = sampler.window(c0, sampler.cursor())
    ms_events = e2.elapsed_time(e3) / args.steps
    _lib.check_device()
    cache.set_timing(False)
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    ms_per_step = ms_max / args.steps
    total_seqs = args.batch if strong or world == 1 else args.batch * world
    value = total_seqs / (ms_per_step * 1e-3)

    # ---------------- end to end through the host-buffer entry point ----------------
    e2e = None
    if not args.no_e2e and not split_mode and not emulated:
        for _ in range(3):
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
        e2e = {"value": total_seqs / (dt / args.steps), "unit": "seq-steps/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": dt / args.steps * 1e3,
               "note": "per rank: pinned host inputs of its shard -> device, the step (with the exchange), its "
                       "output slices -> pinned host; bytes are per rank" if strong else
                       "rl_stack_decode_host with pinned host buffers"}
        _lib.check_device()

    line = None
    if rank == 0:
        ab = algorithmic_bytes(args.layers, ctx, n_q_l, n_kv_l, n_v_l, n_k_l)
        n_attn = cache.n_attn
        attn_ms_per_launch = fam["attn_decode"] / args.steps / max(1, n_attn)
        achieved = ab["attn_decode"] / (attn_ms_per_launch * 1e-3) / 1e9
        families = {}
        for k, nl in (("attn_decode", n_attn), ("attn_combine", n_attn), ("kv_append", n_attn),
                      ("delta_rule", cache.n_delta)):
            per = fam[k] / args.steps / max(1, nl)
            families[k] = {"ms_per_launch": round(per, 5), "share": round(fam[k] / args.steps / ms_events, 4)}
            if k in ab:
                families[k]["gbs"] = round(ab[k] / (per * 1e-3) / 1e9, 1) if per > 0 else None
        gather_bytes = 0
        if strong:
            gather_bytes = sum(x.numel() * x.element_size() for n, x in gathered.items() if n.endswith("_all"))
        par = {"single": "one GPU" if not emulated else "one GPU running rank 0's share of a %d-rank %s step, no exchange"
               % (args.emulate_ranks, plan.mode),
               "seq": "weak: every rank owns a whole batch of %d (same contexts), no collective" % args.batch,
               "heads": "strong: KV / value heads x%d, then sequences x%d; per-layer outputs all-gathered by the library "
                        "(ncclAllGather on a side stream, one grouped call per %d layers, %d bytes received per rank "
                        "per step)" % (plan.head_ways, plan.seq_ways, args.layers_per_exchange or 4, gather_bytes),
               "splitkv": "strong: token ranges of every sequence x%d + DeltaNet heads x%d; (o, max, sum) partials "
                          "all-gathered by the library (ncclAllGather on a side stream, %d bytes received per rank per "
                          "step) and merged by lse_combine_kernel" % (world, world, gather_bytes)}[mode]
        line = {
            "metric": "hybrid-layer decode steps/sec", "value": value, "unit": "seq-steps/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "f16 KV / f32 state", "data": "synthetic",
            "config": {"workload": workload_name(args), "l2": "inputs larger than L2 (%.1f GB streamed per step per rank)"
                       % (ab["step"] / 1e9),
                       "parallelism": par, "ctx_tokens_rank0": sum(ctx), "cache_bytes_rank0": cache.bytes},
            "clocks": clocks,
            "gpu_launches": (cache.launches_per_step + (n_attn if split_mode else 0)) * args.steps,
            "step_hbm_gbs": ab["step"] * world / (ms_per_step * 1e-3) / 1e9,   # rank 0's bytes x ranks
            "roofline": _hbm_roofline("attn_decode_f16_kernel", ab["attn_decode"], attn_ms_per_launch, peaks,
                                      int(1.0246 * ab["attn_decode"]),
                                      "ncu capture of a batch-8 launch scaled by algorithmic bytes"),
            "kernel_families": families,
            "kernel_timing_pass": {"ms_per_step": ms_events, "note": "same K steps repeated as plain launches "
                                   "with CUDA events between the kernels; roofline and shares come from this pass"},
            "graph_replay": not args.no_graph,
        }
        line["roofline"]["ms_per_launch"] = attn_ms_per_launch
        if check is not None:
            line["sharded_step_check"] = check
        if e2e:
            line["e2e"] = e2e
    cache.close()
    if comm:
        comm.close()
    del cache, dev, gathered
    torch.cuda.empty_cache()
    if rank == 0:
        if world == 1 and not args.no_operators and not emulated:
            line["operators"] = run_operators(args, sampler, peaks)
        if world == 1 and not args.no_cpu_baseline and not emulated:
            line["cpu_baseline"] = cpu_reference_leg(args, ctx_full)
        print(json.dumps(line), flush=True)
    sampler.stop()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def sharded_step_check(args, plan, cache, dev, gathered, full, ctx_full, hist, table, seqs, rank, world):
    """One step of the sharded stack on known data for two sequences, first attention layer and first
    DeltaNet layer; rank 0 compares the gathered outputs with the unsharded operators (rl_attn_decode,
    rl_conv1d_update + rl_delta_recurrent over all heads) on the same inputs.  Every rank exits
    non-zero on a mismatch."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from rapidllm_b200 import _lib, ops
    split_mode = plan.mode == "splitkv"
    picks = sorted({0, args.batch - 1})
    known = {}
    for b in picks:
        g = torch.Generator().manual_seed(args.seed * 7919 + b)
        n_hist = ctx_full[b] - 1
        known[b] = {"k": torch.randn(n_hist, N_KV, HD, generator=g).half(), "v": torch.randn(n_hist, N_KV, HD, generator=g).half(),
                    "S": torch.randn(N_V, DK, DV, generator=g) * 0.02, "conv": torch.randn(CONV_DIM, CONV_K, generator=g)}
        if b in seqs:
            lb = seqs.index(b)
            first, n_h = hist[lb]
            kvh = list(plan.kv_heads)
            if n_h > 0:
                ops.kv_append(cache.k_pool(0), cache.v_pool(0), table[lb].cuda(),
                              known[b]["k"][first:first + n_h][:, kvh].contiguous().cuda(),
                              known[b]["v"][first:first + n_h][:, kvh].contiguous().cuda(), pos0=0)
            cache.state(0)[lb].copy_(known[b]["S"][list(plan.v_heads)])
            cache.conv(0)[lb].copy_(known[b]["conv"][plan.conv_channels()])
    cache.decode(dev, len(seqs))
    torch.cuda.synchronize()
    _lib.check_device()
    result = {"sequences": picks, "ok": True}
    bad = torch.zeros(1, device="cuda")
    if rank == 0:
        A0 = gathered["attn_o_final"][0] if split_mode else plan.place_attn(
            torch.zeros(args.batch, N_Q, HD, device="cuda"), gathered["attn_o_all"][0])
        D0 = plan.place_delta(torch.zeros(args.batch, N_V, DV, device="cuda"), gathered["delta_o_all"][0])
        errs = {"attn_max_abs": 0.0, "attn_rel_l2": 0.0, "delta_max_abs": 0.0}
        for b in picks:
            # unsharded attention over the same history + the appended row
            n = ctx_full[b]
            n_pg = (n + PAGE - 1) // PAGE
            kp, vp = ops.new_pool(n_pg, N_KV), ops.new_pool(n_pg, N_KV)
            row = torch.arange(n_pg, dtype=torch.int32, device="cuda")
            ops.kv_append(kp, vp, row, known[b]["k"].cuda(), known[b]["v"].cuda(), pos0=0)
            ops.kv_append(kp, vp, row, full["attn_k"][0, b:b + 1].cuda(), full["attn_v"][0, b:b + 1].cuda(), pos0=n - 1)
            ref = ops.attn_decode(full["attn_q"][0, b:b + 1].cuda(), kp, vp, row.unsqueeze(0),
                                  torch.tensor([n], dtype=torch.int32, device="cuda"), full["attn_gate"][0, b:b + 1].cuda())[0]
            got = A0[b]
            errs["attn_max_abs"] = max(errs["attn_max_abs"], float((got - ref).abs().max()))
            errs["attn_rel_l2"] = max(errs["attn_rel_l2"], float((got - ref).norm() / ref.norm()))
            # unsharded DeltaNet step over all heads
            S = known[b]["S"].cuda().unsqueeze(0).contiguous()
            cst = known[b]["conv"].cuda().unsqueeze(0).contiguous()
            mixed = ops.conv1d_update(full["delta_qkv"][0, b:b + 1].cuda(), full["conv_w"][0].cuda(), cst)
            qk = N_K * DK
            refd = ops.delta_recurrent_step(S, mixed[:, :qk].reshape(1, N_K, DK).contiguous(),
                                            mixed[:, qk:2 * qk].reshape(1, N_K, DK).contiguous(),
                                            mixed[:, 2 * qk:].reshape(1, N_V, DV).contiguous(),
                                            full["delta_beta"][0, b:b + 1].cuda(), full["delta_g"][0, b:b + 1].cuda())[0]
            errs["delta_max_abs"] = max(errs["delta_max_abs"], float((D0[b] - refd).abs().max()))
        _lib.check_device()
        ok = (errs["attn_max_abs"] <= ATTN_MAX_ABS and errs["attn_rel_l2"] <= ATTN_REL_L2 and
              errs["delta_max_abs"] <= DELTA_MAX_ABS and all(math.isfinite(v) for v in errs.values()))
        result.update(errs)
        result["ok"] = bool(ok)
        result["tolerance"] = {"attn_max_abs": ATTN_MAX_ABS, "attn_rel_l2": ATTN_REL_L2, "delta_max_abs": DELTA_MAX_ABS}
        if not ok:
            bad += 1
            print("sharded step check FAILED: %s" % json.dumps(result), file=sys.stderr, flush=True)
    dist.all_reduce(bad)
    if float(bad.item()) > 0:
        dist.barrier()
        dist.destroy_process_group()
        raise SystemExit(3)
    return result


if __name__ == "__main__":
    main()
