"""Compact-KV policy with an F16 compute window (WindowedKV): which cache each call attends over,
and parity of every branch with the oracle (F16-rounded rows inside the window, the dequantised
compact cache past it). Rules: src/kernels/cuda/cuda_engine.cu:18948-18953, 18487-18497, 6033-6036."""
import numpy as np
import pytest
import torch

from helpers import ATTN_MAX_ABS, ATTN_REL_L2, rel_l2

pytestmark = pytest.mark.gpu

N_Q, N_KV, HD = 24, 4, 256


def _close(o, ref, what):
    o = o.cpu().numpy()
    assert np.isfinite(o).all(), what
    assert np.abs(o - ref).max() <= ATTN_MAX_ABS and rel_l2(o, ref) <= ATTN_REL_L2, \
        (what, np.abs(o - ref).max(), rel_l2(o, ref))


def test_window_then_compact(oracle):
    from rapidllm_b200 import _lib
    from rapidllm_b200.kv_window import WindowedKV
    gen = torch.Generator().manual_seed(31)
    win, ctx = 192, 448
    kv = WindowedKV(max_batch=2, ctx=ctx, window_tokens=win)
    n = [300, 150]                                  # final lengths of the two sequences
    k = [torch.randn(ctx, N_KV, HD, generator=gen) for _ in n]
    v = [torch.randn(ctx, N_KV, HD, generator=gen) for _ in n]

    def f16(x):
        return x.half().float().numpy()

    def deq(b, upto):
        return oracle.compact_dequant(*oracle.compact_store(k[b][:upto].numpy(), v[b][:upto].numpy(), 128), 128)

    def chunk(b, T, expect):
        p0 = kv.lens[b]
        q = torch.randn(T, N_Q, HD, generator=gen).bfloat16()
        gate = torch.randn(T, N_Q, HD, generator=gen)
        o = kv.prefill(b, q.cuda(), k[b][p0:p0 + T].cuda(), v[b][p0:p0 + T].cuda(), gate.cuda())
        _lib.check_device()
        assert kv.last_path == expect and kv.lens[b] == p0 + T
        kd, vd = (f16(k[b][:p0 + T]), f16(v[b][:p0 + T])) if expect == "window" else deq(b, p0 + T)
        ref = oracle.attn_prefill_rows(q.float().numpy(), kd, vd, np.arange(p0, p0 + T))
        ref = ref / (1.0 + np.exp(-gate.numpy()))
        _close(o, ref, ("prefill", b, p0, T))

    chunk(0, 100, "window")                         # [0, 100) inside the window
    chunk(1, 64, "window")
    chunk(0, 92, "window")                          # ends exactly at the window edge
    # decode: both inside the window -> F16
    for step in range(3):
        seqs = [0, 1] if step < 2 else [1]
        pos = [kv.lens[s] for s in seqs]
        q = torch.randn(len(seqs), N_Q, HD, generator=gen)
        gate = torch.randn(len(seqs), N_Q, HD, generator=gen)
        kr = torch.stack([k[s][p] for s, p in zip(seqs, pos)])
        vr = torch.stack([v[s][p] for s, p in zip(seqs, pos)])
        o = kv.decode(seqs, q.cuda(), kr.cuda(), vr.cuda(), gate.cuda())
        _lib.check_device()
        # sequence 0 is at the window edge from the first step on: the whole batch goes compact
        expect = "compact" if 0 in seqs else "window"
        assert kv.last_path == expect
        for i, (s, p) in enumerate(zip(seqs, pos)):
            kd, vd = deq(s, p + 1) if expect == "compact" else (f16(k[s][:p + 1]), f16(v[s][:p + 1]))
            _close(o[i], oracle.gated_attn_decode(q[i].numpy(), kd, vd, gate[i].numpy()), ("decode", s, p))
    assert kv.lens == [194, 67]
    chunk(1, 83, "window")                          # sequence 1 still inside: the F16 rows were kept up to date
    chunk(0, 106, "compact")                        # past the window: over the dequantised compact cache
    chunk(1, 60, "compact")                         # straddles the edge: compact, nothing written to the window
    assert kv.lens == [300, 210]
    with pytest.raises(_lib.RlError):
        kv.prefill(0, torch.zeros(200, N_Q, HD).bfloat16().cuda(), k[0][:200].cuda(), v[0][:200].cuda())


def test_sizes_come_from_the_plan():
    import ctypes as C
    from rapidllm_b200 import _lib
    from rapidllm_b200.kv_window import WindowedKV
    inp = _lib.PlanInput(weight_bytes=0, available_bytes=0, pad_bytes=0, ctx=12288, max_batch=1, n_attn_layers=1,
                         n_kv=N_KV, head_dim=HD, n_delta_layers=0, n_v=48, dk=128, dv=128, conv_dim=10240, conv_k=4,
                         page_tokens=64, kv_policy=_lib.RL_KV_POLICY_COMPACT, allow_shrink=0, prefill_chunk=1024)
    out = _lib.PlanResult()
    assert _lib.lib().rl_plan_cache(C.byref(inp), C.byref(out)) == 0 and out.window_tokens == 8192
    kv = WindowedKV(1, out.ctx, out.window_tokens)
    assert kv.bytes() == out.kv_bytes
    assert kv.pages_w == out.window_pages_per_seq and kv.pages_c == out.max_pages_per_seq
