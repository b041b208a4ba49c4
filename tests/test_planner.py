"""rl_plan_cache: host-only arithmetic mirroring plan_memory (src/runtime/planner.cpp:28-44)
and the engine's KV-type policy (cuda_engine.cu:20106-20118) for paged pools."""
import ctypes as C

import pytest

from rapidllm_b200 import _lib

GIB = 1 << 30


def _plan(**kw):
    base = dict(weight_bytes=0, available_bytes=0, pad_bytes=64 << 20, ctx=32768, max_batch=1, n_attn_layers=16,
                n_kv=4, head_dim=256, n_delta_layers=48, n_v=48, dk=128, dv=128, conv_dim=10240, conv_k=4,
                page_tokens=64, kv_policy=_lib.RL_KV_POLICY_AUTO, allow_shrink=0, prefill_chunk=0)
    base.update(kw)
    inp, out = _lib.PlanInput(**base), _lib.PlanResult()
    st = _lib.lib().rl_plan_cache(C.byref(inp), C.byref(out))
    return st, out


def test_sizes_follow_plan_memory():
    st, r = _plan(ctx=4096)
    assert st == 0 and r.ok and r.kv_dtype == _lib.RL_KV_F16 and r.message == b"ok"
    # plan_memory: kv = n_attn * n_kv * hd * 2 (K,V) * 2 B * ctx; state = n_delta * (nv*dk*dv + conv_dim*k) * 4
    assert r.kv_bytes == 16 * 4 * 256 * 2 * 2 * 4096
    assert r.state_bytes == 48 * (48 * 128 * 128 + 10240 * 4) * 4
    assert r.need_bytes == r.kv_bytes + r.state_bytes + (64 << 20)
    assert r.max_pages_per_seq == 64 and r.n_pages == 64 and r.ctx == 4096
    st, r = _plan(ctx=4097, max_batch=3)
    assert r.max_pages_per_seq == 65 and r.n_pages == 195


def test_policy_and_budget():
    # 32 sequences x 32768 tokens of F16 KV = 64 GiB: fits 180 GB next to 30 GB of weights
    st, r = _plan(max_batch=32, weight_bytes=30 * GIB, available_bytes=180 * 10**9)
    assert r.ok and r.kv_dtype == _lib.RL_KV_F16
    # 262144 tokens x 8 sequences = 128 GiB of F16 KV does not fit next to the weights: compact (22.4 KiB/token)
    st, r = _plan(ctx=262144, max_batch=8, weight_bytes=60 * GIB, available_bytes=180 * 10**9)
    assert r.ok and r.kv_dtype == _lib.RL_KV_Q8K_TQ3V
    # ... plus the F16 compute window over the first max(8192, 2 * prefill chunk) tokens of each sequence
    assert r.window_tokens == 8192 and r.window_pages_per_seq == 128
    assert r.window_bytes == 16 * 4 * 256 * 2 * 2 * 8192 * 8
    assert r.kv_bytes == 16 * 4 * _lib.lib().rl_kv_compact_page_bytes() * 4096 * 8 + r.window_bytes
    # forced F16 refuses with the reference's message shape ...
    st, r = _plan(ctx=262144, max_batch=8, weight_bytes=60 * GIB, available_bytes=180 * 10**9,
                  kv_policy=_lib.RL_KV_POLICY_F16)
    assert st == 0 and not r.ok and r.message.startswith(b"OOM: need ") and b"(ctx=262144)" in r.message
    # ... or shrinks to whole pages that fit
    st, r = _plan(ctx=262144, max_batch=8, weight_bytes=60 * GIB, available_bytes=180 * 10**9,
                  kv_policy=_lib.RL_KV_POLICY_F16, allow_shrink=1)
    assert r.ok and 0 < r.ctx < 262144 and r.ctx % 64 == 0 and r.need_bytes <= 180 * 10**9
    assert b"reduced" in r.message
    st2, r2 = _plan(ctx=r.ctx + 64, max_batch=8, weight_bytes=60 * GIB, available_bytes=180 * 10**9,
                    kv_policy=_lib.RL_KV_POLICY_F16)
    assert not r2.ok                                        # one more page would not have fitted
    # forced compact; the window follows the prefill chunk and never exceeds ctx
    st, r = _plan(kv_policy=_lib.RL_KV_POLICY_COMPACT, prefill_chunk=8192)
    assert r.kv_dtype == _lib.RL_KV_Q8K_TQ3V and r.window_tokens == 16384
    st, r = _plan(kv_policy=_lib.RL_KV_POLICY_COMPACT, ctx=4096)
    assert r.window_tokens == 4096 and r.window_pages_per_seq == 64
    st, r = _plan(kv_policy=_lib.RL_KV_POLICY_COMPACT, ctx=1 << 20, max_batch=8, weight_bytes=60 * GIB,
                  available_bytes=180 * 10**9, allow_shrink=1)
    assert r.ok and r.ctx % 64 == 0 and r.need_bytes <= 180 * 10**9 and r.window_tokens == 8192
    st2, r2 = _plan(kv_policy=_lib.RL_KV_POLICY_COMPACT, ctx=r.ctx + 64, max_batch=8, weight_bytes=60 * GIB,
                    available_bytes=180 * 10**9)
    assert not r2.ok
    # nothing left after the weights
    st, r = _plan(weight_bytes=200 * GIB, available_bytes=180 * 10**9, allow_shrink=1)
    assert st == 0 and not r.ok


def test_bad_input_is_refused():
    assert _plan(ctx=0)[0] != 0
    assert _plan(kv_policy=7)[0] != 0
    assert _plan(kv_policy=_lib.RL_KV_POLICY_COMPACT, head_dim=128)[0] != 0
    assert _lib.lib().rl_plan_cache(None, None) != 0
