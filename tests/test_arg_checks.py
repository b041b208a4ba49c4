"""Argument validation of the C ABI: refused before anything touches a device, with the
reference's status codes (include/rapidllm/api.h:11-20) and a message in rl_last_error()."""
import ctypes as C

from rapidllm_b200 import _lib

RANGE, UNSUPPORTED = 6, 4


def _err():
    return _lib.lib().rl_last_error().decode()


def test_null_params_and_bad_shapes_are_refused():
    L = _lib.lib()
    assert L.rl_attn_decode(None, None, None, None, None, None, None, None, 0, None, None) == RANGE
    assert L.rl_attn_prefill(None, None, None, None, None, None, None, None, None, None) == RANGE
    assert "params" in _err()
    pp = _lib.AttnPrefillParams(n_q=24, n_kv=4, head_dim=128, seq=8, br=128, bc=64, pos0=0, page_tokens=64,
                                n_pages=4, n_table=4)
    assert L.rl_attn_prefill(None, None, None, None, None, None, None, None, C.byref(pp), None) == UNSUPPORTED
    assert "head_dim" in _err()
    pp.head_dim, pp.n_q = 256, 25
    assert L.rl_attn_prefill(None, None, None, None, None, None, None, None, C.byref(pp), None) == UNSUPPORTED
    pp.n_q, pp.pos0 = 24, 10_000
    assert L.rl_attn_prefill(None, None, None, None, None, None, None, None, C.byref(pp), None) == RANGE
    assert "exceeds" in _err()
    assert L.rl_attn_prefill_workspace_bytes(None) == 0
    dp = _lib.DeltaRecurrentParams(n_v=48, dk=64, dv=128, eps_l2=1e-6, batch=1, n_slots=1, n_qk=16, head_map=1)
    assert L.rl_delta_recurrent(None, None, None, None, None, None, None, None, C.byref(dp), None) == UNSUPPORTED
    dp.dk, dp.n_qk = 128, 7
    assert L.rl_delta_recurrent(None, None, None, None, None, None, None, None, C.byref(dp), None) == RANGE
    dp.n_qk = 16
    assert L.rl_delta_recurrent_multi(None, None, None, None, None, None, None, None, None, C.byref(dp), 65, 0, 0,
                                      None) == RANGE
    assert L.rl_gated_rmsnorm(None, None, None, None, 1, 48, 64, 1e-6, None) == UNSUPPORTED
    assert L.rl_delta_gates(None, None, None, None, None, None, -1, 48, None) == RANGE
    assert L.rl_rmsnorm(None, None, None, 1, 0, 1e-6, None) == RANGE
    assert L.rl_rmsnorm(None, None, None, 1, 8, 1e-6, None) == RANGE
    qp = _lib.AttnQkPrepareParams(n_q=24, n_kv=4, head_dim=256, rotary_dim=63, rows=1, pos0=0, theta=1e7, eps=1e-6)
    assert L.rl_attn_qk_prepare(None, None, None, None, None, None, None, C.byref(qp), None) == RANGE
    assert L.rl_kv_compact_to_f16(None, None, 0, 1, None, None, None, 0, 1, 4, 4, 100, None, None) == UNSUPPORTED
    assert L.rl_stack_decode(None, None, None) == RANGE
    assert L.rl_stack_set_graph(None, 1) == RANGE
    assert L.rl_cache_create(None, None) == RANGE


def test_zero_sized_calls_are_no_ops():
    L = _lib.lib()
    pp = _lib.AttnPrefillParams(n_q=24, n_kv=4, head_dim=256, seq=0, br=128, bc=64, pos0=0, page_tokens=64,
                                n_pages=4, n_table=4)
    assert L.rl_attn_prefill(None, None, None, None, None, None, None, None, C.byref(pp), None) == 0
    assert L.rl_gated_rmsnorm(None, None, None, None, 0, 48, 128, 1e-6, None) == 0
    assert L.rl_delta_gates(None, None, None, None, None, None, 0, 48, None) == 0
    assert L.rl_rmsnorm(None, None, None, 0, 8, 1e-6, None) == 0
    dp = _lib.DeltaRecurrentParams(n_v=48, dk=128, dv=128, eps_l2=1e-6, batch=0, n_slots=1, n_qk=16, head_map=1)
    assert L.rl_delta_recurrent(None, None, None, None, None, None, None, None, C.byref(dp), None) == 0
    assert L.rl_delta_recurrent_multi(None, None, None, None, None, None, None, None, None, C.byref(dp), 0, 0, 0,
                                      None) == 0
