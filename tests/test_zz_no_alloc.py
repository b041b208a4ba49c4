"""rl_attn_decode_noalloc: decode attention for callers that cannot allocate device memory.

Some hosts of this library run under a fixed memory plan: every byte of HBM was handed out
at start-up (KV pools, weights, activations) and neither cudaMalloc nor a spare workspace is
available when a decode step runs.  For them the split-KV partials live in an array inside
the library's device image.  This test calls that entry point through the C ABI twice in a
row (the array keeps the previous call's contents, so the second call must not be disturbed
by the first) and checks both results against rl_attn_decode with a caller workspace.
The file name sorts last so that a run stopping at the first failure has run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import ATTN_MAX_ABS, ATTN_REL_L2, paged_from_rows, rel_l2

pytestmark = pytest.mark.gpu

N_Q, N_KV, HD = 24, 4, 256


def _case(seed, lens):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(len(lens), N_Q, HD, generator=gen)
    gate = torch.randn(len(lens), N_Q, HD, generator=gen)
    ks = [torch.randn(n, N_KV, HD, generator=gen).half() for n in lens]
    vs = [torch.randn(n, N_KV, HD, generator=gen).half() for n in lens]
    kp, vp, table, sl = paged_from_rows(ks, vs, gen)
    return q.cuda(), gate.cuda(), kp, vp, table, sl


def _noalloc(q, gate, kp, vp, table, sl):
    from rapidllm_b200 import _lib, ops
    p = ops.attn_params(N_Q, N_KV, q.shape[0], kp.shape[0], table.shape[1], table.shape[1] * 64)
    o = torch.full_like(q, float("nan"))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = _lib.lib().rl_attn_decode_noalloc(C.c_void_p(kp.data_ptr()), C.c_void_p(vp.data_ptr()),
                                           C.c_void_p(table.data_ptr()), C.c_void_p(sl.data_ptr()),
                                           C.c_void_p(q.data_ptr()), C.c_void_p(gate.data_ptr()),
                                           C.c_void_p(o.data_ptr()), C.byref(p), stream)
    return st, o


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    from rapidllm_b200 import _lib, ops
    # two different problems back to back: the second sees the first one's leftovers in the array
    for seed, lens in ((101, [700, 64, 1, 2049, 33]), (102, [90, 1300])):
        q, gate, kp, vp, table, sl = _case(seed, lens)
        ref = ops.attn_decode(q, kp, vp, table, sl, gate)          # rl_attn_decode, caller workspace
        st, o = _noalloc(q, gate, kp, vp, table, sl)
        assert st == 0, _lib.lib().rl_last_error()
        _lib.check_device()
        a, b = o.cpu().numpy(), ref.cpu().numpy()
        assert np.isfinite(a).all()
        assert np.abs(a - b).max() <= ATTN_MAX_ABS and rel_l2(a, b) <= ATTN_REL_L2
        # and once more on the same inputs: same answer again
        st, o2 = _noalloc(q, gate, kp, vp, table, sl)
        assert st == 0
        _lib.check_device()
        assert np.abs(o2.cpu().numpy() - b).max() <= ATTN_MAX_ABS and rel_l2(o2.cpu().numpy(), b) <= ATTN_REL_L2


def test_sizes_beyond_the_built_in_array_are_refused():
    from rapidllm_b200 import _lib, ops
    q, gate, kp, vp, table, sl = _case(103, [10])
    p = ops.attn_params(N_Q, N_KV, 1000, kp.shape[0], table.shape[1], table.shape[1] * 64)
    st = _lib.lib().rl_attn_decode_noalloc(C.c_void_p(kp.data_ptr()), C.c_void_p(vp.data_ptr()),
                                           C.c_void_p(table.data_ptr()), C.c_void_p(sl.data_ptr()),
                                           C.c_void_p(q.data_ptr()), None, C.c_void_p(q.data_ptr()),
                                           C.byref(p), None)
    assert st == 6                                                   # RL_ERR_RANGE, nothing launched
    assert b"built-in array" in _lib.lib().rl_last_error()
    assert _lib.device_error() == 0
