"""rl_attn_decode_noalloc: decode attention for callers that cannot allocate device memory.

Some hosts of this library run under a fixed memory plan: every byte of HBM was handed out
at start-up (KV pools, weights, activations) and neither cudaMalloc nor a spare workspace is
available when a decode step runs.  For them the split-KV partials live in an array inside
the library's device image.  This test calls that entry point through the C ABI twice in a
row (the array keeps the previous call's contents, so the second call must not be disturbed
by the first) and checks both results against rl_attn_decode with a caller workspace: the two
entry points run the same kernels over the same division of the work with fixed-order merges,
so the outputs must agree bit for bit, and one of them is also compared with the CPU oracle.
It also checks that calls after a device's first allocate nothing (free device memory is
unchanged) and that the documented size limit sits exactly where the header says.
The file name sorts last so that a run stopping at the first failure has run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import ATTN_MAX_ABS, ATTN_REL_L2, paged_from_rows, rel_l2

pytestmark = pytest.mark.gpu

N_Q, N_KV, HD = 24, 4, 256
BUILT_IN_BYTES = 4 << 20


def _case(seed, lens):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(len(lens), N_Q, HD, generator=gen)
    gate = torch.randn(len(lens), N_Q, HD, generator=gen)
    ks = [torch.randn(n, N_KV, HD, generator=gen).half() for n in lens]
    vs = [torch.randn(n, N_KV, HD, generator=gen).half() for n in lens]
    kp, vp, table, sl = paged_from_rows(ks, vs, gen)
    return q, gate, ks, vs, kp, vp, table, sl


def _noalloc(q, gate, kp, vp, table, sl, out=None, batch=None):
    from rapidllm_b200 import _lib, ops
    p = ops.attn_params(N_Q, N_KV, q.shape[0] if batch is None else batch, kp.shape[0], table.shape[1],
                        table.shape[1] * 64)
    o = torch.full_like(q, float("nan")) if out is None else out
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = _lib.lib().rl_attn_decode_noalloc(C.c_void_p(kp.data_ptr()), C.c_void_p(vp.data_ptr()),
                                           C.c_void_p(table.data_ptr()), C.c_void_p(sl.data_ptr()),
                                           C.c_void_p(q.data_ptr()), C.c_void_p(gate.data_ptr()),
                                           C.c_void_p(o.data_ptr()), C.byref(p), stream)
    return st, o


def test_two_calls_in_a_row_match_the_workspace_entry_point(oracle):
    from rapidllm_b200 import _lib, ops
    # two different problems back to back: the second sees the first one's leftovers in the array
    for seed, lens in ((101, [700, 64, 1, 2049, 33]), (102, [90, 1300])):
        q, gate, ks, vs, kp, vp, table, sl = _case(seed, lens)
        qd, gd = q.cuda(), gate.cuda()
        ref = ops.attn_decode(qd, kp, vp, table, sl, gd)             # rl_attn_decode, caller workspace
        st, o = _noalloc(qd, gd, kp, vp, table, sl)
        assert st == 0, _lib.lib().rl_last_error()
        _lib.check_device()
        assert torch.isfinite(o).all()
        assert torch.equal(o, ref)                                    # same kernels, same plan: same bits
        # and once more on the same inputs: same answer again
        st, o2 = _noalloc(qd, gd, kp, vp, table, sl)
        assert st == 0
        _lib.check_device()
        assert torch.equal(o2, ref)
        # the tolerance of every attention test here, against the CPU oracle
        a = o.cpu().numpy()
        for b, n in enumerate(lens):
            want = oracle.gated_attn_decode(q[b].numpy(), ks[b].float().numpy(), vs[b].float().numpy(),
                                            gate[b].numpy())
            assert np.abs(a[b] - want).max() <= ATTN_MAX_ABS and rel_l2(a[b], want) <= ATTN_REL_L2, (b, n)


def test_later_calls_allocate_nothing():
    """After a device's first call (the library's one-time set-up) free device memory does not move."""
    from rapidllm_b200 import _lib
    q, gate, ks, vs, kp, vp, table, sl = _case(104, [300, 65])
    qd, gd = q.cuda(), gate.cuda()
    out = torch.empty_like(qd)                                        # the test allocates nothing below this line
    st, _ = _noalloc(qd, gd, kp, vp, table, sl, out=out)
    assert st == 0, _lib.lib().rl_last_error()
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        st, _ = _noalloc(qd, gd, kp, vp, table, sl, out=out)
        assert st == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free0
    _lib.check_device()


def _largest_batch_that_fits():
    from rapidllm_b200 import _lib, ops
    lo = 1
    while True:
        p = ops.attn_params(N_Q, N_KV, lo + 1, 8, 1, 64)
        need = _lib.lib().rl_attn_decode_workspace_bytes(C.byref(p))
        if need == 0 or need > BUILT_IN_BYTES:
            return lo
        lo += 1


def test_the_size_limit_is_where_the_header_says():
    """The largest batch whose partials fit the 4 MiB array (132 on a 148-SM part with 24Q/4KV heads)
    is accepted and equals rl_attn_decode; one more is refused with RL_ERR_RANGE before any launch."""
    from rapidllm_b200 import _lib, ops
    limit = _largest_batch_that_fits()
    if torch.cuda.get_device_properties(0).multi_processor_count == 148:
        assert limit == 132
    gen = torch.Generator().manual_seed(105)
    lens = [int(x) for x in torch.randint(1, 64, (limit + 1,), generator=gen)]
    q, gate, ks, vs, kp, vp, table, sl = _case(106, lens)
    qd, gd = q.cuda(), gate.cuda()
    ref = ops.attn_decode(qd[:limit].contiguous(), kp, vp, table[:limit].contiguous(), sl[:limit].contiguous(),
                          gd[:limit].contiguous())
    st, o = _noalloc(qd[:limit].contiguous(), gd[:limit].contiguous(), kp, vp, table[:limit].contiguous(),
                     sl[:limit].contiguous())
    assert st == 0, _lib.lib().rl_last_error()
    _lib.check_device()
    assert torch.equal(o, ref)
    st, _ = _noalloc(qd, gd, kp, vp, table, sl)
    assert st == 6                                                   # RL_ERR_RANGE, nothing launched
    assert b"built-in array" in _lib.lib().rl_last_error()
    assert _lib.device_error() == 0


def test_sizes_beyond_the_built_in_array_are_refused():
    from rapidllm_b200 import _lib
    q, gate, ks, vs, kp, vp, table, sl = _case(103, [10])
    qd, gd = q.cuda(), gate.cuda()
    st, _ = _noalloc(qd, gd, kp, vp, table, sl, batch=1000)
    assert st == 6                                                   # RL_ERR_RANGE, nothing launched
    assert b"built-in array" in _lib.lib().rl_last_error()
    assert _lib.device_error() == 0
