"""Chunked causal attention prefill (tcgen05 kernel, through the C ABI) against the oracle."""
import numpy as np
import pytest
import torch

from helpers import ATTN_MAX_ABS, ATTN_REL_L2, rel_l2

pytestmark = pytest.mark.gpu

N_Q, N_KV, HD = 24, 4, 256


def _inputs(gen, T):
    q = torch.randn(T, N_Q, HD, generator=gen).bfloat16()
    k = torch.randn(T, N_KV, HD, generator=gen).bfloat16()
    v = torch.randn(T, N_KV, HD, generator=gen).bfloat16()
    gate = torch.randn(T, N_Q, HD, generator=gen)
    return q, k, v, gate


def _check(o, ref, what=""):
    o = o.cpu().numpy() if hasattr(o, "cpu") else o
    assert np.isfinite(o).all()
    e, r = np.abs(o - ref).max(), rel_l2(o, ref)
    print("prefill %s max-abs %.3e rel-l2 %.3e" % (what, e, r))
    assert e <= ATTN_MAX_ABS and r <= ATTN_REL_L2, (what, e, r)


@pytest.mark.parametrize("T", [1, 64, 129, 200])
def test_whole_sequence_small(oracle, T):
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(30 + T)
    q, k, v, gate = _inputs(gen, T)
    n_pages = (T + 63) // 64 + 2
    table = torch.randperm(n_pages, generator=gen)[:(T + 63) // 64].int().cuda()
    kp, vp = ops.new_pool(n_pages, N_KV), ops.new_pool(n_pages, N_KV)
    kp.fill_(float("nan"))                      # rows past the end hold NaN
    vp.fill_(float("nan"))
    o = ops.attn_prefill(q.cuda(), kp, vp, table, 0, k.cuda(), v.cuda(), gate.cuda())
    _lib.check_device()
    ref = oracle.attn_prefill(q.float().numpy(), k.float().numpy(), v.float().numpy())
    ref = oracle.sigmoid_gate(ref, gate.numpy())
    _check(o, ref, "T=%d" % T)
    # the cache now holds the chunk's rows: bf16 -> fp16, round to nearest even (exact unless
    # the value is below the fp16 normal range)
    kg = ops.kv_gather(kp, table, T).cpu()
    assert torch.equal(kg, k.float().half())


def test_chunks_over_an_existing_cache(oracle):
    """Three chunks (300 + 150 + 77 rows): each attends to everything cached before it."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(31)
    T = 527
    q, k, v, gate = _inputs(gen, T)
    n_pages = 12
    table = torch.randperm(n_pages, generator=gen)[:9].int().cuda()
    kp, vp = ops.new_pool(n_pages, N_KV), ops.new_pool(n_pages, N_KV)
    outs, pos = [], 0
    for n in (300, 150, 77):
        sl = slice(pos, pos + n)
        outs.append(ops.attn_prefill(q[sl].cuda(), kp, vp, table, pos, k[sl].cuda(), v[sl].cuda(),
                                     gate[sl].cuda()))
        pos += n
    _lib.check_device()
    o = torch.cat(outs).cpu().numpy()
    ref = oracle.sigmoid_gate(oracle.attn_prefill(q.float().numpy(), k.float().numpy(), v.float().numpy()),
                              gate.numpy())
    _check(o, ref, "3 chunks")
    # decode over the same cache agrees with the last prefill row
    lens = torch.tensor([T], dtype=torch.int32, device="cuda")
    od = ops.attn_decode(q[-1:].float().cuda(), kp, vp, table.unsqueeze(0), lens, gate[-1:].cuda())
    assert rel_l2(od[0].cpu().numpy(), o[-1]) < ATTN_REL_L2


@pytest.mark.parametrize("n_draft", [2, 4, 12])
def test_speculative_verify_rows_over_a_cache(oracle, n_draft):
    """The verify pass of speculative decode (Engine::spec_verify, cuda_engine.h:69-77): a handful
    of drafted tokens at positions pos0 .. pos0 + T - 1 attend causally over the cache and one
    another; rejected tokens are simply overwritten by the next append at the rolled-back position."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(50 + n_draft)
    pos0 = 1000 - n_draft // 2                   # straddles a page boundary for the larger drafts
    T = pos0 + n_draft
    q, k, v, gate = _inputs(gen, T)
    n_pages = 20
    table = torch.randperm(n_pages, generator=gen)[:17].int().cuda()
    kp, vp = ops.new_pool(n_pages, N_KV), ops.new_pool(n_pages, N_KV)
    ops.kv_append(kp, vp, table, k[:pos0].half().cuda(), v[:pos0].half().cuda(), pos0=0)
    o = ops.attn_prefill(q[pos0:].cuda(), kp, vp, table, pos0, k[pos0:].cuda(), v[pos0:].cuda(), gate[pos0:].cuda())
    _lib.check_device()
    ref = oracle.attn_prefill_rows(q[pos0:].float().numpy(), k.float().numpy(), v.float().numpy(), np.arange(pos0, T))
    ref = oracle.sigmoid_gate(ref, gate[pos0:].numpy())
    _check(o, ref, "verify %d" % n_draft)
    # accept only the first token: the next decode step appends at pos0 + 1 and must not see the
    # rejected rows
    k_new = torch.randn(1, N_KV, HD, generator=gen)
    v_new = torch.randn(1, N_KV, HD, generator=gen)
    ops.kv_append(kp, vp, table, k_new.half().cuda(), v_new.half().cuda(), pos0=pos0 + 1)
    lens = torch.tensor([pos0 + 2], dtype=torch.int32, device="cuda")
    qd = torch.randn(1, N_Q, HD, generator=gen)
    od = ops.attn_decode(qd.cuda(), kp, vp, table.unsqueeze(0), lens, None)
    kk = torch.cat([k[:pos0 + 1].float().half().float(), k_new.half().float()]).numpy()
    vv = torch.cat([v[:pos0 + 1].float().half().float(), v_new.half().float()]).numpy()
    ref_d = oracle.attn_decode(qd[0].numpy(), kk, vv)
    assert rel_l2(od[0].cpu().numpy(), ref_d) <= ATTN_REL_L2


def test_config3_8192_tokens_sampled_rows(oracle):
    """8192-token prefill in 1024-row chunks; a strided sample of rows against the oracle."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(3)
    T = 8192
    q, k, v, gate = _inputs(gen, T)
    n_pages = T // 64
    table = torch.randperm(n_pages, generator=gen).int().cuda()
    kp, vp = ops.new_pool(n_pages, N_KV), ops.new_pool(n_pages, N_KV)
    outs = []
    for p0 in range(0, T, 1024):
        sl = slice(p0, p0 + 1024)
        outs.append(ops.attn_prefill(q[sl].cuda(), kp, vp, table, p0, k[sl].cuda(), v[sl].cuda(), gate[sl].cuda()))
    _lib.check_device()
    o = torch.cat(outs).cpu().numpy()
    # 192 (query tile, head) items per chunk on 148 SMs: the lowest query tiles of the last KV head are
    # the ones whose KV range is divided (rows 0-255 of a chunk, more parts the longer the cache)
    rows = np.array([0, 1, 63, 64, 127, 128, 1000, 1023, 1024, 1100, 2053, 3272, 4095, 5000, 7168 + 130, 7168 + 255,
                     7168 + 256, 8191], np.int32)
    ref = oracle.attn_prefill_rows(q[rows].float().numpy(), k.float().numpy(), v.float().numpy(), rows)
    ref = oracle.sigmoid_gate(ref, gate[rows].numpy())
    _check(o[rows], ref, "cfg3 rows")


def test_two_chunks_of_4096_sampled_rows(oracle):
    """768 (query tile, head) items per chunk = five full waves of 148 + 28: the second chunk runs those 28
    (the lowest query tiles of the last KV head) divided in parts; sampled rows inside and outside them."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(33)
    T = 8192
    q, k, v, gate = _inputs(gen, T)
    n_pages = T // 64
    table = torch.randperm(n_pages, generator=gen).int().cuda()
    kp, vp = ops.new_pool(n_pages, N_KV), ops.new_pool(n_pages, N_KV)
    outs = []
    for p0 in range(0, T, 4096):
        sl = slice(p0, p0 + 4096)
        outs.append(ops.attn_prefill(q[sl].cuda(), kp, vp, table, p0, k[sl].cuda(), v[sl].cuda(), gate[sl].cuda()))
    _lib.check_device()
    o = torch.cat(outs).cpu().numpy()
    rows = np.array([0, 640, 4095, 4096, 4100, 4223, 4500, 4735, 4736, 6000, 8191], np.int32)
    ref = oracle.attn_prefill_rows(q[rows].float().numpy(), k.float().numpy(), v.float().numpy(), rows)
    ref = oracle.sigmoid_gate(ref, gate[rows].numpy())
    _check(o[rows], ref, "2 x 4096 rows")
