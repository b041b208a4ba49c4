"""Paged F16 GQA decode attention (CUDA, through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from helpers import ATTN_MAX_ABS, ATTN_REL_L2, paged_from_rows, rel_l2

pytestmark = pytest.mark.gpu

N_Q, N_KV, HD = 24, 4, 256


def _case(gen, lens):
    q = torch.randn(len(lens), N_Q, HD, generator=gen)
    gate = torch.randn(len(lens), N_Q, HD, generator=gen)
    ks = [torch.randn(n, N_KV, HD, generator=gen).half() for n in lens]
    vs = [torch.randn(n, N_KV, HD, generator=gen).half() for n in lens]
    return q, gate, ks, vs


def _oracle(oracle, q, gate, ks, vs):
    out = []
    for b in range(len(ks)):
        if ks[b].shape[0] == 0:
            out.append(np.zeros((N_Q, HD), np.float32))
        else:
            out.append(oracle.gated_attn_decode(q[b].numpy(), ks[b].float().numpy(),
                                                vs[b].float().numpy(), gate[b].numpy()))
    return np.stack(out)


def _check(o, ref):
    o = o.cpu().numpy()
    assert np.isfinite(o).all()
    print("attn max-abs %.3e rel-l2 %.3e" % (np.abs(o - ref).max(), rel_l2(o, ref)))
    assert np.abs(o - ref).max() <= ATTN_MAX_ABS, np.abs(o - ref).max()
    assert rel_l2(o, ref) <= ATTN_REL_L2, rel_l2(o, ref)


def test_config0_ctx4096_batch1(oracle):
    """Batch 1, context 4096, 24Q/4KV, head_dim 256, seed 0, scale 1/16, sigmoid gate."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(0)
    q, gate, ks, vs = _case(gen, [4096])
    kp, vp, table, lens = paged_from_rows(ks, vs, gen)
    o = ops.attn_decode(q.cuda(), kp, vp, table, lens, gate.cuda())
    _lib.check_device()
    ref = _oracle(oracle, q, gate, ks, vs)
    _check(o, ref)
    print("cfg0 max-abs %.3e rel-l2 %.3e" % (np.abs(o.cpu().numpy() - ref).max(), rel_l2(o.cpu().numpy(), ref)))


@pytest.mark.parametrize("chunk_pages", [0, 1, 3])
def test_ragged_edges(oracle, chunk_pages):
    """Contexts 1, 63, 64, 65, 1000, 0 and 130 in one ragged batch, shuffled pages."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(10 + chunk_pages)
    q, gate, ks, vs = _case(gen, [1, 63, 64, 65, 1000, 0, 130])
    kp, vp, table, lens = paged_from_rows(ks, vs, gen)
    o = ops.attn_decode(q.cuda(), kp, vp, table, lens, gate.cuda(), chunk_pages=chunk_pages)
    _lib.check_device()
    _check(o, _oracle(oracle, q, gate, ks, vs))


def test_unused_rows_may_hold_anything(oracle):
    """Rows past a sequence's end (and unowned pages) are NaN: the result must not change."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(3)
    q, gate, ks, vs = _case(gen, [70, 5, 129])
    kp, vp, table, lens = paged_from_rows(ks, vs, gen, fill=float("nan"))
    o = ops.attn_decode(q.cuda(), kp, vp, table, lens, gate.cuda())
    _lib.check_device()
    _check(o, _oracle(oracle, q, gate, ks, vs))


def test_no_gate_and_gqa_group_sizes(oracle):
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(4)
    for n_q, n_kv in [(8, 1), (4, 4), (16, 2)]:
        q = torch.randn(2, n_q, HD, generator=gen)
        ks = [torch.randn(n, n_kv, HD, generator=gen).half() for n in (200, 77)]
        vs = [torch.randn(n, n_kv, HD, generator=gen).half() for n in (200, 77)]
        kp, vp, table, lens = paged_from_rows(ks, vs, gen)
        o = ops.attn_decode(q.cuda(), kp, vp, table, lens, None)
        _lib.check_device()
        ref = np.stack([oracle.attn_decode(q[b].numpy(), ks[b].float().numpy(), vs[b].float().numpy())
                        for b in range(2)])
        _check(o, ref)


def test_paged_indexing_and_append_are_bit_exact(oracle):
    """gather(page table) == the contiguous rows; fp32 rows are rounded to nearest even;
    the pool bytes equal the oracle's scatter into the same layout."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(5)
    n = 64 * 3 + 11
    k32 = torch.randn(n, N_KV, HD, generator=gen)
    v32 = torch.randn(n, N_KV, HD, generator=gen)
    table = torch.randperm(9, generator=gen)[:4].int().cuda()
    kp, vp = ops.new_pool(9, N_KV), ops.new_pool(9, N_KV)
    ops.kv_append(kp, vp, table, k32[:100].cuda(), v32[:100].cuda(), pos0=0)
    pos = torch.tensor([100], dtype=torch.int32, device="cuda")
    ops.kv_append(kp, vp, table, k32[100:].cuda(), v32[100:].cuda(), pos=pos)
    _lib.check_device()
    kg = ops.kv_gather(kp, table, n).cpu().numpy().view(np.uint16)
    vg = ops.kv_gather(vp, table, n).cpu().numpy().view(np.uint16)
    assert np.array_equal(kg, oracle.to_f16(k32.numpy()))
    assert np.array_equal(vg, oracle.to_f16(v32.numpy()))
    # element (tok, d) of a slice sits where kv_slice_index says
    tok = torch.arange(64).view(64, 1).expand(64, HD)
    d = torch.arange(HD).view(1, HD).expand(64, HD)
    idx = ops.kv_slice_index(tok, d).reshape(-1)
    page1 = kp[int(table[1])].cpu()                      # tokens 64..127
    for h in range(N_KV):
        rows = page1[h][idx].reshape(64, HD).numpy().view(np.uint16)
        assert np.array_equal(rows, kg[64:128, h])


def test_partials_merge_to_the_full_result(oracle):
    """Two GPUs' worth of token ranges: partial over each half merged by lse_combine."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(6)
    q, gate, ks, vs = _case(gen, [700, 90])
    cut = [384, 64]
    halves = []
    for part in range(2):
        kr = [k[:c] if part == 0 else k[c:] for k, c in zip(ks, cut)]
        vr = [v[:c] if part == 0 else v[c:] for v, c in zip(vs, cut)]
        kp, vp, table, lens = paged_from_rows(kr, vr, gen)
        halves.append(ops.attn_decode(q.cuda(), kp, vp, table, lens, partial=True))
    part_o = torch.stack([h[0].reshape(-1, HD) for h in halves])
    part_ml = torch.stack([h[1].reshape(-1, 2) for h in halves])
    o = ops.lse_combine(part_o, part_ml, gate.cuda().reshape(-1, HD)).reshape(2, N_Q, HD)
    _lib.check_device()
    _check(o, _oracle(oracle, q, gate, ks, vs))


def test_bad_page_id_is_reported_not_faulted():
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(7)
    q, gate, ks, vs = _case(gen, [100])
    kp, vp, table, lens = paged_from_rows(ks, vs, gen)
    bad = table.clone()
    bad[0, 1] = 10 ** 6
    ops.attn_decode(q.cuda(), kp, vp, bad, lens, gate.cuda())
    assert _lib.device_error() == 1
    assert _lib.device_error() == 0            # cleared
    too_long = torch.tensor([10 ** 6], dtype=torch.int32, device="cuda")
    ops.attn_decode(q.cuda(), kp, vp, table, too_long, gate.cuda())
    assert _lib.device_error() == 5


def test_long_ragged_contexts_split_invariance(oracle):
    """Full-size contexts (8K..32K): the split-KV plan must not change the answer, and
    two sequences are checked against the oracle."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(4)
    lens_l = [32768, 8192, 20001, 12345]
    q, gate, ks, vs = _case(gen, lens_l)
    kp, vp, table, lens = paged_from_rows(ks, vs, gen)
    o1 = ops.attn_decode(q.cuda(), kp, vp, table, lens, gate.cuda())
    o2 = ops.attn_decode(q.cuda(), kp, vp, table, lens, gate.cuda(), chunk_pages=64)
    o3 = ops.attn_decode(q.cuda(), kp, vp, table, lens, gate.cuda(), chunk_pages=5)
    _lib.check_device()
    d2, d3 = rel_l2(o2.cpu().numpy(), o1.cpu().numpy()), rel_l2(o3.cpu().numpy(), o1.cpu().numpy())
    print("split plans differ by rel-l2 %.3e %.3e" % (d2, d3))
    assert d2 <= ATTN_REL_L2 and d3 <= ATTN_REL_L2
    # the same call twice gives the same bits (fixed-order merges)
    o1b = ops.attn_decode(q.cuda(), kp, vp, table, lens, gate.cuda())
    assert torch.equal(o1, o1b)
    for b in (1, 3):
        ref = oracle.gated_attn_decode(q[b].numpy(), ks[b].float().numpy(), vs[b].float().numpy(),
                                       gate[b].numpy())
        _check(o1[b], ref)
