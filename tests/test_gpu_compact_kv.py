"""q8-K + TurboQuant-3-V compact cache: bit-exact codes and decode attention vs the oracle
(the CPU restatement of the reference's CUDA store/dequant math; no reference test pins it)."""
import numpy as np
import pytest
import torch

from helpers import ATTN_MAX_ABS, ATTN_REL_L2, rel_l2

pytestmark = pytest.mark.gpu

N_Q, N_KV, HD = 24, 4, 256


def _signs(gen):
    return (2.0 * torch.bernoulli(torch.full((256,), 0.5), generator=gen) - 1.0).float()


def _table(lens, gen, extra=2):
    pages = [(n + 63) // 64 for n in lens]
    n_pages = sum(pages) + extra
    perm = torch.randperm(n_pages, generator=gen).int()
    table = torch.zeros(len(lens), max(1, max(pages)), dtype=torch.int32)
    at = 0
    for b, p in enumerate(pages):
        table[b, :p] = perm[at:at + p]
        at += p
    return table.cuda(), n_pages


@pytest.mark.parametrize("wht_len,use_signs", [(128, False), (256, True)])
def test_codes_are_bit_exact(oracle, wht_len, use_signs):
    """Store (prefill rows, then single-token appends) -> gather == oracle codes and scales."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(2)
    n = 64 * 2 + 37
    k = torch.randn(n, N_KV, HD, generator=gen)
    v = torch.randn(n, N_KV, HD, generator=gen)
    k[3] *= 1e-3                                   # small rows, a zero row, an outlier
    v[5] = 0.0
    k[7, 1, 11] = 40.0
    signs = _signs(gen) if use_signs else None
    sd = signs.cuda() if use_signs else None
    table, n_pages = _table([n], gen)
    pool = ops.new_compact_pool(n_pages, N_KV)
    ops.kv_compact_append(pool, table, k[:101].cuda(), v[:101].cuda(), wht_len, sd, pos0=0)
    for t in range(101, n):                        # decode-style appends, device-resident position
        pos = torch.tensor([t], dtype=torch.int32, device="cuda")
        ops.kv_compact_append(pool, table, k[t:t + 1].cuda(), v[t:t + 1].cuda(), wht_len, sd, pos=pos)
    _lib.check_device()
    k_q, k_sc, v_codes, v_sc = ops.kv_compact_gather(pool, table[0], n, wht_len)
    rk_q, rk_sc, rv_codes, rv_sc = oracle.compact_store(k.numpy(), v.numpy(), wht_len,
                                                        None if signs is None else signs.numpy())
    assert np.array_equal(k_q.cpu().numpy(), rk_q)
    assert np.array_equal(k_sc.cpu().numpy().view(np.uint16), rk_sc)
    assert np.array_equal(v_sc.cpu().numpy().view(np.uint16), rv_sc)
    assert np.array_equal(v_codes.cpu().numpy(), rv_codes)
    # overwriting a token leaves its pair partner untouched
    ops.kv_compact_append(pool, table, k[10:11].cuda(), v[10:11].cuda(), wht_len, sd, pos0=10)
    again = ops.kv_compact_gather(pool, table[0], n, wht_len)
    assert torch.equal(again[2], v_codes) and torch.equal(again[0], k_q)


@pytest.mark.parametrize("wht_len,use_signs,lens", [
    (128, False, [1, 31, 32, 33, 64, 65, 700, 0, 1000]),
    (256, True, [1, 31, 32, 33, 64, 65, 700, 0, 1000]),
    # long sequences: every head spreads over tens of CTAs, and the CTAs whose range runs over a
    # (sequence, head) boundary own fewer records than the others
    (128, False, [9000, 40, 0, 13000, 6001]),
])
def test_decode_over_compact_cache(oracle, wht_len, use_signs, lens):
    """Ragged batch; oracle = dequantise (per-token inverse transform) -> ops::attn_decode -> gate."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(22)
    signs = _signs(gen) if use_signs else None
    sd = signs.cuda() if use_signs else None
    q = torch.randn(len(lens), N_Q, HD, generator=gen)
    gate = torch.randn(len(lens), N_Q, HD, generator=gen)
    ks = [torch.randn(n, N_KV, HD, generator=gen) for n in lens]
    vs = [torch.randn(n, N_KV, HD, generator=gen) for n in lens]
    table, n_pages = _table(lens, gen)
    pool = ops.new_compact_pool(n_pages, N_KV)
    pool.fill_(0xFF)                               # unused rows hold NaN scales / arbitrary codes
    for b, n in enumerate(lens):
        if n:
            ops.kv_compact_append(pool, table[b], ks[b].cuda(), vs[b].cuda(), wht_len, sd, pos0=0)
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    outs = [ops.attn_decode(q.cuda(), pool, None, table, sl, gate.cuda(), wht_len=wht_len, signs=sd,
                            chunk_pages=cp) for cp in (0, 1, 4)]
    _lib.check_device()
    sn = None if signs is None else signs.numpy()
    for b, n in enumerate(lens):
        if n == 0:
            assert not outs[0][b].any()
            continue
        kd, vd = oracle.compact_dequant(*oracle.compact_store(ks[b].numpy(), vs[b].numpy(), wht_len, sn),
                                        wht_len, sn)
        ref = oracle.gated_attn_decode(q[b].numpy(), kd, vd, gate[b].numpy())
        for o in outs:
            ob = o[b].cpu().numpy()
            assert np.isfinite(ob).all()
            assert np.abs(ob - ref).max() <= ATTN_MAX_ABS, (b, np.abs(ob - ref).max())
            assert rel_l2(ob, ref) <= ATTN_REL_L2, (b, rel_l2(ob, ref))
        print("compact decode wht%d len %d: max-abs %.3e rel-l2 %.3e" %
              (wht_len, n, np.abs(outs[0][b].cpu().numpy() - ref).max(), rel_l2(outs[0][b].cpu().numpy(), ref)))


def test_compact_partials_merge_across_token_ranges(oracle):
    """Split-KV across two 'GPUs': rotated-domain partials merged by lse_combine(wht_len)."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(23)
    n, cut = 500, 256
    q = torch.randn(1, N_Q, HD, generator=gen)
    gate = torch.randn(1, N_Q, HD, generator=gen)
    k = torch.randn(n, N_KV, HD, generator=gen)
    v = torch.randn(n, N_KV, HD, generator=gen)
    parts = []
    for a, b in ((0, cut), (cut, n)):
        table, n_pages = _table([b - a], gen)
        pool = ops.new_compact_pool(n_pages, N_KV)
        ops.kv_compact_append(pool, table[0], k[a:b].cuda(), v[a:b].cuda(), 128, None, pos0=0)
        parts.append(ops.attn_decode(q.cuda(), pool, None, table,
                                     torch.tensor([b - a], dtype=torch.int32, device="cuda"), partial=True))
    po = torch.stack([p[0].reshape(-1, HD) for p in parts])
    pml = torch.stack([p[1].reshape(-1, 2) for p in parts])
    o = ops.lse_combine(po, pml, gate.cuda().reshape(-1, HD), wht_len=128).cpu().numpy()
    _lib.check_device()
    kd, vd = oracle.compact_dequant(*oracle.compact_store(k.numpy(), v.numpy(), 128), 128)
    ref = oracle.gated_attn_decode(q[0].numpy(), kd, vd, gate[0].numpy())
    assert np.abs(o - ref).max() <= ATTN_MAX_ABS and rel_l2(o, ref) <= ATTN_REL_L2


@pytest.mark.parametrize("wht_len,use_signs", [(128, False), (256, True)])
def test_f16_window_rebuilt_from_compact_cache_and_prefill_over_it(oracle, wht_len, use_signs):
    """The compact cache persists; a prefill chunk (or verify rows) attends over an F16 window
    dequantised from it (rl_kv_compact_to_f16), as the reference rebuilds its compute window."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(8)
    n_old, n_new = 64 * 3 + 21, 40
    k = torch.randn(n_old, N_KV, HD, generator=gen)
    v = torch.randn(n_old, N_KV, HD, generator=gen)
    signs = _signs(gen) if use_signs else None
    sd = signs.cuda() if use_signs else None
    table, n_pages = _table([n_old], gen)
    pool = ops.new_compact_pool(n_pages, N_KV)
    ops.kv_compact_append(pool, table, k.cuda(), v.cuda(), wht_len, sd, pos0=0)
    # window: its own F16 pools and page table, rebuilt in two pieces (page-unaligned split)
    wt, wn = _table([n_old + n_new], gen)
    kp, vp = ops.new_pool(wn, N_KV), ops.new_pool(wn, N_KV)
    ops.kv_compact_to_f16(pool, table[0], kp, vp, wt[0], 100, 0, 0, wht_len, sd)
    ops.kv_compact_to_f16(pool, table[0], kp, vp, wt[0], n_old - 100, 100, 100, wht_len, sd)
    _lib.check_device()
    kw = ops.kv_gather(kp, wt[0], n_old).cpu().float().numpy()
    vw = ops.kv_gather(vp, wt[0], n_old).cpu().float().numpy()
    sn = None if signs is None else signs.numpy()
    kd, vd = oracle.compact_dequant(*oracle.compact_store(k.numpy(), v.numpy(), wht_len, sn), wht_len, sn)
    # fp16 of the oracle's fp32 dequantisation; the transform's summation order may move a value
    # across an fp16 rounding boundary: allow one fp16 ulp (2^-10 relative, 2^-24 absolute floor)
    assert np.array_equal(kw, kd.astype(np.float16).astype(np.float32))      # K: one exact product
    ulp = np.maximum(np.abs(vd) * 2.0 ** -10, 2.0 ** -24)
    assert (np.abs(vw - vd) <= ulp).all()
    # a prefill chunk over the rebuilt window == the oracle over the dequantised cache + the new rows
    q = torch.randn(n_new, N_Q, HD, generator=gen).bfloat16()
    k2 = torch.randn(n_new, N_KV, HD, generator=gen).bfloat16()
    v2 = torch.randn(n_new, N_KV, HD, generator=gen).bfloat16()
    o = ops.attn_prefill(q.cuda(), kp, vp, wt[0], n_old, k2.cuda(), v2.cuda(), None)
    _lib.check_device()
    k_all = np.concatenate([kd, k2.float().numpy()])
    v_all = np.concatenate([vd, v2.float().numpy()])
    ref = oracle.attn_prefill_rows(q.float().numpy(), k_all, v_all, np.arange(n_old, n_old + n_new))
    o = o.cpu().numpy()
    assert np.abs(o - ref).max() <= ATTN_MAX_ABS and rel_l2(o, ref) <= ATTN_REL_L2


def test_config2_full_size_batch4_ctx131072(oracle):
    """Batch 4 x 131 072 tokens in the 256-point / sign-vector layout, seed 2.  Sequence 0 goes through the
    oracle whole (codes bit for bit, then the decode output); all four are checked through properties
    that do not need the oracle: the division of the KV range must not change the answer, the same call
    gives the same bits twice, and the F16 kernel over a window dequantised from the same cache (an
    independent code path from the stored bytes on) agrees within the attention tolerance."""
    from rapidllm_b200 import _lib, ops
    B, n, wht_len = 4, 131072, 256
    gen = torch.Generator().manual_seed(2)
    signs = _signs(gen)
    sd = signs.cuda()
    q = torch.randn(B, N_Q, HD, generator=gen)
    gate = torch.randn(B, N_Q, HD, generator=gen)
    table, n_pages = _table([n] * B, gen)
    wt, wn = _table([n] * B, gen)
    pool = ops.new_compact_pool(n_pages, N_KV)
    kp, vp = ops.new_pool(wn, N_KV), ops.new_pool(wn, N_KV)
    dgen = torch.Generator(device="cuda").manual_seed(2)
    k0 = v0 = None
    for b in range(B):
        k = torch.randn(n, N_KV, HD, generator=dgen, device="cuda")
        v = torch.randn(n, N_KV, HD, generator=dgen, device="cuda")
        ops.kv_compact_append(pool, table[b], k, v, wht_len, sd, pos0=0)
        ops.kv_compact_to_f16(pool, table[b], kp, vp, wt[b], n, 0, 0, wht_len, sd)
        if b == 0:
            k0, v0 = k.cpu().numpy(), v.cpu().numpy()
        del k, v
    _lib.check_device()
    sl = torch.full((B,), n, dtype=torch.int32, device="cuda")
    o = ops.attn_decode(q.cuda(), pool, None, table, sl, gate.cuda(), wht_len=wht_len, signs=sd)
    o_again = ops.attn_decode(q.cuda(), pool, None, table, sl, gate.cuda(), wht_len=wht_len, signs=sd)
    o_cut = ops.attn_decode(q.cuda(), pool, None, table, sl, gate.cuda(), wht_len=wht_len, signs=sd, chunk_pages=64)
    o_f16 = ops.attn_decode(q.cuda(), kp, vp, wt, sl, gate.cuda())
    _lib.check_device()
    assert torch.equal(o, o_again)
    o, o_cut, o_f16 = o.cpu().numpy(), o_cut.cpu().numpy(), o_f16.cpu().numpy()
    assert np.isfinite(o).all()
    for b in range(B):
        assert rel_l2(o_cut[b], o[b]) <= ATTN_REL_L2
        assert np.abs(o_f16[b] - o[b]).max() <= ATTN_MAX_ABS and rel_l2(o_f16[b], o[b]) <= ATTN_REL_L2, \
            (b, np.abs(o_f16[b] - o[b]).max(), rel_l2(o_f16[b], o[b]))
    print("config 2: compact vs F16-window decode rel-l2 %s" % [float("%.2e" % rel_l2(o_f16[b], o[b])) for b in range(B)])
    # sequence 0 against the oracle
    rk_q, rk_sc, rv_codes, rv_sc = oracle.compact_store(k0, v0, wht_len, signs.numpy())
    k_q, k_sc, v_codes, v_sc = ops.kv_compact_gather(pool, table[0], n, wht_len)
    assert np.array_equal(k_q.cpu().numpy(), rk_q)
    assert np.array_equal(k_sc.cpu().numpy().view(np.uint16), rk_sc)
    assert np.array_equal(v_sc.cpu().numpy().view(np.uint16), rv_sc)
    assert np.array_equal(v_codes.cpu().numpy(), rv_codes)
    kd, vd = oracle.compact_dequant(rk_q, rk_sc, rv_codes, rv_sc, wht_len, signs.numpy())
    ref = oracle.gated_attn_decode(q[0].numpy(), kd, vd, gate[0].numpy())
    err, rl = np.abs(o[0] - ref).max(), rel_l2(o[0], ref)
    print("config 2: sequence 0 vs oracle max-abs %.3e rel-l2 %.3e" % (err, rl))
    assert err <= ATTN_MAX_ABS and rl <= ATTN_REL_L2
