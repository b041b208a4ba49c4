"""Whole decode mixers (rapidllm_b200/mixer.py) against the oracle's restatement of
ops::fused_delta_decode / fused_attn_decode (src/kernels/ops_fused.cpp:84-182), which the CPU suite
pins bit for bit on the reference's outputs.  Model shapes of the operators (16/48 heads of 128,
24/4 heads of 256), a reduced hidden size to keep the oracle's scalar projections short.

Tolerances: the projections run as fp32 library GEMMs (fp32 accumulation in another order than the
oracle's double accumulator) in front of and behind the operators, so the hidden state is compared
with the attention tolerance (max-abs 2e-2, rel-L2 1e-3) per step and the DeltaNet state with
rel-L2 1e-5."""
import numpy as np
import pytest
import torch

from helpers import ATTN_MAX_ABS, ATTN_REL_L2, rel_l2

pytestmark = pytest.mark.gpu

HIDDEN = 512


def _f(rs, *shape):
    return rs.standard_normal(shape).astype(np.float32)


def test_deltanet_mixer_steps(oracle):
    from rapidllm_b200 import _lib
    from rapidllm_b200.mixer import DeltaNetMixer
    torch.backends.cuda.matmul.allow_tf32 = False
    rs = np.random.RandomState(41)
    nk, nv = 16, 48
    cd = 2 * nk * 128 + nv * 128
    w = dict(rms_w=_f(rs, HIDDEN) * 0.1, Wqkv=_f(rs, cd, HIDDEN) / 20, Wz=_f(rs, nv * 128, HIDDEN) / 20,
             Wa=_f(rs, nv, HIDDEN) / 20, Wb=_f(rs, nv, HIDDEN) / 20, Wo=_f(rs, HIDDEN, nv * 128) / 80,
             A_log=_f(rs, nv) * 0.5, dt_bias=_f(rs, nv), conv_w=_f(rs, cd, 4) * 0.5, gnorm=_f(rs, 128))
    for head_map, tiled in ((_lib.RL_HEADS_GROUPED, False), (_lib.RL_HEADS_TILED, True)):
        B = 3
        mix = DeltaNetMixer(w, nk, nv, n_slots=5, head_map=head_map)
        slots = torch.tensor([4, 0, 2], dtype=torch.int32, device="cuda")
        x = _f(rs, B, HIDDEN)
        xd = torch.from_numpy(x).cuda()
        S = [np.zeros((nv, 128, 128), np.float32) for _ in range(B)]
        conv = [np.zeros((cd, 4), np.float32) for _ in range(B)]
        for step in range(4):
            xd = mix.decode(xd, slots)
            _lib.check_device()
            got = xd.cpu().numpy()
            for b in range(B):
                x[b] = oracle.fused_delta_decode(x[b], w, S[b], conv[b], nk, nv, v_tiled=tiled)
                assert np.abs(got[b] - x[b]).max() <= ATTN_MAX_ABS and rel_l2(got[b], x[b]) <= ATTN_REL_L2, \
                    (tiled, step, b, np.abs(got[b] - x[b]).max(), rel_l2(got[b], x[b]))
            xd = torch.from_numpy(x).cuda()          # same inputs every step: errors do not compound
        for b, s in enumerate([4, 0, 2]):
            assert rel_l2(mix.S[s].cpu().numpy(), S[b]) <= 1e-5
            assert np.abs(mix.conv_state[s].cpu().numpy() - conv[b]).max() <= 1e-4
        assert not mix.S[1].any() and not mix.S[3].any()
        print("deltanet mixer tiled=%s: x max-abs %.2e rel-l2 %.2e, S rel-l2 %.2e" %
              (tiled, np.abs(got - x).max(), rel_l2(got, x), rel_l2(mix.S[4].cpu().numpy(), S[0])))


def test_attention_mixer_steps(oracle):
    from rapidllm_b200 import _lib
    from rapidllm_b200.mixer import GatedAttentionMixer
    torch.backends.cuda.matmul.allow_tf32 = False
    rs = np.random.RandomState(42)
    n_q, n_kv, hd = 24, 4, 256
    w = dict(rms_w=_f(rs, HIDDEN) * 0.1, Wq=_f(rs, n_q * 2 * hd, HIDDEN) / 20, Wk=_f(rs, n_kv * hd, HIDDEN) / 20,
             Wv=_f(rs, n_kv * hd, HIDDEN) / 20, Wo=_f(rs, HIDDEN, n_q * hd) / 80, q_norm=_f(rs, hd) * 0.1,
             k_norm=_f(rs, hd) * 0.1)
    B, start = 2, [62, 5000]                      # one sequence crosses a page edge; one far out for RoPE
    max_pages = 80
    mix = GatedAttentionMixer(w, n_pages=B * max_pages + 3)
    perm = torch.randperm(B * max_pages + 3, generator=torch.Generator().manual_seed(1)).int()
    table = perm[:B * max_pages].view(B, max_pages).contiguous().cuda()
    # caches of earlier tokens: random rows in both the oracle's contiguous caches and the pages
    kc = [np.zeros((start[b] + 4, n_kv, hd), np.float32) for b in range(B)]
    vc = [np.zeros((start[b] + 4, n_kv, hd), np.float32) for b in range(B)]
    from rapidllm_b200 import ops
    for b in range(B):
        k0, v0 = _f(rs, start[b], n_kv, hd), _f(rs, start[b], n_kv, hd)
        k0, v0 = k0.astype(np.float16).astype(np.float32), v0.astype(np.float16).astype(np.float32)
        kc[b][:start[b]], vc[b][:start[b]] = k0, v0
        ops.kv_append(mix.k_pool, mix.v_pool, table[b], torch.from_numpy(k0).cuda(), torch.from_numpy(v0).cuda(),
                      pos0=0)
    x = _f(rs, B, HIDDEN)
    for step in range(4):
        pos = [s + step for s in start]
        got = mix.decode(torch.from_numpy(x).cuda(), table, torch.tensor(pos, dtype=torch.int32, device="cuda"))
        _lib.check_device()
        got = got.cpu().numpy()
        for b in range(B):
            x[b] = oracle.fused_attn_decode(x[b], w, kc[b], vc[b], pos[b], n_q, n_kv)
            # the device cache holds fp16 rows: round the oracle's new rows the same way for later steps
            kc[b][pos[b]] = kc[b][pos[b]].astype(np.float16).astype(np.float32)
            vc[b][pos[b]] = vc[b][pos[b]].astype(np.float16).astype(np.float32)
            assert np.abs(got[b] - x[b]).max() <= ATTN_MAX_ABS and rel_l2(got[b], x[b]) <= ATTN_REL_L2, \
                (step, b, np.abs(got[b] - x[b]).max(), rel_l2(got[b], x[b]))
    print("attention mixer: x max-abs %.2e rel-l2 %.2e" % (np.abs(got - x).max(), rel_l2(got, x)))
    # the appended rows equal the oracle's, rounded to fp16
    for b in range(B):
        n = start[b] + 4
        kd = ops.kv_gather(mix.k_pool, table[b], n).float().cpu().numpy()
        assert np.abs(kd - kc[b][:n]).max() <= 2e-3


def test_mixer_stack_two_tokens(oracle):
    """D, D, D, A in layer order for two decode tokens of two sequences: the residual stream after the
    last mixer equals the oracle's fused_delta_decode / fused_attn_decode chained in the same order."""
    from rapidllm_b200 import _lib
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES
    from rapidllm_b200.mixer import MixerStack
    torch.backends.cuda.matmul.allow_tf32 = False
    rs = np.random.RandomState(43)
    nk, nv, n_q, n_kv, hd = 16, 48, 24, 4, 256
    cd = 2 * nk * 128 + nv * 128
    weights = []
    for kind in QWEN35_LAYER_TYPES:
        if kind == _lib.RL_LAYER_FULL_ATTENTION:
            weights.append(dict(rms_w=_f(rs, HIDDEN) * 0.1, Wq=_f(rs, n_q * 2 * hd, HIDDEN) / 20,
                                Wk=_f(rs, n_kv * hd, HIDDEN) / 20, Wv=_f(rs, n_kv * hd, HIDDEN) / 20,
                                Wo=_f(rs, HIDDEN, n_q * hd) / 80, q_norm=_f(rs, hd) * 0.1, k_norm=_f(rs, hd) * 0.1))
        else:
            weights.append(dict(rms_w=_f(rs, HIDDEN) * 0.1, Wqkv=_f(rs, cd, HIDDEN) / 20,
                                Wz=_f(rs, nv * 128, HIDDEN) / 20, Wa=_f(rs, nv, HIDDEN) / 20,
                                Wb=_f(rs, nv, HIDDEN) / 20, Wo=_f(rs, HIDDEN, nv * 128) / 80, A_log=_f(rs, nv) * 0.5,
                                dt_bias=_f(rs, nv), conv_w=_f(rs, cd, 4) * 0.5, gnorm=_f(rs, 128)))
    B, max_pages = 2, 2
    stack = MixerStack(QWEN35_LAYER_TYPES, weights, n_pages=B * max_pages, n_slots=B)
    table = torch.arange(B * max_pages, dtype=torch.int32).view(B, max_pages).cuda()
    S = [[np.zeros((nv, 128, 128), np.float32) for _ in range(B)] for _ in range(3)]
    conv = [[np.zeros((cd, 4), np.float32) for _ in range(B)] for _ in range(3)]
    kc = [np.zeros((4, n_kv, hd), np.float32) for _ in range(B)]
    vc = [np.zeros((4, n_kv, hd), np.float32) for _ in range(B)]
    for pos in range(2):
        x = _f(rs, B, HIDDEN)
        got = stack.decode(torch.from_numpy(x).cuda(), table,
                           torch.full((B,), pos, dtype=torch.int32, device="cuda")).cpu().numpy()
        _lib.check_device()
        for b in range(B):
            xb, d = x[b], 0
            for kind, w in zip(QWEN35_LAYER_TYPES, weights):
                if kind == _lib.RL_LAYER_FULL_ATTENTION:
                    xb = oracle.fused_attn_decode(xb, w, kc[b], vc[b], pos, n_q, n_kv)
                    kc[b][pos] = kc[b][pos].astype(np.float16).astype(np.float32)
                    vc[b][pos] = vc[b][pos].astype(np.float16).astype(np.float32)
                else:
                    xb = oracle.fused_delta_decode(xb, w, S[d][b], conv[d][b], nk, nv)
                    d += 1
            assert np.abs(got[b] - xb).max() <= ATTN_MAX_ABS and rel_l2(got[b], xb) <= ATTN_REL_L2, \
                (pos, b, np.abs(got[b] - xb).max(), rel_l2(got[b], xb))
    print("mixer stack: x max-abs %.2e rel-l2 %.2e" % (np.abs(got[b] - xb).max(), rel_l2(got[b], xb)))


def test_mixers_prefill_chunks(oracle):
    """Prompt chunks through each mixer (chunked delta rule / tensor-core attention) against the oracle's
    decode mixers run token by token."""
    from rapidllm_b200 import _lib
    from rapidllm_b200.mixer import DeltaNetMixer, GatedAttentionMixer
    torch.backends.cuda.matmul.allow_tf32 = False
    rs = np.random.RandomState(44)
    nk, nv, n_q, n_kv, hd = 16, 48, 24, 4, 256
    cd = 2 * nk * 128 + nv * 128
    wd = dict(rms_w=_f(rs, HIDDEN) * 0.1, Wqkv=_f(rs, cd, HIDDEN) / 20, Wz=_f(rs, nv * 128, HIDDEN) / 20,
              Wa=_f(rs, nv, HIDDEN) / 20, Wb=_f(rs, nv, HIDDEN) / 20, Wo=_f(rs, HIDDEN, nv * 128) / 80,
              A_log=_f(rs, nv) * 0.5, dt_bias=_f(rs, nv), conv_w=_f(rs, cd, 4) * 0.5, gnorm=_f(rs, 128))
    wa = dict(rms_w=_f(rs, HIDDEN) * 0.1, Wq=_f(rs, n_q * 2 * hd, HIDDEN) / 20, Wk=_f(rs, n_kv * hd, HIDDEN) / 20,
              Wv=_f(rs, n_kv * hd, HIDDEN) / 20, Wo=_f(rs, HIDDEN, n_q * hd) / 80, q_norm=_f(rs, hd) * 0.1,
              k_norm=_f(rs, hd) * 0.1)
    chunks = [70, 31]
    T = sum(chunks)
    x = _f(rs, T, HIDDEN)
    dm = DeltaNetMixer(wd, nk, nv, n_slots=2)
    am = GatedAttentionMixer(wa, n_pages=3)
    row = torch.tensor([2, 0, 1], dtype=torch.int32).cuda()
    got_d, got_a, p0 = [], [], 0
    for n in chunks:
        xc = torch.from_numpy(x[p0:p0 + n]).cuda()
        got_d.append(dm.prefill(xc, slot=1, start=p0 == 0).cpu().numpy())
        got_a.append(am.prefill(xc, row, p0).cpu().numpy())
        _lib.check_device()
        p0 += n
    got_d, got_a = np.concatenate(got_d), np.concatenate(got_a)
    S, conv = np.zeros((nv, 128, 128), np.float32), np.zeros((cd, 4), np.float32)
    kc, vc = np.zeros((T, n_kv, hd), np.float32), np.zeros((T, n_kv, hd), np.float32)
    ref_d, ref_a = np.empty_like(x), np.empty_like(x)
    for t in range(T):
        ref_d[t] = oracle.fused_delta_decode(x[t], wd, S, conv, nk, nv)
        ref_a[t] = oracle.fused_attn_decode(x[t], wa, kc, vc, t, n_q, n_kv)
        kc[t], vc[t] = kc[t].astype(np.float16).astype(np.float32), vc[t].astype(np.float16).astype(np.float32)
    for name, got, ref in (("deltanet", got_d, ref_d), ("attention", got_a, ref_a)):
        print("%s mixer prefill: x max-abs %.2e rel-l2 %.2e" % (name, np.abs(got - ref).max(), rel_l2(got, ref)))
        assert np.abs(got - ref).max() <= ATTN_MAX_ABS and rel_l2(got, ref) <= ATTN_REL_L2
    assert rel_l2(dm.S[1].cpu().numpy(), S) <= 1e-3           # chunked form: fp16 hi + lo operands
    assert not dm.S[0].any()
