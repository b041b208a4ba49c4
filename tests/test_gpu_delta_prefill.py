"""Chunked (WY-form) DeltaNet prefill on the tensor cores against T sequential oracle steps
(the reference's only prefill form is the token-by-token recurrence)."""
import numpy as np
import pytest
import torch

from helpers import rel_l2, softplus

pytestmark = pytest.mark.gpu

N_V, N_K, D = 48, 16, 128
# chunked form: operands pass through fp16 (state and deltas as hi + lo pairs)
OUT_REL_L2 = 1e-3
OUT_MAX_ABS = 2e-2
STATE_REL_L2 = 1e-5   # the FP32-state bound


def _inputs(gen, T, n_v=N_V, n_k=N_K, s0_scale=0.02):
    S0 = torch.randn(n_v, D, D, generator=gen) * s0_scale
    q = torch.randn(T, n_k, D, generator=gen)
    k = torch.randn(T, n_k, D, generator=gen)
    v = torch.randn(T, n_v, D, generator=gen)
    beta = torch.sigmoid(torch.randn(T, n_v, generator=gen))
    g = -softplus(torch.randn(T, n_v, generator=gen))
    return S0, q, k, v, beta, g


def _oracle(oracle, S0, q, k, v, beta, g, tiled=False):
    n_v = S0.shape[0]
    S = S0.numpy().copy()
    T = q.shape[0]
    qq = np.stack([oracle.repeat_heads(q[t].numpy(), n_v, tiled) for t in range(T)])
    kk = np.stack([oracle.repeat_heads(k[t].numpy(), n_v, tiled) for t in range(T)])
    o = oracle.delta_prefill_seq(S, qq, kk, v.numpy(), beta.numpy(), g.numpy())
    return o, S


@pytest.mark.parametrize("T", [1, 64, 65, 200])
def test_small_sequences(oracle, T):
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(40 + T)
    S0, q, k, v, beta, g = _inputs(gen, T)
    S = S0.cuda().clone()
    o = ops.delta_chunk_prefill(S, q.cuda(), k.cuda(), v.cuda(), beta.cuda(), g.cuda())
    _lib.check_device()
    oref, Sref = _oracle(oracle, S0, q, k, v, beta, g)
    eo, ro, rs = np.abs(o.cpu().numpy() - oref).max(), rel_l2(o.cpu().numpy(), oref), rel_l2(S.cpu().numpy(), Sref)
    print("delta chunk T=%d: o max-abs %.3e rel-l2 %.3e, state rel-l2 %.3e" % (T, eo, ro, rs))
    assert np.isfinite(o.cpu().numpy()).all()
    assert eo <= OUT_MAX_ABS and ro <= OUT_REL_L2 and rs <= STATE_REL_L2


def test_prefill_then_decode_hands_over_the_state(oracle):
    """prefill(300) followed by 20 decode steps == 320 sequential oracle steps (tiled head map)."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(41)
    T, n = 300, 20
    S0, q, k, v, beta, g = _inputs(gen, T + n)
    S = S0.cuda().clone()
    o1 = ops.delta_chunk_prefill(S, q[:T].cuda(), k[:T].cuda(), v[:T].cuda(), beta[:T].cuda(), g[:T].cuda(),
                                 head_map=_lib.RL_HEADS_TILED)
    outs = []
    for t in range(T, T + n):
        outs.append(ops.delta_recurrent_step(S.unsqueeze(0), q[t:t + 1].cuda(), k[t:t + 1].cuda(), v[t:t + 1].cuda(),
                                             beta[t:t + 1].cuda(), g[t:t + 1].cuda(), head_map=_lib.RL_HEADS_TILED))
    _lib.check_device()
    o = torch.cat([o1] + outs).cpu().numpy()
    oref, Sref = _oracle(oracle, S0, q, k, v, beta, g, tiled=True)
    assert rel_l2(o, oref) <= OUT_REL_L2 and np.abs(o - oref).max() <= OUT_MAX_ABS
    assert rel_l2(S.cpu().numpy(), Sref) <= STATE_REL_L2


def test_strong_decay_and_per_value_heads(oracle):
    """Log decays down to -8 per token (exp(G) underflows to ~1e-200 over a chunk in double, 0 in
    fp32): the chunked form must stay finite and accurate."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(42)
    T, n_v = 130, 6
    S0, q, k, v, beta, g = _inputs(gen, T, n_v=n_v, n_k=n_v, s0_scale=1.0)
    g = g * 6.0
    S = S0.cuda().clone()
    o = ops.delta_chunk_prefill(S, q.cuda(), k.cuda(), v.cuda(), beta.cuda(), g.cuda())
    _lib.check_device()
    oref, Sref = _oracle(oracle, S0, q, k, v, beta, g)
    assert np.isfinite(o.cpu().numpy()).all() and np.isfinite(S.cpu().numpy()).all()
    assert rel_l2(o.cpu().numpy(), oref) <= OUT_REL_L2 and rel_l2(S.cpu().numpy(), Sref) <= STATE_REL_L2


def test_config3_8192_tokens(oracle):
    """16 K / 48 V heads, 8192 tokens from a zero state, seed 3: outputs and the final FP32 state."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(3)
    T = 8192
    S0, q, k, v, beta, g = _inputs(gen, T, s0_scale=0.0)
    S = S0.cuda().clone()
    o = ops.delta_chunk_prefill(S, q.cuda(), k.cuda(), v.cuda(), beta.cuda(), g.cuda())
    _lib.check_device()
    oref, Sref = _oracle(oracle, S0, q, k, v, beta, g)
    o = o.cpu().numpy()
    print("delta chunk cfg3: o max-abs %.3e rel-l2 %.3e, state rel-l2 %.3e" %
          (np.abs(o - oref).max(), rel_l2(o, oref), rel_l2(S.cpu().numpy(), Sref)))
    assert rel_l2(o, oref) <= OUT_REL_L2 and np.abs(o - oref).max() <= OUT_MAX_ABS
    assert rel_l2(S.cpu().numpy(), Sref) <= STATE_REL_L2
