"""Gated DeltaNet decode step and causal conv1d (CUDA, through the C ABI) against the oracle."""
import numpy as np
import pytest
import torch

from helpers import STATE_REL_L2, rel_l2, softplus

pytestmark = pytest.mark.gpu

N_V, N_K, DK, DV, CONV_DIM, CONV_K = 48, 16, 128, 128, 10240, 4


def test_config1_1024_steps_with_conv(oracle):
    """16 K / 48 V heads, FP32 S ~ N(0, 0.02), conv k=4 over 10240 channels, 1024
    consecutive steps from seed 1: state rel-L2 <= 1e-5, outputs max-abs <= 1e-4."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(1)
    S0 = torch.randn(N_V, DK, DV, generator=gen) * 0.02
    w = torch.randn(CONV_DIM, CONV_K, generator=gen) * 0.5
    steps = 1024
    xs = torch.randn(steps, CONV_DIM, generator=gen)
    beta = torch.sigmoid(torch.randn(steps, N_V, generator=gen))
    g = -softplus(torch.randn(steps, N_V, generator=gen))
    S = S0.cuda().unsqueeze(0).clone()
    cst = torch.zeros(1, CONV_DIM, CONV_K, device="cuda")
    wd, xd, bd, gd = w.cuda(), xs.cuda(), beta.cuda(), g.cuda()
    outs = []
    for t in range(steps):
        mixed = ops.conv1d_update(xd[t:t + 1], wd, cst)
        qk = mixed[:, :2 * N_K * DK].reshape(1, 2, N_K, DK)
        v = mixed[:, 2 * N_K * DK:].reshape(1, N_V, DV).contiguous()
        outs.append(ops.delta_recurrent_step(S, qk[:, 0].contiguous(), qk[:, 1].contiguous(), v,
                                             bd[t:t + 1], gd[t:t + 1]))
    _lib.check_device()
    o_gpu = torch.cat(outs).cpu().numpy()
    Sr = S0.numpy().copy()
    cr = np.zeros((CONV_DIM, CONV_K), np.float32)
    o_ref = np.empty_like(o_gpu)
    for t in range(steps):
        mixed = oracle.conv1d_update(xs[t].numpy(), w.numpy(), cr)
        q = oracle.repeat_heads(mixed[:N_K * DK].reshape(N_K, DK), N_V)
        k = oracle.repeat_heads(mixed[N_K * DK:2 * N_K * DK].reshape(N_K, DK), N_V)
        v = mixed[2 * N_K * DK:].reshape(N_V, DV)
        o_ref[t] = oracle.delta_step(Sr, q, k, v, beta[t].numpy(), g[t].numpy())
    s_err = rel_l2(S[0].cpu().numpy(), Sr)
    o_err = np.abs(o_gpu - o_ref).max()
    print("cfg1 state rel-l2 %.3e, o max-abs %.3e, conv state max-abs %.3e" %
          (s_err, o_err, np.abs(cst[0].cpu().numpy() - cr).max()))
    assert s_err <= STATE_REL_L2
    assert o_err <= 1e-4
    assert np.array_equal(cst[0].cpu().numpy(), cr)          # the window is a pure shift


def test_l2_normalised_inputs_per_value_heads(oracle):
    """q, k already L2-normalised and repeated per value head (the op normalises again)."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(11)
    S0 = torch.randn(N_V, DK, DV, generator=gen) * 0.02
    q = torch.nn.functional.normalize(torch.randn(N_V, DK, generator=gen), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(N_V, DK, generator=gen), dim=-1)
    v = torch.randn(N_V, DV, generator=gen)
    beta = torch.sigmoid(torch.randn(N_V, generator=gen))
    g = -softplus(torch.randn(N_V, generator=gen))
    S = S0.cuda().clone()
    o = ops.delta_recurrent_step(S, q.cuda(), k.cuda(), v.cuda(), beta.cuda(), g.cuda())
    _lib.check_device()
    Sr = S0.numpy().copy()
    oref = oracle.delta_step(Sr, q.numpy(), k.numpy(), v.numpy(), beta.numpy(), g.numpy())
    assert np.abs(o.cpu().numpy() - oref).max() < 1e-5
    assert rel_l2(S.cpu().numpy(), Sr) < 1e-6


def test_reference_golden_vectors(golden):
    """The reference's own scalar outputs (tests/golden, 4 heads of 128x128, 3 steps)."""
    from rapidllm_b200 import _lib, ops
    S = torch.from_numpy(golden["delta_a_S0"].copy()).cuda()
    for t in range(3):
        a = [torch.from_numpy(golden[f"delta_a_{n}{t}"]).cuda() for n in ("q", "k", "v", "beta", "g")]
        o = ops.delta_recurrent_step(S, *a)
        assert np.abs(o.cpu().numpy() - golden[f"delta_a_o_scalar{t}"]).max() < 2e-5
    _lib.check_device()
    assert rel_l2(S.cpu().numpy(), golden["delta_a_S_scalar"]) < 1e-6


@pytest.mark.parametrize("head_map", [1, 2])
def test_batch_slots_and_head_maps(oracle, head_map):
    """Batch of 5 sequences on shuffled state slots; grouped (h // 3) and tiled (h % 16) maps."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(20 + head_map)
    B, n_slots = 5, 8
    S0 = torch.randn(n_slots, N_V, DK, DV, generator=gen) * 0.02
    slots = torch.randperm(n_slots, generator=gen)[:B].int()
    q = torch.randn(B, N_K, DK, generator=gen)
    k = torch.randn(B, N_K, DK, generator=gen)
    v = torch.randn(B, N_V, DV, generator=gen)
    beta = torch.sigmoid(torch.randn(B, N_V, generator=gen))
    g = -softplus(torch.randn(B, N_V, generator=gen))
    S = S0.cuda().clone()
    o = ops.delta_recurrent_step(S, q.cuda(), k.cuda(), v.cuda(), beta.cuda(), g.cuda(),
                                 slot_ids=slots.cuda(), head_map=head_map)
    _lib.check_device()
    Sr = S0.numpy().copy()
    for b in range(B):
        sl = int(slots[b])
        qq = oracle.repeat_heads(q[b].numpy(), N_V, tiled=(head_map == 2))
        kk = oracle.repeat_heads(k[b].numpy(), N_V, tiled=(head_map == 2))
        oref = oracle.delta_step(Sr[sl], qq, kk, v[b].numpy(), beta[b].numpy(), g[b].numpy())
        assert np.abs(o[b].cpu().numpy() - oref).max() < 2e-5
    assert rel_l2(S.cpu().numpy(), Sr) < 1e-6           # untouched slots stay bit-identical too
    untouched = [s for s in range(n_slots) if s not in slots.tolist()]
    assert np.array_equal(S[untouched].cpu().numpy(), S0[untouched].numpy())
    bad = torch.tensor([0, 1, 2, 3, 99], dtype=torch.int32, device="cuda")
    ops.delta_recurrent_step(S, q.cuda(), k.cuda(), v.cuda(), beta.cuda(), g.cuda(), slot_ids=bad,
                             head_map=head_map)
    assert _lib.device_error() == 4


def test_conv1d_update_and_prefill(oracle, golden):
    from rapidllm_b200 import _lib, ops
    w, xs = golden["conv_w"], golden["conv_x"]
    wd = torch.from_numpy(w).cuda()
    st = torch.zeros(1, *w.shape, device="cuda")
    ys = torch.cat([ops.conv1d_update(torch.from_numpy(x).cuda().unsqueeze(0), wd, st) for x in xs])
    assert np.abs(ys.cpu().numpy() - golden["conv_y_update"]).max() < 2e-6
    assert np.array_equal(st[0].cpu().numpy(), golden["conv_state_end"])
    # prefill form, whole and in two chunks carrying the window
    xd = torch.from_numpy(xs).cuda()
    st2 = torch.zeros(*w.shape, device="cuda")
    y = ops.conv1d_causal_prefill(xd, wd, st2)
    assert np.abs(y.cpu().numpy() - golden["conv_y_prefill"]).max() < 2e-6
    assert np.array_equal(st2.cpu().numpy(), golden["conv_state_end"])
    st3 = torch.zeros(*w.shape, device="cuda")
    ya = ops.conv1d_causal_prefill(xd[:2].contiguous(), wd, st3)
    yb = ops.conv1d_causal_prefill(xd[2:].contiguous(), wd, st3, use_state_in=True)
    assert torch.equal(torch.cat([ya, yb]), y)
    assert np.array_equal(st3.cpu().numpy(), golden["conv_state_end"])
    # other tap counts and a ragged channel count
    gen = torch.Generator().manual_seed(2)
    for dim, k in [(1000, 3), (77, 4), (300, 2)]:
        ww = torch.randn(dim, k, generator=gen)
        x = torch.randn(9, dim, generator=gen)
        s = np.zeros((dim, k), np.float32)
        ref = np.stack([oracle.conv1d_update(x[t].numpy(), ww.numpy(), s) for t in range(9)])
        sd = torch.zeros(1, dim, k, device="cuda")
        got = torch.cat([ops.conv1d_update(x[t:t + 1].cuda(), ww.cuda(), sd) for t in range(9)])
        assert np.abs(got.cpu().numpy() - ref).max() < 2e-6
        assert np.array_equal(sd[0].cpu().numpy(), s)
        assert np.abs(ops.conv1d_causal_prefill(x.cuda(), ww.cuda()).cpu().numpy() - ref).max() < 2e-6
    # the model's width (k 4, dim % 4 == 0: four channels x 16 steps per thread), ragged lengths, window carried
    dim, k = 10240, 4
    ww = torch.randn(dim, k, generator=gen)
    x = torch.randn(100, dim, generator=gen)
    s = np.zeros((dim, k), np.float32)
    ref = np.stack([oracle.conv1d_update(x[t].numpy(), ww.numpy(), s) for t in range(100)])
    sd = torch.zeros(dim, k, device="cuda")
    ya = ops.conv1d_causal_prefill(x[:37].cuda(), ww.cuda(), sd)
    yb = ops.conv1d_causal_prefill(x[37:].cuda(), ww.cuda(), sd, use_state_in=True)
    assert np.abs(torch.cat([ya, yb]).cpu().numpy() - ref).max() < 2e-6
    assert np.array_equal(sd.cpu().numpy(), s)
    whole = ops.conv1d_causal_prefill(x.cuda(), ww.cuda())
    assert torch.equal(whole, torch.cat([ya, yb]))
    _lib.check_device()


@pytest.mark.parametrize("B", [14, 16, 32])
def test_large_batch_streaming_path(oracle, B):
    """Batch x 48 heads takes the persistent TMA-streamed kernel; two steps, shuffled slots.  On 148
    SMs the last round of heads is taken by 80 (batch 14), 28 (batch 16) or 56 (batch 32) of the CTAs."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(33 + B)
    n_slots = B + 4
    S0 = torch.randn(n_slots, N_V, DK, DV, generator=gen) * 0.02
    slots = torch.randperm(n_slots, generator=gen)[:B].int()
    S = S0.cuda().clone()
    Sr = S0.numpy().copy()
    for step in range(2):
        q = torch.randn(B, N_K, DK, generator=gen)
        k = torch.randn(B, N_K, DK, generator=gen)
        v = torch.randn(B, N_V, DV, generator=gen)
        beta = torch.sigmoid(torch.randn(B, N_V, generator=gen))
        g = -softplus(torch.randn(B, N_V, generator=gen))
        o = ops.delta_recurrent_step(S, q.cuda(), k.cuda(), v.cuda(), beta.cuda(), g.cuda(),
                                     slot_ids=slots.cuda(), head_map=1)
        _lib.check_device()
        for b in range(B):
            sl = int(slots[b])
            oref = oracle.delta_step(Sr[sl], oracle.repeat_heads(q[b].numpy(), N_V),
                                     oracle.repeat_heads(k[b].numpy(), N_V), v[b].numpy(), beta[b].numpy(),
                                     g[b].numpy())
            assert np.abs(o[b].cpu().numpy() - oref).max() < 2e-5
    assert rel_l2(S.cpu().numpy(), Sr) < 1e-6
    untouched = [s for s in range(n_slots) if s not in slots.tolist()]
    assert np.array_equal(S[untouched].cpu().numpy(), S0[untouched].numpy())


@pytest.mark.parametrize("n_tok", [1, 2, 4, 12])
def test_multi_token_step_equals_single_steps_and_rolls_back(oracle, n_tok):
    """The speculative-verify form: n_tok tokens in one pass with the state on chip == n_tok
    single launches bit for bit; the backup holds the state before the first token, so restoring
    it and running k tokens gives the state after k accepted tokens."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(40 + n_tok)
    B, n_slots = 2, 3
    S0 = torch.randn(n_slots, 48, 128, 128, generator=gen) * 0.02
    slots = torch.tensor([2, 0], dtype=torch.int32)
    q = torch.randn(B, n_tok, 16, 128, generator=gen)
    k = torch.randn(B, n_tok, 16, 128, generator=gen)
    v = torch.randn(B, n_tok, 48, 128, generator=gen)
    beta = torch.sigmoid(torch.randn(B, n_tok, 48, generator=gen))
    g = -torch.nn.functional.softplus(torch.randn(B, n_tok, 48, generator=gen))
    dev = [x.cuda() for x in (q, k, v, beta, g)]
    S_multi = S0.clone().cuda()
    backup = torch.full_like(S_multi, float("nan"))
    o_multi = ops.delta_recurrent_multi(S_multi, *dev, slot_ids=slots.cuda(), backup=backup)
    _lib.check_device()
    S_single = S0.clone().cuda()
    for t in range(n_tok):
        o_t = ops.delta_recurrent_step(S_single, dev[0][:, t].contiguous(), dev[1][:, t].contiguous(),
                                       dev[2][:, t].contiguous(), dev[3][:, t].contiguous(),
                                       dev[4][:, t].contiguous(), slot_ids=slots.cuda())
        assert torch.equal(o_t, o_multi[:, t])
    assert torch.equal(S_single, S_multi)
    # backup: the touched slots as they were, the untouched slot never written
    assert torch.equal(backup[2].cpu(), S0[2]) and torch.equal(backup[0].cpu(), S0[0])
    assert torch.isnan(backup[1]).all()
    # oracle for sequence 0 (slot 2), first and last token
    Sr = S0[2].numpy().copy()
    for t in range(n_tok):
        ref = oracle.delta_step(Sr, oracle.repeat_heads(q[0, t].numpy(), 48), oracle.repeat_heads(k[0, t].numpy(), 48),
                                v[0, t].numpy(), beta[0, t].numpy(), g[0, t].numpy())
        assert np.abs(o_multi[0, t].cpu().numpy() - ref).max() < 1e-4
    assert rel_l2(S_multi[2].cpu().numpy(), Sr) < 1e-6
    # roll back to k accepted tokens
    if n_tok >= 2:
        kacc = n_tok // 2
        S_multi[2].copy_(backup[2])
        S_multi[0].copy_(backup[0])
        ops.delta_recurrent_multi(S_multi, *[x[:, :kacc].contiguous() for x in dev], slot_ids=slots.cuda())
        S_ref = S0.clone().cuda()
        for t in range(kacc):
            ops.delta_recurrent_step(S_ref, dev[0][:, t].contiguous(), dev[1][:, t].contiguous(),
                                     dev[2][:, t].contiguous(), dev[3][:, t].contiguous(),
                                     dev[4][:, t].contiguous(), slot_ids=slots.cuda())
        assert torch.equal(S_ref, S_multi)


def _fused_oracle_step(oracle, S, C, x, w, beta, g, n_k, n_v, tiled):
    mixed = oracle.conv1d_update(x, w, C)
    q = oracle.repeat_heads(mixed[:n_k * DK].reshape(n_k, DK), n_v, tiled)
    k = oracle.repeat_heads(mixed[n_k * DK:2 * n_k * DK].reshape(n_k, DK), n_v, tiled)
    return oracle.delta_step(S, q, k, mixed[2 * n_k * DK:].reshape(n_v, DV), beta, g)


@pytest.mark.parametrize("batch,head_map_name", [(3, "RL_HEADS_GROUPED"), (3, "RL_HEADS_TILED"), (14, "RL_HEADS_GROUPED"),
                                                 (14, "RL_HEADS_TILED")])
def test_fused_gdn_decode_matches_conv_then_delta(oracle, batch, head_map_name):
    """rl_gdn_decode (conv window + SiLU + l2 norms + delta rule in one kernel, ring windows) over
    six consecutive steps against ops::conv1d_update + ops::delta_recurrent_step: outputs, state,
    and the windows bit for bit after every step.  Batch 3 runs the slice kernel, batch 14 (672
    heads) the streaming kernel on a 148-SM part; slots are shuffled and one is left untouched."""
    from rapidllm_b200 import _lib, ops
    head_map = getattr(_lib, head_map_name)
    tiled = head_map == _lib.RL_HEADS_TILED
    gen = torch.Generator().manual_seed(70 + batch)
    n_slots = batch + 1
    S0 = torch.randn(n_slots, N_V, DK, DV, generator=gen) * 0.02
    C0 = torch.randn(n_slots, CONV_DIM, CONV_K, generator=gen)
    w = torch.randn(CONV_DIM, CONV_K, generator=gen) * 0.5
    slots = torch.randperm(n_slots, generator=gen)[:batch].int()
    S, ring = S0.cuda().clone(), C0.cuda().clone()          # phase 0: the ring equals the shifted window
    phase = torch.zeros(n_slots, dtype=torch.int32, device="cuda")
    Sr, Cr = S0.numpy().copy(), C0.numpy().copy()
    wd, sd = w.cuda(), slots.cuda()
    for step in range(6):
        x = torch.randn(batch, CONV_DIM, generator=gen)
        beta = torch.sigmoid(torch.randn(batch, N_V, generator=gen))
        g = -softplus(torch.randn(batch, N_V, generator=gen))
        o = ops.gdn_decode(S, ring, phase, x.cuda(), wd, beta.cuda(), g.cuda(), N_K, slot_ids=sd, head_map=head_map)
        _lib.check_device()
        o = o.cpu().numpy()
        for b in range(batch):
            sl = int(slots[b])
            ref = _fused_oracle_step(oracle, Sr[sl], Cr[sl], x[b].numpy(), w.numpy(), beta[b].numpy(), g[b].numpy(),
                                     N_K, N_V, tiled)
            assert np.abs(o[b] - ref).max() <= 1e-5, (step, b, np.abs(o[b] - ref).max())
        assert np.array_equal(ops.conv_ring_export(ring, phase).cpu().numpy(), Cr), step
        assert rel_l2(S.cpu().numpy(), Sr) <= 1e-6
    assert phase.cpu().tolist().count(0) == 1 and int(phase[slots[0]]) == 2      # 6 steps = phase 2; the idle slot stays 0
    idle = [s for s in range(n_slots) if s not in slots.tolist()][0]
    assert torch.equal(S[idle].cpu(), S0[idle])


def test_config1_1024_steps_fused(oracle):
    """The single-layer DeltaNet configuration (batch 1, 1024 consecutive steps from seed 1) through the
    fused kernel: state rel-L2 <= 1e-5, outputs max-abs <= 1e-4, window equal bit for bit."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(1)
    S0 = torch.randn(N_V, DK, DV, generator=gen) * 0.02
    w = torch.randn(CONV_DIM, CONV_K, generator=gen) * 0.5
    steps = 1024
    xs = torch.randn(steps, CONV_DIM, generator=gen)
    beta = torch.sigmoid(torch.randn(steps, N_V, generator=gen))
    g = -softplus(torch.randn(steps, N_V, generator=gen))
    S = S0.cuda().unsqueeze(0).clone()
    ring = torch.zeros(1, CONV_DIM, CONV_K, device="cuda")
    phase = torch.zeros(1, dtype=torch.int32, device="cuda")
    wd, xd, bd, gd = w.cuda(), xs.cuda(), beta.cuda(), g.cuda()
    outs = [ops.gdn_decode(S, ring, phase, xd[t:t + 1], wd, bd[t:t + 1], gd[t:t + 1], N_K) for t in range(steps)]
    _lib.check_device()
    o_gpu = torch.cat(outs).cpu().numpy()
    Sr = S0.numpy().copy()
    cr = np.zeros((CONV_DIM, CONV_K), np.float32)
    o_ref = np.empty_like(o_gpu)
    for t in range(steps):
        o_ref[t] = _fused_oracle_step(oracle, Sr, cr, xs[t].numpy(), w.numpy(), beta[t].numpy(), g[t].numpy(), N_K, N_V, False)
    s_err, o_err = rel_l2(S[0].cpu().numpy(), Sr), np.abs(o_gpu - o_ref).max()
    print("cfg1 fused: state rel-l2 %.3e, o max-abs %.3e" % (s_err, o_err))
    assert s_err <= STATE_REL_L2 and o_err <= 1e-4
    assert np.array_equal(ops.conv_ring_export(ring, phase)[0].cpu().numpy(), cr)
