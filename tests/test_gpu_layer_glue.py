"""The element-wise steps around the mixers (rl_attn_qk_prepare, rl_gated_rmsnorm,
rl_delta_gates) against the oracle's restatement of the reference's CPU functions."""
import numpy as np
import pytest
import torch

from helpers import rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,positions", [(1, [4095]), (5, [0, 1, 63, 32767, 131071]), (3, None)])
def test_attn_qk_prepare_matches_oracle(oracle, rows, positions):
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(31)
    qg = torch.randn(rows, 24, 512, generator=gen)
    k = torch.randn(rows, 4, 256, generator=gen)
    qn = torch.randn(256, generator=gen) * 0.1
    kn = torch.randn(256, generator=gen) * 0.1
    pos0 = 1000
    pos = None if positions is None else torch.tensor(positions, dtype=torch.int32).cuda()
    kd = k.clone().cuda()
    q, gate = ops.attn_qk_prepare(qg.cuda(), kd, qn.cuda(), kn.cuda(), pos, pos0=pos0)
    _lib.check_device()
    for r in range(rows):
        p = pos0 + r if positions is None else positions[r]
        q_ref, gate_ref, k_ref = oracle.attn_qk_prepare(qg[r].numpy(), k[r].numpy(), qn.numpy(), kn.numpy(), p)
        assert np.array_equal(gate[r].cpu().numpy(), gate_ref)            # a copy: exact
        # same frequencies (host powf) and the same fp32 angle as the CPU path; cosf / sinf of the
        # device are within 2 ulp, the double-accumulated norm within 1 ulp
        assert np.abs(q[r].cpu().numpy() - q_ref).max() <= 4e-6
        assert np.abs(kd[r].cpu().numpy() - k_ref).max() <= 4e-6
        # a rotation keeps the norm of every pair, whatever the angle
        assert rel_l2(np.linalg.norm(q[r].cpu().numpy(), axis=1), np.linalg.norm(q_ref, axis=1)) <= 1e-6


def test_attn_qk_prepare_without_norm_weights_and_rejects_bad_shapes():
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(32)
    qg = torch.randn(2, 6, 512, generator=gen).cuda()
    k = torch.randn(2, 1, 256, generator=gen).cuda()
    q, gate = ops.attn_qk_prepare(qg, k, None, None, None, pos0=0, rotary_dim=0)   # no RoPE, weight 1
    x = qg[:, :, :256]
    want = x / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True).float() + 1e-6)
    assert (q - want).abs().max().item() <= 2e-6
    with pytest.raises(_lib.RlError):
        ops.attn_qk_prepare(qg, k, rotary_dim=63)
    with pytest.raises(_lib.RlError):
        ops.attn_qk_prepare(torch.randn(2, 6, 256).cuda(), torch.randn(2, 1, 128).cuda())


@pytest.mark.parametrize("rows", [1, 7])
def test_gated_rmsnorm_and_gates_match_oracle(oracle, rows):
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(33)
    x = torch.randn(rows, 48, 128, generator=gen)
    z = torch.randn(rows, 48, 128, generator=gen) * 3
    gm = torch.randn(128, generator=gen)
    y = ops.gated_rmsnorm(x.cuda(), z.cuda(), gm.cuda()).cpu().numpy()
    for r in range(rows):
        ref = oracle.gated_rmsnorm(x[r].reshape(-1).numpy(), z[r].reshape(-1).numpy(), gm.numpy()).reshape(48, 128)
        assert np.abs(y[r] - ref).max() <= 1e-5 and rel_l2(y[r], ref) <= 1e-6
    a = torch.randn(rows, 48, generator=gen) * 4
    b = torch.randn(rows, 48, generator=gen) * 4
    A_log = torch.randn(48, generator=gen)
    dt = torch.randn(48, generator=gen)
    beta, g = ops.delta_gates(a.cuda(), b.cuda(), A_log.cuda(), dt.cuda())
    _lib.check_device()
    for r in range(rows):
        beta_ref, g_ref = oracle.delta_gates(a[r].numpy(), b[r].numpy(), A_log.numpy(), dt.numpy())
        assert rel_l2(beta[r].cpu().numpy(), beta_ref) <= 1e-6
        assert rel_l2(g[r].cpu().numpy(), g_ref) <= 1e-6


def test_hidden_rmsnorm(oracle):
    """rl_rmsnorm over rows of the hidden size (the norm in front of a mixer's projections), also in place."""
    from rapidllm_b200 import _lib, ops
    gen = torch.Generator().manual_seed(77)
    for n in (5120, 96, 1):
        x = torch.randn(5, n, generator=gen) * 3.0
        gamma = torch.randn(n, generator=gen) * 0.1
        y = ops.rmsnorm(x.cuda(), gamma.cuda())
        y0 = ops.rmsnorm(x.cuda(), None)
        xi = x.cuda()
        ops.rmsnorm(xi, gamma.cuda(), out=xi)
        _lib.check_device()
        ref = oracle.qwen3_rmsnorm(x.numpy(), gamma.numpy())
        assert np.abs(y.cpu().numpy() - ref).max() <= 2e-6 * max(1.0, np.abs(ref).max())
        assert torch.equal(xi, y)
        assert np.abs(y0.cpu().numpy() - oracle.qwen3_rmsnorm(x.numpy(), None)).max() <= 2e-6 * np.abs(ref).max() + 2e-6


def test_cast_f32_to_bf16_rounds_to_nearest_even():
    import ctypes as C
    from rapidllm_b200 import _lib
    gen = torch.Generator().manual_seed(5)
    for n in (1, 3, 4, 1021, 4096 * 3 + 2):
        x = (torch.randn(n, generator=gen) * 3).cuda()
        if n > 8:
            x[1], x[2], x[5] = 1.00390625, 1.01171875, -0.0        # ties: to even (down), to even (up); signed zero
        y = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        _lib.check(_lib.lib().rl_cast_f32_to_bf16(C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), n,
                                                  C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        assert torch.equal(y, x.to(torch.bfloat16))
