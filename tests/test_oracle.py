"""The CPU restatement (oracle/rl_oracle.c) against the reference's own outputs.

Golden vectors in tests/golden/ref_vectors.npz were produced by the reference's
compiled CPU operators and by its python/goldens/tiny_hybrid.py (see
tests/golden/make_golden.py).  Integer / same-order fp32 paths must match
bit for bit; the AVX path and the double-precision Python model within a
stated tolerance.
"""
import numpy as np
import pytest

from conftest import rel_l2


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_attn_decode_bit_exact_vs_reference_golden(oracle, golden, tag):
    q, k, v = (golden[f"attn_decode_{tag}_{n}"] for n in "qkv")
    assert np.array_equal(oracle.attn_decode(q, k, v), golden[f"attn_decode_{tag}_o"])
    assert np.array_equal(oracle.attn_decode(q, k, v, pos=k.shape[0] // 2),
                          golden[f"attn_decode_{tag}_o_half"])


def test_attn_prefill_bit_exact_vs_reference_golden(oracle, golden):
    q, k, v = golden["attn_prefill_q"], golden["attn_prefill_k"], golden["attn_prefill_v"]
    assert np.array_equal(oracle.attn_prefill(q, k, v), golden["attn_prefill_o"])
    rows = np.array([0, 7, 18], np.int32)
    o = oracle.attn_prefill_rows(q[rows], k, v, rows)
    assert np.array_equal(o, golden["attn_prefill_o"][rows])


@pytest.mark.parametrize("tag", ["a", "b"])
def test_delta_step_vs_reference_golden(oracle, golden, tag):
    S = golden[f"delta_{tag}_S0"].copy()
    for t in range(3):
        a = [golden[f"delta_{tag}_{n}{t}"] for n in ("q", "k", "v", "beta", "g")]
        o = oracle.delta_step(S, *a)
        assert np.array_equal(o, golden[f"delta_{tag}_o_scalar{t}"])
        # the AVX-512/AVX2 path fuses multiply-adds: same maths, other rounding
        assert rel_l2(o, golden[f"delta_{tag}_o_simd{t}"]) < 1e-5
    assert np.array_equal(S, golden[f"delta_{tag}_S_scalar"])
    assert rel_l2(S, golden[f"delta_{tag}_S_simd"]) < 1e-5


def test_conv1d_vs_reference_golden(oracle, golden):
    w, xs = golden["conv_w"], golden["conv_x"]
    st = np.zeros_like(w)
    ys = np.stack([oracle.conv1d_update(x, w, st) for x in xs])
    assert np.array_equal(ys, golden["conv_y_update"])
    assert np.array_equal(st, golden["conv_state_end"])
    assert np.array_equal(oracle.conv1d_causal_prefill(xs, w), golden["conv_y_prefill"])
    # decode form and prefill form are the same function of the inputs
    assert np.array_equal(golden["conv_y_update"], golden["conv_y_prefill"])
    assert np.array_equal(oracle.l2norm(golden["l2_x"]), golden["l2_y"])


def test_norms_and_rope_bit_exact_vs_reference_golden(oracle, golden):
    for tag in "ab":
        y = oracle.qwen3_rmsnorm(golden[f"rms_{tag}_x"], golden[f"rms_{tag}_gamma"])
        assert np.array_equal(y, golden[f"rms_{tag}_y"])
    for tag in "abc":
        rot, pos = (int(v) for v in golden[f"rope_{tag}_meta"])
        q, k = oracle.rope_partial(golden[f"rope_{tag}_q"], golden[f"rope_{tag}_k"], pos, rotary_dim=rot)
        assert np.array_equal(q, golden[f"rope_{tag}_q_out"]) and np.array_equal(k, golden[f"rope_{tag}_k_out"])
    for tag in "abc":
        y = oracle.gated_rmsnorm(golden[f"gnorm_{tag}_x"], golden[f"gnorm_{tag}_z"], golden[f"gnorm_{tag}_gamma"])
        assert np.array_equal(y, golden[f"gnorm_{tag}_y"])
    # the composite of ops_fused.cpp:154-171 equals its parts
    rng = np.random.default_rng(5)
    qg = rng.standard_normal((24, 512), dtype=np.float32)
    k = rng.standard_normal((4, 256), dtype=np.float32)
    qn = rng.standard_normal(256, dtype=np.float32) * 0.1
    kn = rng.standard_normal(256, dtype=np.float32) * 0.1
    q, gate, k2 = oracle.attn_qk_prepare(qg, k, qn, kn, pos=777)
    q_ref, k_ref = oracle.rope_partial(oracle.qwen3_rmsnorm(qg[:, :256], qn), oracle.qwen3_rmsnorm(k, kn), 777)
    assert np.array_equal(q, q_ref) and np.array_equal(k2, k_ref) and np.array_equal(gate, qg[:, 256:])


def test_tiny_hybrid_python_model(oracle, golden):
    """python/goldens/tiny_hybrid.py delta_step (120-146) and decode attention
    with the sigmoid gate (275-312), double precision, tiny dims."""
    S = golden["tiny_delta_S0"].astype(np.float32)
    eps = float(golden["tiny_delta_eps"])
    for t in range(2):
        a = [golden[f"tiny_delta_{n}{t}"] for n in ("q", "k", "v", "beta", "g")]
        o = oracle.delta_step(S, *a, eps=eps)
        assert np.allclose(o, golden[f"tiny_delta_o{t}"], rtol=1e-4, atol=1e-5)
    assert np.allclose(S, golden["tiny_delta_S_end"], rtol=1e-4, atol=1e-5)
    o = oracle.gated_attn_decode(golden["tiny_attn_q"], golden["tiny_attn_k"],
                                 golden["tiny_attn_v"],
                                 golden["tiny_attn_gate"].reshape(golden["tiny_attn_q"].shape))
    assert np.allclose(o.ravel(), golden["tiny_attn_o"], rtol=1e-4, atol=1e-6)


def test_live_reference_bit_exact(oracle, reference):
    """Random shapes against the reference library built in this container."""
    rng = np.random.default_rng(7)
    for n_q, n_kv, hd, seq in [(24, 4, 256, 130), (4, 4, 16, 9), (12, 2, 128, 65)]:
        q = rng.standard_normal((n_q, hd), dtype=np.float32)
        k = rng.standard_normal((seq, n_kv, hd), dtype=np.float32)
        v = rng.standard_normal((seq, n_kv, hd), dtype=np.float32)
        assert np.array_equal(oracle.attn_decode(q, k, v), reference.attn_decode(q, k, v))
    S1 = (rng.standard_normal((48, 128, 128), dtype=np.float32) * 0.02).astype(np.float32)
    S2 = S1.copy()
    for _ in range(4):
        q = rng.standard_normal((48, 128), dtype=np.float32)
        k = rng.standard_normal((48, 128), dtype=np.float32)
        v = rng.standard_normal((48, 128), dtype=np.float32)
        b = rng.random(48, dtype=np.float32)
        g = -rng.random(48, dtype=np.float32)
        assert np.array_equal(oracle.delta_step(S1, q, k, v, b, g),
                              reference.delta_step(S2, q, k, v, b, g))
    assert np.array_equal(S1, S2)
    w = rng.standard_normal((10240, 4), dtype=np.float32)
    s1 = rng.standard_normal((10240, 4), dtype=np.float32)
    s2 = s1.copy()
    x = rng.standard_normal(10240, dtype=np.float32)
    assert np.array_equal(oracle.conv1d_update(x, w, s1), reference.conv1d_update(x, w, s2))
    assert np.array_equal(s1, s2)


def test_split_partials_combine_to_unsplit(oracle):
    rng = np.random.default_rng(3)
    n_kv, hd, seq = 2, 64, 300
    q = rng.standard_normal((4, hd), dtype=np.float32)
    k = rng.standard_normal((seq, n_kv, hd), dtype=np.float32)
    v = rng.standard_normal((seq, n_kv, hd), dtype=np.float32)
    full = oracle.attn_decode(q, k, v)
    cuts = [0, 64, 128, 129, 300]
    for hq in range(4):
        parts = [oracle.attn_partial(q[hq], k, v, a, b, hq // 2) for a, b in zip(cuts, cuts[1:])]
        o = oracle.lse_combine([p[0] for p in parts], [p[1] for p in parts],
                               np.stack([p[2] for p in parts]))
        assert rel_l2(o, full[hq]) < 1e-6
    # an empty split (m = -1e30, l = 0) must not disturb the result
    m, l, acc = oracle.attn_partial(q[0], k, v, 10, 10, 0)
    assert l == 0.0 and m == np.float32(-1e30)


def test_fp16_round_to_nearest_even(oracle):
    x = np.array([1.0, 1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 65504.0, 1e-8, -2.5, 6.1e-5],
                 np.float32)
    assert np.array_equal(oracle.to_f16(x), x.astype(np.float16).view(np.uint16))
    r = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    assert np.array_equal(oracle.to_f16(r), r.astype(np.float16).view(np.uint16))
    assert np.array_equal(oracle.from_f16(oracle.to_f16(r)),
                          r.astype(np.float16).astype(np.float32))


def test_paged_gather_equals_contiguous(oracle):
    rng = np.random.default_rng(5)
    n_kv, pt, hd, n_pages = 4, 64, 256, 9
    seq = 64 * 5 + 17
    rows = rng.integers(0, 65535, size=(seq, n_kv, hd), dtype=np.uint16)
    table = rng.permutation(n_pages)[:6].astype(np.int32)
    pool = np.zeros((n_pages, n_kv, pt, hd), np.uint16)
    oracle.paged_scatter(pool, table, 0, rows[:100])
    oracle.paged_scatter(pool, table, 100, rows[100:])
    assert np.array_equal(oracle.paged_gather(pool, table, seq), rows)


@pytest.mark.parametrize("wht_len,use_signs", [(128, False), (256, True), (256, False)])
def test_compact_kv_properties(oracle, wht_len, use_signs):
    rng = np.random.default_rng(11)
    T, n_kv, hd = 33, 4, 256
    k = rng.standard_normal((T, n_kv, hd), dtype=np.float32)
    v = rng.standard_normal((T, n_kv, hd), dtype=np.float32)
    signs = (2.0 * rng.integers(0, 2, wht_len) - 1).astype(np.float32) if use_signs else None
    k_q, k_sc, v_codes, v_sc = oracle.compact_store(k, v, wht_len, signs)
    # q8: |q| <= 127, the row maximum maps to +-127, error below one step
    assert np.abs(k_q.astype(np.int32)).max() == 127
    amax = np.abs(k).max(-1)
    s = amax / np.float32(127) + np.float32(1e-8)
    assert np.array_equal(k_sc, s.astype(np.float16).view(np.uint16))
    kd, vd = oracle.compact_dequant(k_q, k_sc, v_codes, v_sc, wht_len, signs)
    assert np.abs(kd - k).max() <= 0.51 * s.max() + 2e-3 * amax.max()
    # the transform is orthonormal and its own inverse
    x = rng.standard_normal(wht_len).astype(np.float32)
    y = oracle.fwht(x)
    assert abs(np.linalg.norm(y) - np.linalg.norm(x)) < 1e-4
    assert np.allclose(oracle.fwht(y), x, atol=1e-5)
    # TQ3: scale is the RMS of the block, reconstruction error is that of an
    # 8-level Lloyd-Max quantiser for N(0,1) (MSE 0.03454 -> rel error ~0.186)
    rms = np.sqrt((v.reshape(T, n_kv, hd // wht_len, wht_len) ** 2).mean(-1))
    assert np.allclose(oracle.from_f16(v_sc), rms, rtol=2e-3)
    rel = rel_l2(vd, v)
    assert 0.15 < rel < 0.22, rel
    # codes are packed 8 per 3 bytes, LSB first
    w = v_codes[0, 0, 0].astype(np.uint32) | (v_codes[0, 0, 1].astype(np.uint32) << 8) | \
        (v_codes[0, 0, 2].astype(np.uint32) << 16)
    cent = oracle.centroids()
    xb = v[0, 0, :wht_len] * (signs if signs is not None else 1)
    yb = oracle.fwht(xb)
    r = np.float32(np.sqrt(np.float32((yb.astype(np.float64) ** 2).sum()) / wht_len))
    for j in range(8):
        idx = (w >> (3 * j)) & 7
        assert idx == np.argmin(np.abs(yb[j] / r - cent)) or \
            abs(abs(yb[j] / r - cent[idx]) - np.abs(yb[j] / r - cent).min()) < 1e-5


def _mixer_weights(golden, prefix, names):
    return {n: golden[f"{prefix}_{n}"] for n in names}


DELTA_W = ("rms_w", "Wqkv", "Wz", "Wa", "Wb", "Wo", "A_log", "dt_bias", "conv_w", "gnorm")
ATTN_W = ("rms_w", "Wq", "Wk", "Wv", "Wo", "q_norm", "k_norm")


def test_whole_mixers_bit_exact_vs_reference_golden(oracle, golden):
    """ops::fused_delta_decode / fused_attn_decode outputs (three tokens, both head maps)."""
    for tag, (nk, nv, tiled) in {"grouped": (1, 3, False), "tiled": (2, 4, True)}.items():
        w = _mixer_weights(golden, f"mixer_delta_{tag}", DELTA_W)
        S = np.zeros((nv, 128, 128), np.float32)
        conv = np.zeros_like(golden[f"mixer_delta_{tag}_conv_out"])
        x = golden[f"mixer_delta_{tag}_x"]
        for t in range(3):
            x = oracle.fused_delta_decode(x, w, S, conv, nk, nv, v_tiled=tiled)
            assert np.array_equal(x, golden[f"mixer_delta_{tag}_x_out"][t]), (tag, t)
        assert np.array_equal(S, golden[f"mixer_delta_{tag}_S_out"])
        assert np.array_equal(conv, golden[f"mixer_delta_{tag}_conv_out"])
    w = _mixer_weights(golden, "mixer_attn", ATTN_W)
    kc, vc = np.zeros((4, 1, 256), np.float32), np.zeros((4, 1, 256), np.float32)
    x = golden["mixer_attn_x"]
    for pos in range(3):
        x = oracle.fused_attn_decode(x, w, kc, vc, pos, 2, 1)
        assert np.array_equal(x, golden["mixer_attn_x_out"][pos]), pos
    assert np.array_equal(kc, golden["mixer_attn_k_cache"]) and np.array_equal(vc, golden["mixer_attn_v_cache"])


def test_whole_mixers_vs_live_reference(oracle, reference, monkeypatch):
    """Larger shapes against oracle/_ref: bit for bit with the reference's scalar norm
    (RAPIDLLM_SIMD=scalar, its own switch), within a few ulp with its AVX norm."""
    rs = np.random.RandomState(9)

    def f(*shape):
        return rs.standard_normal(shape).astype(np.float32)

    hidden, nk, nv, n_q, n_kv = 96, 4, 12, 6, 2
    cd = 2 * nk * 128 + nv * 128
    wd = dict(rms_w=f(hidden) * 0.1, Wqkv=f(cd, hidden) / 8, Wz=f(nv * 128, hidden) / 8, Wa=f(nv, hidden) / 8,
              Wb=f(nv, hidden) / 8, Wo=f(hidden, nv * 128) / 20, A_log=f(nv) * 0.5, dt_bias=f(nv),
              conv_w=f(cd, 4) * 0.5, gnorm=f(128))
    wa = dict(rms_w=f(hidden) * 0.1, Wq=f(n_q * 512, hidden) / 8, Wk=f(n_kv * 256, hidden) / 8,
              Wv=f(n_kv * 256, hidden) / 8, Wo=f(hidden, n_q * 256) / 20, q_norm=f(256) * 0.1, k_norm=f(256) * 0.1)
    x0 = f(hidden)
    for mode in ("scalar", None):
        if mode:
            monkeypatch.setenv("RAPIDLLM_SIMD", mode)
        else:
            monkeypatch.delenv("RAPIDLLM_SIMD")
        S1, S2 = np.zeros((nv, 128, 128), np.float32), np.zeros((nv, 128, 128), np.float32)
        c1, c2 = np.zeros((cd, 4), np.float32), np.zeros((cd, 4), np.float32)
        k1, k2, v1, v2 = (np.zeros((6, n_kv, 256), np.float32) for _ in range(4))
        xa = xb = x0
        for t in range(5):
            xa = oracle.fused_delta_decode(xa, wd, S1, c1, nk, nv)
            xb = reference.fused_delta_decode(xb, wd, S2, c2, nk, nv)
            xa = oracle.fused_attn_decode(xa, wa, k1, v1, t, n_q, n_kv)
            xb = reference.fused_attn_decode(xb, wa, k2, v2, t, n_q, n_kv)
            if mode:
                assert np.array_equal(xa, xb) and np.array_equal(S1, S2) and np.array_equal(k1, k2), t
            else:
                assert np.abs(xa - xb).max() <= 2e-5 * np.abs(xb).max(), t
