"""Generate tests/golden/ref_vectors.npz from the reference itself.

Run in a container that has the reference tree (it cannot travel to the GPU
box, the vectors can):

    make -C oracle && python tests/golden/make_golden.py [--ref /path/to/RapidLLM]

Two sources, both the reference's own code:
  * oracle/_ref/librl_ref.so  -- rapidllm::ops::{attn_decode, attn_prefill,
    delta_recurrent_step_scalar/_simd, conv1d_update, conv1d_causal_prefill,
    l2norm, qwen3_rmsnorm, rope_partial, gated_rmsnorm} compiled from the reference's sources (see oracle/Makefile);
  * python/goldens/tiny_hybrid.py -- the reference's pure-Python model of the
    tiny hybrid net; its delta_step() and its decode-attention arithmetic give
    an independent double-precision statement at tiny dims (dk=dv=8, hd=8).
Inputs are seeded numpy draws and are stored next to the outputs.
"""
import argparse
import importlib.util
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import Reference  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of the RapidLLM tree")
    args = ap.parse_args()
    ref = Reference()
    out = {}
    rng = np.random.default_rng(20240)

    # attention decode: (n_q, n_kv, hd, seq)
    for tag, (n_q, n_kv, hd, seq) in {"a": (6, 2, 64, 37), "b": (24, 4, 256, 96),
                                      "c": (8, 1, 32, 1)}.items():
        q = rng.standard_normal((n_q, hd), dtype=np.float32)
        k = rng.standard_normal((seq, n_kv, hd), dtype=np.float32)
        v = rng.standard_normal((seq, n_kv, hd), dtype=np.float32)
        out[f"attn_decode_{tag}_q"] = q
        out[f"attn_decode_{tag}_k"] = k
        out[f"attn_decode_{tag}_v"] = v
        out[f"attn_decode_{tag}_o"] = ref.attn_decode(q, k, v)
        # a shorter position inside the same cache
        out[f"attn_decode_{tag}_o_half"] = ref.attn_decode(q, k, v, pos=seq // 2)

    # attention prefill
    T, n_q, n_kv, hd = 19, 6, 2, 32
    q = rng.standard_normal((T, n_q, hd), dtype=np.float32)
    k = rng.standard_normal((T, n_kv, hd), dtype=np.float32)
    v = rng.standard_normal((T, n_kv, hd), dtype=np.float32)
    out["attn_prefill_q"], out["attn_prefill_k"], out["attn_prefill_v"] = q, k, v
    out["attn_prefill_o"] = ref.attn_prefill(q, k, v)

    # delta rule, 3 consecutive steps, scalar and simd paths
    for tag, (n_v, dk, dv) in {"a": (4, 128, 128), "b": (6, 16, 24)}.items():
        S0 = (rng.standard_normal((n_v, dk, dv), dtype=np.float32) * 0.02).astype(np.float32)
        out[f"delta_{tag}_S0"] = S0
        Ss, Sv = S0.copy(), S0.copy()
        for t in range(3):
            q = rng.standard_normal((n_v, dk), dtype=np.float32)
            k = rng.standard_normal((n_v, dk), dtype=np.float32)
            v = rng.standard_normal((n_v, dv), dtype=np.float32)
            beta = (1 / (1 + np.exp(-rng.standard_normal(n_v)))).astype(np.float32)
            g = (-np.log1p(np.exp(rng.standard_normal(n_v)))).astype(np.float32)
            for nm, arr in (("q", q), ("k", k), ("v", v), ("beta", beta), ("g", g)):
                out[f"delta_{tag}_{nm}{t}"] = arr
            out[f"delta_{tag}_o_scalar{t}"] = ref.delta_step(Ss, q, k, v, beta, g, simd=False)
            out[f"delta_{tag}_o_simd{t}"] = ref.delta_step(Sv, q, k, v, beta, g, simd=True)
        out[f"delta_{tag}_S_scalar"] = Ss
        out[f"delta_{tag}_S_simd"] = Sv
    out["simd_isa"] = np.array(ref.simd_name())

    # conv1d
    dim, kk = 96, 4
    w = (rng.standard_normal((dim, kk), dtype=np.float32) * 0.5).astype(np.float32)
    st = np.zeros((dim, kk), np.float32)
    xs = rng.standard_normal((7, dim), dtype=np.float32)
    ys = np.stack([ref.conv1d_update(xs[t], w, st) for t in range(7)])
    out["conv_w"], out["conv_x"], out["conv_y_update"], out["conv_state_end"] = w, xs, ys, st
    out["conv_y_prefill"] = ref.conv1d_causal_prefill(xs, w)
    x = rng.standard_normal(128, dtype=np.float32)
    out["l2_x"], out["l2_y"] = x, ref.l2norm(x)

    # tiny_hybrid.py (double-precision python lists)
    spec = importlib.util.spec_from_file_location(
        "tiny_hybrid", os.path.join(args.ref, "python", "goldens", "tiny_hybrid.py"))
    th = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(th)
    NV, DK, DV = th.NV, th.DK, th.DV
    S = (rng.standard_normal((NV, DK, DV)) * 0.1).tolist()
    out["tiny_delta_S0"] = np.array(S, np.float64)
    for t in range(2):
        q = rng.standard_normal((NV, DK)).tolist()
        k = rng.standard_normal((NV, DK)).tolist()
        v = rng.standard_normal((NV, DV)).tolist()
        beta = (1 / (1 + np.exp(-rng.standard_normal(NV)))).tolist()
        g = (-np.log1p(np.exp(rng.standard_normal(NV)))).tolist()
        o = th.delta_step(S, q, k, v, beta, g)
        for nm, arr in (("q", q), ("k", k), ("v", v), ("beta", beta), ("g", g), ("o", o)):
            out[f"tiny_delta_{nm}{t}"] = np.array(arr, np.float64)
    out["tiny_delta_S_end"] = np.array(S, np.float64)
    out["tiny_delta_eps"] = np.array(th.EPS)
    # decode attention + sigmoid gate exactly as one_layer_attn() spells it
    NQ, NKV, HD = th.NQ, th.NKV, th.HD
    pos = 4
    qh = rng.standard_normal((NQ, HD)).tolist()
    kc = rng.standard_normal((pos + 1, NKV, HD)).tolist()
    vc = rng.standard_normal((pos + 1, NKV, HD)).tolist()
    gate = rng.standard_normal(NQ * HD).tolist()
    scale = 1.0 / math.sqrt(HD)
    rep = NQ // NKV
    o = []
    for hq in range(NQ):
        hkv = hq // rep
        scores, m = [], -1e30
        for s in range(pos + 1):
            acc = sum(qh[hq][d] * kc[s][hkv][d] for d in range(HD)) * scale
            scores.append(acc)
            m = max(m, acc)
        z = sum(math.exp(s - m) for s in scores)
        oh = [0.0] * HD
        for s, sc in enumerate(scores):
            a = math.exp(sc - m) / z
            for d in range(HD):
                oh[d] += a * vc[s][hkv][d]
        o.extend([oh[d] * th.sigmoid(gate[hq * HD + d]) for d in range(HD)])
    out["tiny_attn_q"], out["tiny_attn_k"], out["tiny_attn_v"] = map(np.array, (qh, kc, vc))
    out["tiny_attn_gate"], out["tiny_attn_o"] = np.array(gate), np.array(o)

    # the steps around the mixers (own generator, so the vectors above do not move):
    # head RMSNorm with (1 + gamma), partial RoPE, gated RMSNorm
    rng2 = np.random.default_rng(20241)
    for tag, n in {"a": 256, "b": 32}.items():
        x = rng2.standard_normal(n, dtype=np.float32)
        gm = (rng2.standard_normal(n, dtype=np.float32) * 0.1).astype(np.float32)
        out[f"rms_{tag}_x"], out[f"rms_{tag}_gamma"], out[f"rms_{tag}_y"] = x, gm, ref.qwen3_rmsnorm(x, gm)
    for tag, (n_q, n_kv, hd, rot, pos) in {"a": (24, 4, 256, 64, 4095), "b": (6, 2, 64, 64, 131071),
                                           "c": (4, 2, 8, 8, 17)}.items():
        q = rng2.standard_normal((n_q, hd), dtype=np.float32)
        k = rng2.standard_normal((n_kv, hd), dtype=np.float32)
        qr, kr = ref.rope_partial(q, k, pos, rotary_dim=rot, theta=1e7)
        out[f"rope_{tag}_q"], out[f"rope_{tag}_k"] = q, k
        out[f"rope_{tag}_meta"] = np.array([rot, pos], np.int64)
        out[f"rope_{tag}_q_out"], out[f"rope_{tag}_k_out"] = qr, kr
    for tag, (n, gn) in {"a": (48 * 128, 128), "b": (96, 96), "c": (64, 16)}.items():
        x = rng2.standard_normal(n, dtype=np.float32)
        z = rng2.standard_normal(n, dtype=np.float32)
        gm = rng2.standard_normal(gn, dtype=np.float32)
        out[f"gnorm_{tag}_x"], out[f"gnorm_{tag}_z"], out[f"gnorm_{tag}_gamma"] = x, z, gm
        out[f"gnorm_{tag}_y"] = ref.gated_rmsnorm(x, z, gm)

    # the whole decode mixers (ops::fused_delta_decode / fused_attn_decode) with dense fp32 weights,
    # three tokens each.  The reference's own switch RAPIDLLM_SIMD=scalar selects its scalar norm
    # (its qwen3_rmsnorm otherwise takes the AVX kernel for n >= 64, whose summation order differs
    # by an ulp); the vectors above were made without it and do not move.
    os.environ["RAPIDLLM_SIMD"] = "scalar"
    rng3 = np.random.default_rng(20242)
    f = lambda *shape: rng3.standard_normal(shape, dtype=np.float32)  # noqa: E731
    hidden, nk, nv, dk, dv, ck = 32, 1, 3, 128, 128, 4
    cd = 2 * nk * dk + nv * dv
    for tag, tiled in {"grouped": False, "tiled": True}.items():
        w = dict(rms_w=f(hidden) * 0.1, Wqkv=f(cd, hidden) / 6, Wz=f(nv * dv, hidden) / 6, Wa=f(nv, hidden) / 6,
                 Wb=f(nv, hidden) / 6, Wo=f(hidden, nv * dv) / 20, A_log=f(nv) * 0.5, dt_bias=f(nv),
                 conv_w=f(cd, ck) * 0.5, gnorm=f(dv))
        S = np.zeros((nv, dk, dv), np.float32)
        conv = np.zeros((cd, ck), np.float32)
        x = f(hidden)
        for name, arr in w.items():
            out[f"mixer_delta_{tag}_{name}"] = arr
        out[f"mixer_delta_{tag}_x"] = x
        xs = []
        for _ in range(3):
            x = ref.fused_delta_decode(x, w, S, conv, nk, nv, dk, dv, v_tiled=tiled)
            xs.append(x.copy())
        out[f"mixer_delta_{tag}_x_out"] = np.stack(xs)
        out[f"mixer_delta_{tag}_S_out"], out[f"mixer_delta_{tag}_conv_out"] = S, conv
        if tag == "grouped":     # nk = 1 makes both head maps equal; the tiled case uses nk = 2 below
            nk, nv = 2, 4
            cd = 2 * nk * dk + nv * dv
    n_q, n_kv, hd = 2, 1, 256
    w = dict(rms_w=f(hidden) * 0.1, Wq=f(n_q * 2 * hd, hidden) / 6, Wk=f(n_kv * hd, hidden) / 6,
             Wv=f(n_kv * hd, hidden) / 6, Wo=f(hidden, n_q * hd) / 20, q_norm=f(hd) * 0.1, k_norm=f(hd) * 0.1)
    kc = np.zeros((4, n_kv, hd), np.float32)
    vc = np.zeros((4, n_kv, hd), np.float32)
    x = f(hidden)
    for name, arr in w.items():
        out[f"mixer_attn_{name}"] = arr
    out["mixer_attn_x"] = x
    xs = []
    for pos in range(3):
        x = ref.fused_attn_decode(x, w, kc, vc, pos, n_q, n_kv, hd)
        xs.append(x.copy())
    out["mixer_attn_x_out"] = np.stack(xs)
    out["mixer_attn_k_cache"], out["mixer_attn_v_cache"] = kc, vc
    del os.environ["RAPIDLLM_SIMD"]

    path = os.path.join(HERE, "ref_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
