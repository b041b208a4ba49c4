"""ctypes bindings of the CPU checkers (TEST INFRASTRUCTURE ONLY).

`Oracle` wraps oracle/librl_oracle.so (the C restatement, rl_oracle.c);
`Reference` wraps oracle/_ref/librl_ref.so (the reference's own CPU operators
behind ref_shim.cpp) when that library has been built.  Only tests, the smoke
check and the bench's CPU-baseline / reference legs may import this package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "librl_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "librl_ref.so")
REF_CUDA_SO = os.path.join(_HERE, "_ref", "librl_refcuda.so")


def reference_tree() -> str:
    """Where the RapidLLM sources lie: $RAPIDLLM_REFERENCE, else a `reference` directory beside
    this repository; "" when neither exists (then only the restatement is built)."""
    cand = os.environ.get("RAPIDLLM_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.exists(os.path.join(cand, "src", "kernels", "ops.cpp")) else ""


def build(quiet: bool = True) -> None:
    """Compile the restatement (and the reference libraries when its tree is there)."""
    subprocess.run(["make", "-C", _HERE, "REF=" + reference_tree()], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


def _ptr(a, ct):
    return a.ctypes.data_as(C.POINTER(ct))


class Oracle:
    """numpy front-end of rl_oracle.c; every method names the C function it calls."""

    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build()
        self.lib = C.CDLL(ORACLE_SO)
        self.lib.rlo_tq3_centroids.restype = C.POINTER(C.c_float)
        self.lib.rlo_f16_to_f32.restype = C.c_float
        self.lib.rlo_f32_to_f16.restype = C.c_uint16
        self.lib.rlo_f32_to_f16.argtypes = [C.c_float]

    # -- attention ---------------------------------------------------------
    def attn_decode(self, q, k_cache, v_cache, pos=None):
        """rlo_attn_decode: q [n_q,hd], caches [seq,n_kv,hd] fp32 -> o [n_q,hd]."""
        q, qp = _f32(q)
        k, kp = _f32(k_cache)
        v, vp = _f32(v_cache)
        n_q, hd = q.shape
        n_kv = k.shape[1]
        if pos is None:
            pos = k.shape[0] - 1
        o = np.empty_like(q)
        self.lib.rlo_attn_decode(qp, kp, vp, _ptr(o, C.c_float), int(pos), n_q, n_kv, hd)
        return o

    def attn_prefill(self, q, k, v):
        """rlo_attn_prefill: q [T,n_q,hd], k/v [T,n_kv,hd] -> o [T,n_q,hd]."""
        q, qp = _f32(q)
        k, kp = _f32(k)
        v, vp = _f32(v)
        T, n_q, hd = q.shape
        o = np.empty_like(q)
        self.lib.rlo_attn_prefill(qp, kp, vp, _ptr(o, C.c_float), T, n_q, k.shape[1], hd)
        return o

    def attn_prefill_rows(self, q_rows, k_cache, v_cache, row_pos):
        """rlo_attn_prefill_rows: selected query rows at absolute positions row_pos."""
        q, qp = _f32(q_rows)
        k, kp = _f32(k_cache)
        v, vp = _f32(v_cache)
        rp = np.ascontiguousarray(row_pos, dtype=np.int32)
        o = np.empty_like(q)
        self.lib.rlo_attn_prefill_rows(qp, kp, vp, _ptr(o, C.c_float), _ptr(rp, C.c_int),
                                       len(rp), q.shape[1], k.shape[1], q.shape[2])
        return o

    def sigmoid_gate(self, o, gate):
        o = np.array(o, dtype=np.float32, order="C", copy=True)
        g, gp = _f32(gate)
        self.lib.rlo_sigmoid_gate(_ptr(o, C.c_float), gp, C.c_long(o.size))
        return o

    def gated_attn_decode(self, q, k_cache, v_cache, gate, pos=None):
        return self.sigmoid_gate(self.attn_decode(q, k_cache, v_cache, pos), gate)

    def attn_partial(self, qh, k_cache, v_cache, s0, s1, hkv):
        qh, qp = _f32(qh)
        k, kp = _f32(k_cache)
        v, vp = _f32(v_cache)
        hd = qh.shape[0]
        m = C.c_float()
        l = C.c_float()
        acc = np.empty(hd, np.float32)
        self.lib.rlo_attn_partial(qp, kp, vp, int(s0), int(s1), k.shape[1], int(hkv), hd,
                                  C.byref(m), C.byref(l), _ptr(acc, C.c_float))
        return m.value, l.value, acc

    def lse_combine(self, m, l, acc):
        m, mp = _f32(m)
        l, lp = _f32(l)
        acc, ap = _f32(acc)
        o = np.empty(acc.shape[1], np.float32)
        self.lib.rlo_lse_combine(mp, lp, ap, len(m), acc.shape[1], _ptr(o, C.c_float))
        return o

    # -- fp16 / paging -------------------------------------------------------
    def to_f16(self, x):
        x, xp = _f32(x)
        y = np.empty(x.shape, np.uint16)
        self.lib.rlo_f32_to_f16_n(xp, _ptr(y, C.c_uint16), C.c_long(x.size))
        return y

    def from_f16(self, x):
        x = np.ascontiguousarray(x, dtype=np.uint16)
        y = np.empty(x.shape, np.float32)
        self.lib.rlo_f16_to_f32_n(_ptr(x, C.c_uint16), _ptr(y, C.c_float), C.c_long(x.size))
        return y

    def paged_gather(self, pool, table, seq_len):
        """rlo_paged_gather_u16: pool [pages,n_kv,page_tokens,hd] u16 -> [seq,n_kv,hd]."""
        pool = np.ascontiguousarray(pool, dtype=np.uint16)
        table = np.ascontiguousarray(table, dtype=np.int32)
        _, n_kv, pt, hd = pool.shape
        out = np.empty((seq_len, n_kv, hd), np.uint16)
        self.lib.rlo_paged_gather_u16(_ptr(pool, C.c_uint16), _ptr(table, C.c_int32), int(seq_len),
                                      n_kv, pt, hd, _ptr(out, C.c_uint16))
        return out

    def paged_scatter(self, pool, table, s0, rows):
        """rlo_paged_scatter_u16 (in place on pool): rows [n,n_kv,hd] -> tokens s0.."""
        assert pool.dtype == np.uint16 and pool.flags.c_contiguous
        table = np.ascontiguousarray(table, dtype=np.int32)
        rows = np.ascontiguousarray(rows, dtype=np.uint16)
        _, n_kv, pt, hd = pool.shape
        self.lib.rlo_paged_scatter_u16(_ptr(pool, C.c_uint16), _ptr(table, C.c_int32), int(s0),
                                       int(s0 + rows.shape[0]), n_kv, pt, hd,
                                       _ptr(rows, C.c_uint16))

    # -- DeltaNet --------------------------------------------------------------
    def delta_step(self, S, q, k, v, beta, g_log, eps=1e-6):
        """rlo_delta_step: S [n_v,dk,dv] updated in place; returns o [n_v,dv]."""
        assert S.dtype == np.float32 and S.flags.c_contiguous
        q, qp = _f32(q)
        k, kp = _f32(k)
        v, vp = _f32(v)
        b, bp = _f32(beta)
        g, gp = _f32(g_log)
        n_v, dk, dv = S.shape
        o = np.empty((n_v, dv), np.float32)
        self.lib.rlo_delta_step(_ptr(S, C.c_float), qp, kp, vp, bp, gp, _ptr(o, C.c_float), n_v,
                                dk, dv, C.c_float(eps))
        return o

    def delta_prefill_seq(self, S, q, k, v, beta, g_log, eps=1e-6):
        """rlo_delta_prefill_seq: T sequential steps; q,k [T,n_v,dk] ..."""
        assert S.dtype == np.float32 and S.flags.c_contiguous
        q, qp = _f32(q)
        k, kp = _f32(k)
        v, vp = _f32(v)
        b, bp = _f32(beta)
        g, gp = _f32(g_log)
        n_v, dk, dv = S.shape
        T = q.shape[0]
        o = np.empty((T, n_v, dv), np.float32)
        self.lib.rlo_delta_prefill_seq(_ptr(S, C.c_float), qp, kp, vp, bp, gp, _ptr(o, C.c_float),
                                       T, n_v, dk, dv, C.c_float(eps))
        return o

    def repeat_heads(self, x, n_v, tiled=False):
        x, xp = _f32(x)
        n_k, d = x.shape
        y = np.empty((n_v, d), np.float32)
        self.lib.rlo_repeat_heads(xp, _ptr(y, C.c_float), n_k, n_v, d, int(tiled))
        return y

    def delta_gates(self, a, b, A_log, dt_bias):
        a, ap = _f32(a)
        b, bp = _f32(b)
        A, Ap = _f32(A_log)
        d, dp = _f32(dt_bias)
        beta = np.empty_like(a)
        g = np.empty_like(a)
        self.lib.rlo_delta_gates(ap, bp, Ap, dp, _ptr(beta, C.c_float), _ptr(g, C.c_float), a.size)
        return beta, g

    def l2norm(self, x, eps=1e-6):
        x, xp = _f32(x)
        y = np.empty_like(x)
        self.lib.rlo_l2norm(xp, _ptr(y, C.c_float), x.size, C.c_float(eps))
        return y

    def qwen3_rmsnorm(self, x, gamma, eps=1e-6):
        """rlo_qwen3_rmsnorm over the last axis: x [..., n], gamma [n] or None."""
        x, _ = _f32(x)
        y = np.empty_like(x)
        g = None if gamma is None else np.ascontiguousarray(gamma, np.float32)
        rows = x.reshape(-1, x.shape[-1])
        out = y.reshape(-1, x.shape[-1])
        for r in range(rows.shape[0]):
            self.lib.rlo_qwen3_rmsnorm(_ptr(rows[r], C.c_float), None if g is None else _ptr(g, C.c_float),
                                       _ptr(out[r], C.c_float), rows.shape[1], C.c_float(eps))
        return y

    def rope_partial(self, q, k, pos, rotary_dim=64, theta=1e7):
        """rlo_rope_partial: q [n_q,hd], k [n_kv,hd] -> rotated copies."""
        q = np.array(q, np.float32, order="C")
        k = np.array(k, np.float32, order="C")
        self.lib.rlo_rope_partial(_ptr(q, C.c_float), _ptr(k, C.c_float), q.shape[0], k.shape[0], q.shape[1],
                                  int(rotary_dim), int(pos), C.c_float(theta))
        return q, k

    def attn_qk_prepare(self, qg, k, q_norm, k_norm, pos, rotary_dim=64, theta=1e7, eps=1e-6):
        """rlo_attn_qk_prepare: qg [n_q, 2*hd] ([q | gate] per head), k [n_kv, hd] -> q, gate, k."""
        qg, qgp = _f32(qg)
        k = np.array(k, np.float32, order="C")
        qn, qnp = _f32(q_norm)
        kn, knp = _f32(k_norm)
        n_q, hd = qg.shape[0], qg.shape[1] // 2
        q = np.empty((n_q, hd), np.float32)
        gate = np.empty((n_q, hd), np.float32)
        self.lib.rlo_attn_qk_prepare(qgp, _ptr(k, C.c_float), qnp, knp, _ptr(q, C.c_float), _ptr(gate, C.c_float),
                                     n_q, k.shape[0], hd, int(rotary_dim), int(pos), C.c_float(theta),
                                     C.c_float(eps))
        return q, gate, k

    def gated_rmsnorm(self, x, z, gamma, eps=1e-6):
        """rlo_gated_rmsnorm: x, z [n]; gamma [gamma_n] (per head when gamma_n < n)."""
        x, xp = _f32(x)
        z, zp = _f32(z)
        g, gp = _f32(gamma)
        y = np.empty_like(x)
        self.lib.rlo_gated_rmsnorm(xp, zp, gp, _ptr(y, C.c_float), x.size, C.c_float(eps), g.size)
        return y

    def conv1d_update(self, x_t, w, state):
        """rlo_conv1d_update: state [dim,k] updated in place; returns y [dim]."""
        assert state.dtype == np.float32 and state.flags.c_contiguous
        x, xp = _f32(x_t)
        w, wp = _f32(w)
        dim, k = w.shape
        y = np.empty(dim, np.float32)
        self.lib.rlo_conv1d_update(xp, wp, _ptr(state, C.c_float), _ptr(y, C.c_float), dim, k)
        return y

    def conv1d_causal_prefill(self, x, w):
        x, xp = _f32(x)
        w, wp = _f32(w)
        seq, dim = x.shape
        y = np.empty_like(x)
        self.lib.rlo_conv1d_causal_prefill(xp, wp, _ptr(y, C.c_float), seq, dim, w.shape[1])
        return y

    # -- whole decode mixers ---------------------------------------------------
    def gemv(self, W, x):
        """rlo_gemv_f32: W [m,n] @ x [n] with a double accumulator in index order."""
        W, Wp = _f32(W)
        x, xp = _f32(x)
        y = np.empty(W.shape[0], np.float32)
        self.lib.rlo_gemv_f32(Wp, xp, _ptr(y, C.c_float), W.shape[0], W.shape[1])
        return y

    def fused_delta_decode(self, x, w, S, conv_state, n_k, n_v, dk=128, dv=128, eps=1e-6, v_tiled=False):
        """One token through a DeltaNet mixer, in the order of ops::fused_delta_decode
        (src/kernels/ops_fused.cpp:84-135): norm, four projections, conv + SiLU, head repeat and
        gate maths, the delta rule, gated RMSNorm, output projection, residual.  w: dict of
        rms_w, Wqkv, Wz, Wa, Wb, Wo, A_log, dt_bias, conv_w, gnorm.  S [n_v,dk,dv] and
        conv_state [conv_dim,k] are updated in place; returns the new hidden state."""
        x = np.asarray(x, np.float32)
        qdim = n_k * dk
        xn = self.qwen3_rmsnorm(x, w["rms_w"], eps)
        qkv, z = self.gemv(w["Wqkv"], xn), self.gemv(w["Wz"], xn)
        aa, bb = self.gemv(w["Wa"], xn), self.gemv(w["Wb"], xn)
        mixed = self.conv1d_update(qkv, w["conv_w"], conv_state)
        qh = self.repeat_heads(mixed[:qdim].reshape(n_k, dk), n_v, v_tiled)
        kh = self.repeat_heads(mixed[qdim:2 * qdim].reshape(n_k, dk), n_v, v_tiled)
        vh = mixed[2 * qdim:].reshape(n_v, dv)
        beta, g = self.delta_gates(aa, bb, w["A_log"], w["dt_bias"])
        o = self.delta_step(S, qh, kh, vh, beta, g, 1e-6)
        og = self.gated_rmsnorm(o.reshape(-1), z, w["gnorm"], 1e-6)
        return x + self.gemv(w["Wo"], og)

    def fused_attn_decode(self, x, w, k_cache, v_cache, pos, n_q, n_kv, hd=256, rotary_dim=64, theta=1e7,
                          eps=1e-6):
        """One token through a gated-attention mixer, in the order of ops::fused_attn_decode
        (src/kernels/ops_fused.cpp:137-182).  w: dict of rms_w, Wq ([q | gate] rows per head), Wk,
        Wv, Wo, q_norm, k_norm.  k_cache, v_cache fp32 [ctx,n_kv,hd] get row pos; returns the
        new hidden state."""
        x = np.asarray(x, np.float32)
        xn = self.qwen3_rmsnorm(x, w["rms_w"], eps)
        qg = self.gemv(w["Wq"], xn).reshape(n_q, 2 * hd)
        k = self.gemv(w["Wk"], xn).reshape(n_kv, hd)
        v = self.gemv(w["Wv"], xn).reshape(n_kv, hd)
        q, gate, k = self.attn_qk_prepare(qg, k, w["q_norm"], w["k_norm"], pos, rotary_dim, theta, eps)
        k_cache[pos], v_cache[pos] = k, v
        o = self.gated_attn_decode(q, k_cache[:pos + 1], v_cache[:pos + 1], gate)
        return x + self.gemv(w["Wo"], o.reshape(-1))

    # -- compact KV ------------------------------------------------------------
    def centroids(self):
        return np.ctypeslib.as_array(self.lib.rlo_tq3_centroids(), shape=(8,)).copy()

    def fwht(self, x):
        x = np.array(x, dtype=np.float32, order="C", copy=True)
        self.lib.rlo_fwht(_ptr(x, C.c_float), x.size)
        return x

    def compact_store(self, k, v, wht_len=128, signs=None):
        """rlo_compact_store: k,v [T,n_kv,hd] fp32 -> (k_q i8, k_sc u16, v_codes u8, v_sc u16)."""
        k, kp = _f32(k)
        v, vp = _f32(v)
        T, n_kv, hd = k.shape
        nblk = hd // wht_len
        k_q = np.empty((T, n_kv, hd), np.int8)
        k_sc = np.empty((T, n_kv), np.uint16)
        v_codes = np.empty((T, n_kv, hd * 3 // 8), np.uint8)
        v_sc = np.empty((T, n_kv, nblk), np.uint16)
        sp = None
        if signs is not None:
            signs, sp = _f32(signs)
        self.lib.rlo_compact_store(kp, vp, C.c_long(T), n_kv, hd, wht_len, sp, _ptr(k_q, C.c_int8),
                                   _ptr(k_sc, C.c_uint16), _ptr(v_codes, C.c_uint8),
                                   _ptr(v_sc, C.c_uint16))
        return k_q, k_sc, v_codes, v_sc

    def compact_dequant(self, k_q, k_sc, v_codes, v_sc, wht_len=128, signs=None):
        k_q = np.ascontiguousarray(k_q, np.int8)
        k_sc = np.ascontiguousarray(k_sc, np.uint16)
        v_codes = np.ascontiguousarray(v_codes, np.uint8)
        v_sc = np.ascontiguousarray(v_sc, np.uint16)
        T, n_kv, hd = k_q.shape
        k = np.empty((T, n_kv, hd), np.float32)
        v = np.empty((T, n_kv, hd), np.float32)
        sp = None
        if signs is not None:
            signs, sp = _f32(signs)
        self.lib.rlo_compact_dequant(_ptr(k_q, C.c_int8), _ptr(k_sc, C.c_uint16),
                                     _ptr(v_codes, C.c_uint8), _ptr(v_sc, C.c_uint16), C.c_long(T),
                                     n_kv, hd, wht_len, sp, _ptr(k, C.c_float), _ptr(v, C.c_float))
        return k, v


class Reference:
    """The reference's own CPU operators (oracle/_ref/librl_ref.so)."""

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        self.lib = C.CDLL(REF_SO)

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def simd_name(self) -> str:
        buf = C.create_string_buffer(128)
        self.lib.ref_simd_name(buf, 128)
        return buf.value.decode()

    def num_threads(self) -> int:
        return int(self.lib.ref_num_threads())

    def set_threads(self, n: int) -> None:
        self.lib.ref_set_threads(int(n))

    def attn_decode(self, q, k_cache, v_cache, pos=None):
        q, qp = _f32(q)
        k, kp = _f32(k_cache)
        v, vp = _f32(v_cache)
        if pos is None:
            pos = k.shape[0] - 1
        o = np.empty_like(q)
        self.lib.ref_attn_decode(qp, kp, vp, _ptr(o, C.c_float), int(pos), q.shape[0], k.shape[1],
                                 q.shape[1])
        return o

    def attn_prefill(self, q, k, v):
        q, qp = _f32(q)
        k, kp = _f32(k)
        v, vp = _f32(v)
        o = np.empty_like(q)
        self.lib.ref_attn_prefill(qp, kp, vp, _ptr(o, C.c_float), q.shape[0], q.shape[1],
                                  k.shape[1], q.shape[2])
        return o

    def delta_step(self, S, q, k, v, beta, g_log, eps=1e-6, simd=False):
        assert S.dtype == np.float32 and S.flags.c_contiguous
        q, qp = _f32(q)
        k, kp = _f32(k)
        v, vp = _f32(v)
        b, bp = _f32(beta)
        g, gp = _f32(g_log)
        n_v, dk, dv = S.shape
        o = np.empty((n_v, dv), np.float32)
        fn = self.lib.ref_delta_step_simd if simd else self.lib.ref_delta_step_scalar
        fn(_ptr(S, C.c_float), qp, kp, vp, bp, gp, _ptr(o, C.c_float), n_v, dk, dv, C.c_float(eps))
        return o

    def conv1d_update(self, x_t, w, state):
        assert state.dtype == np.float32 and state.flags.c_contiguous
        x, xp = _f32(x_t)
        w, wp = _f32(w)
        dim, k = w.shape
        y = np.empty(dim, np.float32)
        self.lib.ref_conv1d_update(xp, wp, _ptr(state, C.c_float), _ptr(y, C.c_float), dim, k)
        return y

    def conv1d_causal_prefill(self, x, w):
        x, xp = _f32(x)
        w, wp = _f32(w)
        y = np.empty_like(x)
        self.lib.ref_conv1d_causal_prefill(xp, wp, _ptr(y, C.c_float), x.shape[0], x.shape[1],
                                           w.shape[1])
        return y

    def qwen3_rmsnorm(self, x, gamma, eps=1e-6):
        x, xp = _f32(x)
        g, gp = _f32(gamma)
        y = np.empty_like(x)
        self.lib.ref_qwen3_rmsnorm(xp, gp, _ptr(y, C.c_float), x.size, C.c_float(eps))
        return y

    def rope_partial(self, q, k, pos, rotary_dim=64, theta=1e7):
        q = np.array(q, np.float32, order="C")
        k = np.array(k, np.float32, order="C")
        self.lib.ref_rope_partial(_ptr(q, C.c_float), _ptr(k, C.c_float), q.shape[0], k.shape[0], q.shape[1],
                                  int(rotary_dim), int(pos), C.c_float(theta))
        return q, k

    def gated_rmsnorm(self, x, z, gamma, eps=1e-6):
        x, xp = _f32(x)
        z, zp = _f32(z)
        g, gp = _f32(gamma)
        y = np.empty_like(x)
        self.lib.ref_gated_rmsnorm(xp, zp, gp, _ptr(y, C.c_float), x.size, C.c_float(eps), g.size)
        return y

    def fused_delta_decode(self, x, w, S, conv_state, n_k, n_v, dk=128, dv=128, eps=1e-6, v_tiled=False,
                           simd=False):
        """ops::fused_delta_decode with dense fp32 weights; S and conv_state updated in place."""
        assert S.dtype == np.float32 and S.flags.c_contiguous
        assert conv_state.dtype == np.float32 and conv_state.flags.c_contiguous
        x = np.array(x, np.float32, order="C")
        keep = [_f32(w[n]) for n in ("rms_w", "Wqkv", "Wz", "Wa", "Wb", "Wo", "A_log", "dt_bias", "conv_w",
                                     "gnorm")]
        self.lib.ref_fused_delta_decode(_ptr(x, C.c_float), *[p for _, p in keep], _ptr(S, C.c_float),
                                        _ptr(conv_state, C.c_float), x.size, n_k, n_v, dk, dv,
                                        conv_state.shape[1], C.c_float(eps), int(simd), int(v_tiled))
        return x

    def fused_attn_decode(self, x, w, k_cache, v_cache, pos, n_q, n_kv, hd=256, rotary_dim=64, theta=1e7,
                          eps=1e-6, simd=False):
        """ops::fused_attn_decode with dense fp32 weights; the caches get row pos."""
        assert k_cache.dtype == np.float32 and k_cache.flags.c_contiguous
        assert v_cache.dtype == np.float32 and v_cache.flags.c_contiguous
        x = np.array(x, np.float32, order="C")
        keep = [_f32(w[n]) for n in ("rms_w", "Wq", "Wk", "Wv", "Wo", "q_norm", "k_norm")]
        self.lib.ref_fused_attn_decode(_ptr(x, C.c_float), *[p for _, p in keep], _ptr(k_cache, C.c_float),
                                       _ptr(v_cache, C.c_float), x.size, n_q, n_kv, hd, int(rotary_dim),
                                       int(pos), C.c_float(theta), C.c_float(eps), int(simd))
        return x

    def l2norm(self, x, eps=1e-6):
        x, xp = _f32(x)
        y = np.empty_like(x)
        self.lib.ref_l2norm(xp, _ptr(y, C.c_float), x.size, C.c_float(eps))
        return y


class ReferenceCuda:
    """The reference's own CUDA kernels for the compact KV cache (oracle/_ref/librl_refcuda.so =
    its engine translation unit compiled in place behind ref_cuda_shim.cu).  Needs a GPU."""

    def __init__(self):
        if not os.path.exists(REF_CUDA_SO):
            raise FileNotFoundError(REF_CUDA_SO)
        self.lib = C.CDLL(REF_CUDA_SO)
        self.lib.rlref_cuda_error_string.restype = C.c_char_p

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_CUDA_SO)

    def _check(self, code, what):
        if code:
            raise RuntimeError("%s: %s" % (what, self.lib.rlref_cuda_error_string(code).decode()))

    def compact_store(self, k, v):
        """store_k_q8_th_k + store_v_tq3_th_k (cuda_engine.cu:8224-8284): k, v [T, n_kv, 256] fp32 ->
        (k_q i8 [T,n_kv,256], k_sc u16 [T,n_kv], v_codes u8 [T,n_kv,96], v_sc u16 [T,n_kv,2])."""
        k, kp = _f32(k)
        v, vp = _f32(v)
        T, n_kv, hd = k.shape
        assert hd == 256
        k_q = np.empty((T, n_kv, hd), np.int8)
        k_sc = np.empty((T, n_kv), np.uint16)
        v_codes = np.empty((T, n_kv, 96), np.uint8)
        v_sc = np.empty((T, n_kv, 2), np.uint16)
        self._check(self.lib.rlref_cuda_compact_store(kp, vp, T, n_kv, _ptr(k_q, C.c_int8), _ptr(k_sc, C.c_uint16),
                                                      _ptr(v_codes, C.c_uint8), _ptr(v_sc, C.c_uint16)),
                    "rlref_cuda_compact_store")
        return k_q, k_sc, v_codes, v_sc

    def compact_dequant(self, k_q, k_sc, v_codes, v_sc):
        """dequant_k_q8_h_k + dequant_v_tq3_h_k (cuda_engine.cu:8286-8314) -> k, v fp16 bits [T,n_kv,256]."""
        k_q = np.ascontiguousarray(k_q, np.int8)
        k_sc = np.ascontiguousarray(k_sc, np.uint16)
        v_codes = np.ascontiguousarray(v_codes, np.uint8)
        v_sc = np.ascontiguousarray(v_sc, np.uint16)
        T, n_kv, hd = k_q.shape
        k16 = np.empty((T, n_kv, hd), np.uint16)
        v16 = np.empty((T, n_kv, hd), np.uint16)
        self._check(self.lib.rlref_cuda_compact_dequant(_ptr(k_q, C.c_int8), _ptr(k_sc, C.c_uint16),
                                                        _ptr(v_codes, C.c_uint8), _ptr(v_sc, C.c_uint16), T, n_kv,
                                                        _ptr(k16, C.c_uint16), _ptr(v16, C.c_uint16)),
                    "rlref_cuda_compact_dequant")
        return k16.view(np.float16), v16.view(np.float16)

    def attn_decode_tq(self, q, k_q, k_sc, v_codes, v_sc, pos=None):
        """qk_attn_decode_tq_gqa_k (cuda_engine.cu:8382-8454): q [n_q,256] over tokens [0, pos]."""
        q, qp = _f32(q)
        k_q = np.ascontiguousarray(k_q, np.int8)
        k_sc = np.ascontiguousarray(k_sc, np.uint16)
        v_codes = np.ascontiguousarray(v_codes, np.uint8)
        v_sc = np.ascontiguousarray(v_sc, np.uint16)
        T, n_kv, _ = k_q.shape
        pos = T - 1 if pos is None else pos
        o = np.empty_like(q)
        self._check(self.lib.rlref_cuda_attn_decode_tq(qp, int(pos), q.shape[0], n_kv, _ptr(k_q, C.c_int8),
                                                       _ptr(k_sc, C.c_uint16), _ptr(v_codes, C.c_uint8),
                                                       _ptr(v_sc, C.c_uint16), T, _ptr(o, C.c_float)),
                    "rlref_cuda_attn_decode_tq")
        return o
