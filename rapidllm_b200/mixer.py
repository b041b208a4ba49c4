"""Whole decode mixers: what ops::fused_delta_decode and ops::fused_attn_decode do to one token's
hidden state (src/kernels/ops_fused.cpp:84-135, 137-182), for a batch of sequences on the device.

    x -> RMSNorm (1 + gamma) -> input projections -> [conv + SiLU, gate maths | q/gate split, head
    norms, partial RoPE, KV append] -> delta rule | attention over the paged cache -> gated RMSNorm |
    sigmoid gate -> output projection -> x + y

The operators and the steps either side of them are this library's kernels; the dense projections
are plain library GEMMs (torch.matmul), one for all input projections of a mixer and one for the
output.  Weights are fp32 as in FusedDeltaArgs / FusedAttnArgs with QuantKind::F32; `weight_dtype`
stores them narrower for the GEMMs.  Both classes keep no host copy of any position: the attention
mixer takes device-resident positions like the stack entry points.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib, ops
from ._lib import DeltaRecurrentParams, check, lib


def _matmul(x, w):
    if w.dtype == torch.float32:
        return x @ w.t()
    return (x.to(w.dtype) @ w.t()).float()


class DeltaNetMixer:
    """w: rms_w [hidden], Wqkv [2*n_k*dk + n_v*dv, hidden], Wz [n_v*dv, hidden], Wa, Wb [n_v, hidden],
    Wo [hidden, n_v*dv], A_log, dt_bias [n_v], conv_w [conv_dim, k], gnorm [dv]."""

    def __init__(self, w: dict, n_k=16, n_v=48, dk=128, dv=128, n_slots=1, eps=1e-6, head_map=None,
                 weight_dtype=torch.float32, device="cuda"):
        self.n_k, self.n_v, self.dk, self.dv, self.eps = n_k, n_v, dk, dv, eps
        self.head_map = _lib.RL_HEADS_GROUPED if head_map is None else head_map
        dev = lambda t: torch.as_tensor(t).to(device=device, dtype=torch.float32).contiguous()  # noqa: E731
        self.qdim, self.zdim = n_k * dk, n_v * dv
        self.conv_dim = 2 * self.qdim + self.zdim
        # one GEMM for qkv | z | a | b
        self.W_in = torch.cat([dev(w["Wqkv"]), dev(w["Wz"]), dev(w["Wa"]), dev(w["Wb"])]).to(weight_dtype)
        self.W_out = dev(w["Wo"]).to(weight_dtype)
        self.rms_w, self.A_log, self.dt_bias = dev(w["rms_w"]), dev(w["A_log"]), dev(w["dt_bias"])
        self.conv_w, self.gnorm = dev(w["conv_w"]), dev(w["gnorm"])
        self.S = torch.zeros(n_slots, n_v, dk, dv, dtype=torch.float32, device=device)
        self.conv_state = torch.zeros(n_slots, self.conv_dim, self.conv_w.shape[1], dtype=torch.float32, device=device)

    def decode(self, x, slot_ids=None):
        """x fp32 [batch][hidden] -> the new hidden state; state of slot_ids[b] (or b) advances."""
        B = x.shape[0]
        xn = ops.rmsnorm(x, self.rms_w, self.eps)
        proj = _matmul(xn, self.W_in)
        cd, zd, nv = self.conv_dim, self.zdim, self.n_v
        qkv = proj[:, :cd].contiguous()
        z = proj[:, cd:cd + zd].contiguous()
        a = proj[:, cd + zd:cd + zd + nv].contiguous()
        b = proj[:, cd + zd + nv:].contiguous()
        mixed = ops.conv1d_update(qkv, self.conv_w, self.conv_state, slot_ids)
        beta, g = ops.delta_gates(a, b, self.A_log, self.dt_bias)
        # q | k | v are column ranges of `mixed`: passed as strided views, no copies
        o = torch.empty(B, nv, self.dv, dtype=torch.float32, device=x.device)
        p = DeltaRecurrentParams(n_v=nv, dk=self.dk, dv=self.dv, eps_l2=1e-6, batch=B, n_slots=self.S.shape[0],
                                 n_qk=self.n_k, head_map=self.head_map, q_stride=cd, k_stride=cd, v_stride=cd)
        base = mixed.data_ptr()
        check(lib().rl_delta_recurrent(ops._p(self.S), ops._p(slot_ids), C.c_void_p(base),
                                       C.c_void_p(base + 4 * self.qdim), C.c_void_p(base + 8 * self.qdim),
                                       ops._p(beta), ops._p(g), ops._p(o), C.byref(p), ops._stream()))
        og = ops.gated_rmsnorm(o, z.view(B, nv, self.dv), self.gnorm, 1e-6)
        return x + _matmul(og.view(B, zd), self.W_out)


    def prefill(self, x, slot=0, start=True, workspace=None):
        """A chunk of one sequence's prompt: x fp32 [T][hidden] -> new hidden states; the slot's state and
        conv window advance by T tokens (start=True: the sequence begins here, state zero, window empty).
        Same arithmetic as T decode steps, with the delta rule in its chunked form."""
        T = x.shape[0]
        cd, zd, nv = self.conv_dim, self.zdim, self.n_v
        xn = ops.rmsnorm(x, self.rms_w, self.eps)
        proj = _matmul(xn, self.W_in)
        qkv = proj[:, :cd].contiguous()
        z = proj[:, cd:cd + zd].contiguous()
        a = proj[:, cd + zd:cd + zd + nv].contiguous()
        b = proj[:, cd + zd + nv:].contiguous()
        if start:
            self.S[slot].zero_()
        mixed = ops.conv1d_causal_prefill(qkv, self.conv_w, self.conv_state[slot], use_state_in=not start)
        beta, g = ops.delta_gates(a, b, self.A_log, self.dt_bias)
        p = _lib.DeltaChunkParams(n_v=nv, dk=self.dk, dv=self.dv, seq=T, chunk=64, eps_l2=1e-6, n_qk=self.n_k,
                                  head_map=self.head_map, qk_tok_stride=cd, v_tok_stride=cd)
        need = lib().rl_delta_chunk_workspace_bytes(C.byref(p))
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
        o = torch.empty(T, nv, self.dv, dtype=torch.float32, device=x.device)
        base = mixed.data_ptr()
        check(lib().rl_delta_chunk_prefill(ops._p(self.S[slot]), C.c_void_p(base), C.c_void_p(base + 4 * self.qdim),
                                           C.c_void_p(base + 8 * self.qdim), ops._p(beta), ops._p(g), ops._p(o),
                                           ops._p(workspace), workspace.numel(), C.byref(p), ops._stream()))
        og = ops.gated_rmsnorm(o, z.view(T, nv, self.dv), self.gnorm, 1e-6)
        return x + _matmul(og.view(T, zd), self.W_out)


class GatedAttentionMixer:
    """w: rms_w [hidden], Wq [n_q*2*hd, hidden] ([q | gate] rows per head), Wk, Wv [n_kv*hd, hidden],
    Wo [hidden, n_q*hd], q_norm, k_norm [hd].  The KV cache is paged F16 (k_pool, v_pool)."""

    def __init__(self, w: dict, n_pages, n_q=24, n_kv=4, hd=256, rotary_dim=64, theta=1e7, eps=1e-6,
                 weight_dtype=torch.float32, device="cuda"):
        self.n_q, self.n_kv, self.hd, self.rotary_dim, self.theta, self.eps = n_q, n_kv, hd, rotary_dim, theta, eps
        dev = lambda t: torch.as_tensor(t).to(device=device, dtype=torch.float32).contiguous()  # noqa: E731
        self.W_in = torch.cat([dev(w["Wq"]), dev(w["Wk"]), dev(w["Wv"])]).to(weight_dtype)
        self.W_out = dev(w["Wo"]).to(weight_dtype)
        self.rms_w, self.q_norm, self.k_norm = dev(w["rms_w"]), dev(w["q_norm"]), dev(w["k_norm"])
        self.k_pool, self.v_pool = ops.new_pool(n_pages, n_kv, device), ops.new_pool(n_pages, n_kv, device)

    def decode(self, x, page_table, pos):
        """x fp32 [batch][hidden]; page_table int32 [batch][max_pages]; pos int32 [batch] on the
        device (the index this token is written at; it attends to rows 0 .. pos)."""
        B = x.shape[0]
        qn, kn = self.n_q * self.hd, self.n_kv * self.hd
        xn = ops.rmsnorm(x, self.rms_w, self.eps)
        proj = _matmul(xn, self.W_in)
        qg = proj[:, :2 * qn].contiguous().view(B, self.n_q, 2 * self.hd)
        k = proj[:, 2 * qn:2 * qn + kn].contiguous().view(B, self.n_kv, self.hd)
        v = proj[:, 2 * qn + kn:].contiguous().view(B, self.n_kv, self.hd)
        q, gate = ops.attn_qk_prepare(qg, k, self.q_norm, self.k_norm, pos=pos, rotary_dim=self.rotary_dim,
                                      theta=self.theta, eps=self.eps)
        ops.kv_append(self.k_pool, self.v_pool, page_table, k.unsqueeze(1), v.unsqueeze(1), pos=pos)
        o = ops.attn_decode(q, self.k_pool, self.v_pool, page_table, pos + 1, gate)
        return x + _matmul(o.view(B, qn), self.W_out)


class MixerStack:
    """The mixers of a hybrid model in layer order, as Session::forward_hidden walks
    ModelDesc.layers (src/runtime/session.cpp:325-411; slot = index among the layers of a kind,
    src/runtime/model_desc.cpp:12-22), without the MLP blocks between them: one decode token of
    every sequence goes through every layer's mixer, the hidden state carrying the residual.

    layer_types: RL_LAYER_* per layer; weights: one dict per layer (see the two mixer classes).
    All attention layers share page_table / pos; every DeltaNet layer keeps its own state per slot."""

    def __init__(self, layer_types, weights, n_pages, n_slots, device="cuda", **dims):
        self.layers = []
        for kind, w in zip(layer_types, weights):
            if kind == _lib.RL_LAYER_FULL_ATTENTION:
                keys = ("n_q", "n_kv", "hd", "rotary_dim", "theta", "eps", "weight_dtype")
                self.layers.append(GatedAttentionMixer(w, n_pages, device=device,
                                                       **{k: v for k, v in dims.items() if k in keys}))
            else:
                keys = ("n_k", "n_v", "dk", "dv", "eps", "head_map", "weight_dtype")
                self.layers.append(DeltaNetMixer(w, n_slots=n_slots, device=device,
                                                 **{k: v for k, v in dims.items() if k in keys}))

    def decode(self, x, page_table, pos, slot_ids=None):
        """x fp32 [batch][hidden] -> hidden state after the last mixer; pos int32 [batch] on the device is
        the position the token is written at (the caller advances it between steps)."""
        for layer in self.layers:
            if isinstance(layer, GatedAttentionMixer):
                x = layer.decode(x, page_table, pos)
            else:
                x = layer.decode(x, slot_ids)
        return x


def _attn_prefill(self, x, page_table_row, pos0):
    """A chunk of one sequence's prompt: x fp32 [T][hidden] at positions pos0 .. pos0+T-1 -> new hidden
    states; K/V rows go into the cache as fp16 (round to nearest even, like decode), the query rows reach
    the tensor cores as bf16."""
    T = x.shape[0]
    qn, kn = self.n_q * self.hd, self.n_kv * self.hd
    xn = ops.rmsnorm(x, self.rms_w, self.eps)
    proj = _matmul(xn, self.W_in)
    qg = proj[:, :2 * qn].contiguous().view(T, self.n_q, 2 * self.hd)
    k = proj[:, 2 * qn:2 * qn + kn].contiguous().view(T, self.n_kv, self.hd)
    v = proj[:, 2 * qn + kn:].contiguous().view(T, self.n_kv, self.hd)
    q, gate = ops.attn_qk_prepare(qg, k, self.q_norm, self.k_norm, pos0=pos0, rotary_dim=self.rotary_dim,
                                  theta=self.theta, eps=self.eps)
    ops.kv_append(self.k_pool, self.v_pool, page_table_row, k, v, pos0=pos0)
    o = ops.attn_prefill(q.bfloat16(), self.k_pool, self.v_pool, page_table_row, pos0, None, None, gate)
    return x + _matmul(o.view(T, qn), self.W_out)


GatedAttentionMixer.prefill = _attn_prefill
