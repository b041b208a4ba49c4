"""Operator-level mirror of rapidllm::ops for torch CUDA tensors.

Same names and argument meaning as include/rapidllm/kernels/ops.h:118-131;
every function enqueues on the current torch stream through the C ABI and
raises RlError on a bad argument.  No CPU path exists here.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import (AttnDecodeParams, AttnPrefillParams, Conv1dParams, DeltaChunkParams,
                   DeltaRecurrentParams, KvAppendParams, check, lib)

PAGE_TOKENS = 64
HEAD_DIM = 256


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _need(t, dtype, name):
    if t is None:
        return
    if not (t.is_cuda and t.dtype == dtype and t.is_contiguous()):
        raise _lib.RlError(6, f"{name}: need a contiguous CUDA tensor of {dtype}")


def kv_slice_index(tok: torch.Tensor, d: torch.Tensor) -> torch.Tensor:
    """Offset (in halves) of element (tok, d) inside one (page, head) slice."""
    sub = d >> 6
    chunk = ((d & 63) >> 3) ^ (tok & 7)
    return sub * (PAGE_TOKENS * 64) + tok * 64 + chunk * 8 + (d & 7)


def new_pool(n_pages: int, n_kv: int, device="cuda") -> torch.Tensor:
    """A zeroed fp16 pool [n_pages][n_kv][64*256] for K or V."""
    return torch.zeros(n_pages, n_kv, PAGE_TOKENS * HEAD_DIM, dtype=torch.float16, device=device)


def kv_append(k_pool, v_pool, page_table, k_rows, v_rows, pos=None, pos0=0):
    """Write rows [batch][n_tok][n_kv][256] (fp32 -> fp16 RNE, or fp16) at pos[b] (+0..n_tok-1)."""
    n_pages, n_kv = k_pool.shape[0], k_pool.shape[1]
    if k_rows.dim() == 3:
        k_rows, v_rows = k_rows.unsqueeze(0), v_rows.unsqueeze(0)
    if page_table.dim() == 1:
        page_table = page_table.unsqueeze(0)
    kind = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}.get(k_rows.dtype)
    if kind is None:
        raise _lib.RlError(6, "k_rows: need fp32, fp16 or bf16")
    _need(k_rows, k_rows.dtype, "k_rows")
    _need(v_rows, k_rows.dtype, "v_rows")
    _need(page_table, torch.int32, "page_table")
    _need(pos, torch.int32, "pos")
    p = KvAppendParams(n_kv=n_kv, head_dim=HEAD_DIM, batch=k_rows.shape[0], n_tok=k_rows.shape[1],
                       page_tokens=PAGE_TOKENS, n_pages=n_pages,
                       max_pages_per_seq=page_table.shape[1], pos0=pos0, rows_fp16=kind)
    check(lib().rl_kv_append(_p(k_pool), _p(v_pool), _p(page_table), _p(pos), _p(k_rows),
                             _p(v_rows), C.byref(p), _stream()))


def kv_gather(pool, page_table_row, n_tok):
    """Tokens [0, n_tok) of one sequence as contiguous fp16 [n_tok][n_kv][256]."""
    n_pages, n_kv = pool.shape[0], pool.shape[1]
    _need(page_table_row, torch.int32, "page_table_row")
    out = torch.empty(n_tok, n_kv, HEAD_DIM, dtype=torch.float16, device=pool.device)
    check(lib().rl_kv_gather(_p(pool), _p(page_table_row), _p(out), n_tok, n_kv, HEAD_DIM, n_pages,
                             _stream()))
    return out


def new_compact_pool(n_pages: int, n_kv: int, device="cuda") -> torch.Tensor:
    """A zeroed byte pool [n_pages][n_kv][page bytes] for the q8-K / TQ3-V cache."""
    return torch.zeros(n_pages, n_kv, lib().rl_kv_compact_page_bytes(), dtype=torch.uint8, device=device)


def kv_compact_append(pool, page_table, k_rows, v_rows, wht_len=128, signs=None, pos=None, pos0=0):
    """Quantise fp32 rows [batch][n_tok][n_kv][256] into the compact cache at pos[b] (+0..n_tok-1)."""
    n_pages, n_kv = pool.shape[0], pool.shape[1]
    if k_rows.dim() == 3:
        k_rows, v_rows = k_rows.unsqueeze(0), v_rows.unsqueeze(0)
    if page_table.dim() == 1:
        page_table = page_table.unsqueeze(0)
    for t, n in ((k_rows, "k_rows"), (v_rows, "v_rows"), (signs, "signs")):
        _need(t, torch.float32, n)
    _need(page_table, torch.int32, "page_table")
    _need(pos, torch.int32, "pos")
    p = KvAppendParams(n_kv=n_kv, head_dim=HEAD_DIM, batch=k_rows.shape[0], n_tok=k_rows.shape[1],
                       page_tokens=PAGE_TOKENS, n_pages=n_pages,
                       max_pages_per_seq=page_table.shape[1], pos0=pos0, rows_fp16=0, wht_len=wht_len)
    check(lib().rl_kv_compact_append(_p(pool), _p(page_table), _p(pos), _p(k_rows), _p(v_rows),
                                     _p(signs), C.byref(p), _stream()))


def kv_compact_gather(pool, page_table_row, n_tok, wht_len=128):
    """Codes and scales of tokens [0, n_tok) in the reference's packing:
    (k_q int8 [n,n_kv,256], k_sc fp16 [n,n_kv], v_codes u8 [n,n_kv,96], v_sc fp16 [n,n_kv,256/wht])."""
    n_pages, n_kv = pool.shape[0], pool.shape[1]
    dev = pool.device
    k_q = torch.empty(n_tok, n_kv, HEAD_DIM, dtype=torch.int8, device=dev)
    k_sc = torch.empty(n_tok, n_kv, dtype=torch.float16, device=dev)
    v_codes = torch.empty(n_tok, n_kv, 96, dtype=torch.uint8, device=dev)
    v_sc = torch.empty(n_tok, n_kv, HEAD_DIM // wht_len, dtype=torch.float16, device=dev)
    check(lib().rl_kv_compact_gather(_p(pool), _p(page_table_row), _p(k_q), _p(k_sc), _p(v_codes),
                                     _p(v_sc), n_tok, n_kv, n_pages, wht_len, _stream()))
    return k_q, k_sc, v_codes, v_sc


def attn_params(n_q, n_kv, batch, n_pages, max_pages_per_seq, max_seq_len, len_add=0,
                chunk_pages=0, kv_dtype=_lib.RL_KV_F16, wht_len=128, signs=None):
    return AttnDecodeParams(n_q=n_q, n_kv=n_kv, head_dim=HEAD_DIM, kv_dtype=kv_dtype,
                            batch=batch, page_tokens=PAGE_TOKENS, n_pages=n_pages,
                            max_pages_per_seq=max_pages_per_seq, max_seq_len=max_seq_len,
                            len_add=len_add, chunk_pages=chunk_pages, wht_len=wht_len,
                            tq_signs=None if signs is None else signs.data_ptr())


def attn_decode(q, k_pool, v_pool, page_table, seq_lens, gate=None, max_seq_len=None,
                chunk_pages=0, workspace=None, out=None, partial=False, wht_len=128, signs=None):
    """ops::attn_decode for a ragged batch over the paged F16 cache, then o *= sigmoid(gate).

    q, gate [batch][n_q][256] fp32; page_table int32 [batch][max_pages]; seq_lens int32
    [batch] on the device.  With partial=True returns (part_o, part_ml) per (sequence,
    head) for a cross-GPU merge with lse_combine.  A uint8 k_pool (new_compact_pool) selects
    the q8-K / TQ3-V cache (v_pool is then ignored; wht_len 128 or 256, signs for 256).
    """
    _need(q, torch.float32, "q")
    _need(gate, torch.float32, "gate")
    _need(page_table, torch.int32, "page_table")
    _need(seq_lens, torch.int32, "seq_lens")
    batch, n_q, _ = q.shape
    n_pages, n_kv = k_pool.shape[0], k_pool.shape[1]
    if max_seq_len is None:
        max_seq_len = page_table.shape[1] * PAGE_TOKENS
    compact = k_pool.dtype == torch.uint8
    _need(signs, torch.float32, "signs")
    p = attn_params(n_q, n_kv, batch, n_pages, page_table.shape[1], max_seq_len, 0, chunk_pages,
                    _lib.RL_KV_Q8K_TQ3V if compact else _lib.RL_KV_F16, wht_len, signs)
    need = lib().rl_attn_decode_workspace_bytes(C.byref(p))
    if need == 0 and batch > 0:
        raise _lib.RlError(6, lib().rl_last_error().decode())
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    o = out if out is not None else torch.empty_like(q)
    if partial:
        ml = torch.empty(batch, n_q, 2, dtype=torch.float32, device=q.device)
        check(lib().rl_attn_decode_partial(_p(k_pool), _p(v_pool), _p(page_table), _p(seq_lens),
                                           _p(q), _p(o), _p(ml), _p(workspace), workspace.numel(),
                                           C.byref(p), _stream()))
        return o, ml
    check(lib().rl_attn_decode(_p(k_pool), _p(v_pool), _p(page_table), _p(seq_lens), _p(q),
                               _p(gate), _p(o), _p(workspace), workspace.numel(), C.byref(p),
                               _stream()))
    return o


def attn_prefill(q, k_pool, v_pool, page_table_row, pos0=0, k_rows=None, v_rows=None, gate=None, split=True,
                 workspace=None):
    """ops::attn_prefill for one chunk of one sequence over the paged F16 cache.

    q bf16 [T][n_q][256]; k_rows, v_rows bf16 [T][n_kv][256] are appended at pos0 first (or the
    cache already holds them); row t attends to cache rows [0, pos0 + t]; o *= sigmoid(gate).
    """
    _need(q, torch.bfloat16, "q")
    _need(k_rows, torch.bfloat16, "k_rows")
    _need(v_rows, torch.bfloat16, "v_rows")
    _need(gate, torch.float32, "gate")
    _need(page_table_row, torch.int32, "page_table_row")
    T, n_q, _ = q.shape
    n_pages, n_kv = k_pool.shape[0], k_pool.shape[1]
    o = torch.empty(T, n_q, HEAD_DIM, dtype=torch.float32, device=q.device)
    p = AttnPrefillParams(n_q=n_q, n_kv=n_kv, head_dim=HEAD_DIM, seq=T, br=128, bc=64, pos0=pos0,
                          page_tokens=PAGE_TOKENS, n_pages=n_pages, n_table=page_table_row.numel())
    need = lib().rl_attn_prefill_workspace_bytes(C.byref(p))
    ws = None
    if need and split:
        ws = workspace if workspace is not None and workspace.numel() >= need else \
            torch.empty(need, dtype=torch.uint8, device=q.device)
    check(lib().rl_attn_prefill_ws(_p(k_pool), _p(v_pool), _p(page_table_row), _p(q), _p(k_rows),
                                   _p(v_rows), _p(gate), _p(o), _p(ws), 0 if ws is None else ws.numel(),
                                   C.byref(p), _stream()))
    return o


def lse_combine(part_o, part_ml, gate=None, wht_len=0, signs=None):
    """Merge partials [n_parts][rows][256] / [n_parts][rows][2] -> o [rows][256]
    (wht_len 128/256: partials of the compact cache, still in the rotated domain)."""
    _need(part_o, torch.float32, "part_o")
    _need(part_ml, torch.float32, "part_ml")
    n_parts, rows, hd = part_o.shape
    o = torch.empty(rows, hd, dtype=torch.float32, device=part_o.device)
    check(lib().rl_lse_combine(_p(part_o), _p(part_ml), _p(gate), _p(o), n_parts, rows, hd,
                               wht_len, _p(signs), _stream()))
    return o


def delta_recurrent_step(S, q, k, v, beta, g_log, eps_l2=1e-6, slot_ids=None, head_map=None,
                         out=None):
    """ops::delta_recurrent_step for a batch; S [n_slots][n_v][128][128] fp32 in place.

    q,k [batch][n_qk][128]; v [batch][n_v][128]; beta,g_log [batch][n_v]; returns o.
    A 3-D S / 2-D q,k,v (the reference's single-sequence shapes) are accepted.
    """
    single = S.dim() == 3
    if single:
        S, q, k, v = S.unsqueeze(0), q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0)
        beta, g_log = beta.unsqueeze(0), g_log.unsqueeze(0)
    for t, n in ((S, "S"), (q, "q"), (k, "k"), (v, "v"), (beta, "beta"), (g_log, "g_log")):
        _need(t, torch.float32, n)
    _need(slot_ids, torch.int32, "slot_ids")
    n_slots, n_v, dk, dv = S.shape
    batch, n_qk = q.shape[0], q.shape[1]
    if head_map is None:
        head_map = _lib.RL_HEADS_PER_VALUE if n_qk == n_v else _lib.RL_HEADS_GROUPED
    o = out if out is not None else torch.empty(batch, n_v, dv, dtype=torch.float32, device=S.device)
    p = DeltaRecurrentParams(n_v=n_v, dk=dk, dv=dv, eps_l2=eps_l2, batch=batch, n_slots=n_slots,
                             n_qk=n_qk, head_map=head_map, q_stride=0, k_stride=0, v_stride=0)
    check(lib().rl_delta_recurrent(_p(S), _p(slot_ids), _p(q), _p(k), _p(v), _p(beta), _p(g_log),
                                   _p(o), C.byref(p), _stream()))
    return o[0] if single else o


def delta_recurrent_multi(S, q, k, v, beta, g_log, eps_l2=1e-6, slot_ids=None, head_map=None, backup=None):
    """n_tok consecutive delta-rule steps per sequence in one pass (speculative verify).

    S [n_slots][n_v][128][128] in place; q,k [batch][n_tok][n_qk][128]; v [batch][n_tok][n_v][128];
    beta,g_log [batch][n_tok][n_v]; backup (same shape as S) receives the touched heads' state
    before the first token.  Returns o [batch][n_tok][n_v][128]."""
    for t, n in ((S, "S"), (q, "q"), (k, "k"), (v, "v"), (beta, "beta"), (g_log, "g_log"), (backup, "backup")):
        _need(t, torch.float32, n)
    _need(slot_ids, torch.int32, "slot_ids")
    n_slots, n_v, dk, dv = S.shape
    batch, n_tok, n_qk = q.shape[0], q.shape[1], q.shape[2]
    if head_map is None:
        head_map = _lib.RL_HEADS_PER_VALUE if n_qk == n_v else _lib.RL_HEADS_GROUPED
    o = torch.empty(batch, n_tok, n_v, dv, dtype=torch.float32, device=S.device)
    p = DeltaRecurrentParams(n_v=n_v, dk=dk, dv=dv, eps_l2=eps_l2, batch=batch, n_slots=n_slots,
                             n_qk=n_qk, head_map=head_map, q_stride=0, k_stride=0, v_stride=0)
    check(lib().rl_delta_recurrent_multi(_p(S), _p(backup), _p(slot_ids), _p(q), _p(k), _p(v), _p(beta),
                                         _p(g_log), _p(o), C.byref(p), n_tok, 0, 0, _stream()))
    return o


def delta_chunk_prefill(S, q, k, v, beta, g_log, eps_l2=1e-6, head_map=None, workspace=None):
    """T delta-rule steps of one sequence in chunked (WY) form: the result of T calls of
    ops::delta_recurrent_step.  S [n_v][128][128] fp32 in place; q,k [T][n_qk][128];
    v [T][n_v][128]; beta,g_log [T][n_v]; returns o [T][n_v][128]."""
    for t, n in ((S, "S"), (q, "q"), (k, "k"), (v, "v"), (beta, "beta"), (g_log, "g_log")):
        _need(t, torch.float32, n)
    n_v, dk, dv = S.shape
    T, n_qk = q.shape[0], q.shape[1]
    if head_map is None:
        head_map = _lib.RL_HEADS_PER_VALUE if n_qk == n_v else _lib.RL_HEADS_GROUPED
    p = DeltaChunkParams(n_v=n_v, dk=dk, dv=dv, seq=T, chunk=64, eps_l2=eps_l2, n_qk=n_qk, head_map=head_map)
    need = lib().rl_delta_chunk_workspace_bytes(C.byref(p))
    if need == 0 and T > 0:
        raise _lib.RlError(6, lib().rl_last_error().decode())
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=S.device)
    o = torch.empty(T, n_v, dv, dtype=torch.float32, device=S.device)
    check(lib().rl_delta_chunk_prefill(_p(S), _p(q), _p(k), _p(v), _p(beta), _p(g_log), _p(o), _p(workspace),
                                       workspace.numel(), C.byref(p), _stream()))
    return o


def conv1d_update(x_t, w, state, slot_ids=None):
    """ops::conv1d_update: state [n_slots][dim][k] (or [dim][k]) in place; x_t [batch][dim]."""
    single = x_t.dim() == 1
    if single:
        x_t, state = x_t.unsqueeze(0), state.unsqueeze(0)
    for t, n in ((x_t, "x_t"), (w, "w"), (state, "state")):
        _need(t, torch.float32, n)
    batch, dim = x_t.shape
    y = torch.empty_like(x_t)
    p = Conv1dParams(dim=dim, k=w.shape[1], silu=1, batch=batch, n_slots=state.shape[0])
    check(lib().rl_conv1d_update(_p(x_t), _p(w), _p(state), _p(slot_ids), _p(y), C.byref(p),
                                 _stream()))
    return y[0] if single else y


def conv1d_causal_prefill(x, w, state=None, use_state_in=False):
    """ops::conv1d_causal_prefill over x [seq][dim]; optional [dim][k] window in/out."""
    _need(x, torch.float32, "x")
    _need(w, torch.float32, "w")
    _need(state, torch.float32, "state")
    seq, dim = x.shape
    y = torch.empty_like(x)
    p = Conv1dParams(dim=dim, k=w.shape[1], silu=1, batch=1, n_slots=1)
    check(lib().rl_conv1d_causal(_p(x), _p(w), _p(y), _p(state), seq, C.byref(p),
                                 int(use_state_in), _stream()))
    return y


def attn_qk_prepare(qg, k, q_norm=None, k_norm=None, pos=None, pos0=0, rotary_dim=64, theta=1e7, eps=1e-6):
    """The steps of fused_attn_decode between the projections and the cache append: split
    qg [rows][n_q][512] into q and gate, head RMSNorm (1 + gamma) of q and k, partial RoPE at
    pos [rows] (int32) or pos0 + row.  k [rows][n_kv][256] is updated in place; returns q, gate."""
    for t, n in ((qg, "qg"), (k, "k"), (q_norm, "q_norm"), (k_norm, "k_norm")):
        _need(t, torch.float32, n)
    _need(pos, torch.int32, "pos")
    rows, n_q, two_hd = qg.shape
    q = torch.empty(rows, n_q, two_hd // 2, dtype=torch.float32, device=qg.device)
    gate = torch.empty_like(q)
    p = _lib.AttnQkPrepareParams(n_q=n_q, n_kv=k.shape[1], head_dim=two_hd // 2, rotary_dim=rotary_dim,
                                 rows=rows, pos0=pos0, theta=theta, eps=eps)
    check(lib().rl_attn_qk_prepare(_p(qg), _p(k), _p(q_norm), _p(k_norm), _p(pos), _p(q), _p(gate),
                                   C.byref(p), _stream()))
    return q, gate


def rmsnorm(x, gamma=None, eps=1e-6, out=None):
    """ops::qwen3_rmsnorm over the last dimension: x / rms(x) * (1 + gamma)."""
    _need(x, torch.float32, "x")
    _need(gamma, torch.float32, "gamma")
    y = torch.empty_like(x) if out is None else out
    n = x.shape[-1]
    check(lib().rl_rmsnorm(_p(x), _p(gamma), _p(y), x.numel() // n, n, eps, _stream()))
    return y


def gated_rmsnorm(x, z, gamma=None, eps=1e-6):
    """ops::gated_rmsnorm per head: x, z [rows][n_heads][128], gamma [128] -> y."""
    for t, n in ((x, "x"), (z, "z"), (gamma, "gamma")):
        _need(t, torch.float32, n)
    rows, n_heads, hd = x.shape
    y = torch.empty_like(x)
    check(lib().rl_gated_rmsnorm(_p(x), _p(z), _p(gamma), _p(y), rows, n_heads, hd, eps, _stream()))
    return y


def delta_gates(a, b, A_log, dt_bias):
    """beta = sigmoid(b), g_log = -exp(A_log) * softplus(a + dt_bias); a, b [rows][n_v]."""
    for t, n in ((a, "a"), (b, "b"), (A_log, "A_log"), (dt_bias, "dt_bias")):
        _need(t, torch.float32, n)
    rows, n_v = a.shape
    beta, g = torch.empty_like(a), torch.empty_like(a)
    check(lib().rl_delta_gates(_p(a), _p(b), _p(A_log), _p(dt_bias), _p(beta), _p(g), rows, n_v, _stream()))
    return beta, g


def kv_compact_to_f16(pool, src_table_row, k_pool, v_pool, dst_table_row, n_tok, src_pos0=0, dst_pos0=0,
                      wht_len=128, signs=None):
    """Dequantise n_tok tokens of one sequence of the compact cache into paged F16 pools (the
    F16 compute window for prefill chunks / verify rows over a compact cache)."""
    _need(src_table_row, torch.int32, "src_table_row")
    _need(dst_table_row, torch.int32, "dst_table_row")
    _need(signs, torch.float32, "signs")
    check(lib().rl_kv_compact_to_f16(_p(pool), _p(src_table_row), src_pos0, pool.shape[0], _p(k_pool), _p(v_pool),
                                     _p(dst_table_row), dst_pos0, k_pool.shape[0], n_tok, pool.shape[1], wht_len,
                                     _p(signs), _stream()))


def gdn_decode(S, conv_ring, conv_phase, qkv, conv_w, beta, g_log, n_qk, slot_ids=None, head_map=None,
               eps_l2=1e-6, advance=True):
    """The fused Gated DeltaNet decode step of one layer (rl_gdn_decode): conv window + SiLU + l2
    norms + delta rule.  S [n_slots][n_v][128][128], conv_ring [n_slots][conv_dim][4] (ring windows),
    conv_phase int32 [n_slots], qkv [batch][conv_dim], conv_w [conv_dim][4]; returns o.  With
    advance the rings' phases move on afterwards (rl_gdn_phase_advance), as after a layer's step."""
    for t, n in ((S, "S"), (conv_ring, "conv_ring"), (qkv, "qkv"), (conv_w, "conv_w"), (beta, "beta"), (g_log, "g_log")):
        _need(t, torch.float32, n)
    _need(conv_phase, torch.int32, "conv_phase")
    _need(slot_ids, torch.int32, "slot_ids")
    n_slots, n_v, dk, dv = S.shape
    batch = qkv.shape[0]
    if head_map is None:
        head_map = _lib.RL_HEADS_PER_VALUE if n_qk == n_v else _lib.RL_HEADS_GROUPED
    o = torch.empty(batch, n_v, dv, dtype=torch.float32, device=S.device)
    p = _lib.GdnDecodeParams(n_v=n_v, n_qk=n_qk, dk=dk, dv=dv, conv_k=conv_w.shape[1], batch=batch, n_slots=n_slots,
                             head_map=head_map, eps_l2=eps_l2)
    check(lib().rl_gdn_decode(_p(S), _p(conv_ring), _p(conv_phase), _p(slot_ids), _p(qkv), _p(conv_w), _p(beta),
                              _p(g_log), _p(o), C.byref(p), _stream()))
    if advance:
        check(lib().rl_gdn_phase_advance(_p(conv_phase), _p(slot_ids), 1, n_slots, batch, 1, _stream()))
    return o


def conv_ring_export(conv_ring, conv_phase):
    """Ring windows [n_slots][conv_dim][4] -> the reference's shifted windows, oldest tap first."""
    out = torch.empty_like(conv_ring)
    check(lib().rl_conv_ring_export(_p(conv_ring), _p(conv_phase), _p(out), 1, conv_ring.shape[0], -1,
                                    conv_ring.shape[1], _stream()))
    return out
