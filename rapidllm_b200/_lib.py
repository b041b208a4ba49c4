"""ctypes binding of librl_b200.so (the C ABI declared in include/rl_b200.h).

There is no fallback: if the library is missing or a call fails, an exception
is raised.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "librl_b200.so")

RL_OK = 0
RL_KV_F16, RL_KV_Q8K_TQ3V = 0, 1
RL_KV_POLICY_AUTO, RL_KV_POLICY_F16, RL_KV_POLICY_COMPACT = 0, 1, 2
RL_LAYER_LINEAR_ATTENTION, RL_LAYER_FULL_ATTENTION = 0, 1
RL_HEADS_PER_VALUE, RL_HEADS_GROUPED, RL_HEADS_TILED = 0, 1, 2
STATUS_NAMES = ["RL_OK", "RL_ERR_IO", "RL_ERR_FORMAT", "RL_ERR_NOMEM", "RL_ERR_UNSUPPORTED",
                "RL_ERR_DEVICE", "RL_ERR_RANGE", "RL_ERR_INTERNAL"]


class RlError(RuntimeError):
    def __init__(self, status, message):
        self.status = status
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"{name}: {message}")


class AttnDecodeParams(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "n_q", "n_kv", "head_dim", "kv_dtype", "batch", "page_tokens", "n_pages",
        "max_pages_per_seq", "max_seq_len", "len_add", "chunk_pages", "wht_len")] + [
        ("tq_signs", C.c_void_p)]


class AttnPrefillParams(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "n_q", "n_kv", "head_dim", "seq", "br", "bc", "pos0", "page_tokens", "n_pages", "n_table")]


class KvAppendParams(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "n_kv", "head_dim", "batch", "n_tok", "page_tokens", "n_pages", "max_pages_per_seq",
        "pos0", "rows_fp16", "wht_len", "pos_limit")]


class DeltaRecurrentParams(C.Structure):
    _fields_ = [("n_v", C.c_int), ("dk", C.c_int), ("dv", C.c_int), ("eps_l2", C.c_float),
                ("batch", C.c_int), ("n_slots", C.c_int), ("n_qk", C.c_int), ("head_map", C.c_int),
                ("q_stride", C.c_longlong), ("k_stride", C.c_longlong), ("v_stride", C.c_longlong)]


class DeltaChunkParams(C.Structure):
    _fields_ = [("n_v", C.c_int), ("dk", C.c_int), ("dv", C.c_int), ("seq", C.c_int), ("chunk", C.c_int),
                ("eps_l2", C.c_float), ("n_qk", C.c_int), ("head_map", C.c_int),
                ("qk_tok_stride", C.c_longlong), ("v_tok_stride", C.c_longlong)]


class GdnDecodeParams(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_v", "n_qk", "dk", "dv", "conv_k", "batch", "n_slots", "head_map")] + [
        ("eps_l2", C.c_float)]


class Conv1dParams(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("dim", "k", "silu", "batch", "n_slots")]


class AttnQkPrepareParams(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_q", "n_kv", "head_dim", "rotary_dim", "rows", "pos0")] + [
        ("theta", C.c_float), ("eps", C.c_float)]


class PlanInput(C.Structure):
    _fields_ = [("weight_bytes", C.c_ulonglong), ("available_bytes", C.c_ulonglong), ("pad_bytes", C.c_ulonglong)] + [
        (n, C.c_int) for n in ("ctx", "max_batch", "n_attn_layers", "n_kv", "head_dim", "n_delta_layers", "n_v",
                               "dk", "dv", "conv_dim", "conv_k", "page_tokens", "kv_policy", "allow_shrink",
                               "prefill_chunk")]


class PlanResult(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("ok", "kv_dtype", "ctx", "max_pages_per_seq", "n_pages")] + [
        ("kv_bytes", C.c_ulonglong), ("state_bytes", C.c_ulonglong), ("need_bytes", C.c_ulonglong),
        ("window_tokens", C.c_int), ("window_pages_per_seq", C.c_int), ("window_bytes", C.c_ulonglong),
        ("message", C.c_char * 160)]


class CacheConfig(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("layer_types", C.POINTER(C.c_int)),
                ("n_q", C.c_int), ("n_kv", C.c_int), ("head_dim", C.c_int), ("kv_dtype", C.c_int),
                ("page_tokens", C.c_int), ("n_pages", C.c_int),
                ("n_v", C.c_int), ("n_k", C.c_int), ("dk", C.c_int), ("dv", C.c_int),
                ("conv_k", C.c_int), ("head_map", C.c_int), ("n_slots", C.c_int),
                ("max_batch", C.c_int), ("max_pages_per_seq", C.c_int), ("max_seq_len", C.c_int),
                ("wht_len", C.c_int), ("window_tokens", C.c_int), ("tq_signs", C.c_void_p)]


class StackIO(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "attn_q", "attn_gate", "attn_k", "attn_v", "attn_o", "delta_qkv", "delta_beta", "delta_g",
        "delta_o", "conv_w", "page_table", "pos", "slot_ids")] + [
        ("batch", C.c_int), ("attn_ml", C.c_void_p), ("no_append", C.c_int), ("kv_window_ok", C.c_int),
        ("glue", C.c_void_p)]


class StackGlue(C.Structure):
    _fields_ = [("attn_qg", C.c_void_p), ("attn_k_raw", C.c_void_p), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
                ("rotary_dim", C.c_int), ("theta", C.c_float), ("rms_eps", C.c_float),
                ("delta_a", C.c_void_p), ("delta_b", C.c_void_p), ("A_log", C.c_void_p), ("dt_bias", C.c_void_p),
                ("delta_z", C.c_void_p), ("gnorm", C.c_void_p)]


class StackGather(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("comm", "attn_o_all", "delta_o_all", "attn_ml_all", "attn_o_final")] + [
        ("layers_per_exchange", C.c_int), ("reserve_sms", C.c_int)]


COMM_ID_BYTES = 128


class StackPrefillIO(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "attn_q", "attn_k", "attn_v", "attn_gate", "attn_o", "delta_qkv", "delta_beta", "delta_g", "delta_o",
        "conv_w", "page_table_row")] + [("slot", C.c_int), ("pos0", C.c_int), ("T", C.c_int)]


# every symbol include/rl_b200.h declares: name -> (restype, argtypes)
_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t
SYMBOLS = {
    "rl_b200_available": (_i, []),
    "rl_b200_abi_version": (_i, []),
    "rl_last_error": (C.c_char_p, []),
    "rl_device_error": (_i, [_vp]),
    "rl_device_error_string": (C.c_char_p, [_i]),
    "rl_attn_decode_workspace_bytes": (_sz, [C.POINTER(AttnDecodeParams)]),
    "rl_attn_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz,
                            C.POINTER(AttnDecodeParams), _vp]),
    "rl_attn_decode_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, C.POINTER(AttnDecodeParams), _vp]),
    "rl_attn_decode_partial": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz,
                                    C.POINTER(AttnDecodeParams), _vp]),
    "rl_attn_prefill": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.POINTER(AttnPrefillParams), _vp]),
    "rl_attn_prefill_workspace_bytes": (_sz, [C.POINTER(AttnPrefillParams)]),
    "rl_attn_prefill_ws": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, C.POINTER(AttnPrefillParams), _vp]),
    "rl_lse_combine": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "rl_kv_compact_page_bytes": (_sz, []),
    "rl_kv_compact_append": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, C.POINTER(KvAppendParams), _vp]),
    "rl_kv_compact_gather": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "rl_kv_compact_to_f16": (_i, [_vp, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "rl_kv_append": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, C.POINTER(KvAppendParams), _vp]),
    "rl_kv_gather": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "rl_delta_recurrent": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                C.POINTER(DeltaRecurrentParams), _vp]),
    "rl_delta_recurrent_multi": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                      C.POINTER(DeltaRecurrentParams), _i, C.c_longlong, C.c_longlong, _vp]),
    "rl_delta_chunk_workspace_bytes": (_sz, [C.POINTER(DeltaChunkParams)]),
    "rl_delta_chunk_mma_flops": (C.c_double, []),
    "rl_delta_chunk_prefill": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, C.POINTER(DeltaChunkParams), _vp]),
    "rl_gdn_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.POINTER(GdnDecodeParams), _vp]),
    "rl_gdn_phase_advance": (_i, [_vp, _vp, _i, _i, _i, _i, _vp]),
    "rl_conv_ring_export": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "rl_conv_ring_import": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "rl_cache_conv_phase": (_vp, [_vp, _i]),
    "rl_cache_delta_prefill_workspace_bytes": (_sz, [_vp, _i]),
    "rl_cache_delta_prefill": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "rl_cache_conv_export": (_i, [_vp, _i, _vp, _vp]),
    "rl_cache_conv_import": (_i, [_vp, _i, _vp, _vp]),
    "rl_conv1d_update": (_i, [_vp, _vp, _vp, _vp, _vp, C.POINTER(Conv1dParams), _vp]),
    "rl_conv1d_causal": (_i, [_vp, _vp, _vp, _vp, _i, C.POINTER(Conv1dParams), _i, _vp]),
    "rl_plan_cache": (_i, [C.POINTER(PlanInput), C.POINTER(PlanResult)]),
    "rl_attn_qk_prepare": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, C.POINTER(AttnQkPrepareParams), _vp]),
    "rl_gated_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, C.c_float, _vp]),
    "rl_rmsnorm": (_i, [_vp, _vp, _vp, _i, _i, C.c_float, _vp]),
    "rl_cast_f32_to_bf16": (_i, [_vp, _vp, _sz, _vp]),
    "rl_delta_gates": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "rl_cache_create": (_i, [C.POINTER(CacheConfig), C.POINTER(_vp)]),
    "rl_cache_destroy": (None, [_vp]),
    "rl_cache_bytes": (_sz, [_vp]),
    "rl_cache_k_pool": (_vp, [_vp, _i]),
    "rl_cache_v_pool": (_vp, [_vp, _i]),
    "rl_cache_window_k_pool": (_vp, [_vp, _i]),
    "rl_cache_window_v_pool": (_vp, [_vp, _i]),
    "rl_cache_state": (_vp, [_vp, _i]),
    "rl_cache_conv": (_vp, [_vp, _i]),
    "rl_cache_zero": (_i, [_vp, _vp]),
    "rl_stack_decode": (_i, [_vp, C.POINTER(StackIO), _vp]),
    "rl_stack_prefill_workspace_bytes": (_sz, [_vp, _i, _i]),
    "rl_stack_prefill": (_i, [_vp, C.POINTER(StackPrefillIO), _vp, _sz, _vp]),
    "rl_stack_decode_host": (_i, [_vp, C.POINTER(StackIO)]),
    "rl_stack_set_conv_w": (_i, [_vp, _vp]),
    "rl_stack_launches_per_step": (_i, [_vp]),
    "rl_stack_set_timing": (_i, [_vp, _i]),
    "rl_stack_set_graph": (_i, [_vp, _i]),
    "rl_stack_timing": (_i, [_vp, C.POINTER(C.c_float)]),
    "rl_comm_unique_id": (_i, [_vp]),
    "rl_comm_create": (_i, [_vp, _i, _i, C.POINTER(_vp)]),
    "rl_comm_destroy": (None, [_vp]),
    "rl_stack_set_gather": (_i, [_vp, C.POINTER(StackGather)]),
}

_lib = None


def lib():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RlError(1, f"{LIB_PATH} not found: run `python -m rapidllm_b200.build`")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != RL_OK:
        raise RlError(status, lib().rl_last_error().decode(errors="replace"))


def device_error(stream=None) -> int:
    return lib().rl_device_error(stream)


def check_device(stream=None) -> None:
    code = device_error(stream)
    if code != 0:
        raise RlError(5, "device error %d: %s" % (
            code, lib().rl_device_error_string(code).decode() if code > 0 else
            lib().rl_last_error().decode()))
