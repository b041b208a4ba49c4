"""The C ABI library loads and exports every symbol include/rl_b200.h declares.
No compute is called here; this runs without a GPU."""
import ctypes as C
import os
import re

from conftest import ROOT


def _declared():
    src = open(os.path.join(ROOT, "include", "rl_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(rl_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_are_exported_and_bound():
    import __graft_entry__ as ge
    ge.build()
    from rapidllm_b200 import _lib
    names = _declared()
    assert len(names) >= 20
    L = C.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(L, n), f"{n} declared in rl_b200.h but not exported"
    assert set(names) == set(_lib.SYMBOLS), set(names) ^ set(_lib.SYMBOLS)
    assert _lib.lib().rl_b200_abi_version() == 2


def test_argument_errors_follow_reference_status_codes():
    """Bad arguments return RAPID_ERR_* style codes with a message; nothing throws or runs."""
    from rapidllm_b200 import _lib
    L = _lib.lib()
    p = _lib.AttnDecodeParams(n_q=24, n_kv=4, head_dim=128, kv_dtype=0, batch=1, page_tokens=64,
                              n_pages=4, max_pages_per_seq=4, max_seq_len=256)
    assert L.rl_attn_decode(None, None, None, None, None, None, None, None, 0, C.byref(p), None) == 4
    assert b"head_dim" in L.rl_last_error()
    assert L.rl_attn_decode_workspace_bytes(C.byref(p)) == 0
    p.head_dim = 256
    p.n_q = 40                                       # group of 10 > 8
    assert L.rl_attn_decode(None, None, None, None, None, None, None, None, 0, C.byref(p), None) == 4
    d = _lib.DeltaRecurrentParams(n_v=48, dk=64, dv=128, eps_l2=1e-6, batch=1, n_slots=1, n_qk=48)
    assert L.rl_delta_recurrent(None, None, None, None, None, None, None, None, C.byref(d), None) == 4
    d.dk = 128
    d.n_qk = 7
    d.head_map = 1
    assert L.rl_delta_recurrent(None, None, None, None, None, None, None, None, C.byref(d), None) == 6
    c = _lib.Conv1dParams(dim=10240, k=4, silu=0, batch=1, n_slots=1)
    assert L.rl_conv1d_update(None, None, None, None, None, C.byref(c), None) == 4
    assert L.rl_lse_combine(None, None, None, None, 0, 4, 256, 0, None, None) == 6
    assert L.rl_lse_combine(None, None, None, None, 2, 4, 256, 64, None, None) == 4
    assert L.rl_kv_compact_page_bytes() == 2 * 11456
    assert L.rl_device_error_string(1).startswith(b"page-table")
