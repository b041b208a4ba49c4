"""The hybrid stack over the compact cache (q8 K + TQ3 V pages with an F16 compute window) inside
rl_cache: prefill chunks that end inside the window and past it, decode steps over the window and
over the compact pages, two periods of layers, against the oracle (F16-rounded rows while the
window is read, the dequantised compact cache otherwise).  The window policy follows
src/kernels/cuda/cuda_engine.cu:18948-18953, 19048 (decode) and 18487-18497 (prefill)."""
import numpy as np
import pytest
import torch

from helpers import ATTN_MAX_ABS, ATTN_REL_L2, rel_l2, softplus

pytestmark = pytest.mark.gpu

N_Q, N_KV, HD = 24, 4, 256


def _chunk_inputs(cache, T, gen):
    t = {}
    for name, (shape, dtype) in cache.prefill_shapes(T).items():
        if name in ("attn_o", "delta_o"):
            t[name] = torch.zeros(shape, dtype=dtype)
        elif name == "delta_beta":
            t[name] = torch.sigmoid(torch.randn(shape, generator=gen))
        elif name == "delta_g":
            t[name] = -softplus(torch.randn(shape, generator=gen))
        else:
            t[name] = (torch.randn(shape, generator=gen) * (0.5 if name == "conv_w" else 1.0)).to(dtype)
    return t


@pytest.mark.parametrize("wht_len", [128, 256])
def test_window_then_compact_through_the_stack(oracle, wht_len):
    from rapidllm_b200 import _lib
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
    gen = torch.Generator().manual_seed(50 + wht_len)
    signs = (2.0 * torch.bernoulli(torch.full((256,), 0.5), generator=gen) - 1.0) if wht_len == 256 else None
    sn = None if signs is None else signs.numpy()
    window, max_pages, n_slots = 128, 5, 2
    cache = HybridCache(QWEN35_LAYER_TYPES * 2, n_pages=12, n_slots=n_slots, max_batch=2, max_pages_per_seq=max_pages,
                        kv_dtype=_lib.RL_KV_Q8K_TQ3V, wht_len=wht_len, window_tokens=window, tq_signs=signs)
    A = cache.n_attn
    assert A == 2 and cache.window_pages == 2
    assert cache.launches_per_step == A * 4 + 1 + cache.n_delta + 1
    tables = torch.tensor([[7, 2, 5, 0, 3], [1, 4, 6, 8, 9]], dtype=torch.int32).cuda()
    k_rows = [[torch.zeros(0, N_KV, HD) for _ in range(A)] for _ in range(n_slots)]      # what each sequence has stored, fp32
    v_rows = [[torch.zeros(0, N_KV, HD) for _ in range(A)] for _ in range(n_slots)]

    def reference_kv(seq, a, over_window):
        k, v = k_rows[seq][a], v_rows[seq][a]
        if over_window:
            return k.half().float().numpy(), v.half().float().numpy()
        return oracle.compact_dequant(*oracle.compact_store(k.numpy(), v.numpy(), wht_len, sn), wht_len, sn)

    def chunk(seq, T, over_window):
        pos0 = k_rows[seq][0].shape[0]
        t = _chunk_inputs(cache, T, gen)
        dev = {n: x.cuda() for n, x in t.items()}
        cache.prefill(dev, tables[seq], seq, pos0, T)
        _lib.check_device()
        for a in range(A):
            k_rows[seq][a] = torch.cat([k_rows[seq][a], t["attn_k"][a].float()])
            v_rows[seq][a] = torch.cat([v_rows[seq][a], t["attn_v"][a].float()])
            kd, vd = reference_kv(seq, a, over_window)
            rows = np.unique(np.clip(np.array([0, 1, T // 2, T - 2, T - 1]), 0, T - 1))
            ref = oracle.attn_prefill_rows(t["attn_q"][a].float().numpy()[rows], kd, vd, pos0 + rows)
            ref = ref / (1.0 + np.exp(-t["attn_gate"][a].numpy()[rows]))
            o = dev["attn_o"][a].cpu().numpy()[rows]
            assert np.isfinite(o).all()
            assert np.abs(o - ref).max() <= ATTN_MAX_ABS and rel_l2(o, ref) <= ATTN_REL_L2, \
                ("prefill", seq, pos0, T, a, np.abs(o - ref).max(), rel_l2(o, ref))

    def decode(seq, over_window):
        pos = k_rows[seq][0].shape[0]
        sh = cache.io_shapes(1)
        t = {n: torch.randn(sh[n], generator=gen) for n in ("attn_q", "attn_gate", "attn_k", "attn_v", "delta_qkv")}
        t["delta_beta"] = torch.sigmoid(torch.randn(sh["delta_beta"], generator=gen))
        t["delta_g"] = -softplus(torch.randn(sh["delta_g"], generator=gen))
        t["conv_w"] = torch.randn(sh["conv_w"], generator=gen) * 0.5
        t["attn_o"], t["delta_o"] = torch.zeros(sh["attn_o"]), torch.zeros(sh["delta_o"])
        t["pos"] = torch.tensor([pos], dtype=torch.int32)
        t["page_table"] = tables[seq:seq + 1].cpu()
        t["slot_ids"] = torch.tensor([seq], dtype=torch.int32)
        dev = {n: x.cuda() for n, x in t.items()}
        dev["kv_window_ok"] = over_window
        cache.decode(dev, 1)
        _lib.check_device()
        for a in range(A):
            k_rows[seq][a] = torch.cat([k_rows[seq][a], t["attn_k"][a]])
            v_rows[seq][a] = torch.cat([v_rows[seq][a], t["attn_v"][a]])
            kd, vd = reference_kv(seq, a, over_window)
            ref = oracle.gated_attn_decode(t["attn_q"][a, 0].numpy(), kd, vd, t["attn_gate"][a, 0].numpy())
            o = dev["attn_o"][a, 0].cpu().numpy()
            assert np.isfinite(o).all()
            assert np.abs(o - ref).max() <= ATTN_MAX_ABS and rel_l2(o, ref) <= ATTN_REL_L2, \
                ("decode", seq, pos, a, over_window, np.abs(o - ref).max(), rel_l2(o, ref))

    chunk(0, 100, True)            # ends inside the window: appended to it, attended over it
    chunk(1, 90, True)
    chunk(0, 60, False)            # [100, 160) ends past the window: over F16 pages rebuilt from the compact cache
    for _ in range(3):
        decode(1, True)            # positions 90..92 inside the window: the F16 window is read (and kept current)
    decode(1, False)               # the caller no longer vouches for the window: the compact pages hold every token
    for _ in range(2):
        decode(0, False)           # position 160, 161: compact
    chunk(1, 40, False)            # [94, 134) straddles the window edge: compact
    decode(1, False)
    # DeltaNet layers ran beside all this: their state must be finite and untouched slots still zero-free of NaN
    for d in range(cache.n_delta):
        assert torch.isfinite(cache.state(d)).all()
    cache.close()


def test_cache_config_errors():
    from rapidllm_b200 import _lib
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
    with pytest.raises(_lib.RlError):
        HybridCache(QWEN35_LAYER_TYPES, n_pages=4, n_slots=1, max_batch=1, max_pages_per_seq=2,
                    kv_dtype=_lib.RL_KV_Q8K_TQ3V, wht_len=64)
    with pytest.raises(_lib.RlError):
        HybridCache(QWEN35_LAYER_TYPES, n_pages=4, n_slots=1, max_batch=1, max_pages_per_seq=2,
                    kv_dtype=_lib.RL_KV_Q8K_TQ3V, wht_len=256)              # the 256-point layout needs its sign vector
    with pytest.raises(_lib.RlError):
        HybridCache(QWEN35_LAYER_TYPES, n_pages=4, n_slots=1, max_batch=1, max_pages_per_seq=2,
                    kv_dtype=_lib.RL_KV_Q8K_TQ3V, wht_len=128, window_tokens=4096)   # window beyond the context
