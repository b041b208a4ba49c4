"""rl_stack_prefill: a prompt through a small hybrid stack in chunks (the reference's chunked-prefill
driver for the mixers), then one rl_stack_decode step continuing from the caches it left, against
the oracle run token by token: conv + delta rule per token, causal attention rows over the fp16 cache."""
import numpy as np
import pytest
import torch

from helpers import ATTN_MAX_ABS, ATTN_REL_L2, rel_l2, softplus

pytestmark = pytest.mark.gpu

CHUNKED_REL_L2 = 1e-3      # outputs of the chunked form (fp16 operands on the output products)
STATE_REL_L2 = 1e-5        # its FP32 state


def _chunk_inputs(cache, T, gen):
    t = {}
    for name, (shape, dtype) in cache.prefill_shapes(T).items():
        if name in ("attn_o", "delta_o"):
            t[name] = torch.zeros(shape, dtype=dtype)
        elif name == "conv_w":
            continue
        elif name == "delta_beta":
            t[name] = torch.sigmoid(torch.randn(shape, generator=gen))
        elif name == "delta_g":
            t[name] = -softplus(torch.randn(shape, generator=gen))
        else:
            t[name] = torch.randn(shape, generator=gen).to(dtype)
    return t


@pytest.mark.parametrize("head_map_name", ["RL_HEADS_GROUPED", "RL_HEADS_TILED"])
def test_prompt_in_chunks_then_decode(oracle, head_map_name):
    from rapidllm_b200 import _lib
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
    head_map = getattr(_lib, head_map_name)
    tiled = head_map == _lib.RL_HEADS_TILED
    gen = torch.Generator().manual_seed(12)
    types = QWEN35_LAYER_TYPES                      # D, D, D, A
    n_slots, max_pages, n_pages = 3, 5, 9
    cache = HybridCache(types, n_pages=n_pages, n_slots=n_slots, max_batch=2, max_pages_per_seq=max_pages,
                        head_map=head_map)
    A, D, cd = cache.n_attn, cache.n_delta, cache.conv_dim
    slot = 1
    # another sequence's state sits in the slot: a prompt starting at position 0 must not see it
    for d in range(D):
        cache.state(d).normal_(generator=None)
        cache.conv(d).normal_(generator=None)
    row = torch.tensor([7, 2, 5, 0, 3], dtype=torch.int32).cuda()
    conv_w = torch.randn(D, cd, 4, generator=gen) * 0.5
    chunks = [130, 70, 1]                           # page-unaligned boundaries, a one-token chunk
    ins, outs, pos0 = [], [], 0
    for T in chunks:
        t = _chunk_inputs(cache, T, gen)
        dev = {n: x.cuda() for n, x in t.items()}
        dev["conv_w"] = conv_w.cuda()
        cache.prefill(dev, row, slot, pos0, T)
        _lib.check_device()
        ins.append(t)
        outs.append({n: dev[n].cpu().numpy() for n in ("attn_o", "delta_o")})
        pos0 += T
    n_prompt = pos0
    cat = {n: torch.cat([t[n] for t in ins], dim=1) for n in ins[0]}
    got = {n: np.concatenate([o[n] for o in outs], axis=1) for n in outs[0]}
    # DeltaNet layers: conv and delta rule token by token from a zero state
    S_ref, C_ref = [], []
    n_k = cache.n_k
    for d in range(D):
        S = np.zeros((48, 128, 128), np.float32)
        cs = np.zeros((cd, 4), np.float32)
        w = conv_w[d].numpy()
        o = np.empty((n_prompt, 48, 128), np.float32)
        for tok in range(n_prompt):
            mixed = oracle.conv1d_update(cat["delta_qkv"][d, tok].numpy(), w, cs)
            q = oracle.repeat_heads(mixed[:n_k * 128].reshape(n_k, 128), 48, tiled)
            k = oracle.repeat_heads(mixed[n_k * 128:2 * n_k * 128].reshape(n_k, 128), 48, tiled)
            v = mixed[2 * n_k * 128:].reshape(48, 128)
            o[tok] = oracle.delta_step(S, q, k, v, cat["delta_beta"][d, tok].numpy(), cat["delta_g"][d, tok].numpy())
        # the chunked form passes operands through fp16 hi + lo pairs: the tolerance of its own test
        assert rel_l2(got["delta_o"][d], o) <= CHUNKED_REL_L2, (d, rel_l2(got["delta_o"][d], o))
        assert rel_l2(cache.state(d)[slot].cpu().numpy(), S) <= STATE_REL_L2
        assert np.abs(cache.conv_windows(d)[slot].cpu().numpy() - cs).max() == 0.0
        S_ref.append(S)
        C_ref.append(cs)
    # attention layers: row t attends to the fp16-rounded rows [0, t] of the whole prompt
    for a in range(A):
        kf = cat["attn_k"][a].float().half().float().numpy()
        vf = cat["attn_v"][a].float().half().float().numpy()
        rows = np.array([0, 1, 63, 64, 129, 130, 131, 199, 200])
        ref = oracle.attn_prefill_rows(cat["attn_q"][a].float().numpy()[rows], kf, vf, rows)
        ref = ref / (1.0 + np.exp(-cat["attn_gate"][a].numpy()[rows]))
        o = got["attn_o"][a][rows]
        assert np.abs(o - ref).max() <= ATTN_MAX_ABS and rel_l2(o, ref) <= ATTN_REL_L2, \
            (np.abs(o - ref).max(), rel_l2(o, ref))
    # untouched slots kept their contents; one decode step continues from what the prefill left
    assert cache.state(0)[0].abs().sum() > 0
    sh = cache.io_shapes(1)
    t = {n: torch.randn(sh[n], generator=gen) for n in ("attn_q", "attn_gate", "attn_k", "attn_v", "delta_qkv")}
    t["delta_beta"] = torch.sigmoid(torch.randn(sh["delta_beta"], generator=gen))
    t["delta_g"] = -softplus(torch.randn(sh["delta_g"], generator=gen))
    t["attn_o"], t["delta_o"] = torch.zeros(sh["attn_o"]), torch.zeros(sh["delta_o"])
    t["conv_w"] = conv_w
    t["pos"] = torch.tensor([n_prompt], dtype=torch.int32)
    t["page_table"] = row.cpu().view(1, -1)
    t["slot_ids"] = torch.tensor([slot], dtype=torch.int32)
    dev = {n: x.cuda() for n, x in t.items()}
    cache.decode(dev, 1)
    _lib.check_device()
    for d in range(D):
        mixed = oracle.conv1d_update(t["delta_qkv"][d, 0].numpy(), conv_w[d].numpy(), C_ref[d])
        q = oracle.repeat_heads(mixed[:n_k * 128].reshape(n_k, 128), 48, tiled)
        k = oracle.repeat_heads(mixed[n_k * 128:2 * n_k * 128].reshape(n_k, 128), 48, tiled)
        o = oracle.delta_step(S_ref[d], q, k, mixed[2 * n_k * 128:].reshape(48, 128), t["delta_beta"][d, 0].numpy(),
                              t["delta_g"][d, 0].numpy())
        assert rel_l2(dev["delta_o"][d, 0].cpu().numpy(), o) <= CHUNKED_REL_L2
    for a in range(A):
        kf = torch.cat([cat["attn_k"][a].float(), t["attn_k"][a]]).half().float().numpy()
        vf = torch.cat([cat["attn_v"][a].float(), t["attn_v"][a]]).half().float().numpy()
        ref = oracle.gated_attn_decode(t["attn_q"][a, 0].numpy(), kf, vf, t["attn_gate"][a, 0].numpy())
        o = dev["attn_o"][a, 0].cpu().numpy()
        assert np.abs(o - ref).max() <= ATTN_MAX_ABS and rel_l2(o, ref) <= ATTN_REL_L2


def test_argument_errors():
    from rapidllm_b200 import _lib
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
    cache = HybridCache(QWEN35_LAYER_TYPES, n_pages=4, n_slots=1, max_batch=1, max_pages_per_seq=2)
    row = torch.zeros(2, dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.RlError):
        cache.prefill({}, row, 0, 100, 64)                      # past the page table
    with pytest.raises(_lib.RlError):
        cache.prefill({}, row, 3, 0, 16)                        # slot outside the cache
    with pytest.raises(_lib.RlError):
        cache.prefill({}, row, 0, 0, 16)                        # tensors missing
    cache.prefill({}, row, 0, 0, 0)                             # nothing to do


def test_one_deltanet_layer_at_a_time_equals_the_stack_call():
    """rl_cache_delta_prefill (a host that runs its projections between the layers calls the DeltaNet
    prefill per layer) leaves the same state, windows and outputs as rl_stack_prefill over the same
    inputs, bit for bit, across two chunks (the second starts from the carried window)."""
    import ctypes as C
    from rapidllm_b200 import _lib
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
    gen = torch.Generator().manual_seed(13)
    mk = lambda: HybridCache(QWEN35_LAYER_TYPES, n_pages=6, n_slots=2, max_batch=2, max_pages_per_seq=3)
    a, b = mk(), mk()
    D, cd = a.n_delta, a.conv_dim
    row = torch.tensor([4, 1, 2], dtype=torch.int32).cuda()
    conv_w = (torch.randn(D, cd, 4, generator=gen) * 0.5).cuda()
    slot, pos0 = 1, 0
    L = _lib.lib()
    vp = C.c_void_p
    for T in (100, 37):
        t = _chunk_inputs(a, T, gen)
        dev = {n: x.cuda() for n, x in t.items()}
        dev["conv_w"] = conv_w
        a.prefill(dev, row, slot, pos0, T)
        o = torch.zeros(D, T, 48, 128, device="cuda")
        need = L.rl_cache_delta_prefill_workspace_bytes(b._h, T)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        st = vp(torch.cuda.current_stream().cuda_stream)
        for d in range(D):
            _lib.check(L.rl_cache_delta_prefill(b._h, d, slot, pos0, T, vp(dev["delta_qkv"][d].data_ptr()),
                                                vp(conv_w[d].data_ptr()), vp(dev["delta_beta"][d].data_ptr()),
                                                vp(dev["delta_g"][d].data_ptr()), vp(o[d].data_ptr()), vp(ws.data_ptr()),
                                                ws.numel(), st))
        _lib.check_device()
        assert torch.equal(o, dev["delta_o"])
        for d in range(D):
            assert torch.equal(a.state(d), b.state(d))
            assert torch.equal(a.conv_windows(d), b.conv_windows(d))
        pos0 += T
    a.close()
    b.close()
