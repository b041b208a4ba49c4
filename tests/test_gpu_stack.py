"""The layer_types[] decode step (rl_stack_decode / rl_stack_decode_host) against the
oracle run layer by layer, on a small hybrid stack with ragged paged contexts."""
import numpy as np
import pytest
import torch

from helpers import ATTN_MAX_ABS, ATTN_REL_L2, rel_l2, softplus

pytestmark = pytest.mark.gpu


def _inputs(cache, B, gen, lens):
    sh = cache.io_shapes(B)
    t = {n: torch.randn(sh[n], generator=gen) for n in
         ("attn_q", "attn_gate", "attn_k", "attn_v", "delta_qkv")}
    t["conv_w"] = torch.randn(sh["conv_w"], generator=gen) * 0.5
    t["delta_beta"] = torch.sigmoid(torch.randn(sh["delta_beta"], generator=gen))
    t["delta_g"] = -softplus(torch.randn(sh["delta_g"], generator=gen))
    t["attn_o"] = torch.zeros(sh["attn_o"])
    t["delta_o"] = torch.zeros(sh["delta_o"])
    t["pos"] = torch.tensor(lens, dtype=torch.int32)
    return t


def test_stack_decode_matches_oracle_layer_by_layer(oracle):
    from rapidllm_b200 import _lib, ops
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
    gen = torch.Generator().manual_seed(4)
    types = QWEN35_LAYER_TYPES * 2
    lens = [100, 63, 257]                        # tokens already cached per sequence
    B, n_slots, max_pages = 3, 4, 6
    n_pages = 16
    cache = HybridCache(types, n_pages=n_pages, n_slots=n_slots, max_batch=4,
                        max_pages_per_seq=max_pages)
    assert cache.n_attn == 2 and cache.n_delta == 6 and cache.launches_per_step == 2 * 3 + 6 + 1
    # page table: disjoint shuffled pages
    perm = torch.randperm(n_pages, generator=gen).int()
    table = torch.zeros(B, max_pages, dtype=torch.int32)
    at = 0
    for b, n in enumerate(lens):
        p = (n + 1 + 63) // 64
        table[b, :p] = perm[at:at + p]
        at += p
    slots = torch.tensor([2, 0, 3], dtype=torch.int32)
    # fill the caches
    k_hist = [[torch.randn(n, 4, 256, generator=gen).half() for n in lens] for _ in range(2)]
    v_hist = [[torch.randn(n, 4, 256, generator=gen).half() for n in lens] for _ in range(2)]
    for a in range(2):
        for b in range(B):
            ops.kv_append(cache.k_pool(a), cache.v_pool(a), table[b].cuda(), k_hist[a][b].cuda(),
                          v_hist[a][b].cuda(), pos0=0)
    S0 = [torch.randn(n_slots, 48, 128, 128, generator=gen) * 0.02 for _ in range(6)]
    C0 = [torch.randn(n_slots, cache.conv_dim, 4, generator=gen) for _ in range(6)]
    for d in range(6):
        cache.state(d).copy_(S0[d])
        cache.set_conv_windows(d, C0[d])
    t = _inputs(cache, B, gen, lens)
    t["page_table"], t["slot_ids"] = table, slots
    dev = {n: x.cuda() for n, x in t.items()}
    cache.decode(dev, B)
    _lib.check_device()
    attn_o = dev["attn_o"].cpu().numpy()
    delta_o = dev["delta_o"].cpu().numpy()
    # oracle, layer by layer
    for a in range(2):
        for b in range(B):
            k = torch.cat([k_hist[a][b], t["attn_k"][a, b:b + 1].half()]).float().numpy()
            v = torch.cat([v_hist[a][b], t["attn_v"][a, b:b + 1].half()]).float().numpy()
            ref = oracle.gated_attn_decode(t["attn_q"][a, b].numpy(), k, v, t["attn_gate"][a, b].numpy())
            assert np.abs(attn_o[a, b] - ref).max() <= ATTN_MAX_ABS
            assert rel_l2(attn_o[a, b], ref) <= ATTN_REL_L2
    nk = 16 * 128
    for d in range(6):
        Sr = S0[d].numpy().copy()
        Cr = C0[d].numpy().copy()
        for b in range(B):
            sl = int(slots[b])
            mixed = oracle.conv1d_update(t["delta_qkv"][d, b].numpy(), t["conv_w"][d].numpy(), Cr[sl])
            q = oracle.repeat_heads(mixed[:nk].reshape(16, 128), 48)
            k = oracle.repeat_heads(mixed[nk:2 * nk].reshape(16, 128), 48)
            ref = oracle.delta_step(Sr[sl], q, k, mixed[2 * nk:].reshape(48, 128),
                                    t["delta_beta"][d, b].numpy(), t["delta_g"][d, b].numpy())
            assert np.abs(delta_o[d, b] - ref).max() < 1e-4
        assert rel_l2(cache.state(d).cpu().numpy(), Sr) < 1e-6
        assert np.array_equal(cache.conv_windows(d).cpu().numpy(), Cr)

    # the host-buffer entry point gives the same bits
    for d in range(6):
        cache.state(d).copy_(S0[d])
        cache.set_conv_windows(d, C0[d])
    host = {n: (x.pin_memory() if n != "conv_w" else x) for n, x in t.items()}
    host["attn_o"].zero_()
    host["delta_o"].zero_()
    cache.set_conv_w(host["conv_w"])
    cache.decode_host(host, B)
    _lib.check_device()
    assert np.array_equal(host["attn_o"].numpy(), attn_o)
    assert np.array_equal(host["delta_o"].numpy(), delta_o)
    cache.close()


def test_graph_replay_matches_plain_launches():
    """rl_stack_decode replays its step as a CUDA graph from the third call with the same io; the
    positions live in device memory and advance between replays.  Same bits as plain launches."""
    from rapidllm_b200 import _lib
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
    types = QWEN35_LAYER_TYPES
    B, n_slots, max_pages, n_pages = 2, 2, 3, 6
    lens = [61, 120]
    outs = []
    for graph in (True, False):
        gen = torch.Generator().manual_seed(11)
        cache = HybridCache(types, n_pages=n_pages, n_slots=n_slots, max_batch=B, max_pages_per_seq=max_pages)
        cache.set_graph(graph)
        for a in range(cache.n_attn):
            cache.k_pool(a).copy_(torch.randn(cache.k_pool(a).shape, generator=gen).half())
            cache.v_pool(a).copy_(torch.randn(cache.v_pool(a).shape, generator=gen).half())
        for d in range(cache.n_delta):
            cache.state(d).copy_(torch.randn(cache.state(d).shape, generator=gen) * 0.02)
            cache.set_conv_windows(d, torch.randn(cache.conv(d).shape, generator=gen))
        t = _inputs(cache, B, gen, lens)
        t["page_table"] = torch.tensor([[4, 1, 0], [2, 5, 3]], dtype=torch.int32)
        dev = {n: x.cuda() for n, x in t.items()}
        steps = []
        for step in range(5):                    # crosses a page boundary for sequence 0 (61 -> 65)
            if step:
                fresh = _inputs(cache, B, gen, lens)
                for n in ("attn_q", "attn_gate", "attn_k", "attn_v", "delta_qkv", "delta_beta", "delta_g"):
                    dev[n].copy_(fresh[n])       # same device tensors: the io of the captured graph stays valid
                dev["pos"] += 1
            cache.decode(dev, B)
            _lib.check_device()
            steps.append((dev["attn_o"].cpu().clone(), dev["delta_o"].cpu().clone()))
        final = [cache.state(d).cpu().clone() for d in range(cache.n_delta)]
        final += [cache.conv_windows(d).cpu().clone() for d in range(cache.n_delta)]
        final += [cache.k_pool(a).cpu().clone() for a in range(cache.n_attn)]
        outs.append((steps, final))
        cache.close()
    for (ao, do), (ao2, do2) in zip(outs[0][0], outs[1][0]):
        assert torch.equal(ao, ao2) and torch.equal(do, do2)
    for x, y in zip(outs[0][1], outs[1][1]):
        assert torch.equal(x, y)


def test_split_kv_partials_merge_to_the_unsplit_step():
    """Two caches that each hold a token range of every sequence (what two devices hold under
    split-KV) emit partials through rl_stack_decode; rl_lse_combine over the two equals the step of
    one cache that holds everything."""
    from rapidllm_b200 import _lib, ops
    from rapidllm_b200.cache import HybridCache
    gen = torch.Generator().manual_seed(21)
    types = [_lib.RL_LAYER_FULL_ATTENTION] * 2
    lens = [200, 75]                              # cached tokens per sequence; page 64
    head = [128, 64]                              # tokens on the first "device" (whole pages)
    B = 2
    k_hist = [[torch.randn(n, 4, 256, generator=gen).half() for n in lens] for _ in types]
    v_hist = [[torch.randn(n, 4, 256, generator=gen).half() for n in lens] for _ in types]

    def make(tok_from, tok_to):
        cache = HybridCache(types, n_pages=8, n_slots=1, max_batch=B, max_pages_per_seq=4)
        table = torch.tensor([[0, 1, 2, 3], [4, 5, 6, 7]], dtype=torch.int32).cuda()
        for a in range(len(types)):
            for b in range(B):
                ops.kv_append(cache.k_pool(a), cache.v_pool(a), table[b], k_hist[a][b][tok_from[b]:tok_to[b]].cuda(),
                              v_hist[a][b][tok_from[b]:tok_to[b]].cuda(), pos0=0)
        return cache, table

    sh = None
    full, table = make([0, 0], lens)
    sh = full.io_shapes(B)
    t = {n: torch.randn(sh[n], generator=gen).cuda() for n in ("attn_q", "attn_gate", "attn_k", "attn_v")}
    io = dict(t, attn_o=torch.zeros(sh["attn_o"]).cuda(), page_table=table,
              pos=torch.tensor(lens, dtype=torch.int32).cuda())
    full.decode(io, B)
    want = io["attn_o"].clone()
    full.close()

    parts_o, parts_ml = [], []
    for rank in range(2):
        frm = [0, 0] if rank == 0 else head
        to = head if rank == 0 else lens
        cache, table = make(frm, to)
        io = dict(t, attn_o=torch.zeros(sh["attn_o"]).cuda(), attn_ml=torch.zeros(sh["attn_ml"]).cuda(),
                  page_table=table, pos=torch.tensor([to[b] - frm[b] for b in range(B)], dtype=torch.int32).cuda(),
                  no_append=(rank == 0))
        cache.decode(io, B)
        _lib.check_device()
        parts_o.append(io["attn_o"].reshape(-1, 256))
        parts_ml.append(io["attn_ml"].reshape(-1, 2))
        cache.close()
    got = ops.lse_combine(torch.stack(parts_o), torch.stack(parts_ml), t["attn_gate"].reshape(-1, 256))
    got = got.reshape(want.shape)
    assert (got - want).abs().max().item() <= 1e-5
    assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) <= 1e-5


def test_host_entry_graph_replay_matches_plain_launches():
    """rl_stack_decode_host replays copies in + layers + copies out as one graph from the third
    call with the same pinned buffers; contents and positions change between calls."""
    from rapidllm_b200 import _lib
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
    types = QWEN35_LAYER_TYPES
    B, n_slots, max_pages, n_pages = 2, 2, 3, 6
    lens = [61, 120]
    outs = []
    for graph in (True, False):
        gen = torch.Generator().manual_seed(12)
        cache = HybridCache(types, n_pages=n_pages, n_slots=n_slots, max_batch=B, max_pages_per_seq=max_pages)
        cache.set_graph(graph)
        for a in range(cache.n_attn):
            cache.k_pool(a).copy_(torch.randn(cache.k_pool(a).shape, generator=gen).half())
            cache.v_pool(a).copy_(torch.randn(cache.v_pool(a).shape, generator=gen).half())
        for d in range(cache.n_delta):
            cache.state(d).copy_(torch.randn(cache.state(d).shape, generator=gen) * 0.02)
            cache.set_conv_windows(d, torch.randn(cache.conv(d).shape, generator=gen))
        t = _inputs(cache, B, gen, lens)
        t["page_table"] = torch.tensor([[4, 1, 0], [2, 5, 3]], dtype=torch.int32)
        cache.set_conv_w(t["conv_w"])
        host = {n: x.pin_memory() for n, x in t.items() if n != "conv_w"}
        steps = []
        for step in range(5):
            if step:
                fresh = _inputs(cache, B, gen, lens)
                for n in ("attn_q", "attn_gate", "attn_k", "attn_v", "delta_qkv", "delta_beta", "delta_g"):
                    host[n].copy_(fresh[n])
                host["pos"] += 1
            cache.decode_host(host, B)
            _lib.check_device()
            steps.append((host["attn_o"].clone(), host["delta_o"].clone()))
        final = [cache.state(d).cpu().clone() for d in range(cache.n_delta)]
        final += [cache.k_pool(a).cpu().clone() for a in range(cache.n_attn)]
        outs.append((steps, final))
        cache.close()
    for (ao, do), (ao2, do2) in zip(outs[0][0], outs[1][0]):
        assert torch.equal(ao, ao2) and torch.equal(do, do2)
    for x, y in zip(outs[0][1], outs[1][1]):
        assert torch.equal(x, y)


def test_config4_full_batch_one_period_of_the_stack(oracle):
    """One period of the layer pattern (3 DeltaNet + 1 gated attention) at the full batch and contexts of
    the headline workload: 32 sequences, contexts uniform in [8192, 32768], shuffled page table, seed 4.
    DeltaNet layers: every sequence against the oracle.  Attention: the three shortest sequences against
    the oracle; every sequence against a batch-of-one call (another division of the KV range among the
    CTAs); the appended K/V rows read back bit for bit through the page table."""
    from rapidllm_b200 import _lib, ops
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
    gen = torch.Generator().manual_seed(4)
    B = 32
    lens = torch.randint(8192, 32769, (B,), generator=gen).tolist()
    pages = [(n + 1 + 63) // 64 for n in lens]
    n_pages, max_pages = sum(pages) + 3, max(pages)
    cache = HybridCache(QWEN35_LAYER_TYPES, n_pages=n_pages, n_slots=B + 2, max_batch=B, max_pages_per_seq=max_pages)
    assert cache.n_attn == 1 and cache.n_delta == 3
    perm = torch.randperm(n_pages, generator=gen).int()
    table = torch.zeros(B, max_pages, dtype=torch.int32)
    at = 0
    for b, p in enumerate(pages):
        table[b, :p] = perm[at:at + p]
        at += p
    table_d = table.cuda()
    slots = torch.randperm(B + 2, generator=gen)[:B].int()
    dgen = torch.Generator(device="cuda").manual_seed(4)
    short = sorted(range(B), key=lambda b: lens[b])[:3]
    hist = {}
    for b in range(B):
        k = torch.randn(lens[b], 4, 256, generator=dgen, device="cuda").half()
        v = torch.randn(lens[b], 4, 256, generator=dgen, device="cuda").half()
        ops.kv_append(cache.k_pool(0), cache.v_pool(0), table_d[b], k, v, pos0=0)
        if b in short:
            hist[b] = (k.cpu(), v.cpu())
    S0 = [torch.randn(B + 2, 48, 128, 128, generator=gen) * 0.02 for _ in range(3)]
    C0 = [torch.randn(B + 2, cache.conv_dim, 4, generator=gen) for _ in range(3)]
    for d in range(3):
        cache.state(d).copy_(S0[d])
        cache.set_conv_windows(d, C0[d])
    t = _inputs(cache, B, gen, lens)
    t["page_table"], t["slot_ids"] = table, slots
    dev = {n: x.cuda() for n, x in t.items()}
    cache.decode(dev, B)
    _lib.check_device()
    attn_o = dev["attn_o"].cpu().numpy()
    delta_o = dev["delta_o"].cpu().numpy()
    # attention
    for b in short:
        k = torch.cat([hist[b][0], t["attn_k"][0, b:b + 1].half()]).float().numpy()
        v = torch.cat([hist[b][1], t["attn_v"][0, b:b + 1].half()]).float().numpy()
        ref = oracle.gated_attn_decode(t["attn_q"][0, b].numpy(), k, v, t["attn_gate"][0, b].numpy())
        assert np.abs(attn_o[0, b] - ref).max() <= ATTN_MAX_ABS and rel_l2(attn_o[0, b], ref) <= ATTN_REL_L2
    for b in range(B):
        one = ops.attn_decode(dev["attn_q"][0, b:b + 1], cache.k_pool(0), cache.v_pool(0), table_d[b:b + 1],
                              torch.tensor([lens[b] + 1], dtype=torch.int32, device="cuda"),
                              dev["attn_gate"][0, b:b + 1]).cpu().numpy()
        assert rel_l2(attn_o[0, b], one[0]) <= ATTN_REL_L2, (b, rel_l2(attn_o[0, b], one[0]))
        k_new = ops.kv_gather(cache.k_pool(0), table_d[b], lens[b] + 1)[lens[b]].cpu()
        v_new = ops.kv_gather(cache.v_pool(0), table_d[b], lens[b] + 1)[lens[b]].cpu()
        assert torch.equal(k_new, t["attn_k"][0, b].half()) and torch.equal(v_new, t["attn_v"][0, b].half())
    _lib.check_device()
    # DeltaNet
    nk = 16 * 128
    for d in range(3):
        Sr = S0[d].numpy().copy()
        Cr = C0[d].numpy().copy()
        for b in range(B):
            sl = int(slots[b])
            mixed = oracle.conv1d_update(t["delta_qkv"][d, b].numpy(), t["conv_w"][d].numpy(), Cr[sl])
            q = oracle.repeat_heads(mixed[:nk].reshape(16, 128), 48)
            k = oracle.repeat_heads(mixed[nk:2 * nk].reshape(16, 128), 48)
            ref = oracle.delta_step(Sr[sl], q, k, mixed[2 * nk:].reshape(48, 128),
                                    t["delta_beta"][d, b].numpy(), t["delta_g"][d, b].numpy())
            assert np.abs(delta_o[d, b] - ref).max() < 1e-4
        assert rel_l2(cache.state(d).cpu().numpy(), Sr) < 1e-6
        assert np.array_equal(cache.conv_windows(d).cpu().numpy(), Cr)
    cache.close()


def test_stack_decode_with_the_element_wise_steps_inside(oracle):
    """rl_stack_io.glue: the step takes the raw projections and runs q/gate split + head RMSNorm +
    partial RoPE before the attention, the gate maths before and the gated RMSNorm after the delta
    rule itself.  One period of layers, two steps (the second replays the captured graph), against
    the oracle's statements of those steps chained with its operators."""
    from rapidllm_b200 import _lib, ops
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, HybridCache
    gen = torch.Generator().manual_seed(21)
    lens = [70, 5]
    B, max_pages, n_pages = 2, 2, 5
    cache = HybridCache(QWEN35_LAYER_TYPES, n_pages=n_pages, n_slots=B, max_batch=B, max_pages_per_seq=max_pages)
    A, D = cache.n_attn, cache.n_delta
    table = torch.tensor([[3, 1], [4, 0]], dtype=torch.int32)
    k_hist = [torch.randn(n, 4, 256, generator=gen).half() for n in lens]
    v_hist = [torch.randn(n, 4, 256, generator=gen).half() for n in lens]
    for b in range(B):
        ops.kv_append(cache.k_pool(0), cache.v_pool(0), table[b].cuda(), k_hist[b].cuda(), v_hist[b].cuda(), pos0=0)
    S0 = [torch.randn(B, 48, 128, 128, generator=gen) * 0.02 for _ in range(D)]
    C0 = [torch.randn(B, cache.conv_dim, 4, generator=gen) for _ in range(D)]
    for d in range(D):
        cache.state(d).copy_(S0[d])
        cache.set_conv_windows(d, C0[d])
    w = {"q_norm": torch.randn(A, 256, generator=gen) * 0.1, "k_norm": torch.randn(A, 256, generator=gen) * 0.1,
         "A_log": torch.randn(D, 48, generator=gen) * 0.3, "dt_bias": torch.randn(D, 48, generator=gen) * 0.3,
         "gnorm": 1.0 + torch.randn(D, 128, generator=gen) * 0.1, "conv_w": torch.randn(D, cache.conv_dim, 4, generator=gen) * 0.5}
    Sr = [x.numpy().copy() for x in S0]
    Cr = [x.numpy().copy() for x in C0]
    dev_fixed = {n: x.cuda() for n, x in w.items()}
    sh = cache.io_shapes(B)
    raw = {"attn_qg": torch.empty(A, B, 24, 512).cuda(), "attn_k_raw": torch.empty(A, B, 4, 256).cuda(),
           "delta_a": torch.empty(D, B, 48).cuda(), "delta_b": torch.empty(D, B, 48).cuda(),
           "delta_z": torch.empty(D, B, 48, 128).cuda()}
    dev = {"attn_v": torch.empty(sh["attn_v"]).cuda(), "delta_qkv": torch.empty(sh["delta_qkv"]).cuda(),
           "attn_o": torch.zeros(sh["attn_o"]).cuda(), "delta_o": torch.zeros(sh["delta_o"]).cuda(),
           "conv_w": dev_fixed["conv_w"], "page_table": table.cuda(), "pos": torch.tensor(lens, dtype=torch.int32).cuda()}
    dev["glue"] = dict(raw, q_norm=dev_fixed["q_norm"], k_norm=dev_fixed["k_norm"], A_log=dev_fixed["A_log"],
                       dt_bias=dev_fixed["dt_bias"], gnorm=dev_fixed["gnorm"], rotary_dim=64, theta=1e7, rms_eps=1e-6)
    kh = [[k_hist[b].float().numpy()] for b in range(B)]
    vh = [[v_hist[b].float().numpy()] for b in range(B)]
    nk = 16 * 128
    for step in range(3):
        t = {"attn_qg": torch.randn(A, B, 24, 512, generator=gen), "attn_k_raw": torch.randn(A, B, 4, 256, generator=gen),
             "attn_v": torch.randn(A, B, 4, 256, generator=gen), "delta_qkv": torch.randn(D, B, cache.conv_dim, generator=gen),
             "delta_a": torch.randn(D, B, 48, generator=gen), "delta_b": torch.randn(D, B, 48, generator=gen),
             "delta_z": torch.randn(D, B, 48, 128, generator=gen)}
        for n, x in t.items():
            (raw[n] if n in raw else dev[n]).copy_(x)          # same device tensors: the captured graph stays valid
        if step:
            dev["pos"] += 1
        cache.decode(dev, B)
        _lib.check_device()
        attn_o, delta_o = dev["attn_o"].cpu().numpy(), dev["delta_o"].cpu().numpy()
        for b in range(B):
            pos = lens[b] + step
            q, gate, k = oracle.attn_qk_prepare(t["attn_qg"][0, b].numpy(), t["attn_k_raw"][0, b].numpy(),
                                                w["q_norm"][0].numpy(), w["k_norm"][0].numpy(), pos)
            kh[b].append(torch.from_numpy(k).half().float().numpy()[None])
            vh[b].append(t["attn_v"][0, b].half().float().numpy()[None])
            ref = oracle.gated_attn_decode(q, np.concatenate(kh[b]), np.concatenate(vh[b]), gate)
            assert np.abs(attn_o[0, b] - ref).max() <= ATTN_MAX_ABS and rel_l2(attn_o[0, b], ref) <= ATTN_REL_L2, (step, b)
        for d in range(D):
            for b in range(B):
                beta, g = oracle.delta_gates(t["delta_a"][d, b].numpy(), t["delta_b"][d, b].numpy(), w["A_log"][d].numpy(),
                                             w["dt_bias"][d].numpy())
                mixed = oracle.conv1d_update(t["delta_qkv"][d, b].numpy(), w["conv_w"][d].numpy(), Cr[d][b])
                q = oracle.repeat_heads(mixed[:nk].reshape(16, 128), 48)
                k = oracle.repeat_heads(mixed[nk:2 * nk].reshape(16, 128), 48)
                o = oracle.delta_step(Sr[d][b], q, k, mixed[2 * nk:].reshape(48, 128), beta, g)
                ref = oracle.gated_rmsnorm(o.reshape(-1), t["delta_z"][d, b].numpy().reshape(-1), w["gnorm"][d].numpy()).reshape(48, 128)
                assert np.abs(delta_o[d, b] - ref).max() <= 2e-4, (step, d, b, np.abs(delta_o[d, b] - ref).max())
            assert rel_l2(cache.state(d).cpu().numpy(), Sr[d]) < 1e-6
    cache.close()


@pytest.mark.parametrize("B", [1, 40])
def test_overlapped_step_equals_plain_per_layer_launches(B):
    """Inside rl_stack_decode the kernels of a step are launched for programmatic dependent launch and some of
    them work before they wait for the kernel in front (the DeltaNet step, the KV append, the decode kernel's
    page stream).  A short stack makes consecutive kernels and consecutive steps overlap as far as they ever
    can; thirty replayed steps must leave exactly the bits that plain launches, one operator after the other,
    leave (B 1: one CTA per column slice; B 40: persistent CTAs streaming whole heads)."""
    from rapidllm_b200 import _lib, ops
    from rapidllm_b200.cache import HybridCache
    lin, att = _lib.RL_LAYER_LINEAR_ATTENTION, _lib.RL_LAYER_FULL_ATTENTION
    types = [lin, lin, att, lin]
    gen = torch.Generator().manual_seed(70 + B)
    n_steps, max_pages = 30, 2
    cache = HybridCache(types, n_pages=B * max_pages, n_slots=B, max_batch=B, max_pages_per_seq=max_pages)
    lens = [int(x) for x in torch.randint(1, 60, (B,), generator=gen)]
    t = _inputs(cache, B, gen, lens)
    t["page_table"] = torch.randperm(B * max_pages, generator=gen).int().view(B, max_pages)
    dev = {n: x.cuda() for n, x in t.items()}
    # the plain side: its own copies of state, rings, phases and pages
    S = [cache.state(d).normal_(0, 0.02, generator=None).clone() for d in range(cache.n_delta)]
    for d in range(cache.n_delta):
        cache.set_conv_windows(d, torch.randn(cache.conv(d).shape, generator=gen))
    ring = [cache.conv(d).clone() for d in range(cache.n_delta)]
    phase = [torch.zeros(B, dtype=torch.int32, device="cuda") for _ in range(cache.n_delta)]
    kp, vp = cache.k_pool(0).normal_().clone(), cache.v_pool(0).normal_().clone()
    for d in range(cache.n_delta):
        cache.state(d).copy_(S[d])
    cache.k_pool(0).copy_(kp)
    cache.v_pool(0).copy_(vp)
    for step in range(n_steps):
        if step:
            fresh = _inputs(cache, B, gen, lens)
            for n in ("attn_q", "attn_gate", "attn_k", "attn_v", "delta_qkv", "delta_beta", "delta_g"):
                dev[n].copy_(fresh[n])
            dev["pos"] += 1
        cache.decode(dev, B)
        for d in range(cache.n_delta):
            o = ops.gdn_decode(S[d], ring[d], phase[d], dev["delta_qkv"][d], dev["conv_w"][d], dev["delta_beta"][d],
                               dev["delta_g"][d], n_qk=cache.n_k)
            assert torch.equal(o, dev["delta_o"][d]), (step, d)
        ops.kv_append(kp, vp, dev["page_table"], dev["attn_k"][0].unsqueeze(1), dev["attn_v"][0].unsqueeze(1), pos=dev["pos"])
        o = ops.attn_decode(dev["attn_q"][0], kp, vp, dev["page_table"], dev["pos"] + 1, dev["attn_gate"][0])
        assert torch.equal(o, dev["attn_o"][0]), step
    _lib.check_device()
    for d in range(cache.n_delta):
        assert torch.equal(cache.state(d), S[d])
        assert torch.equal(cache.conv(d), ring[d])
    assert torch.equal(cache.k_pool(0), kp) and torch.equal(cache.v_pool(0), vp)
    cache.close()
