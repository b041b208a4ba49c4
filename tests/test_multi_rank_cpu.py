"""World-size-2 (gloo, CPU) checks of the multi-GPU division: the shard plan, the all_gather
of head slices, and the split-KV exchange of (o, max, sum) partials merged like rl_lse_combine
does -- with the oracle standing in for the kernels."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT
from rapidllm_b200.shard import pages_of_part, plan_heads, plan_sequences, token_range_of_part


def test_shard_plans():
    for world in (1, 2, 4, 8):
        shards = [plan_heads(r, world) for r in range(world)]
        assert sorted(h for s in shards for h in s.v_heads) == list(range(48))
        assert all(set(range(s.k_heads.start * 3, s.k_heads.stop * 3)) == set(s.v_heads) for s in shards)
        cover = {}
        for s in shards:
            for h in s.kv_heads:
                cover.setdefault(h, []).append(s.kv_part)
            assert list(s.q_heads) == [6 * h + i for h in s.kv_heads for i in range(6)]
            assert s.rank in s.peers and len(s.peers) == s.kv_split
        assert sorted(cover) == [0, 1, 2, 3]
        assert all(sorted(p) == list(range(max(1, world // 4))) for p in cover.values())
    s = plan_heads(5, 8)
    assert list(s.kv_heads) == [1] and s.kv_split == 2 and s.kv_part == 1 and s.peers == [1, 5]
    assert pages_of_part(7, 2, 0) == [0, 2, 4, 6] and pages_of_part(7, 2, 1) == [1, 3, 5]
    assert [len(plan_sequences(r, 4, 30)) for r in range(4)] == [8, 8, 7, 7]
    with pytest.raises(ValueError):
        plan_heads(0, 3)
    for n_tok in (1, 63, 64, 65, 1000, 32768):
        for world in (1, 2, 4, 8):
            parts = [token_range_of_part(n_tok, world, r) for r in range(world)]
            assert parts[0][0] == 0 and sum(n for _, n in parts) == n_tok
            assert all(parts[r][0] + parts[r][1] == parts[r + 1][0] or parts[r + 1][1] == 0 for r in range(world - 1))
            assert all(f % 64 == 0 for f, _ in parts)


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import Oracle
    orc = Oracle()
    rng = np.random.default_rng(0)                      # same inputs on every rank
    n_q, n_kv, hd, seq = 12, 2, 64, 64 * 5 + 20
    q = rng.standard_normal((n_q, hd), dtype=np.float32)
    k = rng.standard_normal((seq, n_kv, hd), dtype=np.float32)
    v = rng.standard_normal((seq, n_kv, hd), dtype=np.float32)
    full = orc.attn_decode(q, k, v)
    # (1) head sharding: every rank computes its KV head's query heads, one all_gather
    sh = plan_heads(rank, world, n_q=n_q, n_kv=n_kv, n_v=4, n_k=2)
    mine = orc.attn_decode(q[sh.q_heads.start:sh.q_heads.stop], k[:, sh.kv_heads.start:sh.kv_heads.stop],
                           v[:, sh.kv_heads.start:sh.kv_heads.stop])
    parts = [torch.empty(mine.shape) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(mine))
    ok_heads = np.array_equal(torch.cat(parts).numpy(), full)
    # (2) split-KV: rank holds alternating pages of every head; exchange (o, max, sum)
    n_pages = (seq + 63) // 64
    tok = np.concatenate([np.arange(p * 64, min(seq, p * 64 + 64)) for p in pages_of_part(n_pages, world, rank)])
    po = np.empty((n_q, hd), np.float32)
    pml = np.empty((n_q, 2), np.float32)
    for h in range(n_q):
        m, l, acc = orc.attn_partial(q[h], k[tok], v[tok], 0, len(tok), h // (n_q // n_kv))
        po[h], pml[h] = acc, (m, l)
    go = [torch.empty(n_q, hd) for _ in range(world)]
    gml = [torch.empty(n_q, 2) for _ in range(world)]
    dist.all_gather(go, torch.from_numpy(po))
    dist.all_gather(gml, torch.from_numpy(pml))
    merged = np.stack([orc.lse_combine([x[h, 0].item() for x in gml], [x[h, 1].item() for x in gml],
                                       np.stack([x[h].numpy() for x in go])) for h in range(n_q)])
    err = float(np.abs(merged - full).max())
    # (2b) the same exchange with one contiguous page range per rank (token_range_of_part)
    first, n_loc = token_range_of_part(seq, world, rank)
    for h in range(n_q):
        m, l, acc = orc.attn_partial(q[h], k[first:first + n_loc], v[first:first + n_loc], 0, n_loc, h // (n_q // n_kv))
        po[h], pml[h] = acc, (m, l)
    dist.all_gather(go, torch.from_numpy(po))
    dist.all_gather(gml, torch.from_numpy(pml))
    merged = np.stack([orc.lse_combine([x[h, 0].item() for x in gml], [x[h, 1].item() for x in gml],
                                       np.stack([x[h].numpy() for x in go])) for h in range(n_q)])
    err = max(err, float(np.abs(merged - full).max()))
    # (3) a rank that fails is seen by the others on the host, not by a hung collective
    flag = torch.tensor([1 if rank == 1 else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    ret[rank] = (ok_heads, err, int(flag.item()))
    dist.destroy_process_group()


def test_two_ranks_gloo():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    for r in range(world):
        ok_heads, err, flag = ret[r]
        assert ok_heads
        assert err < 1e-5
        assert flag == 1


def _plan_worker(rank, world, port, mode, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from rapidllm_b200.shard import StepPlan
    B, n_q, n_kv, n_v, n_k = 4, 24, 4, 12, 4
    rng = np.random.default_rng(1)                      # the whole problem, the same on every rank
    conv_dim = 2 * n_k * 128 + n_v * 128
    full = {"attn_q": torch.from_numpy(rng.standard_normal((2, B, n_q, 8), dtype=np.float32)),
            "attn_k": torch.from_numpy(rng.standard_normal((2, B, n_kv, 8), dtype=np.float32)),
            "delta_qkv": torch.from_numpy(rng.standard_normal((3, B, conv_dim), dtype=np.float32)),
            "delta_beta": torch.from_numpy(rng.standard_normal((3, B, n_v), dtype=np.float32)),
            "conv_w": torch.from_numpy(rng.standard_normal((3, conv_dim, 4), dtype=np.float32))}
    plan = StepPlan(mode, rank, world, B, n_q, n_kv, n_v, n_k)
    mine = {n: x.contiguous() for n, x in plan.slice_io(full).items()}
    # a stand-in for the kernels: attention output = 2 q, DeltaNet output = the v channels times beta
    attn_o = 2.0 * mine["attn_q"][0]
    nv_l = len(plan.v_heads)
    delta_o = mine["delta_qkv"][0][:, -nv_l * 128:].reshape(len(plan.seqs), nv_l, 128) * mine["delta_beta"][0][..., None]
    ga = [torch.empty_like(attn_o) for _ in range(world)]
    gd = [torch.empty_like(delta_o) for _ in range(world)]
    dist.all_gather(ga, attn_o.contiguous())            # block r = rank r's local output, as rl_stack_gather lays it out
    dist.all_gather(gd, delta_o.contiguous())
    ok = True
    if mode == "heads":
        whole = plan.place_attn(torch.zeros(B, n_q, 8), torch.stack(ga))
        ok = ok and torch.equal(whole, 2.0 * full["attn_q"][0])
    whole_d = plan.place_delta(torch.zeros(B, n_v, 128), torch.stack(gd))
    want = full["delta_qkv"][0][:, 2 * n_k * 128:].reshape(B, n_v, 128) * full["delta_beta"][0][..., None]
    ok = ok and torch.equal(whole_d, want)
    # the conv weights follow the channels
    ok = ok and torch.equal(mine["conv_w"][0], full["conv_w"][0][plan.conv_channels()])
    ret[rank] = bool(ok)
    dist.destroy_process_group()


@pytest.mark.parametrize("mode,world", [("heads", 2), ("heads", 4), ("heads", 8), ("splitkv", 2)])
def test_step_plan_slices_and_gathered_blocks_round_trip(mode, world):
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 31500 + os.getpid() % 2000 + world
    mp.spawn(_plan_worker, args=(world, port, mode, ret), nprocs=world, join=True)
    assert all(ret[r] for r in range(world))


def test_step_plan_rejects_what_does_not_divide():
    from rapidllm_b200.shard import StepPlan
    with pytest.raises(ValueError):
        StepPlan("heads", 0, 3, 32)
    with pytest.raises(ValueError):
        StepPlan("heads", 0, 8, 31)                    # sequences x2 need an even batch
    with pytest.raises(ValueError):
        StepPlan("splitkv", 0, 5, 32)
    p = StepPlan("heads", 5, 8, 32)
    assert (p.head_ways, p.seq_ways, p.head_part, p.seq_part) == (4, 2, 1, 1)
    assert list(p.kv_heads) == [1] and list(p.q_heads) == list(range(6, 12)) and list(p.seqs) == list(range(16, 32))
    assert list(p.v_heads) == list(range(12, 24)) and list(p.k_heads) == [4, 5, 6, 7]
    s = StepPlan("splitkv", 7, 8, 32)
    assert list(s.q_heads) == list(range(24)) and list(s.v_heads) == list(range(42, 48)) and s.token_range(1000) == (896, 104)
