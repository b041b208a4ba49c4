"""One decode step of a small hybrid stack divided over 2 GPUs (one process per GPU, the library's
own all-gather over NCCL on its side stream, rl_stack_set_gather) against the CPU oracle run over
the WHOLE problem: KV / value heads 2-way, and token ranges of every sequence 2-way (split-KV
partials merged by log-sum-exp).  Needs two GPUs; skipped on a single-GPU box.
No rank ever waits on a device-side flag: every wait is NCCL's or the host's, and the child
processes run under a time limit."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = pytest.mark.gpu

N_Q, N_KV, HD, N_V, N_K = 24, 4, 256, 48, 16
CONV_DIM = 2 * N_K * 128 + N_V * 128


def _problem(seed, lens, n_periods):
    """Whole-problem inputs, the same on every rank."""
    g = torch.Generator().manual_seed(seed)
    A, D, B = n_periods, 3 * n_periods, len(lens)
    p = {"attn_q": torch.randn(A, B, N_Q, HD, generator=g), "attn_gate": torch.randn(A, B, N_Q, HD, generator=g),
         "attn_k": torch.randn(A, B, N_KV, HD, generator=g), "attn_v": torch.randn(A, B, N_KV, HD, generator=g),
         "delta_qkv": torch.randn(D, B, CONV_DIM, generator=g),
         "delta_beta": torch.sigmoid(torch.randn(D, B, N_V, generator=g)),
         "delta_g": -torch.nn.functional.softplus(torch.randn(D, B, N_V, generator=g)),
         "conv_w": torch.randn(D, CONV_DIM, 4, generator=g) * 0.5}
    p["k_hist"] = [[torch.randn(n, N_KV, HD, generator=g).half() for n in lens] for _ in range(A)]
    p["v_hist"] = [[torch.randn(n, N_KV, HD, generator=g).half() for n in lens] for _ in range(A)]
    p["S0"] = [torch.randn(B, N_V, 128, 128, generator=g) * 0.02 for _ in range(D)]
    p["C0"] = [torch.randn(B, CONV_DIM, 4, generator=g) for _ in range(D)]
    return p


def _worker(rank, world, port, mode, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from rapidllm_b200 import _lib, ops
    from rapidllm_b200.cache import QWEN35_LAYER_TYPES, Comm, HybridCache
    from rapidllm_b200.shard import StepPlan
    lens = [100, 63, 257, 1]                           # tokens cached per sequence before the step
    n_periods = 2
    prob = _problem(7, lens, n_periods)
    B = len(lens)
    plan = StepPlan(mode, rank, world, B)
    split = mode == "splitkv"
    last = (not split) or rank == world - 1
    # tokens of each sequence held here: history range, and what pos[] is on this rank
    hist, pos = [], []
    for n in lens:
        first, n_loc = plan.token_range(n + 1)
        n_h = n_loc - 1 if last else n_loc
        hist.append((first, max(0, n_h)))
        pos.append(max(0, n_h))
    pages = [(h[1] + 1 + 63) // 64 for h in hist]
    max_pages, n_pages = max(pages), sum(pages) + 1
    cache = HybridCache(QWEN35_LAYER_TYPES * n_periods, n_pages=n_pages, n_slots=B, max_batch=B,
                        max_pages_per_seq=max_pages, n_q=len(plan.q_heads), n_kv=len(plan.kv_heads),
                        n_v=len(plan.v_heads), n_k=len(plan.k_heads))
    g = torch.Generator().manual_seed(100 + rank)
    perm = torch.randperm(n_pages, generator=g).int()
    table = torch.zeros(B, max_pages, dtype=torch.int32)
    at = 0
    for b, p in enumerate(pages):
        table[b, :p] = perm[at:at + p]
        at += p
    kvh, vh = list(plan.kv_heads), list(plan.v_heads)
    for a in range(cache.n_attn):
        for b in range(B):
            first, n_h = hist[b]
            if n_h:
                ops.kv_append(cache.k_pool(a), cache.v_pool(a), table[b].cuda(),
                              prob["k_hist"][a][b][first:first + n_h][:, kvh].contiguous().cuda(),
                              prob["v_hist"][a][b][first:first + n_h][:, kvh].contiguous().cuda(), pos0=0)
    for d in range(cache.n_delta):
        cache.state(d).copy_(prob["S0"][d][:, vh])
        cache.set_conv_windows(d, prob["C0"][d][:, plan.conv_channels()])
    dev = {n: x.contiguous().cuda() for n, x in plan.slice_io(prob).items()}
    sh = cache.io_shapes(B)
    dev["attn_o"] = torch.zeros(sh["attn_o"], device="cuda")
    dev["delta_o"] = torch.zeros(sh["delta_o"], device="cuda")
    dev["page_table"] = table.cuda()
    dev["pos"] = torch.tensor(pos, dtype=torch.int32, device="cuda")
    if split:
        dev["attn_ml"] = torch.zeros(sh["attn_ml"], device="cuda")
        dev["no_append"] = not last

    def bcast(raw):
        t = torch.zeros(_lib.COMM_ID_BYTES, dtype=torch.uint8, device="cuda")
        if raw is not None:
            t.copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
        dist.broadcast(t, 0)
        return t.cpu().numpy().tobytes()
    comm = Comm(rank, world, bcast)
    gs = cache.gather_shapes(B, world)
    gathered = {n: torch.zeros(gs[n], device="cuda") for n in gs if split or not n.startswith("attn_ml") and n != "attn_o_final"}
    cache.set_gather(comm, gathered)
    cache.decode(dev, B)
    torch.cuda.synchronize()
    _lib.check_device()
    out = None
    if rank == 0:
        attn = np.stack([(gathered["attn_o_final"][a] if split else
                          plan.place_attn(torch.zeros(B, N_Q, HD, device="cuda"), gathered["attn_o_all"][a])).cpu().numpy()
                         for a in range(cache.n_attn)])
        delta = np.stack([plan.place_delta(torch.zeros(B, N_V, 128, device="cuda"), gathered["delta_o_all"][d]).cpu().numpy()
                          for d in range(cache.n_delta)])
        out = (attn, delta)
    ret[rank] = out
    dist.barrier()
    cache.close()
    comm.close()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("mode", ["heads", "splitkv"])
def test_two_gpu_sharded_step_matches_the_oracle(oracle, mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from helpers import ATTN_MAX_ABS, ATTN_REL_L2, rel_l2
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 33500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, mode, ret), nprocs=world, join=True)
    attn, delta = ret[0]
    lens = [100, 63, 257, 1]
    prob = _problem(7, lens, 2)
    for a in range(2):
        for b, n in enumerate(lens):
            k = torch.cat([prob["k_hist"][a][b], prob["attn_k"][a, b:b + 1].half()]).float().numpy()
            v = torch.cat([prob["v_hist"][a][b], prob["attn_v"][a, b:b + 1].half()]).float().numpy()
            ref = oracle.gated_attn_decode(prob["attn_q"][a, b].numpy(), k, v, prob["attn_gate"][a, b].numpy())
            assert np.abs(attn[a, b] - ref).max() <= ATTN_MAX_ABS, (mode, a, b)
            assert rel_l2(attn[a, b], ref) <= ATTN_REL_L2, (mode, a, b)
    nk = N_K * 128
    for d in range(6):
        for b in range(len(lens)):
            C = prob["C0"][d][b].numpy().copy()
            S = prob["S0"][d][b].numpy().copy()
            mixed = oracle.conv1d_update(prob["delta_qkv"][d, b].numpy(), prob["conv_w"][d].numpy(), C)
            q = oracle.repeat_heads(mixed[:nk].reshape(N_K, 128), N_V)
            k = oracle.repeat_heads(mixed[nk:2 * nk].reshape(N_K, 128), N_V)
            ref = oracle.delta_step(S, q, k, mixed[2 * nk:].reshape(N_V, 128), prob["delta_beta"][d, b].numpy(),
                                    prob["delta_g"][d, b].numpy())
            assert np.abs(delta[d, b] - ref).max() < 1e-4, (mode, d, b)
