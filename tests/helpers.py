"""Shared builders for the GPU parity tests (seeded synthetic inputs)."""
import numpy as np
import torch

from rapidllm_b200 import ops

ATTN_MAX_ABS = 2e-2      # fp16-KV attention output tolerance (max-abs)
ATTN_REL_L2 = 1e-3       # fp16-KV attention output tolerance (relative L2)
STATE_REL_L2 = 1e-5      # FP32 DeltaNet state after many steps (relative L2)


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def paged_from_rows(k_rows, v_rows, gen, n_extra_pages=3, fill=None):
    """k_rows/v_rows: list of fp16 CPU tensors [len_b][n_kv][256].  Returns pools, table
    (shuffled page ids, int32 cuda [B][max_pages]) and seq_lens (cuda int32)."""
    n_kv = k_rows[0].shape[1]
    lens = [int(x.shape[0]) for x in k_rows]
    pages = [(n + 63) // 64 for n in lens]
    max_pages = max(1, max(pages))
    n_pages = sum(pages) + n_extra_pages
    perm = torch.randperm(n_pages, generator=gen).int()
    table = torch.zeros(len(lens), max_pages, dtype=torch.int32)
    at = 0
    for b, p in enumerate(pages):
        table[b, :p] = perm[at:at + p]
        at += p
    kp, vp = ops.new_pool(n_pages, n_kv), ops.new_pool(n_pages, n_kv)
    if fill is not None:
        kp.fill_(fill)
        vp.fill_(fill)
    table = table.cuda()
    for b, (kr, vr) in enumerate(zip(k_rows, v_rows)):
        if kr.shape[0]:
            ops.kv_append(kp, vp, table[b], kr.cuda(), vr.cuda(), pos0=0)
    return kp, vp, table, torch.tensor(lens, dtype=torch.int32, device="cuda")


def softplus(x):
    return torch.nn.functional.softplus(x)
