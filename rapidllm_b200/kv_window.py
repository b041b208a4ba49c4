"""The compact-KV policy of one attention layer: q8-K / TQ3-V pages persist for the whole
context, an F16 compute window covers the first `window_tokens` tokens of every sequence, and
attention runs over the window while everything it needs is inside it.

Mirrors the engine's rules (src/kernels/cuda/cuda_engine.cu):
  * every token is stored in the compact cache, also while the window is in use, so that the
    first step past the window finds tokens 0 .. window-1 there (6033-6036);
  * a decode step writes and reads the F16 window iff pos < window, else it attends over the
    compact cache alone (18948-18953); a batched step decides once for the whole batch (19048);
  * a prefill chunk [pos0, tend) is stored in the window and attends over it iff
    tend <= window (18487-18490), else it attends over the compact cache (18493-18497) - here
    through F16 scratch pages dequantised from it, which the tensor-core prefill reads.
Sizes come from rl_plan_cache (window_tokens, window_pages_per_seq).
"""
from __future__ import annotations

import torch

from . import _lib, ops

PAGE = ops.PAGE_TOKENS


class WindowedKV:
    def __init__(self, max_batch: int, ctx: int, window_tokens: int, n_q=24, n_kv=4, wht_len=128, signs=None,
                 device="cuda"):
        if not 0 < window_tokens <= ctx:
            raise _lib.RlError(6, "window_tokens %d outside (0, ctx=%d]" % (window_tokens, ctx))
        self.max_batch, self.ctx, self.window, self.n_q, self.n_kv = max_batch, ctx, window_tokens, n_q, n_kv
        self.wht_len, self.signs, self.device = wht_len, signs, device
        self.pages_c, self.pages_w = -(-ctx // PAGE), -(-window_tokens // PAGE)
        self.pool = ops.new_compact_pool(max_batch * self.pages_c, n_kv, device)
        self.k_win = ops.new_pool(max_batch * self.pages_w, n_kv, device)
        self.v_win = ops.new_pool(max_batch * self.pages_w, n_kv, device)
        self.table_c = torch.arange(max_batch * self.pages_c, dtype=torch.int32, device=device).view(max_batch, -1)
        self.table_w = torch.arange(max_batch * self.pages_w, dtype=torch.int32, device=device).view(max_batch, -1)
        self.lens = [0] * max_batch                 # host positions, like the engine's pos_
        self._scratch = None                        # F16 pages for a prefill chunk past the window
        self.last_path = None                       # "window" or "compact": which cache the last call attended over

    def bytes(self):
        n = self.pool.numel() + 2 * self.k_win.numel() * 2
        return n + (0 if self._scratch is None else 2 * self._scratch[0].numel() * 2)

    def _dev(self, values):
        return torch.tensor(values, dtype=torch.int32, device=self.device)

    def decode(self, seqs, q, k_row, v_row, gate):
        """One token per listed sequence: store its K/V row, attend over [0, pos], gate.
        q, gate fp32 [B][n_q][256]; k_row, v_row fp32 [B][n_kv][256]."""
        pos = [self.lens[s] for s in seqs]
        if max(pos) >= self.ctx:
            raise _lib.RlError(6, "sequence is at ctx %d" % self.ctx)
        use_win = max(pos) < self.window            # one decision for the batch
        pos_d = self._dev(pos)
        idx = torch.as_tensor(list(seqs), device=self.device)
        ops.kv_compact_append(self.pool, self.table_c[idx], k_row.unsqueeze(1), v_row.unsqueeze(1), self.wht_len,
                              self.signs, pos=pos_d)
        lens_d = pos_d + 1
        # the window rows of every sequence still inside it stay current, whichever cache this batch reads
        inside = [i for i, p in enumerate(pos) if p < self.window]
        if inside:
            sub = slice(None) if len(inside) == len(pos) else torch.as_tensor(inside, device=self.device)
            ops.kv_append(self.k_win, self.v_win, self.table_w[idx][sub].contiguous(),
                          k_row[sub].unsqueeze(1).contiguous(), v_row[sub].unsqueeze(1).contiguous(),
                          pos=pos_d[sub].contiguous())
        if use_win:
            o = ops.attn_decode(q, self.k_win, self.v_win, self.table_w[idx], lens_d, gate,
                                max_seq_len=self.pages_w * PAGE)
        else:
            o = ops.attn_decode(q, self.pool, None, self.table_c[idx], lens_d, gate,
                                max_seq_len=self.pages_c * PAGE, wht_len=self.wht_len, signs=self.signs)
        for s in seqs:
            self.lens[s] += 1
        self.last_path = "window" if use_win else "compact"
        return o

    def prefill(self, seq, q, k_rows, v_rows, gate=None):
        """One chunk of one sequence at its current position: q bf16 [T][n_q][256], k_rows, v_rows
        fp32 [T][n_kv][256] (already normed and rotated), gate fp32 [T][n_q][256] or None."""
        pos0, T = self.lens[seq], q.shape[0]
        tend = pos0 + T
        if tend > self.ctx:
            raise _lib.RlError(6, "chunk ends at %d, ctx is %d" % (tend, self.ctx))
        ops.kv_compact_append(self.pool, self.table_c[seq], k_rows, v_rows, self.wht_len, self.signs, pos0=pos0)
        if tend <= self.window:
            ops.kv_append(self.k_win, self.v_win, self.table_w[seq], k_rows, v_rows, pos0=pos0)
            o = ops.attn_prefill(q, self.k_win, self.v_win, self.table_w[seq], pos0, None, None, gate)
            self.last_path = "window"
        else:
            if self._scratch is None:
                self._scratch = (ops.new_pool(self.pages_c, self.n_kv, self.device),
                                 ops.new_pool(self.pages_c, self.n_kv, self.device),
                                 torch.arange(self.pages_c, dtype=torch.int32, device=self.device))
            ks, vs, ts = self._scratch
            ops.kv_compact_to_f16(self.pool, self.table_c[seq], ks, vs, ts, tend, 0, 0, self.wht_len, self.signs)
            o = ops.attn_prefill(q, ks, vs, ts, pos0, None, None, gate)
            self.last_path = "compact"
        self.lens[seq] = tend
        return o

    def reset(self, seq):
        self.lens[seq] = 0
