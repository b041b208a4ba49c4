"""How the mixer operators of one decode step are divided among the GPUs of a node.

The reference is single-GPU (README "single-GPU / CPU engine"); this division is new.  Three
axes, none of which moves KV or state between GPUs:
  * sequences   -- every rank owns whole sequences (weak scaling, no exchange at all);
  * heads       -- rank r owns KV heads and DeltaNet value heads (with their key heads: value
                   head h uses key head h // 3, so groups of 3 stay together); outputs are
                   disjoint head slices, gathered with one all_gather;
  * kv_split    -- the ranks that share a KV head hold different pages of every sequence
                   (alternating pages: pages_of_part; or one contiguous page range per rank:
                   token_range_of_part, where the last rank holds the tail and appends) and
                   exchange (o, max, sum) partials, merged by rl_lse_combine.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class HeadShard:
    rank: int
    world: int
    kv_heads: range          # KV heads of this rank
    q_heads: range           # their query heads
    kv_split: int            # ranks sharing each of these KV heads (1 = no split)
    kv_part: int             # this rank's index among them
    v_heads: range           # DeltaNet value heads
    k_heads: range           # DeltaNet key/query heads (grouped map)

    @property
    def peers(self):
        """Ranks that hold the other token parts of the same KV heads (including this one)."""
        first = self.rank - self.kv_part * (self.world // self.kv_split)
        return [first + i * (self.world // self.kv_split) for i in range(self.kv_split)]


def plan_heads(rank: int, world: int, n_q=24, n_kv=4, n_v=48, n_k=16) -> HeadShard:
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank %d outside world %d" % (rank, world))
    if n_v % world or (n_v // world) % (n_v // n_k):
        raise ValueError("value heads %d (groups of %d) do not divide among %d ranks" % (n_v, n_v // n_k, world))
    g = n_q // n_kv
    if world <= n_kv:
        if n_kv % world:
            raise ValueError("KV heads %d do not divide among %d ranks" % (n_kv, world))
        per = n_kv // world
        kv = range(rank * per, (rank + 1) * per)
        split, part = 1, 0
    else:
        if world % n_kv:
            raise ValueError("%d ranks are not a multiple of %d KV heads" % (world, n_kv))
        split = world // n_kv
        kv = range(rank % n_kv, rank % n_kv + 1)
        part = rank // n_kv
    vper = n_v // world
    rep = n_v // n_k
    vh = range(rank * vper, (rank + 1) * vper)
    return HeadShard(rank, world, kv, range(kv.start * g, kv.stop * g), split, part, vh,
                     range(vh.start // rep, vh.stop // rep))


def pages_of_part(n_pages_seq: int, kv_split: int, kv_part: int):
    """Page indices (within a sequence) that part kv_part of a kv_split-way split holds."""
    return list(range(kv_part, n_pages_seq, kv_split))


def plan_sequences(rank: int, world: int, batch: int) -> range:
    per, extra = divmod(batch, world)
    start = rank * per + min(rank, extra)
    return range(start, start + per + (1 if rank < extra else 0))


def token_range_of_part(n_tokens: int, world: int, rank: int, page_tokens: int = 64):
    """(first token, token count) of the contiguous page range rank holds out of n_tokens.

    Whole pages go to every rank but the last, which also holds the partly filled tail page;
    a rank may hold nothing when there are fewer pages than ranks.
    """
    n_pages = (n_tokens + page_tokens - 1) // page_tokens
    p0, p1 = rank * n_pages // world, (rank + 1) * n_pages // world
    first = p0 * page_tokens
    last = n_tokens if rank == world - 1 else p1 * page_tokens
    return first, max(0, last - first)


@dataclass(frozen=True)
class StepPlan:
    """One rank's share of a decode step whose batch is divided over `world` ranks, and how the
    all-gathered outputs (rl_stack_gather: block r = rank r's local output) map back to the whole.

    mode "heads":   KV / value heads over head_ways = min(world, n_kv) ranks, then the sequences
                    over world / head_ways; rank = seq_part * head_ways + head_part.
    mode "splitkv": every rank holds a token range of every sequence and all attention heads
                    (partials merged by the library into attn_o_final); DeltaNet value heads / world.
    mode "seq":     whole sequences per rank, nothing gathered (weak scaling).
    """
    mode: str
    rank: int
    world: int
    batch: int
    n_q: int = 24
    n_kv: int = 4
    n_v: int = 48
    n_k: int = 16

    def __post_init__(self):
        if self.mode not in ("heads", "splitkv", "seq"):
            raise ValueError("unknown mode %r" % self.mode)
        if not 0 <= self.rank < self.world:
            raise ValueError("rank %d outside world %d" % (self.rank, self.world))
        if self.mode == "heads":
            if self.n_kv % self.head_ways or self.world % self.head_ways or self.batch % self.seq_ways:
                raise ValueError("heads x%d / sequences x%d do not divide %d KV heads, batch %d"
                                 % (self.head_ways, self.seq_ways, self.n_kv, self.batch))
        if self.mode != "seq" and (self.n_k % self.delta_ways or self.n_v % self.delta_ways):
            raise ValueError("%d ranks do not divide the DeltaNet heads" % self.delta_ways)

    # ---- how many ways each axis is cut ----
    @property
    def head_ways(self):
        return min(self.world, self.n_kv) if self.mode == "heads" else 1

    @property
    def seq_ways(self):
        return self.world // self.head_ways if self.mode == "heads" else 1

    @property
    def delta_ways(self):
        return {"heads": self.head_ways, "splitkv": self.world, "seq": 1}[self.mode]

    @property
    def head_part(self):
        return self.rank % self.head_ways

    @property
    def delta_part(self):
        return self.rank if self.mode == "splitkv" else self.head_part

    @property
    def seq_part(self):
        return self.rank // self.head_ways if self.mode == "heads" else 0

    # ---- this rank's slices of the whole problem ----
    @property
    def seqs(self):
        return plan_sequences(self.seq_part, self.seq_ways, self.batch)

    @property
    def kv_heads(self):
        per = self.n_kv // self.head_ways
        return range(self.head_part * per, (self.head_part + 1) * per)

    @property
    def q_heads(self):
        g = self.n_q // self.n_kv
        return range(self.kv_heads.start * g, self.kv_heads.stop * g)

    @property
    def v_heads(self):
        per = self.n_v // self.delta_ways
        return range(self.delta_part * per, (self.delta_part + 1) * per)

    @property
    def k_heads(self):
        per = self.n_k // self.delta_ways
        return range(self.delta_part * per, (self.delta_part + 1) * per)

    def conv_channels(self, dk=128, dv=128):
        """Indices, in the full q | k | v channel vector, of this rank's conv channels (in the order
        of the local q | k | v layout)."""
        kq = self.n_k * dk
        out = list(range(self.k_heads.start * dk, self.k_heads.stop * dk))
        out += [kq + c for c in range(self.k_heads.start * dk, self.k_heads.stop * dk)]
        out += [2 * kq + c for c in range(self.v_heads.start * dv, self.v_heads.stop * dv)]
        return out

    def token_range(self, n_tokens, page_tokens=64):
        """(first, count) of the tokens of a sequence of n_tokens this rank holds."""
        if self.mode == "splitkv":
            return token_range_of_part(n_tokens, self.world, self.rank, page_tokens)
        return 0, n_tokens

    def slice_io(self, full):
        """The local tensors of a step from the whole problem's (rl_stack_io names; torch tensors or
        numpy arrays with the layouts of the header)."""
        s, qh, kvh, vh = list(self.seqs), list(self.q_heads), list(self.kv_heads), list(self.v_heads)
        ch = self.conv_channels()
        cut = {
            "attn_q": lambda x: x[:, s][:, :, qh], "attn_gate": lambda x: x[:, s][:, :, qh],
            "attn_k": lambda x: x[:, s][:, :, kvh], "attn_v": lambda x: x[:, s][:, :, kvh],
            "delta_qkv": lambda x: x[:, s][:, :, ch], "delta_beta": lambda x: x[:, s][:, :, vh],
            "delta_g": lambda x: x[:, s][:, :, vh], "conv_w": lambda x: x[:, ch],
        }
        return {n: cut[n](x) for n, x in full.items() if n in cut}

    # ---- gathered blocks -> the whole ----
    def place_attn(self, out, gathered):
        """gathered [world][B_local][n_q_local][256] (one layer of attn_o_all) -> out [batch][n_q][256]."""
        for r in range(self.world):
            p = StepPlan(self.mode, r, self.world, self.batch, self.n_q, self.n_kv, self.n_v, self.n_k)
            out[p.seqs.start:p.seqs.stop, p.q_heads.start:p.q_heads.stop] = gathered[r]
        return out

    def place_delta(self, out, gathered):
        """gathered [world][B_local][n_v_local][dv] (one layer of delta_o_all) -> out [batch][n_v][dv]."""
        for r in range(self.world):
            p = StepPlan(self.mode, r, self.world, self.batch, self.n_q, self.n_kv, self.n_v, self.n_k)
            out[p.seqs.start:p.seqs.stop, p.v_heads.start:p.v_heads.stop] = gathered[r]
        return out
