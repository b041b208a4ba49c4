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
