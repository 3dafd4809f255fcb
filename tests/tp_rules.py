"""Tensor-parallel sharding rules of the decoder (host mirror of what
qeng_decoder_load_matrix keeps on each rank): q/k/v/gate/up are split by output
rows (whole heads / FFN columns per rank, no exchange), o/down by input columns
in whole 32-blocks (partial sums, one all-reduce each)."""
from __future__ import annotations

ROW_SPLIT = {"wo", "wdown"}          # split along K: partial sums
COLUMN_SPLIT = {"wq", "wk", "wv", "wgate", "wup"}


def shard_bounds(name, n, k, rank, world):
    """(row0, row1, col0, col1) of the shard rank holds of the [n, k] matrix `name`."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    if name in ROW_SPLIT:
        if k % (32 * world):
            raise ValueError("%s: K=%d does not split into whole 32-blocks over %d ranks" % (name, k, world))
        return 0, n, k // world * rank, k // world * (rank + 1)
    if name in COLUMN_SPLIT:
        if n % (16 * world):
            raise ValueError("%s: N=%d does not split into whole 16-row tiles over %d ranks" % (name, n, world))
        return n // world * rank, n // world * (rank + 1), 0, k
    raise ValueError("unknown matrix %r" % name)


def shard_matrix(name, q, s, rank, world):
    """Codes and scales of the shard (views of the full host arrays)."""
    r0, r1, c0, c1 = shard_bounds(name, q.shape[0], q.shape[1], rank, world)
    return q[r0:r1, c0:c1], s[r0:r1, c0 // 32:c1 // 32]


def vocab_shard(vocab, rank, world):
    """(v0, v1): LM-head rows a rank keeps.  The head is split only when the vocabulary divides
    evenly (and indices stay exact in f32, the type the (max, index) pairs travel in);
    otherwise every rank keeps the whole head."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    if world > 1 and vocab % world == 0 and vocab <= 1 << 24:
        return vocab // world * rank, vocab // world * (rank + 1)
    return 0, vocab


def pick_token(pairs):
    """pairs [world][batch][2] = (max logit, global index as f32) gathered from the ranks ->
    token per sequence: the largest value, the lowest index on ties (what the unsharded argmax returns)."""
    out = []
    for b in range(len(pairs[0])):
        best_v, best_i = float("-inf"), 1 << 31
        for r in range(len(pairs)):
            v, i = float(pairs[r][b][0]), int(pairs[r][b][1])
            if v > best_v or (v == best_v and i < best_i):
                best_v, best_i = v, i
        out.append(best_i)
    return out


def all_reduces_per_step(layers):
    return 2 * layers
