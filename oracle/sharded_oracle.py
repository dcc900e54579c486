"""CPU checker for vocabulary-sharded sampling.  TEST INFRASTRUCTURE ONLY.

The reference has no tensor-parallel LM head (its only collective is an 8-byte all-reduce,
hydraserve/engine/dp_graph_sync.py:22-40), so the oracle for the sharded configuration is
the reference sampler on the concatenated row (sampler_oracle.sample_row).  This file
restates the sharded algorithm itself on the CPU -- per-slice candidates, exchange, merge --
so that its claim (the union of the slices' top-k candidates yields the row's result) is
checked without a GPU, over a real process group.
"""
from __future__ import annotations

import numpy as np

from . import sampler_oracle as O

F32 = np.float32


def shard_bounds(vocab: int, ranks: int):
    """Contiguous, equal-width slices (the last one takes the remainder)."""
    width = (vocab + ranks - 1) // ranks
    return [(r * width, min(vocab, (r + 1) * width)) for r in range(ranks)]


def local_history(history, lo: int, hi: int) -> np.ndarray:
    """History ids that fall into [lo, hi), renumbered from the slice start."""
    h = np.asarray(history, dtype=np.int64).reshape(-1)
    return (h[(h >= lo) & (h < hi)] - lo).astype(np.int32)


def partial(slice_row, history_local, p, offset: int):
    """One slice of one row -> (global ids, scores) of its top-k with ties at the k-th,
    plus (max score, sum exp(score - max)) of the whole slice."""
    _, scores = O.scaled_scores(slice_row, history_local, p)
    k = min(int(p.top_k), scores.size)
    kth = np.partition(scores, scores.size - k)[scores.size - k]
    ids = np.nonzero(scores >= kth)[0]
    m = scores.max()
    z = np.exp(scores.astype(np.float64) - np.float64(m)).sum()
    return ids + offset, scores[ids], float(m), float(z)


def merge(vocab: int, parts, p, step: int, draws=None) -> O.OracleRow:
    """Union of the slices' candidates -> the row's result: every other token is out (-inf),
    then the reference's filters run as on a full row."""
    scores = np.full(vocab, -np.inf, dtype=F32)
    for ids, vals, _, _ in parts:
        scores[ids] = vals
    return O.sample_from_scores(scores, scores, p, step, draws=draws, want_probabilities=False)


def full_logsumexp(parts) -> float:
    m = max(part[2] for part in parts)
    return float(m + np.log(sum(part[3] * np.exp(part[2] - m) for part in parts)))
