"""CPU checker for the per-step token sampler.  TEST INFRASTRUCTURE ONLY.

This file restates, in numpy, what HydraServe's sampler computes for one logits row
(reference: hydraserve/engine/sampling.py:54-163).  Only tests, the smoke check and the
CPU-baseline leg of the benchmark may import it; the product path never does.

Parity pin: tests/golden/*.npz hold outputs of the unmodified reference sampler run on
seeded inputs (tests/golden/make_golden.py is the generating script); tests/test_oracle.py
checks this restatement against them and against the reference's own unit-test cases
(tests/test_sampling.py:17-111 of the reference).

Arithmetic.  The reference's arithmetic lives in PyTorch (pyproject.toml:15 pins
torch>=2.1).  Steps whose result is fixed by IEEE fp32 (penalties, the temperature
division, comparisons) are restated in fp32 in the same order, and agree bit for bit.
Steps whose low bits depend on the library's summation order (the soft-max denominators;
torch's vectorised CPU sum carries about 5e-6 relative error on a 150k-wide row) are
restated in fp64.  Every cut therefore comes with a margin: how far, relatively, the
deciding quantity was from its threshold.  A cut whose margin is below the noise of the
implementation it is compared with is reported as rounding-sensitive, not as a mismatch.

Tie rules, where the reference leaves them to the sort/topk implementation: a top-p cut
that falls inside a group of equal scores keeps the lowest token ids of the group;
equal log-probabilities are listed by ascending token id.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

F32 = np.float32
SEED_STRIDE = 0x1E3779B97F4A7C15  # reference sampling.py:148


def mixed_seed(seed: int, step: int) -> int:
    """Per-step generator seed (reference sampling.py:148)."""
    return (int(seed) + (int(step) + 1) * SEED_STRIDE) % (2 ** 63)


def has_penalties(p) -> bool:
    """reference sampling.py:94-99"""
    return p.repetition_penalty != 1.0 or p.presence_penalty != 0.0 or p.frequency_penalty != 0.0


def is_plain_greedy(p) -> bool:
    """reference sampling.py:86-91"""
    return p.temperature == 0.0 and not has_penalties(p) and p.logprobs is None


def history_counts(history, vocab: int):
    """Unique in-range token ids and their multiplicities (reference sampling.py:106-110)."""
    h = np.asarray(history, dtype=np.int64).reshape(-1)
    h = h[(h >= 0) & (h < vocab)]
    if h.size == 0:
        return np.zeros(0, np.int64), np.zeros(0, np.int64)
    ids, counts = np.unique(h, return_counts=True)
    return ids, counts


def penalise(row: np.ndarray, history, p) -> np.ndarray:
    """Repetition, presence and frequency penalties, three separately rounded fp32 steps
    per unique history id (reference sampling.py:105-120)."""
    y = np.array(row, dtype=F32, copy=True)
    if not has_penalties(p):
        return y
    ids, counts = history_counts(history, y.size)
    if ids.size == 0:
        return y
    v = y[ids]
    rp = F32(p.repetition_penalty)
    v = np.where(v < 0, v * rp, v / rp).astype(F32)
    v = (v - F32(p.presence_penalty)).astype(F32)
    v = (v - (F32(p.frequency_penalty) * counts.astype(F32)).astype(F32)).astype(F32)
    y[ids] = v
    return y


def exponential_draws(seed64: int, vocab: int) -> np.ndarray:
    """The V Exp(1) variates torch.multinomial consumes on CPU for a generator seeded
    with ``seed64`` (reference sampling.py:146-150: multinomial(p, 1) == argmax(p / q))."""
    import torch

    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed64))
    return torch.empty(vocab, dtype=torch.float32).exponential_(1.0, generator=g).numpy()


@dataclass
class OracleRow:
    token: int
    logprob: float | None
    top_logprobs: tuple
    scores: np.ndarray  # final fp32 scores, -inf where filtered (the reference's `scores`)
    penalised: np.ndarray  # fp32 logits after penalties, before temperature
    kept: np.ndarray  # sorted int64 ids of the final candidate set
    n_after_topk: int
    n_after_minp: int
    n_after_topp: int
    margins: dict = field(default_factory=dict)
    probabilities: np.ndarray | None = None  # fp64 over the final set (non-greedy rows)


def _softmax64(scores: np.ndarray):
    finite = np.isfinite(scores)
    m = scores[finite].max()
    e = np.zeros(scores.shape, np.float64)
    e[finite] = np.exp(scores[finite].astype(np.float64) - np.float64(m))
    z = e.sum()
    return e / z, m, z


def scaled_scores(row, history, p):
    """Penalised logits and the scores the filters see: penalties, then the true fp32
    division by the temperature (reference sampling.py:105-123).  Greedy rows are not scaled."""
    y = penalise(np.asarray(row, dtype=F32), history, p)
    if p.temperature == 0.0:
        return y, y.copy()
    return y, (y / F32(p.temperature)).astype(F32)


def sample_row(row, history, p, step: int, *, draws: np.ndarray | None = None,
               want_probabilities: bool = True) -> OracleRow:
    """One row through penalties -> temperature -> top-k -> min-p -> top-p -> draw ->
    log-probabilities (reference sampling.py:102-163).

    ``draws``: the Exp(1) variates to use for the draw; default = the reference's own
    (``exponential_draws(mixed_seed(seed, step), V)``)."""
    y, scores = scaled_scores(row, history, p)
    return sample_from_scores(y, scores, p, step, draws=draws, want_probabilities=want_probabilities)


def sample_from_scores(y, scores, p, step: int, *, draws: np.ndarray | None = None,
                       want_probabilities: bool = True) -> OracleRow:
    """The filters, the draw and the log-probabilities on already scaled scores
    (reference sampling.py:124-163); -inf entries are tokens that are not candidates."""
    scores = np.array(scores, dtype=F32, copy=True)
    vocab = scores.size
    margins: dict = {}
    greedy = p.temperature == 0.0
    n_k = n_m = n_p = vocab
    if not greedy:
        if p.top_k:  # :124-127, ties at the k-th value stay
            keep = min(int(p.top_k), vocab)
            kth = np.partition(scores, vocab - keep)[vocab - keep]
            scores = np.where(scores < kth, F32(-np.inf), scores)
        n_k = int(np.isfinite(scores).sum())
        if p.min_p:  # :129-132, relative to the soft-max over the top-k survivors
            prob, _, _ = _softmax64(scores)
            thr32 = F32(F32(prob.max()) * F32(p.min_p))
            live = np.isfinite(scores)
            ratio = prob[live] / np.float64(thr32)
            margins["min_p"] = float(np.min(np.abs(ratio - 1.0)))
            scores = np.where(prob.astype(F32) < thr32, F32(-np.inf), scores)
        n_m = int(np.isfinite(scores).sum())
        if p.top_p < 1.0:  # :133-139
            live_ids = np.nonzero(np.isfinite(scores))[0]
            order = live_ids[np.argsort(-scores[live_ids], kind="stable")]  # ties: low id first
            e = np.exp(scores[order].astype(np.float64) - np.float64(scores[order[0]]))
            pr32 = (e / e.sum()).astype(F32)
            cum32 = np.cumsum(pr32.astype(np.float64)).astype(F32)
            over = cum32 > F32(p.top_p)
            n_keep = int(np.argmax(over)) + 1 if over.any() else order.size
            cum64 = np.cumsum(e / e.sum())
            near = [abs(cum64[n_keep - 1] - p.top_p)]
            if n_keep >= 2:
                near.append(abs(cum64[n_keep - 2] - p.top_p))
            margins["top_p"] = float(min(near))
            margins["top_p_step"] = float(e[n_keep - 1] / e.sum())
            cut_value = scores[order[n_keep - 1]]
            margins["top_p_splits_tie"] = bool(
                n_keep < order.size and scores[order[n_keep]] == cut_value)
            dropped = order[n_keep:]
            scores[dropped] = F32(-np.inf)
        n_p = int(np.isfinite(scores).sum())

    kept = np.nonzero(np.isfinite(scores))[0]
    probabilities = None
    if greedy:
        token = int(np.argmax(scores))  # first occurrence = lowest id, :142
        vals = np.sort(scores)[-2:] if vocab > 1 else None
        if vals is not None:
            margins["greedy_tie"] = bool(vals[0] == vals[1])
    else:
        prob64, _, _ = _softmax64(scores)
        probabilities = prob64 if want_probabilities else None
        if draws is None:
            if p.seed is None:
                raise ValueError("the checker needs a seed (the reference would use the global RNG)")
            draws = exponential_draws(mixed_seed(p.seed, step), vocab)
        race = (prob64.astype(F32) / np.asarray(draws, dtype=F32)).astype(F32)
        token = int(np.argmax(race))
        if kept.size > 1:
            top2 = np.partition(race[kept], kept.size - 2)[-2:]
            margins["draw"] = float(1.0 - top2[0] / top2[1]) if top2[1] > 0 else 0.0

    logprob = None
    top = ()
    if p.logprobs is not None:  # :152-163
        m = scores[kept].max()
        z = np.exp(scores[kept].astype(np.float64) - np.float64(m)).sum()
        logp = scores.astype(np.float64) - np.float64(m) - np.log(z)
        logprob = float(F32(logp[token]))
        n = min(int(p.logprobs), vocab)
        if n:
            take = kept[np.lexsort((kept, -scores[kept]))][:n]
            top = tuple((int(i), float(F32(logp[i]))) for i in take)
            if len(top) < n:  # the reference pads with (some filtered id, -inf)
                filler = []
                kept_set = set(kept.tolist())
                i = 0
                while len(top) + len(filler) < n:
                    if i not in kept_set:
                        filler.append((i, float("-inf")))
                    i += 1
                top = top + tuple(filler)
    return OracleRow(token, logprob, top, scores, y, kept, n_k, n_m, n_p, margins, probabilities)


def sample_batch(logits_f32: np.ndarray, histories, params, steps, **kwargs):
    """Rows are independent (reference sampling.py:78-83)."""
    return [sample_row(logits_f32[i], histories[i], params[i], int(steps[i]), **kwargs)
            for i in range(len(params))]
