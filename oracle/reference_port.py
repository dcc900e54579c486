"""Timing stand-in for the reference's CPU sampling path.  TEST / BENCH INFRASTRUCTURE ONLY.

The reference checkout does not travel to the GPU box, so its CPU baseline is timed with
this port: the same sequence of PyTorch CPU operators, per row, that
hydraserve/engine/sampling.py:102-163 issues (clone, host-side histogram of the history,
gather/scatter penalties, topk, soft-max, full-vocabulary sort + cumsum, multinomial,
log-soft-max + topk), driven by the same per-row Python loop as sampling.py:78-83.
tests/test_oracle.py checks it against the golden outputs of the real reference, so what
is timed is known to compute the reference's results.  The precise checker used for
parity is oracle/sampler_oracle.py; this file exists so the baseline costs what the
reference costs.
"""
from __future__ import annotations

import torch

from .sampler_oracle import has_penalties, is_plain_greedy, mixed_seed


def _penalise_(scores: torch.Tensor, history, p) -> None:
    """reference sampling.py:105-120"""
    histogram: dict = {}
    vocab = scores.numel()
    for token in history:
        if 0 <= token < vocab:
            histogram[token] = histogram.get(token, 0) + 1
    if not histogram:
        return
    where = torch.tensor(tuple(histogram), dtype=torch.long)
    times = torch.tensor(tuple(histogram.values()), dtype=scores.dtype)
    picked = scores[where]
    scores[where] = torch.where(picked < 0, picked * p.repetition_penalty, picked / p.repetition_penalty)
    scores[where] -= p.presence_penalty
    scores[where] -= p.frequency_penalty * times


def _filter_(scores: torch.Tensor, p) -> torch.Tensor:
    """reference sampling.py:122-139"""
    scores /= p.temperature
    if p.top_k:
        kth = torch.topk(scores, min(p.top_k, scores.numel())).values[-1]
        scores = scores.masked_fill(scores < kth, float("-inf"))
    prob = torch.softmax(scores, dim=-1)
    if p.min_p:
        scores = scores.masked_fill(prob < prob.max() * p.min_p, float("-inf"))
    if p.top_p < 1.0:
        ordered, order = torch.sort(scores, descending=True)
        drop = torch.softmax(ordered, dim=-1).cumsum(dim=-1) > p.top_p
        drop[1:] = drop[:-1].clone()
        drop[0] = False
        scores[order[drop]] = float("-inf")
    return scores


def sample_row(row: torch.Tensor, history, p, step: int):
    """(token, logprob or None, top-logprob pairs) for one fp32 row."""
    scores = row.clone()
    if history and has_penalties(p):
        _penalise_(scores, history, p)
    if p.temperature == 0.0:
        token = int(scores.argmax())
    else:
        scores = _filter_(scores, p)
        prob = torch.softmax(scores, dim=-1)
        gen = None
        if p.seed is not None:
            gen = torch.Generator(device="cpu")
            gen.manual_seed(mixed_seed(p.seed, step))
        token = int(torch.multinomial(prob, 1, generator=gen))
    if p.logprobs is None:
        return token, None, ()
    logp = torch.log_softmax(scores, dim=-1)
    n = min(p.logprobs, scores.numel())
    pairs = ()
    if n:
        vals, ids = torch.topk(logp, n)
        pairs = tuple(zip(ids.tolist(), vals.tolist()))
    return token, float(logp[token]), pairs


def sample_batch(logits: torch.Tensor, histories, params, steps):
    """reference sampling.py:54-83: batched arg-max when every row is plain greedy,
    else the per-row loop over row.float()."""
    if all(is_plain_greedy(p) for p in params):
        return [(int(t), None, ()) for t in logits.argmax(dim=-1).tolist()]
    histories = [tuple(int(t) for t in h) for h in histories]
    return [sample_row(logits[i].float(), histories[i], params[i], int(steps[i]))
            for i in range(len(params))]
