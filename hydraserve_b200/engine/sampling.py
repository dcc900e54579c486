"""Drop-in for ``hydraserve.engine.sampling`` backed by the sm_100a CUDA sampler.

The names, signatures, validation messages and result types are those of the reference
module (hydraserve/engine/sampling.py:8-163); the arithmetic is not done here.  Every
call packs the per-row parameters and token histories, hands device pointers to the
C-ABI library (``include/hs_sampler.h``) on the caller's current CUDA stream and unpacks
one result record per row.  There is no CPU code path: a tensor that lives on the host
is copied to the GPU and sampled there, and a missing library or GPU raises.

Extensions over the reference, all optional:

* ``request_ids`` (keyword-only).  When given, the token-count histogram of each request
  stays resident on the device between calls and only the tokens appended since the
  previous call are uploaded, instead of rebuilding the histogram from the full history
  every step (the reference's behaviour, sampling.py:106-110, which remains the default
  here).  ``release_request(request_id)`` frees a finished request's histogram, where the
  reference's backends release a request (serving_loop.py:1481-1488).
* ``sample_logits_packed``: the same call returning one array of fixed-size records
  instead of a tuple of per-row objects, for the worker-to-coordinator reply
  (pd_service.py:1097-1104) and the API layer (api/server.py:491-530).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, replace
from typing import Iterable, Sequence

__all__ = ["SamplingParams", "TokenSample", "sample_logits", "sample_logits_packed", "release_request"]

_RANGES = (
    # field, low, high, low-inclusive, message (the reference's wording)
    ("temperature", 0.0, 2.0, True, "temperature must be in [0, 2]"),
    ("top_p", 0.0, 1.0, False, "top_p must be in (0, 1]"),
    ("min_p", 0.0, 1.0, True, "min_p must be in [0, 1]"),
    ("repetition_penalty", 0.0, 2.0, False, "repetition_penalty must be in (0, 2]"),
    ("presence_penalty", -2.0, 2.0, True, "presence_penalty must be in [-2, 2]"),
    ("frequency_penalty", -2.0, 2.0, True, "frequency_penalty must be in [-2, 2]"),
)


@dataclass(frozen=True, slots=True)
class SamplingParams:
    """Per-request sampling parameters (reference sampling.py:8-44)."""

    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: int | None = None
    logprobs: int | None = None
    stop_token_sequences: tuple[tuple[int, ...], ...] = ()

    def __post_init__(self) -> None:
        for name, low, high, closed_low, message in _RANGES:
            value = getattr(self, name)
            above = value >= low if closed_low else value > low
            if not (above and value <= high):
                raise ValueError(message)
        if self.top_k < 0:
            raise ValueError("top_k cannot be negative")
        if self.seed is not None and not 0 <= self.seed < 2**63:
            raise ValueError("seed must be in [0, 2**63)")
        if self.logprobs is not None and not 0 <= self.logprobs <= 20:
            raise ValueError("logprobs must be in [0, 20]")
        for sequence in self.stop_token_sequences:
            if not sequence:
                raise ValueError("stop token sequences cannot be empty")

    def with_seed(self, seed: int) -> "SamplingParams":
        return replace(self, seed=seed)


@dataclass(frozen=True, slots=True)
class TokenSample:
    """One sampled token (reference sampling.py:47-51)."""

    token_id: int
    logprob: float | None = None
    top_logprobs: tuple[tuple[int, float], ...] = ()


_new_object = object.__new__
_set_token_id = TokenSample.token_id.__set__
_set_logprob = TokenSample.logprob.__set__
_set_top_logprobs = TokenSample.top_logprobs.__set__


def _token_only(token_id: int) -> TokenSample:
    """``TokenSample(token_id)`` without the frozen dataclass's ``__init__`` (which goes through
    ``object.__setattr__`` per field): the result path builds one per row and step."""
    sample = _new_object(TokenSample)
    _set_token_id(sample, token_id)
    _set_logprob(sample, None)
    _set_top_logprobs(sample, ())
    return sample


def _has_penalties(params: SamplingParams) -> bool:
    """reference sampling.py:94-99"""
    return not (
        params.repetition_penalty == 1.0
        and params.presence_penalty == 0.0
        and params.frequency_penalty == 0.0
    )


def _is_plain_greedy(params: SamplingParams) -> bool:
    """reference sampling.py:86-91"""
    return params.temperature == 0.0 and params.logprobs is None and not _has_penalties(params)


def _module():
    import sys

    return sys.modules[__name__]


def _checked(logits, histories, params, steps, request_ids):
    if logits.ndim != 2:
        raise ValueError("sampling logits must have shape [batch, vocabulary]")
    histories = tuple(histories)
    params = tuple(params)
    steps = tuple(int(step) for step in steps)
    if not (len(histories) == len(params) == len(steps) == logits.shape[0]):
        raise ValueError("sampling metadata must match the logits batch")
    if request_ids is not None and len(request_ids) != len(params):
        raise ValueError("sampling metadata must match the logits batch")
    return histories, params, steps


def sample_logits(
    logits,
    histories: Iterable[Iterable[int]],
    params: Iterable[SamplingParams],
    *,
    steps: Iterable[int],
    request_ids: Sequence | None = None,
) -> tuple[TokenSample, ...]:
    """Sample one token per logits row (reference sampling.py:54-83).

    ``logits``: ``[batch, vocabulary]`` tensor, bf16 or fp32 (other dtypes are widened to
    fp32), on the GPU or on the host.  ``histories``: prompt + generated ids per row.
    ``steps``: number of tokens generated so far per row; it advances the seeded stream.
    Raises ``ValueError`` for the same shape and length mismatches as the reference.
    """
    histories, params, steps = _checked(logits, histories, params, steps, request_ids)
    this = _module()
    from . import _device

    if os.environ.get("HYDRASERVE_BATCHED_GREEDY", "1") != "0" and all(
        this._is_plain_greedy(config) for config in params
    ):
        return _device.sample_batch(logits, None, params, steps, None, all_plain_greedy=True)
    if os.environ.get("HYDRASERVE_BATCHED_GREEDY", "1") == "0":
        # Per-row routing, as the reference does when its batched fast path is disabled
        # (sampling.py:69, :78-83): every row goes through the module-level _sample_row.
        return tuple(
            this._sample_row(logits[i], histories[i], params[i], steps[i])
            for i in range(len(params))
        )
    return _device.sample_batch(logits, histories, params, steps, request_ids)


def sample_logits_packed(
    logits,
    histories: Iterable[Iterable[int]],
    params: Iterable[SamplingParams],
    *,
    steps: Iterable[int],
    request_ids: Sequence | None = None,
):
    """``sample_logits`` with the result as one ``PackedSamples`` (an array of fixed-size
    records that indexes and iterates like the reference's tuple and pickles as bytes)."""
    histories, params, steps = _checked(logits, histories, params, steps, request_ids)
    from . import _device

    greedy = all(_is_plain_greedy(config) for config in params)
    return _device.sample_batch(logits, None if greedy else histories, params, steps,
                                None if greedy else request_ids, all_plain_greedy=greedy, packed=True)


def release_request(request_id, device=None) -> None:
    """Free the device-resident histogram of a finished request (one that was sampled with
    ``request_ids``); the place of the reference backends' ``release``
    (serving_loop.py:1481-1488).  Unknown ids are ignored."""
    from . import _device

    _device.release_request(request_id, device)


def _sample_row(logits, history, params: SamplingParams, step: int) -> TokenSample:
    """One row (reference sampling.py:102-163); ``logits`` is a 1-D tensor."""
    from . import _device

    return _device.sample_batch(logits.reshape(1, -1), (history,), (params,), (int(step),), None)[0]
