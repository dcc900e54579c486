"""Seeded synthetic inputs for the sampler: the five benchmark configurations.

Every generator is a pure function of its seed (``numpy.random.default_rng``), so the
CPU checker, the GPU tests, the golden-fixture script and ``bench.py`` all see the very
same rows.  Logits are returned as numpy arrays: ``float32`` for fp32 configurations and
``uint16`` bf16 bit patterns for bf16 ones (numpy has no bf16 type); histories are int32
arrays; parameters are :class:`hydraserve_b200.engine.sampling.SamplingParams`.

No dataset is involved anywhere on this path: the shapes, value distributions and
parameter mixes below are the inputs.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .engine.sampling import SamplingParams

__all__ = [
    "Workload",
    "f32_to_bf16_bits",
    "bf16_bits_to_f32",
    "config1",
    "config2",
    "config3",
    "config4",
    "config5",
    "by_name",
]


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round fp32 to bf16 (nearest even) and return the 16-bit patterns."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """Widen bf16 bit patterns to the fp32 values they denote (exact)."""
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


@dataclass
class Workload:
    name: str
    logits: np.ndarray  # [B, V] float32, or uint16 bf16 bit patterns
    dtype: str  # "f32" | "bf16"
    histories: list  # B int32 arrays
    params: list  # B SamplingParams
    steps: list  # B ints
    notes: dict = field(default_factory=dict)

    @property
    def batch(self) -> int:
        return int(self.logits.shape[0])

    @property
    def vocab(self) -> int:
        return int(self.logits.shape[1])

    def logits_f32(self) -> np.ndarray:
        """The values the sampler sees after its exact widening to fp32."""
        if self.dtype == "bf16":
            return bf16_bits_to_f32(self.logits)
        return self.logits

    def rows(self, index) -> "Workload":
        idx = list(range(self.batch))[index] if isinstance(index, slice) else list(index)
        return Workload(
            self.name,
            np.ascontiguousarray(self.logits[idx]),
            self.dtype,
            [self.histories[i] for i in idx],
            [self.params[i] for i in idx],
            [self.steps[i] for i in idx],
            dict(self.notes),
        )


_ZIPF_CDF: dict = {}


def _zipf_ids(rng: np.random.Generator, vocab: int, n: int, s: float = 1.1) -> np.ndarray:
    """n token ids with P(id) proportional to 1/(id+1)^s, bounded to [0, vocab)."""
    key = (vocab, s)
    cdf = _ZIPF_CDF.get(key)
    if cdf is None:
        w = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), s)
        cdf = np.cumsum(w / w.sum())
        cdf[-1] = 1.0
        _ZIPF_CDF[key] = cdf
    return np.searchsorted(cdf, rng.random(n), side="right").astype(np.int32).clip(0, vocab - 1)


def config1(seed: int = 1, batch: int = 4, vocab: int = 151_936) -> Workload:
    """fp32 N(0, 2.5^2) with 8 spikes of +12 per row; row 0 greedy, the others
    T=0.7, top_k=50, top_p=0.9, repetition 1.1 over 256 uniform history ids, seed = row."""
    rng = np.random.default_rng(seed)
    logits = (rng.standard_normal((batch, vocab)) * 2.5).astype(np.float32)
    for r in range(batch):
        spikes = rng.choice(vocab, size=min(8, vocab), replace=False)
        logits[r, spikes] += np.float32(12.0)
    histories = [rng.integers(0, vocab, 256).astype(np.int32) for _ in range(batch)]
    params = [SamplingParams()] + [
        SamplingParams(temperature=0.7, top_k=50, top_p=0.9, min_p=0.0,
                       repetition_penalty=1.1, seed=r)
        for r in range(1, batch)
    ]
    return Workload("config1", logits, "f32", histories, params, [3] * batch)


def config2(seed: int = 2, batch: int = 64, vocab: int = 151_936) -> Workload:
    """bf16 N(0, 3^2) plus a Zipf(1.1) bias over ids; parameter class = row mod 4;
    presence 0.5 / frequency 0.3 over 1..4096 Zipf history ids; 20 logprobs."""
    rng = np.random.default_rng(seed)
    bias = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), 1.1)
    bias = (bias / bias.max() * 6.0).astype(np.float32)
    logits = (rng.standard_normal((batch, vocab)) * 3.0).astype(np.float32) + bias
    histories, params = [], []
    for r in range(batch):
        common = dict(presence_penalty=0.5, frequency_penalty=0.3, logprobs=20, seed=1000 + r)
        kind = r % 4
        if kind == 0:
            p = SamplingParams(temperature=0.0, **common)
        elif kind == 1:
            p = SamplingParams(temperature=1.0, top_p=0.95, **common)
        elif kind == 2:
            p = SamplingParams(temperature=1.0, top_k=20, min_p=0.05, **common)
        else:
            p = SamplingParams(temperature=1.2, top_k=40, top_p=0.8, **common)
        params.append(p)
        histories.append(_zipf_ids(rng, vocab, int(rng.integers(1, 4097))))
    steps = [int(rng.integers(0, 512)) for _ in range(batch)]
    return Workload("config2", f32_to_bf16_bits(logits), "bf16", histories, params, steps)


def config3(seed: int = 3, batch: int = 256, vocab: int = 248_320,
            history_len: int = 32_768) -> Workload:
    """bf16 large-vocabulary stress.  First half: near-flat rows N(0, 0.1^2) with
    top_p 0.99 (tens of thousands kept).  Second half: peaked rows N(0, 4^2) whose values
    around rank top_k are duplicated, so exact ties straddle the top-k boundary
    (top_k 50, top_p 0.9, min_p 0.02).  All penalties on (1.05 / 0.4 / 0.2)."""
    rng = np.random.default_rng(seed)
    half = batch // 2
    top_k = 50
    logits = np.empty((batch, vocab), dtype=np.float32)
    for r in range(batch):
        scale = 0.1 if r < half else 4.0
        logits[r] = (rng.standard_normal(vocab) * scale).astype(np.float32)
    bits = f32_to_bf16_bits(logits)
    del logits
    tie_rows = {}
    for r in range(half, batch):
        row = bf16_bits_to_f32(bits[r])
        kk = min(top_k, vocab)
        lo, hi = max(kk - 3, 1), min(kk + 4, vocab)
        part = np.argpartition(-row, hi - 1)[:hi]
        order = part[np.argsort(-row[part], kind="stable")]
        bits[r, order[lo - 1:hi]] = bits[r, order[kk - 1]]
        tie_rows[r] = order[lo - 1:hi].astype(np.int32)
    pen = dict(repetition_penalty=1.05, presence_penalty=0.4, frequency_penalty=0.2)
    params = [
        SamplingParams(temperature=1.0, top_p=0.99, seed=3000 + r, **pen) if r < half else
        SamplingParams(temperature=1.0, top_k=top_k, top_p=0.9, min_p=0.02, seed=3000 + r, **pen)
        for r in range(batch)
    ]
    histories = [rng.integers(0, vocab, history_len).astype(np.int32) for _ in range(batch)]
    steps = [int(rng.integers(0, 4096)) for _ in range(batch)]
    return Workload("config3", bits, "bf16", histories, params, steps, {"tie_ids": tie_rows})


def config4(seed: int = 4, batch: int = 1024, vocab: int = 151_936) -> Workload:
    """Row-sharded decode: bf16 N(0, 3^2); per-row parameters drawn from the seed."""
    rng = np.random.default_rng(seed)
    bits = np.empty((batch, vocab), dtype=np.uint16)
    for r in range(batch):
        bits[r] = f32_to_bf16_bits((rng.standard_normal(vocab) * 3.0).astype(np.float32))
    histories, params, steps = [], [], []
    for r in range(batch):
        params.append(SamplingParams(
            temperature=float(np.float32(rng.uniform(0.3, 1.5))),
            top_k=int(rng.choice([0, 20, 50, 200])),
            top_p=float(np.float32(rng.uniform(0.7, 1.0))),
            min_p=float(rng.choice([0.0, 0.05])),
            repetition_penalty=float(np.float32(1.0 + rng.uniform(0.0, 0.6))),
            presence_penalty=float(np.float32(rng.uniform(0.0, 0.6))),
            frequency_penalty=float(np.float32(rng.uniform(0.0, 0.6))),
            seed=4000 + r,
        ))
        histories.append(rng.integers(0, vocab, int(rng.integers(512, 8193))).astype(np.int32))
        steps.append(int(rng.integers(0, 2048)))
    return Workload("config4", bits, "bf16", histories, params, steps)


def config5(seed: int = 5, batch: int = 128, vocab: int = 248_320) -> Workload:
    """Vocabulary-sharded sampling: bf16 N(0, 3^2); every row top_k 50, top_p 0.9,
    T 0.8, 20 logprobs.  The full-width rows are generated here; a rank takes the
    contiguous column range ``[rank*V/ranks, (rank+1)*V/ranks)``."""
    rng = np.random.default_rng(seed)
    bits = np.empty((batch, vocab), dtype=np.uint16)
    for r in range(batch):
        bits[r] = f32_to_bf16_bits((rng.standard_normal(vocab) * 3.0).astype(np.float32))
    params = [SamplingParams(temperature=0.8, top_k=50, top_p=0.9, logprobs=20, seed=5000 + r)
              for r in range(batch)]
    histories = [np.zeros(0, dtype=np.int32) for _ in range(batch)]
    return Workload("config5", bits, "bf16", histories, params, [7] * batch)


_BY_NAME = {"config1": config1, "config2": config2, "config3": config3,
            "config4": config4, "config5": config5}


def by_name(name: str, **kwargs) -> Workload:
    return _BY_NAME[name](**kwargs)
