"""Named, seeded test inputs shared by the golden-fixture script, the checker tests and
the GPU parity tests.  A case is a function of its name only."""
from __future__ import annotations

import numpy as np

from hydraserve_b200 import workloads
from hydraserve_b200.engine.sampling import SamplingParams
from hydraserve_b200.workloads import Workload, f32_to_bf16_bits


def small_mixed(seed: int, batch: int, vocab: int, dtype: str) -> Workload:
    """Rows over a small vocabulary that walk through every parameter combination the
    sampler has, with quantised logits so exact ties are everywhere."""
    rng = np.random.default_rng(seed)
    logits = np.empty((batch, vocab), np.float32)
    params, histories, steps = [], [], []
    for r in range(batch):
        scale = float(rng.choice([0.05, 0.5, 2.0, 4.0, 8.0]))
        row = rng.standard_normal(vocab).astype(np.float32) * np.float32(scale)
        style = r % 4
        if style == 1:  # few distinct levels: many ties
            row = np.round(row * 4) / 4
        elif style == 2:  # a dominant spike
            row[rng.integers(0, vocab)] += np.float32(15.0)
        elif style == 3:  # all equal but a handful
            row[:] = np.float32(rng.normal())
            row[rng.choice(vocab, size=min(5, vocab), replace=False)] += np.float32(1.5)
        logits[r] = row
        temperature = float(rng.choice([0.0, 0.3, 0.7, 1.0, 1.5, 2.0]))
        top_k = int(rng.choice([0, 0, 1, 5, 50, vocab, vocab + 10]))
        top_p = float(rng.choice([1.0, 1.0, 0.99, 0.9, 0.5, 0.1]))
        min_p = float(rng.choice([0.0, 0.0, 0.01, 0.1, 0.5, 1.0]))
        rep = float(rng.choice([1.0, 1.0, 1.1, 0.8, 2.0]))
        pres = float(rng.choice([0.0, 0.0, 0.5, -0.5, 2.0]))
        freq = float(rng.choice([0.0, 0.0, 0.3, -0.2, 2.0]))
        logprobs = rng.choice([-1, -1, 0, 1, 5, 20])
        params.append(SamplingParams(
            temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p,
            repetition_penalty=rep, presence_penalty=pres, frequency_penalty=freq,
            seed=int(rng.integers(0, 2**63 - 1)), logprobs=None if logprobs < 0 else int(logprobs)))
        n_hist = int(rng.choice([0, 1, 17, 300, 4000]))
        history = rng.integers(-3, vocab + 3, n_hist).astype(np.int32)  # some ids out of range
        histories.append(history)
        steps.append(int(rng.integers(0, 10_000)))
    if dtype == "bf16":
        return Workload(f"small_{dtype}", f32_to_bf16_bits(logits), "bf16", histories, params, steps)
    return Workload(f"small_{dtype}", logits, "f32", histories, params, steps)


def tiny(vocab: int) -> Workload:
    """Vocabularies of a few entries: unaligned rows, top_k >= V, logprobs > V."""
    rng = np.random.default_rng(100 + vocab)
    batch = 6
    logits = (rng.standard_normal((batch, vocab)) * 2).astype(np.float32)
    params = [
        SamplingParams(),
        SamplingParams(logprobs=20),
        SamplingParams(temperature=1.0, seed=1, logprobs=3),
        SamplingParams(temperature=0.5, top_k=2, seed=2, logprobs=20),
        SamplingParams(temperature=1.3, top_p=0.6, min_p=0.2, seed=3, frequency_penalty=1.0, logprobs=2),
        SamplingParams(temperature=2.0, top_k=1, top_p=0.5, seed=4, repetition_penalty=1.5),
    ]
    histories = [rng.integers(0, vocab, 5).astype(np.int32) for _ in range(batch)]
    return Workload(f"tiny_v{vocab}", logits, "f32", histories, params, list(range(batch)))


VOCABS = [1, 7, 8, 33, 1_000, 4_099, 33_000, 70_001, 151_936]


def random_workload(seed: int) -> Workload:
    """Six rows drawn from a seed: vocabulary size, value distribution, history and sampling
    parameters (edges included); odd seeds are fp32, even ones bf16."""
    rng = np.random.default_rng(1000 + seed)
    vocab = int(VOCABS[seed % len(VOCABS)])
    batch = 6
    logits = np.empty((batch, vocab), np.float32)
    histories, params, steps = [], [], []
    for r in range(batch):
        kind = rng.integers(0, 5)
        if kind == 0:      # near-flat
            x = rng.standard_normal(vocab) * rng.uniform(0.02, 0.5)
        elif kind == 1:    # peaked
            x = rng.standard_normal(vocab) * rng.uniform(2.0, 6.0)
        elif kind == 2:    # few distinct values: long tie groups
            x = np.round(rng.standard_normal(vocab) * rng.uniform(1.0, 4.0) * 2.0) / 2.0
        elif kind == 3:    # part of the vocabulary pushed far down, some values outside the bin window
            x = rng.standard_normal(vocab) * 3.0
            x[rng.random(vocab) < 0.3] = -1.0e4
            x[rng.random(vocab) < 0.01] = 0.0
            x[rng.random(vocab) < 0.002] = 3000.0 * rng.standard_normal()
        else:              # a shifted row: everything negative
            x = rng.standard_normal(vocab) * rng.uniform(0.5, 3.0) - 20.0
        logits[r] = x.astype(np.float32)
        # histories: empty, short, or long with repeats (counts of three and more)
        n_hist = int(rng.choice([0, 3, 200, 5_000]))
        pool = rng.integers(0, vocab, max(1, min(vocab, int(rng.choice([4, 300, 20_000])))))
        histories.append(rng.choice(pool, n_hist).astype(np.int32) if n_hist else np.zeros(0, np.int32))
        penalised = rng.random() < 0.7
        params.append(SamplingParams(
            temperature=float(rng.choice([0.0, 0.3, 0.8, 1.0, 1.7])),
            top_k=int(rng.choice([0, 0, 1, 5, 50, 256, 257, vocab + 5])),
            top_p=float(rng.choice([1.0, 0.999, 0.95, 0.7, 0.3])),
            min_p=float(rng.choice([0.0, 0.0, 0.02, 0.3])),
            repetition_penalty=float(rng.choice([1.0, 1.05, 1.6])) if penalised else 1.0,
            presence_penalty=float(rng.choice([0.0, 0.4, -0.3])) if penalised else 0.0,
            frequency_penalty=float(rng.choice([0.0, 0.2, 1.0])) if penalised else 0.0,
            seed=int(rng.integers(0, 2**31)),
            logprobs=[None, 0, 5, 20][int(rng.integers(0, 4))],
        ))
        steps.append(int(rng.integers(0, 5000)))
    if seed % 2:  # fp32 logits: the fp32 candidate kernel (small top_k) and the general kernel
        return Workload(f"random rows, seed {seed} (vocabulary {vocab}, fp32)", logits, "f32", histories, params, steps)
    return Workload(f"random rows, seed {seed} (vocabulary {vocab})", f32_to_bf16_bits(logits), "bf16", histories,
                    params, steps)



WIDE_VOCABS = [2, 9, 255, 1_000, 4_097, 12_345, 32_000, 50_257, 100_003, 128_256, 151_936, 151_937, 200_064, 248_320, 262_144]
WIDE_BATCHES = [1, 2, 6, 6, 6, 17, 40, 64]

def wide_workload(seed: int):
    """A wider draw than random_workload: 1 to 64 rows (of which six are checked when there are
    more), fifteen vocabulary sizes up to 262,144, constant rows, rows entirely below the bf16
    kernel's bin window, large offsets, ties at the top, and every parameter at both ends of its
    allowed range; every third seed is fp32.  Returns (workload, rows to check or None)."""
    rng = np.random.default_rng(77_000 + seed)
    vocab = int(rng.choice(WIDE_VOCABS)); batch = int(rng.choice(WIDE_BATCHES))
    if vocab > 160_000 and batch > 17: batch = 17
    logits = np.empty((batch, vocab), np.float32)
    histories, params, steps = [], [], []
    for r in range(batch):
        kind = int(rng.integers(0, 9))
        if kind == 0: x = rng.standard_normal(vocab) * rng.uniform(0.02, 0.5)
        elif kind == 1: x = rng.standard_normal(vocab) * rng.uniform(2.0, 8.0)
        elif kind == 2: x = np.round(rng.standard_normal(vocab) * rng.uniform(0.5, 4.0) * 2.0) / 2.0
        elif kind == 3:
            x = rng.standard_normal(vocab) * 3.0
            x[rng.random(vocab) < 0.3] = -1.0e4
            x[rng.random(vocab) < rng.choice([0.001, 0.01, 0.12])] = 0.0
            x[rng.random(vocab) < 0.002] = 3000.0 * rng.standard_normal()
        elif kind == 4: x = rng.standard_normal(vocab) * rng.uniform(0.5, 3.0) - rng.choice([20.0, 200.0])
        elif kind == 5: x = np.full(vocab, float(rng.choice([0.0, -3.25, 11.0])))            # constant row
        elif kind == 6: x = rng.standard_normal(vocab) * 1e-5                                    # everything below the window
        elif kind == 7: x = rng.standard_normal(vocab) * 2.0 + rng.choice([50.0, 900.0])      # big offsets
        else:
            x = rng.standard_normal(vocab) * 2.5
            top = rng.choice(vocab, min(vocab, int(rng.choice([1, 3, 300]))), replace=False)
            x[top] = 9.0                                                                         # ties at the top
        logits[r] = x.astype(np.float32)
        n_hist = int(rng.choice([0, 1, 3, 200, 3_000]))
        pool = rng.integers(0, vocab, max(1, min(vocab, int(rng.choice([1, 4, 300, 20_000])))))
        histories.append(rng.choice(pool, n_hist).astype(np.int32) if n_hist else np.zeros(0, np.int32))
        penalised = rng.random() < 0.7
        params.append(SamplingParams(
            temperature=float(rng.choice([0.0, 0.05, 0.3, 0.8, 1.0, 1.7, 2.0])),
            top_k=int(rng.choice([0, 0, 1, 2, 5, 50, 255, 256, 257, 1000, 20_000, vocab - 1, vocab, vocab + 5])),
            top_p=float(rng.choice([1.0, 0.9999, 0.95, 0.7, 0.3, 0.01])),
            min_p=float(rng.choice([0.0, 0.0, 1e-4, 0.02, 0.3, 0.9])),
            repetition_penalty=float(rng.choice([1.0, 1.05, 1.6, 0.7, 2.0])) if penalised else 1.0,
            presence_penalty=float(rng.choice([0.0, 0.4, -0.3, 2.0, -2.0])) if penalised else 0.0,
            frequency_penalty=float(rng.choice([0.0, 0.2, 1.0, -0.1, 2.0])) if penalised else 0.0,
            seed=int(rng.integers(0, 2**31)),
            logprobs=[None, 0, 1, 5, 20][int(rng.integers(0, 5))],
        ))
        steps.append(int(rng.integers(0, 5000)))
    only = None if batch <= 6 else sorted(rng.choice(batch, 6, replace=False).tolist())
    name = f"wide seed {seed} (vocab {vocab}, batch {batch}, {'f32' if seed % 3 == 0 else 'bf16'})"
    if seed % 3 == 0: return Workload(name, logits, "f32", histories, params, steps), only
    return Workload(name, f32_to_bf16_bits(logits), "bf16", histories, params, steps), only


_CASES = {
    "config1": lambda: workloads.config1(),
    "config2_8rows": lambda: workloads.config2(batch=8),
    "config3_4rows": lambda: workloads.config3(batch=4),
    "config4_8rows": lambda: workloads.config4(batch=8),
    "config5_4rows": lambda: workloads.config5(batch=4),
    "small_f32": lambda: small_mixed(11, 48, 2048, "f32"),
    "small_bf16": lambda: small_mixed(12, 48, 2048, "bf16"),
    "small_odd_f32": lambda: small_mixed(13, 24, 1003, "f32"),
    "small_odd_bf16": lambda: small_mixed(14, 24, 1003, "bf16"),
    "tiny_v1": lambda: tiny(1),
    "tiny_v2": lambda: tiny(2),
    "tiny_v3": lambda: tiny(3),
    "tiny_v9": lambda: tiny(9),
    "tiny_v33": lambda: tiny(33),
}
# the benchmark configurations at full size (config 4: the seeded quarter the GPU test checks)
_CASES["config2_full"] = lambda: workloads.config2()
_CASES["config3_full"] = lambda: workloads.config3()
_CASES["config4_quarter"] = lambda: workloads.config4().rows(
    np.sort(np.random.default_rng(44).choice(1024, 256, replace=False)).tolist())  # the rows the GPU test checks
_CASES["config5_full"] = lambda: workloads.config5()
# seeded random rows whose reference outputs are kept as fixtures (two rounds over the vocabulary sizes)
RANDOM_GOLDEN_SEEDS = tuple(range(18))
for _seed in RANDOM_GOLDEN_SEEDS:
    _CASES[f"random_rows_{_seed}"] = (lambda s=_seed: random_workload(s))

# ... and of the wider generator: the rows the GPU test checks
WIDE_GOLDEN_SEEDS = tuple(range(18))


def _wide_checked(seed: int) -> Workload:
    w, only = wide_workload(seed)
    return w if only is None else w.rows(only)


for _seed in WIDE_GOLDEN_SEEDS:
    _CASES[f"wide_rows_{_seed}"] = (lambda s=_seed: _wide_checked(s))

GOLDEN_CASES = tuple(_CASES)

_cache: dict = {}


def build(name: str) -> Workload:
    if name not in _cache:
        _cache[name] = _CASES[name]()
    return _cache[name]
