"""GPU parity on seeded random rows: vocabulary sizes, value distributions, histories and
sampling parameters drawn from a seed, so that rows reach the kernels' paths in combinations
no hand-written case lists (near-flat rows next to peaked ones in one launch, ties with
penalties, vocabularies with a third of the tokens pushed far down, top_k around the candidate path's limit, rows too short for a
vector load).  Every row is compared with the CPU checker under the reference's own draws; the
same rows are then sampled with seeded Philox draws, which must repeat and land in the
checker's candidate set."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from hydraserve_b200.engine.sampling import SamplingParams  # noqa: E402
from hydraserve_b200.workloads import Workload, f32_to_bf16_bits  # noqa: E402
from tests import parity  # noqa: E402
from tests.test_gpu_parity import GPU_EPS, compare_case, device_logits, oracle_rows, sampler  # noqa: E402,F401

VOCABS = [1, 7, 8, 33, 1_000, 4_099, 33_000, 70_001, 151_936]


def random_workload(seed: int) -> Workload:
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


@pytest.mark.parametrize("seed", range(54))
def test_random_rows_match_checker(sampler, seed):  # noqa: F811
    w = random_workload(seed)
    report = compare_case(sampler, w)
    report.assert_ok(max_sensitive_fraction=0.5, name=w.name)

    # seeded Philox draws: repeatable, and inside the checker's candidate set
    rows, _ = oracle_rows(w)
    first, _ = sampler.sample(device_logits(w), w.histories, w.params, w.steps, None)
    again, _ = sampler.sample(device_logits(w), w.histories, w.params, w.steps, None)
    np.testing.assert_array_equal(first["token"], again["token"])
    assert int((first["status"] != 0).sum()) == 0
    for r, o in enumerate(rows):
        if w.params[r].temperature == 0.0:
            assert int(first["token"][r]) == o.token, f"{w.name}, row {r}: arg max {first['token'][r]} != {o.token}"
            continue
        if parity.allowed_count_slack(o.margins, GPU_EPS) > 0:
            continue  # a cut within rounding of its threshold may move by an element
        kept = set(np.asarray(o.kept).tolist())
        assert int(first["token"][r]) in kept, f"{w.name}, row {r}: token {first['token'][r]} is not a candidate"
