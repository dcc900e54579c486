"""Cases taken from two wider sweeps that were run on the GPU once (thousands of seeded workloads
each): rows of a wider generator than tests/test_gpu_random_rows.py against the CPU checker, and
decode loops in which tokens repeat, resident histograms against the stateless call.

Collected after the established suite on purpose (file name): a surprise here must not keep
`pytest -x` from running the tests before it."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from hydraserve_b200.engine import SamplingParams, release_request, sample_logits  # noqa: E402
from tests.cases import wide_workload  # noqa: E402
from tests.test_gpu_parity import compare_case, sampler  # noqa: E402,F401


@pytest.mark.parametrize("seed", range(30))
def test_wide_rows_match_checker(sampler, seed):  # noqa: F811
    """The wider generator (batches of 1 to 64 rows, vocabularies up to 262,144, constant rows,
    rows below the bin window, parameters at both ends of their ranges): the checked rows of
    every launch against the CPU checker under the reference's own draws."""
    w, only = wide_workload(seed)
    compare_case(sampler, w, only=only).assert_ok(name=w.name)


def _decode_loop_case(seed):
    """A decode loop drawn from a seed: 1 to 12 requests over a vocabulary of 64 to 151,936
    tokens, 12 or 40 steps, empty to 600-token prompts, parameters that make tokens repeat
    (penalties that raise the scores of repeated tokens among them), bf16 on even seeds."""
    rng = np.random.default_rng(5_000 + seed)
    vocab = int(rng.choice([64, 500, 3_000, 40_000, 151_936]))
    batch = int(rng.choice([1, 3, 6, 12]))
    n_steps = int(rng.choice([12, 40]))
    dtype = torch.bfloat16 if seed % 2 == 0 else torch.float32
    scale = float(rng.choice([0.3, 1.5, 4.0]))
    params, prompts = [], []
    for i in range(batch):
        params.append(SamplingParams(
            temperature=float(rng.choice([0.0, 0.4, 1.0, 1.6])), top_k=int(rng.choice([0, 0, 3, 40, 256, 300])),
            top_p=float(rng.choice([1.0, 0.95, 0.6])), min_p=float(rng.choice([0.0, 0.05])),
            repetition_penalty=float(rng.choice([1.0, 0.6, 1.3])), presence_penalty=float(rng.choice([0.0, -1.5, 0.5])),
            frequency_penalty=float(rng.choice([0.0, -0.4, 0.3])), seed=int(rng.integers(0, 2**31)),
            logprobs=[None, 0, 5][int(rng.integers(0, 3))]))
        n = int(rng.choice([0, 2, 50, 600]))
        prompts.append(rng.integers(0, vocab, n).tolist())
    base = torch.from_numpy((rng.standard_normal((batch, vocab)) * scale).astype(np.float32)).cuda()
    shrink_at = int(rng.integers(3, n_steps))
    return vocab, batch, n_steps, dtype, scale, params, prompts, base, shrink_at


# (seeds 1406 to 1729: loops whose first step differed between the two calls while a penalised
# row with an empty prompt was given a slot with request ids and none without)
@pytest.mark.parametrize("seed", [1400, 1401, 1402, 1403, 1404, 1405, 1406, 1432, 1515, 1549, 1620, 1623, 1644,
                                  1671, 1689, 1697, 1729])
def test_decode_loops_in_which_tokens_repeat(seed):
    """Resident histograms (request ids, one new token per step) against the stateless call
    (whole history every step), sample for sample, over loops in which tokens come back often:
    counts pass one, two and three inside the loop, and one request is replayed from two
    tokens back (its history shrinks)."""
    vocab, batch, n_steps, dtype, scale, params, prompts, base, shrink_at = _decode_loop_case(seed)

    def drive(resident):
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        gen = [[] for _ in range(batch)]
        out = []
        for step in range(n_steps):
            logits = (base + 0.3 * scale * torch.randn((batch, vocab), device="cuda", generator=g)).to(dtype)
            s = sample_logits(logits, [p + q for p, q in zip(prompts, gen)], params, steps=[len(q) for q in gen],
                              request_ids=[("loop", seed, i) for i in range(batch)] if resident else None)
            for i, t in enumerate(s):
                gen[i].append(t.token_id)
            out.append(s)
            if step == shrink_at and len(gen[0]) > 2:
                del gen[0][-2:]  # preempted and replayed
        if resident:
            for i in range(batch):
                release_request(("loop", seed, i))
        return out

    with_ids, stateless = drive(True), drive(False)
    for step, (a, b) in enumerate(zip(with_ids, stateless)):
        assert a == b, f"step {step}: rows {[i for i in range(batch) if a[i] != b[i]]} differ"
