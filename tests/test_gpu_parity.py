"""GPU parity: the CUDA sampler, called through its C ABI, against the CPU checker on
the same seeded inputs.  Integer results (tokens, candidate sets) are compared exactly;
floating-point results within 1e-5 relative (tests/parity.py states the tie rules)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import sampler_oracle as O  # noqa: E402
from tests import cases, parity  # noqa: E402

# The CUDA sampler accumulates probability mass exactly (integers of 2^-40) and uses a
# 2-ulp expf whose errors average out over a row; a cut closer than this (relative) to
# its threshold may move by an element.
GPU_EPS = 2e-7

PARITY_CASES = [
    "tiny_v1", "tiny_v2", "tiny_v3", "tiny_v9", "tiny_v33",
    "small_f32", "small_bf16", "small_odd_f32", "small_odd_bf16",
    "config1", "config2_8rows", "config3_4rows", "config4_8rows", "config5_4rows",
]


@pytest.fixture(scope="module")
def sampler(built_library):
    from hydraserve_b200.engine import _device

    s = _device.DeviceSampler("cuda:0", vocab_max=420_000, batch_max=64, resident_slots=64)
    yield s
    s.close()


def device_logits(w):
    if w.dtype == "bf16":
        return torch.from_numpy(w.logits.view(np.int16)).view(torch.bfloat16).cuda()
    return torch.from_numpy(w.logits).cuda()


def oracle_rows(w, draws=True, only=None):
    """Checker results per row (None for rows outside ``only``) and the Exp(1) draws the
    reference would use (ones for rows that are not checked)."""
    x = w.logits_f32()
    rows, noise = [], np.ones((w.batch, w.vocab), np.float32)
    for r in range(w.batch):
        if only is not None and r not in only:
            rows.append(None)
            continue
        p = w.params[r]
        q = None
        if p.temperature != 0.0:
            q = O.exponential_draws(O.mixed_seed(p.seed, w.steps[r]), w.vocab)
            noise[r] = q
        rows.append(O.sample_row(x[r], w.histories[r], p, w.steps[r], draws=q, want_probabilities=False))
    return rows, noise


def compare_case(sampler, w, report=None, request_ids=None, only=None):
    """Every row of ``w`` (or the rows in ``only``; the others are launched with them all the
    same) through the C ABI against the checker."""
    only = None if only is None else set(int(r) for r in only)
    rows, noise = oracle_rows(w, only=only)
    records, scores = sampler.sample(device_logits(w), w.histories, w.params, w.steps, request_ids,
                                     noise=torch.from_numpy(noise), want_scores=True)
    report = report or parity.Report(name=w.name)
    assert int((records["status"] != 0).sum()) == 0, f"rows with a status: {np.nonzero(records['status'])[0][:8]}"
    for r, o in enumerate(rows):
        if o is None:
            continue
        rec = records[r]
        score_row = scores[r].cpu().numpy()
        kept = np.nonzero(np.isfinite(score_row))[0]
        n_top = int(rec["n_top"])
        top = list(zip(rec["top_ids"][:n_top].tolist(), rec["top_logprobs"][:n_top].tolist()))
        if w.params[r].logprobs is not None:
            want = min(w.params[r].logprobs, w.vocab)
            taken, i = {t for t, _ in top}, 0
            while len(top) < want:
                if i not in taken:
                    top.append((i, float("-inf")))
                i += 1
        before = len(report.failures)
        parity.compare_with_oracle(
            report, r, o, token=int(rec["token"]),
            logprob=float(rec["logprob"]) if w.params[r].logprobs is not None else None,
            top=top, kept_n=int(rec["n_kept"]), kept_ids=kept, eps=GPU_EPS, exact_ties=True)
        sensitive = parity.allowed_count_slack(o.margins, GPU_EPS) > 0
        if len(report.failures) == before and not sensitive:
            if int(rec["n_kept"]) != kept.size:
                report.fail(r, f"n_kept {rec['n_kept']} disagrees with the score dump {kept.size}")
            # kept scores (penalised, temperature-scaled) are IEEE-exact steps: bit for bit
            if not np.array_equal(score_row[o.kept], o.scores[o.kept]):
                bad = np.nonzero(score_row[o.kept] != o.scores[o.kept])[0]
                report.fail(r, f"{bad.size} kept scores differ, first id {o.kept[bad[0]]}: "
                               f"{score_row[o.kept][bad[0]]!r} vs {o.scores[o.kept][bad[0]]!r}")
            if w.params[r].temperature != 0.0:
                if int(rec["n_after_topk"]) != o.n_after_topk:
                    report.fail(r, f"n_after_topk {rec['n_after_topk']} != {o.n_after_topk}")
                if int(rec["n_after_minp"]) != o.n_after_minp:
                    report.fail(r, f"n_after_minp {rec['n_after_minp']} != {o.n_after_minp}")
    return report


@pytest.mark.parametrize("name", PARITY_CASES)
def test_rows_match_checker(sampler, name):
    report = compare_case(sampler, cases.build(name))
    report.assert_ok(max_sensitive_fraction=0.5, name=name)


@pytest.mark.parametrize("parts", [2, 4])
@pytest.mark.parametrize("name", ["small_bf16", "small_odd_bf16", "config2_8rows", "config3_4rows", "config4_8rows"])
def test_counting_rows_split_over_several_ctas(sampler, name, parts):
    """A counting row whose tokens are counted by 2 or 4 CTAs (each a range; the last to
    arrive adds the others' count tables to its own) gives the same results as one CTA."""
    sampler.set_count_split(parts)
    try:
        compare_case(sampler, cases.build(name)).assert_ok(max_sensitive_fraction=0.5,
                                                           name=f"{name} (counted by {parts} CTAs per row)")
    finally:
        sampler.set_count_split(0)


@pytest.fixture(scope="module")
def general_sampler(built_library):
    """A sampler that sends bf16 rows through the general (fp32-resident) kernel as well."""
    from hydraserve_b200 import _lib
    from hydraserve_b200.engine import _device

    s = _device.DeviceSampler("cuda:0", vocab_max=250_000, batch_max=64, resident_slots=8,
                              flags=_lib.HS_CREATE_FORCE_GENERAL)
    assert s.query(4, 151_936) == 0
    yield s
    s.close()


@pytest.mark.parametrize("name", [n for n in PARITY_CASES if "bf16" in n or n.startswith("config")])
def test_bf16_rows_match_checker_on_the_general_kernel(general_sampler, name):
    compare_case(general_sampler, cases.build(name)).assert_ok(max_sensitive_fraction=0.5, name=name + " (general kernel)")


def test_bf16_kernel_is_the_one_used_for_bf16(sampler):
    assert sampler.query(4, 151_936, 1) >= 1 and sampler.query(4, 248_320, 1) >= 1
    assert sampler.query(4, 151_936, 0) == 0


def test_penalised_logits_bit_exact(sampler):
    """Greedy rows dump the penalised logits themselves (no temperature, no filter)."""
    from hydraserve_b200.engine.sampling import SamplingParams

    w = cases.build("config2_8rows")
    params = [SamplingParams(repetition_penalty=1.3, presence_penalty=-0.7, frequency_penalty=0.9, logprobs=0)
              for _ in range(w.batch)]
    records, scores = sampler.sample(device_logits(w), w.histories, params, w.steps, None, want_scores=True)
    x = w.logits_f32()
    for r in range(w.batch):
        want = O.penalise(x[r], w.histories[r], params[r])
        np.testing.assert_array_equal(scores[r].cpu().numpy(), np.where(want == 0, np.float32(0), want))
        assert int(records[r]["token"]) == int(np.argmax(want))


def test_greedy_fast_path_lowest_id_on_ties(sampler):
    rng = np.random.default_rng(7)
    for vocab, dtype in ((151_936, "bf16"), (248_320, "bf16"), (1003, "f32"), (5, "bf16"), (1, "f32")):
        x = (rng.standard_normal((9, vocab)) * 3).astype(np.float32)
        if dtype == "bf16":
            from hydraserve_b200.workloads import bf16_bits_to_f32, f32_to_bf16_bits

            bits = f32_to_bf16_bits(x)
            x = bf16_bits_to_f32(bits)
            # duplicate the maximum of some rows at a higher id
            for r in range(0, 9, 2):
                j = int(np.argmax(x[r]))
                if j + 1 < vocab:
                    bits[r, vocab - 1] = bits[r, j]
                    x[r, vocab - 1] = x[r, j]
            t = torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).cuda()
        else:
            t = torch.from_numpy(x).cuda()
        got = sampler.greedy(t).cpu().numpy()
        np.testing.assert_array_equal(got, np.argmax(x, axis=1))


def test_strided_and_unaligned_rows(sampler):
    """Rows that are a view of a wider buffer: stride != vocab and 2-byte aligned only."""
    rng = np.random.default_rng(8)
    base = torch.from_numpy((rng.standard_normal((6, 1200)) * 2).astype(np.float32)).cuda().bfloat16()
    view = base[:, 3:1003]
    got = sampler.greedy(view).cpu().numpy()
    np.testing.assert_array_equal(got, view.float().cpu().numpy().argmax(axis=1))
    w = cases.build("small_odd_bf16")
    full = torch.zeros((w.batch, w.vocab + 21), dtype=torch.bfloat16, device="cuda")
    full[:, 5:5 + w.vocab] = device_logits(w)
    rows, noise = oracle_rows(w)
    records, _ = sampler.sample(full[:, 5:5 + w.vocab], w.histories, w.params, w.steps, None,
                                noise=torch.from_numpy(noise))
    ref_records, _ = sampler.sample(device_logits(w), w.histories, w.params, w.steps, None,
                                    noise=torch.from_numpy(noise))
    np.testing.assert_array_equal(records["token"], ref_records["token"])
    np.testing.assert_array_equal(records["n_kept"], ref_records["n_kept"])


def test_resident_histograms_match_stateless(sampler):
    """request_ids keep the histogram on the device and upload only the new tokens."""
    w = cases.build("config4_8rows")
    rows, noise = oracle_rows(w)
    ids = [f"req-{i}" for i in range(w.batch)]
    # first call: histories cut short; second call: full histories (delta upload)
    short = [h[: max(1, h.size // 2)] for h in w.histories]
    sampler.sample(device_logits(w), short, w.params, w.steps, ids)
    records, scores = sampler.sample(device_logits(w), w.histories, w.params, w.steps, ids,
                                     noise=torch.from_numpy(noise), want_scores=True)
    stateless, scores2 = sampler.sample(device_logits(w), w.histories, w.params, w.steps, None,
                                        noise=torch.from_numpy(noise), want_scores=True)
    np.testing.assert_array_equal(records["token"], stateless["token"])
    assert torch.equal(scores, scores2)
    # a shrunken history (preempt / replay) rebuilds the slot
    records3, scores3 = sampler.sample(device_logits(w), short, w.params, w.steps, ids, want_scores=True)
    stateless3, scores4 = sampler.sample(device_logits(w), short, w.params, w.steps, None, want_scores=True)
    assert torch.equal(scores3, scores4)
    for i in ids:
        sampler.release_request(i)


def test_global_stage_fallback_for_very_wide_rows(sampler):
    """A row too wide for the cluster's shared memory is staged in global scratch."""
    from hydraserve_b200.engine.sampling import SamplingParams
    from hydraserve_b200.workloads import Workload

    vocab = 410_001
    assert sampler.query(1, vocab, 0) == 0 and sampler.query(1, 248_320, 0) == 1
    rng = np.random.default_rng(9)
    x = (rng.standard_normal((3, vocab)) * 3).astype(np.float32)
    params = [SamplingParams(logprobs=5, presence_penalty=0.5),
              SamplingParams(temperature=0.9, top_k=64, top_p=0.9, seed=5, logprobs=20, frequency_penalty=0.2),
              SamplingParams(temperature=1.0, top_p=0.95, min_p=0.001, seed=6, repetition_penalty=1.2)]
    hist = [rng.integers(0, vocab, 3000).astype(np.int32) for _ in range(3)]
    w = Workload("wide", x, "f32", hist, params, [1, 2, 3])
    compare_case(sampler, w).assert_ok(max_sensitive_fraction=0.34)


def test_philox_draws_are_reproducible_and_follow_the_distribution(sampler):
    """Seeded Philox path: same seed -> same token; across seeds the token frequencies
    pass a chi-square test against the checker's filtered distribution."""
    from scipy import stats

    from hydraserve_b200.engine.sampling import SamplingParams

    rng = np.random.default_rng(10)
    vocab, draws = 4096, 64  # 64 rows x 3,200 calls = 204,800 draws
    x = (rng.standard_normal(vocab) * 2.0).astype(np.float32)
    base = SamplingParams(temperature=0.9, top_k=40, top_p=0.95, seed=0)
    o = O.sample_row(x, (), base, 0, draws=np.ones(vocab, np.float32))
    probs = o.probabilities[o.kept]
    logits = torch.from_numpy(np.tile(x, (draws, 1))).cuda()
    counts = np.zeros(vocab, np.int64)
    total = 0
    first = None
    for rep in range(3200):
        params = [base.with_seed(rep * draws + i) for i in range(draws)]
        records, _ = sampler.sample(logits, [()] * draws, params, [rep] * draws, None)
        if rep == 0:
            first = records["token"].copy()
            again, _ = sampler.sample(logits, [()] * draws, params, [rep] * draws, None)
            np.testing.assert_array_equal(first, again["token"])
        np.add.at(counts, records["token"], 1)
        total += draws
    assert counts.sum() == counts[o.kept].sum(), "a token outside the candidate set was drawn"
    expected = probs * total
    big = expected >= 5
    obs = np.append(counts[o.kept][big], counts[o.kept][~big].sum())
    exp = np.append(expected[big], expected[~big].sum())
    if exp[-1] == 0:
        obs, exp = obs[:-1], exp[:-1]
    chi2, pvalue = stats.chisquare(obs, exp * obs.sum() / exp.sum())
    assert pvalue > 1e-4, f"chi-square p={pvalue:.3g} over {total} draws"


def _bf16_round(x):
    """fp32 values rounded to bf16 (round to nearest even), as fp32 and as raw bits."""
    u = np.asarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    bits = u.astype(np.uint16)
    return (bits.astype(np.uint32) << 16).view(np.float32), bits


@pytest.mark.parametrize("draw", ["by_tokens", "by_classes"])
@pytest.mark.parametrize("kind", ["fine", "coarse", "two_values"])
def test_bf16_philox_draws_follow_the_distribution(sampler, kind, draw):
    """The counting kernel's seeded draw against the checker's distribution, both ways it is
    made.  by_tokens (what these fairly flat rows take by default): rejection on tokens, with
    a top-p cut that splits a tie group (coarse, two_values: only the group's lowest ids may
    come out).  by_classes (what peaked rows take; forced here): class by inverse CDF, then a
    uniformly chosen member, by scanning the row for small classes, by rejection for large
    ones.  fine: every class has a few members (scan); coarse: classes of tens to hundreds of
    members (scan, and rejection with the scan as fall-back); two_values: classes of about a
    thousand members (rejection)."""
    from scipy import stats

    from hydraserve_b200.engine.sampling import SamplingParams

    rng = np.random.default_rng({"fine": 21, "coarse": 22, "two_values": 23}[kind])
    vocab, rows, reps = 2048, 64, 3200  # 204,800 draws per kind
    raw = rng.standard_normal(vocab).astype(np.float32)
    if kind == "coarse":
        raw = np.round(raw * 4.0) / 4.0 + 0.125
    elif kind == "two_values":
        raw = np.where(rng.random(vocab) < 0.5, 0.5, 1.0).astype(np.float32)
    x, bits = _bf16_round(raw)
    history = rng.integers(0, vocab, 600).astype(np.int32)  # count classes 0, 1, 2 and a few higher
    base = SamplingParams(temperature=1.0, top_p=0.98, seed=0, repetition_penalty=1.1, presence_penalty=0.3,
                          frequency_penalty=0.1)
    o = O.sample_row(x, history, base, 0, draws=np.ones(vocab, np.float32))
    probs = o.probabilities[o.kept]
    logits = torch.from_numpy(np.tile(bits.view(np.int16), (rows, 1))).view(torch.bfloat16).cuda()
    assert sampler.query(4, vocab) == 1, "bf16 rows must take the counting / candidate kernels"
    counts = np.zeros(vocab, np.int64)
    total = 0
    sampler.set_token_draw(draw == "by_tokens")
    try:
        for rep in range(reps):
            params = [base.with_seed(rep * rows + i) for i in range(rows)]
            records, _ = sampler.sample(logits, [history] * rows, params, [rep] * rows, None)
            assert int((records["status"] != 0).sum()) == 0
            if rep == 0:
                again, _ = sampler.sample(logits, [history] * rows, params, [rep] * rows, None)
                np.testing.assert_array_equal(records["token"], again["token"])
            np.add.at(counts, records["token"], 1)
            total += rows
    finally:
        sampler.set_token_draw(True)
    assert counts.sum() == counts[o.kept].sum(), "a token outside the candidate set was drawn"
    expected = probs * total
    big = expected >= 5
    obs = np.append(counts[o.kept][big], counts[o.kept][~big].sum())
    exp = np.append(expected[big], expected[~big].sum())
    if exp[-1] == 0:
        obs, exp = obs[:-1], exp[:-1]
    chi2, pvalue = stats.chisquare(obs, exp * obs.sum() / exp.sum())
    assert pvalue > 1e-4, f"{kind}/{draw}: chi-square p={pvalue:.3g} over {total} draws ({obs.size} cells)"


def test_candidate_path_ties_and_long_lists(sampler):
    """Rows of the candidate kernel (0 < top_k <= 256) whose lists take the less common
    routes: hundreds of exact ties at the k-th value (all kept; the k-th key is found in a
    bucket of equal keys), top_k = 256 (lists longer than the short-list sort), top_k = 1,
    and the same with penalties; the rows are wide enough to be split over two CTAs."""
    from hydraserve_b200.engine.sampling import SamplingParams
    from hydraserve_b200.workloads import Workload

    rng = np.random.default_rng(31)
    vocab, batch = 70_000, 5
    raw = (rng.standard_normal((batch, vocab)) * 3.0).astype(np.float32)
    # row 0: 30 clear leaders, then 300 tokens tied exactly at the value where k = 50 falls
    raw[0] = np.minimum(raw[0], 5.0)
    lead = rng.choice(vocab, 330, replace=False)
    raw[0, lead[:30]] = 9.0 + np.arange(30, dtype=np.float32) * 0.25
    raw[0, lead[30:]] = 7.0
    x = np.empty_like(raw)
    bits = np.empty(raw.shape, np.uint16)
    for r in range(batch):
        x[r], bits[r] = _bf16_round(raw[r])
    params = [
        SamplingParams(temperature=0.8, top_k=50, top_p=0.95, seed=1, logprobs=20),
        SamplingParams(temperature=1.1, top_k=256, top_p=0.9, min_p=0.01, seed=2, logprobs=5),
        SamplingParams(temperature=0.7, top_k=1, seed=3, logprobs=3),
        SamplingParams(temperature=1.0, top_k=256, seed=4, repetition_penalty=1.2, presence_penalty=0.5,
                       frequency_penalty=0.3, logprobs=20),
        SamplingParams(temperature=0.9, top_k=200, top_p=0.5, seed=5, frequency_penalty=0.4),
    ]
    hist = [rng.integers(0, vocab, 4000).astype(np.int32) for _ in range(batch)]
    # make the leaders of rows 3 and 4 part of their histories, some of them many times
    for r in (3, 4):
        top_ids = np.argsort(-x[r])[:40].astype(np.int32)
        hist[r] = np.concatenate([hist[r], np.repeat(top_ids, rng.integers(1, 6, top_ids.size))])
    w = Workload("candidate_edges", bits, "bf16", hist, params, [0, 1, 2, 3, 4])
    assert sampler.query(4, vocab) == 1
    report = compare_case(sampler, w)
    report.assert_ok(max_sensitive_fraction=0.4)


def test_rows_with_more_classes_than_shared_memory_holds(sampler):
    """Logits spread over every bf16 value of the bin window, two thirds of the tokens in the
    history once or twice: far more than 6,144 non-empty (count class, value) classes per row,
    so the class list spills from shared memory into its global scratch."""
    from hydraserve_b200.engine.sampling import SamplingParams
    from hydraserve_b200.workloads import Workload

    rng = np.random.default_rng(41)
    vocab, batch = 120_000, 4
    # uniformly random bf16 patterns with 2^-14 <= |x| < 2^4 (sign, 18 binades, 7 mantissa bits)
    exponent = rng.integers(113, 131, (batch, vocab)).astype(np.uint16)
    mantissa = rng.integers(0, 128, (batch, vocab)).astype(np.uint16)
    sign = rng.integers(0, 2, (batch, vocab)).astype(np.uint16)
    bits = (sign << 15) | (exponent << 7) | mantissa
    hist = []
    for r in range(batch):
        once = rng.choice(vocab, vocab // 3, replace=False)
        twice = rng.choice(vocab, vocab // 3, replace=False)
        hist.append(np.concatenate([once, twice, twice]).astype(np.int32))
    params = [
        SamplingParams(temperature=1.0, top_p=0.97, seed=1, repetition_penalty=1.3, presence_penalty=0.7,
                       frequency_penalty=0.4, logprobs=20),
        SamplingParams(temperature=0.6, top_k=2000, top_p=0.9, seed=2, presence_penalty=1.0, frequency_penalty=0.5),
        SamplingParams(temperature=1.5, min_p=0.001, seed=3, repetition_penalty=0.8, frequency_penalty=0.2, logprobs=4),
        SamplingParams(temperature=0.0, repetition_penalty=1.5, presence_penalty=0.2, logprobs=10),
    ]
    w = Workload("many_classes", bits, "bf16", hist, params, [3, 2, 1, 0])
    x = w.logits_f32()
    for r in range(batch):
        y = O.penalise(x[r], hist[r], params[r])
        classes = {(int(c), float(v)) for c, v in zip(np.minimum(np.bincount(hist[r], minlength=vocab), 3), x[r])}
        assert len(classes) > 6144 and np.isfinite(y).all()
    compare_case(sampler, w).assert_ok(max_sensitive_fraction=0.5)


def test_rows_with_thousands_of_often_repeated_tokens(sampler):
    """Histories in which 3,000 tokens occur three to six times: their exact counts matter
    (frequency penalty), the list of such tokens is longer than one thread-per-entry pass and
    than the side list's shared-memory form, in the counting and in the candidate kernel."""
    from hydraserve_b200.engine.sampling import SamplingParams
    from hydraserve_b200.workloads import Workload

    rng = np.random.default_rng(43)
    vocab, batch = 60_000, 4
    raw = (rng.standard_normal((batch, vocab)) * 2.5).astype(np.float32)
    bits = np.empty(raw.shape, np.uint16)
    for r in range(batch):
        _, bits[r] = _bf16_round(raw[r])
    hist = []
    for r in range(batch):
        often = rng.choice(vocab, 3000, replace=False)
        # the highest logits are among the often repeated ones, so that they decide the cuts
        often[:50] = np.argsort(-raw[r])[:50]
        reps = rng.integers(3, 7, often.size)
        rest = rng.integers(0, vocab, 5000)
        h = np.concatenate([np.repeat(often, reps), rest]).astype(np.int32)
        rng.shuffle(h)
        hist.append(h)
    params = [
        SamplingParams(temperature=1.0, top_p=0.9, seed=1, frequency_penalty=0.15, presence_penalty=0.1, logprobs=20),
        SamplingParams(temperature=0.9, top_k=64, top_p=0.95, seed=2, frequency_penalty=0.2, repetition_penalty=1.1,
                       logprobs=20),
        SamplingParams(temperature=0.0, frequency_penalty=0.3, logprobs=5),
        SamplingParams(temperature=1.2, top_k=256, min_p=0.002, seed=4, frequency_penalty=0.1),
    ]
    w = Workload("often_repeated", bits, "bf16", hist, params, [0, 1, 2, 3])
    compare_case(sampler, w).assert_ok(max_sensitive_fraction=0.5)


def test_rows_with_more_zeros_than_the_side_list_holds(sampler):
    """Logits rounded to halves: an eighth of a 151,936-token row is exactly (minus) zero, a value
    below the bin window, so those tokens are scored one by one from the side list.  Row 0 has
    more of them than the list's global form holds (16,384) and must be handed to the general
    kernel, with every token still counted; row 1 has fewer and stays; rows 2 and 3 repeat the
    two with filters and penalties."""
    from hydraserve_b200.engine.sampling import SamplingParams
    from hydraserve_b200.workloads import Workload

    rng = np.random.default_rng(53)
    vocab, batch = 151_936, 4
    raw = np.round(rng.standard_normal((batch, vocab)) * 3.4) / 2.0
    raw = np.where(raw == 0.0, -0.0, raw).astype(np.float32)
    for r in (1, 3):  # leave about 15,000 zeros
        zeros = np.nonzero(raw[r] == 0.0)[0]
        raw[r, zeros[15_000:]] = 0.5
    bits = np.empty(raw.shape, np.uint16)
    for r in range(batch):
        _, bits[r] = _bf16_round(raw[r])
    n_zero = [(raw[r] == 0.0).sum() for r in range(batch)]
    assert n_zero[0] > 16_500 and n_zero[2] > 16_500 and 14_000 < n_zero[1] <= 15_000 and 14_000 < n_zero[3] <= 15_000
    hist = [rng.integers(0, vocab, 200).astype(np.int32) for _ in range(batch)]
    params = [
        SamplingParams(temperature=1.0, seed=1, presence_penalty=-0.3, logprobs=0),
        SamplingParams(temperature=1.0, seed=2, presence_penalty=-0.3, logprobs=0),
        SamplingParams(temperature=0.8, top_p=0.999, min_p=1e-5, seed=3, repetition_penalty=1.2, frequency_penalty=0.1, logprobs=5),
        SamplingParams(temperature=1.3, top_k=100_000, seed=4, presence_penalty=0.5),
    ]
    w = Workload("many_zeros", bits, "bf16", hist, params, [0, 1, 2, 3])
    compare_case(sampler, w).assert_ok(max_sensitive_fraction=0.5)


def test_candidate_list_overflow_falls_back_to_counting(sampler):
    """More tokens tied at the k-th value than a candidate list holds: the candidate kernel
    hands the row back and the second counting pass serves it (all ties are kept, as in the
    reference).  One row is wide enough to be split over two CTAs, one is not."""
    from hydraserve_b200.engine.sampling import SamplingParams
    from hydraserve_b200.workloads import Workload

    rng = np.random.default_rng(47)
    for vocab in (20_000, 90_000):
        batch = 3
        raw = (rng.standard_normal((batch, vocab)) * 1.5).astype(np.float32)
        raw = np.minimum(raw, 3.0)
        tied = rng.choice(vocab, 9000, replace=False)
        raw[0, tied] = 4.0                      # 9,000 tokens share the maximum: top_k = 50 keeps them all
        raw[1, tied[:6000]] = 4.0               # 20 leaders, then 6,000 tied at the value where k = 40 falls
        raw[1, tied[6000:6020]] = 6.0 + np.arange(20, dtype=np.float32) * 0.5
        bits = np.empty(raw.shape, np.uint16)
        for r in range(batch):
            _, bits[r] = _bf16_round(raw[r])
        params = [
            SamplingParams(temperature=1.0, top_k=50, seed=1, logprobs=20),
            SamplingParams(temperature=0.8, top_k=40, top_p=0.9, seed=2, presence_penalty=0.5, logprobs=5),
            SamplingParams(temperature=1.0, top_k=50, top_p=0.95, seed=3),  # an ordinary row beside them
        ]
        hist = [rng.integers(0, vocab, 500).astype(np.int32) for _ in range(batch)]
        w = Workload("overflow", bits, "bf16", hist, params, [0, 1, 2])
        rows, _ = oracle_rows(w)
        assert rows[0].n_after_topk >= 9000 and rows[1].n_after_topk >= 5000  # (a few tied tokens are penalised)
        compare_case(sampler, w).assert_ok(max_sensitive_fraction=0.67)


def test_fp32_rows_with_small_top_k_take_the_candidate_kernel(sampler, general_sampler):
    """fp32 logits (the reference's CPU-runnable check): rows with 0 < top_k <= 256 are served by
    the fp32 candidate kernel, the others by the general kernel launched next to it (two
    launches per call); the results are the general kernel's."""
    w = cases.build("config1")
    assert w.dtype == "f32"
    before = sampler.query(3, w.vocab)
    got, _ = sampler.sample(device_logits(w), w.histories, w.params, w.steps, None)
    assert sampler.query(3, w.vocab) - before >= 2
    want, _ = general_sampler.sample(device_logits(w), w.histories, w.params, w.steps, None)
    # (not the sampled token: which token a seeded draw lands on depends on the kernel's order
    # of the candidates; the sets and the cuts do not)
    for field in ("status", "n_kept", "n_after_topk", "n_after_minp", "n_cut_ties", "cut_bits"):
        np.testing.assert_array_equal(got[field], want[field], err_msg=field)
    compare_case(sampler, w).assert_ok(max_sensitive_fraction=0.5, name="config1 (fp32 candidate kernel)")


def test_fp32_candidate_list_overflow_falls_back_to_the_general_kernel(sampler):
    """fp32 rows with more tokens tied at the k-th value than a candidate list holds: the
    candidate kernel reports the row (status 4) and the general kernel samples it."""
    from hydraserve_b200.engine.sampling import SamplingParams
    from hydraserve_b200.workloads import Workload

    rng = np.random.default_rng(48)
    vocab, batch = 30_000, 3
    raw = np.minimum((rng.standard_normal((batch, vocab)) * 1.5).astype(np.float32), 3.0)
    tied = rng.choice(vocab, 9000, replace=False)
    raw[0, tied] = 4.0
    raw[1, tied[:6000]] = 4.0
    raw[1, tied[6000:6020]] = 6.0 + np.arange(20, dtype=np.float32) * 0.5
    params = [
        SamplingParams(temperature=1.0, top_k=50, seed=1, logprobs=20),
        SamplingParams(temperature=0.8, top_k=40, top_p=0.9, seed=2, presence_penalty=0.5, logprobs=5),
        SamplingParams(temperature=1.0, top_k=50, top_p=0.95, seed=3),
    ]
    hist = [rng.integers(0, vocab, 500).astype(np.int32) for _ in range(batch)]
    w = Workload("fp32 overflow", raw, "f32", hist, params, [0, 1, 2])
    rows, _ = oracle_rows(w)
    assert rows[0].n_after_topk >= 9000 and rows[1].n_after_topk >= 5000
    compare_case(sampler, w).assert_ok(max_sensitive_fraction=0.67)
