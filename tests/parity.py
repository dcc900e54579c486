"""Comparison rules shared by the checker tests and the GPU parity tests.

The reference leaves three things to its sort / topk / sum implementation, so a literal
equality test would be ill-posed there:

* which members of a group of EQUAL scores survive when the top-p cut falls inside the
  group, and the order of equal values in the top-N log-probability list;
* the last bits of the soft-max denominators (torch's vectorised fp32 CPU sum is off by
  about 5e-6 relative on a 150k-wide row), which can move a top-p cut by a few elements
  when neighbouring elements carry a few 1e-6 of probability each.

Everything else is compared exactly.  A row whose deciding quantity lies closer to its
threshold than the stated noise ``eps`` is "rounding-sensitive": it is allowed the small
deviation that noise can cause, and counted so a test can bound how many there are.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

REL = 1e-5  # relative tolerance for penalised logits and log-probabilities


def close(a: float, b: float, rel: float = REL, abs_: float = 2e-6) -> bool:
    if math.isinf(a) or math.isinf(b):
        return a == b
    return abs(a - b) <= max(abs_, rel * max(abs(a), abs(b)))


# (case name, rows compared, rounding-sensitive rows, rows whose top-p cut split a tie group),
# one entry per finished comparison; tests/conftest.py prints them after the run
COUNTS: list = []


@dataclass
class Report:
    rows: int = 0
    sensitive: int = 0
    tie_split: int = 0
    failures: list = field(default_factory=list)
    name: str = ""

    def fail(self, row, message):
        self.failures.append(f"row {row}: {message}")

    def assert_ok(self, max_sensitive_fraction: float = 1.0, name: str = ""):
        COUNTS.append((name or self.name or "?", self.rows, self.sensitive, self.tie_split))
        assert not self.failures, "\n".join(self.failures[:20])
        assert self.sensitive <= max_sensitive_fraction * max(self.rows, 1), (
            f"{self.sensitive} of {self.rows} rows were rounding-sensitive")


def allowed_count_slack(margins: dict, eps: float) -> int:
    """How many elements a top-p / min-p cut may move under relative noise eps."""
    slack = 0
    if "top_p" in margins and margins["top_p"] < eps:
        slack = max(slack, int(math.ceil(eps / max(margins.get("top_p_step", eps), 1e-12))) + 1)
    if "min_p" in margins and margins["min_p"] < eps:
        slack = max(slack, 1_000_000)  # a min-p tie group can be any size
    return slack


def check_top_logprobs(report, row, got, oracle_row, logp_of_id, rel=REL, members=True):
    """got: sequence of (id, value).  Values must match the checker's sorted values;
    ids must be genuine members carrying that value (ties may be listed in any order,
    filler entries at -inf may name any filtered id)."""
    want = oracle_row.top_logprobs
    if len(got) != len(want):
        report.fail(row, f"top_logprobs length {len(got)} != {len(want)}")
        return
    kept = set(oracle_row.kept.tolist())
    seen = set()
    for k, ((gi, gv), (_, wv)) in enumerate(zip(got, want)):
        if not close(gv, wv, rel):
            report.fail(row, f"top_logprobs[{k}] value {gv} != {wv}")
            return
        if math.isinf(wv):
            # (with a split tie group the implementation may have kept other members of the
            # group than the checker, so one of the checker's may be among its fillers)
            if members and gi in kept:
                report.fail(row, f"top_logprobs[{k}] filler id {gi} is a kept token")
            continue
        if not members:
            continue  # a split tie group: only the values are defined
        if gi not in kept or gi in seen or not close(logp_of_id(gi), gv, rel):
            report.fail(row, f"top_logprobs[{k}] id {gi} does not carry value {gv}")
            return
        seen.add(gi)


def oracle_logp(oracle_row):
    scores = oracle_row.scores
    kept = oracle_row.kept
    m = scores[kept].max()
    z = np.exp(scores[kept].astype(np.float64) - np.float64(m)).sum()
    return lambda i: float(scores[i].astype(np.float64) - np.float64(m) - np.log(z))


def compare_with_oracle(report: Report, row: int, oracle_row, *, token, logprob, top, kept_n,
                        kept_ids=None, kept_sum=None, cut_value=None, eps: float,
                        exact_ties: bool, check_token: bool = True):
    """One row of some implementation against the checker.

    exact_ties: the implementation follows the lowest-id tie rule (the CUDA sampler), so
    set membership is compared even when the cut splits a tie group.  For the reference
    (arbitrary tie order) pass False: membership inside a split tie group is skipped.
    """
    report.rows += 1
    m = oracle_row.margins
    slack = allowed_count_slack(m, eps)
    sensitive = slack > 0
    n_want = int(oracle_row.kept.size)
    same_set = True
    if kept_n is not None and kept_n >= 0:
        if kept_n != n_want:
            same_set = False
            if abs(kept_n - n_want) > slack:
                report.fail(row, f"kept count {kept_n} != {n_want} (margins {m})")
                return
        elif not sensitive:
            if cut_value is not None and not (np.float32(cut_value) == oracle_row.scores[oracle_row.kept].min()):
                report.fail(row, f"cut value {cut_value} != {oracle_row.scores[oracle_row.kept].min()}")
            splits = bool(m.get("top_p_splits_tie", False))
            if splits:
                report.tie_split += 1
            if exact_ties or not splits:
                if kept_ids is not None and not np.array_equal(np.sort(np.asarray(kept_ids)), oracle_row.kept):
                    report.fail(row, "kept ids differ")
                if kept_sum is not None and int(kept_sum) != int(oracle_row.kept.astype(np.int64).sum()):
                    report.fail(row, "kept id checksum differs")
            else:
                same_set = False
    if sensitive:
        report.sensitive += 1
    comparable = same_set and not sensitive
    if check_token and comparable:
        if m.get("draw", 1.0) > 1e-5 and token != oracle_row.token:
            report.fail(row, f"token {token} != {oracle_row.token} (margins {m})")
    if oracle_row.logprob is None:
        return
    if logprob is None:
        report.fail(row, "logprob missing")
        return
    if sensitive or (kept_n is not None and kept_n >= 0 and kept_n != n_want):
        return  # a moved cut renormalises every value; the count check above bounds it
    logp = oracle_logp(oracle_row)
    in_kept = token in set(oracle_row.kept.tolist())
    if in_kept and not close(logprob, logp(token)):
        report.fail(row, f"logprob {logprob} != {logp(token)} for token {token}")
    if not in_kept and same_set:
        report.fail(row, f"token {token} is not in the candidate set")
    check_top_logprobs(report, row, top, oracle_row, logp, members=same_set)
