"""Runs the UNMODIFIED reference sampler against the CPU checker on seeded random workloads,
beyond the ones kept as fixtures, and lists the rows on which they differ by more than the
comparison rules of tests/parity.py allow.

Run where the reference checkout is available (it is not on the GPU box):

    python tests/golden/compare_reference.py /path/to/reference random 18 5000 [seconds]
    python tests/golden/compare_reference.py /path/to/reference wide 18 2000 [seconds]

Nothing is written.  The generators are those of tests/cases.py (`random_workload`,
`wide_workload`); of a wide workload only the rows the GPU test checks are run.
"""
from __future__ import annotations

import importlib.util
import sys
import time
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
if len(sys.argv) < 5:
    raise SystemExit("usage: python tests/golden/compare_reference.py /path/to/reference random|wide FIRST LAST [seconds]")
KIND, FIRST, LAST = sys.argv[2], int(sys.argv[3]), int(sys.argv[4])
BUDGET = float(sys.argv[5]) if len(sys.argv) > 5 else 600.0
sys.argv = [sys.argv[0], sys.argv[1]]  # what make_golden.py reads

_spec = importlib.util.spec_from_file_location("make_golden", HERE / "make_golden.py")
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)  # imports the reference, defines run_reference_row

from oracle import sampler_oracle as O  # noqa: E402
from tests import cases, parity  # noqa: E402

EPS = {"random": 2e-5, "wide": 1e-4}[KIND]  # the summation noise allowed to the reference (tests/test_oracle.py)


def workload(seed: int):
    if KIND == "random":
        return cases.random_workload(seed)
    w, only = cases.wide_workload(seed)
    return w if only is None else w.rows(only)


def main() -> None:
    import torch

    torch.set_num_threads(1)
    started = time.time()
    rows = sensitive = differing = 0
    seed = FIRST
    for seed in range(FIRST, LAST):
        if time.time() - started > BUDGET:
            break
        w = workload(seed)
        x = w.logits_f32()
        report = parity.Report()
        for r in range(w.batch):
            sample, scores = make_golden.run_reference_row(x[r], w.histories[r], w.params[r], w.steps[r])
            o = O.sample_row(x[r], w.histories[r], w.params[r], w.steps[r])
            kept_n, kept_ids, kept_sum, cut = -1, None, 0, None
            if scores is not None:
                kept_ids = np.nonzero(np.isfinite(scores))[0]
                kept_n, kept_sum = kept_ids.size, int(kept_ids.astype(np.int64).sum())
                cut = float(scores[kept_ids].min())
            parity.compare_with_oracle(
                report, r, o, token=sample.token_id, logprob=sample.logprob, top=list(sample.top_logprobs),
                kept_n=kept_n, kept_ids=kept_ids, kept_sum=kept_sum, cut_value=cut, eps=EPS, exact_ties=False)
        rows += report.rows
        sensitive += report.sensitive
        if report.failures:
            differing += 1
            print(f"seed {seed}: {w.name}: {[f[:300] for f in report.failures[:3]]}", flush=True)
    print(f"{KIND} workloads, seeds {FIRST} to {seed}: {rows} rows, {sensitive} rounding-sensitive, "
          f"{differing} workloads with a difference beyond the rules, {time.time() - started:.0f} s")


if __name__ == "__main__":
    main()
